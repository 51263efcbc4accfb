"""The vectorised CPU seed mat-vec (the timed baseline): equal to its scalar form bit for bit and within 2e-6 of the
double-precision spec on the reference's shape list (tests/test_cpu_seed4.c:49-63, 182-195).  No GPU."""
import numpy as np
import pytest


@pytest.mark.parametrize("rows,K", [(768, 2560), (2560, 768), (640, 2560), (100, 512), (17, 64)])
def test_vector_equals_scalar_and_spec(oracle, rows, K):
    m = oracle.Matrix(rows, K, rows * 7 + K, eb=-22)
    x = oracle.normal(K, K)
    yv = oracle.cpu_seed4_matvec(m, x, threads=3)
    ys = oracle.cpu_seed4_matvec(m, x, scalar=True)
    assert np.array_equal(yv.view(np.uint32), ys.view(np.uint32))
    y64, mag = oracle.matvec_f64(m, x)
    assert np.max(np.abs(yv - y64[0]) / mag[0]) < 2e-6


def test_thread_counts_agree(oracle):
    m = oracle.Matrix(300, 512, 9)
    x = oracle.normal(3, 512)
    y1 = oracle.cpu_seed4_matvec(m, x, threads=1)
    y4 = oracle.cpu_seed4_matvec(m, x, threads=4)
    assert np.array_equal(y1.view(np.uint32), y4.view(np.uint32))


@pytest.mark.parametrize("rows,kb,threads", [(16, 4, 1), (768, 320, 1), (2560, 96, 4), (1000, 34, 7), (37, 10, 2)])
def test_tiled_layout_gives_the_same_rows(oracle, rows, kb, threads):
    """The CPU-tiled layout: the same arithmetic in the same order as the row-major kernel, so the same bits
    (tests/test_cpu_seed4.c:38-46, 63)."""
    m = oracle.Matrix(rows, kb * 8, rows + kb, eb=-21)
    x = oracle.normal(rows, kb * 8)
    t = oracle.Tiled(m)
    assert np.array_equal(t.matmul(x, threads)[0], oracle.cpu_seed4_matvec(m, x, scalar=True))


@pytest.mark.parametrize("rows,kb,ntok,threads", [(40, 8, 3, 1), (640, 320, 4, 3), (100, 16, 8, 2)])
def test_tiled_tokens_equal_one_token_calls(oracle, rows, kb, ntok, threads):
    """ntok tokens at once: each token's rows equal a one-token call, bit for bit (tests/test_cpu_seed4.c:70-93)."""
    m = oracle.Matrix(rows, kb * 8, 5 * rows + ntok, eb=-21)
    x = oracle.normal(ntok, ntok * kb * 8).reshape(ntok, kb * 8)
    t = oracle.Tiled(m)
    y = t.matmul(x, threads)
    for k in range(ntok):
        assert np.array_equal(y[k], t.matmul(x[k:k + 1], 1)[0])


def test_tiled_refusals_and_job_lists(oracle):
    with pytest.raises(ValueError):
        oracle.Tiled(oracle.Matrix(16, 24, 1))          # 3 blocks per row: the layout pairs blocks
    ms = [oracle.Matrix(40 + 16 * i, 64, 3 + i, eb=-18) for i in range(5)]
    ts = [oracle.Tiled(m) for m in ms]
    xs = [oracle.normal(9 + i, 64 * (1 + i % 3)).reshape(-1, 64) for i in range(5)]
    for t, x, y in zip(ts, xs, oracle.tiled_jobs(list(zip(ts, xs)), 3)):
        assert np.array_equal(y, t.matmul(x))
    with pytest.raises(ValueError):
        ts[0].matmul(np.zeros((9, 64), np.float32))     # more than 8 tokens
