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
