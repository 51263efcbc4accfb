"""The LM head's affine int4 dense mat-vec (kc_mv with MF_Q4) and the greedy arg-max, through the C ABI.

Bounds follow the reference's kernel test (tests/test_mova_kernels.c:181-215): |y - ref| <= |ref| / 128 + 48 * 1.2e-7 *
sum |w x| (one bf16 ulp plus f32 accumulation), twice that with the residual add; token 0's rows are the same bits
for every T."""
import numpy as np
import pytest

from oracle import binding as B

pytestmark = pytest.mark.gpu


def q4_weights(R, K, seed):
    rng = np.random.default_rng(seed)
    codes = rng.integers(0, 2 ** 32, (R, K // 8), dtype=np.uint64).astype(np.uint32)
    scales = B.f2bf((rng.random((R, K // 64), np.float32) * 0.02 + 0.001))
    biases = B.f2bf((rng.random((R, K // 64), np.float32) * -0.2 + 0.02))
    return codes, scales, biases


def bf16v(a):
    return (B.f2bf(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("R,K", [(24, 256), (24, 512), (24, 4096), (37, 2048), (1000, 64), (16, 8192), (40, 1024), (5000, 1024), (5000, 2048), (2400, 4096)])
def test_q4_dense_tokens_add_and_batch_invariance(R, K):
    from nanoseedlm_b200 import kernels
    codes, scales, biases = q4_weights(R, K, R + K)
    rng = np.random.default_rng(K)
    x = bf16v(rng.random((8, K), np.float32) * 2 - 1)
    first = None
    for T in range(1, 9):
        add = int(T == 3)
        y0 = bf16v(rng.random((T, R), np.float32) * 2 - 1)
        y = kernels.kt_mv_q4(codes, scales, biases, x[:T], T, add, y0 if add else None)
        ref, mag = B.q4_mv(codes, scales, biases, x[:T], add, y0 if add else None)
        bound = np.abs(ref) / 128 + 48 * 1.2e-7 * mag * (2 if add else 1) + 1e-30
        assert (np.abs(y - ref) <= bound).all(), (T, float(np.max(np.abs(y - ref) / bound)))
        if T == 1:
            first = y[0].copy()
        elif not add:
            assert np.array_equal(y[0], first), f"token 0 differs between T=1 and T={T}"


def test_q4_refuses_what_it_does_not_serve():
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    codes, scales, biases = q4_weights(8, 96, 1)       # K not a multiple of 64
    with pytest.raises(RuntimeError, match="multiple of 64"):
        kernels.kt_mv_q4(codes, scales, biases, np.zeros((1, 96), np.float32), 1)


@pytest.mark.parametrize("V,n", [(151936, 3), (1000, 5), (7, 2), (1024, 1)])
def test_argmax_ties_to_the_lowest_id_and_probability(V, n):
    from nanoseedlm_b200 import kernels
    rng = np.random.default_rng(V)
    logits = (rng.standard_normal((n, V)) * 3).astype(np.float32)
    logits[0, V // 2] = logits[0, V - 1] = logits[0].max() + 1          # an exact tie: the lower id wins
    out, prob = kernels.kt_argmax(logits, prob=True)
    ro, rp = B.argmax(logits)
    assert np.array_equal(out, ro) and out[0] == V // 2
    np.testing.assert_allclose(prob, rp, rtol=2e-5)
    assert np.array_equal(kernels.kt_argmax(logits), ro)
