"""The MoVA router and the SEED4P4 per-head maps through the C ABI, against the oracle.

Shapes and tolerances follow the reference's own kernel tests: tests/test_mova_kernels.c:376-445 (router: ids exact,
weights within 1e-5; the top-k step with many exact ties, lowest id first) and :882-945 (per-head maps against the
scalar sum over the exact weights, |a - b| <= |b| / 128 + 2e-6)."""
import numpy as np
import pytest

from oracle import binding as B

pytestmark = pytest.mark.gpu


def bfr(a):
    return (B.f2bf(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)


@pytest.fixture(scope="module")
def K():
    from nanoseedlm_b200 import kernels
    return kernels


@pytest.fixture(scope="module")
def L():
    from nanoseedlm_b200 import lib
    return lib


@pytest.mark.parametrize("d,n,k,T", [(512, 20, 4, 5), (2048, 128, 8, 8), (2048, 100, 8, 3), (64, 1024, 64, 2)])
def test_router(K, L, d, n, k, T):
    rng = np.random.default_rng(d + n)
    W = B.f2bf((rng.random((n, d), np.float32) * 2 - 1) * 0.05)
    bias = B.f2bf((rng.random(n, np.float32) * 2 - 1) * 0.01)
    x = bfr(rng.standard_normal((T, d), np.float32))
    a = L.RouterArgs(d, n, k, d // 2, 2.5)
    ind, wt, score, sel = K.kt_router(a, W, bias, x, T)
    so, eo, io, wo = B.mova_router(W, bias, x, k, d // 2, 2.5)
    # f32 sums against the oracle's double sums: a logit may round to the neighbouring BF16 value, rarely
    diff = np.abs(score - so)
    assert diff.max() < 2e-3 and (diff > 1e-6).mean() < 0.02
    np.testing.assert_array_equal(sel, score + (bias.astype(np.uint32) << 16).view(np.float32)[None, :])
    # the selection from the kernel's own scores is exact
    i2, w2 = B.mova_topk(score, sel, k, 2.5)
    np.testing.assert_array_equal(ind, i2)
    np.testing.assert_array_equal(wt, w2)
    clean = diff.max(axis=1) <= 1e-6
    np.testing.assert_array_equal(ind[clean], io[clean])
    np.testing.assert_allclose(wt[clean], wo[clean], atol=1e-5, rtol=0)


@pytest.mark.parametrize("n,k", [(100, 8), (64, 4), (512, 10), (1024, 64), (1, 1)])
def test_router_topk_ties_to_lowest_id(K, L, n, k):
    rng = np.random.default_rng(n)
    T = 6
    sc = (rng.random((T, n), np.float32) * 0.5 + 0.5).astype(np.float32)
    se = (np.floor(rng.random((T, n)) * 12) / 16).astype(np.float32)   # few distinct values: many ties
    a = L.RouterArgs(2048, n, k, 1024, 2.5)
    ind, wt = K.kt_router_topk(a, sc, se, T)
    io, wo = B.mova_topk(sc, se, k, 2.5)
    np.testing.assert_array_equal(ind, io)
    np.testing.assert_array_equal(wt, wo)


def test_router_refuses_bad_sizes(K, L):
    a = L.RouterArgs(2048, 2000, 8, 1024, 1.0)
    with pytest.raises(RuntimeError, match="out of range"):
        K.kt_router_topk(a, np.zeros((1, 2000), np.float32), np.zeros((1, 2000), np.float32), 1)


def stacked(H, O, I, seed):
    mats = [B.Matrix(O, I, seed + h, eb=-22 + h) for h in range(H)]
    assert (O * I // 8) % 2 == 0
    return (mats, np.concatenate([m.seeds.ravel() for m in mats]), np.concatenate([m.coefs.ravel() for m in mats]),
            np.array([m.eb for m in mats], np.int32), np.concatenate([m.codes.ravel() for m in mats]))


@pytest.mark.parametrize("O,I,T,gate", [(96, 128, 3, 0), (128, 192, 5, 1), (128, 192, 37, 1), (6144, 128, 2, 1),
                                        (6, 8, 1, 0), (10, 24, 8, 1), (33, 2048, 4, 0)])
def test_heads_mv(K, O, I, T, gate):
    H = 3
    mats, seeds, coefs, eb, codes = stacked(H, O, I, 1000 + O)
    rng = np.random.default_rng(O * I)
    x = bfr((rng.random((T, H * I), np.float32) * 2 - 1) * 2)
    g = bfr((rng.random((T, H, O), np.float32) * 2 - 1) * 3)
    y = K.kt_heads_seed(H, O, I, seeds, coefs, eb, codes, x, H * I, I, g if gate else None, T)
    for h in range(H):
        Wd = B.decode_rows_f32(mats[h]).astype(np.float64)
        acc = x[:, h * I:(h + 1) * I].astype(np.float64) @ Wd.T          # [T][O]
        want = bfr(acc.astype(np.float32))
        if gate:
            want = bfr(want * B.softplus_gate(g[:, h, :]))
        got = y[:, h, :]
        slack = np.abs(want) / 128 + 2e-6
        assert (np.abs(got - want) <= slack).all(), (h, np.abs(got - want).max())
        # and nearly all of them are the same BF16 value
        assert (got == want).mean() > 0.98


def test_heads_mv_rows_independent_of_batch(K):
    """A row's result does not depend on how many rows share the call (engine/kernels_moe.cu:239-240)."""
    H, O, I = 2, 64, 256
    mats, seeds, coefs, eb, codes = stacked(H, O, I, 77)
    x = bfr(np.random.default_rng(3).standard_normal((11, H * I), np.float32))
    full = K.kt_heads_seed(H, O, I, seeds, coefs, eb, codes, x, H * I, I, None, 11)
    for t in (0, 7, 8, 10):
        one = K.kt_heads_seed(H, O, I, seeds, coefs, eb, codes, x[t:t + 1], H * I, I, None, 1)
        np.testing.assert_array_equal(one[0], full[t])


@pytest.mark.parametrize("O,I", [(96, 128), (128, 192), (6, 8)])
def test_heads_deq_bit_exact(K, O, I):
    H = 3
    mats, seeds, coefs, eb, codes = stacked(H, O, I, 500 + I)
    got = K.kt_heads_deq(H, O, I, seeds, coefs, eb, codes)
    for h in range(H):
        np.testing.assert_array_equal(got[h], B.decode_rows_bf16(mats[h]).reshape(O, I))


def test_heads_refuse_other_formats(K, L):
    L.load().kc_heads_deq(None, 0, L.WSlice(), None, 1, 8, 8, None)   # 0 = MF_BF16
    with pytest.raises(RuntimeError, match="not served"):
        L.check()
