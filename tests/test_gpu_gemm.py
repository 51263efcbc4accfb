"""The tcgen05 prompt GEMM (dense and grouped) against the oracle, through the C ABI.

Shapes and bars follow the reference's test_mm (tests/test_mova_kernels.c:246-317): R = 40 (not a tile multiple),
K = 128, T = 45 tokens with a residual add, 50 pairs over 3 slices with xdiv 2 in a tile table; seed weights rounded to
bf16 (default mode) or exact (three-term mode); results within one bf16 ulp plus 2 x 64 x 1.2e-7 x sum|w x|."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bfr(a):
    a = np.asarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def close_bf(got, ref, extra):
    return np.abs(got.astype(np.float64) - ref) <= np.abs(ref) / 128.0 + 1e-30 + extra


def make(oracle, S, R, K, seed):
    from nanoseedlm_b200 import kernels
    mats = [oracle.Matrix(R, K, seed * 10 + s, eb=(-19, -17, -21)[s % 3]) for s in range(S)]
    return mats, kernels.SeedWeight.from_matrices(mats)


def ref_rows(oracle, mats, slices, xrows, exact):
    """y[p] = sum_c wv x, wv = f32 weights or their bf16 rounding; also sum|wv x|."""
    out, mag = [], []
    for s, x in zip(slices, xrows):
        w = oracle.decode_rows_f32(mats[s]).astype(np.float64) if exact else bfr(oracle.decode_rows_f32(mats[s])).astype(np.float64)
        out.append(w @ x.astype(np.float64))
        mag.append(np.abs(w) @ np.abs(x.astype(np.float64)))
    return np.array(out), np.array(mag)


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("R,K,T", [(40, 128, 45), (128, 64, 16), (300, 512, 130), (24, 72, 5)])
def test_mm_dense_residual(oracle, exact, R, K, T):
    from nanoseedlm_b200 import kernels
    mats, w = make(oracle, 1, R, K, R + K)
    x = oracle.normal(T, T * K, bf16=True).reshape(T, K)
    y0 = oracle.normal(T + 1, T * R, bf16=True).reshape(T, R)
    y = kernels.kt_mm(w, x, T, add=1, y0=y0, exact=exact)
    acc, mag = ref_rows(oracle, mats, [0] * T, x, exact)
    ref = bfr(y0 + bfr(acc.astype(np.float32))).astype(np.float64)
    # the accumulated term is itself rounded to bf16 before the add: where f32 summation order moves it across a
    # rounding boundary the result moves by one bf16 ulp of |acc| (visible where y0 + acc cancels)
    ok = close_bf(y, ref, 2 * 64 * 1.2e-7 * mag + np.abs(acc) / 128)
    assert ok.all(), np.argwhere(~ok)[:5]
    assert np.mean(close_bf(y, ref, 2 * 64 * 1.2e-7 * mag)) > 0.999
    y2 = kernels.kt_mm(w, x, T, exact=exact, packed=not exact)
    assert close_bf(y2, bfr(acc.astype(np.float32)).astype(np.float64), 64 * 1.2e-7 * mag).all()


@pytest.mark.parametrize("exact", [False, True])
@pytest.mark.parametrize("mode", ["host", "dev", "packed"])
def test_mm_grouped_tile_table(oracle, exact, mode):
    if exact and mode == "packed":
        pytest.skip("the packed-input entry points are the bf16-weight mode's")
    from nanoseedlm_b200 import kernels
    R, K, S, P, xdiv = 40, 128, 3, 50, 2
    mats, w = make(oracle, S, R, K, 77)
    x = oracle.normal(5, 45 * K, bf16=True).reshape(45, K)
    slc = [(p * 7) % S for p in range(P)]
    perm, tiles = [], []
    for s in range(S):
        st = len(perm)
        perm += [p for p in range(P) if slc[p] == s]
        for o in range(st, len(perm), 128):
            tiles.append((s, o, min(128, len(perm) - o)))
    y = kernels.kt_mm_grouped(w, P, xdiv, perm, tiles, x, exact=exact, mode=mode)
    acc, mag = ref_rows(oracle, mats, slc, [x[p // xdiv] for p in range(P)], exact)
    ok = close_bf(y, bfr(acc.astype(np.float32)).astype(np.float64), 64 * 1.2e-7 * mag)
    assert ok.all(), np.argwhere(~ok)[:5]


def test_mm_grouped_many_pairs_per_expert(oracle):
    """More than one tile per expert (300 pairs on 2 slices) and the oracle's own grouped reference."""
    from nanoseedlm_b200 import kernels
    R, K, S, P = 136, 256, 2, 300
    mats, w = make(oracle, S, R, K, 5)
    x = oracle.normal(9, P * K, bf16=True).reshape(P, K)
    inds = np.array([(p * 5 + p // 7) % S for p in range(P)], np.int32)
    perm, tiles, nt = kernels.kt_bucket(inds, S)
    y = kernels.kt_mm_grouped(w, P, 1, perm, tiles, x, mode="dev")
    ref = oracle.mm_pairs(mats, inds, 1, x)
    _, mag = ref_rows(oracle, mats, inds, x, False)
    assert close_bf(y, ref.astype(np.float64), 64 * 1.2e-7 * mag).all()


def test_moe_layer_prompt_rows_match_decode_rows(oracle):
    """The grouped prompt path (T > 8) against the mat-vec path on the same rows: same routing; outputs differ only
    by the prompt path's bf16 rounding of the seed weights."""
    from nanoseedlm_b200 import moe
    d, ff, E, k, T = 256, 64, 16, 4, 40
    h = moe.HostLayer(oracle, d, ff, E, seed=3)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, T)
    x = oracle.normal(1, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(2, T * E).reshape(T, E)
    out_mm, ind_mm = m.forward_host(x, logits)
    m.set_grouped_min_tokens(10 ** 6)
    out_mv, ind_mv = m.forward_host(x, logits)
    assert np.array_equal(ind_mm, ind_mv)
    assert np.max(np.abs(out_mm - out_mv)) <= 2e-2 * np.max(np.abs(out_mv))
    rind, _ = oracle.route(logits, k)
    assert np.array_equal(ind_mm, rind)
    m.close()
