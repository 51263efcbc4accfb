"""P = 3 seeds (format SEED4, the nibble-word blocks) through the mat-vec entry points and the bit-exact decode.

Bounds as the reference's kernel test for this format (tests/test_mova_kernels.c:160-243): one bf16 ulp plus
64 x 1.2e-7 x sum |w x| of f32 accumulation, twice that with the residual add; token 0's rows the same bits for every T;
gate+up within one bf16 flip of g or u."""
import numpy as np
import pytest

from oracle import binding as B

pytestmark = pytest.mark.gpu
F32B = 64 * 1.2e-7


@pytest.fixture(scope="module")
def K():
    from nanoseedlm_b200 import kernels
    return kernels


def exact(m):
    return B.decode3_rows_f32(m).astype(np.float64)


@pytest.mark.parametrize("R,Kc", [(24, 256), (7, 72), (512, 2048), (5, 8)])
def test_p3_decode_bit_exact(K, R, Kc):
    m = B.Matrix3(R, Kc, R + Kc, eb=-21)
    m.nibs[0, 0], m.seeds[0, 0] = 0x8880, 65535          # the most negative coefficients
    w = K.SeedWeight3([m])
    ref = B.decode3_rows_f32(m)
    assert np.array_equal(K.kt_decode3(w).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(K.kt_decode3(w, bf16=True), B.f2bf(ref).reshape(R, Kc))


def test_p3_decode_reference_fixture(K):
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "seed4_p3_golden.npz"))
    rows, Kc, eb = (int(v) for v in g["row_shape"])
    m = B.Matrix3(rows, Kc, 0, eb=eb)
    m.seeds, m.nibs = g["row_seeds"], g["row_nibs"]
    assert np.array_equal(K.kt_decode3(K.SeedWeight3([m])).view(np.uint32), g["row_f32"].view(np.uint32))


@pytest.mark.parametrize("Kc", [256, 512, 72, 2048])
def test_p3_dense_tokens_add_and_batch_invariance(K, Kc):
    R = 24
    m = B.Matrix3(R, Kc, 3 * Kc, eb=-20)
    w, W = K.SeedWeight3([m]), exact(m)
    rng = np.random.default_rng(Kc)
    x = B.bfr(rng.random((8, Kc), np.float32) * 2 - 1)
    first = None
    for T in range(1, 9):
        add = int(T == 3)
        y0 = B.bfr(rng.random((T, R), np.float32) * 2 - 1)
        y = K.kt_mv3(w, x[:T], T, add, y0 if add else None)
        acc = x[:T].astype(np.float64) @ W.T
        mag = np.abs(x[:T].astype(np.float64)) @ np.abs(W.T)
        ref = B.bfr(y0 + B.bfr(acc.astype(np.float32))) if add else B.bfr(acc.astype(np.float32))
        bound = np.abs(ref) / 128 + F32B * mag * (2 if add else 1) + 1e-30
        assert (np.abs(y - ref) <= bound).all(), (T, float(np.max(np.abs(y - ref) / bound)))
        if T == 1:
            first = y[0].copy()
        elif not add:
            assert np.array_equal(y[0], first)


def test_p3_gather_and_gate_up(K):
    R, Kc, S = 24, 512, 3
    mats = [B.Matrix3(R, Kc, 40 + s, eb=-19 - s) for s in range(S)]
    mu = [B.Matrix3(R, Kc, 60 + s, eb=-21 + s) for s in range(S)]
    w, wu = K.SeedWeight3(mats), K.SeedWeight3(mu)
    sel = [2, 0, 1, 2, 1, 0]
    x = B.bfr(np.random.default_rng(2).random((3, Kc), np.float32) * 2 - 1)
    y = K.kt_mv3_sel(w, sel, 2, x)
    a = K.kt_mv3_gu(w, wu, sel, 2, x)
    for p, e in enumerate(sel):
        xr = x[p // 2].astype(np.float64)
        g, u = exact(mats[e]) @ xr, exact(mu[e]) @ xr
        mg, mu_ = np.abs(exact(mats[e])) @ np.abs(xr), np.abs(exact(mu[e])) @ np.abs(xr)
        ref = B.bfr(g.astype(np.float32))
        assert (np.abs(y[p] - ref) <= np.abs(ref) / 128 + F32B * mg + 1e-30).all()
        gb, ub = B.bfr(g.astype(np.float32)).astype(np.float64), B.bfr(u.astype(np.float32)).astype(np.float64)
        silu = B.bfr(gb.astype(np.float32) * B.bfr(1.0 / (1.0 + np.exp(-gb)).astype(np.float32)))
        want = B.bfr(silu * ub.astype(np.float32))
        # within one bf16 flip of g or u (each moves the product by about one part in 128) plus the accumulation slack
        slack = np.abs(want) / 32 + 4 * F32B * (mg * np.abs(ub) + mu_ * np.abs(silu)) + 1e-6
        assert (np.abs(a[p] - want) <= slack).all(), float(np.max(np.abs(a[p] - want) / slack))


@pytest.mark.parametrize("exact_mode", [False, True])
@pytest.mark.parametrize("R,Kc,T", [(40, 128, 45), (300, 512, 130), (24, 72, 5)])
def test_p3_gemm_dense(K, exact_mode, R, Kc, T):
    """kc_mm / kc_mm_packed with MF_SEED4: seed weights rounded to bf16 (default) or exact (three terms), the reference's bound
    for its GEMM (tests/test_mova_kernels.c:246-317)."""
    m = B.Matrix3(R, Kc, 7 * R + Kc, eb=-20)
    w = K.SeedWeight3([m])
    W = exact(m) if exact_mode else B.bfr(B.decode3_rows_f32(m)).astype(np.float64)
    rng = np.random.default_rng(T)
    x = B.bfr(rng.standard_normal((T, Kc)).astype(np.float32))
    y0 = B.bfr(rng.standard_normal((T, R)).astype(np.float32))
    acc, mag = x.astype(np.float64) @ W.T, np.abs(x.astype(np.float64)) @ np.abs(W.T)
    y = K.kt_mm(w, x, T, add=1, y0=y0, exact=exact_mode)
    ref = B.bfr(y0 + B.bfr(acc.astype(np.float32))).astype(np.float64)
    assert (np.abs(y - ref) <= np.abs(ref) / 128 + 2 * F32B * mag + np.abs(acc) / 128 + 1e-30).all()
    y2 = K.kt_mm(w, x, T, exact=exact_mode, packed=not exact_mode)
    ref2 = B.bfr(acc.astype(np.float32)).astype(np.float64)
    assert (np.abs(y2 - ref2) <= np.abs(ref2) / 128 + F32B * mag + 1e-30).all()


@pytest.mark.parametrize("mode", ["host", "dev", "packed"])
def test_p3_gemm_grouped(K, mode):
    R, Kc, S, P, xdiv = 40, 128, 3, 50, 2
    mats = [B.Matrix3(R, Kc, 90 + s, eb=-19 - s) for s in range(S)]
    w = K.SeedWeight3(mats)
    x = B.bfr(np.random.default_rng(5).standard_normal((25, Kc)).astype(np.float32))
    slc = [(p * 7) % S for p in range(P)]
    perm, tiles = [], []
    for s in range(S):
        st = len(perm)
        perm += [p for p in range(P) if slc[p] == s]
        for o in range(st, len(perm), 128):
            tiles.append((s, o, min(128, len(perm) - o)))
    y = K.kt_mm_grouped(w, P, xdiv, perm, tiles, x, mode=mode)
    for p in range(P):
        Wp = B.bfr(B.decode3_rows_f32(mats[slc[p]])).astype(np.float64)
        xr = x[p // xdiv].astype(np.float64)
        ref = B.bfr((Wp @ xr).astype(np.float32)).astype(np.float64)
        assert (np.abs(y[p] - ref) <= np.abs(ref) / 128 + F32B * (np.abs(Wp) @ np.abs(xr)) + 1e-30).all(), p


@pytest.mark.parametrize("R,Kc", [(512, 2048), (2048, 512), (96, 64)])
def test_p3_gathers_at_config1_sizes(K, R, Kc):
    """The tuned pair kernel's P = 3 form at the routed experts' shapes: 20 pairs over 5 slices, the gather and gate+up forms
    against the exact weights; a pair's row must not depend on the list it is part of."""
    S, xdiv = 5, 4
    mats = [B.Matrix3(R, Kc, 300 + s, eb=-20 - s % 3) for s in range(S)]
    mu = [B.Matrix3(R, Kc, 400 + s, eb=-21 + s % 2) for s in range(S)]
    w, wu = K.SeedWeight3(mats), K.SeedWeight3(mu)
    rng = np.random.default_rng(R)
    sel = rng.integers(0, S, 20)
    x = B.bfr(rng.standard_normal((5, Kc)).astype(np.float32))
    y = K.kt_mv3_sel(w, sel, xdiv, x)
    a = K.kt_mv3_gu(w, wu, sel, xdiv, x)
    Wg, Wu = [exact(m) for m in mats], [exact(m) for m in mu]
    for p, e in enumerate(sel):
        xr = x[p // xdiv].astype(np.float64)
        g, u = Wg[e] @ xr, Wu[e] @ xr
        mg, mu_ = np.abs(Wg[e]) @ np.abs(xr), np.abs(Wu[e]) @ np.abs(xr)
        ref = B.bfr(g.astype(np.float32))
        assert (np.abs(y[p] - ref) <= np.abs(ref) / 128 + F32B * mg + 1e-30).all(), p
        gb, ub = B.bfr(g.astype(np.float32)).astype(np.float64), B.bfr(u.astype(np.float32)).astype(np.float64)
        silu = B.bfr(gb.astype(np.float32) * B.bfr(1.0 / (1.0 + np.exp(-gb)).astype(np.float32)))
        want = B.bfr(silu * ub.astype(np.float32))
        slack = np.abs(want) / 32 + 4 * F32B * (mg * np.abs(ub) + mu_ * np.abs(silu)) + 1e-6
        assert (np.abs(a[p] - want) <= slack).all(), p
    alone = K.kt_mv3_sel(w, sel[7:8], 1, x[7 // xdiv:7 // xdiv + 1])
    assert np.array_equal(alone[0].view(np.uint32), y[7].view(np.uint32))
