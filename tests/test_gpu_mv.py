"""Parity of the CUDA seed mat-vec kernels with the CPU oracle, called through the C ABI.

Bars: decoded weights bit-exact; mat-vec results within one bf16 ulp plus the f32 accumulation bound the reference's
own kernel tests use (64 * 1.2e-7 * sum|w x|, tests/test_mova_kernels.c:27-30,171), and raw f32 results within
2e-6 * sum|w x| of the double-precision spec (tests/test_cpu_seed4.c:182-195; well inside the 1e-3 relative bar)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

F32B = 64 * 1.2e-7


def bfr(oracle, a):
    import ctypes as C
    a = np.asarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def close_bf(got, ref, extra):
    return np.abs(got.astype(np.float64) - ref) <= np.abs(ref) / 128.0 + 1e-30 + extra


def weights(oracle, S, R, K, seed, ebs=(-19, -17, -21, -22, -20)):
    from nanoseedlm_b200 import kernels
    mats = [oracle.Matrix(R, K, seed * 100 + s, eb=ebs[s % len(ebs)]) for s in range(S)]
    return mats, kernels.SeedWeight.from_matrices(mats)


@pytest.mark.parametrize("R,K", [(24, 256), (7, 72), (40, 128), (512, 2048), (33, 4096), (5, 8)])
def test_decode_bit_exact(oracle, R, K):
    from nanoseedlm_b200 import kernels
    mats, w = weights(oracle, 2, R, K, 1)
    for s in range(2):
        f = kernels.kt_decode(w, s)
        assert np.array_equal(f.view(np.uint32), oracle.decode_rows_f32(mats[s]).view(np.uint32))
        b = kernels.kt_decode(w, s, bf16=True)
        assert np.array_equal(b, oracle.decode_rows_bf16(mats[s]))


def test_decode_matches_reference_fixture(oracle, golden):
    from nanoseedlm_b200 import kernels
    rows, K, eb = (int(v) for v in golden["row_shape"])
    w = kernels.SeedWeight(golden["row_seeds"][None], golden["row_coefs"][None], golden["row_codes"][None], [eb], rows, K)
    assert np.array_equal(kernels.kt_decode(w).view(np.uint32), golden["row_f32"].view(np.uint32))


def test_decode_every_seed_and_coefficient(oracle):
    """All 65535 seeds once, every coefficient nibble value and exponent code: the format lock of the device decode."""
    from nanoseedlm_b200 import kernels
    R, K = 64, 8192   # 65536 blocks
    m = oracle.Matrix(R, K, 0, eb=-24)
    n = R * K // 8
    m.seeds[:] = (np.arange(n) % 65535 + 1).astype(np.uint16)
    m.coefs[:] = (np.arange(n) * 40503 % 65536).astype(np.uint16)
    w = kernels.SeedWeight.from_matrices([m])
    assert np.array_equal(kernels.kt_decode(w).view(np.uint32), oracle.decode_rows_f32(m).view(np.uint32))


@pytest.mark.parametrize("K", [256, 512, 2048, 4096, 72, 640])
def test_mv_dense_tokens_add_and_batch_invariance(oracle, K):
    # reference: tests/test_mova_kernels.c:160-201 (R 24, T 1..8, residual add at T = 3, token 0 equals T = 1)
    from nanoseedlm_b200 import kernels
    R = 24
    mats, w = weights(oracle, 1, R, K, K)
    x = oracle.normal(K + 1, 8 * K, bf16=True).reshape(8, K)
    y64, mag = oracle.matvec_f64(mats[0], x, T=8)
    y1 = None
    for T in range(1, 9):
        add = int(T == 3)
        y0 = oracle.normal(T, T * R, bf16=True).reshape(T, R)
        y = kernels.kt_mv(w, x[:T], T, add=add, y0=y0 if add else None)
        if T == 1:
            y1 = y.copy()
        elif not add:
            assert np.array_equal(y[0].view(np.uint32), y1[0].view(np.uint32)), f"token 0 of T={T} differs from T=1"
        acc = bfr(oracle, y64[:T].astype(np.float32))
        ref = bfr(oracle, y0 + acc).astype(np.float64) if add else bfr(oracle, y64[:T].astype(np.float32)).astype(np.float64)
        ok = close_bf(y, ref, F32B * mag[:T] * (2 if add else 1))
        assert ok.all(), (T, np.argwhere(~ok)[:4])


@pytest.mark.parametrize("R,K", [(24, 256), (24, 512), (2048, 512), (512, 2048), (24, 136)])
def test_mv_gather(oracle, R, K):
    # reference: tests/test_mova_kernels.c:203-220 (6 pairs, xdiv 2)
    from nanoseedlm_b200 import kernels
    mats, w = weights(oracle, 3, R, K, R + K)
    sel = [2, 0, 1, 2, 1, 0]
    x = oracle.normal(9, 3 * K, bf16=True).reshape(3, K)
    y = kernels.kt_mv_sel(w, sel, 2, x)
    yr = kernels.kt_mv_sel(w, sel, 2, x, raw=True)
    for p, s in enumerate(sel):
        y64, mag = oracle.matvec_f64(mats[s], x[p // 2])
        assert close_bf(y[p], bfr(oracle, y64[0].astype(np.float32)).astype(np.float64), F32B * mag[0]).all()
        assert np.max(np.abs(yr[p] - y64[0]) / mag[0]) < 2e-6


@pytest.mark.parametrize("R,K", [(24, 256), (24, 512), (512, 2048), (24, 72)])
def test_mv_gate_up_swiglu(oracle, R, K):
    # reference: tests/test_mova_kernels.c:221-243 (within one bf16 flip of g or u)
    from nanoseedlm_b200 import kernels
    mg, wg = weights(oracle, 2, R, K, 3 * R + K)
    mu, wu = weights(oracle, 2, R, K, 5 * R + K)
    sel = [1, 0, 1, 1, 0, 0]
    x = oracle.normal(21, 3 * K, bf16=True).reshape(3, K)
    a = kernels.kt_mv_gu(wg, wu, sel, 2, x)
    for p, s in enumerate(sel):
        g64, _ = oracle.matvec_f64(mg[s], x[p // 2])
        u64, _ = oracle.matvec_f64(mu[s], x[p // 2])
        gg = bfr(oracle, g64[0].astype(np.float32)).astype(np.float64)
        uu = bfr(oracle, u64[0].astype(np.float32)).astype(np.float64)
        ref = oracle.mv_gu(mg[s], mu[s], x[p // 2]).astype(np.float64)
        slack = (np.abs(uu) * (np.abs(gg) + 1) + np.abs(gg) * np.abs(uu)) / 128 + 1e-7
        assert close_bf(a[p], ref, slack).all()
        exact = np.mean(a[p] == ref.astype(np.float32))
        assert exact > 0.9   # nearly every output is the oracle's value bit for bit


def test_config0_matvec_against_cpu_path(oracle):
    """BASELINE config 0: N = 2048 outputs x K = 4096 inputs, M = 1, fp32 x ~ N(0,1): decoded W bit-exact, y within
    1e-3 relative (measured against |y| with the sum|w x| floor of the reference's tests)."""
    from nanoseedlm_b200 import kernels
    m = oracle.Matrix(2048, 4096, 42, eb=-22)
    w = kernels.SeedWeight.from_matrices([m])
    x = oracle.normal(43, 4096)
    assert np.array_equal(kernels.kt_decode(w).view(np.uint32), oracle.decode_rows_f32(m).view(np.uint32))
    y = kernels.kt_mv(w, x, 1, raw=True)[0]
    y64, mag = oracle.matvec_f64(m, x)
    ycpu = oracle.cpu_seed4_matvec(m, x, threads=4)
    assert np.max(np.abs(y - y64[0]) / mag[0]) < 2e-6
    big = np.abs(y64[0]) > 1e-3 * mag[0]
    assert np.max(np.abs(y[big] - y64[0][big]) / np.abs(y64[0][big])) < 1e-3
    assert np.max(np.abs(y - ycpu) / mag[0]) < 4e-6


def test_other_formats_are_refused_loudly(oracle):
    import ctypes as C
    import torch
    from nanoseedlm_b200 import kernels, lib
    mats, w = weights(oracle, 1, 8, 64, 2)
    x = torch.zeros(64, device="cuda")
    y = torch.zeros(8, device="cuda")
    lib.load().kc_mv(None, 2, w.slice(0), 64, 8, C.c_void_p(x.data_ptr()), 64, C.c_void_p(y.data_ptr()), 8, 1, 0,
                     C.c_void_p(kernels.stream_table().data_ptr()))      # 2 = MF_Q8
    assert "format 2" in lib.last_error()


@pytest.mark.parametrize("R,K,S,P", [(96, 2048, 5, 23), (512, 2048, 12, 64), (2048, 512, 12, 64), (40, 64, 3, 9), (64, 256, 20, 20),
                                     (96, 2048, 5, 200), (256, 512, 40, 330), (16, 128, 7, 1300)])
def test_pairs_that_share_a_slice_share_its_expansion_and_change_nothing(oracle, R, K, S, P):
    """Lists of more than 64 pairs are sorted by slice and a slice's rows expanded once for two pairs at a time (shorter lists
    run pair by pair, lists of more than 1024 pairs ungrouped).  Every pair's row must equal the same pair computed ALONE, bit for bit, whatever pairs share
    the call: for the gate+up form (f32 and packed bf16 inputs, input row by pair / xdiv or by a row index, a device-side
    pair count) and the gather form (rounded and raw)."""
    from nanoseedlm_b200 import kernels
    mats, w = weights(oracle, S, R, K, 11 * R + K, ebs=tuple(-22 + (i % 5) for i in range(S)))
    _, w2 = weights(oracle, S, R, K, 13 * R + K, ebs=tuple(-21 + (i % 4) for i in range(S)))
    rng = np.random.default_rng(P)
    for sel in (rng.integers(0, S, P), np.zeros(P, np.int64) + (S - 1), np.arange(P) % S):
        xdiv = 4
        x = oracle.normal(31 + P, ((P + xdiv - 1) // xdiv) * K, bf16=True).reshape(-1, K)
        sample = sorted(set(rng.integers(0, P, 12).tolist() + [0, P - 1]))
        gu = kernels.kt_mv_gu(w, w2, sel, xdiv, x)
        for p in sample:      # the pair alone: one pair, its slice, its input row
            alone = kernels.kt_mv_gu(w, w2, [sel[p]], 1, x[p // xdiv])
            assert np.array_equal(gu[p].view(np.uint32), alone[0].view(np.uint32)), (p, sel[p])
        xrow = rng.integers(0, x.shape[0], P)
        ref = kernels.kt_mv_gu(w, w2, sel, 1, x[xrow])
        assert np.array_equal(kernels.kt_mv_gu_rows(w, w2, sel, xrow, x), ref)
        assert np.array_equal(kernels.kt_mv_gu_rows(w, w2, sel, xrow, x, bf16=True), ref)   # inputs are bf16 values
        part = kernels.kt_mv_gu_rows(w, w2, sel, xrow, x, count=P // 2)                     # only the first P // 2 pairs are valid
        assert np.array_equal(part[:P // 2], ref[:P // 2]) and not part[P // 2:].any()
        xp = oracle.normal(41 + P, P * K, bf16=True).reshape(P, K)
        dn, dn_raw = kernels.kt_mv_sel(w, sel, 1, xp), kernels.kt_mv_sel(w, sel, 1, xp, raw=True)
        for p in sample:
            assert np.array_equal(dn[p], kernels.kt_mv_sel(w, [sel[p]], 1, xp[p])[0])
            assert np.array_equal(dn_raw[p], kernels.kt_mv_sel(w, [sel[p]], 1, xp[p], raw=True)[0])


@pytest.mark.parametrize("T,E,k,R,K", [(1, 128, 8, 64, 2048), (8, 128, 8, 64, 2048), (5, 512, 10, 48, 512), (3, 40, 1, 24, 256), (8, 1024, 32, 8, 64)])
def test_router_folded_into_the_gate_up_kernel(oracle, T, E, k, R, K):
    """nsl_mv_gu_routed = the router + kc_mv_gu in one launch: ids identical to the oracle's, weights and activations
    identical to the two separate calls."""
    from nanoseedlm_b200 import kernels
    S = min(E, 24)      # experts draw their matrices from a pool (ids stay the router's)
    pool, _ = weights(oracle, S, R, K, 17 * R + K)
    pool2, _ = weights(oracle, S, R, K, 19 * R + K)
    wg = kernels.SeedWeight.from_matrices([pool[e % S] for e in range(E)])
    wu = kernels.SeedWeight.from_matrices([pool2[e % S] for e in range(E)])
    logits = oracle.normal(7 * T + E, T * E).reshape(T, E)
    x = oracle.normal(9 * T + E, T * K, bf16=True).reshape(T, K)
    a, ind, wt = kernels.kt_mv_gu_routed(wg, wu, logits, k, x)
    ri, rw = oracle.route(logits, k)
    i2, w2 = kernels.kt_route(logits, k)
    assert np.array_equal(ind, ri) and np.array_equal(ind, i2) and np.array_equal(wt, w2)
    assert np.max(np.abs(wt - rw) / rw) < 1e-5
    assert np.array_equal(a, kernels.kt_mv_gu(wg, wu, ind.ravel(), k, x))


def test_misaligned_streams_of_a_dense_slice_take_the_any_shape_kernel(oracle):
    """A dense call whose streams do not start on the boundaries the chunked kernels' 16-byte loads need (a slice cut out of
    a larger buffer at an odd offset) is served by the any-shape kernel: same results as the aligned copy."""
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    mats, w = weights(oracle, 1, 40, 256, 3)
    x = oracle.normal(77, 256, bf16=True)
    want = kernels.kt_mv(w, x, 1, raw=True)
    nb = 40 * 256 // 8
    seeds = torch.zeros(nb + 8, dtype=torch.int16, device="cuda")
    seeds[1:nb + 1] = w.seeds[0]                                   # two bytes off a 16-byte boundary
    sl = w.slice(0)
    sl.p[0] = seeds.data_ptr() + 2
    xd, yd = kernels.dev(x.reshape(1, 256)), torch.zeros(1, 40, device="cuda")
    one = (L.WSlice * 1)(sl)
    import ctypes as C
    L.load().nsl_mv_raw(None, C.cast(one, C.c_void_p), 256, 40, C.c_void_p(xd.data_ptr()), 256, C.c_void_p(yd.data_ptr()), 40, None, 1, 1,
                        C.c_void_p(kernels.stream_table().data_ptr()))
    torch.cuda.synchronize()
    L.check()
    y64, mag = oracle.matvec_f64(mats[0], x)
    assert np.max(np.abs(yd.cpu().numpy()[0] - y64[0]) / mag[0]) < 2e-6 and np.max(np.abs(want[0] - y64[0]) / mag[0]) < 2e-6
