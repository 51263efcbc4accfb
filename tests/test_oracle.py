"""The CPU oracle against the reference's known answers and against fixtures produced by the reference's own code
(tests/golden/make_golden.py).  No GPU."""
import ctypes as C

import numpy as np
import pytest


def test_period_and_first_states(oracle):
    # reference: tests/test_lfsr.c:15-30
    assert oracle.lib().orc_period() == 65535
    assert list(oracle.states(1, 6)) == [0x8000, 0x4000, 0x2000, 0x1000, 0x8800, 0x4400]
    assert oracle.states(0xACE1, 1)[0] != 0xACE1


def test_fnv_golden_over_all_seeds(oracle):
    # reference: tests/test_lfsr.c:41-56
    assert oracle.lib().orc_fnv24_all_seeds() == 0x740E86E513D34463


def test_stream_table_linear_and_windows(oracle):
    # reference: tests/test_lfsr.c:87-93; window rule nslm/lib_rows.c:59,71
    t = oracle.table32()
    s = np.arange(65536)
    assert np.array_equal(t[s], t[s & 0xFF] ^ t[s & 0xFF00])
    for seed in (1, 0xACE1, 65535, 777):
        st = oracle.states(seed, 32)
        win = seed | (int(t[seed]) << 16)
        assert all(((win >> k) & 0xFFFF) == st[k - 1] for k in range(1, 33))


def test_states_match_reference_fixture(oracle, golden):
    for i, seed in enumerate(golden["st_seeds"]):
        assert np.array_equal(oracle.states(int(seed), 48), golden["states"][i])
        assert int(oracle.table32()[int(seed)]) == int(golden["stream"][i])


def test_block_decode_matches_reference_fixture(oracle, golden):
    for i in range(len(golden["blk_seed"])):
        got = oracle.decode_block_bf16(int(golden["blk_seed"][i]), int(golden["blk_coef"][i]), int(golden["blk_e"][i]))
        assert np.array_equal(got, golden["blk_bf16"][i]), i


def test_block_decode_against_double(oracle):
    # reference: tests/test_search4.c:38-56
    rng = np.random.default_rng(3)
    r32 = np.float32(1.0) / np.float32(32767.0)
    for it in range(500):
        seed, coef, e = int(rng.integers(1, 65536)), int(rng.integers(0, 65536)), -20 + it % 9
        st = oracle.states(seed, 32).astype(np.int64)
        q = [oracle.lib().orc_q4(C.c_uint16(coef), p) for p in range(4)]
        want = []
        for c in range(8):
            isum = sum((int(st[4 * c + p]) - 32768) * q[p] for p in range(4))
            w = np.float32(isum) * (r32 * np.float32(2.0 ** e))
            u = int(np.float32(w).view(np.uint32))
            u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFFFFFF
            want.append(u >> 16)
        assert list(oracle.decode_block_bf16(seed, coef, e)) == want


def test_rows_match_reference_fixture_mid_byte_rows(oracle, golden):
    rows, K, eb = (int(v) for v in golden["row_shape"])
    m = oracle.Matrix(rows, K, 0, eb=eb)
    m.seeds[:], m.coefs[:], m.codes[:] = golden["row_seeds"], golden["row_coefs"], golden["row_codes"]
    w = oracle.decode_rows_f32(m)
    assert np.array_equal(w.view(np.uint32), golden["row_f32"].view(np.uint32))
    bf = oracle.decode_rows_bf16(m)
    u = golden["row_f32"].view(np.uint32).astype(np.uint64)
    assert np.array_equal(bf, ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16))


def test_route_matches_reference_fixture(oracle, golden):
    # reference: tests/test_qwen4_kernels.c:223-245 (the tie goes to the higher expert: 300 before 7)
    ind, wt = oracle.route(golden["route_logits"], 10)
    assert np.array_equal(ind, golden["route_ind"]) and ind[0, 0] == 300 and ind[0, 1] == 7
    assert np.array_equal(wt, golden["route_wt"])


def test_against_reference_library_when_built(oracle):
    R = oracle.ref()
    if R is None:
        pytest.skip("oracle/_ref not built here (it needs the reference tree)")
    rng = np.random.default_rng(11)
    u16p = C.POINTER(C.c_uint16)
    for _ in range(3000):
        seed, coef, e = int(rng.integers(1, 65536)), int(rng.integers(0, 65536)), int(rng.integers(-30, 1))
        o = np.zeros(8, np.uint16)
        R.ref_decode_block(C.c_uint16(seed), C.c_uint16(coef), e, o.ctypes.data_as(u16p))
        assert np.array_equal(o, oracle.decode_block_bf16(seed, coef, e))


def test_bucket_grouping(oracle):
    # reference: tests/test_qwen4_engine.c:34-61 (skewed selections, half on expert 0)
    for n, rows, k in ((128, 512, 10), (64, 128, 8)):
        P = rows * k
        x = 12345
        inds = np.zeros(P, np.int32)
        for i in range(P):
            x = (x * 1664525 + 1013904223) & 0xFFFFFFFF
            inds[i] = ((x >> 8) % n) * ((x >> 4) & 1)
        perm, tiles = oracle.bucket(inds, n)
        at = 0
        ti = 0
        for e in range(n):
            ids = np.nonzero(inds == e)[0]
            assert np.array_equal(perm[at:at + len(ids)], ids)
            for s in range(at, at + len(ids), 128):
                assert tiles[ti] == (e, s, min(128, at + len(ids) - s))
                ti += 1
            at += len(ids)
        assert ti == len(tiles)


def test_rounding_points(oracle):
    g = np.array([0.5, -1.25, 3.0, 0.0], np.float32)
    u = np.array([2.0, 0.5, -1.0, 7.0], np.float32)
    a = oracle.swiglu(g, u)
    oracle.lib().orc_bfr.restype = C.c_float
    oracle.lib().orc_bfr.argtypes = [C.c_float]
    for i in range(4):
        s = np.float32(oracle.lib().orc_silu_bf(C.c_float(float(g[i]))))
        assert a[i] == np.float32(oracle.lib().orc_bfr(C.c_float(float(s * u[i]))))
    assert a[3] == 0.0 and a[0] > 0
    m = oracle.Matrix(24, 256, 5, eb=-19)
    x = oracle.normal(1, 256, bf16=True)
    y64, _ = oracle.matvec_f64(m, x)
    y = oracle.mv(m, x)
    assert np.all(np.abs(y[0] - y64[0]) <= np.abs(y64[0]) / 128 + 1e-30)   # one bf16 ulp
    assert np.array_equal(y.view(np.uint32) & 0xFFFF, np.zeros_like(y.view(np.uint32)))


def test_mova_router_against_the_double_form(oracle):
    """The oracle's MoVA router against the double-precision form the reference's kernel test checks its backends with
    (tests/test_mova_kernels.c:386-411): n 20, top 4, two partitions, BF16 weights and bias, scale 2.5."""
    rng = np.random.default_rng(11)
    d, n, k, T = 512, 20, 4, 6
    W = oracle.f2bf((rng.random((n, d), np.float32) * 2 - 1) * 0.05)
    bias = oracle.f2bf((rng.random(n, np.float32) * 2 - 1) * 0.01)
    x = rng.standard_normal((T, d)).astype(np.float32)
    score, sel, ind, wt = oracle.mova_router(W, bias, x, k, d // 2, 2.5)
    Wf = (W.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    bf = (bias.astype(np.uint32) << 16).view(np.float32).astype(np.float64)

    def bfr(v):
        return (oracle.f2bf(np.asarray(v, np.float32)).astype(np.uint32) << 16).view(np.float32).astype(np.float64)

    for t in range(T):
        s0 = Wf[:, :d // 2] @ x[t, :d // 2].astype(np.float64)
        s1 = Wf[:, d // 2:] @ x[t, d // 2:].astype(np.float64)
        sc = 1 / (1 + np.exp(-(bfr(s0) + bfr(s1))))
        se = sc + bf
        chosen = []
        for _ in range(k):
            best = -1
            for e in range(n):
                if e not in chosen and (best < 0 or se[e] > se[best]):
                    best = e
            chosen.append(best)
        assert list(ind[t]) == chosen
        assert np.abs(wt[t] - sc[chosen] / sc[chosen].sum() * 2.5).max() < 1e-5


def test_mova_topk_ties_go_to_the_lowest_id(oracle):
    sc = np.full((1, 8), 0.5, np.float32)
    se = np.array([[0.25, 0.5, 0.5, 0.125, 0.5, 0.25, 0.75, 0.75]], np.float32)
    ind, wt = oracle.mova_topk(sc, se, 5, 2.0)
    assert list(ind[0]) == [6, 7, 1, 2, 4]
    assert np.allclose(wt[0], 0.4)
    g = oracle.softplus_gate(np.array([0.0, 3.0, -3.0], np.float32))
    assert g[0] == 1.0 and g[1] > 3.0 and 0 < g[2] < 0.2   # softplus with beta ln 2: 1 at 0, ~x for large x


def test_q4_reference_form(oracle):
    """The oracle's affine int4 mat-vec against a direct numpy statement of weight = s q + b per group of 64."""
    rng = np.random.default_rng(5)
    R, K, T = 6, 128, 2
    codes = rng.integers(0, 2 ** 32, (R, K // 8), dtype=np.uint64).astype(np.uint32)
    s = oracle.f2bf(rng.random((R, K // 64), np.float32) * 0.02 + 0.001)
    b = oracle.f2bf(rng.random((R, K // 64), np.float32) * -0.2)
    x = rng.standard_normal((T, K)).astype(np.float32)
    q = ((codes[:, :, None] >> (4 * np.arange(8, dtype=np.uint32))) & 15).reshape(R, K).astype(np.float64)
    tof = lambda h: (h.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    w = np.repeat(tof(s), 64, axis=1) * q + np.repeat(tof(b), 64, axis=1)
    want = x.astype(np.float64) @ w.T
    y, mag = oracle.q4_mv(codes, s, b, x)
    assert np.all(np.abs(y - want) <= np.abs(want) / 128 + 1e-12)       # the oracle rounds to bf16
    assert np.allclose(mag, np.abs(x.astype(np.float64)) @ np.abs(w.T))
    out, prob = oracle.argmax(np.array([[0.0, 2.0, 2.0, -1.0]], np.float32))
    assert out[0] == 1 and abs(prob[0] - 1 / (2 + np.exp(-2) + np.exp(-3))) < 1e-12


def test_p3_decode_matches_reference_fixture(oracle):
    """P = 3 (SEED4) blocks and rows against outputs of the reference's own code (tests/golden/make_golden_p3.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "seed4_p3_golden.npz"))
    for i in range(len(g["blk_seed"])):
        got = oracle.decode3_block_bf16(g["blk_seed"][i], g["blk_nib"][i], g["blk_bias"][i])
        assert np.array_equal(got, g["blk_bf16"][i]), i
    rows, K, eb = (int(v) for v in g["row_shape"])
    m = oracle.Matrix3(rows, K, 0, eb=eb)
    m.seeds, m.nibs = g["row_seeds"], g["row_nibs"]
    assert np.array_equal(oracle.decode3_rows_f32(m).view(np.uint32), g["row_f32"].view(np.uint32))


def test_kv_q8_cache_follows_the_reference_tests_quantizer(oracle):
    """tests/test_mova_kernels.c:584-604: per (row, head) scale = max|x| / 127 (1 for a zero row), code = lrintf(x / scale),
    and the values a kernel reads from the cache are bf16(code * scale)."""
    rng = np.random.default_rng(8)
    bits = oracle.f2bf((rng.random((40, 2, 128), np.float32) * 2 - 1) * 2)
    bits[5, 1] = 0                                                      # a zero row: scale 1, codes 0
    x = (bits.astype(np.uint32) << 16).view(np.float32)
    codes, sc, deq = oracle.kv_q8_cache(bits)
    assert codes.dtype == np.int8 and sc.dtype == np.float32 and deq.dtype == np.uint16 and deq.shape == bits.shape
    assert sc[5, 1] == 1 and not codes[5, 1].any() and not deq[5, 1].any()
    m = np.abs(x).max(-1)
    live = m > 0
    assert np.array_equal(sc[live], (m[live] / np.float32(127)).astype(np.float32))
    assert np.abs(codes.astype(np.int32)).max() == 127                   # every live row reaches +-127 at its largest value
    for r, h in [(0, 0), (7, 1), (39, 0)]:                               # scalar restatement of the C loop
        for e in range(128):
            q = int(np.rint(np.float32(x[r, h, e]) / sc[r, h]))
            assert q == codes[r, h, e]
            assert oracle.f2bf(np.float32(np.float32(q) * sc[r, h]))[()] == deq[r, h, e]
    back = (deq.astype(np.uint32) << 16).view(np.float32)
    assert np.all(np.abs(back - x) <= sc[..., None] / 2 + np.abs(x) / 256 + 1e-30)   # half a step + the BF16 rounding


def test_attn_decode_reference_form(oracle):
    """The double-precision statement the attention kernels are compared with (tests/test_mova_kernels.c:690-712): one head
    against an explicit loop, the GQA head -> KV head map, and the gate's two roundings."""
    rng = np.random.default_rng(2)
    nh, nkv, NP = 4, 2, 50
    q = oracle.bfr(rng.standard_normal((2, nh, 128)).astype(np.float32))
    g = oracle.bfr(rng.standard_normal((2, nh, 128)).astype(np.float32))
    Kc = oracle.f2bf(rng.standard_normal((NP, nkv, 128)).astype(np.float32))
    Vc = oracle.f2bf(rng.standard_normal((NP, nkv, 128)).astype(np.float32))
    K = (Kc.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    V = (Vc.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    pos, kv0, scale = [20, 0], [3, 40], np.float32(1 / np.sqrt(128.0))
    out, att = oracle.attn_decode(q, Kc, Vc, pos, kv0, nkv, scale, g)
    t, h = 0, 3
    kvh = h // (nh // nkv)
    s = np.array([np.dot(q[t, h].astype(np.float64) * np.float64(scale), K[kv0[t] + p, kvh]) for p in range(pos[t] + 1)])
    w = np.exp(s - s.max())
    ref = sum(w[p] / w.sum() * V[kv0[t] + p, kvh] for p in range(pos[t] + 1))
    assert np.allclose(att[t, h], ref, rtol=1e-12, atol=1e-14)
    assert np.array_equal(att[1, 0], V[40, 0])                            # a row at position 0 returns its only value row
    want = oracle.bfr(oracle.bfr(att.astype(np.float32)) * oracle.softplus_gate(g))
    assert np.array_equal(out.view(np.uint32), want.view(np.uint32))
    plain, _ = oracle.attn_decode(q, Kc, Vc, pos, kv0, nkv, scale, None)
    assert np.array_equal(plain.view(np.uint32), oracle.bfr(att.astype(np.float32)).view(np.uint32))
