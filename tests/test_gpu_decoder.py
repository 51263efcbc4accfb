"""The whole decoder step (include/nslm_decoder.h) on a small configuration against a host reference composed of the CPU
oracle's pieces -- grouped RMSNorm, dense seed mat-vecs, RoPE + cache write, decode attention (double precision), router,
routed and shared experts, combine, residual adds, the affine-int4 head, arg-max -- with the engine's bf16 rounding points;
three steps in a row so that later steps attend the keys earlier steps wrote.  Also: the small kernels alone (kc_gnorm,
kc_rope_kv with BF16 and 8-bit caches, kc_embed), the decoder with its routed experts behind a one-rank peer-memory window,
and a step of more than MV_MAXT rows (the tensor-core path of the dense projections)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

EPS, THETA = 1e-6, 1e6


def bfr(a):
    a = np.asarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def bf_bits(a):
    return (bfr(a).view(np.uint32) >> 16).astype(np.uint16)


def bf_val(b):
    return (np.asarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def gnorm(x, w):
    x = np.asarray(x, np.float32)
    hw = x.shape[-1] // 2
    out = np.empty_like(x)
    for g in (slice(0, hw), slice(hw, None)):
        r = (1.0 / np.sqrt((x[..., g].astype(np.float64) ** 2).mean(-1, keepdims=True) + EPS)).astype(np.float32)
        out[..., g] = bfr(bf_val(w[g]) * (x[..., g] * r))
    return out


def rope(vec, pos):
    """vec [..., 128] -> rotated, pairs (p, p + 64)."""
    inv = (THETA ** (-np.arange(64) / 64.0)).astype(np.float32)
    th = np.float32(pos) * inv
    sn, cs = np.sin(th).astype(np.float32), np.cos(th).astype(np.float32)
    a, b = vec[..., :64], vec[..., 64:]
    return np.concatenate([a * cs - b * sn, b * cs + a * sn], -1)


def make_weights(oracle, moe, n_layer, d, n_head, n_kv, n_exp, ff, ffs, vocab, seed=1):
    rng = np.random.default_rng(seed)
    norm = lambda: bf_bits(rng.uniform(0.8, 1.2, d).astype(np.float32))
    HQ, HK = n_head * 128, n_kv * 128
    layers = []
    for l in range(n_layer):
        m = lambda R, K, j: oracle.Matrix(R, K, 1000 * seed + 20 * l + j, eb=-20)
        layers.append({"norm_attn": norm(), "norm_ffn": norm(), "wq": m(HQ, d, 0), "wk": m(HK, d, 1), "wv": m(HK, d, 2), "wo": m(d, HQ, 3),
                       "router": m(n_exp + 1, d, 4), "sg": m(ffs, d, 5), "su": m(ffs, d, 6), "sd": m(d, ffs, 7),
                       "experts": moe.HostLayer(oracle, d, ff, n_exp, seed=50 * seed + l, eb=-20)})
    head = (rng.integers(0, 2 ** 32, (vocab, d // 8), dtype=np.uint64).astype(np.uint32), bf_bits(rng.uniform(0.001, 0.02, (vocab, d // 64)).astype(np.float32)),
            bf_bits(rng.uniform(-0.2, 0.0, (vocab, d // 64)).astype(np.float32)))
    return {"layers": layers, "embed": bf_bits(rng.standard_normal((vocab, d)).astype(np.float32) * 0.5), "norm_out": norm(), "head": head}


class HostDecoder:
    """The reference: one step over T rows, each its own sequence slot of `ctx` positions; caches kept between steps."""

    def __init__(self, oracle, hw, d, n_head, n_kv, n_exp, k, slots, ctx, dense_bf16=False):
        self.o, self.hw, self.d, self.n_head, self.n_kv, self.n_exp, self.k = oracle, hw, d, n_head, n_kv, n_exp, k
        self.dense_bf16, self.wcache = dense_bf16, {}
        self.K = [np.zeros((slots * ctx, n_kv, 128), np.uint16) for _ in hw["layers"]]
        self.V = [np.zeros((slots * ctx, n_kv, 128), np.uint16) for _ in hw["layers"]]

    def dense(self, m, x, T, add=0, y0=None):
        """A dense projection: the seed mat-vec, or (dense_bf16) the product with the weights rounded to bf16 once."""
        if not self.dense_bf16:
            return self.o.mv(m, x, T, add=add, y0=y0)
        if id(m) not in self.wcache:
            self.wcache[id(m)] = bfr(self.o.decode_rows_f32(m)).astype(np.float64)
        acc = bfr((np.asarray(x, np.float64).reshape(T, -1) @ self.wcache[id(m)].T).astype(np.float32))
        return bfr(np.asarray(y0, np.float32).reshape(T, -1) + acc) if add else acc

    def step(self, ids, pos, kv0):
        o, d, T = self.o, self.d, len(ids)
        x = bf_val(self.hw["embed"][ids])
        for l, hl in enumerate(self.hw["layers"]):
            h = gnorm(x, hl["norm_attn"])
            q = self.dense(hl["wq"], h, T).reshape(T, self.n_head, 128)
            kk = self.dense(hl["wk"], h, T).reshape(T, self.n_kv, 128)
            vv = self.dense(hl["wv"], h, T).reshape(T, self.n_kv, 128)
            for t in range(T):
                q[t] = bfr(rope(q[t], pos[t]))
                self.K[l][kv0[t] + pos[t]] = bf_bits(rope(kk[t], pos[t]))
                self.V[l][kv0[t] + pos[t]] = bf_bits(vv[t])
            att, _ = o.attn_decode(q, self.K[l], self.V[l], pos, kv0, self.n_kv, np.float32(1 / np.sqrt(128.0)))
            x = self.dense(hl["wo"], att.reshape(T, -1), T, add=1, y0=x)
            h = gnorm(x, hl["norm_ffn"])
            logits = self.dense(hl["router"], h, T)
            ind, wt = o.route(np.ascontiguousarray(logits[:, :self.n_exp]), self.k)
            ex = hl["experts"]
            D = np.zeros((T * self.k, d), np.float32)
            sh = np.zeros((T, d), np.float32)
            for t in range(T):
                for j in range(self.k):
                    e = int(ind[t, j])
                    a = o.mv_gu(ex.matrix(o, "gate", e), ex.matrix(o, "up", e), h[t])
                    D[t * self.k + j] = o.mv(ex.matrix(o, "down", e), a)[0]
                if self.dense_bf16:
                    a = o.swiglu(self.dense(hl["sg"], h[t], 1)[0], self.dense(hl["su"], h[t], 1)[0])
                    sh[t] = self.dense(hl["sd"], a, 1)[0]
                else:
                    sh[t] = o.mv(hl["sd"], o.mv_gu(hl["sg"], hl["su"], h[t]))[0]
            br = o.q4_moe_combine(D, wt, sh, np.ascontiguousarray(logits[:, self.n_exp]), T, d, self.k)
            x = bfr(x + br)
        lm, _ = o.q4_mv(*self.hw["head"], gnorm(x, self.hw["norm_out"]))
        return x, lm


CFG = dict(n_layer=2, d=256, n_head=4, n_kv=2, n_exp=8, top_k=2, ff_exp=64, ff_shared=64, vocab=512, ctx=8)


@pytest.mark.parametrize("windowed,dense_bf16", [(False, 0), (True, 0), (False, 1)])
def test_decoder_steps_against_the_host_reference(oracle, windowed, dense_bf16):
    import torch
    from nanoseedlm_b200 import decoder, ep, lib as L, moe
    c = CFG
    T = 3
    hw = make_weights(oracle, moe, c["n_layer"], c["d"], c["n_head"], c["n_kv"], c["n_exp"], c["ff_exp"], c["ff_shared"], c["vocab"])
    cfg = decoder.make_cfg(max_rows=T, eps=EPS, theta=THETA, dense_bf16=dense_bf16, **c)
    win = ep.P2PWindow.create(1, 0, T, c["d"], c["top_k"]) if windowed else None
    dec = decoder.host_decoder(cfg, hw, win)
    ref = HostDecoder(oracle, hw, c["d"], c["n_head"], c["n_kv"], c["n_exp"], c["top_k"], T, c["ctx"], dense_bf16=bool(dense_bf16))
    kv0 = [t * c["ctx"] for t in range(T)]
    nxt = torch.zeros(T, dtype=torch.int32, device="cuda")
    ids = np.array([5, 77, 300], np.int32)
    for step in range(3):
        pos = [step] * T
        dec.step(torch.from_numpy(ids).cuda(), decoder.row_info(pos, kv0), T, nxt)
        torch.cuda.synchronize()
        L.check()
        x, lm = ref.step(ids, pos, kv0)
        got_x, got_lm = dec.hidden(T).cpu().numpy(), dec.logits(T).cpu().numpy()
        sx, sl = np.max(np.abs(x)), np.max(np.abs(lm))
        # every intermediate is rounded to bf16: a flip of one of them moves later values by about a bf16 ulp
        assert np.max(np.abs(got_x - x)) <= 3e-2 * sx, (step, np.max(np.abs(got_x - x)) / sx)
        assert np.mean(np.abs(got_x - x) <= 4e-3 * sx) > 0.9
        assert np.max(np.abs(got_lm - lm)) <= 3e-2 * sl
        top2 = np.sort(lm, axis=1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.05 * sl      # rows whose best token does not hang on a rounding
        assert np.array_equal(nxt.cpu().numpy()[clear], np.argmax(lm, axis=1)[clear])
        ids = np.argmax(lm, axis=1).astype(np.int32)
    if win is not None:
        assert win.status() == 0
        win.close()
    dec.close()


def test_small_kernels_alone(oracle):
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    lib = L.load()
    rng = np.random.default_rng(3)
    T, d = 5, 384
    x = bfr(rng.standard_normal((T, d)).astype(np.float32) * 3)
    w = bf_bits(rng.uniform(0.5, 1.5, d).astype(np.float32))
    xd, wd, yd = kernels.dev(x), kernels.dev(w), torch.zeros(T, d, device="cuda")
    lib.kc_gnorm(None, d, EPS, xd.data_ptr(), wd.data_ptr(), yd.data_ptr(), T)
    torch.cuda.synchronize()
    want = gnorm(x, w)
    got = yd.cpu().numpy()
    assert np.mean(got == want) > 0.98 and np.max(np.abs(got - want)) <= np.max(np.abs(want)) / 64      # rsqrt: a bf16 flip now and then
    # rope + cache write: BF16 cache, then the 8-bit cache (codes and scales as the reference's quantizer gives them)
    n_head, n_kv, rows = 4, 2, 40
    q = bfr(rng.standard_normal((T, n_head, 128)).astype(np.float32))
    k = bfr(rng.standard_normal((T, n_kv, 128)).astype(np.float32))
    v = bfr(rng.standard_normal((T, n_kv, 128)).astype(np.float32))
    pos, kv0 = [0, 3, 7, 1, 6], [0, 8, 16, 24, 32]
    inv = (THETA ** (-np.arange(64) / 64.0)).astype(np.float32)
    ri = (L.RowInfo * T)()
    for t in range(T):
        ri[t].pos, ri[t].kv0 = pos[t], kv0[t]
    rid = torch.empty(16 * T, dtype=torch.uint8, device="cuda")
    rid.copy_(torch.frombuffer(bytearray(bytes(ri)), dtype=torch.uint8))
    invd = kernels.dev(inv)
    for q8 in (False, True):
        qd, kd, vd = kernels.dev(q), kernels.dev(k), kernels.dev(v)
        kc = torch.zeros(rows, n_kv, 128, dtype=torch.int8 if q8 else torch.int16, device="cuda")
        vc = torch.zeros_like(kc)
        ks, vs = torch.zeros(rows, n_kv, device="cuda"), torch.zeros(rows, n_kv, device="cuda")
        kv = L.KvView()
        kv.a.k, kv.a.v, kv.nv, kv.fmt = kc.data_ptr(), vc.data_ptr(), rows, 1 if q8 else 0
        if q8:
            kv.a.ks, kv.a.vs = ks.data_ptr(), vs.data_ptr()
        lib.kc_rope_kv(None, qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), kv, rid.data_ptr(), invd.data_ptr(), n_head, n_kv, T)
        torch.cuda.synchronize()
        L.check()
        for t in range(T):
            want_q = bfr(rope(q[t], pos[t]))
            assert np.max(np.abs(qd.cpu().numpy()[t] - want_q)) <= np.max(np.abs(want_q)) / 100      # sincosf on the device vs libm
            want_k, want_v = bf_bits(rope(k[t], pos[t])), bf_bits(v[t])
            row = kv0[t] + pos[t]
            if not q8:
                gk = bf_val(kc.cpu().numpy().view(np.uint16)[row])
                assert np.max(np.abs(gk - bf_val(want_k))) <= np.max(np.abs(bf_val(want_k))) / 100
                assert np.array_equal(vc.cpu().numpy().view(np.uint16)[row], want_v)
            else:
                codes, sc, _ = oracle.kv_q8_cache(want_v[None])
                assert np.array_equal(vc.cpu().numpy()[row], codes[0]) and np.array_equal(vs.cpu().numpy()[row], sc[0])
                kdeq = kc.cpu().numpy()[row].astype(np.float32) * ks.cpu().numpy()[row][:, None]
                assert np.max(np.abs(kdeq - bf_val(want_k))) <= np.max(np.abs(bf_val(want_k))) / 50
    # embedding rows
    table = bf_bits(rng.standard_normal((50, d)).astype(np.float32))
    ids = np.array([3, 49, 0, 7], np.int32)
    td, idd, out = kernels.dev(table), kernels.dev(ids), torch.zeros(4, d, device="cuda")
    w0 = L.WSlice()
    w0.p[0] = td.data_ptr()
    lib.kc_embed(None, 0, w0, d, idd.data_ptr(), out.data_ptr(), 4)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), bf_val(table[ids]))


@pytest.mark.parametrize("R,K,T", [(40, 256, 1), (40, 256, 5), (300, 2048, 8), (40, 128, 12), (300, 512, 40), (136, 256, 130), (2048, 2048, 32),
                                   (513, 2048, 32), (24, 256, 9), (40, 512, 64), (16, 256, 17)])
def test_stored_bf16_weights(oracle, R, K, T):
    """kc_mv (T <= 8) and kc_mm (more rows) with MF_BF16 weights [R][K]: y = bf16(W . x) with f32 sums, and the residual form."""
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    lib = L.load()
    rng = np.random.default_rng(R + K + T)
    W = bfr(rng.standard_normal((R, K)).astype(np.float32) * 0.05)
    x = bfr(rng.standard_normal((T, K)).astype(np.float32))
    y0 = bfr(rng.standard_normal((T, R)).astype(np.float32))
    wd, xd = kernels.dev(bf_bits(W)), kernels.dev(x)
    w = L.WSlice()
    w.p[0] = wd.data_ptr()
    acc = x.astype(np.float64) @ W.astype(np.float64).T
    mag = np.abs(x).astype(np.float64) @ np.abs(W).astype(np.float64).T
    fn = lib.kc_mv if T <= 8 else lib.kc_mm
    for add in (0, 1):
        yd = kernels.dev(y0.copy())
        fn(None, 0, w, K, R, xd.data_ptr(), K, yd.data_ptr(), R, T, add, None)
        torch.cuda.synchronize()
        L.check()
        want = bfr(y0 + bfr(acc.astype(np.float32))) if add else bfr(acc.astype(np.float32))
        got = yd.cpu().numpy()
        slack = 64 * 1.2e-7 * mag + (np.abs(acc) / 128 if add else 0)
        assert (np.abs(got.astype(np.float64) - want) <= np.abs(want) / 128.0 + 1e-30 + slack).all()
    assert lib.nsl_mm_status() == 0
    if 8 < T <= 64 and K % 256 == 0:      # the decode-batch GEMM: a row's result does not depend on the rows it shares the call with
        y9 = kernels.dev(np.zeros((9, R), np.float32))
        lib.kc_mm(None, 0, w, K, R, xd.data_ptr(), K, y9.data_ptr(), R, 9, 0, None)
        yT = kernels.dev(np.zeros((T, R), np.float32))
        lib.kc_mm(None, 0, w, K, R, xd.data_ptr(), K, yT.data_ptr(), R, T, 0, None)
        torch.cuda.synchronize()
        assert torch.equal(y9[:9], yT[:9])


def test_decoder_step_of_more_rows_than_a_mat_vec_takes(oracle):
    """Twelve rows: the dense projections and the shared expert take the tensor-core GEMM, the routed experts the pair
    mat-vec over 24 pairs.  The GEMM rounds seed weights to bf16, so this is not compared value by value with the
    mat-vec path: the step must run clean and give finite rows and tokens inside the vocabulary."""
    import torch
    from nanoseedlm_b200 import decoder, lib as L
    c = dict(CFG, n_layer=1)
    T = 12
    cfg = decoder.make_cfg(max_rows=T, eps=EPS, theta=THETA, **c)
    dec = decoder.random_decoder(cfg, seed=3)
    nxt = torch.full((T,), -1, dtype=torch.int32, device="cuda")
    ids = torch.arange(T, dtype=torch.int32, device="cuda")
    dec.step(ids, decoder.row_info([0] * T, [t * c["ctx"] for t in range(T)]), T, nxt)
    torch.cuda.synchronize()
    L.check()
    assert L.load().nsl_mm_status() == 0
    h = dec.hidden(T).cpu().numpy()
    assert np.isfinite(h).all() and np.abs(h).max() > 0
    n = nxt.cpu().numpy()
    assert ((n >= 0) & (n < c["vocab"])).all()
    dec.close()
