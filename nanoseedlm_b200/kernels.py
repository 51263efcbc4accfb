"""Host-side mirror of the reference's kernel test backend (tests/kernel_backend.h: KtWeight and the kt_* calls;
tests/kernel_backend_cuda.c:26-34, 94-…): upload, launch the kc_* entry point on a stream, synchronise, copy back.

Every function here calls the CUDA library through its C ABI; numpy arrays in, numpy arrays out.  torch supplies
device memory and the stream only."""
import ctypes as C

import numpy as np
import torch

from . import lib as L


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr() if t is not None else 0)


def dev(a, dtype=None):
    """numpy -> device tensor of the same bits (u16 travels as int16, u32 as int32)."""
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        a = a.view(np.int16)
    elif a.dtype == np.uint32:
        a = a.view(np.int32)
    t = torch.from_numpy(a).cuda()
    return t if dtype is None else t.to(dtype)


_table = {}


def stream_table():
    """The 65536-entry lfsr_stream32 table on the current device (the G argument of the kc_* calls)."""
    d = torch.cuda.current_device()
    if d not in _table:
        host = np.zeros(65536, np.uint32)
        L.load().nsl_stream_table(C.c_void_p(host.ctypes.data))
        _table[d] = dev(host)
    return _table[d]


class SeedWeight:
    """S slices of an R x K SEED4P4 tensor on the device plus the device table of their WSlice entries
    (the reference's KtWeight for MF_SEED4P4: streams w = seeds, s = coefficient words, e = codes, b = biases)."""

    def __init__(self, seeds, coefs, codes, eb, R, K):
        S = len(eb)
        self.S, self.R, self.K = S, R, K
        self.seeds = dev(np.asarray(seeds, np.uint16).reshape(S, -1))
        self.coefs = dev(np.asarray(coefs, np.uint16).reshape(S, -1))
        self.codes = dev(np.asarray(codes, np.uint8).reshape(S, -1))
        self.eb = [int(e) for e in eb]
        arr = (L.WSlice * S)()
        for s in range(S):
            arr[s] = self.slice(s)
        self.table_host = arr
        self.table = torch.empty(S * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
        self.table.copy_(torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8))

    @classmethod
    def from_matrices(cls, mats):
        m0 = mats[0]
        return cls(np.stack([m.seeds for m in mats]), np.stack([m.coefs for m in mats]),
                   np.stack([m.codes for m in mats]), [m.eb for m in mats], m0.rows, m0.K)

    def slice(self, s):
        w = L.WSlice()
        w.p[0] = self.seeds[s].data_ptr()
        w.p[1] = self.coefs[s].data_ptr()
        w.p[2] = 0
        w.p[3] = self.codes[s].data_ptr()
        w.eb = self.eb[s]
        return w

    @property
    def nbytes(self):
        return self.seeds.numel() * 2 + self.coefs.numel() * 2 + self.codes.numel()


class SeedWeight3:
    """S slices of an R x K P = 3 (MF_SEED4) tensor on the device and the device table of their WSlice entries."""

    def __init__(self, mats):
        self.S, self.R, self.K = len(mats), mats[0].rows, mats[0].K
        self.seeds = dev(np.stack([m.seeds for m in mats]).reshape(self.S, -1))
        self.nibs = dev(np.stack([m.nibs for m in mats]).reshape(self.S, -1))
        self.eb = [int(m.eb) for m in mats]
        arr = (L.WSlice * self.S)()
        for s in range(self.S):
            arr[s] = self.slice(s)
        self.table = torch.empty(self.S * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
        self.table.copy_(torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8))

    def slice(self, s):
        w = L.WSlice()
        w.p[0], w.p[1] = self.seeds[s].data_ptr(), self.nibs[s].data_ptr()
        w.eb = self.eb[s]
        return w


def kt_decode3(w, s=0, bf16=False):
    out = torch.empty(w.R * w.K, dtype=torch.int16 if bf16 else torch.float32, device="cuda")
    fn = L.load().nsl_decode3_bf16 if bf16 else L.load().nsl_decode3_f32
    fn(_stream(), w.slice(s), w.K, w.R, _ptr(out), _ptr(stream_table()))
    _done()
    o = out.cpu().numpy()
    return (o.view(np.uint16) if bf16 else o).reshape(w.R, w.K)


def kt_mv3(w, x, T, add=0, y0=None, s=0):
    """kc_mv with MF_SEED4 on slice s."""
    xd = dev(np.asarray(x, np.float32).reshape(T, w.K))
    yd = dev(np.asarray(y0, np.float32).reshape(T, w.R)) if y0 is not None else torch.zeros(T, w.R, device="cuda")
    L.load().kc_mv(_stream(), L.MF_SEED4, w.slice(s), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, T, add, _ptr(stream_table()))
    _done()
    return yd.cpu().numpy()


def kt_mv3_sel(w, sel, xdiv, x):
    sel = np.asarray(sel, np.int32)
    xd, seld = dev(np.asarray(x, np.float32).reshape(-1, w.K)), dev(sel)
    yd = torch.zeros(sel.size, w.R, device="cuda")
    L.load().kc_mv_sel(_stream(), L.MF_SEED4, _ptr(w.table), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, _ptr(seld), sel.size, xdiv,
                       _ptr(stream_table()))
    _done()
    return yd.cpu().numpy()


def kt_mv3_gu(wg, wu, sel, xdiv, x):
    sel = np.asarray(sel, np.int32)
    xd, seld = dev(np.asarray(x, np.float32).reshape(-1, wg.K)), dev(sel)
    ad = torch.zeros(sel.size, wg.R, device="cuda")
    L.load().kc_mv_gu(_stream(), L.MF_SEED4, _ptr(wg.table), _ptr(wu.table), wg.K, wg.R, _ptr(xd), wg.K, _ptr(ad), wg.R,
                      _ptr(seld), sel.size, xdiv, _ptr(stream_table()))
    _done()
    return ad.cpu().numpy()


def _done():
    torch.cuda.synchronize()
    L.check()
    st = L.load().nsl_mm_status()
    if st:
        raise RuntimeError(f"a GEMM block gave up on a bounded wait (code {st})")


def kt_decode(w, s=0, bf16=False):
    out = torch.empty(w.R * w.K, dtype=torch.int16 if bf16 else torch.float32, device="cuda")
    fn = L.load().nsl_decode_bf16 if bf16 else L.load().nsl_decode_f32
    fn(_stream(), w.slice(s), w.K, w.R, _ptr(out), _ptr(stream_table()))
    _done()
    o = out.cpu().numpy()
    return (o.view(np.uint16) if bf16 else o).reshape(w.R, w.K)


def kt_mv(w, x, T, add=0, y0=None, s=0, raw=False):
    """Dense mat-vec of slice s: x [T][K] -> y [T][R]."""
    xd = dev(np.asarray(x, np.float32).reshape(T, w.K))
    yd = dev(np.asarray(y0, np.float32).reshape(T, w.R)) if y0 is not None else torch.zeros(T, w.R, device="cuda")
    if raw:
        one = (L.WSlice * 1)(w.slice(s))
        L.load().nsl_mv_raw(_stream(), C.cast(one, C.c_void_p), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, None, T, 1,
                            _ptr(stream_table()))
    else:
        L.load().kc_mv(_stream(), L.MF_SEED4P4, w.slice(s), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, T, add,
                       _ptr(stream_table()))
    _done()
    return yd.cpu().numpy()


def kt_mv_sel(w, sel, xdiv, x, raw=False):
    """Gather mat-vec: pair p uses slice sel[p] and input row p // xdiv."""
    sel = np.asarray(sel, np.int32)
    P = sel.size
    xd = dev(np.asarray(x, np.float32).reshape(-1, w.K))
    yd = torch.zeros(P, w.R, device="cuda")
    seld = dev(sel)
    if raw:
        L.load().nsl_mv_raw(_stream(), _ptr(w.table), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, _ptr(seld), P, xdiv,
                            _ptr(stream_table()))
    else:
        L.load().kc_mv_sel(_stream(), L.MF_SEED4P4, _ptr(w.table), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, _ptr(seld),
                           P, xdiv, _ptr(stream_table()))
    _done()
    return yd.cpu().numpy()


def kt_mv_gu(wg, wu, sel, xdiv, x):
    sel = np.asarray(sel, np.int32)
    P = sel.size
    xd = dev(np.asarray(x, np.float32).reshape(-1, wg.K))
    ad = torch.zeros(P, wg.R, device="cuda")
    seld = dev(sel)
    L.load().kc_mv_gu(_stream(), L.MF_SEED4P4, _ptr(wg.table), _ptr(wu.table), wg.K, wg.R, _ptr(xd), wg.K, _ptr(ad),
                      wg.R, _ptr(seld), P, xdiv, _ptr(stream_table()))
    _done()
    return ad.cpu().numpy()


def kt_mv_gu_routed(wg, wu, logits, k, x, raw=False):
    """nsl_mv_gu_routed: the router and the gate + up + SwiGLU mat-vec in one launch -> (a [T*k][R], ind, wt)."""
    logits = np.asarray(logits, np.float32)
    T, E = logits.shape
    xd, ld = dev(np.asarray(x, np.float32).reshape(T, wg.K)), dev(logits)
    ad = torch.zeros(T * k, wg.R, device="cuda")
    ind = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    wt = torch.zeros(T, k, device="cuda")
    L.load().nsl_mv_gu_routed(_stream(), _ptr(wg.table), _ptr(wu.table), wg.K, wg.R, _ptr(xd), wg.K, _ptr(ad), wg.R, E, k,
                              _ptr(ld), E, T, _ptr(ind), _ptr(wt), int(raw), _ptr(stream_table()))
    _done()
    return ad.cpu().numpy(), ind.cpu().numpy(), wt.cpu().numpy()


def kt_mv_gu_rows(wg, wu, sel, xrow, x, bf16=False, count=None, raw=False):
    """nsl_mv_gu_rows: pair p uses slice sel[p] and input row xrow[p]; bf16 packs the inputs first; count (optional) = the
    number of valid pairs, read on the device."""
    sel = np.asarray(sel, np.int32)
    P = sel.size
    xd = dev(np.asarray(x, np.float32).reshape(-1, wg.K))
    if bf16:
        packed = torch.zeros(xd.numel(), dtype=torch.int16, device="cuda")
        L.load().kc_pack_input_bf16(_stream(), _ptr(xd), _ptr(packed), xd.numel())
        xd = packed
    ad = torch.zeros(P, wg.R, device="cuda")
    seld, rowd = dev(sel), dev(np.asarray(xrow, np.int32))
    cnt = dev(np.array([P if count is None else count], np.int32))
    L.load().nsl_mv_gu_rows(_stream(), _ptr(wg.table), _ptr(wu.table), wg.K, wg.R, _ptr(xd), wg.K, int(bf16), _ptr(ad), wg.R,
                            _ptr(seld), _ptr(rowd), P, _ptr(cnt), int(raw), _ptr(stream_table()))
    _done()
    return ad.cpu().numpy()


def kt_mv_q4(codes, scales, biases, x, T, add=0, y0=None):
    """kc_mv with fmt MF_Q4 (the LM head): codes u32 [R][K/8], scales / biases bf16 bits per group of 64."""
    codes = np.ascontiguousarray(codes, np.uint32)
    R, K = codes.shape[0], codes.shape[1] * 8
    keep = [dev(codes), dev(np.asarray(scales, np.uint16)), dev(np.asarray(biases, np.uint16))]
    w = L.WSlice()
    w.p[0], w.p[1], w.p[2] = (t.data_ptr() for t in keep)
    xd = dev(np.asarray(x, np.float32).reshape(T, K))
    yd = dev(np.asarray(y0, np.float32).reshape(T, R)) if y0 is not None else torch.zeros(T, R, device="cuda")
    L.load().kc_mv(_stream(), L.MF_Q4, w, K, R, _ptr(xd), K, _ptr(yd), R, T, add, None)
    _done()
    return yd.cpu().numpy()


def kt_argmax(logits, prob=False):
    ld = dev(np.asarray(logits, np.float32))
    n, V = ld.shape
    out = torch.zeros(n, dtype=torch.int32, device="cuda")
    pr = torch.zeros(n, device="cuda") if prob else None
    L.load().kc_argmax_p(_stream(), _ptr(ld), _ptr(out), _ptr(pr), V, n)
    _done()
    return (out.cpu().numpy(), pr.cpu().numpy()) if prob else out.cpu().numpy()


def kt_attn(a, q, Kc, Vc, pos, kv0, g=None, nv=None, scales=None):
    """kc_attn (tests/kernel_backend_cuda.c: kt_attn, kt_attn_q8): Kc / Vc [rows][n_kv][128] as bf16 bits, or int8 codes
    with scales = (ks, vs) [rows][n_kv] f32 (the 8-bit cache); rows of the cache below nv (default: all) sit in segment a,
    the rest in segment b."""
    T = len(pos)
    q8 = scales is not None
    Kc, Vc = np.asarray(Kc, np.int8 if q8 else np.uint16), np.asarray(Vc, np.int8 if q8 else np.uint16)
    nv = Kc.shape[0] if nv is None else nv
    two = nv < Kc.shape[0]
    keep = [dev(Kc[:nv]), dev(Vc[:nv]), dev(Kc[nv:]) if two else None, dev(Vc[nv:]) if two else None]
    kv = L.KvView()
    kv.a.k, kv.a.v = keep[0].data_ptr(), keep[1].data_ptr()
    if two:
        kv.b.k, kv.b.v = keep[2].data_ptr(), keep[3].data_ptr()
    if q8:
        ks, vs = (np.asarray(x, np.float32) for x in scales)
        keep += [dev(ks[:nv]), dev(vs[:nv]), dev(ks[nv:]) if two else None, dev(vs[nv:]) if two else None]
        kv.a.ks, kv.a.vs = keep[4].data_ptr(), keep[5].data_ptr()
        if two:
            kv.b.ks, kv.b.vs = keep[6].data_ptr(), keep[7].data_ptr()
    kv.nv, kv.fmt = nv, 1 if q8 else 0
    ri = (L.RowInfo * T)()
    for t in range(T):
        ri[t].pos, ri[t].kv0 = int(pos[t]), int(kv0[t])
    rid = torch.empty(T * 16, dtype=torch.uint8, device="cuda")
    rid.copy_(torch.frombuffer(bytearray(bytes(ri)), dtype=torch.uint8))
    qd = dev(np.asarray(q, np.float32))
    gd = dev(np.asarray(g, np.float32)) if g is not None else None
    part = torch.zeros(T * a.n_head * a.n_splits * 130, device="cuda")
    o = torch.zeros(T, a.n_head, 128, device="cuda")
    L.load().kc_attn(_stream(), a, _ptr(qd), kv, _ptr(rid), _ptr(part), _ptr(gd), _ptr(o), T)
    _done()
    return o.cpu().numpy()


def kt_route(logits, k):
    logits = np.asarray(logits, np.float32)
    T, E = logits.shape
    ld = dev(logits)
    ind = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    wt = torch.zeros(T, k, device="cuda")
    L.load().nsl_route(_stream(), E, k, _ptr(ld), E, _ptr(ind), _ptr(wt), T)
    _done()
    return ind.cpu().numpy(), wt.cpu().numpy()


def kt_route_cfg(logits, k):
    """The same through kq4_route and a Qwen4Cfg-shaped block of ints."""
    logits = np.asarray(logits, np.float32)
    T, E = logits.shape
    cfg = np.zeros(128, np.int32)
    cfg[21], cfg[22] = E, k
    ld = dev(logits)
    ind = torch.zeros(T, k, dtype=torch.int32, device="cuda")
    wt = torch.zeros(T, k, device="cuda")
    L.load().kq4_route(_stream(), C.c_void_p(cfg.ctypes.data), _ptr(ld), _ptr(ind), _ptr(wt), T)
    _done()
    return ind.cpu().numpy(), wt.cpu().numpy()


def kt_router(a, W, bias, x, T):
    """kc_router (tests/kernel_backend_cuda.c:176-184): W [n][d], bias [n] BF16 bits; returns inds, wts, score, sel."""
    Wd, bd, xd = dev(np.asarray(W, np.uint16)), dev(np.asarray(bias, np.uint16)), dev(np.asarray(x, np.float32))
    score, sel = torch.zeros(T, a.n, device="cuda"), torch.zeros(T, a.n, device="cuda")
    ind = torch.zeros(T, a.top_k, dtype=torch.int32, device="cuda")
    wt = torch.zeros(T, a.top_k, device="cuda")
    L.load().kc_router(_stream(), a, _ptr(Wd), _ptr(bd), _ptr(xd), _ptr(score), _ptr(sel), _ptr(ind), _ptr(wt), T)
    _done()
    return ind.cpu().numpy(), wt.cpu().numpy(), score.cpu().numpy(), sel.cpu().numpy()


def kt_router_topk(a, score, sel, T):
    """kc_router_topk (tests/kernel_backend_cuda.c:185-192)."""
    sd, ed = dev(np.asarray(score, np.float32)), dev(np.asarray(sel, np.float32))
    ind = torch.zeros(T, a.top_k, dtype=torch.int32, device="cuda")
    wt = torch.zeros(T, a.top_k, device="cuda")
    L.load().kc_router_topk(_stream(), a, _ptr(sd), _ptr(ed), _ptr(ind), _ptr(wt), T)
    _done()
    return ind.cpu().numpy(), wt.cpu().numpy()


def _heads_slice(seeds, coefs, ebias, ecodes):
    keep = [dev(np.asarray(seeds, np.uint16)), dev(np.asarray(coefs, np.uint16)), dev(np.asarray(ebias, np.int32)),
            dev(np.asarray(ecodes, np.uint8))]
    w = L.WSlice()
    for i in range(4):
        w.p[i] = keep[i].data_ptr()
    w.eb = int(np.asarray(ebias).ravel()[0])
    return w, keep


def kt_heads_seed(H, O, I, seeds, coefs, ebias, ecodes, x, xs, hs, g, T):
    """kc_heads_mv on a stacked SEED4P4 map [H][O][I] (tests/kernel_backend_cuda.c:546-562): y [T][H][O]."""
    w, keep = _heads_slice(seeds, coefs, ebias, ecodes)
    a = L.HmvArgs(H, O, I, xs, hs, int(g is not None))
    xd = dev(np.asarray(x, np.float32))
    gd = dev(np.asarray(g, np.float32)) if g is not None else None
    y = torch.zeros(T, H, O, device="cuda")
    L.load().kc_heads_mv(_stream(), a, L.MF_SEED4P4, w, _ptr(stream_table()), _ptr(xd), _ptr(gd), _ptr(y), T)
    _done()
    return y.cpu().numpy()


def kt_heads_deq(H, O, I, seeds, coefs, ebias, ecodes):
    """kc_heads_deq (tests/kernel_backend_cuda.c:564-565): the map as BF16 bits [H][O][I]."""
    w, keep = _heads_slice(seeds, coefs, ebias, ecodes)
    out = torch.zeros(H * O * I, dtype=torch.int16, device="cuda")
    L.load().kc_heads_deq(_stream(), L.MF_SEED4P4, w, _ptr(stream_table()), H, O, I, _ptr(out))
    _done()
    return out.cpu().numpy().view(np.uint16).reshape(H, O, I)


def kt_swiglu(g, u):
    gd, ud = dev(np.asarray(g, np.float32)), dev(np.asarray(u, np.float32))
    ad = torch.empty_like(gd)
    L.load().kc_swiglu(_stream(), _ptr(gd), _ptr(ud), _ptr(ad), gd.numel())
    _done()
    return ad.cpu().numpy()


def kt_q4_moe_combine(D, wt, sh, sg, T, d, k):
    Dd, wd = dev(np.asarray(D, np.float32)), dev(np.asarray(wt, np.float32))
    shd = dev(np.asarray(sh, np.float32)) if sh is not None else None
    sgd = dev(np.asarray(sg, np.float32)) if sg is not None else None
    out = torch.zeros(T, d, device="cuda")
    L.load().kq4_moe_combine(_stream(), d, k, _ptr(Dd), _ptr(wd), _ptr(shd), _ptr(sgd), 1, _ptr(out), T)
    _done()
    return out.cpu().numpy()


def kt_moe_combine(D, w, shared, x, T, d, k):
    Dd, wd, sd = dev(np.asarray(D, np.float32)), dev(np.asarray(w, np.float32)), dev(np.asarray(shared, np.float32))
    xd = dev(np.asarray(x, np.float32).copy())
    L.load().kc_moe_combine(_stream(), _ptr(Dd), _ptr(wd), _ptr(sd), _ptr(xd), d, k, T)
    _done()
    return xd.cpu().numpy()


def kt_pack_bf16(x):
    xd = dev(np.asarray(x, np.float32).ravel())
    yd = torch.zeros(xd.numel(), dtype=torch.int16, device="cuda")
    L.load().kc_pack_input_bf16(_stream(), _ptr(xd), _ptr(yd), xd.numel())
    _done()
    return yd.cpu().numpy().view(np.uint16)


def kt_bucket(inds, n):
    """-> (perm, [(slice, start, count)], ntiles) as kc_bucket leaves them."""
    inds = np.asarray(inds, np.int32).ravel()
    P = inds.size
    mt = P // L.MMT_BN + n
    di = dev(inds)
    perm = torch.zeros(max(P, 1), dtype=torch.int32, device="cuda")
    tiles = torch.zeros(mt * 4, dtype=torch.int32, device="cuda")
    work = torch.zeros(2 * n + 3, dtype=torch.int32, device="cuda")
    L.load().kc_bucket(_stream(), _ptr(di), P, n, _ptr(perm), _ptr(tiles), _ptr(work))
    _done()
    nt = int(work[0].item())
    tl = tiles.cpu().numpy().reshape(mt, 4)
    return perm.cpu().numpy()[:P], [tuple(int(v) for v in tl[i, :3]) for i in range(nt)], nt


def kt_mm(w, x, T, add=0, y0=None, s=0, exact=False, packed=False):
    """Dense prompt GEMM of slice s: x [T][K] -> y [T][R] (w: a SeedWeight, or a SeedWeight3 for the P = 3 format)."""
    lib = L.load()
    fmt = L.MF_SEED4 if isinstance(w, SeedWeight3) else L.MF_SEED4P4
    lib.kc_seed_gemm_f32(int(exact))
    xd = dev(np.asarray(x, np.float32).reshape(T, w.K))
    yd = dev(np.asarray(y0, np.float32).reshape(T, w.R)) if y0 is not None else torch.zeros(T, w.R, device="cuda")
    if packed:
        xp = torch.zeros(T * w.K, dtype=torch.int16, device="cuda")
        lib.kc_pack_input_bf16(_stream(), _ptr(xd), _ptr(xp), T * w.K)
        lib.kc_mm_packed(_stream(), fmt, w.slice(s), w.K, w.R, _ptr(xp), w.K, _ptr(yd), w.R, T, add,
                         _ptr(stream_table()))
    else:
        lib.kc_mm(_stream(), fmt, w.slice(s), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, T, add,
                  _ptr(stream_table()))
    _done()
    lib.kc_seed_gemm_f32(0)
    return yd.cpu().numpy()


def kt_mm_grouped(w, P, xdiv, perm, tiles, x, exact=False, mode="host"):
    """Grouped prompt GEMM over a tile table.  mode: 'host' (kc_mm_grouped), 'dev' (kc_mm_grouped_dev) or 'packed'."""
    lib = L.load()
    fmt = L.MF_SEED4 if isinstance(w, SeedWeight3) else L.MF_SEED4P4
    lib.kc_seed_gemm_f32(int(exact))
    xd = dev(np.asarray(x, np.float32).reshape(-1, w.K))
    yd = torch.zeros(P, w.R, device="cuda")
    pd = dev(np.asarray(perm, np.int32))
    tl = np.zeros((max(len(tiles), 1), 4), np.int32)
    for i, t in enumerate(tiles):
        tl[i, :3] = t
    td = dev(tl)
    nt = len(tiles)
    if mode == "host":
        lib.kc_mm_grouped(_stream(), fmt, _ptr(w.table), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, xdiv, _ptr(pd),
                          _ptr(td), nt, _ptr(stream_table()))
    else:
        ntd = dev(np.array([nt], np.int32))
        if mode == "dev":
            lib.kc_mm_grouped_dev(_stream(), fmt, _ptr(w.table), w.K, w.R, _ptr(xd), w.K, _ptr(yd), w.R, xdiv,
                                  _ptr(pd), _ptr(td), _ptr(ntd), nt + 3, _ptr(stream_table()))
        else:
            xp = torch.zeros(xd.numel(), dtype=torch.int16, device="cuda")
            lib.kc_pack_input_bf16(_stream(), _ptr(xd), _ptr(xp), xd.numel())
            lib.kc_mm_grouped_packed(_stream(), fmt, _ptr(w.table), w.K, w.R, _ptr(xp), w.K, _ptr(yd), w.R,
                                     xdiv, _ptr(pd), _ptr(td), _ptr(ntd), nt + 3, _ptr(stream_table()))
    _done()
    lib.kc_seed_gemm_f32(0)
    return yd.cpu().numpy()
