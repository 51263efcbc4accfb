"""ctypes binding of the CPU oracle (oracle/liboracle.so) and, where it was built, of the reference's own C sources
(oracle/_ref/libnslm_ref.so).  TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the bench's CPU
baseline leg -- never by the product package."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None


def build(ref_root=None):
    """Compile liboracle.so (and oracle/_ref when the reference tree is present: ref_root, else $NSLM_REFERENCE_ROOT, else a
    checkout named `reference` beside this repository)."""
    subprocess.run(["make", "-s", "-C", HERE] + ([f"REF={ref_root}"] if ref_root else []), check=True)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _declare(_LIB)
    return _LIB


def ref():
    """The reference's own code, or None when oracle/_ref was not built (it only builds where the reference tree is)."""
    global _REF
    if _REF is None:
        path = os.path.join(HERE, "_ref", "libnslm_ref.so")
        if not os.path.exists(path):
            return None
        _REF = C.CDLL(path)
        _REF.ref_stream32.restype = C.c_uint32
    return _REF


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def _declare(L):
    L.orc_lfsr_step.restype = C.c_uint16
    L.orc_lfsr_step.argtypes = [C.c_uint16]
    L.orc_stream32.restype = C.c_uint32
    L.orc_stream32.argtypes = [C.c_uint16]
    L.orc_fnv24_all_seeds.restype = C.c_uint64
    L.orc_period.restype = C.c_int
    L.orc_scale.restype = C.c_float
    L.orc_scale.argtypes = [C.c_int]
    L.orc_silu_bf.restype = C.c_float
    L.orc_silu_bf.argtypes = [C.c_float]
    L.orc_cpu_seed4_time.restype = C.c_double
    L.orc_softplus_gate.restype = C.c_float
    L.orc_softplus_gate.argtypes = [C.c_float]
    L.orc_mova_topk.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    L.orc_mova_router.argtypes = [C.c_int] * 4 + [C.c_float] + [C.c_void_p] * 7
    L.orc_bucket.restype = C.c_int


u16, u8, i32, f32, f64, u32 = C.c_uint16, C.c_uint8, C.c_int32, C.c_float, C.c_double, C.c_uint32


class Matrix:
    """One SEED4P4 slice: rows x K weights as seeds/coefs [rows][K/8] (u16) and exponent-code nibbles (u8)."""

    def __init__(self, rows, K, seed, eb=-22):
        self.rows, self.K, self.eb = rows, K, eb
        nb = rows * (K // 8)
        self.seeds = np.zeros(nb, np.uint16)
        self.coefs = np.zeros(nb, np.uint16)
        self.codes = np.zeros((nb + 1) // 2, np.uint8)
        lib().orc_gen_matrix(C.c_uint64(seed), rows, K, _p(self.seeds, u16), _p(self.coefs, u16), _p(self.codes, u8))

    def args(self):
        return _p(self.seeds, u16), _p(self.coefs, u16), _p(self.codes, u8), C.c_int(self.eb)

    @property
    def nbytes(self):
        return self.seeds.nbytes + self.coefs.nbytes + self.codes.nbytes


def normal(seed, n, bf16=False):
    out = np.zeros(n, np.float32)
    lib().orc_gen_normal(C.c_uint64(seed), C.c_size_t(n), int(bf16), _p(out, f32))
    return out


def table32():
    t = np.zeros(65536, np.uint32)
    lib().orc_table32(_p(t, u32))
    return t


def states(seed, n):
    out = np.zeros(n, np.uint16)
    lib().orc_lfsr_states(C.c_uint16(seed), n, _p(out, u16))
    return out


def decode_block_bf16(seed, coef, e):
    out = np.zeros(8, np.uint16)
    lib().orc_decode_block_bf16(C.c_uint16(seed), C.c_uint16(coef), e, _p(out, u16))
    return out


def decode_rows_f32(m):
    out = np.zeros(m.rows * m.K, np.float32)
    lib().orc_decode_rows_f32(*m.args(), m.rows, m.K, _p(out, f32))
    return out.reshape(m.rows, m.K)


def decode_rows_bf16(m):
    out = np.zeros(m.rows * m.K, np.uint16)
    lib().orc_decode_rows_bf16(*m.args(), m.rows, m.K, _p(out, u16))
    return out.reshape(m.rows, m.K)


def matvec_f64(m, x, T=1):
    """x [T][K] f32 -> (y [T][rows] f64, mag [T][rows] f64 = sum |w x|)."""
    x = np.ascontiguousarray(x, np.float32).reshape(T, m.K)
    y = np.zeros((T, m.rows), np.float64)
    mag = np.zeros((T, m.rows), np.float64)
    lib().orc_matvec_f64(*m.args(), m.rows, m.K, _p(x, f32), m.K, T, _p(y, f64), m.rows, _p(mag, f64))
    return y, mag


def mv(m, x, T=1, add=0, y0=None):
    x = np.ascontiguousarray(x, np.float32).reshape(T, m.K)
    y = np.zeros((T, m.rows), np.float32) if y0 is None else np.array(y0, np.float32).reshape(T, m.rows).copy()
    lib().orc_mv(*m.args(), m.rows, m.K, _p(x, f32), m.K, T, add, _p(y, f32), m.rows)
    return y


def mv_gu(g, u, x):
    x = np.ascontiguousarray(x, np.float32)
    a = np.zeros(g.rows, np.float32)
    lib().orc_mv_gu(*g.args(), *u.args(), g.rows, g.K, _p(x, f32), _p(a, f32))
    return a


def swiglu(g, u):
    g = np.ascontiguousarray(g, np.float32)
    u = np.ascontiguousarray(u, np.float32)
    a = np.zeros_like(g)
    lib().orc_swiglu(_p(g, f32), _p(u, f32), _p(a, f32), g.size)
    return a


def route(logits, k):
    logits = np.ascontiguousarray(logits, np.float32)
    T, E = logits.shape
    ind = np.zeros((T, k), np.int32)
    wt = np.zeros((T, k), np.float32)
    for t in range(T):
        lib().orc_route(_p(logits[t], f32), E, k, _p(ind[t], i32), _p(wt[t], f32))
    return ind, wt


def f2bf(a):
    """f32 array -> BF16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def mova_topk(score, sel, k, scale):
    score, sel = np.ascontiguousarray(score, np.float32), np.ascontiguousarray(sel, np.float32)
    T, n = score.shape
    ind, wt = np.zeros((T, k), np.int32), np.zeros((T, k), np.float32)
    for t in range(T):
        lib().orc_mova_topk(score[t].ctypes.data, sel[t].ctypes.data, n, k, scale, ind[t].ctypes.data, wt[t].ctypes.data)
    return ind, wt


def mova_router(W, bias, x, k, hw, scale):
    """W [n][d] and bias [n] as BF16 bit patterns, x [T][d] f32 -> score, sel, inds, wts."""
    W, bias = np.ascontiguousarray(W, np.uint16), np.ascontiguousarray(bias, np.uint16)
    x = np.ascontiguousarray(x, np.float32)
    (n, d), T = W.shape, x.shape[0]
    score, sel = np.zeros((T, n), np.float32), np.zeros((T, n), np.float32)
    ind, wt = np.zeros((T, k), np.int32), np.zeros((T, k), np.float32)
    for t in range(T):
        lib().orc_mova_router(d, hw, n, k, scale, W.ctypes.data, bias.ctypes.data, x[t].ctypes.data, score[t].ctypes.data,
                              sel[t].ctypes.data, ind[t].ctypes.data, wt[t].ctypes.data)
    return score, sel, ind, wt


def softplus_gate(g):
    g = np.ascontiguousarray(g, np.float32)
    return np.array([lib().orc_softplus_gate(float(v)) for v in g.ravel()], np.float32).reshape(g.shape)


def q4_moe_combine(D, wt, sh, sg, T, d, k):
    out = np.zeros((T, d), np.float32)
    D, wt, sh, sg = (np.ascontiguousarray(a, np.float32) for a in (D, wt, sh, sg))
    lib().orc_q4_moe_combine(d, k, _p(D, f32), _p(wt, f32), _p(sh, f32), _p(sg, f32), 1, _p(out, f32), T)
    return out


def moe_combine(D, w, shared, x, T, d, k):
    x = np.array(x, np.float32).copy()
    D, w, shared = (np.ascontiguousarray(a, np.float32) for a in (D, w, shared))
    lib().orc_moe_combine(_p(D, f32), _p(w, f32), _p(shared, f32), _p(x, f32), d, k, T)
    return x


class Tile(C.Structure):
    _fields_ = [("slice", i32), ("start", i32), ("count", i32), ("pad", i32)]


def bucket(inds, n, bn=128):
    inds = np.ascontiguousarray(inds, np.int32).ravel()
    perm = np.zeros(inds.size, np.int32)
    tiles = (Tile * (inds.size // bn + n + 1))()
    nt = lib().orc_bucket(_p(inds, i32), inds.size, n, bn, _p(perm, i32), tiles)
    return perm, [(t.slice, t.start, t.count) for t in tiles[:nt]]


def mm_pairs(mats, slice_of_pair, xdiv, x, exact=False):
    """mats: list of Matrix (same shape); x [rows_in][K]; returns y [P][rows] as the grouped prompt GEMM rounds it."""
    S = len(mats)
    rows, K = mats[0].rows, mats[0].K
    sp = (C.POINTER(u16) * S)(*[_p(m.seeds, u16) for m in mats])
    cp = (C.POINTER(u16) * S)(*[_p(m.coefs, u16) for m in mats])
    ep = (C.POINTER(u8) * S)(*[_p(m.codes, u8) for m in mats])
    eb = np.array([m.eb for m in mats], np.int32)
    sl = np.ascontiguousarray(slice_of_pair, np.int32)
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros((sl.size, rows), np.float32)
    lib().orc_mm_pairs(sp, cp, ep, _p(eb, i32), _p(sl, i32), sl.size, xdiv, rows, K, _p(x, f32), K, int(exact),
                       _p(y, f32), rows)
    return y


class _OrcMoe(C.Structure):
    _fields_ = [("d", C.c_int), ("ff", C.c_int), ("E", C.c_int), ("k", C.c_int)] + \
               [(n, C.POINTER(u16)) for n in ("gs", "gc", "us", "uc", "ds", "dc")] + \
               [(n, C.POINTER(u8)) for n in ("ge", "ue", "de")] + \
               [(n, C.POINTER(i32)) for n in ("geb", "ueb", "deb")]


def moe_layer(layer, x, logits, k):
    """layer: object with d, ff, E and stacked arrays gate/up/down = dict(seeds, coefs, codes, eb)."""
    T = x.shape[0]
    m = _OrcMoe(layer.d, layer.ff, layer.E, k,
                _p(layer.gate["seeds"], u16), _p(layer.gate["coefs"], u16),
                _p(layer.up["seeds"], u16), _p(layer.up["coefs"], u16),
                _p(layer.down["seeds"], u16), _p(layer.down["coefs"], u16),
                _p(layer.gate["codes"], u8), _p(layer.up["codes"], u8), _p(layer.down["codes"], u8),
                _p(layer.gate["eb"], i32), _p(layer.up["eb"], i32), _p(layer.down["eb"], i32))
    x = np.ascontiguousarray(x, np.float32)
    logits = np.ascontiguousarray(logits, np.float32)
    out = np.zeros((T, layer.d), np.float32)
    ind = np.zeros((T, k), np.int32)
    wt = np.zeros((T, k), np.float32)
    lib().orc_moe_layer(C.byref(m), _p(x, f32), _p(logits, f32), T, _p(out, f32), _p(ind, i32), _p(wt, f32))
    return out, ind, wt


def cpu_seed4_matvec(m, x, threads=1, scalar=False):
    tab = table32()
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros(m.rows, np.float32)
    if scalar:
        lib().orc_cpu_seed4_matvec_scalar(_p(m.seeds, u16), _p(m.coefs, u16), _p(m.codes, u8), m.eb, _p(tab, u32),
                                          _p(x, f32), m.rows, m.K // 8, _p(y, f32))
    else:
        lib().orc_cpu_seed4_matvec_mt(_p(m.seeds, u16), _p(m.coefs, u16), _p(m.codes, u8), m.eb, _p(tab, u32),
                                      _p(x, f32), m.rows, m.K // 8, _p(y, f32), threads)
    return y


def cpu_seed4_time(m, x, threads, reps):
    x = np.ascontiguousarray(x, np.float32)
    y = np.zeros(m.rows, np.float32)
    return lib().orc_cpu_seed4_time(_p(m.seeds, u16), _p(m.coefs, u16), _p(m.codes, u8), m.eb, _p(x, f32), m.rows,
                                    m.K // 8, _p(y, f32), threads, reps), y


class Tiled:
    """A Matrix in the CPU-tiled layout (16-row tiles, vector loads): the fastest CPU form of the path."""

    def __init__(self, m):
        L = lib()
        L.orc_cpu_seed4_tile.restype = C.c_void_p
        self.h = L.orc_cpu_seed4_tile(_p(m.seeds, u16), _p(m.coefs, u16), _p(m.codes, u8), m.eb, m.rows, m.K // 8)
        if not self.h:
            raise ValueError("the tiled layout needs an even number of blocks per row")
        self.rows, self.K = m.rows, m.K

    def __del__(self):
        if getattr(self, "h", None):
            lib().orc_cpu_seed4_tiled_free(C.c_void_p(self.h))
            self.h = None

    def matmul(self, x, threads=1):
        """x [ntok][K] (ntok <= 8) -> y [ntok][rows], unrounded f32."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.K)
        y = np.zeros((x.shape[0], self.rows), np.float32)
        rc = lib().orc_cpu_seed4_tiled_matmul_mt(C.c_void_p(self.h), _p(table32(), u32), _p(x, f32), x.shape[0],
                                                 _p(y, f32), threads)
        if rc:
            raise ValueError("1..8 tokens")
        return y

    def time(self, x, threads, reps):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.K)
        y = np.zeros((x.shape[0], self.rows), np.float32)
        L = lib()
        L.orc_cpu_seed4_tiled_time.restype = C.c_double
        return L.orc_cpu_seed4_tiled_time(C.c_void_p(self.h), _p(x, f32), x.shape[0], _p(y, f32), threads, reps), y


class _TiledJob(C.Structure):
    _fields_ = [("m", C.c_void_p), ("x", C.c_void_p), ("ntok", C.c_int), ("y", C.c_void_p)]


def tiled_jobs(jobs, threads):
    """jobs: list of (Tiled, x [ntok][K]); all of them in one parallel region; returns the list of y [ntok][rows]."""
    arr = (_TiledJob * len(jobs))()
    keep, ys = [], []
    for i, (t, x) in enumerate(jobs):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, t.K)
        y = np.zeros((x.shape[0], t.rows), np.float32)
        keep.append(x)
        ys.append(y)
        arr[i] = _TiledJob(t.h, x.ctypes.data, x.shape[0], y.ctypes.data)
    if lib().orc_cpu_seed4_tiled_jobs(arr, len(jobs), _p(table32(), u32), threads):
        raise ValueError("a job has no matrix or more than 8 tokens")
    return ys


def q4_mv(codes, scales, biases, x, add=0, y0=None):
    """The LM head's affine int4 mat-vec: codes u32 [R][K/8], scales / biases bf16 bits [R][K/64], x [T][K] ->
    (y [T][R] bf16-rounded, mag [T][R] = sum |w x|)."""
    codes = np.ascontiguousarray(codes, np.uint32)
    R, K = codes.shape[0], codes.shape[1] * 8
    x = np.ascontiguousarray(x, np.float32).reshape(-1, K)
    T = x.shape[0]
    y = np.zeros((T, R), np.float32) if y0 is None else np.array(y0, np.float32).reshape(T, R).copy()
    mag = np.zeros((T, R), np.float64)
    s, b = np.ascontiguousarray(scales, np.uint16), np.ascontiguousarray(biases, np.uint16)
    lib().orc_q4_mv(codes.ctypes.data_as(C.c_void_p), s.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), K, R,
                    x.ctypes.data_as(C.c_void_p), T, int(add), y.ctypes.data_as(C.c_void_p), mag.ctypes.data_as(C.c_void_p))
    return y, mag


def argmax(logits):
    logits = np.ascontiguousarray(logits, np.float32)
    n, V = logits.shape
    out, prob = np.zeros(n, np.int32), np.zeros(n, np.float64)
    for i in range(n):
        lib().orc_argmax(logits[i].ctypes.data_as(C.c_void_p), V, out[i:].ctypes.data_as(C.c_void_p),
                         prob[i:].ctypes.data_as(C.c_void_p))
    return out, prob


class Matrix3:
    """A seeded P = 3 (SEED4) matrix: seeds and nibble words [rows][K/8] (code in bits 0-3, three int4 coefficients above)."""

    def __init__(self, rows, K, seed, eb=-22):
        rng = np.random.default_rng(seed)
        self.rows, self.K, self.eb = rows, K, eb
        self.seeds = rng.integers(1, 65536, (rows, K // 8)).astype(np.uint16)
        self.nibs = rng.integers(0, 65536, (rows, K // 8)).astype(np.uint16)


def decode3_block_bf16(seed, nib, bias):
    out = np.zeros(8, np.uint16)
    lib().orc_decode3_block_bf16(C.c_uint16(int(seed)), C.c_uint16(int(nib)), int(bias), out.ctypes.data_as(C.c_void_p))
    return out


def decode3_rows_f32(m):
    out = np.zeros((m.rows, m.K), np.float32)
    lib().orc_decode3_rows_f32(m.seeds.ctypes.data_as(C.c_void_p), m.nibs.ctypes.data_as(C.c_void_p), m.eb, m.rows, m.K,
                               out.ctypes.data_as(C.c_void_p))
    return out


def bfr(a):
    """f32 values rounded to bf16 (round to nearest even), as f32."""
    return (f2bf(np.asarray(a, np.float32)).astype(np.uint32) << 16).view(np.float32)


def attn_decode(q, Kc, Vc, pos, kv0, n_kv, scale, g=None):
    """Decode attention in double precision, as the reference's kernel test states it (tests/test_mova_kernels.c:684-712):
    q [T][n_head][128] f32, Kc / Vc bf16 bits [rows][n_kv][128]; row t attends cache rows kv0[t] .. kv0[t] + pos[t]; returns
    the gated, bf16-rounded outputs the kernels are compared with and the ungated double values."""
    q = np.asarray(q, np.float64)
    T, n_head, _ = q.shape
    K = (np.asarray(Kc, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    V = (np.asarray(Vc, np.uint16).astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    att = np.zeros((T, n_head, 128))
    for t in range(T):
        rows = slice(int(kv0[t]), int(kv0[t]) + int(pos[t]) + 1)
        for h in range(n_head):
            kvh = h // (n_head // n_kv)
            s = (K[rows, kvh] @ (q[t, h] * np.float64(np.float32(scale))))
            w = np.exp(s - s.max())
            att[t, h] = (w / w.sum()) @ V[rows, kvh]
    out = bfr(att.astype(np.float32))
    if g is not None:
        out = bfr(out * softplus_gate(np.asarray(g, np.float32)))
    return out, att


def kv_q8_cache(bits):
    """A BF16 cache [rows][n_kv][128] (bit patterns) quantized to the 8-bit KV format as the reference's kernel test does it
    (tests/test_mova_kernels.c:584-604): per (row, head) scale = max|x| / 127 (1 if the row is zero), code = lrintf(x /
    scale), all in f32.  Returns (codes int8, scales f32 [rows][n_kv], the BF16 bits of code * scale: the values a kernel
    reads from this cache)."""
    x = (np.asarray(bits, np.uint16).astype(np.uint32) << 16).view(np.float32)
    m = np.max(np.abs(x), axis=-1)
    sc = np.where(m > 0, (m / np.float32(127.0)).astype(np.float32), np.float32(1.0)).astype(np.float32)
    codes = np.rint((x / sc[..., None]).astype(np.float32)).astype(np.int8)      # rint: halves to even, as lrintf
    deq = (codes.astype(np.float32) * sc[..., None]).astype(np.float32)
    return codes, sc, f2bf(deq).reshape(x.shape)

