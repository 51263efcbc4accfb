"""Python handle of the expert cache's host side (include/nslm_cache.h): the pinned arena of all experts' units, the pool of
VRAM slots, and the two upload paths (the copy kernel reading the arena over PCIe, or pinned asynchronous copies on a side
stream).  The reference builds the same around its kc_cache_* kernels in engine/qwen4_cuda.c:368-451 and :1143-1162."""
import ctypes as C

import numpy as np

from . import lib as L

KERNEL, DMA = 0, 1


class ExpertCache:
    @classmethod
    def random(cls, layers, E, d, ff, slots, seed=0):
        """A cache whose arena holds random bytes (timing of the upload paths; no oracle involved)."""
        self = cls.__new__(cls)
        self.lib = L.load()
        self.layers, self.E, self.d, self.ff = layers, E, d, ff
        lens = np.zeros((3, 4), np.uint64)
        for i, (R, K) in enumerate(((ff, d), (ff, d), (d, ff))):
            lens[i] = [R * K // 8 * 2, R * K // 8 * 2, 0, R * K // 16]
        self.h = self.lib.nsl_xcache_create(layers, E, lens.ctypes.data, slots)
        if not self.h:
            raise RuntimeError(L.last_error() or "nsl_xcache_create failed")
        ub = self.unit_bytes = self.lib.nsl_xcache_unit_bytes(self.h)
        rng = np.random.default_rng(seed)
        whole = np.ctypeslib.as_array(C.cast(self.lib.nsl_xcache_host_unit(self.h, 0), C.POINTER(C.c_uint8)), (ub * layers * E,))
        block = rng.integers(0, 256, 1 << 24, dtype=np.uint8)
        for o in range(0, whole.size, block.size):
            n = min(block.size, whole.size - o)
            whole[o:o + n] = block[:n]
        if self.lib.nsl_xcache_finish(self.h, None):
            raise RuntimeError(L.last_error() or "nsl_xcache_finish failed")
        return self

    def __init__(self, host_layers, slots):
        """host_layers: moe.HostLayer objects of one shape (every expert's gate / up / down streams on the host)."""
        self.lib = L.load()
        h0 = host_layers[0]
        self.layers, self.E, self.d, self.ff = len(host_layers), h0.E, h0.d, h0.ff
        lens = np.zeros((3, 4), np.uint64)
        for i, (R, K) in enumerate(((h0.ff, h0.d), (h0.ff, h0.d), (h0.d, h0.ff))):
            lens[i] = [R * K // 8 * 2, R * K // 8 * 2, 0, R * K // 16]
        self.h = self.lib.nsl_xcache_create(self.layers, self.E, lens.ctypes.data, slots)
        if not self.h:
            raise RuntimeError(L.last_error() or "nsl_xcache_create failed")
        ub = self.lib.nsl_xcache_unit_bytes(self.h)
        eb = np.zeros((self.layers, 3, self.E), np.int32)
        for l, h in enumerate(host_layers):
            for i, st in enumerate((h.gate, h.up, h.down)):
                eb[l, i] = st["eb"]
                for x in range(self.E):
                    unit = np.ctypeslib.as_array(C.cast(self.lib.nsl_xcache_host_unit(self.h, l * self.E + x), C.POINTER(C.c_uint8)), (ub,))
                    for s, key in ((0, "seeds"), (1, "coefs"), (3, "codes")):
                        off = self.lib.nsl_xcache_offset(self.h, i, s)
                        raw = np.ascontiguousarray(st[key][x]).view(np.uint8).ravel()
                        unit[off:off + raw.size] = raw
        if self.lib.nsl_xcache_finish(self.h, eb.ctypes.data):
            raise RuntimeError(L.last_error() or "nsl_xcache_finish failed")
        self.unit_bytes = ub

    def table(self, layer, tensor):
        """Device address of the layer's WSlice table for tensor 0 (gate), 1 (up) or 2 (down)."""
        return self.lib.nsl_xcache_table(self.h, layer, tensor)

    def fetch(self, stream, layer, inds, count, mode=KERNEL):
        if self.lib.nsl_xcache_fetch(self.h, C.c_void_p(stream), layer, C.c_void_p(inds), count, mode):
            raise RuntimeError(L.last_error() or "nsl_xcache_fetch failed")

    def layer_start(self, stream, layer, mode=KERNEL):
        if self.lib.nsl_xcache_layer_start(self.h, C.c_void_p(stream), layer, mode):
            raise RuntimeError(L.last_error() or "nsl_xcache_layer_start failed")

    def stats(self):
        v = (C.c_uint64 * 5)()
        p = [C.byref(v, 8 * i) for i in range(5)]
        if self.lib.nsl_xcache_stats(self.h, *[C.cast(q, C.c_void_p) for q in p]):
            raise RuntimeError(L.last_error() or "nsl_xcache_stats failed")
        return dict(zip(("hits", "misses", "units", "bytes", "runs"), [int(x) for x in v]))

    def close(self):
        if self.h:
            self.lib.nsl_xcache_destroy(self.h)
            self.h = None
