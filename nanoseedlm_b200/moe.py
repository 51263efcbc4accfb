"""Synthetic SEED4P4 expert layers and the Python handle of the C host layer (include/nslm_moe.h).

The arithmetic lives in the CUDA library; this module builds inputs (seeded, on the host for oracle-checked cases or
directly on the device for large timing-only layers), owns their device memory through torch, and calls the C entry
points.  Layout of an expert stack: seeds and coefficient words [E][R][K/8] u16, exponent codes [E][R*K/16] u8, one
exponent bias per expert (reference: nslm/model_st.h:13-16), plus the device array of E WSlice entries that the
kernels index by expert id (reference: engine/kernels_cuda.h:19-24, engine/qwen4_cuda.c:197-216)."""
import ctypes as C

import numpy as np
import torch

from . import lib as L
from .kernels import _ptr, dev, stream_table


class ExpertStack:
    def __init__(self, seeds, coefs, codes, eb, R, K):
        """seeds / coefs / codes: device tensors (int16, int16, uint8) shaped [E, ...]; eb: list of E ints."""
        self.E, self.R, self.K = len(eb), R, K
        self.seeds, self.coefs, self.codes, self.eb = seeds, coefs, codes, [int(e) for e in eb]
        arr = (L.WSlice * self.E)()
        for e in range(self.E):
            arr[e].p[0] = seeds[e].data_ptr()
            arr[e].p[1] = coefs[e].data_ptr()
            arr[e].p[2] = 0
            arr[e].p[3] = codes[e].data_ptr()
            arr[e].eb = self.eb[e]
        self.table = torch.empty(self.E * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
        self.table.copy_(torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8))

    @classmethod
    def from_host(cls, seeds, coefs, codes, eb, R, K):
        return cls(dev(np.asarray(seeds, np.uint16)), dev(np.asarray(coefs, np.uint16)), dev(np.asarray(codes, np.uint8)),
                   eb, R, K)

    @classmethod
    def from_blk4(cls, image, E, R, K):
        """A .blk4 expert bank (bytes or a uint8 array) -> its experts on the device, through the library's own ingestion:
        nsl_blk4_split for the streams and nsl_wslice_table for the slice table."""
        lib = L.load()
        img = np.frombuffer(bytes(image), np.uint8) if not isinstance(image, np.ndarray) else np.ascontiguousarray(image, np.uint8)
        nb = R * K // 8
        seeds, coefs = np.zeros((E, nb), np.uint16), np.zeros((E, nb), np.uint16)
        bias, codes = np.zeros(E, np.int32), np.zeros((E, nb // 2), np.uint8)
        if lib.nsl_blk4_split(img.ctypes.data, img.size, E, R, K, seeds.ctypes.data, coefs.ctypes.data, bias.ctypes.data, codes.ctypes.data):
            raise ValueError("not a .blk4 bank of this shape")
        st = cls.__new__(cls)
        st.E, st.R, st.K = E, R, K
        st.seeds, st.coefs, st.codes, st.eb = dev(seeds), dev(coefs), dev(codes), [int(b) for b in bias]
        table = (L.WSlice * E)()
        if lib.nsl_wslice_table(st.seeds.data_ptr(), st.coefs.data_ptr(), st.codes.data_ptr(), bias.ctypes.data, E, R, K, table):
            raise ValueError(L.last_error())
        st.table = torch.empty(E * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
        st.table.copy_(torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8))
        return st

    @classmethod
    def random_on_device(cls, E, R, K, gen, eb=-22):
        nb = R * K // 8
        seeds = torch.randint(1, 65536, (E, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
        coefs = torch.randint(0, 65536, (E, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
        codes = torch.randint(0, 256, (E, nb // 2), generator=gen, device="cuda", dtype=torch.int32).to(torch.uint8)
        return cls(seeds, coefs, codes, [eb] * E, R, K)

    @property
    def nbytes_per_expert(self):
        return self.R * self.K // 8 * 4 + self.R * self.K // 16


class HostLayer:
    """A seeded layer on the host, in the form the oracle reads (oracle.binding.moe_layer)."""

    def __init__(self, oracle, d, ff, E, seed, eb=-22):
        self.d, self.ff, self.E = d, ff, E
        self.gate, self.up, self.down = ({} for _ in range(3))
        for which, (R, K) in (("gate", (ff, d)), ("up", (ff, d)), ("down", (d, ff))):
            nb = R * K // 8
            seeds = np.zeros((E, nb), np.uint16)
            coefs = np.zeros((E, nb), np.uint16)
            codes = np.zeros((E, nb // 2), np.uint8)
            for e in range(E):
                m = oracle.Matrix(R, K, seed * 1000003 + e * 3 + {"gate": 0, "up": 1, "down": 2}[which], eb=eb)
                seeds[e], coefs[e], codes[e] = m.seeds, m.coefs, m.codes
            getattr(self, which).update(seeds=seeds, coefs=coefs, codes=codes, eb=np.full(E, eb, np.int32))

    def matrix(self, oracle, which, e):
        R, K = (self.ff, self.d) if which in ("gate", "up") else (self.d, self.ff)
        src = getattr(self, which)
        m = oracle.Matrix(R, K, 0, eb=int(src["eb"][e]))
        m.seeds[:], m.coefs[:], m.codes[:] = src["seeds"][e], src["coefs"][e], src["codes"][e]
        return m


class DeviceLayer:
    def __init__(self, gate, up, down):
        self.gate, self.up, self.down = gate, up, down
        self.d, self.ff, self.E = gate.K, gate.R, gate.E

    @classmethod
    def from_host(cls, h, lo=0, hi=None):
        """The host layer's experts [lo, hi) (all of them by default) on the device."""
        mk = lambda s, R, K: ExpertStack.from_host(s["seeds"][lo:hi], s["coefs"][lo:hi], s["codes"][lo:hi], s["eb"][lo:hi], R, K)
        return cls(mk(h.gate, h.ff, h.d), mk(h.up, h.ff, h.d), mk(h.down, h.d, h.ff))

    @classmethod
    def concat(cls, a, b):
        """a's experts followed by b's (copies)."""
        cat = lambda x, y: ExpertStack(torch.cat([x.seeds, y.seeds]), torch.cat([x.coefs, y.coefs]), torch.cat([x.codes, y.codes]),
                                       x.eb + y.eb, x.R, x.K)
        return cls(cat(a.gate, b.gate), cat(a.up, b.up), cat(a.down, b.down))

    @classmethod
    def from_host_ranges(cls, h, ranges):
        """The host layer's experts of several [lo, hi) ranges, one after the other (a rank's own experts, then the
        ones it mirrors)."""
        pick = np.concatenate([np.arange(lo, hi) for lo, hi in ranges])
        mk = lambda s, R, K: ExpertStack.from_host(s["seeds"][pick], s["coefs"][pick], s["codes"][pick], s["eb"][pick], R, K)
        return cls(mk(h.gate, h.ff, h.d), mk(h.up, h.ff, h.d), mk(h.down, h.d, h.ff))

    @classmethod
    def random_on_device(cls, d, ff, E, gen):
        return cls(ExpertStack.random_on_device(E, ff, d, gen), ExpertStack.random_on_device(E, ff, d, gen),
                   ExpertStack.random_on_device(E, d, ff, gen))

    @property
    def nbytes_per_expert(self):
        return self.gate.nbytes_per_expert + self.up.nbytes_per_expert + self.down.nbytes_per_expert


class Moe:
    """Handle of the C host layer for one layer shape; set_layer() switches the resident layer it runs."""

    def __init__(self, layer, top_k, max_tokens):
        self.lib = L.load()
        self.layer, self.k, self.max_tokens = layer, top_k, max_tokens
        torch.cuda.synchronize()   # the layer's tensors were written on torch's stream; the C layer uses its own
        self.G = stream_table()
        self.h = self.lib.nsl_moe_create(layer.d, layer.ff, layer.E, top_k, max_tokens, _ptr(layer.gate.table),
                                         _ptr(layer.up.table), _ptr(layer.down.table), _ptr(self.G))
        if not self.h:
            raise RuntimeError(L.last_error() or "nsl_moe_create failed")
        d, E = layer.d, layer.E
        f32 = C.POINTER(C.c_float)
        self.hx = np.ctypeslib.as_array(C.cast(self.lib.nsl_moe_host_x(self.h), f32), (max_tokens, d))
        self.hlogits = np.ctypeslib.as_array(C.cast(self.lib.nsl_moe_host_logits(self.h), f32), (max_tokens, E))
        self.hout = np.ctypeslib.as_array(C.cast(self.lib.nsl_moe_host_out(self.h), f32), (max_tokens, d))

    def set_layer(self, layer):
        self.layer = layer
        self.lib.nsl_moe_set_layer(self.h, _ptr(layer.gate.table), _ptr(layer.up.table), _ptr(layer.down.table))

    def set_grouped_min_tokens(self, t):
        self.lib.nsl_moe_set_grouped_min_tokens(self.h, t)

    def set_rounding(self, bf16_points):
        self.lib.nsl_moe_set_rounding(self.h, int(bf16_points))

    def set_dependent_launch(self, on):
        self.lib.nsl_moe_set_dependent_launch(self.h, int(on))

    def forward_host(self, x, logits):
        """numpy x [T][d], logits [T][E] -> (out [T][d], ind [T][k]) through nsl_moe_forward_host."""
        x = np.ascontiguousarray(x, np.float32)
        logits = np.ascontiguousarray(logits, np.float32)
        T = x.shape[0]
        out = np.zeros((T, self.layer.d), np.float32)
        ind = np.zeros((T, self.k), np.int32)
        rc = self.lib.nsl_moe_forward_host(self.h, x.ctypes.data, logits.ctypes.data, T, out.ctypes.data, ind.ctypes.data)
        if rc:
            raise RuntimeError(L.last_error() or "nsl_moe_forward_host failed")
        L.check()
        return out, ind

    def forward_block(self, block):
        """One full batch from the caller's own pinned block (a pinned torch tensor or an address: max_tokens rows of d floats, then
        max_tokens rows of logits); the result lands in self.hout."""
        ptr = block.data_ptr() if hasattr(block, "data_ptr") else int(block)
        if self.lib.nsl_moe_submit_block(self.h, C.c_void_p(ptr)) or self.lib.nsl_moe_wait(self.h):
            raise RuntimeError(L.last_error() or "nsl_moe_submit_block failed")

    def set_direct_output(self, on):
        """Whether the pinned forms' combine kernel stores straight into the pinned output (default) or a copy brings it."""
        self.lib.nsl_moe_set_direct_output(self.h, int(on))

    def set_one_launch(self, on):
        """Whether a decode step is one launch or (default) three dependent launches."""
        self.lib.nsl_moe_set_one_launch(self.h, int(on))

    def step_status(self):
        """0, or 1 when a wait inside a one-launch step ran out since the last call."""
        return int(self.lib.nsl_moe_step_status(self.h))

    def forward_pinned(self, T):
        """Inputs already in self.hx / self.hlogits; the result lands in self.hout."""
        if self.lib.nsl_moe_forward_pinned(self.h, T):
            raise RuntimeError(L.last_error() or "nsl_moe_forward_pinned failed")

    def submit_pinned(self, T):
        """forward_pinned without the wait: pair with wait(); two Moe objects used alternately overlap their steps."""
        if self.lib.nsl_moe_submit_pinned(self.h, T):
            raise RuntimeError(L.last_error() or "nsl_moe_submit_pinned failed")

    def wait(self):
        if self.lib.nsl_moe_wait(self.h):
            raise RuntimeError("nsl_moe_wait: the stream reported an error")

    def forward_dev(self, x, logits, out, stream=None):
        """Device tensors; enqueues launches on the given (or the current torch) stream."""
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        if self.lib.nsl_moe_forward_dev(self.h, C.c_void_p(s), _ptr(x), _ptr(logits), x.shape[0], _ptr(out)):
            raise RuntimeError(L.last_error() or "nsl_moe_forward_dev failed")

    def close(self):
        if self.h:
            self.lib.nsl_moe_destroy(self.h)
            self.h = None
