"""Python handle of the decoder's host side (include/nslm_decoder.h) and builders of synthetic decoders: random-init weights
of BASELINE config 4's architecture, made on the device for timing or from host arrays for oracle-checked tests."""
import ctypes as C

import numpy as np
import torch

from . import lib as L
from .kernels import SeedWeight, _ptr, dev, stream_table
from .moe import DeviceLayer, ExpertStack


class NslDecoderCfg(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layer", "d", "n_head", "n_kv", "n_exp", "top_k", "ff_exp", "ff_shared", "vocab", "max_rows",
                                         "ctx", "exp_lo", "exp_hi")] + [("eps", C.c_float), ("rope_theta", C.c_float), ("dense_bf16", C.c_int32)]


class NslDecoderLayer(C.Structure):
    _fields_ = [("norm_attn", C.c_void_p), ("norm_ffn", C.c_void_p), ("wq", L.WSlice), ("wk", L.WSlice), ("wv", L.WSlice), ("wo", L.WSlice),
                ("router", L.WSlice), ("eg", C.c_void_p), ("eu", C.c_void_p), ("ed", C.c_void_p), ("sg", L.WSlice), ("su", L.WSlice),
                ("sd", L.WSlice)]


def _dense_random(R, K, gen, eb=-22):
    """One dense SEED4P4 matrix with random streams on the device -> (WSlice, tensors to keep alive)."""
    st = ExpertStack.random_on_device(1, R, K, gen, eb=eb)
    w = L.WSlice()
    w.p[0], w.p[1], w.p[3], w.eb = st.seeds[0].data_ptr(), st.coefs[0].data_ptr(), st.codes[0].data_ptr(), eb
    return w, st


def _dense_host(m):
    sw = SeedWeight.from_matrices([m])
    return sw.slice(0), sw


class Decoder:
    def __init__(self, cfg, layers, embed, norm_out, head, keep, win=None):
        """cfg: NslDecoderCfg; layers: list of NslDecoderLayer; embed / head: WSlice; norm_out: device tensor; keep: whatever owns
        the device memory the structures point at; win: an ep.P2PWindow, or None."""
        self.lib = L.load()
        self.cfg, self.keep, self.G = cfg, keep, stream_table()
        arr = (NslDecoderLayer * len(layers))(*layers)
        w = C.byref(win.struct()) if win is not None else None
        self.h = self.lib.nsl_decoder_create(C.byref(cfg), arr, embed, _ptr(norm_out), head, _ptr(self.G), w)
        if not self.h:
            raise RuntimeError(L.last_error() or "nsl_decoder_create failed")

    def step(self, ids, ri, T, nxt, stream=None):
        """ids (int32 [T]), ri (RowInfo bytes, 16 T) and nxt (int32 [T]) are device tensors; only launches are enqueued."""
        s = stream if stream is not None else torch.cuda.current_stream().cuda_stream
        if self.lib.nsl_decoder_step(C.c_void_p(self.h), C.c_void_p(s), _ptr(ids), _ptr(ri), T, _ptr(nxt)):
            raise RuntimeError(L.last_error() or "nsl_decoder_step failed")

    def hidden(self, T):
        """The last step's final hidden rows [T][d] (before the output norm)."""
        out = torch.empty(T, self.cfg.d, device="cuda")
        if self.lib.nsl_decoder_copy_out(C.c_void_p(self.h), 0, T, _ptr(out)):
            raise RuntimeError("nsl_decoder_copy_out failed")
        return out

    def logits(self, T):
        out = torch.empty(T, self.cfg.vocab, device="cuda")
        if self.lib.nsl_decoder_copy_out(C.c_void_p(self.h), 1, T, _ptr(out)):
            raise RuntimeError("nsl_decoder_copy_out failed")
        return out

    def fill_cache(self, layer, k, v):
        """k / v: bf16 device tensors copied into the start of the layer's caches."""
        if self.lib.nsl_decoder_fill_cache(C.c_void_p(self.h), layer, _ptr(k), _ptr(v), k.numel()):
            raise RuntimeError(L.last_error() or "nsl_decoder_fill_cache failed")

    def close(self):
        if self.h:
            self.lib.nsl_decoder_destroy(C.c_void_p(self.h))
            self.h = None


def row_info(pos, kv0):
    """RowInfo array as a device byte tensor."""
    ri = (L.RowInfo * len(pos))()
    for t, (p, k) in enumerate(zip(pos, kv0)):
        ri[t].pos, ri[t].kv0 = int(p), int(k)
    out = torch.empty(16 * len(pos), dtype=torch.uint8, device="cuda")
    out.copy_(torch.frombuffer(bytearray(bytes(ri)), dtype=torch.uint8))
    return out


def make_cfg(n_layer, d, n_head, n_kv, n_exp, top_k, ff_exp, ff_shared, vocab, max_rows, ctx, exp_lo=0, exp_hi=None, eps=1e-6, theta=1e6,
             dense_bf16=0):
    return NslDecoderCfg(n_layer, d, n_head, n_kv, n_exp, top_k, ff_exp, ff_shared, vocab, max_rows, ctx, exp_lo,
                         n_exp if exp_hi is None else exp_hi, eps, theta, dense_bf16)


def random_decoder(cfg, seed=0, win=None):
    """Random-init weights of the configured architecture, generated on the device (timing)."""
    gen = torch.Generator(device="cuda").manual_seed(seed)
    gen_exp = torch.Generator(device="cuda").manual_seed(seed * 1000 + 17 + cfg.exp_lo)      # a rank's own experts
    d, HQ, HK = cfg.d, cfg.n_head * 128, cfg.n_kv * 128
    keep, layers = [], []
    bf16_ones = lambda n: (torch.rand(n, generator=gen, device="cuda") * 0.2 + 0.9).to(torch.bfloat16)
    for _ in range(cfg.n_layer):
        lay = NslDecoderLayer()
        na, nf = bf16_ones(d), bf16_ones(d)
        lay.norm_attn, lay.norm_ffn = na.data_ptr(), nf.data_ptr()
        ws = {}
        for name, (R, K) in (("wq", (HQ, d)), ("wk", (HK, d)), ("wv", (HK, d)), ("wo", (d, HQ)), ("router", (cfg.n_exp + 1, d)),
                             ("sg", (cfg.ff_shared, d)), ("su", (cfg.ff_shared, d)), ("sd", (d, cfg.ff_shared))):
            w, st = _dense_random(R, K, gen)
            setattr(lay, name, w)
            ws[name] = st
        ex = DeviceLayer.random_on_device(d, cfg.ff_exp, cfg.exp_hi - cfg.exp_lo, gen_exp)
        lay.eg, lay.eu, lay.ed = ex.gate.table.data_ptr(), ex.up.table.data_ptr(), ex.down.table.data_ptr()
        keep += [na, nf, ws, ex]
        layers.append(lay)
    table = (torch.randn(cfg.vocab, d, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    embed = L.WSlice()
    embed.p[0] = table.data_ptr()
    norm_out = bf16_ones(d)
    codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (cfg.vocab, d // 8), generator=gen, device="cuda", dtype=torch.int32)
    sc = (torch.rand(cfg.vocab, d // 64, generator=gen, device="cuda") * 0.02 + 0.001).to(torch.bfloat16)
    bi = (torch.rand(cfg.vocab, d // 64, generator=gen, device="cuda") * -0.2).to(torch.bfloat16)
    head = L.WSlice()
    head.p[0], head.p[1], head.p[2] = codes.data_ptr(), sc.data_ptr(), bi.data_ptr()
    keep += [table, norm_out, codes, sc, bi]
    torch.cuda.synchronize()
    return Decoder(cfg, layers, embed, norm_out, head, keep, win)


def host_decoder(cfg, hw, win=None):
    """A decoder from host weights hw (tests): hw["layers"][l] = dict(norm_attn, norm_ffn (uint16 [d]), wq, wk, wv, wo, router, sg,
    su, sd (oracle matrices), experts (a moe.HostLayer)); hw["embed"] uint16 [vocab][d]; hw["norm_out"]; hw["head"] = (codes,
    scales, biases)."""
    keep, layers = [], []
    for hl in hw["layers"]:
        lay = NslDecoderLayer()
        na, nf = dev(hl["norm_attn"]), dev(hl["norm_ffn"])
        lay.norm_attn, lay.norm_ffn = na.data_ptr(), nf.data_ptr()
        for name in ("wq", "wk", "wv", "wo", "router", "sg", "su", "sd"):
            w, sw = _dense_host(hl[name])
            setattr(lay, name, w)
            keep.append(sw)
        ex = DeviceLayer.from_host(hl["experts"], cfg.exp_lo, cfg.exp_hi)
        lay.eg, lay.eu, lay.ed = ex.gate.table.data_ptr(), ex.up.table.data_ptr(), ex.down.table.data_ptr()
        keep += [na, nf, ex]
        layers.append(lay)
    table = dev(hw["embed"])
    embed = L.WSlice()
    embed.p[0] = table.data_ptr()
    norm_out = dev(hw["norm_out"])
    codes, sc, bi = (dev(a) for a in hw["head"])
    head = L.WSlice()
    head.p[0], head.p[1], head.p[2] = codes.data_ptr(), sc.data_ptr(), bi.data_ptr()
    keep += [table, norm_out, codes, sc, bi]
    torch.cuda.synchronize()
    return Decoder(cfg, layers, embed, norm_out, head, keep, win)
