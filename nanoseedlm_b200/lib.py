"""ctypes view of libnslm_b200.so: the C ABI declared in include/nslm_kernels.h and include/nslm_moe.h.

There is no fallback: if the library is missing the import of the kernels fails with instructions to build it, and
every call goes to the CUDA kernels.  torch is used only for device memory and streams."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnslm_b200.so")

MF_SEED4P4 = 4
MF_SEED4 = 1
MF_Q4 = 3
MV_MAXT = 8
MMT_BN = 128
MMT_BM = 64


class WSlice(C.Structure):
    _fields_ = [("p", C.c_void_p * 4), ("eb", C.c_int32), ("gs", C.c_int32), ("pad", C.c_int32 * 2)]


class MmTile(C.Structure):
    _fields_ = [("slice", C.c_int32), ("start", C.c_int32), ("count", C.c_int32), ("pad", C.c_int32)]


class CachePool(C.Structure):
    _fields_ = [("unit_slot", C.c_void_p), ("slot_unit", C.c_void_p), ("slot_last", C.c_void_p), ("tick", C.c_void_p),
                ("stats", C.c_void_p), ("jobs", C.c_void_p), ("njobs", C.c_void_p), ("vram", C.c_void_p),
                ("host", C.c_void_p), ("unit_bytes", C.c_uint64), ("slots", C.c_int32), ("per_layer", C.c_int32),
                ("ntens", C.c_int32), ("tab", C.c_void_p), ("off", (C.c_uint32 * 4) * 3), ("hits", C.c_uint64),
                ("misses", C.c_uint64)]


class RouterArgs(C.Structure):
    _fields_ = [("d", C.c_int32), ("n", C.c_int32), ("top_k", C.c_int32), ("hw", C.c_int32), ("scale", C.c_float)]


class HmvArgs(C.Structure):
    _fields_ = [("H", C.c_int32), ("O", C.c_int32), ("I", C.c_int32), ("xs", C.c_int32), ("hs", C.c_int32),
                ("gate", C.c_int32), ("pad", C.c_int32 * 2)]


class AttnArgs(C.Structure):
    _fields_ = [("n_head", C.c_int32), ("n_kv", C.c_int32), ("chunk", C.c_int32), ("n_splits", C.c_int32), ("scale", C.c_float)]


class RowInfo(C.Structure):
    _fields_ = [("pos", C.c_int32), ("kv0", C.c_int32), ("pad", C.c_int32 * 2)]


class KvSeg(C.Structure):
    _fields_ = [("k", C.c_void_p), ("v", C.c_void_p), ("ks", C.c_void_p), ("vs", C.c_void_p)]


class KvView(C.Structure):
    _fields_ = [("a", KvSeg), ("b", KvSeg), ("nv", C.c_int32), ("fmt", C.c_int32)]


assert C.sizeof(AttnArgs) == 20 and C.sizeof(RowInfo) == 16 and C.sizeof(KvView) == 72


class NslEpWindow(C.Structure):
    _fields_ = [("win", C.c_void_p * 16), ("n", C.c_int32), ("me", C.c_int32), ("t_loc", C.c_int32), ("reserved", C.c_int32),
                ("bytes", C.c_uint64),
                ("chunk_bytes", C.c_uint64), ("recv_off", C.c_uint64), ("parts_off", C.c_uint64), ("dflag_off", C.c_uint64),
                ("cflag_off", C.c_uint64), ("local_off", C.c_uint64)]


assert C.sizeof(NslEpWindow) == 200
assert C.sizeof(WSlice) == 48 and C.sizeof(MmTile) == 16 and C.sizeof(RouterArgs) == 20 and C.sizeof(HmvArgs) == 32

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t

# name -> (restype, argtypes): every symbol include/nslm_kernels.h declares
PROTOTYPES = {
    "kc_mv": (None, [_vp, _i, WSlice, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp]),
    "kc_mv_sel": (None, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "kc_mv_gu": (None, [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "kc_seed_gemm_f32": (None, [_i]),
    "kc_mm": (None, [_vp, _i, WSlice, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp]),
    "kc_mm_grouped": (None, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _i, _vp]),
    "kc_bucket": (None, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "kc_mm_grouped_dev": (None, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp]),
    "kc_pack_input_bf16": (None, [_vp, _vp, _vp, _sz]),
    "kc_mm_packed": (None, [_vp, _i, WSlice, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp]),
    "kc_mm_grouped_packed": (None, [_vp, _i, _vp, _i, _i, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp]),
    "kc_swiglu": (None, [_vp, _vp, _vp, _vp, _i]),
    "kc_moe_combine": (None, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "kq4_route": (None, [_vp, _vp, _vp, _vp, _vp, _i]),
    "kq4_route_ld": (None, [_vp, _vp, _vp, _i, _vp, _vp, _i]),
    "kq4_moe_combine": (None, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _i]),
    "kc_router": (None, [_vp, RouterArgs, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "kc_router_topk": (None, [_vp, RouterArgs, _vp, _vp, _vp, _vp, _i]),
    "kc_heads_mv": (None, [_vp, HmvArgs, _i, WSlice, _vp, _vp, _vp, _vp, _i]),
    "kc_heads_deq": (None, [_vp, _i, WSlice, _vp, _i, _i, _i, _vp]),
    "nsl_attn_batch_invariant": (None, [_i]),
    "kc_attn": (None, [_vp, AttnArgs, _vp, KvView, _vp, _vp, _vp, _vp, _i]),
    "kc_argmax": (None, [_vp, _vp, _vp, _i, _i]),
    "kc_argmax_p": (None, [_vp, _vp, _vp, _vp, _i, _i]),
    "kc_cache_admit": (None, [_vp, C.POINTER(CachePool), _i, _vp, _i, _i]),
    "kc_cache_copy": (None, [_vp, C.POINTER(CachePool), _i]),
    "nsl_bucket_noalloc": (None, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "nsl_route": (None, [_vp, _i, _i, _vp, _i, _vp, _vp, _i]),
    "nsl_swiglu_packed": (None, [_vp, _vp, _vp, _vp, _i]),
    "nsl_mv_step": (_i, [_vp, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "nsl_mv_raw": (None, [_vp, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "nsl_mv_gu_raw": (None, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _i, _vp]),
    "nsl_decode_f32": (None, [_vp, WSlice, _i, _i, _vp, _vp]),
    "nsl_decode_bf16": (None, [_vp, WSlice, _i, _i, _vp, _vp]),
    "nsl_decode3_f32": (None, [_vp, WSlice, _i, _i, _vp, _vp]),
    "nsl_decode3_bf16": (None, [_vp, WSlice, _i, _i, _vp, _vp]),
    "nsl_mm_status": (_i, []),
    "nsl_stream_table": (None, [_vp]),
    "nsl_last_error": (C.c_char_p, []),
    "nsl_launch_count": (C.c_uint64, []),
    "nsl_sm_count": (_i, []),
    "nsl_dependent_launch": (None, [_i]),
    "nsl_mv_gu_routed": (None, [_vp, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _i, _i, _vp, _i, _i, _vp, _vp, _i, _vp]),
    # include/nslm_moe.h
    "nsl_moe_create": (_vp, [_i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "nsl_moe_destroy": (None, [_vp]),
    "nsl_moe_set_layer": (None, [_vp, _vp, _vp, _vp]),
    "nsl_moe_set_grouped_min_tokens": (None, [_vp, _i]),
    "nsl_moe_forward_dev": (_i, [_vp, _vp, _vp, _vp, _i, _vp]),
    "nsl_moe_forward_host": (_i, [_vp, _vp, _vp, _i, _vp, _vp]),
    "nsl_moe_host_x": (_vp, [_vp]),
    "nsl_moe_host_logits": (_vp, [_vp]),
    "nsl_moe_host_out": (_vp, [_vp]),
    "nsl_moe_forward_pinned": (_i, [_vp, _i]),
    "nsl_moe_submit_pinned": (_i, [_vp, _i]),
    "nsl_moe_submit_block": (_i, [_vp, _vp]),
    "nsl_moe_wait": (_i, [_vp]),
    "nsl_moe_dev_ind": (_vp, [_vp]),
    "nsl_moe_dev_wt": (_vp, [_vp]),
    "nsl_moe_stream": (_vp, [_vp]),
    "nsl_moe_set_rounding": (None, [_vp, _i]),
    "nsl_moe_set_dependent_launch": (None, [_vp, _i]),
    "nsl_moe_set_direct_output": (None, [_vp, _i]),
    "nsl_moe_set_one_launch": (None, [_vp, _i]),
    "nsl_moe_step_status": (_i, [_vp]),
    # include/nslm_pack.h
    "nsl_blk4_bytes": (_sz, [_i, _i, _i]),
    "nsl_blk4_split": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "nsl_blk4_join": (_i, [_vp, _sz, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "nsl_wslice_table": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    # include/nslm_ep.h
    "nsl_ep_plan": (None, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "nsl_mv_gu_rows": (None, [_vp, _vp, _vp, _i, _i, _vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _vp]),
    "nsl_mv_sel_rows": (None, [_vp, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _i, _vp, _i, _vp]),
    "nsl_ep_combine": (None, [_vp, _vp, _vp, _vp, _i, _i, _vp]),
    "nsl_ep_reduce": (None, [_vp, _vp, _i, _i, _i, _vp]),
    "nsl_ep_window_alloc": (_i, [_sz, C.POINTER(C.c_void_p), _vp]),
    "nsl_ep_window_open": (_i, [_vp, C.POINTER(C.c_void_p)]),
    "nsl_ep_window_close": (_i, [_vp]),
    "nsl_ep_window_free": (_i, [_vp]),
    "nsl_ep_p2p_dispatch": (None, [_vp, NslEpWindow, _vp]),
    "nsl_ep_p2p_wait_dispatch": (None, [_vp, NslEpWindow]),
    "nsl_ep_p2p_plan": (None, [_vp, NslEpWindow, C.c_uint64, C.c_uint64, _i, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "nsl_ep_p2p_route_dispatch": (None, [_vp, NslEpWindow, _i, _i, _vp, _i, _vp, _i, C.c_uint64, C.c_uint64, _vp, _vp]),
    "nsl_ep_p2p_combine": (None, [_vp, NslEpWindow, _vp, _vp, _vp, _i]),
    "nsl_ep_p2p_reduce": (None, [_vp, NslEpWindow, _i, _vp]),
    "nsl_ep_p2p_status": (_i, [NslEpWindow]),
    # include/nslm_decoder.h
    "nsl_decoder_create": (_vp, [_vp, _vp, WSlice, _vp, WSlice, _vp, _vp]),
    "nsl_decoder_destroy": (None, [_vp]),
    "nsl_decoder_step": (_i, [_vp, _vp, _vp, _vp, _i, _vp]),
    "nsl_decoder_hidden": (_vp, [_vp]),
    "nsl_decoder_logits": (_vp, [_vp]),
    "nsl_decoder_copy_out": (_i, [_vp, _i, _i, _vp]),
    "nsl_decoder_kcache": (_vp, [_vp, _i]),
    "nsl_decoder_vcache": (_vp, [_vp, _i]),
    "nsl_decoder_fill_cache": (_i, [_vp, _i, _vp, _vp, _sz]),
    "nsl_residual_add": (None, [_vp, _vp, _vp, _sz]),
    "kc_embed": (None, [_vp, _i, WSlice, _i, _vp, _vp, _i]),
    "kc_gnorm": (None, [_vp, _i, C.c_float, _vp, _vp, _vp, _i]),
    "kc_rope_kv": (None, [_vp, _vp, _vp, _vp, KvView, _vp, _vp, _i, _i, _i]),
    # include/nslm_cache.h
    "nsl_xcache_create": (_vp, [_i, _i, _vp, _i]),
    "nsl_xcache_destroy": (None, [_vp]),
    "nsl_xcache_host_unit": (_vp, [_vp, _i]),
    "nsl_xcache_offset": (C.c_uint32, [_vp, _i, _i]),
    "nsl_xcache_unit_bytes": (C.c_uint64, [_vp]),
    "nsl_xcache_finish": (_i, [_vp, _vp]),
    "nsl_xcache_table": (_vp, [_vp, _i, _i]),
    "nsl_xcache_pool": (_vp, [_vp]),
    "nsl_xcache_fetch": (_i, [_vp, _vp, _i, _vp, _i, _i]),
    "nsl_xcache_prefetch": (_i, [_vp, _vp, _i, _i]),
    "nsl_xcache_layer_start": (_i, [_vp, _vp, _i, _i]),
    "nsl_xcache_stats": (_i, [_vp, _vp, _vp, _vp, _vp, _vp]),
    "nsl_xcache_set_ops": (None, [_vp]),
}

_lib = None


def load():
    """The library handle with every prototype set.  Raises when the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: run `python -m nanoseedlm_b200.build` (there is no CPU path)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(lib, name)   # AttributeError if the library does not export a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def last_error():
    return load().nsl_last_error().decode()


def check():
    """Raise if a call since the last check was refused for its arguments."""
    msg = last_error()
    if msg:
        raise RuntimeError(msg)
