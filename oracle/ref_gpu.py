"""ctypes binding of the reference's own CUDA kernels (oracle/_ref/libnslm_ref_gpu.so: engine/kernels_moe.cu and
engine/kernels_qwen4.cu compiled unmodified for sm_100a by oracle/Makefile).  TEST INFRASTRUCTURE ONLY: the GPU tests and the
bench's `ref_gpu` leg call it as the thing this library is compared with; nothing in the product imports it.

The two libraries export the same kc_* / kq4_* names with the same argument structs (that is the drop-in boundary), so the
prototypes are the product's own table (nanoseedlm_b200.lib.PROTOTYPES), restricted to what the reference exports."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "_ref", "libnslm_ref_gpu.so")
_LIB = None


def available():
    return os.path.exists(PATH)


def lib():
    """The reference kernels' library with prototypes set, or None when it was not built (it builds where the reference's
    sources and nvcc are)."""
    global _LIB
    if _LIB is None and available():
        from nanoseedlm_b200 import lib as L
        h = C.CDLL(PATH)
        for name, (res, args) in L.PROTOTYPES.items():
            if not name.startswith(("kc_", "kq4_")):
                continue
            try:
                fn = getattr(h, name)
            except AttributeError:
                continue
            fn.restype, fn.argtypes = res, args
        _LIB = h
    return _LIB


def qwen4_cfg(n_exp, top_k):
    """A block shaped like the reference's Qwen4Cfg (nslm/qwen4_cfg.h:9-22) with the two fields kq4_route reads."""
    import numpy as np
    cfg = np.zeros(128, np.int32)
    cfg[21], cfg[22] = n_exp, top_k
    return cfg
