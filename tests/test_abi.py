"""The C-ABI library loads and exports every symbol include/nslm_kernels.h declares (no compute calls).  No GPU."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = ""
    for name in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if name.endswith(".h"):
            text += open(os.path.join(ROOT, "include", name)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:kc|kq4|nsl)_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("kc_mv", "kc_mv_sel", "kc_mv_gu", "kc_mm_grouped_dev", "kc_bucket", "kc_cache_admit", "kc_cache_copy",
                 "kq4_route_ld", "kq4_moe_combine", "kc_swiglu", "kc_moe_combine", "kc_pack_input_bf16"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from nanoseedlm_b200 import build, lib
    if not os.path.exists(lib.LIB_PATH):
        build.build_library()
    handle = C.CDLL(lib.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(handle, n)]
    assert not missing, missing
    assert sorted(lib.PROTOTYPES) == declared_symbols()


def test_struct_layouts_match_the_reference_abi():
    from nanoseedlm_b200 import lib
    assert C.sizeof(lib.WSlice) == 48 and lib.WSlice.eb.offset == 32        # engine/kernels_cuda.h:19-24
    assert C.sizeof(lib.MmTile) == 16                                        # engine/kernels_moe.metal:130
    assert lib.CachePool.unit_bytes.offset == 72 and lib.CachePool.tab.offset == 96   # engine/kernels_cuda.h:32-47
    assert lib.CachePool.off.offset == 104 and C.sizeof(lib.CachePool) == 168


def test_host_stream_table_matches_oracle(oracle):
    import numpy as np
    from nanoseedlm_b200 import lib
    t = np.zeros(65536, np.uint32)
    lib.load().nsl_stream_table(C.c_void_p(t.ctypes.data))
    assert np.array_equal(t, oracle.table32())
