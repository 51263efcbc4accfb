"""Empty inputs through the C ABI: zero pairs, zero tokens, zero tiles.  Nothing may be launched with an empty grid (a CUDA
launch error), nothing written, no error recorded; the reference's hosts make such calls (a layer whose rows all miss a
rank, a batch of zero prompt rows: engine/qwen4_cuda.c:1058-1078 runs with whatever P the step has)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_empty_calls_launch_nothing_and_record_no_error(oracle):
    import torch
    from nanoseedlm_b200 import kernels, lib as L, moe
    lib = L.load()
    d, ff, E = 256, 64, 4
    lay = moe.DeviceLayer.from_host(moe.HostLayer(oracle, d, ff, E, seed=3))
    G = kernels.stream_table()
    x = torch.ones(4, d, device="cuda")
    y = torch.full((4, d), 7.0, device="cuda")
    a = torch.full((4, ff), 7.0, device="cuda")
    sel = torch.zeros(4, dtype=torch.int32, device="cuda")
    wt = torch.ones(4, device="cuda")
    before = lib.nsl_launch_count()
    w0 = L.WSlice()
    w0.p[0], w0.p[1], w0.p[3], w0.eb = lay.gate.seeds[0].data_ptr(), lay.gate.coefs[0].data_ptr(), lay.gate.codes[0].data_ptr(), lay.gate.eb[0]
    lib.kc_mv(None, L.MF_SEED4P4, w0, d, ff, x.data_ptr(), d, a.data_ptr(), ff, 0, 0, G.data_ptr())                       # no tokens
    lib.kc_mv_sel(None, L.MF_SEED4P4, lay.down.table.data_ptr(), ff, d, a.data_ptr(), ff, y.data_ptr(), d, sel.data_ptr(), 0, 1, G.data_ptr())
    lib.kc_mv_gu(None, L.MF_SEED4P4, lay.gate.table.data_ptr(), lay.up.table.data_ptr(), d, ff, x.data_ptr(), d, a.data_ptr(), ff,
                 sel.data_ptr(), 0, 1, G.data_ptr())
    lib.kc_mm(None, L.MF_SEED4P4, w0, d, ff, x.data_ptr(), d, a.data_ptr(), ff, 0, 0, G.data_ptr())
    lib.kc_mm_grouped(None, L.MF_SEED4P4, lay.gate.table.data_ptr(), d, ff, x.data_ptr(), d, a.data_ptr(), ff, 1, sel.data_ptr(), None, 0,
                      G.data_ptr())
    lib.kc_swiglu(None, a.data_ptr(), a.data_ptr(), a.data_ptr(), 0)
    lib.kq4_moe_combine(None, d, 2, y.data_ptr(), wt.data_ptr(), None, None, 0, y.data_ptr(), 0)
    lib.kc_moe_combine(None, y.data_ptr(), wt.data_ptr(), y.data_ptr(), y.data_ptr(), d, 2, 0)
    lib.nsl_route(None, E, 2, x.data_ptr(), E, sel.data_ptr(), wt.data_ptr(), 0)
    lib.kc_argmax(None, x.data_ptr(), sel.data_ptr(), d, 0)
    lib.kc_pack_input_bf16(None, x.data_ptr(), a.data_ptr(), 0)
    kv = L.KvView()
    lib.kc_attn(None, L.AttnArgs(8, 2, 64, 4, 0.1), None, kv, None, None, None, None, 0)
    torch.cuda.synchronize()      # a launch with an empty grid would surface here
    L.check()
    assert lib.nsl_launch_count() == before
    assert float(y.min()) == 7.0 and float(a.min()) == 7.0


def test_bucket_of_no_pairs_gives_no_tiles(oracle):
    from nanoseedlm_b200 import kernels
    perm, tiles, nt = kernels.kt_bucket(np.zeros(0, np.int32), 8)
    assert nt == 0 and tiles == [] and perm.size == 0
