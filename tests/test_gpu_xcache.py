"""The expert cache's host side (include/nslm_cache.h) on the GPU: a three-layer stack of MoE layers run through the cache
gives the same bits as the same layers with every expert resident -- with either upload path (the copy kernel, or pinned
asynchronous copies on the side stream), with and without the next layer's prefetch, over steps whose routing forces
evictions.  The reference's engine tests make the same statement (tests/test_qwen4_engine.c:514-533, 604-629: cache on /
off and prefetch on / off give identical logits)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def forward(lib, L, G, stream, tables, x, logits, k, d, ff, E, cache=None, mode=0, prefetch=False):
    """x -> layer 0 -> layer 1 -> ...: each layer routes its own logits, runs gate+up+SwiGLU, down and the combine."""
    import torch
    T = x.shape[0]
    P = T * k
    ind = torch.zeros(P, dtype=torch.int32, device="cuda")
    wt = torch.zeros(P, device="cuda")
    A, Dx = torch.zeros(P, ff, device="cuda"), torch.zeros(P, d, device="cuda")
    cur = x.clone()
    s = C.c_void_p(stream.cuda_stream)
    for l, (tg, tu, td) in enumerate(tables):
        if cache is not None and prefetch:
            cache.layer_start(stream.cuda_stream, l, mode)
        lib.nsl_route(s, E, k, logits[l].data_ptr(), E, ind.data_ptr(), wt.data_ptr(), T)
        if cache is not None:
            cache.fetch(stream.cuda_stream, l, ind.data_ptr(), P, mode)
        lib.kc_mv_gu(s, L.MF_SEED4P4, C.c_void_p(tg), C.c_void_p(tu), d, ff, cur.data_ptr(), d, A.data_ptr(), ff, ind.data_ptr(), P, k, G.data_ptr())
        lib.kc_mv_sel(s, L.MF_SEED4P4, C.c_void_p(td), ff, d, A.data_ptr(), ff, Dx.data_ptr(), d, ind.data_ptr(), P, 1, G.data_ptr())
        nxt = torch.zeros(T, d, device="cuda")
        lib.kq4_moe_combine(s, d, k, Dx.data_ptr(), wt.data_ptr(), None, None, 0, nxt.data_ptr(), T)
        stream.synchronize()
        cur = (nxt * 8).bfloat16().float()      # keep the activations bf16-valued and of order one
    return cur.cpu().numpy()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("prefetch", [False, True])
def test_cache_on_off_and_prefetch_on_off_give_identical_results(oracle, mode, prefetch):
    import torch
    from nanoseedlm_b200 import cache, kernels, lib as L, moe
    lib = L.load()
    d, ff, E, NLAY, k, T = 256, 64, 12, 3, 4, 3
    hl = [moe.HostLayer(oracle, d, ff, E, seed=70 + l) for l in range(NLAY)]
    resident = [moe.DeviceLayer.from_host(h) for h in hl]
    res_tables = [(r.gate.table.data_ptr(), r.up.table.data_ptr(), r.down.table.data_ptr()) for r in resident]
    xc = cache.ExpertCache(hl, slots=2 * E + 2)      # 26 of 36 units fit: later layers push earlier ones out
    xc_tables = [tuple(xc.table(l, i) for i in range(3)) for l in range(NLAY)]
    G = kernels.stream_table()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for step in range(4):
            x = torch.from_numpy(oracle.normal(100 + step, T * d, bf16=True).reshape(T, d)).cuda()
            logits = [torch.from_numpy(oracle.normal(200 + 10 * step + l, T * E).reshape(T, E)).cuda() for l in range(NLAY)]
            want = forward(lib, L, G, stream, res_tables, x, logits, k, d, ff, E)
            got = forward(lib, L, G, stream, xc_tables, x, logits, k, d, ff, E, cache=xc, mode=mode, prefetch=prefetch)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), step
    L.check()
    st = xc.stats()
    assert st["misses"] > 0 and st["units"] >= 2 * E + 2 and st["bytes"] == st["units"] * xc.unit_bytes
    if mode == 1:
        assert 0 < st["runs"] <= st["units"]
    xc.close()


def test_prefetch_needs_room_for_two_layers(oracle):
    from nanoseedlm_b200 import cache, lib as L, moe
    hl = [moe.HostLayer(oracle, 64, 64, 4, seed=5 + l) for l in range(2)]
    xc = cache.ExpertCache(hl, slots=5)
    with pytest.raises(RuntimeError, match="two layers"):
        xc.layer_start(0, 0)
    xc.close()
