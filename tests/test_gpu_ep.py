"""Expert-parallel layer on one GPU (all experts local, no collective): its device steps -- the pair plan on received
bf16 rows, the row-indexed mat-vecs with a device-side pair count, the per-token pre-sum and the rank-order reduce --
against the plain MoE layer and the oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("d,ff,E,k,T", [(2048, 512, 16, 4, 5), (512, 128, 32, 10, 64)])
def test_single_rank_ep_equals_moe_layer(oracle, d, ff, E, k, T):
    import torch
    from nanoseedlm_b200 import ep, moe
    h = moe.HostLayer(oracle, d, ff, E, seed=23)
    layer = moe.DeviceLayer.from_host(h)
    x = oracle.normal(3, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(4, T * E).reshape(T, E)
    m = moe.Moe(layer, k, T)
    m.set_grouped_min_tokens(10 ** 6)
    ref, rind = m.forward_host(x, logits)
    epl = ep.ExpertParallelMoe(ep.CudaBackend(layer), d, k, E, T)
    out = epl.step(torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda())
    torch.cuda.synchronize()
    from nanoseedlm_b200 import lib
    lib.check()
    assert np.max(np.abs(out.cpu().numpy() - ref)) <= 1e-6 * np.max(np.abs(ref))
    oi, _ = oracle.route(logits, k)
    assert np.array_equal(rind, oi)
    m.close()


def test_plan_keeps_local_pairs_in_token_order(oracle):
    import ctypes as C
    import torch
    from nanoseedlm_b200 import lib as L
    n_ranks, t_loc, k, lo, hi = 3, 5, 4, 10, 30
    rng = np.random.default_rng(0)
    stride = t_loc * k + 7
    ind = rng.integers(0, 40, (n_ranks, stride)).astype(np.int32)
    wt = rng.random((n_ranks, stride)).astype(np.float32)
    di, dw = torch.from_numpy(ind).cuda(), torch.from_numpy(wt).cuda()
    T, P = n_ranks * t_loc, n_ranks * t_loc * k
    sel, xrow = torch.zeros(P, dtype=torch.int32, device="cuda"), torch.zeros(P, dtype=torch.int32, device="cuda")
    wsel, off, cnt = torch.zeros(P, device="cuda"), torch.zeros(T + 1, dtype=torch.int32, device="cuda"), torch.zeros(1, dtype=torch.int32, device="cuda")
    L.load().nsl_ep_plan(None, di.data_ptr(), dw.data_ptr(), n_ranks, t_loc, k, stride, 9, lo, hi, sel.data_ptr(),
                         xrow.data_ptr(), wsel.data_ptr(), off.data_ptr(), cnt.data_ptr())
    torch.cuda.synchronize()
    want_sel, want_row, want_w, want_off = [], [], [], []
    for r in range(n_ranks):
        for t in range(t_loc):
            want_off.append(len(want_sel))
            for j in range(k):
                e = int(ind[r, t * k + j])
                if lo <= e < hi:
                    want_sel.append(e - lo); want_row.append(r * 9 + t); want_w.append(wt[r, t * k + j])
    n = len(want_sel)
    assert int(cnt.item()) == n and off.cpu().tolist() == want_off + [n]
    assert sel.cpu().tolist()[:n] == want_sel and xrow.cpu().tolist()[:n] == want_row
    assert np.array_equal(wsel.cpu().numpy()[:n], np.array(want_w, np.float32))


def test_p2p_exchange_single_rank_and_graphs(oracle):
    """The peer-memory exchange with one rank (its own window): several steps, directly and as two CUDA graphs per
    step, equal the plain MoE layer; no wait runs out."""
    import torch
    from nanoseedlm_b200 import ep, lib, moe
    d, ff, E, k, T = 512, 128, 32, 10, 16
    h = moe.HostLayer(oracle, d, ff, E, seed=29)
    layer = moe.DeviceLayer.from_host(h)
    m = moe.Moe(layer, k, T)
    m.set_grouped_min_tokens(10 ** 6)
    xs = [oracle.normal(30 + i, T * d, bf16=True).reshape(T, d) for i in range(3)]
    ls = [oracle.normal(40 + i, T * E).reshape(T, E) for i in range(3)]
    refs = [m.forward_host(x, l)[0].copy() for x, l in zip(xs, ls)]
    epl = ep.ExpertParallelMoe(ep.CudaBackend(layer), d, k, E, T, collectives="p2p")
    dx = [torch.from_numpy(x).cuda() for x in xs]
    dl = [torch.from_numpy(l).cuda() for l in ls]
    for i in (0, 1, 2, 0):
        out = epl.step(dx[i], dl[i]).cpu().numpy()
        assert np.max(np.abs(out - refs[i])) <= 1e-6 * np.max(np.abs(refs[i]))
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        g = ep.GraphedSteps(epl, [layer], list(zip(dx, dl)), whole=[(1, 0), (2, 0)])      # inputs 1 and 2: the whole step as one graph
        assert set(g.whole) == {(1, 0), (2, 0)}
        for i in (2, 1, 0, 1):
            out = g.step(i, 0)
            stream.synchronize()
            assert np.max(np.abs(out.cpu().numpy() - refs[i])) <= 1e-6 * np.max(np.abs(refs[i]))
    assert epl.window.status() == 0
    lib.check()
    epl.window.close()
    m.close()


@pytest.mark.parametrize("fused,mirror", [(False, False), (True, False), (True, True)])
def test_p2p_exchange_four_ranks_driven_from_one_stream(oracle, fused, mirror):
    """Four ranks' windows in one process, their kernels issued on one stream with every rank's producers before any
    rank's consumers (so no kernel ever waits for a later one): dispatch slots, flags, epochs and the owner-indexed
    partial rows all line up with the plain MoE layer over the whole batch, for several steps."""
    import torch
    from nanoseedlm_b200 import ep, lib, moe
    N, d, ff, E, k, t_loc = 4, 512, 128, 32, 10, 6
    T = N * t_loc
    h = moe.HostLayer(oracle, d, ff, E, seed=31)
    m = moe.Moe(moe.DeviceLayer.from_host(h), k, T)
    m.set_grouped_min_tokens(10 ** 6)
    wins = ep.P2PWindow.local_group(N, t_loc, d, k)
    rng = lambda r: (r * E // N, (r + 1) * E // N)
    held = lambda r: [rng(r), rng((r + N // 2) % N)] if mirror else [rng(r)]     # mirrored: the partner's experts too
    eps = [ep.ExpertParallelMoe(ep.CudaBackend(moe.DeviceLayer.from_host_ranges(h, held(r))), d, k, E, t_loc,
                                collectives="p2p", window=wins[r], mirror=mirror) for r in range(N)]
    for step in range(3):
        x = oracle.normal(50 + step, T * d, bf16=True).reshape(T, d)
        logits = oracle.normal(60 + step, T * E).reshape(T, E)
        ref = m.forward_host(x, logits)[0]
        dx, dl = torch.from_numpy(x).cuda(), torch.from_numpy(logits).cuda()
        for r, e in enumerate(eps):
            if fused:      # router + packing + dispatch in one kernel
                e.be.route_pack_dispatch(e, dx[r * t_loc:(r + 1) * t_loc], dl[r * t_loc:(r + 1) * t_loc])
            else:          # a ready-made chunk copied into the windows
                e.be.route_and_pack(e, dx[r * t_loc:(r + 1) * t_loc], dl[r * t_loc:(r + 1) * t_loc])
                e.be.p2p_dispatch(e)
        for e in eps:
            e.be.local_experts(e)
        for e in eps:
            e.be.reduce(e)
        torch.cuda.synchronize()
        out = np.concatenate([e.out.cpu().numpy() for e in eps])
        assert np.max(np.abs(out - ref)) <= 1e-5 * np.max(np.abs(ref))
        counts = [int(e.be.count.item()) for e in eps]
        assert sum(counts) == T * k
        if mirror:      # a pair of ranks splits its joint list in the middle
            assert all(0 <= counts[r] - counts[r + N // 2] <= 1 for r in range(N // 2))
    assert all(w.status() == 0 for w in wins)
    lib.check()
    for w in wins:
        w.close()
    m.close()


def test_p2p_refuses_an_inconsistent_window():
    from nanoseedlm_b200 import ep, lib as L
    w = L.NslEpWindow()
    w.n, w.me, w.t_loc, w.bytes, w.chunk_bytes = 2, 0, 4, 1024, 64
    L.load().nsl_ep_p2p_wait_dispatch(None, w)      # null windows: nothing is launched
    with pytest.raises(RuntimeError, match="inconsistent"):
        L.check()


def test_p2p_wait_runs_out_and_reports():
    """A wait on a counter that nothing bumps (rank 1 of 2 never dispatches) ends by itself after its bound, records which
    rank it waited for, and leaves the stream and the context usable."""
    import time
    import torch
    from nanoseedlm_b200 import ep, lib as L
    t_loc, d, k = 4, 256, 2
    wins = ep.P2PWindow.local_group(2, t_loc, d, k)
    w0 = wins[0].struct()
    chunk = torch.zeros(wins[0].wl["chunk_bytes"], dtype=torch.uint8, device="cuda")
    L.load().nsl_ep_p2p_dispatch(None, w0, chunk.data_ptr())          # rank 0's rows arrive; rank 1's never do
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    L.load().nsl_ep_p2p_wait_dispatch(None, w0)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 1.0 < waited < 10.0                                        # the bound is about two seconds
    assert wins[0].status() == 1 * 256 + (1 + 1)                      # code 1 = dispatch, waited for rank 1
    assert wins[0].status() == 0                                      # reading clears it
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0
    L.check()
    for w in wins:
        w.close()
