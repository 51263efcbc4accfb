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
