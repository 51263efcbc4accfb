"""Worker of tests/test_gpu_ep_multi.py: one process per GPU (torchrun), the expert-parallel step with the peer-memory
exchange against the CPU oracle's layer on this rank's tokens, against the same step with NCCL all-to-alls, and replayed
from CUDA graphs.

A check that fails on one rank must not end that process while the other ranks' kernels may still store into its window
or wait on its counters: failures are collected, every rank drains its stream, the ranks agree on the outcome with an
all-reduce, the windows are closed after a barrier, and only then does a failing rank raise."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from oracle import binding as oracle
    from nanoseedlm_b200 import ep, lib, moe
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    d, ff, E, k, t_loc = 512, 128, 32, 10, 6
    T = world * t_loc
    h = moe.HostLayer(oracle, d, ff, E, seed=37)                     # the same layer on every rank
    lo, hi = rank * E // world, (rank + 1) * E // world
    mine = moe.DeviceLayer.from_host(h, lo, hi)
    p2p = ep.ExpertParallelMoe(ep.CudaBackend(mine), d, k, E, t_loc, collectives="p2p")
    raw = ep.ExpertParallelMoe(ep.CudaBackend(mine, rounding=False), d, k, E, t_loc, collectives="p2p")
    partner = (rank + world // 2) % world
    both = moe.DeviceLayer.from_host_ranges(h, [(lo, hi), (partner * E // world, (partner + 1) * E // world)])
    mir = ep.ExpertParallelMoe(ep.CudaBackend(both), d, k, E, t_loc, collectives="p2p", mirror=True) if world % 2 == 0 else None
    a2a = ep.ExpertParallelMoe(ep.CudaBackend(mine), d, k, E, t_loc, collectives="a2a")
    m = moe.Moe(moe.DeviceLayer.from_host(h), k, T)
    m.set_grouped_min_tokens(10 ** 6)
    failures = []

    def check(ok, what):
        if not ok:
            failures.append(f"rank {rank}: {what}")

    worst, worst_oracle = 0.0, 0.0
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    for step in range(5):
        x = oracle.normal(80 + step, T * d, bf16=True).reshape(T, d)
        logits = oracle.normal(90 + step, T * E).reshape(T, E)
        dx, dl = torch.from_numpy(x[sl]).cuda(), torch.from_numpy(logits[sl]).cuda()
        o1 = p2p.step(dx, dl).clone()
        o2 = a2a.step(dx, dl).clone()
        o4 = raw.step(dx, dl).clone()
        torch.cuda.synchronize()
        check(torch.equal(o1, o2), f"step {step}: p2p and all-to-all results differ")
        ref = m.forward_host(x, logits)[0][sl]
        worst = max(worst, float(np.max(np.abs(o1.cpu().numpy() - ref)) / np.max(np.abs(ref))))
        # f32 throughout against the CPU reference forward on this rank's tokens: the 1e-3 bar, identical routing ids
        oref, oind, _ = oracle.moe_layer(h, x[sl], logits[sl], k)
        check(np.array_equal(raw.be.ind.cpu().numpy(), oind), f"step {step}: routing ids differ from the oracle's")
        worst_oracle = max(worst_oracle, float(np.max(np.abs(o4.cpu().numpy() - oref)) / np.max(np.abs(oref))))
        if mir is not None:      # mirrored pairs of ranks: another split of the same pairs, the same sums up to their order
            o3 = mir.step(dx, dl).clone()
            torch.cuda.synchronize()
            worst = max(worst, float(np.max(np.abs(o3.cpu().numpy() - ref)) / np.max(np.abs(ref))))
    # the same steps replayed from CUDA graphs (two launches per step)
    stream = torch.cuda.Stream()
    x = oracle.normal(99, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(98, T * E).reshape(T, E)
    dx, dl = torch.from_numpy(x[sl]).cuda(), torch.from_numpy(logits[sl]).cuda()
    want = a2a.step(dx, dl).clone()
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.stream(stream):
        g = ep.GraphedSteps(p2p, [mine], [(dx, dl)])
        for _ in range(3):
            out = g.step(0, 0)
        stream.synchronize()
    check(torch.equal(out, want), "graphed p2p step differs")
    dist.barrier()
    with torch.cuda.stream(stream):      # the whole step as one graph
        g1 = ep.GraphedSteps(p2p, [mine], [(dx, dl)], whole=[(0, 0)])
        for _ in range(3):
            out = g1.step(0, 0)
        stream.synchronize()
    check(torch.equal(out, want), "p2p step captured as one graph differs")
    # the whole decoder step with its routed experts behind the window: this rank's rows against the same rows through a
    # decoder that holds every expert locally (same weights on every rank)
    from nanoseedlm_b200 import decoder
    import test_gpu_decoder as TD
    c = dict(TD.CFG, n_exp=8 if 8 % world == 0 else 4 * world)
    hw = TD.make_weights(oracle, moe, c["n_layer"], c["d"], c["n_head"], c["n_kv"], c["n_exp"], c["ff_exp"], c["ff_shared"], c["vocab"], seed=2)
    Td, e_loc = 2, c["n_exp"] // world
    dwin = ep.P2PWindow.create(world, rank, Td, c["d"], c["top_k"])
    dec_ep = decoder.host_decoder(decoder.make_cfg(max_rows=Td, exp_lo=rank * e_loc, exp_hi=(rank + 1) * e_loc, eps=TD.EPS, theta=TD.THETA, **c), hw, dwin)
    dec_1 = decoder.host_decoder(decoder.make_cfg(max_rows=Td, eps=TD.EPS, theta=TD.THETA, **c), hw)
    ids = torch.tensor([3 + rank, 100 + 7 * rank], dtype=torch.int32, device="cuda")
    n1, n2 = torch.zeros(Td, dtype=torch.int32, device="cuda"), torch.zeros(Td, dtype=torch.int32, device="cuda")
    for step in range(3):
        ri = decoder.row_info([step] * Td, [0, c["ctx"]])
        dec_ep.step(ids, ri, Td, n1)
        dec_1.step(ids, ri, Td, n2)
        torch.cuda.synchronize()
        a, b = dec_ep.hidden(Td).cpu().numpy(), dec_1.hidden(Td).cpu().numpy()
        check(np.max(np.abs(a - b)) <= 2e-2 * np.max(np.abs(b)) and np.mean(np.abs(a - b) <= 1e-3 * np.max(np.abs(b))) > 0.9,
              f"decoder step {step}: expert-parallel rows differ from the one-GPU decoder's ({np.max(np.abs(a - b)) / np.max(np.abs(b)):.2e})")
        ids = n2.clone()
    torch.cuda.synchronize()                                          # this rank's kernels have all finished
    status = p2p.window.status() or dwin.status() or raw.window.status() or (mir.window.status() if mir is not None else 0)
    check(status == 0, f"a wait ran out (status {status})")
    check(worst <= 1e-5, f"against the one-GPU layer: {worst}")
    check(worst_oracle <= 1e-3, f"against the oracle: {worst_oracle}")
    err = lib.last_error()
    check(not err, f"library error: {err}")
    bad = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(bad)                                              # every rank has drained and knows the outcome
    dist.barrier()
    dec_ep.close()
    dec_1.close()
    for w in (p2p.window, raw.window, dwin) + ((mir.window,) if mir is not None else ()):
        w.close()
    dist.barrier()
    if failures:
        print("\n".join(failures), file=sys.stderr)
    if rank == 0 and int(bad.item()) == 0:
        print(f"EP_P2P_OK world={world} worst_rel={worst:.2e} worst_vs_oracle={worst_oracle:.2e}")
    dist.destroy_process_group()
    if failures or int(bad.item()):
        sys.exit(1)


if __name__ == "__main__":
    main()
