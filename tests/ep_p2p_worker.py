"""Worker of tests/test_gpu_ep_multi.py: one process per GPU (torchrun), the expert-parallel step with the peer-memory
exchange against the same step with NCCL all-to-alls, and against the plain MoE layer on rank 0's tokens."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


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
    partner = (rank + world // 2) % world
    both = moe.DeviceLayer.from_host_ranges(h, [(lo, hi), (partner * E // world, (partner + 1) * E // world)])
    mir = ep.ExpertParallelMoe(ep.CudaBackend(both), d, k, E, t_loc, collectives="p2p", mirror=True) if world % 2 == 0 else None
    a2a = ep.ExpertParallelMoe(ep.CudaBackend(mine), d, k, E, t_loc, collectives="a2a")
    m = moe.Moe(moe.DeviceLayer.from_host(h), k, T)
    m.set_grouped_min_tokens(10 ** 6)
    worst = 0.0
    for step in range(5):
        x = oracle.normal(80 + step, T * d, bf16=True).reshape(T, d)
        logits = oracle.normal(90 + step, T * E).reshape(T, E)
        sl = slice(rank * t_loc, (rank + 1) * t_loc)
        dx, dl = torch.from_numpy(x[sl]).cuda(), torch.from_numpy(logits[sl]).cuda()
        o1 = p2p.step(dx, dl).clone()
        o2 = a2a.step(dx, dl).clone()
        torch.cuda.synchronize()
        assert torch.equal(o1, o2), f"rank {rank} step {step}: p2p and all-to-all results differ"
        ref = m.forward_host(x, logits)[0][sl]
        worst = max(worst, float(np.max(np.abs(o1.cpu().numpy() - ref)) / np.max(np.abs(ref))))
        if mir is not None:      # mirrored pairs of ranks: another split of the same pairs, the same sums up to their order
            o3 = mir.step(dx, dl).clone()
            torch.cuda.synchronize()
            worst = max(worst, float(np.max(np.abs(o3.cpu().numpy() - ref)) / np.max(np.abs(ref))))
    # the same steps replayed from CUDA graphs (two launches per step)
    stream = torch.cuda.Stream()
    x = oracle.normal(99, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(98, T * E).reshape(T, E)
    sl = slice(rank * t_loc, (rank + 1) * t_loc)
    dx, dl = torch.from_numpy(x[sl]).cuda(), torch.from_numpy(logits[sl]).cuda()
    want = a2a.step(dx, dl).clone()
    torch.cuda.synchronize()
    dist.barrier()
    with torch.cuda.stream(stream):
        g = ep.GraphedSteps(p2p, [mine], [(dx, dl)])
        for _ in range(3):
            out = g.step(0, 0)
        stream.synchronize()
    assert torch.equal(out, want), f"rank {rank}: graphed p2p step differs"
    status = p2p.window.status() or (mir.window.status() if mir is not None else 0)
    lib.check()
    dist.barrier()
    p2p.window.close()
    if mir is not None:
        mir.window.close()
    assert status == 0, f"rank {rank}: a wait ran out (status {status})"
    assert worst <= 1e-5, worst
    if rank == 0:
        print(f"EP_P2P_OK world={world} worst_rel={worst:.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
