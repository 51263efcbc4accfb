"""The expert-parallel dispatch / combine plumbing on 2 CPU ranks (gloo): every rank's output equals the single-rank
result for its tokens.  The device steps are replaced by the oracle (tests/ep_cpu_backend.py).  No GPU."""
import os
import sys
import tempfile

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _worker(rank, world, store_path, d, ff, E, k, t_loc, out_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, HERE)
    from oracle import binding as B
    from nanoseedlm_b200 import ep, moe
    from ep_cpu_backend import OracleBackend
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
    h = moe.HostLayer(B, d, ff, E, seed=17)
    e_loc = E // world
    layer = ep.ExpertParallelMoe(OracleBackend(B, h, rank * e_loc, (rank + 1) * e_loc), d, k, E, t_loc)
    T = world * t_loc
    x = B.normal(5, T * d, bf16=True).reshape(T, d)
    logits = B.normal(6, T * E).reshape(T, E)
    mine = slice(rank * t_loc, (rank + 1) * t_loc)
    for _ in range(2):   # twice: the buffers are reused
        out = layer.step(torch.from_numpy(x[mine].copy()), torch.from_numpy(logits[mine].copy())).numpy().copy()
    np.save(out_path + f".{rank}.npy", out)
    dist.destroy_process_group()


def test_two_ranks_equal_single_rank(oracle):
    from nanoseedlm_b200 import moe
    d, ff, E, k, t_loc, world = 128, 64, 8, 3, 3, 2
    with tempfile.TemporaryDirectory() as tmp:
        store, outp = os.path.join(tmp, "store"), os.path.join(tmp, "out")
        mp.spawn(_worker, args=(world, store, d, ff, E, k, t_loc, outp), nprocs=world, join=True)
        got = np.concatenate([np.load(outp + f".{r}.npy") for r in range(world)])
    h = moe.HostLayer(oracle, d, ff, E, seed=17)
    T = world * t_loc
    x = oracle.normal(5, T * d, bf16=True).reshape(T, d)
    logits = oracle.normal(6, T * E).reshape(T, E)
    ind, wt = oracle.route(logits, k)
    ref = np.zeros((T, d), np.float32)
    for t in range(T):
        for j in range(k):
            e = int(ind[t, j])
            a = oracle.mv_gu(h.matrix(oracle, "gate", e), h.matrix(oracle, "up", e), x[t])
            ref[t] += wt[t, j] * oracle.mv(h.matrix(oracle, "down", e), a)[0]
    assert np.max(np.abs(got - ref)) <= 1e-5 * np.max(np.abs(ref))   # summation order differs (per-rank partial sums)


def test_chunk_layout_is_whole_rows():
    from nanoseedlm_b200 import ep
    for t_loc, d, k in ((8, 2048, 10), (64, 2048, 10), (3, 128, 3), (1, 64, 32)):
        lay = ep.chunk_layout(t_loc, d, k)
        assert lay["bytes"] % lay["row"] == 0 and lay["ind_off"] % 4 == 0 and lay["wt_off"] % 4 == 0
        assert lay["wt_off"] + 4 * t_loc * k <= lay["bytes"] and lay["rows"] * lay["row"] == lay["bytes"]


def test_window_layout_is_aligned_and_disjoint():
    """The peer-memory window: every area starts on its alignment, areas do not overlap, flags sit 128 bytes apart."""
    from nanoseedlm_b200 import ep
    for N, t_loc, d, k in [(1, 64, 2048, 10), (2, 32, 2048, 10), (8, 8, 2048, 10), (4, 6, 512, 10), (16, 4, 256, 3)]:
        wl, lay = ep.window_layout(N, t_loc, d, k), ep.chunk_layout(t_loc, d, k)
        assert wl["chunk_bytes"] == lay["bytes"] and wl["chunk_bytes"] % 16 == 0
        areas = [(wl["recv_off"], N * wl["chunk_bytes"], 256), (wl["parts_off"], N * t_loc * d * 4, 256),
                 (wl["dflag_off"], N * 128, 128), (wl["cflag_off"], N * 128, 128), (wl["local_off"], 64, 128)]
        end = 0
        for off, size, align in areas:
            assert off % align == 0 and off >= end
            end = off + size
        assert end <= wl["bytes"]
