"""CPU stand-in for the expert-parallel layer's device steps, built on the oracle: lets the dispatch / combine plumbing
(nanoseedlm_b200.ep.ExpertParallelMoe) run under gloo without a GPU.  Test infrastructure."""
import numpy as np
import torch


def bf16_bits(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class OracleBackend:
    def __init__(self, oracle, host_layer, lo, hi):
        self.o, self.h, self.lo, self.hi = oracle, host_layer, lo, hi
        self.device = torch.device("cpu")

    def setup(self, ep):
        pass

    def route_and_pack(self, ep, x, logits):
        lay = ep.lay
        ind, wt = self.o.route(logits.numpy(), ep.k)
        chunk = ep.send[0].numpy()
        chunk[:ep.t_loc * lay["row"]] = bf16_bits(x.numpy()).view(np.uint8).ravel()
        chunk[lay["ind_off"]:lay["wt_off"]] = ind.view(np.uint8).ravel()
        chunk[lay["wt_off"]:lay["wt_off"] + 4 * ep.t_loc * ep.k] = wt.view(np.uint8).ravel()

    def local_experts(self, ep):
        lay, o = ep.lay, self.o
        recv = ep.recv.numpy()
        part = ep.partial.numpy()
        part[:] = 0
        for r in range(ep.N):
            c = recv[r]
            x = (c[:ep.t_loc * lay["row"]].view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(ep.t_loc, ep.d)
            ind = c[lay["ind_off"]:lay["wt_off"]].view(np.int32).reshape(ep.t_loc, ep.k)
            wt = c[lay["wt_off"]:lay["wt_off"] + 4 * ep.t_loc * ep.k].view(np.float32).reshape(ep.t_loc, ep.k)
            for t in range(ep.t_loc):
                acc = np.zeros(ep.d, np.float32)
                for j in range(ep.k):
                    e = int(ind[t, j])
                    if self.lo <= e < self.hi:
                        a = o.mv_gu(self.h.matrix(o, "gate", e), self.h.matrix(o, "up", e), x[t])
                        acc = acc + wt[t, j] * o.mv(self.h.matrix(o, "down", e), a)[0]
                part[r, t] = acc

    def reduce(self, ep):
        parts = ep.parts.numpy()
        acc = parts[0].copy()
        for r in range(1, ep.N):
            acc = acc + parts[r]
        ep.out.numpy()[:] = acc
