"""Expert-parallel dispatch / combine layer: one process per GPU, experts sharded evenly, two all-to-alls per step.

The reference is single-GPU and shards nothing (engine/mova_cuda.c:590); this layer is new and sits where its engine
calls the routed experts (engine/qwen4_cuda.c:1071-1078).  Rank r owns experts [r E/N, (r+1) E/N) and t_loc tokens.

A step, on every rank:
  1. route the local tokens (top-k over all E experts) and pack their rows to bf16;
  2. DISPATCH all-to-all: every rank receives every rank's chunk = [t_loc rows of bf16 | ids | weights] (at decode batch
     sizes a token needs most ranks -- 5.9 of 8 at top-10 over 512 experts -- so the chunk carries all local rows);
  3. plan: keep the (token, expert) pairs whose expert is local, in token order;
  4. the local experts' gate+up+SwiGLU and down mat-vecs over those pairs, reading the received rows in place;
  5. pre-sum each token's local experts into one partial row;
  6. COMBINE all-to-all: the partial rows go back to the ranks that own the tokens;
  7. the owner adds the N partial rows in rank order.
Steps 1, 3-5 and 7 are supplied by a backend: CudaBackend calls the C ABI (include/nslm_ep.h); the tests' CPU backend
does the same steps with the oracle so that the plumbing runs under gloo without a GPU."""
import ctypes as C

import numpy as np
import torch
import torch.distributed as dist


def chunk_layout(t_loc, d, k):
    """Byte layout of one rank's dispatch chunk, padded so that a chunk is a whole number of bf16 rows."""
    row = 2 * d
    x_bytes = t_loc * row
    ind_off = x_bytes
    wt_off = ind_off + 4 * t_loc * k
    total = wt_off + 4 * t_loc * k
    total = (total + row - 1) // row * row
    return {"row": row, "ind_off": ind_off, "wt_off": wt_off, "bytes": total, "rows": total // row}


def window_layout(N, t_loc, d, k):
    """Byte layout of a rank's peer-memory window (include/nslm_ep.h, NslEpWindow): receive chunks, partial rows, the two
    flag arrays (one 128-byte line per rank) and the owner's private words."""
    lay = chunk_layout(t_loc, d, k)
    up = lambda v, a=256: (v + a - 1) // a * a
    parts_off = up(N * lay["bytes"])
    dflag_off = up(parts_off + N * t_loc * d * 4)
    cflag_off = dflag_off + N * 128
    local_off = cflag_off + N * 128
    return {"t_loc": t_loc, "chunk_bytes": lay["bytes"], "recv_off": 0, "parts_off": parts_off, "dflag_off": dflag_off,
            "cflag_off": cflag_off, "local_off": local_off, "bytes": up(local_off + 128)}


class P2PWindow:
    """This rank's view of all ranks' windows: ptrs[r] = rank r's window as mapped in this process."""

    def __init__(self, lib, ptrs, me, wl, owned, opened):
        self.lib, self.ptrs, self.me, self.wl, self.owned, self.opened = lib, ptrs, me, wl, owned, opened

    @classmethod
    def create(cls, N, me, t_loc, d, k, group=None):
        """One window per rank, allocated by its owner and opened by the others through CUDA inter-process handles that
        travel over the process group."""
        from . import lib as L
        lib = L.load()
        wl = window_layout(N, t_loc, d, k)
        ptr, handle = C.c_void_p(), (C.c_ubyte * 64)()
        if lib.nsl_ep_window_alloc(wl["bytes"], C.byref(ptr), handle):
            raise RuntimeError(L.last_error() or "nsl_ep_window_alloc failed")
        ptrs, opened = [0] * N, []
        if N > 1:
            handles = [None] * N
            dist.all_gather_object(handles, bytes(handle), group=group)
            for r in range(N):
                if r == me:
                    continue
                q = C.c_void_p()
                if lib.nsl_ep_window_open((C.c_ubyte * 64).from_buffer_copy(handles[r]), C.byref(q)):
                    raise RuntimeError(L.last_error() or "nsl_ep_window_open failed")
                ptrs[r] = q.value
                opened.append(q.value)
        ptrs[me] = ptr.value
        return cls(lib, ptrs, me, wl, [ptr.value], opened)

    @classmethod
    def local_group(cls, N, t_loc, d, k):
        """N windows inside this process (no handles): for driving N ranks' kernels from one stream on one GPU, every
        rank's producers before any rank's consumers, so that no kernel waits for a later one."""
        from . import lib as L
        lib = L.load()
        wl = window_layout(N, t_loc, d, k)
        ptrs = []
        for _ in range(N):
            ptr = C.c_void_p()
            if lib.nsl_ep_window_alloc(wl["bytes"], C.byref(ptr), None):
                raise RuntimeError(L.last_error() or "nsl_ep_window_alloc failed")
            ptrs.append(ptr.value)
        return [cls(lib, ptrs, me, wl, ptrs if me == 0 else [], []) for me in range(N)]

    def struct(self):
        from . import lib as L
        w, wl = L.NslEpWindow(), self.wl
        for r, q in enumerate(self.ptrs):
            w.win[r] = q
        w.n, w.me, w.t_loc, w.bytes = len(self.ptrs), self.me, wl["t_loc"], wl["bytes"]
        for f in ("chunk_bytes", "recv_off", "parts_off", "dflag_off", "cflag_off", "local_off"):
            setattr(w, f, wl[f])
        return w

    def status(self):
        """0, or the code of a wait that ran out (see nsl_ep_p2p_status).  Synchronises the device."""
        torch.cuda.synchronize()
        return self.lib.nsl_ep_p2p_status(self.struct())

    def close(self):
        for q in self.opened:
            self.lib.nsl_ep_window_close(C.c_void_p(q))
        for q in self.owned:
            self.lib.nsl_ep_window_free(C.c_void_p(q))
        self.opened, self.owned = [], []


class ExpertParallelMoe:
    def __init__(self, backend, d, k, n_exp_total, t_loc, group=None, collectives="a2a", window=None, mirror=False):
        """collectives: "a2a" -- two all-to-alls and a rank-order sum on the owner; "gather" -- the same data movement as
        an all-gather of the chunks and a reduce-scatter of the partial rows (the sum is then formed by the collective,
        in its own order); "p2p" -- no collective call: the kernels store into the other ranks' windows over NVLink and
        wait on flags (window: a P2PWindow, made here when omitted; passing one of P2PWindow.local_group's lets one
        process drive several ranks).
        mirror (p2p only, an even number of ranks): rank r and rank r + N/2 hold each other's experts as well (the backend's
        layer = the own experts followed by the partner's) and split the pairs of their joint expert set in the middle,
        so that a pair of ranks is balanced to within one (token, expert) pair whatever the routing."""
        self.be, self.d, self.k, self.E, self.t_loc, self.group = backend, d, k, n_exp_total, t_loc, group
        self.collectives = collectives
        if window is not None:
            self.N, self.rank = len(window.ptrs), window.me
        else:
            self.N = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        assert n_exp_total % self.N == 0, "experts must divide evenly over the ranks"
        self.e_loc = n_exp_total // self.N
        self.lo, self.hi = self.rank * self.e_loc, (self.rank + 1) * self.e_loc
        self.lay = chunk_layout(t_loc, d, k)
        self.lo2, self.hi2, self.upper = 0, 0, 0
        if mirror:
            assert collectives == "p2p" and self.N % 2 == 0, "mirrored ranks need the peer-memory exchange and an even rank count"
            partner = (self.rank + self.N // 2) % self.N
            self.lo2, self.hi2, self.upper = partner * self.e_loc, (partner + 1) * self.e_loc, int(self.rank > partner)
        dev = backend.device
        self.send = torch.zeros(self.N, self.lay["bytes"], dtype=torch.uint8, device=dev)
        self.recv = torch.zeros(self.N, self.lay["bytes"], dtype=torch.uint8, device=dev)
        self.partial = torch.zeros(self.N, t_loc, d, dtype=torch.float32, device=dev)
        self.parts = torch.zeros(self.N, t_loc, d, dtype=torch.float32, device=dev)
        self.out = torch.zeros(t_loc, d, dtype=torch.float32, device=dev)
        self.window = None
        if collectives == "p2p":
            self.window = window or P2PWindow.create(self.N, self.rank, t_loc, d, k, group)
            self.win = self.window.struct()
            self.recv_ptr = self.window.ptrs[self.rank] + self.window.wl["recv_off"]
        else:
            self.recv_ptr = self.recv.data_ptr()
        backend.setup(self)

    def _all_to_all(self, out, inp):
        if self.N == 1:
            out.copy_(inp)
        else:
            dist.all_to_all_single(out.view(-1), inp.view(-1), group=self.group)

    def step(self, x, logits):
        """x [t_loc][d] f32 (bf16-valued), logits [t_loc][E] -> out [t_loc][d] (this rank's tokens)."""
        be = self.be
        if self.collectives == "p2p":
            be.route_pack_dispatch(self, x, logits)        # router + bf16 rows straight into every rank's window
            be.local_experts(self)
            be.reduce(self)
            return self.out
        be.route_and_pack(self, x, logits)                 # fills send[0]
        self.dispatch()
        be.local_experts(self)                             # plan + mat-vecs + per-token pre-sum -> partial [N][t_loc][d]
        self.combine()
        return self.out

    def dispatch(self, replicate=True):
        if self.N > 1 and self.collectives == "gather":
            dist.all_gather_into_tensor(self.recv.view(-1), self.send[0], group=self.group)
            return
        if self.N > 1 and replicate:
            self.send[1:] = self.send[0]
        self._all_to_all(self.recv, self.send)

    def combine(self, reduce=True):
        if self.N > 1 and self.collectives == "gather":
            dist.reduce_scatter_tensor(self.out.view(-1), self.partial.view(-1), group=self.group)
            return
        self._all_to_all(self.parts, self.partial)
        if reduce:
            self.be.reduce(self)                           # out = sum_r parts[r], rank order


class GraphedSteps:
    """The device work of a step as CUDA graphs.  With the peer-memory exchange ("p2p") two graphs hold the whole step:
    (route + pack + dispatch) per input batch and (wait + plan + mat-vecs + combine + reduce) per resident layer.  With
    collective calls it is three graphs -- (route + pack + replicate), (plan + mat-vecs + pre-sum) and (reduce) -- with
    the two all-to-alls issued between them as ordinary NCCL calls.  One first graph per input batch
    and one second graph per resident layer are captured up front; a step then costs three graph launches and two
    collective calls on the host instead of a dozen kernel launches.  (Capturing the collectives themselves into a graph
    did not complete on this system, so they stay outside.)

    whole (peer-memory exchange only): the (input batch, layer) pairs whose step is captured as ONE graph, as an engine that
    replays a graph per decode forward would hold it: no second graph launch, and the dispatch kernel's dependents come in
    while it drains."""

    def __init__(self, ep, layers, inputs, whole=()):
        self.ep, be = ep, ep.be
        stream = torch.cuda.current_stream()

        def capture(fn):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                fn()
            return g

        gather = ep.N > 1 and ep.collectives == "gather"
        self.p2p = ep.collectives == "p2p"

        def first(x, logits):
            if self.p2p:
                be.route_pack_dispatch(ep, x, logits)
                return
            be.route_and_pack(ep, x, logits)
            if ep.N > 1 and not gather:
                ep.send[1:] = ep.send[0]

        def second(layer):
            be.set_layer(layer)
            be.local_experts(ep)
            if self.p2p:
                be.reduce(ep)

        self.first = [capture(lambda x=x, l=l: first(x, l)) for x, l in inputs]
        self.second = [capture(lambda layer=layer: second(layer)) for layer in layers]
        self.third = None if gather or self.p2p else capture(lambda: be.reduce(ep))
        self.whole = {}
        if self.p2p:
            for i, j in whole:
                if (i, j) not in self.whole:
                    x, l = inputs[i]
                    self.whole[(i, j)] = capture(lambda x=x, l=l, layer=layers[j]: (first(x, l), second(layer)))

    def step(self, i_input, i_layer):
        ep = self.ep
        g = self.whole.get((i_input, i_layer))
        if g is not None:
            g.replay()
            return ep.out
        self.first[i_input].replay()
        if self.p2p:      # the exchanges are inside the graphs: two launches make a step
            self.second[i_layer].replay()
            return ep.out
        ep.dispatch(replicate=False)
        self.second[i_layer].replay()
        ep.combine(reduce=False)
        if self.third is not None:
            self.third.replay()
        return ep.out


class CudaBackend:
    """The steps on the GPU through the C ABI; layer = this rank's experts (moe.DeviceLayer with e_loc experts)."""

    def __init__(self, layer, rounding=True):
        from . import lib as L
        from .kernels import stream_table
        self.L, self.lib, self.layer = L, L.load(), layer
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.G = stream_table()
        self.raw = int(not rounding)      # 1: f32 throughout (no bf16 rounding points), for comparison with the CPU forward

    def setup(self, ep):
        T, k, d, ff = ep.N * ep.t_loc, ep.k, ep.d, self.layer.ff
        P = T * k
        z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=self.device)
        self.ind, self.wt = z(ep.t_loc, k, dt=torch.int32), z(ep.t_loc, k)
        self.sel, self.xrow, self.wsel = z(P, dt=torch.int32), z(P, dt=torch.int32), z(P)
        self.tok_off, self.count = z(T + 1, dt=torch.int32), z(1, dt=torch.int32)
        self.A, self.D = z(P, ff), z(P, d)

    def set_layer(self, layer):
        self.layer = layer

    def _s(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def route_and_pack(self, ep, x, logits):
        lib, s, lay = self.lib, self._s(), ep.lay
        chunk = ep.send[0]
        ind = chunk[lay["ind_off"]:lay["wt_off"]].view(torch.int32)
        wt = chunk[lay["wt_off"]:lay["wt_off"] + 4 * ep.t_loc * ep.k].view(torch.float32)
        lib.nsl_route(s, ep.E, ep.k, logits.data_ptr(), ep.E, ind.data_ptr(), wt.data_ptr(), ep.t_loc)
        lib.kc_pack_input_bf16(s, x.data_ptr(), chunk.data_ptr(), ep.t_loc * ep.d)

    def local_experts(self, ep):
        lib, s, lay, lyr = self.lib, self._s(), ep.lay, self.layer
        base = ep.recv_ptr
        T = ep.N * ep.t_loc
        p2p = ep.collectives == "p2p"
        out = (self.sel.data_ptr(), self.xrow.data_ptr(), self.wsel.data_ptr(), self.tok_off.data_ptr(), self.count.data_ptr())
        if p2p:      # the wait for every rank's chunk is the first thing the plan kernel does
            lib.nsl_ep_p2p_plan(s, ep.win, lay["ind_off"], lay["wt_off"], ep.k, lay["rows"], ep.lo, ep.hi, ep.lo2, ep.hi2,
                                ep.upper, *out)
        else:
            lib.nsl_ep_plan(s, base + lay["ind_off"], base + lay["wt_off"], ep.N, ep.t_loc, ep.k, lay["bytes"] // 4,
                            lay["rows"], ep.lo, ep.hi, *out)
        P = T * ep.k
        lib.nsl_dependent_launch(1)   # the three kernels after the plan come in while their predecessor drains
        try:
            lib.nsl_mv_gu_rows(s, lyr.gate.table.data_ptr(), lyr.up.table.data_ptr(), lyr.d, lyr.ff, base, ep.d, 1,
                               self.A.data_ptr(), lyr.ff, self.sel.data_ptr(), self.xrow.data_ptr(), P, self.count.data_ptr(),
                               self.raw, self.G.data_ptr())
            lib.nsl_mv_sel_rows(s, lyr.down.table.data_ptr(), lyr.ff, lyr.d, self.A.data_ptr(), lyr.ff, self.D.data_ptr(), lyr.d,
                                self.sel.data_ptr(), P, self.count.data_ptr(), self.raw, self.G.data_ptr())
            if p2p:
                lib.nsl_ep_p2p_combine(s, ep.win, self.D.data_ptr(), self.wsel.data_ptr(), self.tok_off.data_ptr(), ep.d)
            else:
                lib.nsl_ep_combine(s, self.D.data_ptr(), self.wsel.data_ptr(), self.tok_off.data_ptr(), T, ep.d, ep.partial.data_ptr())
        finally:
            lib.nsl_dependent_launch(0)

    def p2p_dispatch(self, ep):
        """The chunk route_and_pack left in send[0] -> every rank's window."""
        self.lib.nsl_ep_p2p_dispatch(self._s(), ep.win, ep.send.data_ptr())

    def route_pack_dispatch(self, ep, x, logits):
        """route_and_pack + p2p_dispatch as one kernel that stores straight into the windows."""
        lay = ep.lay
        self.lib.nsl_ep_p2p_route_dispatch(self._s(), ep.win, ep.E, ep.k, logits.data_ptr(), ep.E, x.data_ptr(), ep.d,
                                           lay["ind_off"], lay["wt_off"], self.ind.data_ptr(), self.wt.data_ptr())

    def reduce(self, ep):
        if ep.collectives == "p2p":
            self.lib.nsl_ep_p2p_reduce(self._s(), ep.win, ep.d, ep.out.data_ptr())
        else:
            self.lib.nsl_ep_reduce(self._s(), ep.parts.data_ptr(), ep.N, ep.t_loc, ep.d, ep.out.data_ptr())


def _emulate(ranks, steps, mirror=False, d=2048, ff=512, n_exp=512, k=10, batch=64):
    """N ranks of the peer-memory step driven from ONE stream on ONE GPU (every rank's producers before any rank's
    consumers, so that no kernel waits for a later one): each rank's kernels have the sizes of an N-GPU run, which makes
    their durations readable from a profiler's launch list without N GPUs.  Prints the serial time per step."""
    from . import lib as L, moe
    t_loc = batch // ranks
    gen = torch.Generator(device="cuda").manual_seed(1)
    wins = P2PWindow.local_group(ranks, t_loc, d, k)
    held = (2 if mirror else 1) * n_exp // ranks      # timing only: the mirrored experts are random too
    eps = [ExpertParallelMoe(CudaBackend(moe.DeviceLayer.random_on_device(d, ff, held, gen)), d, k, n_exp, t_loc,
                             collectives="p2p", window=wins[r], mirror=mirror) for r in range(ranks)]
    x = torch.randn(batch, d, generator=gen, device="cuda")
    logits = torch.randn(batch, n_exp, generator=gen, device="cuda")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for s in range(steps + 1):
        if s == 1:
            e0.record()
        for r, e in enumerate(eps):
            e.be.route_pack_dispatch(e, x[r * t_loc:(r + 1) * t_loc], logits[r * t_loc:(r + 1) * t_loc])
        for e in eps:
            e.be.local_experts(e)
        for e in eps:
            e.be.reduce(e)
    e1.record()
    torch.cuda.synchronize()
    status = [w.status() for w in wins]
    pairs = [int(e.be.count.item()) for e in eps]
    L.check()
    for w in wins:
        w.close()
    print(f"{ranks} emulated ranks, {steps} steps: {e0.elapsed_time(e1) * 1e3 / steps:.1f} us per step for all ranks in series "
          f"({e0.elapsed_time(e1) * 1e3 / steps / ranks:.1f} us per rank); pairs per rank {pairs}; wait status {status}")


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="the expert-parallel step of N ranks emulated on one GPU (kernel sizes of an N-GPU run)")
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--mirror", action="store_true", help="ranks r and r + N/2 hold each other's experts and split their pairs")
    a = ap.parse_args()
    _emulate(a.ranks, a.steps, a.mirror)
