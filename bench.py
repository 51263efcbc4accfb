#!/usr/bin/env python
"""Benchmark of the seed-decode MoE hot path on B200 (BASELINE.json: seed-decode MoE GEMV tokens/s and GB/s against the
roofline at 1 / 2 / 4 / 8 GPUs, next to the CPU seed path timed on the same host).

    python bench.py --gpus 1 --steps 2000 --warmup 10           # this library (CUDA kernels behind the C ABI)
    python bench.py --impl reference --steps 3 --warmup 1        # the CPU seed path on the host cores
    torchrun --nproc-per-node N ... bench.py --gpus N            # expert-parallel decode (config 3) on N GPUs

N = 1.  The headline is BASELINE config 1 at M = 8 (the multi-token-prediction verify batch): a step = router top-8 over
128 experts (in the prologue of the gate+up kernel), the routed experts' gate + up + SwiGLU and down projections
regenerated from their seeds pair by pair, and the weighted combine.  Steps rotate over enough
independent synthetic layers that every step's packed streams come from HBM, not L2.  The same JSON line carries
`workloads` (config 0, config 1 at M = 1 and 4, config 2, the LM head, decode attention: time per step and roofline
each) and `ep_base` = config 3 with all 512 experts on the one GPU, the base of the strong-scaling series that the N > 1
lines continue.

N > 1.  Config 3: 512 experts sharded over the ranks, 64 sequences x 1 token, top-10, dispatch and combine by the kernels
themselves over NVLink peer memory.  Before the timed region one step on seeded inputs is compared with the one-GPU layer
(`parity`).

value = tokens/s with inputs resident in HBM (CUDA events, max over ranks); e2e = the same through the C host layer with
HOST buffers (H2D of the step's inputs from pinned memory, D2H of its output, one step in flight); roofline = the dominant
kernel against the measured HBM peak and against the logic-pipe floor that actually bounds it; cpu_baseline = the CPU
restatement of the reference's seed mat-vec on the host cores, on the same bytes as one timed step."""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, FF, E, TOPK = 2048, 512, 128, 8
BYTES_PER_MATRIX = D * FF // 8 * 4 + D * FF // 16        # 589,824: seeds + coefficient words + exponent codes
BLOCKS_PER_MATRIX = D * FF // 8                           # 131,072 blocks of 8 weights
ALU_FLOOR = 53 / 64        # clocks per block per SM: 53 logic-pipe operations per block, 64 logic lanes per SM and clock
                           # (ncu agrees: 113.4 k blocks per SM in 141.3 k active cycles with sm__pipe_alu_cycles_active
                           # at 70 %; profiles/logic_pipe_rates.md)
METRIC = "seed_decode_moe_gemv_tokens_per_s"
# DRAM bytes per launch of the gate+up kernel from ncu (profiles/mv_pair_gate_up_config1.md): per distinct expert
# (gate + up streams: pairs that share an expert find its streams in L2) and the rest (activations, tables)
NCU_TRAFFIC_PER_DISTINCT = 1.114e6
NCU_TRAFFIC_FIXED = 0.9e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def bf16r(a):
    a = np.ascontiguousarray(a, np.float32)
    return (a.view(np.uint32) + 0x7FFF + ((a.view(np.uint32) >> 16) & 1) & 0xFFFF0000).view(np.float32)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            self.t.join(timeout=2)

    def summary(self):
        sm = sorted(float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit())
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


# ---- the CPU path ---------------------------------------------------------------------------------------------------------
class CpuMoe:
    """One MoE step on the host cores with the CPU seed kernels (the gcc restatement of nslm/lib_cpu_seed4.c) in their
    fastest form: the CPU-tiled layout, the rows that share an expert multiplied together (up to 8 per call, the
    kernel's limit), every routed expert's gate and up products in one parallel region over all host threads, then
    every down product in a second one.  experts: {id: (gate, up, down) oracle matrices}; ids outside it draw from a pool
    of seeded matrices (timing only)."""

    def __init__(self, n_exp, top_k, threads, experts=None, pool=24):
        from oracle import binding as B
        self.B, self.n_exp, self.top_k, self.threads = B, n_exp, top_k, threads
        self.own = {e: tuple(B.Tiled(m) for m in ms) for e, ms in (experts or {}).items()}
        self.pool = None if experts else [(B.Tiled(B.Matrix(FF, D, 300 + i)), B.Tiled(B.Matrix(FF, D, 400 + i)),
                                           B.Tiled(B.Matrix(D, FF, 500 + i))) for i in range(pool)]

    def mats(self, e):
        return self.own[e] if e in self.own else self.pool[e % len(self.pool)]

    def groups(self, logits):
        ind, wt = self.B.route(logits, self.top_k)
        by = {}
        for t in range(ind.shape[0]):
            for j in range(self.top_k):
                by.setdefault(int(ind[t, j]), []).append((t, float(wt[t, j])))
        out = []
        for e, rows in sorted(by.items()):
            for c in range(0, len(rows), 8):
                out.append((e, rows[c:c + 8]))
        return out

    def run(self, x, groups):
        """The groups' share of the layer output; returns (out [M][D], pairs done)."""
        B = self.B
        xs = [x[[t for t, _ in rows]] for _, rows in groups]
        gu = B.tiled_jobs([(self.mats(e)[0], xe) for (e, _), xe in zip(groups, xs)] +
                          [(self.mats(e)[1], xe) for (e, _), xe in zip(groups, xs)], self.threads)
        n = len(groups)
        act = [g / (1.0 + np.exp(-g)) * u for g, u in zip(gu[:n], gu[n:])]
        dn = B.tiled_jobs([(self.mats(e)[2], a) for (e, _), a in zip(groups, act)], self.threads)
        out = np.zeros_like(x)
        for (_, rows), y in zip(groups, dn):
            for i, (t, w) in enumerate(rows):
                out[t] += w * y[i]
        return out, sum(len(rows) for _, rows in groups)


def cpu_inputs(M, n_exp, seed=99):
    rng = np.random.default_rng(seed)
    return bf16r(rng.standard_normal((M, D)).astype(np.float32)), rng.standard_normal((M, n_exp)).astype(np.float32)


def host_experts(layer, ids):
    """The streams of a device layer's experts `ids` copied back to the host as oracle matrices (the same bytes the GPU reads)."""
    from oracle import binding as B
    out = {}
    for e in ids:
        ms = []
        for st, (R, K) in ((layer.gate, (FF, D)), (layer.up, (FF, D)), (layer.down, (D, FF))):
            m = B.Matrix(R, K, 0, eb=st.eb[e])
            m.seeds[:] = st.seeds[e].cpu().numpy().view(np.uint16)
            m.coefs[:] = st.coefs[e].cpu().numpy().view(np.uint16)
            m.codes[:] = st.codes[e].cpu().numpy()
            ms.append(m)
        out[e] = tuple(ms)
    return out


def cpu_baseline_cfg1(threads, M, layer=None, x=None, logits=None, gpu_out=None, seconds=12.0):
    """The CPU path on a bounded sample: whole steps of the headline's workload, repeated for about `seconds`.  With a
    device layer given, the CPU works on the SAME bytes as one of the GPU's timed steps (the routed experts' streams
    copied back) and its output is compared with the GPU's."""
    from oracle import binding as B
    if x is None:
        x, logits = cpu_inputs(M, E)
    ind, _ = B.route(logits, TOPK)
    ids = sorted(set(ind.ravel().tolist()))
    cpu = CpuMoe(E, TOPK, threads, host_experts(layer, ids) if layer is not None else None)
    groups = cpu.groups(logits)
    out, _ = cpu.run(x, groups)   # warm-up
    times, t_end = [], time.perf_counter() + seconds
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 200):
        t0 = time.perf_counter()
        cpu.run(x, groups)
        times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    res = {"value": M / dt, "unit": "tok/s", "cores": threads, "kind": "port", "ms_per_step": dt * 1e3,
           "gweights_per_s": len(ids) * 3 * D * FF / dt / 1e9,
           "sample": f"{len(times)} whole steps (median) of {M} rows x top-{TOPK} of {E} experts = {len(ids)} distinct experts x "
                     f"(gate, up, down) on {threads} host threads, on the bytes of one of the GPU's timed steps: CPU-tiled layout, "
                     "rows sharing an expert multiplied together; the reference's own kernel needs Clang, this is its gcc "
                     "restatement (oracle/cpu_seed4_tiled.c)"}
    if gpu_out is not None:
        res["gpu_vs_cpu_max_rel"] = float(np.max(np.abs(gpu_out - out)) / np.max(np.abs(out)))
    return res


def cpu_cfg0_protocol():
    """BASELINE config 0 on the host cores by the reference bench's protocol (harness/nslm-cpu-seed-bench.c:22, 46-49, 57-66):
    N = 2048 x K = 4096, one token, threads 1 and all, best of 20 after a warm-up, CLOCK_MONOTONIC, nproc and the load
    average printed, the largest error against the double-precision spec relative to sum |w x|."""
    from oracle import binding as B
    m = B.Matrix(2048, 4096, 42, eb=-22)
    x = B.normal(43, 4096)
    y64, mag = B.matvec_f64(m, x)
    tiled = B.Tiled(m)
    nproc = os.cpu_count() or 1
    res = {"shape": "2048 x 4096, 1 token", "nproc": nproc, "loadavg": open("/proc/loadavg").read().split()[:3], "protocol": "best of 20 after one warm-up call",
           "threads": {}}
    for th in sorted({1, nproc}):
        dt, y = tiled.time(x, th, 20)
        res["threads"][str(th)] = {"ms": dt * 1e3, "gweights_per_s": 2048 * 4096 / dt / 1e9, "packed_gbs": 2048 * 4096 * 0.5625 / dt / 1e9,
                                   "max_err_vs_f64_spec": float(np.max(np.abs(y[0] - y64[0]) / mag[0]))}
    return res


def run_reference(args, workload):
    threads = os.cpu_count() or 1
    M, n_exp, top_k = (EP_B, EP_E, EP_K) if workload == "cfg3" else (args.tokens, E, TOPK)
    cpu = CpuMoe(n_exp, top_k, threads)
    x, logits = cpu_inputs(M, n_exp)
    groups = cpu.groups(logits)
    pairs = M * top_k
    t0 = time.perf_counter()
    cpu.run(x, groups)
    full = time.perf_counter() - t0
    # each step = a bounded sample of the step's expert groups, so that steps + warm-up end within about 150 s
    budget = 150.0 / max(1, args.steps + args.warmup)
    take = max(1, min(len(groups), int(len(groups) * budget / full)))
    for i in range(args.warmup):
        cpu.run(x, [groups[(i * take + g) % len(groups)] for g in range(take)])
    done, t0 = 0, time.perf_counter()
    for i in range(args.steps):
        done += cpu.run(x, [groups[(i * take + g) % len(groups)] for g in range(take)])[1]
    dt = (time.perf_counter() - t0) / args.steps
    value = M * (done / args.steps / pairs) / dt      # rows/s of whole steps at the sampled (row, expert) pair rate
    cfg = ep_config(args.gpus) if workload == "cfg3" else workload_config(M)
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": f"each step = {take} of the step's {len(groups)} (expert, <= 8 rows) groups "
                                       f"({done // args.steps} of {pairs} (row, expert) pairs), scaled to whole steps; CPU-tiled "
                                       f"seed kernels on {threads} host threads (gcc restatement of nslm/lib_cpu_seed4.c; the "
                                       "original needs Clang)"},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(M):
    which = "config 1: synthetic MoE expert layer at decode" if M <= 8 else "config 2: synthetic MoE prefill / continuous-batching grouped GEMM"
    return {"workload": f"BASELINE {which}, hidden {D}, {E} seed-encoded (SEED4P4) "
                        f"SwiGLU experts of intermediate {FF}, softmax top-{TOPK}, M={M} tokens, all experts resident",
            "tokens": M, "experts": E, "top_k": TOPK, "hidden": D, "intermediate": FF}


def l2_policy(layers, n_exp=E):
    return (f"steps rotate over {layers} independent layers ({layers * n_exp * 3 * BYTES_PER_MATRIX / 1e9:.1f} GB of packed streams, "
            "far larger than the 126 MB L2), so each step's experts are read from HBM")


# ---- config 1 / config 2: one GPU's MoE layer ---------------------------------------------------------------------------
class Cfg1:
    """The resident synthetic layers and input batches shared by the config-1 / config-2 measurements."""

    def __init__(self, NL, rank=0):
        import torch
        from nanoseedlm_b200 import lib as L, moe
        self.torch, self.L, self.moe, self.lib = torch, L, moe, L.load()
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        self.layers = [moe.DeviceLayer.random_on_device(D, FF, E, gen) for _ in range(NL)]
        self.NL, self.rank = NL, rank
        self.stream = torch.cuda.Stream()
        torch.cuda.synchronize()

    def inputs(self, M, NB=16):
        rng = np.random.default_rng(99 + self.rank + 1000 * M)
        hx = bf16r(rng.standard_normal((NB, M, D)).astype(np.float32))
        hl = rng.standard_normal((NB, M, E)).astype(np.float32)
        distinct = [len(set(np.argsort(-hl[b], axis=1, kind="stable")[:, :TOPK].ravel().tolist())) for b in range(NB)]
        return hx, hl, distinct


ONE_LAUNCH = False     # --one-launch: the decode step as the one fused launch (nsl_mv_step) instead of three dependent launches


def measure_layer(c, M, K, W, sample_clocks=True, with_e2e=True, dependent_launch=True):
    """Config 1 (M <= 8) or config 2 (M = 512) on one GPU: tokens/s of whole steps (CUDA graph of `chunk` steps replayed),
    the dominant kernel timed launch by launch, and the end-to-end forms."""
    torch, L, lib, layers, NL, stream = c.torch, c.L, c.lib, c.layers, c.NL, c.stream
    NB = 16
    hx, hl, distinct = c.inputs(M, NB)
    dx, dl = torch.from_numpy(hx).cuda(), torch.from_numpy(hl).cuda()
    dout = torch.zeros(M, D, device="cuda")
    m = c.moe.Moe(layers[0], TOPK, M)
    m.set_dependent_launch(dependent_launch)
    m.set_one_launch(ONE_LAUNCH)
    res = {"tokens": M}

    def enqueue(step, s):
        m.set_layer(layers[step % NL])
        m.forward_dev(dx[step % NB], dl[step % NB], dout, stream=s.cuda_stream)

    with torch.cuda.stream(stream):
        for i in range(W):
            enqueue(i, stream)
        stream.synchronize()
        # the steps are captured as a CUDA graph of `chunk` steps (the reference engine replays a graph per decode
        # forward, engine/qwen4_cuda.c:1213-1231); K steps = K // chunk replays plus the remainder launched directly
        chunk = min(K, 200)
        launches0 = lib.nsl_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(chunk):
                enqueue(W + i, stream)
        launches = (lib.nsl_launch_count() - launches0) // chunk * K
        graph.replay()   # one untimed replay: graph upload
        stream.synchronize()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(torch.cuda.current_device()) if sample_clocks else None
        if sampler:
            sampler.__enter__()
        e0.record(stream)
        for _ in range(K // chunk):
            graph.replay()
        for i in range(K % chunk):
            enqueue(W + i, stream)
        e1.record(stream)
        e1.synchronize()
        if sampler:
            sampler.__exit__()
            res["clocks"] = sampler.summary()
        torch.cuda.synchronize()
    ms_per_step = e0.elapsed_time(e1) / K
    res.update(ms_per_step=ms_per_step, value=M / (ms_per_step * 1e-3), gpu_launches=int(launches),
               packed_gbs=sum(distinct[(W + i) % NB] for i in range(K)) / K * 3 * BYTES_PER_MATRIX / (ms_per_step * 1e-3) / 1e9)

    # ---- the dominant kernel, CUDA events around each of its launches on the launching stream --------------------------
    G = m.G
    P = M * TOPK
    A = torch.zeros(P, FF, device="cuda")
    ind = torch.zeros(P, dtype=torch.int32, device="cuda")
    wt = torch.zeros(P, device="cuda")
    perm = torch.zeros(P, dtype=torch.int32, device="cuda")
    tiles = torch.zeros((P // 128 + E + 1) * 4, dtype=torch.int32, device="cuda")
    work = torch.zeros(2 * E + 3, dtype=torch.int32, device="cuda")
    xp = torch.zeros(M * D, dtype=torch.int16, device="cuda")
    with torch.cuda.stream(stream):
        evs = []
        KR = min(K, 400)
        for i in range(KR):
            lay, b = layers[(W + i) % NL], (W + i) % NB
            if M > 8:
                lib.nsl_route(stream.cuda_stream, E, TOPK, dl[b].data_ptr(), E, ind.data_ptr(), wt.data_ptr(), M)
                lib.kc_bucket(stream.cuda_stream, ind.data_ptr(), P, E, perm.data_ptr(), tiles.data_ptr(), work.data_ptr())
                lib.kc_pack_input_bf16(stream.cuda_stream, dx[b].data_ptr(), xp.data_ptr(), M * D)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            if M > 8:      # as the layer launches it: the rows packed to bf16 beforehand
                lib.kc_mm_grouped_packed(stream.cuda_stream, L.MF_SEED4P4, lay.gate.table.data_ptr(), D, FF, xp.data_ptr(), D,
                                         A.data_ptr(), FF, TOPK, perm.data_ptr(), tiles.data_ptr(), work.data_ptr(), P // 128 + E, G.data_ptr())
            else:
                lib.nsl_mv_gu_routed(stream.cuda_stream, lay.gate.table.data_ptr(), lay.up.table.data_ptr(), D, FF, dx[b].data_ptr(), D,
                                     A.data_ptr(), FF, E, TOPK, dl[b].data_ptr(), E, M, ind.data_ptr(), wt.data_ptr(), 0, G.data_ptr())
            a1.record(stream)
            evs.append((a0, a1, b))
        stream.synchronize()
        k_ms = sum(a0.elapsed_time(a1) for a0, a1, _ in evs)
        k_distinct = sum(distinct[b] for _, _, b in evs) / KR
    k_us = k_ms * 1e3 / KR
    res["kernel"] = {"us_per_launch": k_us, "distinct_experts_per_launch": k_distinct, "launches_timed": KR}

    # ---- e2e: host buffers through the C host layer, H2D and D2H inside every step -------------------------------------
    if with_e2e:
        for i in range(W):
            m.set_layer(layers[i % NL])
            m.hx[:M], m.hlogits[:M] = hx[i % NB], hl[i % NB]
            m.forward_pinned(M)
        KE = min(K, 2000)
        t0 = time.perf_counter()
        for i in range(KE):
            m.set_layer(layers[(W + i) % NL])
            m.hx[:M], m.hlogits[:M] = hx[(W + i) % NB], hl[(W + i) % NB]
            m.forward_pinned(M)
        e2e_sync_s = (time.perf_counter() - t0) / KE
        # the same from the caller's OWN pinned blocks (rows then logits, one block per batch): no staging copy on the host
        blocks = [torch.cat([torch.from_numpy(hx[b]).reshape(-1), torch.from_numpy(hl[b]).reshape(-1)]).pin_memory() for b in range(NB)] if M <= 8 else []
        e2e_block_s = None
        if blocks:
            for i in range(W):
                m.set_layer(layers[i % NL])
                m.forward_block(blocks[i % NB])
            t0 = time.perf_counter()
            for i in range(KE):
                m.set_layer(layers[(W + i) % NL])
                m.forward_block(blocks[(W + i) % NB])
                checksum_b = float(m.hout[0, 0])      # the host reads every step's result
            e2e_block_s = (time.perf_counter() - t0) / KE
        # the same with the result brought by a device-to-host copy instead of the combine kernel's stores into pinned memory
        m.set_direct_output(0)
        for i in range(W):
            m.forward_pinned(M)
        t0 = time.perf_counter()
        for i in range(KE // 2):
            m.set_layer(layers[(W + i) % NL])
            m.hx[:M], m.hlogits[:M] = hx[(W + i) % NB], hl[(W + i) % NB]
            m.forward_pinned(M)
        e2e_copy_s = (time.perf_counter() - t0) / (KE // 2)
        m.set_direct_output(1)
        # two independent batches on two handles used alternately: step i + 1 is submitted (its H2D copies and launches)
        # before the host waits for step i's output.  Only independent batches can do this (a decoder's layer L + 1 needs
        # layer L), so it is reported beside the headline, not as it.
        m2 = c.moe.Moe(layers[0], TOPK, M)
        m2.set_dependent_launch(dependent_launch)
        m2.set_one_launch(ONE_LAUNCH)
        ms, checksum = (m, m2), 0.0

        def submit(i):
            h = ms[i & 1]
            h.set_layer(layers[(W + i) % NL])
            h.hx[:M], h.hlogits[:M] = hx[(W + i) % NB], hl[(W + i) % NB]
            h.submit_pinned(M)

        for i in range(4):
            submit(i)
            ms[i & 1].wait()
        t0 = time.perf_counter()
        submit(0)
        for i in range(1, KE):
            submit(i)
            ms[(i - 1) & 1].wait()
            checksum += float(ms[(i - 1) & 1].hout[0, 0])     # the host reads every step's result
        ms[(KE - 1) & 1].wait()
        e2e_two_s = (time.perf_counter() - t0) / KE
        m2.close()
        head_s = e2e_block_s if e2e_block_s is not None else e2e_sync_s
        res["e2e"] = {"value": M / head_s, "unit": "tok/s", "h2d_bytes_per_step": M * D * 4 + M * E * 4, "d2h_bytes_per_step": M * D * 4,
                      "ms_per_step": head_s * 1e3, "steps_in_flight": 1,
                      "call": ("nsl_moe_submit_block + nsl_moe_wait: the step's rows and logits copied from the caller's pinned memory (one H2D copy), "
                               "the layer, the result rows stored into pinned host memory by the combine kernel, a sync, the host reads the result"
                               if e2e_block_s is not None else
                               "nsl_moe_forward_pinned: H2D of the rows and logits from the layer's pinned staging buffers, the layer, a D2H copy, a sync"),
                      "via_staging_buffers": {"value": M / e2e_sync_s, "ms_per_step": e2e_sync_s * 1e3,
                                              "note": "nsl_moe_forward_pinned after copying the inputs into the layer's own pinned buffers on the host"},
                      "with_d2h_copy_instead": {"value": M / e2e_copy_s, "ms_per_step": e2e_copy_s * 1e3},
                      "two_independent_batches": {"value": M / e2e_two_s, "ms_per_step": e2e_two_s * 1e3}}
    # one timed step's inputs and output, for the CPU baseline's comparison on the same bytes
    m.set_layer(layers[0])
    out0, _ = m.forward_host(hx[0], hl[0])
    res["step0"] = (hx[0], hl[0], out0)
    L.check()
    m.close()
    return res


def measure_ref_gpu(c, M, K, W, mine_out=None):
    """The reference's OWN CUDA kernels (engine/kernels_moe.cu + engine/kernels_qwen4.cu compiled unmodified for sm_100a into
    oracle/_ref/libnslm_ref_gpu.so) on the same layers, inputs and rotation as measure_layer: per step kq4_route_ld, kc_mv_gu,
    kc_mv_sel and kq4_moe_combine (engine/qwen4_cuda.c:1033-1078; for M > 8 prompt rows its kc_bucket + kc_mm_grouped_dev x 3 +
    kc_swiglu path, :1058-1064), captured as a CUDA graph and timed with CUDA events.  The checker's use of the reference: a
    reported baseline and a parity check of one step, never the product path."""
    from oracle import ref_gpu
    ref = ref_gpu.lib()
    if ref is None:
        return {"unavailable": "oracle/_ref/libnslm_ref_gpu.so was not built (needs the reference's sources and nvcc)"}
    torch, L, layers, NL, stream = c.torch, c.L, c.layers, c.NL, c.stream
    NB, P = 16, M * TOPK
    hx, hl, _ = c.inputs(M, NB)
    dx, dl = torch.from_numpy(hx).cuda(), torch.from_numpy(hl).cuda()
    cfg = ref_gpu.qwen4_cfg(E, TOPK)
    cfgp = C.c_void_p(cfg.ctypes.data)
    from nanoseedlm_b200 import kernels
    G = kernels.stream_table()
    ind = torch.zeros(P, dtype=torch.int32, device="cuda")
    wt = torch.zeros(P, device="cuda")
    A = torch.zeros(P, FF, device="cuda")
    Dx = torch.zeros(P, D, device="cuda")
    sh, sg = torch.zeros(M, D, device="cuda"), torch.zeros(M, device="cuda")      # no shared expert in config 1: a zero term
    out = torch.zeros(M, D, device="cuda")
    if M > 8:
        U = torch.zeros(P, FF, device="cuda")
        perm = torch.zeros(P, dtype=torch.int32, device="cuda")
        tiles = torch.zeros((P // 128 + E + 1) * 4, dtype=torch.int32, device="cuda")
        work = torch.zeros(2 * E + 3, dtype=torch.int32, device="cuda")
        mt = P // 128 + E

    def enqueue(step):
        lay, b, s = layers[step % NL], step % NB, stream.cuda_stream
        ref.kq4_route_ld(s, cfgp, dl[b].data_ptr(), E, ind.data_ptr(), wt.data_ptr(), M)
        if M > 8:
            ref.kc_bucket(s, ind.data_ptr(), P, E, perm.data_ptr(), tiles.data_ptr(), work.data_ptr())
            for tab, dst in ((lay.gate, A), (lay.up, U)):
                ref.kc_mm_grouped_dev(s, L.MF_SEED4P4, tab.table.data_ptr(), D, FF, dx[b].data_ptr(), D, dst.data_ptr(), FF, TOPK, perm.data_ptr(),
                                      tiles.data_ptr(), work.data_ptr(), mt, G.data_ptr())
            ref.kc_swiglu(s, A.data_ptr(), U.data_ptr(), A.data_ptr(), P * FF)
            ref.kc_mm_grouped_dev(s, L.MF_SEED4P4, lay.down.table.data_ptr(), FF, D, A.data_ptr(), FF, Dx.data_ptr(), D, 1, perm.data_ptr(),
                                  tiles.data_ptr(), work.data_ptr(), mt, G.data_ptr())
            ref.kq4_moe_combine(s, D, TOPK, Dx.data_ptr(), wt.data_ptr(), sh.data_ptr(), sg.data_ptr(), 0, out.data_ptr(), M)
            return
        ref.kc_mv_gu(s, L.MF_SEED4P4, lay.gate.table.data_ptr(), lay.up.table.data_ptr(), D, FF, dx[b].data_ptr(), D, A.data_ptr(), FF,
                     ind.data_ptr(), P, TOPK, G.data_ptr())
        ref.kc_mv_sel(s, L.MF_SEED4P4, lay.down.table.data_ptr(), FF, D, A.data_ptr(), FF, Dx.data_ptr(), D, ind.data_ptr(), P, 1, G.data_ptr())
        ref.kq4_moe_combine(s, D, TOPK, Dx.data_ptr(), wt.data_ptr(), sh.data_ptr(), sg.data_ptr(), 0, out.data_ptr(), M)

    res = {"kernels": "the reference's engine/kernels_moe.cu + engine/kernels_qwen4.cu, unmodified, nvcc -O3 sm_100a", "launches_per_step": 4 if M <= 8 else 8}
    with torch.cuda.stream(stream):
        enqueue(0)      # step 0 = the step measure_layer hands to the parity checks (layer 0, batch 0)
        stream.synchronize()
        if mine_out is not None:
            r = out.cpu().numpy()
            res["this_library_vs_reference_max_rel"] = float(np.max(np.abs(mine_out - r)) / np.max(np.abs(r)))
        for i in range(W):
            enqueue(i)
        stream.synchronize()
        chunk = min(K, 100 if M <= 8 else 10)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(chunk):
                enqueue(W + i)
        graph.replay()
        stream.synchronize()
        reps = max(1, min(K, 400 if M <= 8 else 40) // chunk)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            graph.replay()
        e1.record(stream)
        e1.synchronize()
    ms = e0.elapsed_time(e1) / (reps * chunk)
    res.update(ms_per_step=ms, value=M / (ms * 1e-3), unit="tok/s", steps=reps * chunk)
    return res


def alu_roofline(us, blocks, sm_mhz, sms):
    """Clocks per expanded block per SM against the logic pipe's floor."""
    clk = us * 1e-6 * sm_mhz * 1e6 * sms / blocks
    return {"blocks_expanded_per_launch": blocks, "clk_per_block_per_sm": clk, "floor_clk_per_block_per_sm": ALU_FLOOR,
            "frac": ALU_FLOOR / clk, "alu_floor_time_us": us * ALU_FLOOR / clk}


def layer_roofline(r, M, sm_mhz, sms, peaks, peak_kind):
    """The roofline object of a config-1 / config-2 measurement: HBM fraction of the dominant kernel and, since the kernel
    is bound by the integer / logic pipe, that pipe's floor.  `alu.frac` counts one expansion per DISTINCT expert (the algorithmic minimum);
    `alu.frac_of_expanded_blocks` counts the blocks the kernel does expand (config 1: every pair)."""
    k = r["kernel"]
    mats = 1 if M > 8 else 2      # config 2 times the gate GEMM, config 1 the gate+up mat-vec
    nbytes = k["distinct_experts_per_launch"] * mats * BYTES_PER_MATRIX + M * D * 4 + M * TOPK * FF * 4
    achieved = nbytes / (k["us_per_launch"] * 1e-6) / 1e9
    name = "seed_gemm_kernel (kc_mm_grouped_dev, gate projection)" if M > 8 else "mv_pair_kernel<gate+up> with the router in its prologue (nsl_mv_gu_routed)"
    out = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
           "peak_kind": peak_kind, "us_per_launch": k["us_per_launch"], "algorithmic_bytes_per_launch": nbytes,
           "traffic": (k["distinct_experts_per_launch"] * NCU_TRAFFIC_PER_DISTINCT + NCU_TRAFFIC_FIXED) if M <= 8 else None,
           "traffic_source": "ncu dram bytes per launch at M = 8 (profiles/), scaled by the launch's distinct experts" if M <= 8 else None,
           "note": "bound by the integer / logic pipe (LFSR expansion: 53 logic operations per 8 weights), not by HBM: see alu"}
    if sm_mhz:
        blocks = k["distinct_experts_per_launch"] * mats * BLOCKS_PER_MATRIX
        out["alu"] = alu_roofline(k["us_per_launch"], blocks, sm_mhz, sms)
        out["alu"]["bytes_time_us"] = nbytes / (peaks["hbm_gbs"] * 1e9) * 1e6
        if M <= 8:
            out["alu"]["frac_of_expanded_blocks"] = out["alu"]["frac"] * M * TOPK / k["distinct_experts_per_launch"]
            out["alu"]["note"] = ("frac: one expansion per distinct expert (the algorithmic minimum); frac_of_expanded_blocks: the kernel expands "
                                  "every (row, expert) pair, since sharing an expansion between pairs measured no faster at <= 64 pairs")
        else:
            tf = 2.0 * M * TOPK * FF * D / (k["us_per_launch"] * 1e-6) / 1e12
            out["tensor"] = {"achieved_tflops": tf, "peak_tflops": peaks["bf16_tflops"], "frac": tf / peaks["bf16_tflops"],
                             "note": "the tensor pipe idles by construction: regenerating a weight tile is the work"}
    return out


def measure_cfg0(K, W):
    """BASELINE config 0: one dense seed mat-vec, 2048 outputs x 4096 inputs, one token (raw f32 output as the CPU path gives
    it); 32 matrices rotated (151 MB) so that every launch reads HBM."""
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    lib = L.load()
    R, Kd, NM = 2048, 4096, 32
    gen = torch.Generator(device="cuda").manual_seed(42)
    nb = R * Kd // 8
    seeds = torch.randint(1, 65536, (NM, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
    coefs = torch.randint(0, 65536, (NM, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
    codes = torch.randint(0, 256, (NM, nb // 2), generator=gen, device="cuda", dtype=torch.int32).to(torch.uint8)
    slices = []
    for i in range(NM):
        w = L.WSlice()
        w.p[0], w.p[1], w.p[3], w.eb = seeds[i].data_ptr(), coefs[i].data_ptr(), codes[i].data_ptr(), -22
        slices.append((L.WSlice * 1)(w))
    x = torch.randn(1, Kd, generator=gen, device="cuda")
    y = torch.zeros(1, R, device="cuda")
    G = kernels.stream_table()
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    def step(i):
        lib.nsl_mv_raw(stream.cuda_stream, C.cast(slices[i % NM], C.c_void_p), Kd, R, x.data_ptr(), Kd, y.data_ptr(), R, None, 1, 1, G.data_ptr())

    with torch.cuda.stream(stream):
        for i in range(W):
            step(i)
        stream.synchronize()
        chunk = min(K, 256)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(chunk):
                step(i)
        g.replay()
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(max(1, K // chunk)):
            g.replay()
        e1.record(stream)
        e1.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (max(1, K // chunk) * chunk)
    L.check()
    return {"us": us, "bytes": nb * 4 + nb // 2 + Kd * 4 + R * 4, "blocks": nb, "weights": R * Kd}


LM_V, LM_D = 151936, 2048   # the LM head of the reference's Qwen-class model (affine int4, groups of 64)


def measure_lmhead(T, K, W, lib=None):
    """The dense affine-int4 LM head (kc_mv with MF_Q4) + greedy arg-max, an HBM-bound kernel.  lib: the library whose kc_mv /
    kc_argmax are timed (default: this one; the reference's kernels for the `ref_gpu` leg)."""
    import torch
    from nanoseedlm_b200 import lib as L
    lib = lib or L.load()
    NM = 4
    gen = torch.Generator(device="cuda").manual_seed(77)
    mats = []
    for _ in range(NM):      # NM independent heads (0.7 GB), rotated so that every step reads HBM
        codes = torch.randint(-2 ** 31, 2 ** 31 - 1, (LM_V, LM_D // 8), generator=gen, device="cuda", dtype=torch.int32)
        sc = (torch.rand(LM_V, LM_D // 64, generator=gen, device="cuda") * 0.02 + 0.001).to(torch.bfloat16)
        bi = (torch.rand(LM_V, LM_D // 64, generator=gen, device="cuda") * -0.2).to(torch.bfloat16)
        w = L.WSlice()
        w.p[0], w.p[1], w.p[2] = codes.data_ptr(), sc.data_ptr(), bi.data_ptr()
        mats.append((w, codes, sc, bi))
    x = torch.randn(T, LM_D, generator=gen, device="cuda").to(torch.bfloat16).float()
    y = torch.zeros(T, LM_V, device="cuda")
    tok = torch.zeros(T, dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    s = C.c_void_p(stream.cuda_stream)

    def step(i):
        lib.kc_mv(s, L.MF_Q4, mats[i % NM][0], LM_D, LM_V, x.data_ptr(), LM_D, y.data_ptr(), LM_V, T, 0, None)
        lib.kc_argmax(s, y.data_ptr(), tok.data_ptr(), LM_V, T)

    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for i in range(W):
            step(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(K):
            step(W + i)
        e1.record(stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1) / K
        evs = []
        for i in range(min(K, 50)):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            lib.kc_mv(s, L.MF_Q4, mats[i % NM][0], LM_D, LM_V, x.data_ptr(), LM_D, y.data_ptr(), LM_V, T, 0, None)
            a1.record(stream)
            evs.append((a0, a1))
        stream.synchronize()
        mv_us = sum(a.elapsed_time(b) for a, b in evs) / len(evs) * 1e3
    L.check()
    nbytes = LM_V * LM_D // 2 + 2 * LM_V * (LM_D // 64) * 2 + T * LM_D * 4 + T * LM_V * 4
    return {"ms_per_step": ms, "tokens": T, "mv_us": mv_us, "bytes": nbytes}


def measure_attn(K, W):
    """Decode attention of BASELINE config 4's shape (GQA 16 query / 2 KV heads of 128, BF16 cache of 4096 positions, 32
    sequences = 134 MB of K and V per layer), an HBM-bound kernel; 3 layers rotated."""
    import torch
    from nanoseedlm_b200 import lib as L
    lib = L.load()
    NH, NKV, CTX, NSEQ, NL = 16, 2, 4096, 32, 3
    NS = int(os.environ.get("NSL_ATTN_SPLITS", "32"))      # 32 splits: the reference host's choice for 32 rows of 4096 keys
    invariant = os.environ.get("NSL_ATTN_INVARIANT", "0") == "1"      # time the form with one block per caller split instead
    lib.nsl_attn_batch_invariant(int(invariant))
    gen = torch.Generator(device="cuda").manual_seed(5)
    caches = [(torch.randn(NSEQ * CTX, NKV, 128, generator=gen, device="cuda").to(torch.bfloat16),
               torch.randn(NSEQ * CTX, NKV, 128, generator=gen, device="cuda").to(torch.bfloat16)) for _ in range(NL)]
    q = torch.randn(NSEQ, NH, 128, generator=gen, device="cuda").to(torch.bfloat16).float()
    g = torch.randn(NSEQ, NH, 128, generator=gen, device="cuda").to(torch.bfloat16).float()
    o = torch.zeros(NSEQ, NH, 128, device="cuda")
    part = torch.zeros(NSEQ * NH * NS * 130, device="cuda")
    ri = (L.RowInfo * NSEQ)()
    for t in range(NSEQ):
        ri[t].pos, ri[t].kv0 = CTX - 1, t * CTX
    rid = torch.empty(NSEQ * 16, dtype=torch.uint8, device="cuda")
    rid.copy_(torch.frombuffer(bytearray(bytes(ri)), dtype=torch.uint8))
    a = L.AttnArgs(NH, NKV, CTX // NS, NS, float(1 / np.sqrt(128.0)))
    views = []
    for kc, vc in caches:
        kv = L.KvView()
        kv.a.k, kv.a.v, kv.nv, kv.fmt = kc.data_ptr(), vc.data_ptr(), NSEQ * CTX, 0
        views.append(kv)
    stream = torch.cuda.Stream()
    s = C.c_void_p(stream.cuda_stream)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for i in range(W):
            lib.kc_attn(s, a, q.data_ptr(), views[i % NL], rid.data_ptr(), part.data_ptr(), g.data_ptr(), o.data_ptr(), NSEQ)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(K):
            lib.kc_attn(s, a, q.data_ptr(), views[(W + i) % NL], rid.data_ptr(), part.data_ptr(), g.data_ptr(), o.data_ptr(), NSEQ)
        e1.record(stream)
        e1.synchronize()
        ms = e0.elapsed_time(e1) / K
    lib.nsl_attn_batch_invariant(0)
    L.check()
    return {"ms_per_step": ms, "tokens": NSEQ, "bytes": 2 * NSEQ * CTX * NKV * 128 * 2 + 3 * NSEQ * NH * 128 * 4, "splits": NS,
            "form": "one block per caller split (batch-invariant)" if invariant else "balanced blocks (default)"}


def measure_upload(K, W):
    """The expert cache's upload paths on config 1's shape: 4 layers x 128 experts in the pinned arena (0.9 GB), 256 slots in
    VRAM; every step asks for 52 experts (a config-1 verify batch's distinct experts) of the next layer, so that nearly all
    of them are misses; time on the consumer stream from before the admit until the units are usable."""
    import torch
    from nanoseedlm_b200 import cache, lib as L
    NL, SL, NREQ = 4, 256, 52
    xc = cache.ExpertCache.random(NL, E, D, FF, SL)
    rng = np.random.default_rng(3)
    reqs = [torch.from_numpy(np.sort(rng.choice(E, NREQ, replace=False)).astype(np.int32)).cuda() for _ in range(16)]
    stream = torch.cuda.Stream()
    out = {"workload": f"expert-cache upload: {NL} layers x {E} experts of {xc.unit_bytes} B pinned on the host, {SL} VRAM slots, "
                       f"{NREQ} experts of the next layer requested per step", "unit_bytes": int(xc.unit_bytes)}
    with torch.cuda.stream(stream):
        for mode, name in ((cache.KERNEL, "copy_kernel"), (cache.DMA, "dma_side_stream")):
            steps = max(8, min(K, 40))
            for i in range(W):
                xc.fetch(stream.cuda_stream, i % NL, reqs[i % 16].data_ptr(), NREQ, mode)
            stream.synchronize()
            st0 = xc.stats()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record(stream)
            for i in range(steps):
                xc.fetch(stream.cuda_stream, (W + i) % NL, reqs[(W + i) % 16].data_ptr(), NREQ, mode)
            e1.record(stream)
            e1.synchronize()
            wall = time.perf_counter() - t0
            st1 = xc.stats()
            units, nbytes = st1["units"] - st0["units"] if mode == cache.DMA else st1["misses"] - st0["misses"], 0
            nbytes = units * xc.unit_bytes
            ms = e0.elapsed_time(e1)
            out[name] = {"steps": steps, "units_uploaded": int(units), "us_per_unit": ms * 1e3 / max(units, 1), "pcie_gbs": nbytes / (ms * 1e-3) / 1e9,
                         "ms_per_step": ms / steps, "host_ms_per_step": wall * 1e3 / steps,
                         "runs": int(st1["runs"] - st0["runs"]) if mode == cache.DMA else None}
    L.check()
    xc.close()
    return out


# ---- config 4: the whole synthetic decoder ---------------------------------------------------------------------------------
C4 = dict(n_layer=48, d=D, n_head=16, n_kv=2, n_exp=512, top_k=10, ff_exp=FF, ff_shared=FF, vocab=151936, ctx=4096)
C4_BATCH = 32


def c4_config(world, layers, batch=C4_BATCH):
    C4_BATCH = batch      # noqa: N806 (the profiling option's batch, printed as it ran)
    return {"workload": f"BASELINE config 4: random-init synthetic MoE decoder, {layers} layers, hidden {D}, GQA 16 query / 2 KV heads of 128, BF16 KV "
                        f"cache with 4096 prefilled positions, 512 seed-encoded routed experts (top-10) + 1 shared expert per layer, vocab 151936 "
                        f"with an affine int4 LM head, decode at batch {C4_BATCH}, experts sharded over {world} GPU(s)",
            "tokens": C4_BATCH, "experts": 512, "top_k": 10, "hidden": D, "intermediate": FF, "layers": layers, "parallelism": f"ep{world}"}


def measure_cfg4(args, K, W):
    """One decode step of the whole decoder for 32 sequences at position 4095 (the rows split over the ranks, the routed experts
    sharded over them), replayed as a CUDA graph; tokens/s = 32 / the step time (max over ranks)."""
    import torch
    import torch.distributed as dist
    from nanoseedlm_b200 import decoder, ep, lib as L
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    c = dict(C4, n_layer=args.c4_layers)
    batch = args.c4_batch if args.c4_batch > 0 and world == 1 else C4_BATCH
    T = batch // world
    e_loc = c["n_exp"] // world
    cfg = decoder.make_cfg(max_rows=T, exp_lo=rank * e_loc, exp_hi=(rank + 1) * e_loc, dense_bf16=int(not args.c4_dense_seed), **c)
    win = ep.P2PWindow.create(world, rank, T, D, c["top_k"]) if world > 1 else None
    dec = decoder.random_decoder(cfg, seed=11, win=win)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    n = T * c["ctx"] * c["n_kv"] * 128
    for l in range(c["n_layer"]):      # the prefilled context
        kk = torch.randn(n, generator=gen, device="cuda").to(torch.bfloat16)
        dec.fill_cache(l, kk, kk.flip(0))
    del kk
    pos, kv0 = [c["ctx"] - 1] * T, [t * c["ctx"] for t in range(T)]
    ri = decoder.row_info(pos, kv0)
    hid = torch.randint(0, c["vocab"], (8, T), generator=gen, device="cuda", dtype=torch.int32)
    pin = hid.cpu().pin_memory()
    ids = torch.zeros(T, dtype=torch.int32, device="cuda")
    nxt = torch.zeros(T, dtype=torch.int32, device="cuda")
    pnext = torch.zeros(T, dtype=torch.int32).pin_memory()
    stream = torch.cuda.Stream()
    lib = L.load()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with torch.cuda.stream(stream):
        launches0 = lib.nsl_launch_count()
        dec.step(ids, ri, T, nxt, stream.cuda_stream)
        stream.synchronize()
        launches = lib.nsl_launch_count() - launches0
        for _ in range(W):
            dec.step(ids, ri, T, nxt, stream.cuda_stream)
        stream.synchronize()
        captured = not args.no_graph
        if captured:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                dec.step(ids, ri, T, nxt, stream.cuda_stream)
            run = g.replay
        else:
            run = lambda: dec.step(ids, ri, T, nxt, stream.cuda_stream)
        run()
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            e0.record(stream)
            for i in range(K):
                ids.copy_(hid[i % 8], non_blocking=True)
                run()
            e1.record(stream)
            e1.synchronize()
        ms = e0.elapsed_time(e1) / K
        # e2e: this step's token ids from pinned host memory, the next tokens back to the host, every step
        if world > 1:
            dist.barrier()
        KE = max(3, min(K, 20))
        t0 = time.perf_counter()
        for i in range(KE):
            ids.copy_(pin[i % 8], non_blocking=True)
            run()
            pnext.copy_(nxt, non_blocking=True)
            stream.synchronize()
        e2e_s = (time.perf_counter() - t0) / KE
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0].item()), float(t[1].item())
    L.check()
    status = 0
    if win is not None:
        status = win.status()
        t = torch.tensor([status], device="cuda", dtype=torch.int64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        status = int(t.item())
        dist.barrier()
    toks = nxt.cpu().numpy()
    dec.close()
    if win is not None:
        win.close()
    torch.cuda.empty_cache()
    if status:
        raise SystemExit(f"config 4: a wait of the expert-parallel exchange ran out (status {status}); the timing is void")
    if rank != 0:
        return None
    return {"value": batch / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms, "gpu_launches": int(launches) * K, "cuda_graph": captured,
            "clocks": clocks.summary(), "config": c4_config(world, c["n_layer"], batch),
            "dense_matrices": "regenerated from their seeds in every call" if args.c4_dense_seed else
                              "expanded once at load to BF16 in HBM (27 MB a layer), the values the tensor-core path rounds seed weights to; "
                              "the routed experts are regenerated from their seeds in every call",
            "e2e": {"value": batch / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4 * T, "d2h_bytes_per_step": 4 * T, "ms_per_step": e2e_s * 1e3,
                    "steps_in_flight": 1},
            "next_tokens_in_vocab": bool(((toks >= 0) & (toks < c["vocab"])).all()),
            "packed_bytes_per_gpu": c["n_layer"] * e_loc * 3 * BYTES_PER_MATRIX}


# ---- config 3: expert-parallel decode ---------------------------------------------------------------------------------------
EP_E, EP_K, EP_B = 512, 10, 64   # BASELINE config 3: 512 routed experts sharded over the ranks, 64 sequences x 1 token, top-10


def ep_config(world):
    return {"workload": f"BASELINE config 3: expert-parallel synthetic MoE decode, {EP_E} seed-encoded experts (hidden {D}, "
                        f"intermediate {FF}) sharded evenly over {world} GPU(s), {EP_B} sequences x 1 token, top-{EP_K}, "
                        "dispatch of bf16 rows and combine of f32 partial sums by the kernels themselves over NVLink peer memory "
                        "(--ep-collectives a2a: NCCL all-to-alls)",
            "tokens": EP_B, "experts": EP_E, "top_k": EP_K, "hidden": D, "intermediate": FF, "parallelism": f"ep{world}"}


def measure_ep(args, K, W, quiet_clocks=False):
    """Config 3 at any N (N = 1: all experts on one GPU, the base of the strong-scaling series).  Returns rank 0's result."""
    import torch
    import torch.distributed as dist
    from nanoseedlm_b200 import ep, lib as L, moe

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    lib = L.load()
    share = max(1, args.ep_share) if world == 1 else 1      # one GPU running the share a rank has at `share` GPUs (profiling)
    n_exp, n_rows = EP_E // share, EP_B // share
    e_loc, t_loc = n_exp // world, n_rows // world
    NL = max(2, min(args.layers, int(6e9 // (e_loc * 3 * BYTES_PER_MATRIX))))
    mirror = bool(args.ep_mirror) and world % 2 == 0 and args.ep_collectives == "p2p"

    def experts_of(r, n_layers=NL):      # rank r's experts of every layer: the same bytes on whichever rank generates them
        g = torch.Generator(device="cuda").manual_seed(4321 + r)
        return [moe.DeviceLayer.random_on_device(D, FF, e_loc, g) for _ in range(n_layers)]

    layers = experts_of(rank)
    if mirror:              # this rank also holds its partner's experts (own first, then the partner's)
        layers = [moe.DeviceLayer.concat(a, b) for a, b in zip(layers, experts_of((rank + world // 2) % world))]
    be = ep.CudaBackend(layers[0])
    epl = ep.ExpertParallelMoe(be, D, EP_K, n_exp, t_loc, collectives=args.ep_collectives, mirror=mirror)
    NB = 8
    rng = np.random.default_rng(7)      # the whole batch on every rank; a rank takes its rows
    gx = bf16r(rng.standard_normal((NB, n_rows, D)).astype(np.float32))
    gl = rng.standard_normal((NB, n_rows, n_exp)).astype(np.float32)
    rows = slice(rank * t_loc, (rank + 1) * t_loc)
    hx, hl = np.ascontiguousarray(gx[:, rows]), np.ascontiguousarray(gl[:, rows])
    dx, dl = torch.from_numpy(hx).cuda(), torch.from_numpy(hl).cuda()
    px, pl = torch.from_numpy(hx).pin_memory(), torch.from_numpy(hl).pin_memory()
    pout = torch.zeros(t_loc, D).pin_memory()
    sx, sl = torch.zeros(t_loc, D, device="cuda"), torch.zeros(t_loc, n_exp, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    def one(i):
        be.set_layer(layers[i % NL])
        return epl.step(dx[i % NB], dl[i % NB])

    # ---- parity, before anything is timed: one step on batch 0 and layer 0 against the ONE-GPU layer over all 512 experts
    # (rank 0 regenerates every rank's experts of layer 0 from their seeds and runs the plain mat-vec path on all 64 rows)
    parity = None
    with torch.cuda.stream(stream):
        mine = one(0).clone()
        stream.synchronize()
    if world > 1:
        allout = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allout, mine)
        got = torch.cat(allout).cpu().numpy()
    else:
        got = mine.cpu().numpy()
    if rank == 0:
        whole = layers[0] if world == 1 and not mirror else None
        if whole is None:
            parts = [experts_of(r, 1)[0] for r in range(world)]
            whole = parts[0]
            for p in parts[1:]:
                whole = moe.DeviceLayer.concat(whole, p)
        m1 = moe.Moe(whole, EP_K, n_rows)
        m1.set_grouped_min_tokens(10 ** 6)
        want, _ = m1.forward_host(gx[0], gl[0])
        m1.close()
        del whole
        rel = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
        parity = {"checked": True, "max_rel": rel, "bar": 1e-5, "against": "the one-GPU MoE layer (all 512 experts, plain mat-vec path) on the same "
                  "seeded batch and layer; the partial sums are added per rank first, so the order of the f32 sums differs"}
    torch.cuda.empty_cache()

    with torch.cuda.stream(stream):
        for i in range(W):
            one(i)
        stream.synchronize()
        launches0 = lib.nsl_launch_count()
        one(W)
        stream.synchronize()
        launches = (lib.nsl_launch_count() - launches0) * K
        captured = not args.no_graph
        if captured:
            combos = sorted({(i % NB, i % NL) for i in range(2 * W + K + 1)}) if args.ep_collectives == "p2p" else ()
            gs = ep.GraphedSteps(epl, layers, [(dx[b], dl[b]) for b in range(NB)], whole=combos)      # one graph per step
            run_step = lambda i: gs.step(i % NB, i % NL)
        else:
            run_step = one
        for i in range(W):
            run_step(i)
        stream.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            e0.record(stream)
            for i in range(K):
                run_step(W + i)
            e1.record(stream)
            e1.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        # e2e: the rank's token rows and logits from pinned host memory, its output rows back, every step
        KE = min(K, 500)
        for i in range(W):
            sx.copy_(px[i % NB], non_blocking=True); sl.copy_(pl[i % NB], non_blocking=True)
            be.set_layer(layers[i % NL]); pout.copy_(epl.step(sx, sl), non_blocking=True); stream.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for i in range(KE):
            sx.copy_(px[(W + i) % NB], non_blocking=True); sl.copy_(pl[(W + i) % NB], non_blocking=True)
            be.set_layer(layers[(W + i) % NL]); pout.copy_(epl.step(sx, sl), non_blocking=True); stream.synchronize()
        e2e_s = (time.perf_counter() - t0) / KE
    pairs = int(be.count.item())
    if world > 1:
        t = torch.tensor([ms, e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_s = float(t[0].item()), float(t[1].item())
    L.check()
    p2p_status = None
    if epl.window is not None:
        p2p_status = epl.window.status()          # non-zero: a bounded wait on another rank ran out
        if world > 1:
            t = torch.tensor([p2p_status], device="cuda", dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            p2p_status = int(t.item())
            dist.barrier()
        epl.window.close()
    del layers, be, epl
    torch.cuda.empty_cache()
    if p2p_status:
        raise SystemExit(f"expert-parallel p2p exchange: a wait ran out (status {p2p_status}); the timing is void")
    ms_per_step = ms / K
    if rank != 0:
        return None
    if parity is not None:
        parity["status"] = p2p_status or 0
        if not parity["max_rel"] <= parity["bar"]:
            raise SystemExit(f"expert-parallel step differs from the one-GPU layer: max relative error {parity['max_rel']:.3e}; the timing is void")
    peaks, peak_kind = measured_peaks()
    # the whole step against the packed-bytes roofline: the experts a step touches, in expectation over the routing
    # (E (1 - (1 - k/E)^B) distinct experts of 3 matrices each), read once by whichever rank owns them
    distinct = n_exp * (1.0 - (1.0 - EP_K / n_exp) ** n_rows)
    gbs = distinct * 3 * BYTES_PER_MATRIX / (ms_per_step * 1e-3) / 1e9
    res = {"value": n_rows / (ms_per_step * 1e-3), "ms_per_step": ms_per_step, "gpu_launches": int(launches), "cuda_graph": captured,
           "collectives": args.ep_collectives, "mirrored_ranks": mirror, "clocks": clocks.summary(), "l2_policy": l2_policy(NL, e_loc),
           "pairs_on_rank0_last_step": pairs, "parity": parity,
           "e2e": {"value": n_rows / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": t_loc * D * 4 + t_loc * n_exp * 4,
                   "d2h_bytes_per_step": t_loc * D * 4, "ms_per_step": e2e_s * 1e3, "steps_in_flight": 1},
           "roofline": {"bound": "hbm", "kernel": "the step's seed mat-vecs (gate+up and down over the ranks' pairs: mv_grp_kernel beyond 64 pairs a rank, else mv_pair_kernel)",
                        "achieved": gbs, "peak": peaks["hbm_gbs"] * world, "unit": "GB/s", "frac": gbs / (peaks["hbm_gbs"] * world),
                        "peak_kind": peak_kind, "traffic": None, "expected_distinct_experts": distinct,
                        "note": "whole step (mat-vecs + exchange) over the aggregate HBM peak of the ranks; the kernels are bound by "
                                "the logic pipe, see the 1-GPU line for the per-kernel roofline"}}
    sm = res["clocks"].get("sm_mhz")
    if sm:      # the logic-pipe floor of the step: every distinct expert's three matrices expanded once, over all the ranks' SMs
        blocks = distinct * 3 * BLOCKS_PER_MATRIX
        res["roofline"]["alu"] = alu_roofline(ms_per_step * 1e3, blocks, sm, lib.nsl_sm_count() * world)
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="config 1: 1..8 (default 8); config 2: prompt rows (default 512)")
    ap.add_argument("--layers", type=int, default=20)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="N = 1: the headline only, without the `workloads` and `ep_base` objects")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--c4-dense-seed", action="store_true", help="config 4: regenerate the dense matrices from their seeds in every call too")
    ap.add_argument("--c4-batch", type=int, default=0, help="config 4: sequences per step (32 = the configuration; fewer only for profiling "
                                                             "one rank's dense and attention sizes on one GPU)")
    ap.add_argument("--c4-layers", type=int, default=48, help="config 4: decoder layers (48 = the configuration; fewer only for profiling)")
    ap.add_argument("--one-launch", action="store_true", help="config 1: the decode step as one fused launch instead of three dependent launches")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="config 1: ordinary launches instead of programmatic dependent launches (for comparison)")
    ap.add_argument("--ep-collectives", default="p2p", choices=["p2p", "a2a", "gather"],
                    help="config 3: p2p (default): no collective call, the kernels store into the other ranks' memory over "
                         "NVLink and wait on counters; a2a: two NCCL all-to-alls; gather: all-gather + reduce-scatter")
    ap.add_argument("--ep-mirror", type=int, default=0,
                    help="config 3, p2p, even rank counts: 1 = ranks r and r + N/2 hold each other's experts too and split their "
                         "joint pairs in the middle (balance to within one pair; twice the expert bytes per GPU)")
    ap.add_argument("--ep-share", type=int, default=1,
                    help="config 3 on ONE GPU, profiling: run the share one rank has at this many GPUs (512 / n experts, 64 / n rows x "
                         "top-10: the pair count and expert count of a rank's mat-vecs, without the other ranks)")
    ap.add_argument("--workload", default=None, choices=["cfg0", "cfg1", "cfg2", "cfg3", "cfg4", "lmhead", "attn", "upload", "p3"],
                    help="one workload alone as the line (profiling): cfg1 one GPU's MoE decode layer; cfg2 the same layer on 512 "
                         "prompt rows (grouped tcgen05 GEMM); cfg3 expert-parallel decode (the default at >1 GPU); cfg0 / lmhead / attn")
    args = ap.parse_args()
    global ONE_LAUNCH
    ONE_LAUNCH = args.one_launch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        workload = args.workload or ("cfg1" if max(world, args.gpus) == 1 else "cfg3")
        args.tokens = args.tokens or (512 if workload == "cfg2" else 8)
        if rank == 0:
            run_reference(args, workload)
        return
    import torch
    import torch.distributed as dist
    from nanoseedlm_b200 import lib as L
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = L.load()
    peaks, peak_kind = measured_peaks()
    sms = lib.nsl_sm_count()
    K, W = args.steps, max(args.warmup, 3)
    workload = args.workload or ("cfg1" if world == 1 else "cfg3")
    base = {"metric": METRIC, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic"}

    if workload == "cfg3":
        r = measure_ep(args, K, W)
        if rank == 0:
            line = dict(base, value=r.pop("value"), ms_per_step=r.pop("ms_per_step"), config=ep_config(world), workload_id="cfg3", **r)
            if world == 1 and args.ep_share > 1:
                line["workload_id"] = f"cfg3_share_of_{args.ep_share}"
                line["config"] = dict(line["config"], share=f"one rank's share at {args.ep_share} GPUs: {EP_E // args.ep_share} experts, "
                                                            f"{EP_B // args.ep_share} rows x top-{EP_K}, alone on one GPU (no exchange partner)")
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()
        return

    if workload == "cfg4":
        r = measure_cfg4(args, min(K, 30), min(W, 3))
        if rank == 0:
            print(json.dumps(dict(base, metric="synthetic_moe_decoder_tokens_per_s", value=r.pop("value"), ms_per_step=r.pop("ms_per_step"),
                                  config=r.pop("config"), workload_id="cfg4", steps=min(K, 30), warmup=min(W, 3), **r)))
        if world > 1:
            dist.destroy_process_group()
        return

    if workload in ("cfg0", "lmhead", "attn", "upload", "p3"):      # one secondary workload alone
        print(json.dumps(dict(base, **secondary(workload, K, W, peaks, peak_kind, sms, args))))
        return

    M = args.tokens or (512 if workload == "cfg2" else 8)
    if workload == "cfg1" and not 1 <= M <= 8:
        raise SystemExit("config 1 is the decode / verify batch: --tokens 1..8 (use --workload cfg2 for prompt rows)")
    c = Cfg1(args.layers)
    r = measure_layer(c, M, K, W, dependent_launch=not args.no_dependent_launch)
    clocks = r["clocks"]
    line = dict(base, value=r["value"], ms_per_step=r["ms_per_step"], config=workload_config(M), workload_id=f"cfg1_m{M}" if M <= 8 else "cfg2",
                l2_policy=l2_policy(args.layers), packed_gbs=r["packed_gbs"], gpu_launches=r["gpu_launches"], clocks=clocks, e2e=r["e2e"],
                roofline=layer_roofline(r, M, clocks.get("sm_mhz"), sms, peaks, peak_kind))
    extra = args.workload is None and not args.no_extra
    if extra:
        Kx = min(K, 1000)
        wl = {}
        for m_ in (1, 4):
            rr = measure_layer(c, m_, Kx, W, sample_clocks=False)
            wl[f"cfg1_m{m_}"] = {"ms_per_step": rr["ms_per_step"], "value": rr["value"], "unit": "tok/s", "e2e": rr["e2e"],
                                 "roofline": layer_roofline(rr, m_, clocks.get("sm_mhz"), sms, peaks, peak_kind)}
        rr = measure_layer(c, 512, min(K, 200), W, sample_clocks=False)
        wl["cfg2"] = {"ms_per_step": rr["ms_per_step"], "value": rr["value"], "unit": "tok/s", "e2e": rr["e2e"],
                      "roofline": layer_roofline(rr, 512, clocks.get("sm_mhz"), sms, peaks, peak_kind),
                      "layer_alu": alu_roofline(rr["ms_per_step"] * 1e3, 3 * E * BLOCKS_PER_MATRIX, clocks.get("sm_mhz") or 1965.0, sms)}
        line["workloads"] = wl
    step0 = r["step0"]
    layer0 = c.layers[0]
    if M <= 8 and not args.no_extra:      # the reference's own CUDA kernels on the same layers and inputs (a baseline, like the CPU's)
        line["ref_gpu"] = measure_ref_gpu(c, M, min(K, 400), W, mine_out=step0[2])
        if extra and "ms_per_step" in line["ref_gpu"]:
            keep = ("ms_per_step", "value", "unit", "launches_per_step")
            line["ref_gpu"]["m1"] = {k_: v for k_, v in measure_ref_gpu(c, 1, min(K, 400), W).items() if k_ in keep}
            line["ref_gpu"]["cfg2"] = {k_: v for k_, v in measure_ref_gpu(c, 512, 40, W).items() if k_ in keep}
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_cfg1(os.cpu_count() or 1, M, layer0 if M <= 8 else None, step0[0], step0[1], step0[2] if M <= 8 else None)
    del c, r
    torch.cuda.empty_cache()
    if extra and "ms_per_step" in line.get("ref_gpu", {}):      # the reference's kc_mv (MF_Q4) + kc_argmax on the LM head
        from oracle import ref_gpu
        rl = measure_lmhead(8, 100, W, lib=ref_gpu.lib())
        line["ref_gpu"]["lmhead"] = {"ms_per_step": rl["ms_per_step"], "value": rl["tokens"] / (rl["ms_per_step"] * 1e-3), "unit": "tok/s"}
        torch.cuda.empty_cache()
    if extra:
        for name in ("cfg0", "lmhead", "attn", "upload", "p3"):
            line["workloads"][name] = secondary(name, min(K, 1000), W, peaks, peak_kind, sms, args, sm_mhz=clocks.get("sm_mhz"))
            torch.cuda.empty_cache()
        try:      # the whole decoder of config 4 on this one GPU (44 GB of experts): reported, with its error if it cannot run
            r4 = measure_cfg4(args, 10, 2)
            line["workloads"]["cfg4"] = {k_: r4[k_] for k_ in ("value", "unit", "ms_per_step", "e2e", "gpu_launches", "cuda_graph", "next_tokens_in_vocab", "dense_matrices")}
            line["workloads"]["cfg4"]["workload"] = r4["config"]["workload"]
        except Exception as ex:      # noqa: BLE001
            line["workloads"]["cfg4"] = {"error": repr(ex)}
        torch.cuda.empty_cache()
        rr = measure_ep(args, min(K, 400), W)
        line["ep_base"] = {"workload": ep_config(1)["workload"], "value": rr["value"], "unit": "tok/s", "ms_per_step": rr["ms_per_step"],
                           "e2e": rr["e2e"], "parity": rr["parity"], "roofline": rr["roofline"],
                           "note": "config 3 with all 512 experts on this one GPU: the base of the strong-scaling series the N > 1 lines "
                                   "continue (speed-up at N = this ms_per_step / the N-GPU line's ms_per_step)"}
    print(json.dumps(line))


def measure_p3(K, W):
    """The config-1 / config-2 layer with P = 3 (MF_SEED4) experts: 8 decode rows through kc_mv_gu / kc_mv_sel (the pair
    kernel's P = 3 form) and 512 prompt rows through kc_bucket + kc_mm_grouped_dev (the tcgen05 GEMM with the
    P = 3 tile producer).  4 layers rotated (0.8 GB of packed streams)."""
    import torch
    from nanoseedlm_b200 import kernels, lib as L
    lib = L.load()
    NL, nb = 4, D * FF // 8
    gen = torch.Generator(device="cuda").manual_seed(303)
    keep, tabs = [], []
    for _ in range(NL):
        lay = []
        for _m in range(3):      # gate, up [FF][D]; down [D][FF]: the same block count
            seeds = torch.randint(1, 65536, (E, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
            nibs = torch.randint(0, 65536, (E, nb), generator=gen, device="cuda", dtype=torch.int32).to(torch.int16)
            arr = (L.WSlice * E)()
            for e in range(E):
                arr[e].p[0], arr[e].p[1], arr[e].eb = seeds[e].data_ptr(), nibs[e].data_ptr(), -22
            tab = torch.empty(E * C.sizeof(L.WSlice), dtype=torch.uint8, device="cuda")
            tab.copy_(torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8))
            keep += [seeds, nibs]
            lay.append(tab)
        tabs.append(lay)
    G = kernels.stream_table()
    stream = torch.cuda.Stream()
    s = stream.cuda_stream
    out = {}
    for M in (8, 512):
        P = M * TOPK
        rng = np.random.default_rng(5 + M)
        x = torch.from_numpy(bf16r(rng.standard_normal((M, D)).astype(np.float32))).cuda()
        lg = torch.from_numpy(rng.standard_normal((M, E)).astype(np.float32)).cuda()
        ind, wt = torch.zeros(P, dtype=torch.int32, device="cuda"), torch.zeros(P, device="cuda")
        A, U, Dx = torch.zeros(P, FF, device="cuda"), torch.zeros(P, FF, device="cuda"), torch.zeros(P, D, device="cuda")
        perm = torch.zeros(P, dtype=torch.int32, device="cuda")
        tiles = torch.zeros((P // 128 + E + 1) * 4, dtype=torch.int32, device="cuda")
        work = torch.zeros(2 * E + 3, dtype=torch.int32, device="cuda")
        res, sh, sg = torch.zeros(M, D, device="cuda"), torch.zeros(M, D, device="cuda"), torch.zeros(M, device="cuda")
        mt = P // 128 + E

        def step(i):
            g, u, d = (t.data_ptr() for t in tabs[i % NL])
            lib.nsl_route(s, E, TOPK, lg.data_ptr(), E, ind.data_ptr(), wt.data_ptr(), M)
            if M <= 8:
                lib.kc_mv_gu(s, L.MF_SEED4, g, u, D, FF, x.data_ptr(), D, A.data_ptr(), FF, ind.data_ptr(), P, TOPK, G.data_ptr())
                lib.kc_mv_sel(s, L.MF_SEED4, d, FF, D, A.data_ptr(), FF, Dx.data_ptr(), D, ind.data_ptr(), P, 1, G.data_ptr())
            else:
                lib.kc_bucket(s, ind.data_ptr(), P, E, perm.data_ptr(), tiles.data_ptr(), work.data_ptr())
                for tab, dst in ((g, A), (u, U)):
                    lib.kc_mm_grouped_dev(s, L.MF_SEED4, tab, D, FF, x.data_ptr(), D, dst.data_ptr(), FF, TOPK, perm.data_ptr(), tiles.data_ptr(),
                                          work.data_ptr(), mt, G.data_ptr())
                lib.kc_swiglu(s, A.data_ptr(), U.data_ptr(), A.data_ptr(), P * FF)
                lib.kc_mm_grouped_dev(s, L.MF_SEED4, d, FF, D, A.data_ptr(), FF, Dx.data_ptr(), D, 1, perm.data_ptr(), tiles.data_ptr(),
                                      work.data_ptr(), mt, G.data_ptr())
            lib.kq4_moe_combine(s, D, TOPK, Dx.data_ptr(), wt.data_ptr(), sh.data_ptr(), sg.data_ptr(), 1, res.data_ptr(), M)

        n = min(K, 200)
        with torch.cuda.stream(stream):
            for i in range(max(W, 3)):
                step(i)
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for i in range(n):
                step(W + i)
            e1.record(stream)
            e1.synchronize()
        L.check()
        ms = e0.elapsed_time(e1) / n
        out[f"m{M}"] = {"ms_per_step": ms, "value": M / (ms * 1e-3), "unit": "tok/s", "finite": bool(torch.isfinite(res).all().item())}
    out["mm_status"] = int(lib.nsl_mm_status())
    return out


def secondary(name, K, W, peaks, peak_kind, sms, args, sm_mhz=None):
    """cfg0, the LM head or decode attention as a result object with its roofline."""
    if name == "cfg0":
        r = measure_cfg0(K, W)
        gbs = r["bytes"] / (r["us"] * 1e-6) / 1e9
        out = {"workload": "BASELINE config 0: dense seed mat-vec, 2048 outputs x 4096 inputs, 1 token, raw f32 output; 32 matrices rotated (151 MB)",
               "ms_per_step": r["us"] * 1e-3, "value": 1.0 / (r["us"] * 1e-6), "unit_note": "mat-vecs / s", "gweights_per_s": r["weights"] / (r["us"] * 1e-6) / 1e9,
               "roofline": {"bound": "hbm", "kernel": "mv_smemx_kernel (nsl_mv_raw / kc_mv)", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": gbs / peaks["hbm_gbs"], "peak_kind": peak_kind, "alu": alu_roofline(r["us"], r["blocks"], sm_mhz or 1965.0, sms)}}
        if not args.no_cpu:
            out["cpu_baseline"] = cpu_cfg0_protocol()
        return out
    if name == "upload":
        return measure_upload(K, W)
    if name == "p3":
        r = measure_p3(K, W)
        return dict(r, workload=f"the config-1 / config-2 layer with P = 3 (MF_SEED4) experts: hidden {D}, {E} experts of intermediate {FF}, top-{TOPK}; "
                                "8 decode rows (the pair kernel's P = 3 form) and 512 prompt rows (tcgen05 GEMM with the P = 3 tile producer)")
    if name == "lmhead":
        r = measure_lmhead(8, min(K, 300), W)
        gbs = r["bytes"] / (r["mv_us"] * 1e-6) / 1e9
        return {"workload": f"dense affine-int4 LM head {LM_V} x {LM_D} (groups of 64) + greedy arg-max, 8 tokens; 4 heads rotated (0.7 GB)",
                "ms_per_step": r["ms_per_step"], "value": r["tokens"] / (r["ms_per_step"] * 1e-3), "unit": "tok/s",
                "roofline": {"bound": "hbm", "kernel": "q4_mv_ksplit_kernel (kc_mv, MF_Q4)", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": gbs / peaks["hbm_gbs"], "peak_kind": peak_kind, "us_per_launch": r["mv_us"], "bytes_per_launch": r["bytes"]}}
    r = measure_attn(min(K, 500), W)
    gbs = r["bytes"] / (r["ms_per_step"] * 1e-3) / 1e9
    return {"workload": f"decode attention, 16 query / 2 KV heads of 128, BF16 cache of 4096 positions x 32 sequences (134 MB per layer), {r['splits']} splits, "
                        f"{r['form']}; 3 layers rotated",
            "ms_per_step": r["ms_per_step"], "value": r["tokens"] / (r["ms_per_step"] * 1e-3), "unit": "tok/s",
            "roofline": {"bound": "hbm", "kernel": "attn_flat_mma_kernel + attn_reduce_kernel (kc_attn)", "achieved": gbs, "peak": peaks["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "peak_kind": peak_kind, "bytes_per_step": r["bytes"]}}


if __name__ == "__main__":
    main()
