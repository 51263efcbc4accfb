#!/usr/bin/env python
"""Benchmark of the seed-decode MoE expert layer (BASELINE.json config 1) on B200.

    python bench.py --gpus 1 --steps 200 --warmup 10              # this library (CUDA kernels behind the C ABI)
    python bench.py --impl reference --steps 3 --warmup 1          # the CPU seed path on the host cores

A step is one pass of the hot path over one batch: router top-8 over 128 experts, the routed experts' gate + up +
SwiGLU and down projections regenerated from their seeds, and the weighted combine, for M tokens (default 8, the
multi-token-prediction verify batch; --tokens 1 or 4 give the other rows of config 1).  Steps rotate over enough
independent synthetic layers that every step's packed streams come from HBM, not L2.

One JSON line is printed (rank 0).  value = tokens/s with inputs resident in HBM; e2e = the same through
nsl_moe_forward_pinned with host buffers (H2D of the step's inputs from pinned memory, D2H of its output, every step);
roofline = the dominant kernel (gate+up mat-vec) against the measured HBM copy peak; cpu_baseline = the CPU
restatement of the reference's seed mat-vec timed on this host."""
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
WEIGHTS_PER_TOKEN = TOPK * 3 * D * FF                      # 25,165,824


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


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


class CpuMoe:
    """One MoE step on the host cores with the CPU seed kernels (the gcc restatement of nslm/lib_cpu_seed4.c) in their
    fastest form: the CPU-tiled layout, the rows that share an expert multiplied together (up to 8 per call, the
    kernel's limit), every routed expert's gate and up products in one parallel region over all host threads, then
    every down product in a second one.  Experts draw their matrices from a pool of `pool` distinct ones."""

    def __init__(self, n_exp, top_k, threads, pool=8):
        from oracle import binding as B
        self.B, self.n_exp, self.top_k, self.threads = B, n_exp, top_k, threads
        self.gate = [B.Tiled(B.Matrix(FF, D, 300 + i)) for i in range(pool)]
        self.up = [B.Tiled(B.Matrix(FF, D, 400 + i)) for i in range(pool)]
        self.down = [B.Tiled(B.Matrix(D, FF, 500 + i)) for i in range(pool)]

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
        B, P = self.B, len(self.gate)
        xs = [x[[t for t, _ in rows]] for _, rows in groups]
        gu = B.tiled_jobs([(self.gate[e % P], xe) for (e, _), xe in zip(groups, xs)] +
                          [(self.up[e % P], xe) for (e, _), xe in zip(groups, xs)], self.threads)
        n = len(groups)
        act = [g / (1.0 + np.exp(-g)) * u for g, u in zip(gu[:n], gu[n:])]
        dn = B.tiled_jobs([(self.down[e % P], a) for (e, _), a in zip(groups, act)], self.threads)
        out = np.zeros_like(x)
        for (_, rows), y in zip(groups, dn):
            for i, (t, w) in enumerate(rows):
                out[t] += w * y[i]
        return out, sum(len(rows) for _, rows in groups)


def cpu_inputs(M, n_exp, seed=99):
    rng = np.random.default_rng(seed)
    return rng.standard_normal((M, D)).astype(np.float32), rng.standard_normal((M, n_exp)).astype(np.float32)


def cpu_baseline(threads, M, n_exp=E, top_k=TOPK, seconds=12.0):
    """The CPU path on a bounded sample: whole steps of the same workload, repeated for about `seconds`."""
    cpu = CpuMoe(n_exp, top_k, threads)
    x, logits = cpu_inputs(M, n_exp)
    groups = cpu.groups(logits)
    cpu.run(x, groups)   # warm-up
    times, t_end = [], time.perf_counter() + seconds
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 200):
        t0 = time.perf_counter()
        cpu.run(x, groups)
        times.append(time.perf_counter() - t0)
    dt = float(np.median(times))
    distinct = len({e for e, _ in groups})
    return {"value": M / dt, "unit": "tok/s", "cores": threads, "kind": "port", "ms_per_step": dt * 1e3,
            "gweights_per_s": distinct * 3 * D * FF / dt / 1e9,
            "sample": f"{len(times)} whole steps (median) of {M} rows x top-{top_k} of {n_exp} experts = {distinct} distinct experts x "
                      f"(gate, up, down) on {threads} host threads: CPU-tiled layout, rows sharing an expert multiplied together; "
                      "the reference's own kernel needs Clang, this is its gcc restatement (oracle/cpu_seed4_tiled.c)"}


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
    cfg = ep_config(args.gpus, args.layers) if workload == "cfg3" else workload_config(M)
    line = {"impl": "reference", "metric": "seed_decode_moe_gemv_tokens_per_s", "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong" if workload == "cfg3" else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": f"each step = {take} of the step's {len(groups)} (expert, <= 8 rows) groups "
                                       f"({done // args.steps} of {pairs} (row, expert) pairs), scaled to whole steps; CPU-tiled "
                                       f"seed kernels on {threads} host threads (gcc restatement of nslm/lib_cpu_seed4.c; the "
                                       "original needs Clang)"},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(M, layers=None):
    which = "config 1: synthetic MoE expert layer at decode" if M <= 8 else "config 2: synthetic MoE prefill / continuous-batching grouped GEMM"
    c = {"workload": f"BASELINE {which}, hidden {D}, {E} seed-encoded (SEED4P4) "
                     f"SwiGLU experts of intermediate {FF}, softmax top-{TOPK}, M={M} tokens, all experts resident",
         "tokens": M, "experts": E, "top_k": TOPK, "hidden": D, "intermediate": FF}
    if layers:
        c["l2_policy"] = (f"steps rotate over {layers} independent layers ({layers * E * 3 * BYTES_PER_MATRIX / 1e9:.1f} GB of "
                          "packed streams, far larger than the 126 MB L2), so each step's experts are read from HBM")
    return c


def run_ours(args):
    import torch
    import torch.distributed as dist
    from nanoseedlm_b200 import lib as L, moe

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = L.load()
    M, K, W, NL = args.tokens, args.steps, max(args.warmup, 3), args.layers
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    layers = [moe.DeviceLayer.random_on_device(D, FF, E, gen) for _ in range(NL)]
    torch.cuda.synchronize()
    m = moe.Moe(layers[0], TOPK, M)
    m.set_dependent_launch(not args.no_dependent_launch)

    # inputs: a pool of distinct batches (bf16-valued activations, N(0,1) logits), on the host and on the device
    NB = 16
    rng = np.random.default_rng(99 + rank)
    hx = rng.standard_normal((NB, M, D)).astype(np.float32)
    hx = (hx.view(np.uint32) + 0x7FFF + ((hx.view(np.uint32) >> 16) & 1) & 0xFFFF0000).view(np.float32)
    hl = rng.standard_normal((NB, M, E)).astype(np.float32)
    dx, dl = torch.from_numpy(hx).cuda(), torch.from_numpy(hl).cuda()
    dout = torch.zeros(M, D, device="cuda")
    distinct = [len(set(np.argsort(-hl[b], axis=1, kind="stable")[:, :TOPK].ravel().tolist())) for b in range(NB)]

    stream = torch.cuda.Stream()
    peaks, peak_kind = measured_peaks()

    def enqueue(step, s):
        m.set_layer(layers[step % NL])
        m.forward_dev(dx[step % NB], dl[step % NB], dout, stream=s.cuda_stream)

    # ---- value: inputs resident in HBM; the K steps are captured once as a CUDA graph and replayed ------------------
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
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local) as clocks:
            e0.record(stream)
            for _ in range(K // chunk):
                graph.replay()
            for i in range(K % chunk):
                enqueue(W + i, stream)
            e1.record(stream)
            e1.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / K
    value = world * M / (ms_per_step * 1e-3)

    # ---- roofline of the dominant kernel (gate+up mat-vec): CUDA events around each of its launches ------------------
    G = m.G
    A = torch.zeros(M * TOPK, FF, device="cuda")
    ind = torch.zeros(M * TOPK, dtype=torch.int32, device="cuda")
    wt = torch.zeros(M * TOPK, device="cuda")
    perm = torch.zeros(M * TOPK, dtype=torch.int32, device="cuda")
    tiles = torch.zeros((M * TOPK // 128 + E + 1) * 4, dtype=torch.int32, device="cuda")
    work = torch.zeros(2 * E + 3, dtype=torch.int32, device="cuda")
    gu_ms, gu_bytes = 0.0, 0.0
    with torch.cuda.stream(stream):
        evs = []
        KR = min(K, 400)   # launches of the dominant kernel timed one by one
        for i in range(KR):
            lay, b = layers[(W + i) % NL], (W + i) % NB
            lib.nsl_route(stream.cuda_stream, E, TOPK, dl[b].data_ptr(), E, ind.data_ptr(), wt.data_ptr(), M)
            if M > 8:
                lib.kc_bucket(stream.cuda_stream, ind.data_ptr(), M * TOPK, E, perm.data_ptr(), tiles.data_ptr(), work.data_ptr())
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            if M > 8:
                lib.kc_mm_grouped_dev(stream.cuda_stream, L.MF_SEED4P4, lay.gate.table.data_ptr(), D, FF, dx[b].data_ptr(), D,
                                      A.data_ptr(), FF, TOPK, perm.data_ptr(), tiles.data_ptr(), work.data_ptr(),
                                      M * TOPK // 128 + E, G.data_ptr())
            else:
                lib.kc_mv_gu(stream.cuda_stream, L.MF_SEED4P4, lay.gate.table.data_ptr(), lay.up.table.data_ptr(), D, FF,
                             dx[b].data_ptr(), D, A.data_ptr(), FF, ind.data_ptr(), M * TOPK, TOPK, G.data_ptr())
            a1.record(stream)
            evs.append((a0, a1, b))
        stream.synchronize()
        for a0, a1, b in evs:
            gu_ms += a0.elapsed_time(a1)
            gu_bytes += distinct[b] * (1 if M > 8 else 2) * BYTES_PER_MATRIX + M * D * 4 + M * TOPK * FF * 4
    gu_us = gu_ms * 1e3 / KR
    achieved = gu_bytes / KR / (gu_us * 1e-6) / 1e9

    # ---- e2e: host buffers through the C host layer, H2D and D2H inside every step -----------------------------------
    for i in range(W):
        m.set_layer(layers[i % NL])
        m.hx[:M], m.hlogits[:M] = hx[i % NB], hl[i % NB]
        m.forward_pinned(M)
    if world > 1:
        dist.barrier()
    KE = min(K, 2000)
    t0 = time.perf_counter()
    for i in range(KE):
        m.set_layer(layers[(W + i) % NL])
        m.hx[:M], m.hlogits[:M] = hx[(W + i) % NB], hl[(W + i) % NB]
        m.forward_pinned(M)
    e2e_sync_s = (time.perf_counter() - t0) / KE
    # the same with two handles used alternately: step i + 1 is submitted (its H2D copies and launches) before the host
    # waits for step i's output, so copies and launch latency hide under the other step's kernels
    m2 = moe.Moe(layers[0], TOPK, M)
    m2.set_dependent_launch(not args.no_dependent_launch)
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
    e2e_s = (time.perf_counter() - t0) / KE
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    L.check()

    if rank == 0:
        line = {"metric": "seed_decode_moe_gemv_tokens_per_s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K,
                "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "config": workload_config(M, NL),
                "packed_gbs": world * sum(distinct[(W + i) % NB] for i in range(K)) / K * 3 * BYTES_PER_MATRIX / (ms_per_step * 1e-3) / 1e9,
                "gpu_launches": int(launches), "clocks": clocks.summary(),
                "e2e": {"value": world * M / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": M * D * 4 + M * E * 4,
                        "d2h_bytes_per_step": M * D * 4, "ms_per_step": e2e_s * 1e3, "steps_in_flight": 2,
                        "one_step_in_flight": {"value": world * M / e2e_sync_s, "ms_per_step": e2e_sync_s * 1e3}},
                "roofline": {"bound": "hbm", "kernel": "mv_shx_kernel<gate+up> (kc_mv_gu)", "achieved": achieved, "peak": peaks["hbm_gbs"],
                             "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_kind": peak_kind, "traffic": 57.5e6 if M == 8 else None,
                             "us_per_launch": gu_us,
                             "note": "the kernel is bound by the integer/logic pipe (LFSR expansion: 53 logic ops per 8 weights), "
                                     "at about 65 % of that roofline; HBM traffic equals the algorithmic bytes (ncu, profiles/)"}}
        if M <= 8 and line["clocks"].get("sm_mhz"):
            # the second roofline of this kernel: the logic pipe.  Each (row, expert) pair expands gate and up once:
            # 2 * FF * D / 8 blocks of 8 weights; an SM retires 64 logic lane-ops per clock and a block needs 53 of them
            blocks = M * TOPK * 2 * FF * D // 8
            clk = gu_us * 1e-6 * line["clocks"]["sm_mhz"] * 1e6 * lib.nsl_sm_count() / blocks
            line["roofline"]["alu"] = {"blocks_per_launch": blocks, "clk_per_block_per_sm": clk, "floor_clk_per_block_per_sm": 53 / 64,
                                       "frac": 53 / 64 / clk, "bytes_time_us": gu_bytes / KR / (peaks["hbm_gbs"] * 1e9) * 1e6,
                                       "alu_floor_time_us": gu_us * 53 / 64 / clk}
        if M > 8:   # prompt rows: the dominant kernel is the grouped tcgen05 GEMM (gate projection timed)
            tf = 2.0 * M * TOPK * FF * D / (gu_us * 1e-6) / 1e12
            line["roofline"] = {"bound": "tensor", "kernel": "seed_gemm_kernel<1> (kc_mm_grouped_dev, gate projection)", "achieved": tf,
                                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops"], "peak_kind": peak_kind,
                                "traffic": None, "us_per_launch": gu_us, "packed_gbs": achieved,
                                "note": "producer-bound: regenerating a weight tile costs ~100 instructions per 8 weights, the tensor "
                                        "pipe idles by construction (ncu: sm__pipe_tensor_cycles_active 3 %)"}
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(os.cpu_count() or 1, M)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


EP_E, EP_K, EP_B = 512, 10, 64   # BASELINE config 3: 512 experts sharded over the ranks, 64 sequences x 1 token, top-10


def ep_config(world, layers):
    return {"workload": f"BASELINE config 3: expert-parallel synthetic MoE decode, {EP_E} seed-encoded experts (hidden {D}, "
                        f"intermediate {FF}) sharded evenly over {world} GPU(s), {EP_B} sequences x 1 token, top-{EP_K}, "
                        "dispatch of bf16 rows and combine of f32 partial sums by the kernels themselves over NVLink peer memory "
                        "(--ep-collectives a2a: NCCL all-to-alls)",
            "tokens": EP_B, "experts": EP_E, "top_k": EP_K, "hidden": D, "intermediate": FF, "parallelism": f"ep{world}",
            "l2_policy": f"steps rotate over {layers} independent layers per rank ({layers * EP_E // world * 3 * BYTES_PER_MATRIX / 1e9:.2f} GB "
                         "of packed streams per GPU), larger than the 126 MB L2"}


def run_ep(args):
    """Config 3 at any N (N = 1: all experts on one GPU, the base of the strong-scaling series)."""
    import torch
    import torch.distributed as dist
    from nanoseedlm_b200 import ep, lib as L, moe

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = L.load()
    K, W = args.steps, max(args.warmup, 3)
    e_loc, t_loc = EP_E // world, EP_B // world
    NL = max(2, min(args.layers, int(6e9 // (e_loc * 3 * BYTES_PER_MATRIX))))
    mirror = bool(args.ep_mirror) and world % 2 == 0 and args.ep_collectives == "p2p"

    def experts_of(r):      # rank r's experts of every layer: the same bytes on whichever rank generates them
        g = torch.Generator(device="cuda").manual_seed(4321 + r)
        return [moe.DeviceLayer.random_on_device(D, FF, e_loc, g) for _ in range(NL)]

    layers = experts_of(rank)
    if mirror:              # this rank also holds its partner's experts (own first, then the partner's)
        layers = [moe.DeviceLayer.concat(a, b) for a, b in zip(layers, experts_of((rank + world // 2) % world))]
    be = ep.CudaBackend(layers[0])
    epl = ep.ExpertParallelMoe(be, D, EP_K, EP_E, t_loc, collectives=args.ep_collectives, mirror=mirror)
    NB = 8
    rng = np.random.default_rng(7 + rank)
    hx = rng.standard_normal((NB, t_loc, D)).astype(np.float32)
    hx = (hx.view(np.uint32) + 0x7FFF + ((hx.view(np.uint32) >> 16) & 1) & 0xFFFF0000).view(np.float32)
    hl = rng.standard_normal((NB, t_loc, EP_E)).astype(np.float32)
    dx, dl = torch.from_numpy(hx).cuda(), torch.from_numpy(hl).cuda()
    px, pl = torch.from_numpy(hx).pin_memory(), torch.from_numpy(hl).pin_memory()
    pout = torch.zeros(t_loc, D).pin_memory()
    sx, sl = torch.zeros(t_loc, D, device="cuda"), torch.zeros(t_loc, EP_E, device="cuda")
    stream = torch.cuda.Stream()
    torch.cuda.synchronize()

    def one(i):
        be.set_layer(layers[i % NL])
        epl.step(dx[i % NB], dl[i % NB])

    with torch.cuda.stream(stream):
        for i in range(W):
            one(i)
        stream.synchronize()
        # one step = 6 kernels of this library with the peer-memory exchange (9 kernels + 2 collective calls otherwise); with
        # --no-graph every launch is issued directly, else the kernels replay as CUDA graphs (see ep.GraphedSteps)
        launches0 = lib.nsl_launch_count()
        one(W)
        stream.synchronize()
        launches = (lib.nsl_launch_count() - launches0) * K
        captured = not args.no_graph
        if captured:
            gs = ep.GraphedSteps(epl, layers, [(dx[b], dl[b]) for b in range(NB)])
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
        if p2p_status:
            raise SystemExit(f"expert-parallel p2p exchange: a wait ran out (status {p2p_status}); the timing is void")
    ms_per_step = ms / K
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        line = {"metric": "seed_decode_moe_gemv_tokens_per_s", "value": EP_B / (ms_per_step * 1e-3), "unit": "tok/s",
                "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": ep_config(world, NL),
                "gpu_launches": int(launches), "cuda_graph": captured, "collectives": args.ep_collectives, "mirrored_ranks": mirror,
                "clocks": clocks.summary(),
                "e2e": {"value": EP_B / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": t_loc * D * 4 + t_loc * EP_E * 4,
                        "d2h_bytes_per_step": t_loc * D * 4, "ms_per_step": e2e_s * 1e3},
                "roofline": None}
        # the whole step against the packed-bytes roofline: the experts a step touches, in expectation over the routing
        # (E (1 - (1 - k/E)^B) distinct experts of 3 matrices each), read once by whichever rank owns them
        distinct = EP_E * (1.0 - (1.0 - EP_K / EP_E) ** EP_B)
        step_bytes = distinct * 3 * BYTES_PER_MATRIX
        gbs = step_bytes / (ms_per_step * 1e-3) / 1e9
        line["roofline"] = {"bound": "hbm", "kernel": "the step's seed mat-vecs (mv_shx_kernel: gate+up and down over the ranks' pairs)",
                            "achieved": gbs, "peak": peaks["hbm_gbs"] * world, "unit": "GB/s", "frac": gbs / (peaks["hbm_gbs"] * world),
                            "peak_kind": peak_kind, "traffic": None, "expected_distinct_experts": distinct,
                            "note": "whole step (mat-vecs + exchange) over the aggregate HBM peak of the ranks; the kernels are bound by "
                                    "the logic pipe, see the 1-GPU config-1 line for the per-kernel roofline"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


LM_V, LM_D = 151936, 2048   # the LM head of the reference's Qwen-class model (affine int4, groups of 64)


def run_lmhead(args):
    """Not the headline: the dense affine-int4 LM head (kc_mv with MF_Q4) + greedy arg-max, an HBM-bound kernel."""
    import torch
    from nanoseedlm_b200 import lib as L
    lib = L.load()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    T, K, W, NM = min(args.tokens, 8), args.steps, max(args.warmup, 3), 4
    lib.nsl_q4_set_variant(int(os.environ.get("NSL_Q4_VARIANT", "1")))
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

    with torch.cuda.stream(stream):
        for i in range(W):
            step(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(torch.cuda.current_device()) as clocks:
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
    peaks, kind = measured_peaks()
    nbytes = LM_V * LM_D // 2 + 2 * LM_V * (LM_D // 64) * 2 + T * LM_D * 4 + T * LM_V * 4
    gbs = nbytes / (mv_us * 1e-6) / 1e9
    print(json.dumps({"metric": "lm_head_q4_tokens_per_s", "value": T / (ms * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": K, "warmup": W,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 x int4 -> f32",
                      "data": "synthetic", "gpu_launches": 2 * K, "clocks": clocks.summary(),
                      "config": {"workload": f"dense affine-int4 LM head {LM_V} x {LM_D} (groups of 64) + greedy arg-max, {T} tokens; "
                                             f"{NM} heads rotated (0.7 GB) so that every step reads HBM", "tokens": T},
                      "roofline": {"bound": "hbm", "kernel": "q4_mv_kernel (kc_mv, MF_Q4)", "achieved": gbs, "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "peak_kind": kind, "traffic": None,
                                   "us_per_launch": mv_us, "bytes_per_launch": nbytes}}))


ATTN_FORMS = {0: "attn_split_kernel", 1: "attn_flat_mma_kernel<2>", 2: "attn_split_mma_kernel<2>", 3: "attn_flat_mma_kernel<3>",
              4: "attn_flat_mma_kernel<2>, two blocks an SM", 5: "attn_flat_mma_kernel<2, bulk copies>",
              6: "attn_flat_mma_kernel<3, bulk copies>", 7: "attn_flat_mma_kernel<2, two warps a ring>"}


def run_attn(args):
    """Not the headline: decode attention of the reference's config 4 (GQA 16 query / 2 KV heads of 128, BF16 cache of 4096
    positions, 32 sequences = 134 MB of K and V per layer), an HBM-bound kernel."""
    import torch
    from nanoseedlm_b200 import lib as L
    lib = L.load()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    NH, NKV, CTX, NSEQ, NS, NL = 16, 2, 4096, 32, int(os.environ.get("NSL_ATTN_SPLITS", "32")), 3      # 32 splits: the reference host's choice for 32 rows of 4096 keys
    variant = int(os.environ.get("NSL_ATTN_VARIANT", "1"))
    lib.nsl_attn_set_variant(variant)
    K, W = args.steps, max(args.warmup, 3)
    gen = torch.Generator(device="cuda").manual_seed(5)
    q8 = os.environ.get("NSL_ATTN_KV", "bf16") == "q8"      # the 8-bit cache: int8 codes and one f32 scale per (row, KV head)
    if q8:
        caches = [(torch.randint(-127, 128, (NSEQ * CTX, NKV, 128), generator=gen, device="cuda", dtype=torch.int8),
                   torch.randint(-127, 128, (NSEQ * CTX, NKV, 128), generator=gen, device="cuda", dtype=torch.int8)) for _ in range(NL)]
        scales = [(torch.rand(NSEQ * CTX, NKV, generator=gen, device="cuda") / 64 + 0.01,
                   torch.rand(NSEQ * CTX, NKV, generator=gen, device="cuda") / 64 + 0.01) for _ in range(NL)]
    else:
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
    for i, (kc, vc) in enumerate(caches):
        kv = L.KvView()
        kv.a.k, kv.a.v, kv.nv, kv.fmt = kc.data_ptr(), vc.data_ptr(), NSEQ * CTX, 1 if q8 else 0
        if q8:
            kv.a.ks, kv.a.vs = scales[i][0].data_ptr(), scales[i][1].data_ptr()
        views.append(kv)
    stream = torch.cuda.Stream()
    s = C.c_void_p(stream.cuda_stream)

    def step(i):
        lib.kc_attn(s, a, q.data_ptr(), views[i % NL], rid.data_ptr(), part.data_ptr(), g.data_ptr(), o.data_ptr(), NSEQ)

    with torch.cuda.stream(stream):
        for i in range(W):
            step(i)
        stream.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(torch.cuda.current_device()) as clocks:
            e0.record(stream)
            for i in range(K):
                step(W + i)
            e1.record(stream)
            e1.synchronize()
        ms = e0.elapsed_time(e1) / K
    L.check()
    peaks, kind = measured_peaks()
    nbytes = 2 * NSEQ * CTX * NKV * ((128 + 4) if q8 else 128 * 2) + 3 * NSEQ * NH * 128 * 4
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "decode_attention_tokens_per_s", "value": NSEQ / (ms * 1e-3), "unit": "tok/s", "n_gpus": 1, "steps": K,
                      "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": ("int8" if q8 else "bf16") + " cache, f32 math",
                      "data": "synthetic", "gpu_launches": 2 * K, "clocks": clocks.summary(),
                      "config": {"workload": f"decode attention, {NH} query / {NKV} KV heads of 128, {'8-bit' if q8 else 'BF16'} cache of {CTX} positions x {NSEQ} "
                                             f"sequences ({nbytes / 1e6:.0f} MB per layer), {NS} splits; {NL} layers rotated", "tokens": NSEQ},
                      "roofline": {"bound": "hbm", "kernel": ATTN_FORMS.get(variant, ATTN_FORMS[1]) + " + attn_reduce_kernel (kc_attn)", "achieved": gbs,
                                   "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "peak_kind": kind, "traffic": None,
                                   "bytes_per_step": nbytes}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=None, help="config 1: 1..8 (default 8); config 2: prompt rows (default 512)")
    ap.add_argument("--layers", type=int, default=20)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-dependent-launch", action="store_true",
                    help="config 1: ordinary launches instead of programmatic dependent launches (for comparison)")
    ap.add_argument("--ep-collectives", default="p2p", choices=["p2p", "a2a", "gather"],
                    help="config 3: p2p (default): no collective call, the kernels store into the other ranks' memory over "
                         "NVLink and wait on counters; a2a: two NCCL all-to-alls; gather: all-gather + reduce-scatter")
    ap.add_argument("--ep-mirror", type=int, default=0,
                    help="config 3, p2p, even rank counts: 1 = ranks r and r + N/2 hold each other's experts too and split their "
                         "joint pairs in the middle (balance to within one pair; twice the expert bytes per GPU)")
    ap.add_argument("--workload", default=None, choices=["cfg1", "cfg2", "cfg3", "lmhead", "attn"],
                    help="cfg1: one GPU's MoE decode layer (default at 1 GPU); cfg2: the same layer on 512 prompt rows (grouped "
                         "tcgen05 GEMM); cfg3: expert-parallel decode (default at >1 GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
        workload = args.workload or ("cfg1" if world == 1 else "cfg3")
        args.tokens = args.tokens or (512 if workload == "cfg2" else 8)
        if int(os.environ.get("RANK", "0")) == 0:
            run_reference(args, workload)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload or ("cfg1" if world == 1 else "cfg3")
    if args.tokens is None:
        args.tokens = 512 if workload == "cfg2" else 8
    if workload == "cfg1" and not 1 <= args.tokens <= 8:
        raise SystemExit("config 1 is the decode / verify batch: --tokens 1..8 (use --workload cfg2 for prompt rows)")
    if workload == "attn":
        run_attn(args)
    elif workload == "lmhead":
        run_lmhead(args)
    elif workload == "cfg3":
        run_ep(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
