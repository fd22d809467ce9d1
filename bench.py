#!/usr/bin/env python
"""Benchmark of the quantized-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]

One "step" is one pass of a Llama-2-70B-shaped A8W8 FFN layer over a batch of
M = 4096 tokens: DynamicQuant(x) -> A8W8 gate/up (K=8192 -> N=57344), then
DynamicQuant(h) -> A8W8 down (K=28672 -> N=8192), bf16 in and out, int8 weights
with per-channel fp32 scales.  With N GPUs the output columns of both
projections are sharded over the ranks (no collective on the data path), so the
total work is fixed and the whole-job rate is total ops / slowest rank's time.

Rank 0 prints one JSON line.  `value` is measured with the inputs resident in
HBM; `e2e` is the same step through the public Python API with pinned host
buffers copied in and the outputs copied back inside the timed region.
`--impl reference` times the CPU restatement of the reference's torch path
(oracle/) on a bounded sample of the same workload, on rank 0 only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN, INTER, TOKENS = 8192, 28672, 4096
N_GU, N_DN = 2 * INTER, HIDDEN
WORKLOAD = ("llama2-70b FFN, A8W8: DynamicQuant + gate/up 8192->57344, DynamicQuant + down 28672->8192, "
            "M=4096, bf16 activations/outputs, int8 weights")


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        busy = [c for c in sm if c > 500] or sm
        return dict(sm_mhz=statistics.median(busy) if busy else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


# ----------------------------------------------------------------------------------------------
# native arm
# ----------------------------------------------------------------------------------------------
class FfnShard:
    """This rank's column shard of the layer, resident on the device."""

    def __init__(self, rank, world, device, tokens=TOKENS):
        import flashnn_b200
        from flashnn_b200 import workloads as W
        self.W = W
        w = W.ffn_layer(tokens, rank, world, HIDDEN, INTER)
        self.host = w
        self.device = device
        self.x, self.h = w["x"].to(device), w["h"].to(device)
        self.w_gu, self.w_dn = w["w_gu"].to(device), w["w_dn"].to(device)
        self.col_gu, self.col_dn = w["col_gu"].to(device), w["col_dn"].to(device)
        self.dq = flashnn_b200.DynamicQuantize()
        self.gemm = flashnn_b200.GemmA8W8(torch.bfloat16)
        self.n_gu, self.n_dn = self.w_gu.shape[0], self.w_dn.shape[0]
        self.tokens = tokens

    def step(self, x=None, h=None):
        x = self.x if x is None else x
        h = self.h if h is None else h
        qx, sx = self.dq(x)
        y_gu = self.gemm(qx, self.w_gu, sx, self.col_gu)
        qh, sh = self.dq(h)
        y_dn = self.gemm(qh, self.w_dn, sh, self.col_dn)
        return y_gu, y_dn

    def ops(self):  # this rank's algorithmic integer ops per step
        return self.W.a8w8_ops(self.tokens, self.n_gu, HIDDEN) + self.W.a8w8_ops(self.tokens, self.n_dn, INTER)


def flush_l2(buf):
    buf.zero_()


def time_steps(fn, steps, warmup, flush_buf):
    """Per-step CUDA-event times (ms) on the current stream, L2 flushed before every step."""
    for _ in range(warmup):
        flush_l2(flush_buf)
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        flush_l2(flush_buf)
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def time_rotating(fns, rounds, warmup_rounds=2):
    """Average device time (ms) of one call when the calls in `fns` (same kernel, disjoint operand copies
    that together exceed L2) run back to back between one pair of CUDA events: no launch gap inside the
    timed region, every launch reads cold operands."""
    for _ in range(warmup_rounds):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(rounds):
        for fn in fns:
            fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (rounds * len(fns))


def time_rotating_graph(fns, rounds, replays=5):
    """As time_rotating, but the `rounds * len(fns)` calls are captured once into a CUDA graph and the graph is
    replayed: the way a decode loop is run in production, and free of the Python / ctypes cost per call (about as
    long as one of these kernels).  Returns the best replay's average device time (ms) per call."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for fn in fns:
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    # thread-local capture: other threads of this process (a collective library's watchdog) may keep calling CUDA
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        for _ in range(rounds):
            for fn in fns:
                fn()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) / (rounds * len(fns)))
    del graph
    return best


def cpu_baseline_sample(host, sample_rows, reps_budget_s=12.0):
    """The CPU restatement of the reference's torch path on the first `sample_rows` tokens of the
    same workload (`host` = the full layer's CPU tensors): returns (TOPS, seconds per pass, threads)."""
    from flashnn_b200 import workloads as W
    from oracle import quant_oracle as O
    w = dict(host)
    w["x"], w["h"] = host["x"][:sample_rows].contiguous(), host["h"][:sample_rows].contiguous()

    def one_pass():
        qx, sx = O.dynamic_quantize(w["x"], saturate=False)
        O.gemm_a8w8(qx, w["w_gu"], sx.float(), w["col_gu"], torch.bfloat16)
        qh, sh = O.dynamic_quantize(w["h"], saturate=False)
        O.gemm_a8w8(qh, w["w_dn"], sh.float(), w["col_dn"], torch.bfloat16)

    one_pass()  # warm-up
    times = []
    t_all = time.perf_counter()
    while len(times) < 5 and (time.perf_counter() - t_all) < reps_budget_s:
        t0 = time.perf_counter()
        one_pass()
        times.append(time.perf_counter() - t0)
    best = min(times)
    ops = W.a8w8_ops(sample_rows, N_GU, HIDDEN) + W.a8w8_ops(sample_rows, N_DN, INTER)
    return ops / best / 1e12, best, torch.get_num_threads()


def run_native(args):
    import torch.distributed as dist
    from flashnn_b200 import _lib
    from flashnn_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N with N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()
    shard = FfnShard(rank, world, device)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: K steps, inputs resident in HBM ----
    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(device).uuid))
    barrier()
    if rank == 0:
        sampler.start()  # sampled from the warm-up steps (same load) to the end of the timed steps
    wall0 = time.perf_counter()
    times = time_steps(shard.step, args.steps, args.warmup, flush_buf)
    barrier()
    wall = time.perf_counter() - wall0
    # the timed region lasts tens of milliseconds; keep the same step running (untimed) until nvidia-smi has
    # delivered a usable number of samples of the clocks under this load
    probe_t0 = time.perf_counter()
    while time.perf_counter() - probe_t0 < 0.6:
        for _ in range(10):
            shard.step()
        torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    if clocks is not None:
        clocks["sampled_over"] = "warm-up + timed steps + 0.6 s of the same step repeated"
    assert _lib.device_status() == 0
    total_ms = torch.tensor([sum(times)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(total_ms.item()) / args.steps
    total_ops = W.a8w8_ops(TOKENS, N_GU, HIDDEN) + W.a8w8_ops(TOKENS, N_DN, INTER)
    value = total_ops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers ----
    hx, hh = shard.host["x"].pin_memory(), shard.host["h"].pin_memory()
    out_gu = torch.empty(TOKENS, shard.n_gu, dtype=torch.bfloat16).pin_memory()
    out_dn = torch.empty(TOKENS, shard.n_dn, dtype=torch.bfloat16).pin_memory()

    # Two side streams: the second input goes up while the first projection computes, and each output goes
    # down as soon as its projection is done (PCIe is full duplex).  Everything is joined back into the
    # launching stream before the step ends, so the CUDA events on that stream bracket all of it.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def e2e_step():
        main = torch.cuda.current_stream(device)
        x = hx.to(device, non_blocking=True)  # first on the host-to-device engine: the first projection waits for it
        s_in.wait_stream(main)                 # (orders the second upload behind the timed region's start only)
        with torch.cuda.stream(s_in):
            h = hh.to(device, non_blocking=True)
        qx, sx = shard.dq(x)
        y_gu = shard.gemm(qx, shard.w_gu, sx, shard.col_gu)
        s_out.wait_stream(main)
        with torch.cuda.stream(s_out):
            out_gu.copy_(y_gu, non_blocking=True)
        main.wait_stream(s_in)
        qh, sh = shard.dq(h)
        y_dn = shard.gemm(qh, shard.w_dn, sh, shard.col_dn)
        s_out.wait_stream(main)
        with torch.cuda.stream(s_out):
            out_dn.copy_(y_dn, non_blocking=True)
        main.wait_stream(s_out)
        for t in (h, y_gu, y_dn):
            t.record_stream(s_out)
        h.record_stream(main)

    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    e2e_times = time_steps(e2e_step, e2e_steps, 2, flush_buf)
    barrier()
    e2e_ms = torch.tensor([sum(e2e_times)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_ms.item()) / e2e_steps
    h2d = hx.numel() * 2 + hh.numel() * 2
    d2h = out_gu.numel() * 2 + out_dn.numel() * 2

    # ---- optional all-gather of the sharded outputs, timed apart ----
    allgather_ms = None
    if world > 1:
        y_gu, y_dn = shard.step()
        full_gu = torch.empty(world, TOKENS, shard.n_gu, dtype=torch.bfloat16, device=device)
        full_dn = torch.empty(world, TOKENS, shard.n_dn, dtype=torch.bfloat16, device=device)

        def gather():
            dist.all_gather_into_tensor(full_gu, y_gu)
            dist.all_gather_into_tensor(full_dn, y_dn)

        barrier()
        ag = time_steps(gather, 5, 2, flush_buf)
        t = torch.tensor([statistics.median(ag)], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allgather_ms = float(t.item())
        del full_gu, full_dn

    line = None
    if rank == 0:
        # ---- per-kernel figures (rank 0's shard), each timed alone with CUDA events ----
        qx, sx = shard.dq(shard.x)
        gu_ms = statistics.median(time_steps(lambda: shard.gemm(qx, shard.w_gu, sx, shard.col_gu), 10, 3, flush_buf))
        gu_ops = W.a8w8_ops(TOKENS, shard.n_gu, HIDDEN)
        achieved = gu_ops / (gu_ms * 1e-3) / 1e12
        int8_peak = 2.0 * peaks["bf16_sustained"]
        # DRAM bytes of one gate/up launch on one GPU from profiles/a8w8_gate_up_4096x57344x8192.md (one ncu capture:
        # 619.2 MB read + 452.5 MB written); with G ranks the weight and output parts shrink by G, the activations do not
        a_bytes = TOKENS * HIDDEN
        traffic = int(a_bytes + (1071694336 - a_bytes) / world)
        roofline = dict(bound="tensor", kernel="a8w8_umma_pair_kernel (gate/up projection of this rank)",
                        achieved=round(achieved, 1), peak=round(int8_peak, 1), unit="TFLOP/s",
                        frac=round(achieved / int8_peak, 4), traffic=traffic,
                        traffic_note="ncu capture at one GPU" + ("" if world == 1 else f", scaled to 1/{world} of the columns"),
                        peak_source=f"2 x {peaks['source']} sustained bf16 cuBLAS rate (int8 dense runs at twice the bf16 rate; "
                                    "no int8 figure is in MEASURED_PEAKS.json); ops are int8 multiply-adds counted as 2",
                        nominal_frac=round(achieved / 4500.0, 4), launch_ms=round(gu_ms, 4))
        extra = dict(kernel_ms=dict(a8w8_gate_up=round(gu_ms, 4)))
        dq_ms = statistics.median(time_steps(lambda: shard.dq(shard.x), 10, 3, flush_buf))
        extra["kernel_ms"]["dynamic_quant_4096x8192"] = round(dq_ms, 4)
        extra["dynamic_quant_gbs"] = round(W.dynamic_quant_bytes(TOKENS, HIDDEN) / (dq_ms * 1e-3) / 1e9, 1)
        extra.update(extra_shapes(device, flush_buf, peaks))
        # ---- CPU baseline: the reference's torch path (restated in oracle/) on a bounded sample ----
        cpu = None
        if world == 1:
            tops, secs, threads = cpu_baseline_sample(shard.host, args.cpu_rows)
            cpu = dict(value=round(tops, 4), unit="TOPS", cores=threads, kind="port",
                       sample=f"first {args.cpu_rows} of {TOKENS} tokens, full layer, best of <=5 passes, {secs:.2f} s per pass")
        line = {
            "metric": "a8w8_ffn_layer_tops", "value": round(value, 2), "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 (int32 accumulate, bf16 out)",
            "data": "synthetic", "impl": "native",
            "config": {"workload": WORKLOAD, "tokens": TOKENS, "sharding": f"columns over {world} rank(s), no collective",
                       "l2": "flushed before every step (256 MiB write); weights per step also exceed L2 at N<=4",
                       "timing": "CUDA events per step on the launching stream, max over ranks"},
            "e2e": {"value": round(total_ops / (e2e_ms_per_step * 1e-3) / 1e12, 3), "unit": "TOPS",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms_per_step, 3),
                    "note": "pinned host x,h copied in, both outputs copied back, every step (copies on side streams, "
                            "joined into the timed stream before the step ends); weights stay resident"},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "allgather_ms": allgather_ms, "wall_s": round(wall, 3), "extra": extra,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def extra_shapes(device, flush_buf, peaks):
    """Figures for the other benchmark configurations (rank 0, one GPU)."""
    import flashnn_b200
    from flashnn_b200 import workloads as W
    out = {}
    # headline A8W8 shape
    m = n = k = 8192
    a = W.rand_int8((m, k), 0).to(device)
    b = W.rand_int8((n, k), 1).to(device)
    row = W.rand_uniform((m,), 2, 0.005, 0.02).to(device)
    col = W.rand_uniform((n,), 3, 0.001, 0.01).to(device)
    gemm = flashnn_b200.GemmA8W8(torch.bfloat16)
    ts = time_steps(lambda: gemm(a, b, row, col), 20, 5, flush_buf)
    ms = statistics.median(ts)
    out["a8w8_8192x8192x8192"] = dict(ms=round(ms, 4), best_ms=round(min(ts), 4), tops=round(W.a8w8_ops(m, n, k) / ms / 1e9, 1),
                                       frac_of_nominal_4500=round(W.a8w8_ops(m, n, k) / ms / 1e9 / 4500, 4),
                                       frac_of_2x_measured_bf16_burst=round(W.a8w8_ops(m, n, k) / ms / 1e9 / (2 * peaks["bf16"]), 4))
    del a, b
    # A8W8 small config (launch/latency bound)
    w = W.a8w8_small()
    a, b, row, col = (w[k_].to(device) for k_ in ("a", "b", "alpha_row", "alpha_col"))
    ms = statistics.median(time_steps(lambda: gemm(a, b, row, col), 20, 5, flush_buf))
    out["a8w8_16x4096x4096"] = dict(ms=round(ms, 4), gbs=round(W.a8w8_bytes(16, 4096, 4096) / ms / 1e6, 1))
    # DynamicQuant + A8W8 prefill chain
    w = W.dq_a8w8_prefill()
    x, wt, col = w["x"].to(device), w["w"].to(device), w["alpha_col"].to(device)
    dq = flashnn_b200.DynamicQuantize()
    ms_dq = statistics.median(time_steps(lambda: dq(x), 20, 5, flush_buf))
    q, s = dq(x)
    ms_g = statistics.median(time_steps(lambda: gemm(q, wt, s, col), 20, 5, flush_buf))
    out["dq_a8w8_4096x11008x4096"] = dict(dq_ms=round(ms_dq, 4), dq_gbs=round(W.dynamic_quant_bytes(4096, 4096) / ms_dq / 1e6, 1),
                                          gemm_ms=round(ms_g, 4), gemm_tops=round(W.a8w8_ops(4096, 11008, 4096) / ms_g / 1e9, 1))
    del x, wt
    # A16W4 decode GEMV: four weight copies (4 x 117 MB > L2) used in rotation, launches back to back
    wo = flashnn_b200.GemmWeightOnly(torch.bfloat16)
    for m_ in (1, 4, 16):
        w = W.a16w4_decode(m_)
        x, sc = w["x"].to(device), w["scale"].to(device)
        qws = [w["qw"].to(device) for _ in range(4)]
        scs = [sc.clone() for _ in range(4)]
        calls = [(lambda q=q, s_=s_: wo(x, q, s_)) for q, s_ in zip(qws, scs)]
        ms_eager = time_rotating(calls, rounds=10)
        ms = time_rotating_graph(calls, rounds=10)
        # the same with the caller's promise that weights are never written in-stream (FNN_OPT_STATIC_WEIGHTS): a
        # decode call may then start fetching weights while the call before it drains
        from flashnn_b200 import _lib as L
        L.set_option(L.OPT_STATIC_WEIGHTS, 1)
        try:
            ms_sw = time_rotating_graph(calls, rounds=10)
        finally:
            L.set_option(L.OPT_STATIC_WEIGHTS, 0)
        single = statistics.median(time_steps(lambda: wo(x, qws[0], scs[0]), 20, 5, flush_buf))
        gbs = W.a16w4_bytes(m_, 28672, 8192, 128) / ms / 1e6
        gbs_sw = W.a16w4_bytes(m_, 28672, 8192, 128) / ms_sw / 1e6
        out[f"a16w4_gemv_m{m_}"] = dict(ms=round(ms, 4), gbs=round(gbs, 1), frac_of_measured_hbm=round(gbs / peaks["hbm"], 4),
                                        timing="40 calls over 4 rotating weight copies captured in one CUDA graph, best of 5 replays",
                                        eager_python_calls_ms=round(ms_eager, 4),
                                        single_launch_ms_with_event_overhead=round(single, 4),
                                        static_weights_option=dict(ms=round(ms_sw, 4), gbs=round(gbs_sw, 1),
                                                                   frac_of_measured_hbm=round(gbs_sw / peaks["hbm"], 4)))
        del qws, scs
    return out


# ----------------------------------------------------------------------------------------------
# reference arm: the reference's CPU (torch) implementation of the same path, restated in oracle/
# ----------------------------------------------------------------------------------------------
def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from flashnn_b200 import workloads as W
    from oracle import quant_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)  # torchrun pins OMP_NUM_THREADS to 1; this arm runs on rank 0 alone
    rows = args.cpu_rows
    w = W.ffn_layer(rows, 0, 1, HIDDEN, INTER)

    def step():
        qx, sx = O.dynamic_quantize(w["x"], saturate=False)
        O.gemm_a8w8(qx, w["w_gu"], sx.float(), w["col_gu"], torch.bfloat16)
        qh, sh = O.dynamic_quantize(w["h"], saturate=False)
        O.gemm_a8w8(qh, w["w_dn"], sh.float(), w["col_dn"], torch.bfloat16)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    ops = W.a8w8_ops(rows, N_GU, HIDDEN) + W.a8w8_ops(rows, N_DN, INTER)
    value = ops / dt / 1e12
    threads = torch.get_num_threads()
    sample = f"each step = first {rows} of {TOKENS} tokens through the full layer on the host CPU"
    print(json.dumps({
        "metric": "a8w8_ffn_layer_tops", "value": round(value, 4), "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 operands multiplied in fp32 (the reference's torch path)", "data": "synthetic",
        "impl": "reference",
        "config": {"workload": WORKLOAD, "tokens": TOKENS, "sample": sample},
        "cpu_baseline": {"value": round(value, 4), "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def run_case(args):
    """One kernel of the path on one GPU, launched `steps` times after `warmup` (used for profiler
    captures and quick A/B timing).  Prints one small JSON line."""
    import flashnn_b200
    from flashnn_b200 import workloads as W
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    name = args.case
    if name == "a8w8":
        m, n, k = args.m or 8192, args.n or 8192, args.k or 8192
        a, b = W.rand_int8((m, k), 0).to(device), W.rand_int8((n, k), 1).to(device)
        row, col = W.rand_uniform((m,), 2, 0.005, 0.02).to(device), W.rand_uniform((n,), 3, 0.001, 0.01).to(device)
        op = flashnn_b200.GemmA8W8(torch.bfloat16)
        fn = lambda: op(a, b, row, col)
        work, unit = W.a8w8_ops(m, n, k) / 1e12, "TOPS"
    elif name == "gemv":
        m, n, k = args.m or 1, args.n or 28672, args.k or 8192
        w = W.a16w4_decode(m, n, k)
        x, qw, sc = w["x"].to(device), w["qw"].to(device), w["scale"].to(device)
        op = flashnn_b200.GemmWeightOnly(torch.bfloat16)
        fn = lambda: op(x, qw, sc)
        work, unit = W.a16w4_bytes(m, n, k, 128) / 1e9, "GB/s"
    elif name == "gemv8":
        m, n, k = args.m or 1, args.n or 28672, args.k or 8192
        g = torch.Generator().manual_seed(1)
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(device)
        qw = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).to(device)
        sc = (torch.rand(k // 128, n, generator=g) * 0.045 + 0.005).to(torch.bfloat16).to(device)
        op = flashnn_b200.GemmWeightOnly(torch.bfloat16)
        fn = lambda: op(x, qw, sc)
        work, unit = (n * k + 2 * (k // 128) * n + 2 * m * k + 2 * m * n) / 1e9, "GB/s"
    elif name == "wo":
        m, n, k = args.m or 2048, args.n or 8192, args.k or 8192
        w = W.a16w8_prefill(m, n, k)
        x, qw, sc = w["x"].to(device), w["w"].to(device), w["scale"].to(device)
        op = flashnn_b200.GemmWeightOnly(torch.float16)
        fn = lambda: op(x, qw, sc)
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"
    elif name == "dq":
        m, k = args.m or 4096, args.k or 8192
        x = W.rand_normal((m, k), 0, torch.bfloat16, outliers=True).to(device)
        op = flashnn_b200.DynamicQuantize()
        fn = lambda: op(x)
        work, unit = W.dynamic_quant_bytes(m, k) / 1e9, "GB/s"
    elif name == "moe":
        # Mixtral-8x7B-shaped expert layer (gate/up): E = 8, top-2, K = 4096 -> N = 28672, int8 weights
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from tests.moe_util import make_moe_case
        m, n, k = args.m or 64, args.n or 28672, args.k or 4096
        e, top_k, bm = 8, 2, (16 if m <= 64 else 128)
        c = {kk: v.to(device) for kk, v in make_moe_case(m, e, n, k, top_k, bm, seed=0).items()}
        out = torch.empty(m, top_k, n, dtype=torch.bfloat16, device=device)
        fn = lambda: flashnn_b200.fused_moe_a8w8_forward(c["a"], c["b"], out, c["alpha_row"], c["alpha_col"], c["topk_w"],
                                                         c["topk_ids"], c["sorted_ids"], c["expert_ids"], c["npp"], True, top_k, bm)
        if m <= 256:
            work, unit = (e * n * k + m * top_k * n * 2 + m * k) / 1e9, "GB/s"
        else:
            work, unit = 2.0 * m * top_k * n * k / 1e12, "TOPS"
    elif name in ("rmsdq", "lndq"):
        m, k = args.m or 4096, args.k or 8192
        x = W.rand_normal((m, k), 0, torch.bfloat16, outliers=True).to(device)
        op = (flashnn_b200.RMSNormDquant(k, 1e-5) if name == "rmsdq" else flashnn_b200.LayernormDquant(k, 1e-5))
        op = op.to(device=device, dtype=torch.bfloat16)
        fn = lambda: op(x)
        work, unit = W.dynamic_quant_bytes(m, k) / 1e9, "GB/s"
    else:
        raise SystemExit(f"unknown case {name}")
    ts = time_steps(fn, args.steps, args.warmup, flush_buf)
    ms = statistics.median(ts)
    print(json.dumps({"case": name, "m": m, "n": locals().get("n"), "k": k, "ms": round(ms, 5), "best_ms": round(min(ts), 5),
                      "rate": round(work / (ms * 1e-3), 1), "unit": unit}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["native", "reference"], default="native")
    ap.add_argument("--cpu-rows", type=int, default=256, help="tokens in the CPU-baseline sample")
    ap.add_argument("--case", choices=["a8w8", "gemv", "gemv8", "dq", "wo", "rmsdq", "lndq", "moe"], help="run one kernel only (profiling / A-B timing)")
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
