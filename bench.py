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
`--impl reference` times the reference's own CPU (torch) implementation of the
same layer on the host cores, on rank 0 only: the unmodified reference classes
when the reference tree is installed under baseline/_ref (or the environment
variable FLASHNN_REFERENCE names a checkout of it), else the restatement in
oracle/ (reported as kind "port").
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
E2E_ROW_BLOCKS = 4  # the end-to-end step walks the rows in this many blocks so that copies and kernels overlap
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


def find_reference():
    """Directory that holds the reference project's own `flashnn` package, or None."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("FLASHNN_REFERENCE", "")):
        if cand and os.path.exists(os.path.join(cand, "flashnn", "quant_gemm.py")):
            return cand
    return None


def load_reference_cpu():
    """The unmodified reference with its torch backend selected: (module, None), or (None, reason)."""
    path = find_reference()
    if path is None:
        return None, "no reference tree under baseline/_ref (nor named by FLASHNN_REFERENCE)"
    try:
        for name in [n for n in sys.modules if n == "flashnn" or n.startswith("flashnn.")]:
            del sys.modules[name]
        sys.path.insert(0, path)
        import flashnn  # the reference's package (this repository's alias of the same name sits later on the path)
        if not os.path.abspath(flashnn.__file__).startswith(os.path.abspath(path)):
            return None, f"`import flashnn` resolved to {flashnn.__file__}, not to the reference"
        flashnn.set_use_triton(False)
        return flashnn, None
    except Exception as e:  # missing dependency of the reference on this host, ...
        return None, f"importing the reference failed: {type(e).__name__}: {e}"


def reference_cpu_layer(rows):
    """(step function, kind, note): one pass of the FFN layer on the host CPU over the first `rows` tokens, through the
    reference's own DynamicQuantize / GemmA8W8 classes (kind "reference") or, without them, the oracle port."""
    from flashnn_b200 import workloads as W
    w = W.ffn_layer(rows, 0, 1, HIDDEN, INTER)
    ref, why = load_reference_cpu()
    if ref is not None:
        dq, gemm = ref.DynamicQuantize(), ref.GemmA8W8(torch.bfloat16)

        def step():
            qx, sx = dq(w["x"])
            gemm(qx, w["w_gu"], sx.float(), w["col_gu"])  # the torch path multiplies the two scales: one dtype for both
            qh, sh = dq(w["h"])
            gemm(qh, w["w_dn"], sh.float(), w["col_dn"])
        return step, "reference", "unmodified reference classes, set_use_triton(False), from " + os.path.relpath(find_reference(), ROOT)
    from oracle import quant_oracle as O

    def step():
        qx, sx = O.dynamic_quantize(w["x"], saturate=False)
        O.gemm_a8w8(qx, w["w_gu"], sx.float(), w["col_gu"], torch.bfloat16)
        qh, sh = O.dynamic_quantize(w["h"], saturate=False)
        O.gemm_a8w8(qh, w["w_dn"], sh.float(), w["col_dn"], torch.bfloat16)
    return step, "port", "oracle port (" + why + ")"


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

    def __init__(self, rank, world, device, tokens=TOKENS, share=None):
        """`share`: another FfnShard of the same rank whose device weights are reused (only the activations differ)."""
        import flashnn_b200
        from flashnn_b200 import workloads as W
        self.W = W
        w = W.ffn_layer(tokens, rank, world, HIDDEN, INTER, weights=share is None)
        self.host = w
        self.device = device
        self.x, self.h = w["x"].to(device), w["h"].to(device)
        if share is None:
            self.w_gu, self.w_dn = w["w_gu"].to(device), w["w_dn"].to(device)
            self.col_gu, self.col_dn = w["col_gu"].to(device), w["col_dn"].to(device)
        else:
            self.w_gu, self.w_dn, self.col_gu, self.col_dn = share.w_gu, share.w_dn, share.col_gu, share.col_dn
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


def cpu_baseline_sample(sample_rows, budget_s=25.0):
    """The reference's CPU path on the first `sample_rows` tokens of the same workload:
    returns (TOPS, seconds per pass, threads, kind, note)."""
    from flashnn_b200 import workloads as W
    torch.set_num_threads(os.cpu_count() or 1)
    step, kind, note = reference_cpu_layer(sample_rows)
    step()  # warm-up
    times = []
    t_all = time.perf_counter()
    while len(times) < 3 and (not times or (time.perf_counter() - t_all) + times[-1] < budget_s):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    best = min(times)
    ops = W.a8w8_ops(sample_rows, N_GU, HIDDEN) + W.a8w8_ops(sample_rows, N_DN, INTER)
    return ops / best / 1e12, best, torch.get_num_threads(), kind, note


def int8_yardstick(device, flush_buf, sustained_seconds=0.0):
    """The library int8 GEMM (torch._int_mm -> cuBLASLt) at 8192^3 on the same event harness: the measured int8
    tensor-core rate of this GPU.  Burst: L2 flushed, launches timed one by one, best of 10.  With
    `sustained_seconds` > 0 also back to back for about that long (the GPU settles under its power cap, so this is run
    after every other measurement).  Returns a dict, or one with "error" if the library declines."""
    try:
        n = 8192
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=device)
        bt = b.t()  # [K, N] view with K contiguous: the layout the weights of this path have
        ts = time_steps(lambda: torch._int_mm(a, bt), 10, 3, flush_buf)
        out = dict(burst_tops=round(2.0 * n ** 3 / (min(ts) * 1e-3) / 1e12, 1), shape="8192^3",
                   how="torch._int_mm (cuBLASLt int8), CUDA events; burst = best of 10 launches with L2 flushed")
        if sustained_seconds > 0:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(20, int(sustained_seconds / (statistics.median(ts) * 1e-3)))
            e0.record()
            for _ in range(reps):
                torch._int_mm(a, bt)
            e1.record()
            torch.cuda.synchronize()
            out["sustained_tops"] = round(2.0 * n ** 3 * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12, 1)
            out["how"] += f"; sustained = {reps} launches back to back"
        return out
    except Exception as e:
        return dict(error=f"{type(e).__name__}: {e}")


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
    # Each rank uploads only its 1/G of the rows of x and h (pinned host memory -> device); with G > 1 the ranks then
    # all-gather the rows over NVLink (NCCL) inside the timed region, so the host link carries every activation byte
    # once per node instead of once per rank.  The outputs of this rank's columns go back to pinned host memory.
    rows_per = TOKENS // world
    r0 = rank * rows_per
    hx = shard.host["x"][r0:r0 + rows_per].contiguous().pin_memory()
    hh = shard.host["h"][r0:r0 + rows_per].contiguous().pin_memory()
    out_gu = torch.empty(TOKENS, shard.n_gu, dtype=torch.bfloat16).pin_memory()
    out_dn = torch.empty(TOKENS, shard.n_dn, dtype=torch.bfloat16).pin_memory()

    # Two side streams and row blocks.  The host link is what bounds this step (839 MB cross it, against 1.8 ms of
    # kernels), so the step is issued the way a caller who cares would issue it: rows are independent, so each
    # projection runs on blocks of E2E_ROW_BLOCKS-th of the rows, a block's output goes down while the next block
    # computes (PCIe is full duplex: uploads ride on s_in, downloads on s_out), and with one GPU a block's rows
    # go up while the block before computes.  Everything is joined back into the launching stream before the step
    # ends, so the CUDA events on that stream bracket all of it.
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    blocks = E2E_ROW_BLOCKS
    rb = TOKENS // blocks

    def gather_rows(part, k):
        full = torch.empty(TOKENS, k, dtype=torch.bfloat16, device=device)
        dist.all_gather_into_tensor(full, part)  # enqueued on the current stream
        return full

    def upload(host_rows, k):
        """-> list of (rows on the device, event or None) per row block, issued on s_in."""
        out = []
        with torch.cuda.stream(s_in):
            if world == 1:
                for c in range(blocks):
                    t = host_rows[c * rb:(c + 1) * rb].to(device, non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(s_in)
                    out.append((t, ev))
            else:
                t = host_rows.to(device, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                out.append((t, ev))
        return out

    def project(ups, k, w, col, host_out, keep):
        main = torch.cuda.current_stream(device)
        if world > 1:  # this rank's rows are up: gather everybody's over NVLink, then walk the row blocks
            part, ev = ups[0]
            main.wait_event(ev)
            full = gather_rows(part, k)
            part.record_stream(main)
            rows = [full[c * rb:(c + 1) * rb] for c in range(blocks)]
        for c in range(blocks):
            if world == 1:
                x_c, ev = ups[c]
                main.wait_event(ev)
                x_c.record_stream(main)
            else:
                x_c = rows[c]
            q, sc = shard.dq(x_c)
            y = shard.gemm(q, w, sc, col)
            s_out.wait_stream(main)
            with torch.cuda.stream(s_out):
                host_out[c * rb:(c + 1) * rb].copy_(y, non_blocking=True)
            y.record_stream(s_out)
            keep.append(y)

    def e2e_step():
        main = torch.cuda.current_stream(device)
        s_in.wait_stream(main)  # the uploads start inside the timed region
        ups_x = upload(hx, HIDDEN)
        ups_h = upload(hh, INTER)
        keep = []
        project(ups_x, HIDDEN, shard.w_gu, shard.col_gu, out_gu, keep)
        project(ups_h, INTER, shard.w_dn, shard.col_dn, out_dn, keep)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    e2e_times = time_steps(e2e_step, e2e_steps, 2, flush_buf)
    barrier()
    e2e_ms = torch.tensor([sum(e2e_times)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_ms.item()) / e2e_steps
    # whole-job bytes over the host link per step
    h2d = world * (hx.numel() * 2 + hh.numel() * 2)
    d2h = world * (out_gu.numel() * 2 + out_dn.numel() * 2)

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

    # ---- the other half of the metric, at this N: decode-shaped work on this rank's column shard (all ranks) ----
    sharded = sharded_decode_extras(rank, world, device, flush_buf, peaks, barrier, shard)

    line = None
    if rank == 0:
        # ---- per-kernel figures (rank 0's shard), each timed alone with CUDA events ----
        qx, sx = shard.dq(shard.x)
        gu_ms = statistics.median(time_steps(lambda: shard.gemm(qx, shard.w_gu, sx, shard.col_gu), 10, 3, flush_buf))
        yard = int8_yardstick(device, flush_buf)
        gu_ops = W.a8w8_ops(TOKENS, shard.n_gu, HIDDEN)
        achieved = gu_ops / (gu_ms * 1e-3) / 1e12
        # a launch timed alone is held against a burst figure: the measured int8 library GEMM when it ran, else twice
        # the measured bf16 burst rate (int8 dense runs at twice the bf16 rate)
        if "burst_tops" in yard:
            int8_peak, peak_source = yard["burst_tops"], "measured in this run: torch._int_mm (cuBLASLt int8) 8192^3, best launch with L2 flushed"
        else:
            int8_peak, peak_source = 2.0 * peaks["bf16"], f"2 x {peaks['source']} burst bf16 cuBLAS rate (the int8 library GEMM did not run: {yard.get('error')})"
        # DRAM bytes of one gate/up launch on one GPU from profiles/a8w8_gate_up_4096x57344x8192.md (one ncu capture:
        # 619.2 MB read + 452.5 MB written); with G ranks the weight and output parts shrink by G, the activations do not
        a_bytes = TOKENS * HIDDEN
        traffic = int(a_bytes + (1071694336 - a_bytes) / world)
        roofline = dict(bound="tensor", kernel="a8w8_umma_pair_kernel (gate/up projection of this rank)",
                        achieved=round(achieved, 1), peak=round(int8_peak, 1), unit="TFLOP/s",
                        frac=round(achieved / int8_peak, 4), traffic=traffic,
                        traffic_note="ncu capture at one GPU" + ("" if world == 1 else f", scaled to 1/{world} of the columns"),
                        peak_source=peak_source + "; ops are int8 multiply-adds counted as 2",
                        frac_of_2x_measured_bf16_burst=round(achieved / (2.0 * peaks["bf16"]), 4),
                        nominal_frac=round(achieved / 4500.0, 4), launch_ms=round(gu_ms, 4))
        extra = dict(kernel_ms=dict(a8w8_gate_up=round(gu_ms, 4)), int8_yardstick=yard)
        dq_ms = statistics.median(time_steps(lambda: shard.dq(shard.x), 10, 3, flush_buf))
        dqh_ms = statistics.median(time_steps(lambda: shard.dq(shard.h), 10, 3, flush_buf))
        extra["kernel_ms"]["dynamic_quant_4096x8192"] = round(dq_ms, 4)
        extra["kernel_ms"]["dynamic_quant_4096x28672"] = round(dqh_ms, 4)
        extra["dynamic_quant_gbs"] = round(W.dynamic_quant_bytes(TOKENS, HIDDEN) / (dq_ms * 1e-3) / 1e9, 1)
        extra["dynamic_quant_28672_gbs"] = round(W.dynamic_quant_bytes(TOKENS, INTER) / (dqh_ms * 1e-3) / 1e9, 1)
        qh, sh = shard.dq(shard.h)
        dn_ms = statistics.median(time_steps(lambda: shard.gemm(qh, shard.w_dn, sh, shard.col_dn), 10, 3, flush_buf))
        extra["kernel_ms"]["a8w8_down"] = round(dn_ms, 4)
        extra["a8w8_down_tops"] = round(W.a8w8_ops(TOKENS, shard.n_dn, INTER) / (dn_ms * 1e-3) / 1e12, 1)
        extra["sharded_decode"] = sharded
        if world == 1:
            extra.update(extra_shapes(device, flush_buf, peaks))
            if not args.no_triton_reference:
                extra["reference_triton"] = reference_triton_figures()
            # last of all: a second of back-to-back library GEMMs leaves the GPU at its power-capped clocks
            sus = int8_yardstick(device, flush_buf, sustained_seconds=1.0)
            if "sustained_tops" in sus:
                yard["sustained_tops"] = sus["sustained_tops"]
                yard["how"] = sus["how"]
        # ---- CPU baseline: the reference's torch path on the host cores ----
        cpu = None
        if world == 1:
            tops, secs, threads, kind, note = cpu_baseline_sample(args.cpu_rows)
            cpu = dict(value=round(tops, 4), unit="TOPS", cores=threads, kind=kind,
                       sample=(f"first {args.cpu_rows} of {TOKENS} tokens" if args.cpu_rows < TOKENS else f"all {TOKENS} tokens")
                              + f", full layer, best of <=3 passes, {secs:.2f} s per pass; {note}")
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
                    "row_blocks": E2E_ROW_BLOCKS,
                    "note": "every step: each rank copies its 1/G of the rows of x and h up from pinned host memory" +
                            ("" if world == 1 else ", the ranks all-gather them over NVLink (NCCL, inside the timed region)") +
                            ", and copies its output columns back; the two projections run on row blocks (DynamicQuantize + "
                            "GemmA8W8 per block, through the module classes), so a block's output goes down while the next "
                            "computes (copies on side streams, joined into the timed stream before the step ends); byte "
                            "counts are whole-job; weights stay resident"},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
            "allgather_ms": allgather_ms, "wall_s": round(wall, 3), "extra": extra,
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line), flush=True)


def sharded_decode_extras(rank, world, device, flush_buf, peaks, barrier, layer):
    """The decode-shaped half of the metric on this rank's column shard, at this number of GPUs: the A16W4 GEMV
    (N = 28672 / G columns, K = 8192, group 128) at M = 1, 4, 16 and the A8W8 FFN layer at M = 1 and 64.  Every rank
    runs its shard; times are the max over ranks, rates are whole-job (all ranks' bytes / that time)."""
    import torch.distributed as dist
    import flashnn_b200
    from flashnn_b200 import workloads as W

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    n_full, k, group = 28672, 8192, 128
    n_shard = n_full // world
    wo = flashnn_b200.GemmWeightOnly(torch.bfloat16)
    w = W.a16w4_decode(16, n_full, k, group)
    qw = w["qw"][rank * n_shard // 2:(rank + 1) * n_shard // 2].contiguous()
    sc = w["scale"][:, rank * n_shard:(rank + 1) * n_shard].contiguous()
    copies = max(4, min(32, -(-(300 << 20) // max(1, qw.numel()))))  # rotating weight copies that together exceed L2
    qws = [qw.to(device) for _ in range(copies)]
    scs = [sc.to(device) for _ in range(copies)]
    for m_ in (1, 4, 16):
        x = w["x"][:m_].contiguous().to(device)
        calls = [(lambda q=q, s_=s_: wo(x, q, s_)) for q, s_ in zip(qws, scs)]
        barrier()
        ms = max_over_ranks(time_rotating_graph(calls, rounds=max(2, 40 // copies)))
        gbs = world * W.a16w4_bytes(m_, n_shard, k, group) / ms / 1e6
        out[f"a16w4_gemv_m{m_}"] = dict(ms=round(ms, 4), gbs_whole_job=round(gbs, 1), gbs_per_gpu=round(gbs / world, 1),
                                        frac_of_measured_hbm=round(gbs / world / peaks["hbm"], 4), columns_per_rank=n_shard)
    del qws, scs
    out["a16w4_gemv_timing"] = (f"{copies} rotating weight copies per rank (> L2 together), calls captured in one CUDA graph "
                                "and replayed, best of 5, max over ranks")
    # decode-shaped A8W8 FFN layer on this rank's shard: DynamicQuant + gate/up, DynamicQuant + down.  A decode loop
    # replays a CUDA graph, so the steps are captured (over rotating copies of the weights that together exceed L2)
    # and replayed; the eager figure (four launches per step issued from Python) is host-bound and reported beside it.
    per_rank_bytes = layer.w_gu.numel() + layer.w_dn.numel()
    ncopy = max(2, min(8, -(-(300 << 20) // per_rank_bytes)))
    weights = [(layer.w_gu, layer.w_dn)] + [(layer.w_gu.clone(), layer.w_dn.clone()) for _ in range(ncopy - 1)]
    for m_ in (1, 64):
        shard = FfnShard(rank, world, device, tokens=m_, share=layer)

        def step_with(wg, wd):
            qx, sx = shard.dq(shard.x)
            shard.gemm(qx, wg, sx, shard.col_gu)
            qh, sh = shard.dq(shard.h)
            shard.gemm(qh, wd, sh, shard.col_dn)

        calls = [(lambda wg=wg, wd=wd: step_with(wg, wd)) for wg, wd in weights]
        barrier()
        ms = max_over_ranks(time_rotating_graph(calls, rounds=max(2, 16 // ncopy)))
        barrier()
        eager = max_over_ranks(statistics.median(time_steps(shard.step, 10, 3, flush_buf)))
        byts = world * (W.a8w8_bytes(m_, shard.n_gu, HIDDEN) + W.a8w8_bytes(m_, shard.n_dn, INTER)
                        + W.dynamic_quant_bytes(m_, HIDDEN) + W.dynamic_quant_bytes(m_, INTER))
        out[f"a8w8_ffn_m{m_}"] = dict(ms=round(ms, 4), gbs_whole_job=round(byts / ms / 1e6, 1),
                                      frac_of_measured_hbm=round(byts / ms / 1e6 / world / peaks["hbm"], 4),
                                      eager_python_calls_ms=round(eager, 4),
                                      note=f"steps of four launches over {ncopy} rotating weight copies captured in one CUDA graph "
                                           "and replayed, best of 5, max over ranks; eager = the same step issued from Python "
                                           "with L2 flushed before it")
        del shard
    del weights
    return out


def reference_triton_figures(timeout_s=900):
    """The reference's own Triton kernels on this GPU (secondary baseline), timed by `bench.py --case ref_triton` in a
    child process so that a JIT failure or a crash of that code cannot take the benchmark down."""
    if find_reference() is None:
        return dict(unavailable="no reference tree under baseline/_ref (nor named by FLASHNN_REFERENCE)")
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--case", "ref_triton"], capture_output=True, text=True,
                           timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return dict(unavailable=f"the reference's Triton kernels did not finish within {timeout_s} s")
    for ln in reversed(r.stdout.strip().splitlines()):
        if ln.startswith("{"):
            return json.loads(ln)
    return dict(unavailable="no result line", rc=r.returncode, stderr_tail=r.stderr[-600:])


def run_ref_triton(args):
    """Times the unmodified reference's Triton path (set_use_triton(True)) with the same CUDA-event harness:
    GemmA8W8 at 8192^3 and at the prefill chain's 4096 x 11008 x 4096, DynamicQuantize at 4096 x 4096 and
    4096 x 8192, GemmWeightOnly A16W4 (group 128) at M = 1, N = 28672, K = 8192.  Each case reports its time or
    the exception text."""
    from flashnn_b200 import workloads as W
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    path = find_reference()
    for name in [n for n in sys.modules if n == "flashnn" or n.startswith("flashnn.")]:
        del sys.modules[name]
    sys.path.insert(0, path)
    out = {"source": os.path.relpath(path, ROOT)}
    try:
        import flashnn
        import triton
        flashnn.set_use_triton(True)
        out["triton_version"] = triton.__version__
    except Exception as e:
        print(json.dumps({"unavailable": f"import failed: {type(e).__name__}: {e}"}), flush=True)
        return
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def timed(label, make):
        try:
            fn, work, unit = make()
            ts = time_steps(fn, 10, 3, flush_buf)
            ms = statistics.median(ts)
            out[label] = dict(ms=round(ms, 4), rate=round(work / (ms * 1e-3), 1), unit=unit)
        except Exception as e:
            out[label] = dict(error=f"{type(e).__name__}: {str(e)[:300]}")
        torch.cuda.synchronize()

    def a8w8(m, n, k):
        def make():
            a, b = W.rand_int8((m, k), 0).to(device), W.rand_int8((n, k), 1).to(device)
            row = W.rand_uniform((m,), 2, 0.005, 0.02, torch.bfloat16).to(device)  # the Triton launcher wants scale dtype == out dtype
            col = W.rand_uniform((n,), 3, 0.001, 0.01, torch.bfloat16).to(device)
            op = flashnn.GemmA8W8(torch.bfloat16)
            return (lambda: op(a, b, row, col)), W.a8w8_ops(m, n, k) / 1e12, "TOPS"
        return make

    def dq(m, k):
        def make():
            x = W.rand_normal((m, k), 0, torch.bfloat16, outliers=True).to(device)
            op = flashnn.DynamicQuantize()
            return (lambda: op(x)), W.dynamic_quant_bytes(m, k) / 1e9, "GB/s"
        return make

    def a16w4(m):
        def make():
            w = W.a16w4_decode(m)
            x, qw, sc = w["x"].to(device), w["qw"].to(device), w["scale"].to(device)
            op = flashnn.GemmWeightOnly(torch.bfloat16)
            return (lambda: op(x, qw, sc)), W.a16w4_bytes(m, 28672, 8192, 128) / 1e9, "GB/s"
        return make

    timed("gemm_a8w8_8192x8192x8192", a8w8(8192, 8192, 8192))
    timed("gemm_a8w8_4096x11008x4096", a8w8(4096, 11008, 4096))
    timed("dynamic_quant_4096x4096", dq(4096, 4096))
    timed("dynamic_quant_4096x8192", dq(4096, 8192))
    timed("gemm_a16w4_m1_28672x8192", a16w4(1))
    timed("gemm_a16w4_m16_28672x8192", a16w4(16))
    out["timing"] = "CUDA events per call, L2 flushed before each, median of 10 after 3 warm-up calls (JIT compile excluded)"
    print(json.dumps(out), flush=True)


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
    torch.set_num_threads(os.cpu_count() or 1)  # torchrun pins OMP_NUM_THREADS to 1; this arm runs on rank 0 alone
    rows = min(args.cpu_rows, TOKENS)
    step, kind, note = reference_cpu_layer(rows)
    t0 = time.perf_counter()
    step()  # first warm-up step, also the probe for the size of the sample
    probe = time.perf_counter() - t0
    # bounded: the whole run (warm-up + timed steps) should end within about four minutes
    while rows > 64 and probe * (args.steps + args.warmup) > 240.0:
        rows //= 2
        step, kind, note = reference_cpu_layer(rows)
        t0 = time.perf_counter()
        step()
        probe = time.perf_counter() - t0
    for _ in range(max(0, args.warmup - 1)):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    ops = W.a8w8_ops(rows, N_GU, HIDDEN) + W.a8w8_ops(rows, N_DN, INTER)
    value = ops / dt / 1e12
    threads = torch.get_num_threads()
    sample = (f"each step = all {TOKENS} tokens" if rows == TOKENS else f"each step = first {rows} of {TOKENS} tokens") + \
        f" through the full layer on the host CPU; {note}"
    print(json.dumps({
        "metric": "a8w8_ffn_layer_tops", "value": round(value, 4), "unit": "TOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "int8 operands multiplied in fp32 (the reference's torch path)", "data": "synthetic",
        "impl": "reference",
        "config": {"workload": WORKLOAD, "tokens": TOKENS, "sample": sample},
        "cpu_baseline": {"value": round(value, 4), "unit": "TOPS", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def run_sweep(args):
    """The reference's own benchmark sweeps on one GPU: GemmA8W8 over M x 20 (N, K) pairs
    (benchmark/benchmark_gemm_a8w8.py:13-44, fp16 scales and output as there) and DynamicQuantize over M x 6 row
    lengths (benchmark/benchmark_dynamic_quant.py:11).  Prints two markdown tables (TOPS; GB/s) and one JSON line."""
    import flashnn_b200
    from flashnn_b200 import _lib
    from flashnn_b200 import workloads as W
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    nk, ms_list = W.reference_sweep_shapes()
    gemm = flashnn_b200.GemmA8W8(torch.float16)
    g = torch.Generator(device=device).manual_seed(0)
    rows = []
    print("### GemmA8W8, TOPS (2 M N K / time), fp16 scales and output, CUDA events, L2 flushed, median of 5\n")
    print("| N | K | " + " | ".join(f"M={m}" for m in ms_list) + " |")
    print("|---|---|" + "---|" * len(ms_list))
    for n, k in nk:
        b = torch.randint(-128, 127, (n, k), dtype=torch.int8, device=device, generator=g)
        col = torch.rand(1, n, device=device, generator=g).half()
        cells = []
        for m in ms_list:
            a = torch.randint(-128, 127, (m, k), dtype=torch.int8, device=device, generator=g)
            row = torch.rand(m, 1, device=device, generator=g).half()
            ms = statistics.median(time_steps(lambda: gemm(a, b, row, col), 5, 2, flush_buf))
            tops = W.a8w8_ops(m, n, k) / ms / 1e9
            rows.append(dict(op="a8w8", m=m, n=n, k=k, ms=round(ms, 5), tops=round(tops, 1),
                             gbs=round(W.a8w8_bytes(m, n, k) / ms / 1e6, 1)))
            cells.append(f"{tops:.0f}" if m > 40 else f"{tops:.1f} ({W.a8w8_bytes(m, n, k) / ms / 1e6:.0f} GB/s)")
        print(f"| {n} | {k} | " + " | ".join(cells) + " |", flush=True)
        del b
    dq = flashnn_b200.DynamicQuantize()
    print("\n### DynamicQuantize, GB/s (3 M K + 2 M bytes / time), fp16 input\n")
    print("| K | " + " | ".join(f"M={m}" for m in ms_list) + " |")
    print("|---|" + "---|" * len(ms_list))
    for k in W.DYNAMIC_QUANT_SWEEP_K:
        cells = []
        for m in ms_list:
            x = torch.rand(m, k, device=device, generator=g).half()
            ms = statistics.median(time_steps(lambda: dq(x), 5, 2, flush_buf))
            gbs = W.dynamic_quant_bytes(m, k) / ms / 1e6
            rows.append(dict(op="dq", m=m, k=k, ms=round(ms, 5), gbs=round(gbs, 1)))
            cells.append(f"{gbs:.0f} ({ms * 1e3:.1f} us)")
        print(f"| {k} | " + " | ".join(cells) + " |", flush=True)
    assert _lib.device_status() == 0
    print()
    print(json.dumps({"case": "sweep", "points": rows}), flush=True)


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
        from flashnn_b200 import _lib
        if args.tile:
            _lib.set_option(_lib.OPT_A8W8_PAIR_TILE, args.tile)
        if args.balanced:
            _lib.set_option(_lib.OPT_A8W8_BALANCED, args.balanced)
        if args.epilogue_warps:
            _lib.set_option(_lib.OPT_A8W8_EPILOGUE_WARPS, args.epilogue_warps)
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
    elif name == "wog":
        # A16W4 prefill with group-wise scales (group 128): the decode config's weight at prefill batch sizes
        m, n, k = args.m or 2048, args.n or 28672, args.k or 8192
        w = W.a16w4_decode(1, n, k, group=args.group if args.group > 0 else 128)
        x = W.rand_normal((m, k), 0, torch.bfloat16).to(device)
        qw, sc = w["qw"].to(device), w["scale"].to(device)
        if args.group == -1:  # per-channel scales on the same weights
            sc = sc[0].contiguous()
        op = flashnn_b200.GemmWeightOnly(torch.bfloat16)
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
        from flashnn_b200.workloads import make_moe_case
        m, n, k = args.m or 64, args.n or 28672, args.k or 4096
        e, top_k, bm = 8, 2, args.bm or (16 if m <= 64 else 128)
        c = {kk: v.to(device) for kk, v in make_moe_case(m, e, n, k, top_k, bm, seed=0).items()}
        out = torch.empty(m, top_k, n, dtype=torch.bfloat16, device=device)
        fn = lambda: flashnn_b200.fused_moe_a8w8_forward(c["a"], c["b"], out, c["alpha_row"], c["alpha_col"], c["topk_w"],
                                                         c["topk_ids"], c["sorted_ids"], c["expert_ids"], c["npp"], True, top_k, bm)
        if m <= 256:
            work, unit = (e * n * k + m * top_k * n * 2 + m * k) / 1e9, "GB/s"
        else:
            work, unit = 2.0 * m * top_k * n * k / 1e12, "TOPS"
    elif name == "moe4":
        # the same expert layer with packed-int4 weights and per-group (128) bf16 scales
        from flashnn_b200.workloads import make_moe_w4_case
        m, n, k = args.m or 64, args.n or 28672, args.k or 4096
        e, top_k, bm = 8, 2, args.bm or (16 if m <= 64 else 64)
        c = {kk: (None if v is None else v.to(device)) for kk, v in
             make_moe_w4_case(m, e, n, k, top_k, bm, seed=0, dtype=torch.bfloat16, group=128).items() if kk != "w4"}
        out = torch.empty(m, top_k, n, dtype=torch.bfloat16, device=device)
        fn = lambda: flashnn_b200.fused_moe_a16w4_forward(c["a"], c["b"], out, c["scale"], None, c["topk_w"], c["topk_ids"],
                                                          c["sorted_ids"], c["expert_ids"], c["npp"], True, top_k, bm)
        if m <= 256:
            work, unit = (e * n * k // 2 + e * n * (k // 128) * 2 + m * top_k * n * 2 + m * k * 2) / 1e9, "GB/s"
        else:
            work, unit = 2.0 * m * top_k * n * k / 1e12, "TFLOP/s"
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
    ap.add_argument("--cpu-rows", type=int, default=TOKENS, help="tokens in the CPU-baseline sample (default: the whole workload)")
    ap.add_argument("--no-triton-reference", action="store_true", help="skip timing the reference's Triton kernels (extra.reference_triton)")
    ap.add_argument("--case", choices=["a8w8", "gemv", "gemv8", "dq", "wo", "wog", "rmsdq", "lndq", "moe", "moe4", "ref_triton", "sweep"],
                    help="run one kernel only (profiling / A-B timing), the reference's Triton kernels, or the reference's shape sweep")
    ap.add_argument("--tile", type=int, default=0, help="with --case a8w8: force this CTA-pair tile width (tuning)")
    ap.add_argument("--balanced", type=int, default=0, help="with --case a8w8: 1 forces, 2 forbids the K-balanced mode of the CTA-pair kernel")
    ap.add_argument("--epilogue-warps", type=int, default=0, help="with --case a8w8: 4 keeps four epilogue warps per CTA for every K")
    ap.add_argument("--bm", type=int, default=0, help="with --case moe / moe4: slots per block (default 16 up to 64 tokens, else 128 / 64)")
    ap.add_argument("--group", type=int, default=0, help="with --case wog: scale group size (-1: per channel)")
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    args = ap.parse_args()
    if args.case == "ref_triton":
        run_ref_triton(args)
    elif args.case == "sweep":
        run_sweep(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_native(args)


if __name__ == "__main__":
    main()
