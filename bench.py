#!/usr/bin/env python
"""Benchmark of the block-quantised GEMV path on B200 (prints ONE JSON line on rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload q8_0_gemv] [--impl reference]

Workload ``q8_0_gemv`` (default) is the decode GEMV of the first benchmark configuration: W 4096 x 4096
(seed 0, N(0, 0.02), packed to Q8_0), x fp32[4096] (seed 1), batch 1.  One such matrix is 17.8 MB and
would sit in the 126 MB L2, so a pass sweeps COPIES distinct weight copies (same values, different
addresses, 570 MB in all): every launch streams its weights from HBM.  The 32 products of a pass are
submitted eight at a time, the reference's own batched form (zen::quant::gemv_batch, src/quant.cpp:1441-1502:
up to kMaxBatch = 8 matvecs sharing one input per submission; zen_cuda_dev_gemv / zen_cuda_gemv_q8_0_batch
here), on both arms.  A step is PASSES_PER_STEP passes, replayed from a CUDA graph (28 ms, so that a clock
sampler sees the timed region).  The line's ``detail`` object carries the same products launched one at a
time and as one list launch, and the other terms of the headline metric, each measured by the workload of
the same name in a short form: the prefill GEMM (``q8_0_gemm``), the lm_head (``lm_head``) and the greedy
decode (``decode``), the last two on all N GPUs.

  value      whole-job GB/s, algorithmic bytes (34 B per 32-weight block + x + y) / device time, inputs
             resident in HBM, CUDA events on the launching stream, max over ranks.
  e2e        the same metric through the host-pointer C-ABI call a ZenInfer build would make
             (zen_cuda_gemv_q8_0): x travels host->device and y device->host inside the timed region.
  roofline   achieved = algorithmic bytes per launch / mean launch time inside the timed region;
             peak = MEASURED_PEAKS.json hbm_gbs (a measured device-to-device copy rate).
  cpu_baseline  the reference's own CPU kernels (oracle/_ref, built from the reference sources) on
             the same workload, bounded sample, on this box's host cores.

With --gpus N (under torchrun) every rank owns one 4096-row shard of a (4096*N) x 4096 matrix per copy
(weak scaling); the path's one exchange step, the all-gather of the output shards, is fused into the
product kernel as peer stores (--gather nccl: an NCCL all-gather after each launch instead).

Other workloads (--workload): q8_0_gemm (config 1, the tcgen05 prefill product), layer_sweep (config 2, the
seven projections of a layer in Q8_0 / Q4_0 / Q6_K), lm_head (config 3, Q6_K 128256 x 4096, --gpus N shards the
rows), decode (config 4, greedy decode of the Llama-3-8B shape; --gpus N runs the sharded decoder, --cut chooses
its cut).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 4096, 4096
COPIES = 32
GROUP = 8                 # products per submission: zen::quant::gemv_batch, up to kMaxBatch = 8 tensors sharing one input
PASSES_PER_STEP = 300     # a step of the default workload: 300 passes over the 32 copies, about 28 ms
BLOCK_BYTES, BLOCK_ELEMS = 34, 32
ALGO_BYTES_PER_LAUNCH = ROWS * (COLS // BLOCK_ELEMS) * BLOCK_BYTES + COLS * 4 + ROWS * 4  # 17,858,560: one product launched alone
ALGO_BYTES_PER_GROUP = GROUP * (ROWS * (COLS // BLOCK_ELEMS) * BLOCK_BYTES + ROWS * 4) + COLS * 4  # 142,753,792: eight products sharing one read of x
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from ncu captures of `bench.py --profile`
# and `bench.py --workload q8_0_gemm --profile`: an eight-tensor decode launch reads 142,679,808 B and writes 3,889,920 B
# (142,753,792 B algorithmic); the prefill kernel (group-scale form, two weight digits = 117 MB of planes) reads
# 141,972,736 B and writes 21,978,112 B of DRAM (the per-block kernel: 81,239,808 + 13,685,504 B for 94,109,696 B algorithmic).
GEMV_NCU_TRAFFIC_BYTES = 146_569_728
GEMM_NCU_TRAFFIC_BYTES = 163_950_848
WORKLOAD = ("Q8_0 decode GEMV batch 1, W 4096x4096 (config 0), %d rotating weight copies, submitted %d products at a time "
            "(zen::quant::gemv_batch: tensors sharing one input)" % (COPIES, GROUP))


def peaks() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.rows, self.proc = index, [], None
        self.window = [None, None]  # host-clock bounds of the timed region

    def mark_start(self) -> None:
        self.window[0] = time.time()

    def mark_end(self) -> None:
        self.window[1] = time.time()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi needs a moment before its first line (seconds on a box with eight GPUs): wait for it here, before
            # any warm-up, so that short timed regions still fall between samples
            t0 = time.time()
            while not self.rows and self.proc.poll() is None and time.time() - t0 < 10.0:
                time.sleep(0.02)
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self) -> dict:
        lo, hi = self.window
        inside = [r for t, r in self.rows if lo is not None and hi is not None and lo <= t <= hi + 0.05]
        scope = "timed region"
        if not inside:  # a timed region shorter than one sampling period: use the samples taken under the same load around it
            inside, scope = [r for _, r in self.rows], "warm-up + timed region (timed region shorter than one sample period)"
        sm, mx, reasons = [], [], set()
        for r in inside:
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except Exception:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "scope": scope}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm), "scope": scope}


def config0() -> dict:
    """The `config` object of the default workload, the same for the GPU arm and the reference arm."""
    return {"workload": WORKLOAD, "rows_per_gpu": ROWS, "columns": COLS, "batch": 1, "activations": "int8 (bit-exact reference codes)",
            "generator": "numpy.random.default_rng(seed).standard_normal(float32): W seed 0 x 0.02 packed to Q8_0, x seed 1",
            "l2": "inputs larger than the last-level cache: rotating weight copies, every product streams its weights from memory"}


def make_inputs():
    from zeninfer_b200 import blocks
    w = np.random.default_rng(0).standard_normal((ROWS, COLS), dtype=np.float32) * np.float32(0.02)
    packed = np.ascontiguousarray(blocks.quantize_q8_0(w))
    x = np.random.default_rng(1).standard_normal(COLS, dtype=np.float32)
    return packed, x


def cpu_description() -> dict:
    """Model name and core counts of the host the CPU baseline runs on (every CPU figure is quoted with them)."""
    model = "unknown"
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.lower().startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    physical = None
    try:
        import psutil
        physical = psutil.cpu_count(logical=False)
    except Exception:
        pass
    return {"cpu_model": model, "logical_cpus": os.cpu_count(), "physical_cores": physical}


class CpuReference:
    """The reference's own CPU path (zen::quant::gemv through oracle/_ref) on the workload; the plain-C
    restatement stands in only where the compiled reference did not travel with the tree."""

    def __init__(self, packed: np.ndarray, x: np.ndarray, copies: int) -> None:
        os.environ.setdefault("ZEN_CPU_Q8_ACT", "1")  # same arithmetic as the GPU arm: int8 activations
        import oracle
        self.x, self.copies = x, copies
        self.kind = "reference" if oracle.reference_available() else "port"
        self.ws = [packed.copy() for _ in range(copies)]  # distinct addresses: the CPU caches do not hold them all
        self.groups = [self.ws[g:g + GROUP] for g in range(0, copies, GROUP)]
        outs = [np.empty(ROWS, np.float32) for _ in range(GROUP)]
        if self.kind == "reference":
            zr = oracle.Reference()
            self.cores = min(zr.pool_workers(), os.cpu_count() or 1)
            # one submission = GROUP products sharing x (zen::quant::gemv_batch); workers=0: the reference's own policy
            self.run = lambda ws: zr.gemv_batch(oracle.Q8_0, ws, x, [ROWS] * len(ws), COLS, workers=0, outs=outs)
            self.run_with = lambda ws, n: zr.gemv_batch(oracle.Q8_0, ws, x, [ROWS] * len(ws), COLS, workers=n, outs=outs)
        else:
            zo = oracle.Oracle()
            self.cores = 1
            self.run = lambda ws: [zo.gemv(oracle.Q8_0, w, x, ROWS, COLS, int8_acts=True) for w in ws]
            self.run_with = None
        self.run(self.groups[0])

    def sample(self, budget_s: float) -> dict:
        t0 = time.perf_counter()
        n = 0
        while True:
            self.run(self.groups[n % len(self.groups)])
            n += 1
            if time.perf_counter() - t0 > budget_s:
                break
        dt = time.perf_counter() - t0
        return {"value": ALGO_BYTES_PER_GROUP * n / dt / 1e9, "unit": "GB/s", "cores": self.cores, "kind": self.kind,
                "sample": f"{n} gemv_batch submissions of {GROUP} products over {self.copies} weight copies in {dt:.2f} s, int8 activations (ZEN_CPU_Q8_ACT=1), reference worker policy",
                "workers": "0 (the reference's planner default; its pool is capped at 32 threads)", **cpu_description()}

    def worker_sweep(self, budget_each_s: float) -> dict:
        """GB/s with an explicit worker count: 1, the physical cores, min(32, logical CPUs)."""
        if self.run_with is None:
            return {}
        desc = cpu_description()
        counts = sorted({1, desc["physical_cores"] or 1, min(32, desc["logical_cpus"] or 1)})
        out = {}
        for workers in counts:
            self.run_with(self.groups[0], workers)
            t0, n = time.perf_counter(), 0
            while n == 0 or time.perf_counter() - t0 < budget_each_s:
                self.run_with(self.groups[n % len(self.groups)], workers)
                n += 1
            out[str(workers)] = ALGO_BYTES_PER_GROUP * n / (time.perf_counter() - t0) / 1e9
        return out


def cpu_reference_leg(packed: np.ndarray, x: np.ndarray, budget_s: float, copies: int) -> dict:
    ref = CpuReference(packed, x, copies)
    leg = ref.sample(budget_s)
    leg["gbs_by_workers"] = ref.worker_sweep(min(2.0, budget_s / 6))
    return leg


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    packed, x = make_inputs()
    ref = CpuReference(packed, x, 16)
    # a step is a bounded sample of the workload; the whole run is sized to about a minute
    per_step_budget = max(0.02, min(20.0, 60.0 / max(1, args.steps + args.warmup)))
    leg = None
    for _ in range(args.warmup):
        leg = ref.sample(per_step_budget)
    vals, calls, t0 = [], 0, time.perf_counter()
    for _ in range(args.steps):
        leg = ref.sample(per_step_budget)
        vals.append(leg["value"])
    elapsed = time.perf_counter() - t0
    value = statistics.mean(vals)
    leg["value"] = value
    leg["sample"] = f"{args.steps} steps of {per_step_budget:.2f} s each, gemv_batch submissions of {GROUP} products over 16 weight copies, int8 activations (ZEN_CPU_Q8_ACT=1), reference worker policy"
    print(json.dumps({
        "impl": "reference", "metric": "q8_0_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed * 1e3 / max(1, args.steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config0(), "notes": "16 rotating weight copies (285 MB, larger than the CPU caches), two submissions of eight per pass",
        "cpu_baseline": leg, "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))



# ---- workload q8_0_gemm: the prefill GEMM of the second benchmark configuration --------------------------------
GEMM_T, GEMM_ROWS, GEMM_COLS, GEMM_COPIES = 512, 14336, 4096, 4
GEMM_OPS = 2 * GEMM_T * GEMM_ROWS * GEMM_COLS  # 60,129,542,144 int8 operations per product


def int8_peak_tops() -> tuple[float, str]:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return 2.0 * float(json.load(f)["bf16_tflops"]), "2 x measured dense bf16 (int8 dense is twice bf16 on this part)"
    except Exception:
        return 2.0 * 1590.0, "2 x fallback bf16"


def run_gemm_workload(args, brief: bool = False) -> dict:
    """Q8_0 prefill GEMM, Llama-3-8B FFN-up shape: activations fp32 512x4096 (seed 2), W 14336x4096 Q8_0 (seed 3),
    out fp32 512x14336.  A step is one product (activation quantise + tcgen05 GEMM) on the next of GEMM_COPIES weight
    copies with its own output buffer (4 x 100 MB, larger than L2)."""
    import torch
    from zeninfer_b200 import Backend, blocks
    if not brief and (int(os.environ.get("WORLD_SIZE", "1")) != 1 or args.gpus != 1):
        raise SystemExit("workload q8_0_gemm is a single-GPU workload")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(local)
    be = Backend()
    w = np.random.default_rng(3).standard_normal((GEMM_ROWS, GEMM_COLS), dtype=np.float32) * np.float32(0.02)
    packed = np.ascontiguousarray(blocks.quantize_q8_0(w))
    del w
    x_host = np.random.default_rng(2).standard_normal((GEMM_T, GEMM_COLS), dtype=np.float32)
    handles = [be.dev_upload("Q8_0", packed, GEMM_ROWS, GEMM_COLS) for _ in range(GEMM_COPIES)]
    d_x = torch.from_numpy(x_host).to(dev)
    outs = [torch.empty((GEMM_T, GEMM_ROWS), dtype=torch.float32, device=dev) for _ in range(GEMM_COPIES)]
    from zeninfer_b200.backend import ACT_FP32, ACT_INT8
    ws_bytes = be.gemm_workspace_bytes(GEMM_T, GEMM_COLS, ACT_FP32)      # large enough for either mode
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)
    main_mode = ACT_FP32 if args.act == "fp32" else ACT_INT8

    def one_pass(mode=main_mode):
        for h, o in zip(handles, outs):
            be.dev_gemm_q8_0([h], [o.data_ptr()], d_x.data_ptr(), GEMM_T, ws.data_ptr(), ws_bytes, stream.cuda_stream, act_mode=mode)

    steps = 1 if args.profile else 250 if brief else max(1, args.steps // GEMM_COPIES)  # a graph replay is GEMM_COPIES steps
    with torch.cuda.stream(stream):
        one_pass()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        with ClockSampler(local) as clocks:
            t_warm, n_warm = time.time(), 0
            while n_warm * GEMM_COPIES < args.warmup or (time.time() - t_warm < 0.3 and not args.profile):
                graph.replay(); n_warm += 1
                stream.synchronize()
            be.dev_check(stream.cuda_stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            clocks.mark_start()
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            clocks.mark_end()
        ms = e0.elapsed_time(e1)
    be.dev_check(stream.cuda_stream)
    n_products = steps * GEMM_COPIES
    per_product_us = ms * 1e3 / n_products
    # the other activation mode, plain launches over the same rotating copies (the products are long enough to hide them)
    other_mode = ACT_INT8 if main_mode == ACT_FP32 else ACT_FP32
    other_us = None
    if not args.profile:
        with torch.cuda.stream(stream):
            for _ in range(3):
                one_pass(other_mode)
            stream.synchronize()
            e0.record(stream)
            n_other = 10 if brief else 25
            for _ in range(n_other):
                one_pass(other_mode)
            e1.record(stream)
            stream.synchronize()
        other_us = e0.elapsed_time(e1) * 1e3 / (n_other * GEMM_COPIES)
        with torch.cuda.stream(stream):
            one_pass()                       # the outputs hold the timed mode's results again
        be.dev_check(stream.cuda_stream)
    mode_name = {ACT_INT8: "int8_activations", ACT_FP32: "fp32_equivalent_activations"}
    value = GEMM_OPS / (per_product_us * 1e-6) / 1e12
    peak, peak_kind = int8_peak_tops()

    if args.profile:
        return {"metric": "q8_0_prefill_gemm_int8_tops", "profile_run": True, "value": value, "unit": "TOPS", "launch_us": per_product_us,
                "launches": "per product: group_digits_acts_kernel, gg_zero_split_tiles_kernel, gemm_groups_kernel (the first product of a tensor also builds its two-digit planes: group_digits_q8_0_kernel); 4 products untimed, 4 + 4 replayed"}
    # e2e: the host-pointer call, activations host->device and the 29 MB result device->host inside the timed region
    copies = [packed] + [packed.copy() for _ in range(GEMM_COPIES - 1)]
    be.set_q8_act_mode(main_mode)
    for c in copies:
        y_host = be.gemm("Q8_0", c, x_host, GEMM_T, GEMM_ROWS, GEMM_COLS)
    e2e_steps = 1 if brief else 3
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for c in copies:
            be.gemm("Q8_0", c, x_host, GEMM_T, GEMM_ROWS, GEMM_COLS)
    e2e_s = time.perf_counter() - t0
    e2e_value = GEMM_OPS * e2e_steps * GEMM_COPIES / e2e_s / 1e12
    assert np.array_equal(y_host, outs[-1].cpu().numpy()), "host-pointer and device-pointer paths disagree"

    be.set_q8_act_mode(ACT_INT8)
    for c in copies:
        be.release_weights(c)
    for h in handles:
        be.dev_free(h)
    cpu = None
    if not args.no_cpu_baseline and not brief:
        import oracle
        if oracle.reference_available():
            zr = oracle.Reference()
            run, kind, cores = (lambda: zr.gemm(oracle.Q8_0, packed, x_host, GEMM_T, GEMM_ROWS, GEMM_COLS, workers=0)), "reference", min(zr.pool_workers(), os.cpu_count() or 1)
        else:
            zo = oracle.Oracle()
            run, kind, cores = (lambda: zo.gemm(oracle.Q8_0, packed[:256], x_host, GEMM_T, 256, GEMM_COLS)), "port", 1
        run()
        t0, n = time.perf_counter(), 0
        while time.perf_counter() - t0 < args.cpu_budget:
            run(); n += 1
        dt = time.perf_counter() - t0
        frac = 1.0 if kind == "reference" else 256 / GEMM_ROWS
        cpu = {**cpu_description(), "value": GEMM_OPS * frac * n / dt / 1e12, "unit": "TOPS", "cores": cores, "kind": kind,
               "sample": f"{n} full products in {dt:.1f} s, the reference's default fp32-activation K-blocked kernel (it has no int8 GEMM), its own worker policy"}

    return ({
        "metric": "q8_0_prefill_gemm_int8_tops", "value": value, "unit": "TOPS", "n_gpus": 1, "steps": n_products, "warmup": args.warmup,
        "ms_per_step": per_product_us / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "Q8_0 prefill GEMM 512 x 14336 x 4096 (config 1): activation digits + tcgen05 kind::i8 GEMM per step",
                   "l2": f"inputs larger than L2: {GEMM_COPIES} weight copies and output buffers, 100 MB per product", "launch": "CUDA graph replay"},
        "roofline": {"bound": "tensor", "achieved": value, "peak": peak, "unit": "TOPS", "frac": value / peak, "peak_kind": peak_kind, "traffic": GEMM_NCU_TRAFFIC_BYTES,
                     "launch_us": per_product_us, "algorithmic_ops_per_launch": GEMM_OPS, "activations": mode_name[main_mode],
                     "other_mode": {"activations": mode_name[other_mode], "launch_us": other_us, "tops_of_the_same_product": GEMM_OPS / (other_us * 1e-6) / 1e12,
                                    "note": "fp32-equivalent activations = the reference's default prefill arithmetic; int8 = its ZEN_CPU_Q8_ACT route; the group-scale kernel runs the same three MMAs per 32 columns for both"},
                     "note": "time includes the activation kernel; weights and activations are two int8 digits under one scale per 256 weights, a group accumulates in TMEM; tensor pipe 46 % busy, L2 39 % of its peak (950 MB of operand traffic per product): it waits for operands with two 64 KB K tiles in flight per SM"},
        "cpu_baseline": cpu, "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "TOPS", "h2d_bytes_per_step": GEMM_T * GEMM_COLS * 4, "d2h_bytes_per_step": GEMM_T * GEMM_ROWS * 4,
                "api": "zen_cuda_gemm_q8_0 (host pointers)", "steps": e2e_steps * GEMM_COPIES},
        "gpu_launches": 2 * n_products,
    })


# ---- workload layer_sweep: mixed-format decode GEMV sweep over one Llama-3-8B layer (third benchmark configuration) ----
LAYER_TENSORS = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
                 ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336))
# what a decode step launches: projections that share an input go out as one launch (zen::quant::gemv_batch)
LAYER_LAUNCHES = (("qkv", ("q", "k", "v")), ("o", ("o",)), ("gate_up", ("gate", "up")), ("down", ("down",)))
FORMAT_BLOCK = {"Q4_0": (32, 18), "Q8_0": (32, 34), "Q6_K": (256, 210), "Q4_K": (256, 144), "Q5_K": (256, 176)}
SWEEP_MIN_BYTES = 300e6   # bytes a timing loop sweeps before it meets an address again: well past the 126 MB L2


def tensor_bytes(fmt: str, rows: int, cols: int) -> int:
    elems, nbytes = FORMAT_BLOCK[fmt]
    return rows * (cols // elems) * nbytes


def run_layer_sweep(args) -> dict:
    """All seven projections of one layer (weights N(0, 0.02), inputs N(0, 1), one generator seeded 4) in Q4_0, Q8_0 and
    Q6_K, batch 1.  Every launch kind is timed on its own over enough rotating weight copies to exceed L2, and the
    whole layer (four launches) is timed as a sequence over rotating layer copies.  value = the Q8_0 layer."""
    import torch
    from zeninfer_b200 import Backend, blocks
    from zeninfer_b200.backend import ACT_FP32, ACT_INT8, FORMAT_IDS
    if int(os.environ.get("WORLD_SIZE", "1")) != 1 or args.gpus != 1:
        raise SystemExit("workload layer_sweep is a single-GPU workload")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    be = Backend()
    rng = np.random.default_rng(4)
    dense = {name: rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02) for name, rows, cols in LAYER_TENSORS}
    shape = {name: (rows, cols) for name, rows, cols in LAYER_TENSORS}
    x_host = {4096: rng.standard_normal(4096, dtype=np.float32), 14336: rng.standard_normal(14336, dtype=np.float32)}
    d_x = {k: torch.from_numpy(v).to(dev) for k, v in x_host.items()}
    d_y = {name: torch.zeros(rows, dtype=torch.float32, device=dev) for name, rows, _ in LAYER_TENSORS}
    stream = torch.cuda.Stream(device=dev)
    peak, peak_kind = peaks()
    reps = 1 if args.profile else max(3, args.steps // 100)

    def time_graph(enqueue, launches_per_replay):
        with torch.cuda.stream(stream):
            enqueue()
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                enqueue()
            for _ in range(1 if args.profile else max(3, args.warmup)):
                graph.replay()
            stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        be.dev_check(stream.cuda_stream)
        return e0.elapsed_time(e1) * 1e3 / (reps * launches_per_replay)  # microseconds per launch

    detail, packed_q8, launches_total = {}, None, 0
    with ClockSampler(0) as clocks:
        clocks.mark_start()
        for fmt in [f for f in ("Q8_0", "Q4_0", "Q6_K", "Q4_K", "Q5_K") if f in args.formats.split(",")]:
            mode = ACT_INT8 if fmt == "Q8_0" else ACT_FP32
            if fmt in ("Q4_K", "Q5_K"):   # no quantiser for these (the reference has none): valid random super-blocks, weights of the order of 0.02
                packed = {name: blocks.random_k_blocks(FORMAT_IDS[fmt], *shape[name], seed=40 + i) for i, name in enumerate(dense)}
            else:
                packed = {name: np.ascontiguousarray(blocks.quantize(FORMAT_IDS[fmt], dense[name])) for name in dense}
            if fmt == "Q8_0":
                packed_q8 = packed
            layer_bytes = sum(tensor_bytes(fmt, *shape[n]) for n in shape)
            layer_copies = int(SWEEP_MIN_BYTES // layer_bytes) + 1
            per_kind, copies = {}, {}

            def launch(hs, names, cols, next_handle, fmt=fmt, mode=mode):
                """One product launch; it also hints the tensor the next launch reads to L2 (no result changes)."""
                be.dev_gemv_fused(hs, [d_y[n].data_ptr() for n in names], d_x[cols].data_ptr(), 1, mode, stream.cuda_stream, warm_next=next_handle)

            for kind, names in LAYER_LAUNCHES:
                nbytes = sum(tensor_bytes(fmt, *shape[n]) for n in names)
                ncopy = max(layer_copies, int(SWEEP_MIN_BYTES // nbytes) + 1)
                copies[kind] = [[be.dev_upload(fmt, packed[n], *shape[n]) for n in names] for _ in range(ncopy)]
                cols = shape[names[0]][1]
                algo = nbytes + 4 * cols + 4 * sum(shape[n][0] for n in names)

                def enqueue(kind=kind, names=names, cols=cols):
                    for c, hs in enumerate(copies[kind]):
                        launch(hs, names, cols, copies[kind][(c + 1) % len(copies[kind])][0])

                us = time_graph(enqueue, ncopy)
                launches_total += (reps + max(3, args.warmup) + 2) * ncopy
                per_kind[kind] = {"rows": [shape[n][0] for n in names], "columns": cols, "algorithmic_bytes": algo, "copies": ncopy,
                                  "us": us, "gbs": algo / us / 1e3, "frac": algo / us / 1e3 / peak}

            def enqueue_layer():
                order = [(c, kind, names) for c in range(layer_copies) for kind, names in LAYER_LAUNCHES]
                for i, (c, kind, names) in enumerate(order):
                    nc, nkind, _ = order[(i + 1) % len(order)]
                    launch(copies[kind][c], names, shape[names[0]][1], copies[nkind][nc][0])

            layer_us = time_graph(enqueue_layer, layer_copies)
            launches_total += (reps + max(3, args.warmup) + 2) * layer_copies * len(LAYER_LAUNCHES)
            layer_algo = sum(v["algorithmic_bytes"] for v in per_kind.values())
            per_kind["layer"] = {"algorithmic_bytes": layer_algo, "copies": layer_copies, "us": layer_us, "gbs": layer_algo / layer_us / 1e3,
                                 "frac": layer_algo / layer_us / 1e3 / peak, "launches": len(LAYER_LAUNCHES)}
            detail[fmt] = per_kind
            for kind in copies:
                for hs in copies[kind]:
                    for h in hs:
                        be.dev_free(h)
        clocks.mark_end()

    if args.profile or packed_q8 is None:
        return {"metric": "layer_decode_gemv_hbm_gbs", "profile_run": args.profile, "detail": detail,
                "launches": "per format: q|k|v, o, gate|up, down copies in turn (one untimed pass, two replays each), then the layer sequence"}
    # e2e: the Q8_0 layer through the host-pointer calls (zen_cuda_gemv_q8_0_batch / zen_cuda_gemv_q8_0), host buffers
    hosts = [{n: (packed_q8[n] if c == 0 else packed_q8[n].copy()) for n in packed_q8} for c in range(2)]

    def host_layer(hc):
        for kind, names in LAYER_LAUNCHES:
            cols = shape[names[0]][1]
            if len(names) > 1:
                be.gemv_batch("Q8_0", [hc[n] for n in names], x_host[cols], [shape[n][0] for n in names], cols)
            else:
                be.gemv("Q8_0", hc[names[0]], x_host[cols], shape[names[0]][0], cols)

    for hc in hosts:
        host_layer(hc)
    e2e_steps, t0 = 10, time.perf_counter()
    for i in range(e2e_steps):
        host_layer(hosts[i % 2])
    e2e_s = time.perf_counter() - t0
    q8 = detail["Q8_0"]
    e2e_value = q8["layer"]["algorithmic_bytes"] * e2e_steps / e2e_s / 1e9

    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        os.environ.setdefault("ZEN_CPU_Q8_ACT", "1")
        if oracle.reference_available():
            zr = oracle.Reference()
            run = lambda n: zr.gemv(oracle.Q8_0, packed_q8[n], x_host[shape[n][1]], shape[n][0], shape[n][1], workers=0)
            kind, cores = "reference", min(zr.pool_workers(), os.cpu_count() or 1)
        else:
            zo = oracle.Oracle()
            run = lambda n: zo.gemv(oracle.Q8_0, packed_q8[n], x_host[shape[n][1]], shape[n][0], shape[n][1], int8_acts=True)
            kind, cores = "port", 1
        t0, n = time.perf_counter(), 0
        while n == 0 or time.perf_counter() - t0 < args.cpu_budget:
            for name in shape:
                run(name)
            n += 1
        dt = time.perf_counter() - t0
        cpu = {**cpu_description(), "value": q8["layer"]["algorithmic_bytes"] * n / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
               "sample": f"{n} passes over the seven Q8_0 projections of the layer in {dt:.1f} s, one call per projection, int8 activations"}

    dom = q8["gate_up"]
    return ({
        "metric": "layer_decode_gemv_hbm_gbs", "value": q8["layer"]["gbs"], "unit": "GB/s", "n_gpus": 1, "steps": reps, "warmup": max(3, args.warmup),
        "ms_per_step": q8["layer"]["us"] / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "decode GEMV sweep over one Llama-3-8B layer, batch 1, Q8_0 / Q4_0 / Q6_K (config 2) and Q4_K / Q5_K; value = the Q8_0 layer, "
                               "four launches (q|k|v, o, gate|up, down)",
                   "l2": f"inputs larger than L2: every timing loop sweeps at least {SWEEP_MIN_BYTES / 1e6:.0f} MB of distinct weight copies",
                   "launch": "CUDA graph replay"},
        "roofline": {"bound": "hbm", "achieved": dom["gbs"], "peak": peak, "unit": "GB/s", "frac": dom["frac"], "peak_kind": peak_kind, "traffic": None,
                     "kernel": "gemv_q8_0_kernel<1,1> on gate|up (2 x 14336 x 4096)", "launch_us": dom["us"],
                     "algorithmic_bytes_per_launch": dom["algorithmic_bytes"]},
        "detail": detail, "cpu_baseline": cpu, "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 4 * (3 * 4096 + 14336), "d2h_bytes_per_step": 4 * sum(r for _, r, _ in LAYER_TENSORS),
                "api": "zen_cuda_gemv_q8_0_batch + zen_cuda_gemv_q8_0 (host pointers)", "steps": e2e_steps},
        "gpu_launches": launches_total,
    })


# ---- workload lm_head: row-sharded Q6_K lm_head, fused all-gather of the logits, greedy pick (fourth configuration) ----
LM_ROWS, LM_COLS = 128256, 4096


def torch_q6_k_pack(w):
    """fp32 [rows, K] on the GPU -> uint8 [rows, K/256*210] raw GGUF Q6_K super-blocks: zeninfer_b200.blocks.quantize_q6_k
    (a plain valid encoder: group scale amax/31, super-block d maps the largest group scale to 127, codes
    round(x / (d*sc)) + 32) and pack_q6_k restated on torch, because packing half a billion weights with numpy takes a
    minute of box time.  Benchmark input preparation only."""
    import torch
    rows, k = w.shape
    n = rows * (k // 256)
    grp = w.reshape(n, 16, 16)
    gscale = grp.abs().amax(dim=2) / 31.0
    d = (gscale.amax(dim=1) / 127.0).to(torch.float16)
    d32 = d.to(torch.float32)
    sc = torch.where(d32[:, None] > 0, torch.round(gscale / d32[:, None].clamp_min(1e-30)), torch.zeros_like(gscale)).clamp_(1, 127)
    eff = d32[:, None] * sc
    q = torch.where(eff[..., None] > 0, torch.round(grp / eff[..., None].clamp_min(1e-30)), torch.zeros_like(grp))
    q = (q.clamp_(-32, 31) + 32).to(torch.uint8).reshape(n, 2, 4, 32)
    out = torch.zeros((n, 210), dtype=torch.uint8, device=w.device)
    ql, qh = out[:, :128].view(n, 2, 2, 32), out[:, 128:192].view(n, 2, 32)
    ql[:, :, 0, :] = (q[:, :, 0, :] & 15) | ((q[:, :, 2, :] & 15) << 4)
    ql[:, :, 1, :] = (q[:, :, 1, :] & 15) | ((q[:, :, 3, :] & 15) << 4)
    qh[:] = (q[:, :, 0, :] >> 4) | ((q[:, :, 1, :] >> 4) << 2) | ((q[:, :, 2, :] >> 4) << 4) | ((q[:, :, 3, :] >> 4) << 6)
    out[:, 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[:, 208:210] = d.view(torch.uint8).view(n, 2)
    return out.view(rows, -1)


def lm_head_shard(first: int, last: int, dev=None) -> np.ndarray:
    """Rows [first, last) of W 128256 x 4096 ~ N(0, 0.02), packed to Q6_K.  With `dev` the rows are drawn and packed
    on the GPU (torch generator seeded 5, one draw per 8016-row chunk from the start, so every rank sees the same
    matrix); without it, numpy's generator seeded 5 and the numpy packer.  Only the own rows are packed."""
    out, chunk = [], 8016
    if dev is not None:
        import torch
        gen = torch.Generator(device=dev)
        gen.manual_seed(5)
        for r0 in range(0, LM_ROWS, chunk):
            r1 = min(LM_ROWS, r0 + chunk)
            if r0 >= last:
                break
            w = torch.randn((r1 - r0, LM_COLS), generator=gen, device=dev, dtype=torch.float32)
            a, b = max(first, r0), min(last, r1)
            if a < b:
                out.append(torch_q6_k_pack(w[a - r0:b - r0] * 0.02).cpu().numpy())
        return np.ascontiguousarray(np.concatenate(out, axis=0))
    from zeninfer_b200 import blocks
    rng = np.random.default_rng(5)
    for r0 in range(0, LM_ROWS, chunk):
        r1 = min(LM_ROWS, r0 + chunk)
        if r0 >= last:
            break
        w = rng.standard_normal((r1 - r0, LM_COLS), dtype=np.float32)
        a, b = max(first, r0), min(last, r1)
        if a < b:
            out.append(blocks.quantize_q6_k(w[a - r0:b - r0] * np.float32(0.02)))
    return np.ascontiguousarray(np.concatenate(out, axis=0))


def run_gemm_formats(args) -> dict:
    """The config 1 shape (512 x 14336 x 4096) for every format's many-row product, next to the same rows in chunks of
    eight through the decode kernel: Q8_0 with fp32-equivalent activations, Q4_0, Q6_K, Q4_K and Q5_K (the reference
    multiplies these with fp32 activations).  Per format GEMM_COPIES weight copies take turns (larger than L2 together
    with the outputs); a timed step is one product.  One GPU."""
    import torch
    from zeninfer_b200 import Backend, blocks
    from zeninfer_b200.backend import ACT_FP32
    if int(os.environ.get("WORLD_SIZE", "1")) != 1 or args.gpus != 1:
        raise SystemExit("workload gemm_formats is a single-GPU workload")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    be = Backend()
    T, R, K = GEMM_T, GEMM_ROWS, GEMM_COLS
    tokens_list = [T] if args.profile else [16, 128, T]
    d_x = torch.from_numpy(np.random.default_rng(2).standard_normal((T, K), dtype=np.float32)).to(dev)
    stream = torch.cuda.Stream(device=dev)
    S = stream.cuda_stream
    detail = {}
    wanted = [f for f in args.formats.split(",") if f]
    with ClockSampler(0) as clocks:
        clocks.mark_start()
        for name in wanted:
            if name == "Q8_0":
                w = np.random.default_rng(3).standard_normal((R, K), dtype=np.float32) * np.float32(0.02)
                packed = np.ascontiguousarray(blocks.quantize_q8_0(w))
            elif name == "Q4_0":
                w = np.random.default_rng(3).standard_normal((R, K), dtype=np.float32) * np.float32(0.02)
                packed = np.ascontiguousarray(blocks.quantize_q4_0(w))
            elif name == "Q6_K":
                packed = lm_head_shard(0, R, dev)
            else:
                packed = blocks.random_k_blocks(blocks.Q4_K if name == "Q4_K" else blocks.Q5_K, R, K, 3)
            copies = 2 if args.profile else GEMM_COPIES
            handles = [be.dev_upload(name, packed, R, K) for _ in range(copies)]
            y = torch.empty((T, R), dtype=torch.float32, device=dev)
            ws_bytes = max(be.gemm_workspace_bytes(T, K, ACT_FP32), be.gemm_q6_k_workspace_bytes(T, K), be.gemm_q4_0_workspace_bytes(T, R, K),
                           be.gemm_kquant_workspace_bytes(T, R, K))
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)

            def tensor(h, n):
                if name == "Q8_0":
                    be.dev_gemm_q8_0([h], [y.data_ptr()], d_x.data_ptr(), n, ws.data_ptr(), ws_bytes, S, act_mode=ACT_FP32)
                elif name == "Q4_0":
                    be.dev_gemm_q4_0(h, y.data_ptr(), d_x.data_ptr(), n, ws.data_ptr(), ws_bytes, S)
                elif name == "Q6_K":
                    be.dev_gemm_q6_k(h, y.data_ptr(), d_x.data_ptr(), n, ws.data_ptr(), ws_bytes, S)
                else:
                    be.dev_gemm_kquant(h, y.data_ptr(), d_x.data_ptr(), n, ws.data_ptr(), ws_bytes, S)

            def chunks(h, n):
                for t0 in range(0, n, 8):
                    be.dev_gemv([h], [y[t0:].data_ptr()], d_x[t0:].data_ptr(), min(8, n - t0), ACT_FP32, S)

            rows_out = {}
            for n in tokens_list:
                for label, fn in (("tensor_cores", tensor), ("decode_kernel_chunks_of_8", chunks)):
                    if args.profile and label != "tensor_cores":
                        continue
                    with torch.cuda.stream(stream):
                        for h in handles:      # outside the capture: a tensor's first many-row product builds its two-digit planes
                            fn(h, n)
                        stream.synchronize()
                        graph = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(graph, stream=stream):
                            for h in handles:
                                fn(h, n)
                        for _ in range(1 if args.profile else 3):
                            graph.replay()
                        stream.synchronize()
                        reps = 1 if args.profile else 5
                        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        e0.record(stream)
                        for _ in range(reps):
                            graph.replay()
                        e1.record(stream)
                        stream.synchronize()
                    us = e0.elapsed_time(e1) * 1e3 / (reps * len(handles))
                    rows_out.setdefault(str(n), {})[label] = {"us": us, "tops": 2.0 * n * R * K / us / 1e6}
            be.dev_check(S)
            detail[name] = rows_out
            for h in handles:
                be.dev_free(h)
            del ws, y
        clocks.mark_end()
    first = detail[wanted[0]][str(T)]["tensor_cores"]
    return {"metric": "many_row_product_tops_by_format", "value": first["tops"], "unit": "TOPS", "n_gpus": 1, "higher_is_better": True, "dtype": "s8 x s8 -> s32, fp32 scales",
            "data": "synthetic", "profile_run": args.profile,
            "config": {"workload": f"{T} x {R} x {K} (the config 1 shape) by weight format, fp32-equivalent activations (two int8 digits); also 16 and 128 rows",
                       "value_is": f"{wanted[0]} at {T} rows"},
            "detail": detail, "clocks": clocks.summary(), "vs_baseline": None}


def run_lm_head(args, brief: bool = False) -> dict | None:
    """Q6_K lm_head 128256 x 4096 at batch 1 (value) and batch 8, rows sharded over the ranks.  A step on every rank: the
    shard product with the all-gather fused in (or followed by an NCCL all-gather), then the greedy pick over the
    gathered logits.  Total work is fixed as N grows: strong scaling."""
    import torch
    import torch.distributed as dist
    from zeninfer_b200 import Backend, shard
    from zeninfer_b200.backend import ACT_FP32

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    be = Backend()
    plan = shard.shard_plan(LM_ROWS, world)
    first, last = plan[rank]
    my_rows, widest = last - first, max(b - a for a, b in plan)
    packed = lm_head_shard(first, last, dev if (brief or args.device_pack) else None)
    shard_bytes = tensor_bytes("Q6_K", my_rows, LM_COLS)
    ncopy = int(SWEEP_MIN_BYTES // shard_bytes) + 1
    handles = [be.dev_upload("Q6_K", packed, my_rows, LM_COLS) for _ in range(ncopy)]
    hidden = np.random.default_rng([5, 1]).standard_normal((8, LM_COLS), dtype=np.float32)
    d_h = torch.from_numpy(hidden).to(dev)
    stream = torch.cuda.Stream(device=dev)
    fused = world > 1 and args.gather == "fused"
    peak, peak_kind = peaks()
    results = {}

    with ClockSampler(local) as clocks:
        for tokens in (1, 8):
            d_local = torch.zeros((tokens, my_rows), dtype=torch.float32, device=dev)
            d_all = torch.zeros((world, tokens * widest), dtype=torch.float32, device=dev)
            d_pick = torch.full((tokens,), -7, dtype=torch.int64, device=dev)
            # two or more rows: the tensor-core product, then (several GPUs, equal shards) an NCCL all-gather of the logits
            tensor = tokens >= 2 and not args.no_q6k_tensor and my_rows == widest
            pg = shard.PeerGather(be, world, rank, tokens * widest) if fused and not tensor else None
            segs = [(d_all.data_ptr() + 4 * r * tokens * widest, b - a, a, b - a) for r, (a, b) in enumerate(plan)]
            if world == 1:
                segs = [(d_local.data_ptr(), LM_ROWS, 0, LM_ROWS)]

            ws_bytes = be.gemm_q6_k_workspace_bytes(tokens, LM_COLS)
            d_ws = torch.zeros(ws_bytes if tensor else 16, dtype=torch.uint8, device=dev)

            def one_pass():
                for h in handles:
                    if tensor:
                        be.dev_gemm_q6_k(h, d_local.data_ptr(), d_h.data_ptr(), tokens, d_ws.data_ptr(), ws_bytes, stream.cuda_stream)
                        if world > 1:
                            dist.all_gather_into_tensor(d_all.view(world * tokens, widest), d_local)
                    elif fused:
                        pg.gemv([h], d_h.data_ptr(), tokens, ACT_FP32, stream.cuda_stream, d_y=[d_local.data_ptr()])
                        pg.fetch(d_all.data_ptr(), stream.cuda_stream)
                    else:
                        be.dev_gemv([h], [d_local.data_ptr()], d_h.data_ptr(), tokens, ACT_FP32, stream.cuda_stream)
                        if world > 1:
                            send = d_local if my_rows == widest else torch.nn.functional.pad(d_local, (0, widest - my_rows))
                            dist.all_gather_into_tensor(d_all.view(world * tokens, widest), send.contiguous())
                    be.dev_greedy_pick(segs, tokens, d_pick.data_ptr(), stream.cuda_stream)

            with torch.cuda.stream(stream):
                one_pass()
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_pass()
                for _ in range(max(3, args.warmup)):
                    graph.replay()
                stream.synchronize()
                be.dev_check(stream.cuda_stream)
                replays = (200 if brief else max(1, args.steps // ncopy))
                if world > 1:
                    dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                if tokens == 1:
                    clocks.mark_start()
                e0.record(stream)
                for _ in range(replays):
                    graph.replay()
                e1.record(stream)
                stream.synchronize()
                if tokens == 1:
                    clocks.mark_end()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms = e0.elapsed_time(e1)
            be.dev_check(stream.cuda_stream)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            steps = replays * ncopy
            # what was timed is right: the pick equals the first maximum of the gathered logits, and the own shard of the
            # gathered logits equals the local product
            if world > 1:
                mine = d_all[rank, : tokens * my_rows].view(tokens, my_rows)
                assert bool((mine == d_local).all().item()), "gathered shard differs from the local product"
                full = torch.cat([d_all[r, : tokens * (b - a)].view(tokens, b - a) for r, (a, b) in enumerate(plan)], dim=1)
            else:
                full = d_local
            assert bool((shard.greedy_pick(full) == d_pick).all().item()), "device pick differs from the first maximum of the logits"
            algo = tensor_bytes("Q6_K", LM_ROWS, LM_COLS) + tokens * 4 * (LM_COLS + LM_ROWS)
            results[tokens] = {"us_per_step": ms * 1e3 / steps, "gbs": algo / (ms * 1e-3 / steps) / 1e9, "steps": steps,
                               "algorithmic_bytes": algo, "picks_per_s": tokens * steps / (ms * 1e-3),
                               "kernel": ("gemm_groups_kernel (tcgen05)" + (", NCCL all-gather" if world > 1 else "")) if tensor else "gemv_kq_kernel (dp4a)"}
            if pg is not None:
                stream.synchronize()
                pg.close()

    for h in handles:
        be.dev_free(h)

    # e2e (single GPU): the host-pointer Q6_K call, hidden state host->device and all logits device->host per step
    e2e = None
    if world == 1:
        be.gemm("Q6_K", packed, hidden[:1], 1, LM_ROWS, LM_COLS)
        e2e_steps, t0 = 10, time.perf_counter()
        for _ in range(e2e_steps):
            y = be.gemm("Q6_K", packed, hidden[:1], 1, LM_ROWS, LM_COLS)
        e2e_s = time.perf_counter() - t0
        e2e = {"value": results[1]["algorithmic_bytes"] * e2e_steps / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * LM_COLS,
               "d2h_bytes_per_step": 4 * LM_ROWS, "api": "zen_cuda_gemm_q6_k (host pointers, tokens = 1)", "steps": e2e_steps}
        be.release_weights(packed)
    if rank != 0:
        return None
    cpu = None
    if world == 1 and not args.no_cpu_baseline and not brief:
        import oracle
        if oracle.reference_available():
            zr = oracle.Reference()
            run, kind, cores = (lambda: zr.gemv(oracle.Q6_K, packed, hidden[0], LM_ROWS, LM_COLS, workers=0)), "reference", min(zr.pool_workers(), os.cpu_count() or 1)
        else:
            zo = oracle.Oracle()
            run, kind, cores = (lambda: zo.gemv(oracle.Q6_K, packed, hidden[0], LM_ROWS, LM_COLS)), "port", 1
        run()
        t0, n = time.perf_counter(), 0
        while n == 0 or time.perf_counter() - t0 < args.cpu_budget:
            run(); n += 1
        dt = time.perf_counter() - t0
        cpu = {**cpu_description(), "value": results[1]["algorithmic_bytes"] * n / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
               "sample": f"{n} full lm_head products (batch 1) in {dt:.1f} s, the reference's Q6_K kernel, its own worker policy"}
    r1 = results[1]
    per_gpu = r1["gbs"] / world
    return ({
        "metric": "lm_head_q6_k_hbm_gbs", "value": r1["gbs"], "unit": "GB/s", "n_gpus": world, "steps": r1["steps"], "warmup": max(3, args.warmup),
        "ms_per_step": r1["us_per_step"] / 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "Q6_K lm_head 128256 x 4096 (config 3), batch 1 (value) and batch 8, rows sharded over the GPUs, logits all-gathered, greedy pick",
                   "gather": ("none (one GPU)" if world == 1 else "fused into the product kernel (peer stores over NVLink)" if fused else "NCCL all-gather"),
                   "l2": f"inputs larger than L2: {ncopy} rotating copies of the {shard_bytes / 1e6:.0f} MB shard per GPU", "launch": "CUDA graph replay"},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak, "peak_kind": peak_kind, "traffic": None,
                     "kernel": "gemv_kq_kernel<Q6_K codes unpacked, 1> (per GPU; step time includes the gather wait and the pick)", "launch_us": r1["us_per_step"],
                     "algorithmic_bytes_per_launch": r1["algorithmic_bytes"] // world,
                     "device_layout": "6-bit codes unpacked on upload to one int8 per weight: the kernel streams 1.30 x the algorithmic (file) bytes, "
                                      "272 B per 256 weights for 210, and no longer rebuilds codes from ql | qh (ZEN_CUDA_Q6K_CODES=0 keeps the file's planes: 143 us)"},
        "detail": {"batch1": r1, "batch8": results[8]}, "cpu_baseline": cpu, "clocks": clocks.summary(), "e2e": e2e,
        "gpu_launches": sum(r["steps"] for r in results.values()) * (4 if fused else 3),
    })


# ---- workload decode: full greedy decode of a random-init Llama-3-8B-shaped Q8_0 model (fifth configuration) ----------
def torch_q8_0_pack(w):
    """fp32 [rows, K] on the GPU -> uint8 [rows, K/32*34] raw GGUF Q8_0 blocks, the packer of zeninfer_b200.blocks
    (scale = amax/127 stored as fp16, codes from the unrounded scale, round half away from zero) on torch, because
    packing eight billion weights with numpy would take minutes of box time.  Benchmark input preparation only."""
    import torch
    rows, k = w.shape
    blk = w.view(rows, k // 32, 32)
    scale = blk.abs().amax(dim=2) / 127.0
    inv = torch.where(scale > 0, 1.0 / scale, torch.zeros_like(scale))
    v = blk * inv[..., None]
    t = torch.trunc(v)
    q = (t + torch.where((v - t).abs() >= 0.5, torch.sign(v), torch.zeros_like(v))).clamp_(-127, 127).to(torch.int8)
    out = torch.empty((rows, k // 32, 34), dtype=torch.uint8, device=w.device)
    out[..., 0:2] = scale.to(torch.float16).view(torch.uint8).view(rows, k // 32, 2)
    out[..., 2:] = q.view(torch.uint8)
    return out.view(rows, -1)


def run_decode(args, brief: bool = False) -> dict | None:
    """Config: 32 layers, d 4096, 32 query / 8 KV heads of 128, SwiGLU 14336, vocab 128256, eps 1e-5, theta 500000,
    weights N(0, 0.02) seed 6, a prompt of 512 uniform-random ids, then greedy decode steps.  The prompt is consumed as
    blocks of tensor-core products and timed separately (prefill_ms); sharded, the block's partial products are summed by
    two NCCL all-reduces per layer.  A step is one decoded token: the launches of 32 layers, the lm_head and the pick, replayed from two CUDA
    graphs (RMSNorm and the residual adds are folded into the projection launches)."""
    import torch
    from zeninfer_b200 import Backend
    from zeninfer_b200.backend import ACT_INT8
    from zeninfer_b200.llama import LlamaConfig, LlamaDecoder, tensor_plan
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    be = Backend()
    cfg = LlamaConfig(layers=args.layers) if args.layers else LlamaConfig()
    prompt_len = args.prompt_len
    steps = 2 if args.profile else 125 if (brief or args.steps == DEFAULT_STEPS) else args.steps      # the default run: 3 warm-up + 125 timed = the 128 greedy steps
    warm = 1 if args.profile else max(3, args.warmup)

    def tensors():
        gen = torch.Generator(device=dev)
        gen.manual_seed(6)
        for name, shape, is_matrix in tensor_plan(cfg):
            if is_matrix:
                w = torch.randn(shape, generator=gen, device=dev, dtype=torch.float32) * 0.02
                yield name, torch_q8_0_pack(w).cpu().numpy(), True
            else:
                yield name, (1.0 + 0.02 * torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)).cpu().numpy(), False

    t0 = time.perf_counter()
    dec = LlamaDecoder(be, cfg, tensors(), act_mode=ACT_INT8, max_positions=1024, fused=args.fuse, rank=rank, world=world,
                       gather="nccl" if args.gather == "nccl" else "peer", cut=args.cut)
    load_s = time.perf_counter() - t0
    dec.capture()
    token_prefill = args.token_prefill or not dec.can_prefill_blocks()     # sharded: blocks need the column cut and the NCCL group
    prompt = np.random.default_rng(6).integers(0, cfg.vocab, size=prompt_len, dtype=np.int64)
    stream = dec.stream
    with ClockSampler(local) as clocks:
        with torch.cuda.stream(stream):
            dec.reset()
            dec.feed_prompt(prompt.tolist(), batched_prefill=not token_prefill)      # first run: kernel attributes, workspace allocation
            stream.synchronize()
            dec.reset()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(stream)
            dec.feed_prompt(prompt.tolist(), batched_prefill=not token_prefill)      # the prompt as tensor-core blocks (or token by token), then the first pick
            p1.record(stream)
            stream.synchronize()
            prefill_ms = p0.elapsed_time(p1)
            for _ in range(warm):
                dec.step(want_token=True)
            stream.synchronize()
            be.dev_check(stream.cuda_stream)
            if world > 1:
                torch.cuda.synchronize()
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            clocks.mark_start()
            e0.record(stream)
            for _ in range(steps):
                dec.step(want_token=True)
            e1.record(stream)
            stream.synchronize()
            clocks.mark_end()
            if world > 1:
                torch.cuda.synchronize()
                dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:       # the step's time is the slowest rank's
            t = torch.tensor([ms, prefill_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, prefill_ms = float(t[0].item()), float(t[1].item())
    be.dev_check(stream.cuda_stream)
    last_pos = int(dec.pos.item())
    assert last_pos == prompt_len + warm + steps, "position counter out of step"
    assert bool(torch.isfinite(dec.logits).all().item()), "non-finite logits"
    tok_s = steps / (ms * 1e-3)
    layer_bytes = sum(tensor_bytes("Q8_0", r, c) for _, r, c in LAYER_TENSORS)
    weight_bytes = cfg.layers * layer_bytes + tensor_bytes("Q8_0", cfg.vocab, cfg.embedding)
    mean_pos = prompt_len + warm + steps / 2
    kv_bytes = int(cfg.layers * 2 * cfg.kv_width * 4 * mean_pos)
    algo = weight_bytes + kv_bytes
    peak, peak_kind = peaks()
    peak *= world
    achieved = algo / (ms * 1e-3 / steps) / 1e9

    if args.profile:
        dec.close()
        return {"metric": "decode_tokens_per_s", "profile_run": True, "value": tok_s, "unit": "tokens/s", "layers": cfg.layers, "prefill_ms": prefill_ms} if rank == 0 else None
    # e2e: the public generate() call; every picked token is read back to the host as it is produced
    stamps = []
    e2e_new = 33
    picked = dec.generate(prompt.tolist(), e2e_new, on_token=lambda _t: stamps.append(time.perf_counter()))
    e2e_tok_s = (e2e_new - 1) / (stamps[-1] - stamps[0])
    if world > 1:           # every rank picked the same tokens; the rate is the slowest rank's
        ids = torch.tensor(picked, device=dev)
        lo, hi = ids.clone(), ids.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        assert bool((lo == hi).all().item()), "the ranks picked different tokens"
        t = torch.tensor([e2e_tok_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        e2e_tok_s = float(t.item())
    if rank != 0:
        dec.close()
        return None

    cpu = None
    if world == 1 and not args.no_cpu_baseline and not brief:
        import oracle
        from zeninfer_b200 import blocks
        os.environ.setdefault("ZEN_CPU_Q8_ACT", "1")
        if oracle.reference_available():
            zr = oracle.Reference()
            rng = np.random.default_rng(6)
            mats = {(r, c): np.ascontiguousarray(blocks.quantize_q8_0(rng.standard_normal((r, c), dtype=np.float32) * np.float32(0.02)))
                    for r, c in {(r, c) for _, r, c in LAYER_TENSORS}}
            xs = {c: rng.standard_normal(c, dtype=np.float32) for c in (4096, 14336)}
            def one_layer():
                for _, r, c in LAYER_TENSORS:
                    zr.gemv(oracle.Q8_0, mats[(r, c)], xs[c], r, c, workers=0)
            one_layer()
            t0, n = time.perf_counter(), 0
            while n == 0 or time.perf_counter() - t0 < args.cpu_budget:
                one_layer(); n += 1
            dt = time.perf_counter() - t0
            per_token = dt / n * (cfg.layers + tensor_bytes("Q8_0", cfg.vocab, cfg.embedding) / layer_bytes)
            cpu = {**cpu_description(), "value": 1.0 / per_token, "unit": "tokens/s", "cores": min(zr.pool_workers(), os.cpu_count() or 1), "kind": "reference",
                   "sample": f"{n} passes over the seven Q8_0 projections of one layer in {dt:.1f} s (reference kernels, int8 activations, its own "
                             f"worker policy), scaled to 32 layers + lm_head by bytes; attention, norms and sampling not included, so an upper bound "
                             f"for the reference's decode rate on these cores"}

    fn, fs, fr, fp = ("n" in dec.fuse), ("s" in dec.fuse), ("r" in dec.fuse), ("p" in dec.fuse)
    per_layer = 5 + (0 if (fn and fr) else 2) + (0 if (fs or fp) else 1)   # q|k|v, attention block, o, gate|up, down + norm / residual / SwiGLU launches
    launches_per_step = 1 + (0 if fn else 1) + per_layer * cfg.layers + 1 + 1 + 2   # embed, layers, advance, lm_head, pick (2): per rank
    gathers = ((2 if dec.col_cut else 4) * cfg.layers + 1) if world > 1 else 0
    line = ({
        "metric": "decode_tokens_per_s", "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "greedy decode, random-init Llama-3-8B shape in Q8_0 (config 4): 32 layers, d 4096, 32/8 heads of 128, ffn 14336, "
                               f"vocab 128256; prompt of {prompt_len} random ids (untimed here, see prefill_ms), then {warm} + {steps} decode steps",
                   "activations": "int8 (bit-exact reference codes)", "l2": "inputs larger than L2: 8.5 GB of weights stream per token",
                   "launch": f"two CUDA graphs per token, {launches_per_step} kernel launches (folded into the projections: '{dec.fuse}')", "weights": "torch.randn on the device, seed 6, N(0, 0.02)",
                   "sharding": ("none (one GPU)" if world == 1 else f"output rows of every matrix over {world} GPUs, rank-local heads and KV cache, "
                                f"{gathers} exchanges per token inside the step graphs "
                                + ("(o and down cut by columns, their partial products all-reduced into the residual stream; logits gathered), "
                                   if dec.col_cut else "(all-gathers of attention output, o, SwiGLU activation, down; logits), ")
                                + ("NCCL collectives" if args.gather == "nccl" else "each one launch of a peer-store kernel over NVLink")),
                   "load_s": load_s, "prefill": ("token by token" if token_prefill else "blocks of up to 512 tokens through the tcgen05 GEMM + causal block attention"
                               + (", two all-reduces of the block's partial products per layer (NCCL)" if world > 1 else "")),
                   "prefill_ms": prefill_ms, "prefill_tokens_per_s": prompt_len / (prefill_ms * 1e-3)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None,
                     "kernel": "whole token step (projections through gemv_q8_0_kernel<1,1>)", "launch_us": ms * 1e3 / steps,
                     "algorithmic_bytes_per_launch": algo, "weight_bytes": weight_bytes, "kv_bytes": kv_bytes},
        "cpu_baseline": cpu, "clocks": clocks.summary(),
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 8, "d2h_bytes_per_step": 8,
                "api": "LlamaDecoder.generate: each picked token id is read back to the host, and fed to the next step from pinned host memory, "
                       "as the reference's generate loop does", "steps": e2e_new - 1},
        "gpu_launches": steps * (launches_per_step + (gathers if dec.peer is not None else 0)) * world,
    })
    dec.close()
    return line


DEFAULT_STEPS = 20


def brief_detail(line: dict | None, keep: tuple[str, ...]) -> dict | None:
    """The figures of a workload's line that the default line's `detail` carries."""
    if line is None:
        return None
    out = {k: line[k] for k in ("metric", "value", "unit", "n_gpus", "ms_per_step", "scaling") if k in line}
    out["frac_of_peak"] = line["roofline"]["frac"]
    out["peak"] = {"value": line["roofline"]["peak"], "unit": line["roofline"]["unit"], "kind": line["roofline"]["peak_kind"]}
    out["workload"] = line["config"]["workload"]
    if line["roofline"].get("other_mode"):
        out["other_mode"] = line["roofline"]["other_mode"]
    for k in keep:
        if k in line["config"]:
            out[k] = line["config"][k]
    if line.get("detail"):
        out["detail"] = line["detail"]
    out["e2e"] = line.get("e2e")
    out["clocks"] = line.get("clocks")
    return out


def run_gemv_workload(args) -> dict | None:
    import torch
    import torch.distributed as dist
    from zeninfer_b200 import Backend
    from zeninfer_b200.backend import ACT_INT8

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)

    be = Backend()  # raises if the CUDA library or a B200 is missing: there is no fallback
    packed, x_host = make_inputs()

    # --- resident inputs: COPIES weight shards on this rank, x and the outputs in HBM ---
    handles = [be.dev_upload("Q8_0", packed, ROWS, COLS) for _ in range(COPIES)]
    groups = [handles[g:g + GROUP] for g in range(0, COPIES, GROUP)]
    d_x = torch.from_numpy(x_host).to(dev)
    ys = torch.zeros((COPIES, ROWS), dtype=torch.float32, device=dev)
    y_ptrs = [ys[i].data_ptr() for i in range(COPIES)]
    d_all = torch.zeros((world, GROUP * ROWS), dtype=torch.float32, device=dev) if world > 1 else None
    stream = torch.cuda.Stream(device=dev)
    fused = world > 1 and args.gather == "fused"
    pg = None
    if fused:
        from zeninfer_b200.shard import PeerGather
        pg = PeerGather(be, world, rank, GROUP * ROWS)  # collective: IPC handles travel through torch.distributed, once

    def one_pass():
        for g, hs in enumerate(groups):
            outs = y_ptrs[g * GROUP:(g + 1) * GROUP]
            if fused:   # the product kernel stores its outputs into every rank's gather region and publishes the launch;
                        # the next launch waits on the device until all ranks have published: no collective launch
                pg.gemv(hs, d_x.data_ptr(), 1, ACT_INT8, stream.cuda_stream, d_y=outs)
                continue
            be.dev_gemv(hs, outs, d_x.data_ptr(), 1, ACT_INT8, stream.cuda_stream)
            if world > 1:
                dist.all_gather_into_tensor(d_all.view(-1), ys[g * GROUP:(g + 1) * GROUP].reshape(-1))

    passes = 1 if args.profile else PASSES_PER_STEP

    def time_passes(enqueue, steps, warm_steps, clocks=None):
        """Captures one pass, replays it `passes` times per step; returns the milliseconds of `steps` timed steps (max
        over ranks).  The replay counts are fixed, never time-based: every rank replays the same number of collectives."""
        with torch.cuda.stream(stream):
            enqueue()  # first launch sets function attributes; keep it out of the capture
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                enqueue()
            for n in range(warm_steps * passes):
                graph.replay()
                if n % 64 == 63:
                    stream.synchronize()
            stream.synchronize()
            be.dev_check(stream.cuda_stream)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if clocks:
                clocks.mark_start()
            e0.record(stream)
            for _ in range(steps * passes):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
            if clocks:
                clocks.mark_end()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            ms = e0.elapsed_time(e1)
        be.dev_check(stream.cuda_stream)
        del graph
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    with ClockSampler(local) as clocks:
        ms = time_passes(one_pass, args.steps, args.warmup, clocks)
    launches = args.steps * passes * len(groups)
    total_bytes = ALGO_BYTES_PER_GROUP * launches * world
    value = total_bytes / (ms * 1e-3) / 1e9
    per_launch_us = ms * 1e3 / launches
    achieved = ALGO_BYTES_PER_GROUP / (per_launch_us * 1e-6) / 1e9
    peak, peak_kind = peaks()

    # --- correctness of what was timed (not part of the timed region) ---
    y_dev = ys[0].cpu().numpy()
    assert bool((ys == ys[0][None, :]).all().item()), "the copies' products differ"
    if world > 1:
        if fused:
            pg.fetch(d_all.data_ptr(), stream.cuda_stream)
            stream.synchronize()
            be.dev_check(stream.cuda_stream)
        # every rank holds the same weights and input here, so every gathered shard must equal the local products
        assert bool((d_all.view(world, GROUP, ROWS) == ys[None, -GROUP:, :]).all().item()), "gathered shards differ from the local products"

    # --- the same 32 products submitted differently (one GPU): one tensor per launch, and all of them as one list launch ---
    variants = {"batch8": {"gbs": achieved, "us_per_product": per_launch_us / GROUP, "frac": achieved / peak, "launches_per_pass": len(groups),
                           "api": "zen_cuda_dev_gemv, eight tensors sharing the input per launch (zen::quant::gemv_batch); this is `value`"}}
    if args.profile:
        if pg is not None:
            stream.synchronize()
            pg.close()
        return {"metric": "q8_0_gemv_hbm_gbs", "profile_run": True, "value": value, "unit": "GB/s", "launch_us": per_launch_us,
                "launches": {"untimed": len(groups), "captured_replays": 2 * len(groups)}} if rank == 0 else None
    if world == 1:
        short = max(3, args.steps // 4)
        ys.zero_()

        def single_pass():   # each launch also asks L2 for the start of the tensor the next launch reads (a hint, no result changes)
            for i, h in enumerate(handles):
                be.dev_gemv_fused([h], [y_ptrs[i]], d_x.data_ptr(), 1, ACT_INT8, stream.cuda_stream, warm_next=handles[(i + 1) % COPIES])

        ms_s = time_passes(single_pass, short, 1)
        assert bool((ys == torch.from_numpy(y_dev).to(dev)[None, :]).all().item()), "single launches differ from batched launches"
        timed = [("single_launch", ms_s, COPIES, "zen_cuda_dev_gemv_fused, one tensor per launch, next tensor hinted to L2")]
        # The persistent list launch keeps state in device memory between its CTAs; a profiler that serialises or replays
        # kernels does not get along with it (an ncu launch list of this command stopped there), so it is left out under one.
        under_profiler = any(k in os.environ for k in ("CUDA_INJECTION64_PATH", "NV_COMPUTE_PROFILER_PERFWORKS_DIR", "NV_NSIGHT_INJECTION_PORT_BASE"))
        if not args.no_list and not under_profiler:
            ys.zero_()
            lst = be.gemv_list_create([dict(handles=[h], d_y=[y_ptrs[i]], d_x=d_x.data_ptr()) for i, h in enumerate(handles)], ACT_INT8)
            ms_l = time_passes(lambda: be.dev_gemv_list(lst, stream.cuda_stream), short, 1)
            assert bool((ys == torch.from_numpy(y_dev).to(dev)[None, :]).all().item()), "the list launch differs from batched launches"
            be.gemv_list_destroy(lst)
            timed.append(("list", ms_l, 1, "zen_cuda_dev_gemv_list, all 32 products as items of one persistent launch"))
        for name, ms_v, lp, api in timed:
            us = ms_v * 1e3 / (short * passes * COPIES)
            variants[name] = {"gbs": ALGO_BYTES_PER_LAUNCH / us / 1e3, "us_per_product": us, "frac": ALGO_BYTES_PER_LAUNCH / us / 1e3 / peak,
                              "launches_per_pass": lp, "api": api}

    # --- e2e: the host-pointer C-ABI call, host buffers, copies inside the timed region ---
    from zeninfer_b200.backend import GemvTask
    e2e_copies = [packed.copy() for _ in range(COPIES)]  # distinct host addresses => distinct resident tensors
    y_out = [np.empty(ROWS, np.float32) for _ in range(GROUP)]
    task_groups = [(GemvTask * GROUP)(*[GemvTask(w.ctypes.data, y.ctypes.data, ROWS, COLS) for w, y in zip(e2e_copies[g:g + GROUP], y_out)])
                   for g in range(0, COPIES, GROUP)]
    call = be.lib.zen_cuda_gemv_q8_0_batch    # the entry point a ZenInfer build binds for gemv_batch: host pointers in, host pointers out
    xp = x_host.ctypes.data
    for _ in range(3):                         # upload, warm, capture
        for tasks in task_groups:
            if not call(xp, tasks, GROUP):
                raise RuntimeError("zen_cuda_gemv_q8_0_batch failed: " + be.last_error())
    y_single = be.gemv("Q8_0", e2e_copies[0], x_host, ROWS, COLS)
    e2e_passes = max(30, min(args.steps * 15, 300))
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_passes):
        for tasks in task_groups:
            if not call(xp, tasks, GROUP):
                raise RuntimeError("zen_cuda_gemv_q8_0_batch failed: " + be.last_error())
    e2e_s = time.perf_counter() - t0
    # and one product per call (zen_cuda_gemv_q8_0), for the detail
    single_call, wp0, yp0 = be.lib.zen_cuda_gemv_q8_0, [w.ctypes.data for w in e2e_copies], y_out[0].ctypes.data
    for wp in wp0:
        single_call(wp, xp, yp0, ROWS, COLS)
    t1 = time.perf_counter()
    for _ in range(max(10, e2e_passes // 4)):
        for wp in wp0:
            if not single_call(wp, xp, yp0, ROWS, COLS):
                raise RuntimeError("zen_cuda_gemv_q8_0 failed: " + be.last_error())
    single_us = (time.perf_counter() - t1) * 1e6 / (max(10, e2e_passes // 4) * COPIES)
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = ALGO_BYTES_PER_GROUP * len(task_groups) * e2e_passes * world / e2e_s / 1e9
    assert np.array_equal(y_single, y_dev) and all(np.array_equal(y, y_dev) for y in y_out), "host-pointer and device-pointer paths disagree"
    variants["batch8"]["e2e_us_per_call"] = e2e_s * 1e6 / (e2e_passes * len(task_groups))
    if "single_launch" in variants:
        variants["single_launch"]["e2e_us_per_call"] = single_us
        variants["single_launch"]["e2e_gbs"] = ALGO_BYTES_PER_LAUNCH / single_us / 1e3
    for w in e2e_copies:
        be.release_weights(w)
    if pg is not None:
        stream.synchronize()
        pg.close()
    for h in handles:
        be.dev_free(h)
    if rank != 0:
        return None

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = cpu_reference_leg(packed, x_host, args.cpu_budget, 16)

    return {
        "metric": "q8_0_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": config0(),
        "notes": f"a step is {PASSES_PER_STEP} passes over {COPIES} weight copies ({COPIES * ALGO_BYTES_PER_LAUNCH / 1e6:.0f} MB per pass), CUDA graph replay, "
                 f"{len(groups)} launches of {GROUP} tensors per pass" + (
            "" if world == 1 else
            "; output shards all-gathered by the product kernel itself (peer stores over NVLink, device-side epoch flags)" if fused else "; NCCL all-gather of output shards after each launch"),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": GEMV_NCU_TRAFFIC_BYTES, "launch_us": per_launch_us, "algorithmic_bytes_per_launch": ALGO_BYTES_PER_GROUP,
                     "kernel": f"gemv_q8_0_kernel<1,1>, {GROUP} tensors of 4096 x 4096 per launch"},
        "cpu_baseline": cpu,
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": COLS * 4 * len(task_groups) * PASSES_PER_STEP, "d2h_bytes_per_step": ROWS * 4 * COPIES * PASSES_PER_STEP,
                "api": "zen_cuda_gemv_q8_0_batch (host pointers, eight tensors per call, weights resident by address)", "calls": e2e_passes * len(task_groups),
                "us_per_call": e2e_s * 1e6 / (e2e_passes * len(task_groups))},
        "gpu_launches": launches,
        "detail": {"config0_submission": variants},
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=DEFAULT_STEPS)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="q8_0_gemv")
    ap.add_argument("--cpu-budget", type=float, default=12.0, help="seconds of CPU time for the cpu_baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", action="store_true",
                    help="a short form of the workload for a profiler capture: one untimed pass, one captured-graph replay as warm-up and one "
                         "as the timed step, no end-to-end leg, no CPU baseline, no detail (its figures are not benchmark values)")
    ap.add_argument("--layers", type=int, default=0, help="workload decode: number of layers (default: the configuration's 32)")
    ap.add_argument("--formats", default="Q8_0,Q4_0,Q6_K,Q4_K,Q5_K", help="workloads layer_sweep and gemm_formats: formats to run")
    ap.add_argument("--act", default="int8", choices=["int8", "fp32"], help="workload q8_0_gemm: activation mode of the timed product (the other one is timed briefly beside it)")
    ap.add_argument("--no-list", action="store_true", help="default workload: skip the persistent list launch among the config 0 submission variants")
    ap.add_argument("--no-q6k-tensor", action="store_true", help="workload lm_head: batch 8 through the decode kernel (dp4a) instead of the tensor-core product")
    ap.add_argument("--no-detail", action="store_true", help="default workload: skip the short runs of the other workloads that fill `detail`")
    ap.add_argument("--device-pack", action="store_true", help="workload lm_head: draw and pack the Q6_K matrix on the GPU (torch) instead of numpy")
    ap.add_argument("--cut", default="rows+cols", choices=["rows", "rows+cols"],
                    help="workload decode, N > 1: every matrix by output rows (four gathers per layer), or o and down by columns "
                         "(two all-reduces per layer)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N > 1: how the output shards are all-gathered after each product -- by the product kernel itself "
                         "(peer stores over NVLink, the default) or by an NCCL all-gather launched after it")
    ap.add_argument("--fuse", default="nrp", help="workload decode: operators folded into the projection launches (letters n, s, r, p; see LlamaDecoder)")
    ap.add_argument("--token-prefill", action="store_true", help="workload decode: consume the prompt token by token instead of in tensor-core blocks")
    ap.add_argument("--prompt-len", type=int, default=512, help="workload decode: prompt tokens consumed before the timed steps")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl != "reference" else args.warmup
    if args.profile:
        args.no_detail = args.no_cpu_baseline = True
        args.steps, args.warmup = 1, 1

    if args.impl == "reference":
        run_reference_arm(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    runners = {"q8_0_gemm": run_gemm_workload, "layer_sweep": run_layer_sweep, "lm_head": run_lm_head, "decode": run_decode, "gemm_formats": run_gemm_formats}
    if args.workload in runners:
        line = runners[args.workload](args)
    elif args.workload == "q8_0_gemv":
        line = run_gemv_workload(args)
        if not args.no_detail:
            # the other terms of the headline metric, each by its own workload in a short form (all ranks take part in the
            # sharded ones; the prefill product is a one-GPU workload)
            detail = line["detail"] if line is not None else {}
            if world == 1:
                detail["q8_0_gemm"] = brief_detail(run_gemm_workload(args, brief=True), ())
            detail["lm_head"] = brief_detail(run_lm_head(args, brief=True), ("gather",))
            detail["decode"] = brief_detail(run_decode(args, brief=True), ("sharding", "prefill", "prefill_ms", "prefill_tokens_per_s", "launch"))
    else:
        raise SystemExit(f"unknown workload {args.workload!r}")
    if line is not None:
        print(json.dumps(line))
    if world > 1:
        # Multi-rank exit: meet once more, then leave without tearing NCCL down under live CUDA graphs (a
        # destroy_process_group here was seen to block for ever); all results are already out.
        import torch
        import torch.distributed as dist
        sys.stdout.flush()
        torch.cuda.synchronize()
        dist.barrier()
        os._exit(0)


if __name__ == "__main__":
    main()
