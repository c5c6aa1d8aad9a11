"""Benchmark of the grouped pointer-table combine (the MoE hot path's dominant kernel).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One step = one full combine of one synthetic batch through the public operator
`grouped_weighted_scatter_add(expert_tensors, indices, weights, out_shape)`:
plan build (inverse map, one cooperative launch) + token-major gather kernel, output
freshly produced. The default workload is the combine microbenchmark
(T=8192 tokens, D=16384, E=256 experts, top-8, bf16; 256 disjoint expert output
matrices, 2.15 GB of rows, which exceeds the 126 MB L2, so every step streams
from HBM).

Rank 0 prints ONE JSON line. Keys beyond the usual ones:
  value     whole-job GB/s of algorithmic bytes, inputs resident in HBM
  e2e       the same metric through the C-ABI host-buffer call fmoe_combine_host
            (pinned host inputs -> device -> combine -> host), copies timed
  roofline  the gather kernel alone: algorithmic bytes / its CUDA-event time,
            against the measured HBM copy bandwidth of this GPU pool
  cpu_baseline  the reference's own CPU path (the unmodified package, when
            oracle/install_ref.py has installed it; else its C port in oracle/),
            timed in this run on a stated sample of the same workload
  graph_replay  the form the reference's microbenchmark times (zero `out`, replay a
            CUDA graph of the call with prebuilt metadata), with and without the
            zero-fill; one GPU only, outside the headline timing
  also      the other single-GPU configurations, a few steps each, outside the
            headline timing: the skewed (Zipf) combine and the dispatch + combine
            chain under autograd, each with its own roofline entry
  ep_layer  the expert-parallel MoE layer at this world size, with a parity record
            (sampled tokens against an fp32 evaluation over all experts, forward
            and token gradients, and the device status word)

With --gpus N > 1 (under torchrun) every rank runs an independent replica of the
combine workload: the combine has no cross-GPU step ("replicas only"); the aggregate
is the sum over ranks divided by the slowest rank's time. The expert-parallel layer
in `ep_layer` is the part that shards (experts over ranks, tokens exchanged).

`--impl reference` times the reference's CPU implementation of the path on the box's
host cores, same workload, same metric, inputs built on the host.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "combine_hbm_gbs"
UNIT = "GB/s"

WORKLOADS = {
    # name: (T, D, E, K, routing)
    "combine_cfg2_bf16_T8192_D16384_E256_top8": (8192, 16384, 256, 8, "softmax"),
    "combine_cfg3_zipf_bf16_T8192_D16384_E256_top8": (8192, 16384, 256, 8, "zipf"),
    # a quarter of the tokens of cfg2, same row width: the size used for ncu captures
    "combine_ncu_bf16_T2048_D16384_E256_top8": (2048, 16384, 256, 8, "softmax"),
    "combine_small_bf16_T1024_D4096_E64_top8": (1024, 4096, 64, 8, "softmax"),
    # the reference's own microbenchmark preset ("GIGACHAT_700B": B=2, S=2048, D=16384, E=256,
    # top-4, fp32 tensors, random targets), the shape behind its published 2.61 ms on an H100
    "combine_reference_preset_fp32_T4096_D16384_E256_top4": (4096, 16384, 256, 4, "random_targets"),
}
DEFAULT_WORKLOAD = "combine_cfg2_bf16_T8192_D16384_E256_top8"
# dispatch permute + combine, forward and backward under autograd: (T, D, E, K)
CFG4 = {
    "dispatch_combine_cfg4_bf16_T16384_D7168_E256_top8": (16384, 7168, 256, 8),
    # a quarter of the tokens: the size used for ncu captures
    "dispatch_combine_ncu_bf16_T4096_D7168_E256_top8": (4096, 7168, 256, 8),
}
# expert FFN alone (two grouped GEMMs, SwiGLU fused): (experts, rows, D, ff)
GEMM = {
    "grouped_swiglu_ffn_E32_R65536_D7168_ff2048": (32, 65536, 7168, 2048),  # one rank of 8
    "grouped_swiglu_ffn_E256_R65536_D7168_ff2048": (256, 65536, 7168, 2048),  # a single rank
    "grouped_swiglu_ffn_ncu_E8_R8192_D7168_ff2048": (8, 8192, 7168, 2048),  # small case for ncu
    "grouped_swiglu_ffn_ncu_E32_R8192_D7168_ff2048": (32, 8192, 7168, 2048),  # 256 rows per expert, for ncu
}

# DRAM bytes (read + write) of one gather launch on the default workload: an ncu capture
# (dram__bytes_read.sum + dram__bytes_write.sum) of the quarter-size case, scaled by its
# 4x tokens; traffic grows in proportion to tokens.
NCU_TRAFFIC_BYTES = {DEFAULT_WORKLOAD: 4 * (537_092_352 + 45_110_528)}

FALLBACK_HBM_GBS = 6650.0


def measured_tflops():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["bf16_tflops_sustained"]), "measured (sustained)"
        except Exception:
            pass
    return 1400.0, "fallback"


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {
            "sm_mhz": statistics.median(self.samples),
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def host_copy(wl):
    """Pinned host copies of the workload (bf16 rows as uint16 bit patterns for numpy)."""
    import torch

    pin = torch.cuda.is_available()
    experts = [torch.empty(e.shape, dtype=e.dtype, pin_memory=pin) for e in wl.experts]
    for h, d in zip(experts, wl.experts):
        h.copy_(d)
    idx = wl.indices.cpu()
    w = wl.weights.cpu()
    if pin:
        idx, w = idx.pin_memory(), w.pin_memory()
        torch.cuda.synchronize()
    return experts, idx, w


def host_threads():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def cpu_pass_port(host, T, D):
    """One combine on the host cores with the reference's CPU arithmetic for the tensors' dtype
    (oracle port: bf16 product and per-call fp32 accumulation for bf16, plain fp32 otherwise)."""
    import numpy as np
    import torch

    import oracle

    experts, idx, w = host
    oracle.use_all_cores()
    if experts[0].dtype == torch.float32:
        ex = [e.numpy() for e in experts]
        t0 = time.perf_counter()
        oracle.combine(ex, idx.numpy(), w.numpy(), T)
        return time.perf_counter() - t0
    ex = [e.view(torch.int16).numpy().view(np.uint16) for e in experts]
    t0 = time.perf_counter()
    oracle.combine_bf16(ex, idx.numpy(), w.view(torch.int16).numpy().view(np.uint16), T)
    return time.perf_counter() - t0


class CpuArm:
    """The reference's CPU path on this box's host cores, on a bounded sample of a combine
    workload: the rows of the first `n_experts` expert matrices (all T output rows). It starts
    from a quarter of the experts and takes the whole workload when a timed trial pass says that
    a full pass stays under two seconds. kind "reference" runs the unmodified package's
    `grouped_weighted_scatter_add` on CPU tensors (src/fastmoe/kernels/ops.py:373-384, torch's
    own thread pool); kind "port" runs the C/OpenMP restatement of it when the package is not
    installed on this machine."""

    def __init__(self, host, T, D, force_port=False):
        import torch

        import oracle

        self.host, self.T, self.D = host, T, D
        self.ref = None if force_port else oracle.reference_ops()
        experts, idx, w = host
        self.kind = "port" if self.ref is None else "reference"
        if self.ref is not None:
            torch.set_num_threads(host_threads())
            self.cores = torch.get_num_threads()
        else:
            self.cores = oracle.use_all_cores()
        E = len(experts)
        self._take(max(1, E // 4))
        trial = self.one_pass()
        if trial * E / self.n_experts <= 2.0:
            self._take(E)

    def _take(self, n_experts):
        experts, idx, w = self.host
        self.n_experts = n_experts
        self.rows = sum(int(e.shape[0]) for e in experts[:n_experts])
        es = experts[0].element_size()
        self.bytes = (self.rows * self.D * es + self.T * self.D * es
                      + self.rows * (idx.element_size() + w.element_size()) + n_experts * 20)  # fmt: skip

    def one_pass(self):
        experts, idx, w = self.host
        sub = (experts[: self.n_experts], idx[: self.rows], w[: self.rows])
        if self.ref is None:
            return cpu_pass_port(sub, self.T, self.D)
        t0 = time.perf_counter()
        self.ref.grouped_weighted_scatter_add(sub[0], sub[1], sub[2], (self.T, self.D))
        return time.perf_counter() - t0

    def describe(self):
        what = ("the unmodified reference package's CPU path (torch index_add_ per expert)" if self.ref is not None
                else "C/OpenMP port of the reference's CPU path")  # fmt: skip
        return (f"{what} on the rows of the first {self.n_experts} of {len(self.host[0])} expert matrices "
                f"({self.rows} rows into all {self.T} output rows); GB/s counts that sample's algorithmic bytes")  # fmt: skip


# The reference publishes one number for this path: 2.61 ms for its grouped kernel on an H100
# at its own preset (README.md:88). In this bench's unit that is the preset's algorithmic
# bytes over 2.61 ms.
PUBLISHED_MS = {"combine_reference_preset_fp32_T4096_D16384_E256_top4": 2.61}


def workload_config(name):
    T, D, E, K, routing = WORKLOADS[name]
    return {"workload": name, "T": T, "D": D, "E": E, "top_k": K, "routing": routing}


def run_reference(args, rank):
    """The reference arm: the reference's CPU path on this box's host cores, inputs built on the host."""
    if rank != 0:
        return
    import torch

    from fastmoe_b200.workloads import make_combine_workload

    T, D, E, K, routing = WORKLOADS[args.workload]
    dtype = torch.float32 if "_fp32_" in args.workload else torch.bfloat16
    wl = make_combine_workload(T, D, E, K, dtype, routing, seed=0, device="cpu")
    arm = CpuArm((wl.experts, wl.indices, wl.weights), T, D, force_port=args.cpu_port)
    for _ in range(args.warmup):
        arm.one_pass()
    t = [arm.one_pass() for _ in range(args.steps)]
    total = sum(t)
    value = arm.bytes * args.steps / total / 1e9
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "bf16",
        "data": "synthetic",
        "config": workload_config(args.workload),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": arm.cores, "kind": arm.kind, "sample": arm.describe()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def bind_to_gpu_cores(index):
    """Restricts this process to the host cores NVML reports as local to GPU `index`, so that the
    pinned staging buffers allocated afterwards come from that GPU's memory node. Returns the
    number of cores, or None when NVML or the affinity call is not available."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cores = {64 * i + b for i, word in enumerate(mask) for b in range(64) if (word >> b) & 1}
        cores &= os.sched_getaffinity(0)
        if cores:
            os.sched_setaffinity(0, cores)
            return len(cores)
    except Exception:
        pass
    return None


def combine_record(name, rank, world, device, steps, warmup, keep=False):
    """Times `steps` combines of workload `name` through the public operator. Returns a dict
    (elapsed_ms over the steps, per-launch kernel and plan times, host enqueue time, ...) and,
    with keep=True, the workload and the last output for the callers that go on with them."""
    import torch
    import torch.distributed as dist

    from fastmoe_b200.kernels import ops
    from fastmoe_b200.workloads import make_combine_workload

    T, D, E, K, routing = WORKLOADS[name]
    dtype = torch.float32 if "_fp32_" in name else torch.bfloat16
    wl = make_combine_workload(T, D, E, K, dtype, routing, seed=rank, device=device)
    nbytes = wl.algorithmic_bytes()
    shape = (T, D)

    def step():
        return ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, shape)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        out = step()
    barrier()
    launches0 = ops.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device.index) as clocks:
        # the timed region: `steps` calls back to back, nothing else on the stream
        barrier()
        start.record()
        t0 = time.perf_counter()
        for _ in range(steps):
            out = step()
        host_s = time.perf_counter() - t0  # time to ENQUEUE the steps: the host's share
        end.record()
        barrier()
        elapsed_ms = start.elapsed_time(end)
        launches = ops.launch_count - launches0
        # the same steps once more with a pair of CUDA events around every launch, for the
        # per-kernel durations: four event records per step between the kernels cost about
        # 20 us a step, which is why the headline pass above runs without them
        ops.kernel_events = {}  # entry point -> (start, end) events, on the launching stream
        start.record()
        for _ in range(steps):
            out = step()
        end.record()
        barrier()
    instrumented_ms = start.elapsed_time(end)
    gather_ms = [s.elapsed_time(e) for s, e in ops.kernel_events.get("fmoe_combine_gather", [])]
    plan_ms = [s.elapsed_time(e) for s, e in ops.kernel_events.get("fmoe_combine_plan", [])]
    ops.kernel_events = None
    assert ops.read_status(device) == 0, "kernels flagged skipped rows"
    assert float(out.float().abs().mean()) > 0.0
    rec = {
        "elapsed_ms": elapsed_ms, "bytes": nbytes, "launches": launches, "clocks": clocks.summary(),
        "kernel_ms": statistics.mean(gather_ms) if gather_ms else None,
        "plan_ms": statistics.mean(plan_ms) if plan_ms else None,
        "instrumented_ms_per_step": instrumented_ms / steps,
        "host_enqueue_ms_per_step": host_s / steps * 1e3, "rows": wl.N, "max_rows_per_expert": max(wl.counts),
    }  # fmt: skip
    return (rec, wl, out) if keep else (rec, None, None)


def graph_replay_record(wl, shape, steps):
    """The combine as the reference's microbenchmark times it (run_on_cloud.py:64-91): metadata
    built once, the call with `out=` and `metadata=` captured in a CUDA graph, every step zeroes
    `out` and replays. The call ADDS into `out`, so against the headline form (a fresh result)
    each step also writes the zeros and reads them back: T*D*s more bytes each way
    (`extra_bytes_per_step`), which `value` does not count."""
    import torch

    from fastmoe_b200.kernels import ops

    out = torch.zeros(shape, device=wl.indices.device, dtype=wl.experts[0].dtype)
    metadata = ops.prepare_grouped_metadata(wl.experts, out.device)

    def launch():
        ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, shape, out=out, metadata=metadata)

    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    out.zero_()
    with torch.cuda.graph(graph):
        launch()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for with_zero in (True, False):  # the second pass leaves the zero-fill out and keeps adding
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            if with_zero:
                out.zero_()
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        if with_zero:
            ms_zero = start.elapsed_time(end) / steps
            fresh = ops.grouped_weighted_scatter_add(wl.experts, wl.indices, wl.weights, shape)
            assert torch.equal(out, fresh), "graph replay into a zeroed output differs from the plain call"
            del fresh
        else:
            ms_plain = start.elapsed_time(end) / steps
    nbytes = wl.algorithmic_bytes()
    return {
        "form": "out.zero_() + replay of a CUDA graph of grouped_weighted_scatter_add(out=, metadata=)",
        "steps": steps, "ms_per_step": ms_zero, "value": nbytes / (ms_zero / 1e3) / 1e9, "unit": UNIT,
        "ms_per_step_without_zero_fill": ms_plain, "value_without_zero_fill": nbytes / (ms_plain / 1e3) / 1e9,
        "extra_bytes_per_step": 2 * out.numel() * out.element_size(),
    }  # fmt: skip


def roofline_of(rec, name):
    peak, peak_kind = measured_peak()
    achieved = rec["bytes"] / (rec["kernel_ms"] / 1e3) / 1e9 if rec["kernel_ms"] else None
    return {
        "bound": "hbm",
        "kernel": "gather_sum_kernel (combine forward)",
        "achieved": achieved,
        "peak": peak,
        "peak_kind": peak_kind,
        "unit": "GB/s",
        "frac": achieved / peak if achieved else None,
        "frac_of_8TBs_spec": achieved / 8000.0 if achieved else None,
        "kernel_ms": rec["kernel_ms"],
        "algorithmic_bytes": rec["bytes"],
        "traffic": NCU_TRAFFIC_BYTES.get(name),
        "plan_build_ms": rec["plan_ms"],
        "measured_in": "a second pass of the same steps with CUDA events around every launch "
                       "(%.4f ms per step with the events, the headline pass runs without them)"
                       % rec["instrumented_ms_per_step"],
    }


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    from fastmoe_b200 import _lib
    from fastmoe_b200.kernels import ops

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _lib.lib()  # fail now if the CUDA library is missing
    local_cores = bind_to_gpu_cores(local_rank) if world > 1 else None

    T, D, E, K, routing = WORKLOADS[args.workload]
    dtype = torch.float32 if "_fp32_" in args.workload else torch.bfloat16
    rec, wl, out = combine_record(args.workload, rank, world, device, args.steps, args.warmup, keep=True)
    nbytes, elapsed_ms = rec["bytes"], rec["elapsed_ms"]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the reference's own timing form: zero `out`, replay a CUDA graph of the call with
    # prebuilt metadata (run_on_cloud.py:64-91); at N=1, outside the headline timing ------
    graph_rec = None
    if world == 1 and not args.no_also:
        graph_rec = graph_replay_record(wl, (T, D), max(3, min(args.steps, 20)))

    # ---- end to end through the C ABI with host buffers ----------------------------
    host = host_copy(wl)
    hex_, hidx, hw = host
    import ctypes

    lib = _lib.lib()
    sizes = (ctypes.c_int64 * E)(*wl.counts)
    ptrs = (ctypes.c_void_p * E)(*[h.data_ptr() for h in hex_])
    fm_dtype = _lib.FMOE_F32 if dtype == torch.float32 else _lib.FMOE_BF16
    arena_bytes = lib.fmoe_combine_host_arena_bytes(sizes, E, wl.N, T, D, fm_dtype)
    arena = torch.empty(arena_bytes, dtype=torch.uint8, device=device)
    out_host = torch.empty(T, D, dtype=dtype).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream
    h2d = sum(h.numel() * h.element_size() for h in hex_) + hidx.numel() * 8 + hw.numel() * hw.element_size()
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        _lib.call("fmoe_combine_host", ptrs, sizes, hidx.data_ptr(), _lib.FMOE_I64, hw.data_ptr(),
                  fm_dtype, out_host.data_ptr(), E, wl.N, T, D, fm_dtype,
                  arena.data_ptr(), arena_bytes, stream)  # fmt: skip

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()  # returns after its stream has drained
    barrier()
    e2e_s = time.perf_counter() - t0
    if ops.combine_mode() == "gather":  # the same kernels in the same order: identical bits
        assert torch.equal(out_host.to(device), out), "host-buffer call and device call disagree"
    else:  # the scatter form adds in bf16, in arrival order: equal within the bf16 bound only
        ref = out_host.to(device).float()
        assert float((out.float() - ref).abs().max() / ref.abs().max()) <= 2e-2

    # ---- aggregate over ranks -------------------------------------------------------
    stats = torch.tensor([elapsed_ms, e2e_s], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_s = stats.tolist()
    value = nbytes * world * args.steps / (elapsed_ms / 1e3) / 1e9
    e2e_value = nbytes * world * e2e_steps / e2e_s / 1e9
    n_rows = wl.N
    del wl, out, arena, out_host
    torch.cuda.empty_cache()

    # CPU baseline on rank 0 at N=1 only: a few passes of the bounded sample
    cpu_baseline = None
    if rank == 0 and world == 1:
        arm = CpuArm(host, T, D, force_port=args.cpu_port)
        arm.one_pass()
        cpu_t = [arm.one_pass() for _ in range(3)]
        cpu_baseline = {
            "value": arm.bytes / statistics.median(cpu_t) / 1e9, "unit": UNIT, "cores": arm.cores, "kind": arm.kind,
            "sample": arm.describe() + "; median of 3 passes after 1 warm-up", "ms": statistics.median(cpu_t) * 1e3,
        }  # fmt: skip
        if arm.kind == "reference":  # the C port of the same path beside it, on the whole workload
            import oracle

            cpu_pass_port(host, T, D)
            port_s = statistics.median(cpu_pass_port(host, T, D) for _ in range(3))
            cpu_baseline["port"] = {"value": nbytes / port_s / 1e9, "unit": UNIT, "cores": oracle.num_threads(),
                                    "ms": port_s * 1e3, "sample": "C/OpenMP port, the full workload"}  # fmt: skip
    del host, hex_, hidx, hw

    # ---- the other single-GPU configurations, outside the headline timing -------------
    also = None
    if args.workload == DEFAULT_WORKLOAD and world == 1 and not args.no_also:
        sub_steps = max(3, min(args.steps, 10))
        r3, _, _ = combine_record("combine_cfg3_zipf_bf16_T8192_D16384_E256_top8", rank, world, device, sub_steps, 3)
        also = {"combine_cfg3": {
            "config": workload_config("combine_cfg3_zipf_bf16_T8192_D16384_E256_top8"),
            "value": r3["bytes"] * sub_steps / (r3["elapsed_ms"] / 1e3) / 1e9, "unit": UNIT,
            "ms_per_step": r3["elapsed_ms"] / sub_steps, "steps": sub_steps, "max_rows_per_expert": r3["max_rows_per_expert"],
            "roofline": roofline_of(r3, "combine_cfg3_zipf_bf16_T8192_D16384_E256_top8"),
        }}  # fmt: skip
        torch.cuda.empty_cache()
        also["dispatch_combine_cfg4"] = cfg4_record("dispatch_combine_cfg4_bf16_T16384_D7168_E256_top8", rank, world,
                                                    local_rank, sub_steps, 3, cpu=False)  # fmt: skip
        torch.cuda.empty_cache()

    # second part of the headline metric: the expert-parallel MoE layer at this world size
    ep = None
    if args.workload == DEFAULT_WORKLOAD and not args.no_ep:
        ep = ep_layer_bench(rank, world, local_rank, min(args.steps, 20), min(args.warmup, 5), None, args.ep_mode)

    if rank != 0:
        return

    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": elapsed_ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (value / (nbytes / (PUBLISHED_MS[args.workload] / 1e3) / 1e9)
                        if args.workload in PUBLISHED_MS and world == 1 else None),
        "dtype": "f32" if dtype == torch.float32 else "bf16",
        "data": "synthetic",
        "config": workload_config(args.workload),
        "notes": {
            "rows": n_rows, "l2": "inputs (%.2f GB) exceed the 126 MB L2; no flush needed" % (nbytes / 1e9),
            "multi_gpu": "replicas only (the combine has no cross-GPU step; ep_layer is the sharded part)",
            "host_enqueue_ms_per_step": rec["host_enqueue_ms_per_step"],
            "pinned_buffers": (f"allocated after binding the rank to its GPU's {local_cores} local cores"
                               if local_cores else "allocated with the process's default affinity"),
        },
        "graph_replay": graph_rec,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "call": "fmoe_combine_host (C ABI, pinned host buffers)"},
        "gpu_launches": rec["launches"],
        "roofline": roofline_of(rec, args.workload),
        "cpu_baseline": cpu_baseline,
        "clocks": rec["clocks"],
        "also": also,
        "ep_layer": ep,
    }  # fmt: skip
    print(json.dumps(line), flush=True)
    fail_on_parity(ep)


EP_WORKLOAD = "ep_moe_layer_cfg5_bf16_8192tok_D7168_E256_top8_swiglu2048"


def ep_layer_bench(rank, world, local_rank, steps, warmup, micro_batches=None, mode="fused", expert_groups=None):
    """Expert-parallel MoE layer forward: 8192 tokens per rank, D=7168, 256 experts sharded
    evenly over the ranks, top-8 softmax router, SwiGLU experts 7168->2048->7168, weights
    N(0, 0.02). Micro-batches run on their own streams, the exchange of one overlapping the
    experts of another. Every micro-batch streams the rank's expert weights from HBM once
    more (22.5 GB / world each time) and thins the rows per expert: measured, the grouped
    GEMMs for 65536 rows take 4.52 / 4.66 / 5.51 ms in 1 / 2 / 4 launches at 32 experts per
    rank and 5.08 / 5.43 / 5.91 ms at 64, and at 2 and 4 ranks one micro-batch was fastest
    (2 ranks: 8.7 ms against 10.2 ms with two; 8 ranks: 8.5 ms against 9.0 ms). The default is
    therefore 1 micro-batch; --micro-batches overrides it (the configuration's nominal value
    is 4). Returns tokens/s over all ranks (max time over ranks)."""
    import torch
    import torch.distributed as dist

    from fastmoe_b200.consts import MoEImplementation
    from fastmoe_b200.models.tiny_model import MoEFeedForward, pipelined_moe_forward

    dev = torch.device("cuda", local_rank)
    T, D, FF, E, K = 8192, 7168, 2048, 256, 8
    MB = micro_batches or 1
    with torch.device(dev):
        moe = MoEFeedForward(D, FF, E, K, MoEImplementation.FAST, expert_type="swiglu")
    moe = moe.to(torch.bfloat16)
    e_local = moe.num_local_experts
    gen = torch.Generator(device=dev)
    with torch.no_grad():
        gen.manual_seed(0)
        moe.router.weight.normal_(0, 0.02, generator=gen)
        for e in range(e_local):  # seeded by the GLOBAL expert id: the same experts at every world size
            gen.manual_seed(1000 + rank * e_local + e)
            moe.experts.w_gate_up[e].normal_(0, 0.02, generator=gen)
            moe.experts.w_down[e].normal_(0, 0.02, generator=gen)
        gen.manual_seed(100 + rank)
        x = torch.randn(T, D, generator=gen, device=dev, dtype=torch.bfloat16)
    chunks = [c.view(1, T // MB, D) for c in x.chunk(MB, 0)]
    streams = [torch.cuda.Stream(device=dev) for _ in range(MB)]
    main = torch.cuda.current_stream()

    # With several ranks the default is the fused exchange: dispatch by peer stores from the
    # permute kernel, return trip in the down-projection's epilogue, no payload collective and
    # no host synchronisation (fastmoe_b200/ep_fused.py). "nccl" selects the all-to-all path.
    fused, ep_mode = None, "single rank"
    if world > 1:
        ep_mode = "nccl all_to_all"
        if mode == "fused":
            try:
                from fastmoe_b200.ep_fused import FusedExpertParallel

                fused = FusedExpertParallel(moe, max_tokens=T, expert_groups=expert_groups)
                if os.environ.get("FASTMOE_B200_EP_STAGGER") is not None:  # A/B switch for measurements
                    fused.stagger_copies = os.environ["FASTMOE_B200_EP_STAGGER"] != "0"
                ep_mode = "fused peer stores"
            except Exception as exc:  # symmetric memory unavailable: every rank falls back alike
                ep_mode = f"nccl all_to_all (fused path unavailable: {type(exc).__name__})"
        ok = torch.tensor([1 if fused is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            fused = None

    def step():
        if fused is not None:
            return [fused(x.view(1, T, D))]
        for s in streams:
            s.wait_stream(main)
        with torch.no_grad():
            outs = pipelined_moe_forward(moe, chunks, streams)
        for s in streams:
            main.wait_stream(s)
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        outs = step()
    barrier()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        outs = step()
    end.record()
    barrier()
    ms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms[0]) / steps
    assert all(bool(torch.isfinite(o.float()).all()) for o in outs)
    y_fwd = torch.cat([o.reshape(-1, D) for o in outs], 0)  # [T, D], this rank's tokens in order

    # the same layer as a training step: forward + backward (tokens, router and expert gradients)
    xt = x.view(1, T, D)
    gy = torch.randn(1, T, D, generator=gen, device=dev, dtype=torch.bfloat16)

    def train_step():
        for prm in moe.parameters():
            prm.grad = None
        xi = xt.detach().requires_grad_(True)
        y = fused.forward_with_grad(xi) if fused is not None else moe(xi)
        y.backward(gy)
        return xi.grad

    train_steps = max(2, min(steps, 5))
    train_step()
    barrier()
    start.record()
    for _ in range(train_steps):
        gx = train_step()
    end.record()
    barrier()
    tms = torch.tensor([start.elapsed_time(end)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    train_ms = float(tms[0]) / train_steps
    assert bool(torch.isfinite(gx.float()).all())
    parity = ep_parity(moe, x, y_fwd, gx.reshape(T, D), gy.reshape(T, D), rank, world, dev, FF)
    del gx, gy, y_fwd
    cpu_baseline = None
    if rank == 0:  # CPU baseline: the expert FFN of a 256-token sample through torch's CPU matmul
        import os

        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        torch.set_num_threads(cores)
        Ts, Es = 256, 8  # 256 tokens x top-8 = 2048 routed rows, spread over 8 experts
        g = torch.Generator().manual_seed(0)
        xs = torch.randn(Ts * K, D, generator=g)
        wgu = torch.empty(Es, 2 * FF, D).normal_(0, 0.02, generator=g)
        wd = torch.empty(Es, D, FF).normal_(0, 0.02, generator=g)
        t0 = time.perf_counter()
        with torch.no_grad():
            for e, chunk in enumerate(xs.chunk(Es, 0)):
                h = chunk @ wgu[e].t()
                (torch.nn.functional.silu(h[:, :FF]) * h[:, FF:]) @ wd[e].t()
        cpu_s = time.perf_counter() - t0
        cpu_baseline = {"value": Ts / cpu_s, "unit": "tokens/s", "cores": cores, "kind": "port", "ms": cpu_s * 1e3,
                        "sample": "expert FFN only (the dominant cost) for 256 tokens x top-8 = 2048 routed rows "
                                  "over 8 experts, fp32 torch CPU matmul"}  # fmt: skip
        del xs, wgu, wd
    gemm_flops = 6 * T * K * D * FF  # per rank and step: three D x FF products per routed row
    a2a_bytes = T * K * D * 2 * (world - 1) / world  # leaving each GPU, per direction
    groups = fused.expert_groups if fused is not None else 1
    del moe, fused
    torch.cuda.empty_cache()
    return {
        "tokens_per_s": T * world / (ms / 1e3),
        "ms_per_step": ms,
        "tokens_per_rank": T, "micro_batches": MB, "pass": "forward",
        "expert_groups": groups,
        "overlap": ("dispatch of expert group g+1 (peer stores, side stream) runs beside the grouped GEMMs of "
                    "group g; results return from the down-projection's epilogue" if groups > 1 else "none"),
        "parity": parity,
        "train_tokens_per_s": T * world / (train_ms / 1e3), "train_ms_per_step": train_ms,
        "train_pass": "forward + backward (tokens, router, expert weights), no optimizer",
        "gemm_tflops_per_gpu": gemm_flops / (ms / 1e3) / 1e12,
        "gemm_flops_per_rank": gemm_flops,
        "a2a_bytes_out_per_rank_per_direction": a2a_bytes,
        "experts_per_rank": e_local,
        "exchange": ep_mode,
        "cpu_baseline": cpu_baseline,
        "config": {"D": D, "ff": FF, "E": E, "top_k": K, "experts": "swiglu", "weights": "N(0,0.02) seeded per expert"},
    }  # fmt: skip


def ep_parity(moe, x, y, gx, gy, rank, world, dev, FF, sample=128):
    """Checks what the timed layer computed, on every rank: `sample` of this rank's tokens are
    evaluated again in fp32 over ALL experts (any rank can regenerate any expert from its
    global-id seed), forward and token gradient (through the experts and through the router),
    and compared with the layer's output `y` and the training step's `gx` for upstream gradient
    `gy`. The ground truth is the single-rank layer over all experts
    (MoEFeedForward.forward, src/fastmoe/models/tiny_model.py:411-420, with SwiGLU experts).
    Returns relative errors (largest over ranks) and the device status word; raises if any is
    out of bounds."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F

    from fastmoe_b200.kernels import ops, routing

    T, D = x.shape
    K, E, el = moe.top_k, moe.num_experts, moe.num_local_experts
    status = ops.read_status(dev, reset=False)
    with torch.no_grad():
        _, idx_all = routing.route_topk(moe.router(x), K, w_dtype=x.dtype)  # the layer's routing decision
    pick = torch.randperm(T, generator=torch.Generator(device=dev).manual_seed(4242 + rank), device=dev)[:sample]
    idx = idx_all[pick]
    xs = x[pick].float().requires_grad_(True)
    gate = torch.softmax(torch.gather(xs @ moe.router.weight.detach().float().t(), 1, idx), dim=-1)
    gen = torch.Generator(device=dev)
    ref = torch.zeros(sample, D, device=dev)
    for e in torch.unique(idx).tolist():
        gen.manual_seed(1000 + e)
        wgu = torch.empty(2 * FF, D, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        wd = torch.empty(D, FF, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        if rank * el <= e < (rank + 1) * el:  # regenerated weights must be the ones the layer holds
            assert torch.equal(wgu, moe.experts.w_gate_up[e - rank * el]) and torch.equal(wd, moe.experts.w_down[e - rank * el])
        rows, ks = (idx == e).nonzero(as_tuple=True)
        h = xs[rows] @ wgu.float().t()
        act = (F.silu(h[:, :FF]) * h[:, FF:])
        act = act + (act.bfloat16().float() - act).detach()  # the layer rounds the activations to bf16 once
        ref = ref.index_add(0, rows, (act @ wd.float().t()) * gate[rows, ks][:, None])
        del wgu, wd
    (ref * gy[pick].float()).sum().backward()
    fwd_err = float((y[pick].float() - ref.detach()).abs().max() / ref.detach().abs().max())
    dx_err = float((gx[pick].float() - xs.grad).abs().max() / xs.grad.abs().max())
    errs = torch.tensor([fwd_err, dx_err, float(status)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    fwd_err, dx_err, status = float(errs[0]), float(errs[1]), int(errs[2])
    ops.read_status(dev)  # clear
    ok = status == 0 and fwd_err <= 2e-2 and dx_err <= 2e-2
    return {"fwd_rel_err": fwd_err, "dx_rel_err": dx_err, "status": status, "ok": ok,
            "sample": f"{sample} tokens per rank", "bound": 2e-2,
            "against": "fp32 evaluation over all experts of the same bf16 values"}  # fmt: skip


def fail_on_parity(ep):
    """Called after the JSON line is out: a run whose expert-parallel layer computed the wrong
    thing (or dropped rows, or gave up a wait) ends with a non-zero exit code and says why."""
    if ep is not None and not ep["parity"]["ok"]:
        raise SystemExit(f"bench.py: expert-parallel layer failed its parity check: {ep['parity']}")


def run_ep(args, rank, world, local_rank):
    import torch

    torch.cuda.set_device(local_rank)
    if args.gemm_sms:
        from fastmoe_b200 import _lib

        _lib.tune("gemm_sms", args.gemm_sms)
    r = ep_layer_bench(rank, world, local_rank, args.steps, args.warmup, args.micro_batches, args.ep_mode,
                       args.ep_groups)
    if rank != 0:
        return
    peak, kind = measured_tflops()
    line = {
        "metric": "ep_moe_layer_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": EP_WORKLOAD, **r["config"], "tokens_per_rank": r["tokens_per_rank"],
                   "micro_batches": r["micro_batches"], "expert_groups": r["expert_groups"],
                   "parallelism": f"ep{world}", "pass": "forward"},
        "e2e": None, "gpu_launches": None,
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (share of the whole layer step)",
                     "achieved": r["gemm_tflops_per_gpu"], "peak": peak, "peak_kind": kind, "unit": "TFLOP/s",
                     "frac": r["gemm_tflops_per_gpu"] / peak, "traffic": None},
        "ep_layer": r,
    }  # fmt: skip
    print(json.dumps(line), flush=True)
    fail_on_parity(r)


def run_gemm(args, rank, world, local_rank):
    """The expert FFN as two grouped GEMM launches (gate/up with fused SwiGLU, then down)."""
    import torch

    from fastmoe_b200.kernels import experts, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    E, R, D, FF = GEMM[args.workload]
    gen = torch.Generator(device=dev).manual_seed(rank)
    cnt = torch.full((E,), R // E, dtype=torch.int64, device=dev)
    jitter = torch.randint(-(R // E // 8), R // E // 8 + 1, (E // 2,), generator=gen, device=dev)
    cnt[: E // 2] += jitter
    cnt[E // 2 :] -= jitter  # ragged, same total
    off = torch.cumsum(cnt, 0) - cnt
    x = torch.randn(R, D, generator=gen, device=dev, dtype=torch.bfloat16)
    wgu = torch.empty(E, 2 * FF, D, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
    wd = torch.empty(E, D, FF, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
    flops = 6 * R * D * FF

    def step():
        with torch.no_grad():
            return experts.grouped_swiglu_ffn(x, wgu, wd, off, cnt, covers_all_rows=True)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    ops.kernel_events = {}
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record()
        for _ in range(args.steps):
            y = step()
        end.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(end) / args.steps
    pairs = ops.kernel_events.get("fmoe_grouped_gemm", [])
    ops.kernel_events = None
    each = [a.elapsed_time(b) for a, b in pairs]
    gate_up_ms, down_ms = statistics.mean(each[0::2]), statistics.mean(each[1::2])
    assert ops.read_status(dev) == 0 and bool(torch.isfinite(y.float()).all())

    # forward + backward (data and weight gradients on the same kernels), fewer steps
    xg, wgu_g, wd_g = x.clone().requires_grad_(True), wgu.requires_grad_(True), wd.requires_grad_(True)
    gy = torch.randn(R, D, generator=gen, device=dev, dtype=torch.bfloat16)

    def train_step():
        xg.grad = wgu_g.grad = wd_g.grad = None
        experts.grouped_swiglu_ffn(xg, wgu_g, wd_g, off, cnt, covers_all_rows=True).backward(gy)

    fb_steps = max(2, min(args.steps, 5))
    train_step()
    torch.cuda.synchronize()
    start.record()
    for _ in range(fb_steps):
        train_step()
    end.record()
    torch.cuda.synchronize()
    fb_ms = start.elapsed_time(end) / fb_steps
    assert ops.read_status(dev) == 0
    if rank != 0:
        return
    peak, kind = measured_tflops()
    achieved = flops / (ms / 1e3) / 1e12
    line = {
        "metric": "grouped_swiglu_ffn_tflops", "value": achieved * world, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "experts": E, "rows": R, "D": D, "ff": FF,
                   "l2": "weights (%.1f GB) exceed the 126 MB L2" % (E * 3 * D * FF * 2 / 1e9)},
        "e2e": None, "gpu_launches": 2 * args.steps,
        "roofline": {"bound": "tensor", "kernel": "grouped_gemm_kernel (gate/up + down)", "achieved": achieved,
                     "peak": peak, "peak_kind": kind, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "gate_up_ms": gate_up_ms, "gate_up_tflops": 4 * R * D * FF / gate_up_ms / 1e9,
                     "down_ms": down_ms, "down_tflops": 2 * R * D * FF / down_ms / 1e9,
                     "fwd_bwd_ms": fb_ms, "fwd_bwd_tflops": 3 * flops / fb_ms / 1e9,
                     "fwd_bwd_note": "forward + data and weight gradients of both products = 3x the forward "
                                     "FLOPs (the forward keeps its pre-activations, nothing is recomputed), "
                                     "SwiGLU derivative as one streaming kernel in between"},
        "clocks": clocks.summary(),
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def cfg4_record(name, rank, world, local_rank, steps, warmup, cpu=True):
    """Index build + dispatch permute + combine, forward and backward, identity experts.
    Returns the record of one workload: whole-chain GB/s of algorithmic bytes and a roofline
    entry per kernel (None on ranks other than 0)."""
    import torch
    import torch.distributed as dist

    from fastmoe_b200.kernels import ops, routing
    from fastmoe_b200.workloads import routing_uniform

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    T, D, E, K = CFG4[name]
    N, s = T * K, 2
    idx_cpu, w_cpu = routing_uniform(T, E, K, seed=rank)
    idx, gate = idx_cpu.to(dev), w_cpu.to(dev).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, generator=torch.Generator(device=dev).manual_seed(7 + rank), device=dev,
                         dtype=torch.bfloat16)  # router logits, only to time the top-k/softmax kernel
    gen = torch.Generator(device=dev).manual_seed(rank)
    x = torch.randn(T, D, generator=gen, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    grad_out = torch.randn(T, D, generator=gen, device=dev, dtype=torch.bfloat16)
    # per-kernel algorithmic bytes (payload only; index bytes are < 0.1%)
    alg = {
        "fmoe_permute_fwd": T * D * s + N * D * s,
        "fmoe_combine_gather": N * D * s + T * D * s,
        "fmoe_combine_bwd": T * D * s + 2 * N * D * s,
        "fmoe_permute_bwd": N * D * s + T * D * s,
    }
    total_bytes = sum(alg.values())

    def step():
        x.grad = gate.grad = None
        routing.route_topk(logits, K)  # timed; the chain below uses the fixed uniform routing
        ix = routing.build_index(idx, gate, E)
        permuted = routing.permute_rows(x, ix.slot_of, K)
        out = ops.grouped_weighted_scatter_add([permuted], ix.reverse_map, ix.sorted_w, (T, D))
        out.backward(grad_out)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(warmup, 3)):
        step()
    barrier()
    launches0 = ops.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        barrier()
        start.record()
        for _ in range(steps):
            step()
        end.record()
        barrier()
        elapsed_ms = start.elapsed_time(end)
        launches = ops.launch_count - launches0
        ops.kernel_events = {}  # a second pass with events around every launch, for the per-kernel times
        for _ in range(steps):
            step()
        barrier()
    events, ops.kernel_events = ops.kernel_events, None
    stats = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    elapsed_ms = float(stats[0])
    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    kernels = {}
    for kname, pairs in events.items():
        ms = statistics.mean(a.elapsed_time(b) for a, b in pairs)
        entry = {"ms": ms, "calls": len(pairs)}
        if kname in alg:
            entry.update(algorithmic_bytes=alg[kname], achieved=alg[kname] / ms / 1e6, frac=alg[kname] / ms / 1e6 / peak)
        kernels[kname] = entry
    top = max(alg, key=lambda k: kernels[k]["ms"])

    cpu_baseline = None
    if cpu:  # the oracle port of the same chain (fp32 arithmetic) on the first 2048 tokens
        import oracle

        oracle.use_all_cores()
        Ts = min(T, 2048)
        o_ix = oracle.build_index(idx_cpu[:Ts].numpy(), w_cpu[:Ts].numpy(), E)
        xs = x.detach()[:Ts].float().cpu().numpy()
        gs = grad_out[:Ts].float().cpu().numpy()
        t0 = time.perf_counter()
        perm = oracle.permute(xs, o_ix["reverse_map"])
        oracle.combine([perm], o_ix["reverse_map"], o_ix["sorted_w"], Ts)
        g_rows, _ = oracle.combine_bwd(perm, o_ix["reverse_map"], o_ix["sorted_w"], gs)
        oracle.permute_bwd(g_rows, o_ix["reverse_map"], Ts)
        cpu_s = time.perf_counter() - t0
        cpu_baseline = {"value": total_bytes * Ts / T / cpu_s / 1e9, "unit": UNIT, "cores": oracle.num_threads(),
                        "kind": "port", "ms": cpu_s * 1e3,
                        "sample": f"the first {Ts} of {T} tokens, one pass of permute + combine + both backwards "
                                  "in fp32; bytes counted as in the bf16 workload"}  # fmt: skip
    return {
        "metric": "dispatch_combine_hbm_gbs", "value": total_bytes * world * steps / (elapsed_ms / 1e3) / 1e9,
        "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": max(warmup, 3),
        "ms_per_step": elapsed_ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "T": T, "D": D, "E": E, "top_k": K, "routing": "uniform"},
        "notes": {"l2": "inputs (1.9 GB of routed rows) exceed the 126 MB L2", "multi_gpu": "replicas only"},
        "e2e": None, "gpu_launches": launches,
        "roofline": {"bound": "hbm", "kernel": top, "achieved": kernels[top]["achieved"], "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": kernels[top]["frac"], "traffic": None},
        "kernels": kernels, "cpu_baseline": cpu_baseline, "clocks": clocks.summary(),
    }  # fmt: skip


def run_cfg4(args, rank, world, local_rank):
    line = cfg4_record(args.workload, rank, world, local_rank, args.steps, args.warmup)
    if line is not None:
        print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + sorted(CFG4) + sorted(GEMM) + [EP_WORKLOAD], default=DEFAULT_WORKLOAD)
    ap.add_argument("--micro-batches", type=int, default=None, help="expert-parallel layer: micro-batches per step")
    ap.add_argument("--ep-mode", choices=["fused", "nccl"], default="fused",
                    help="expert-parallel layer with several ranks: fused peer-store exchange or NCCL all-to-all")
    ap.add_argument("--gemm-sms", type=int, default=None, help="expert-parallel layer: SMs for the grouped GEMM")
    ap.add_argument("--ep-groups", type=int, default=None,
                    help="expert-parallel layer, fused exchange: groups the local experts are split into for the "
                         "overlap of dispatch and GEMMs (default: 4 with several ranks)")
    ap.add_argument("--no-ep", action="store_true", help="skip the expert-parallel layer part of the default run")
    ap.add_argument("--no-also", action="store_true", help="skip the graph-replay, skewed-combine and dispatch+combine sub-records")
    ap.add_argument("--cpu-port", action="store_true",
                    help="CPU baseline: time the C port even where the reference package is installed")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="launch-shape knob of the library (fmoe_tune), for sweeps; repeatable")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    if world > 1:
        import torch
        import torch.distributed as dist

        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    for item in args.tune:
        from fastmoe_b200 import _lib

        key, _, val = item.partition("=")
        _lib.tune(key, int(val))
    try:
        if args.workload in CFG4:
            run_cfg4(args, rank, world, local_rank)
        elif args.workload in GEMM:
            run_gemm(args, rank, world, local_rank)
        elif args.workload == EP_WORKLOAD:
            run_ep(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist

            dist.destroy_process_group()


if __name__ == "__main__":
    main()
