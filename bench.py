"""Benchmark of the tmq_b200 hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--n ELEMS]

Headline workload (N=1): the standalone soft-staircase pass of the baseline configuration "Standalone soft-staircase
transfer, fp32, 64M elements": one step = ONE fused kernel doing forward + backward + quantization-loss
reduction + clamp over a 2^26-element weight tensor (w uniform in [-1.5,1.5), upstream grad N(0,1), hardness
cycling through {0.1, 0.5, 0.9, 1.0}).  Algorithmic traffic 20 B/element (read w, g; write y, grad, clamped w).

Prints one JSON line (rank 0).  `value` is device-resident throughput; `e2e` is the same pass through the public
operator call with pinned HOST buffers (H2D of w and g, D2H of the three outputs and the loss, every step).
With --gpus N every rank processes its own 2^26-element shard (weak scaling) and the loss scalar is all-reduced
over NCCL inside the step.  `--impl reference` times the reference's CPU path for the same workload on all host
threads: the reference's own tmq/tmq.py (SoftStep / SoftStepDerivative autograd functions, torch.mean, backward,
torch.clamp: PyTorch CPU eager) when a checkout is present (TMQ_REFERENCE_DIR or a checkout beside this repository), else
its restatement oracle/softstep_torch.py; one step = the full 2^26-element pass.  For N > 1 the default run also measures
the three partitionings that move data (column-sharded prefill GEMM, data-parallel ResNet-18 QAT, batch-sharded packed
ResNet-18 inference) and reports them under `extra`.
"""
import argparse
import ctypes
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

GEMV_ROWS_PER_PASS = 16     # activation rows one skinny-kernel launch takes
HARDNESS = [0.1, 0.5, 0.9, 1.0]
SHARPNESS, STRENGTH, LO, HI = 5.0, 5e-4, -1.0, 1.0
BYTES_PER_ELEM = 20
NCU_TRAFFIC_BYTES_PER_ELEM = 623554048 / 33554432   # measured DRAM bytes per element of the fused kernel (ncu, 2^25 elements)
METRIC = "softstep_fwd_bwd_loss_clamp_GBps"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return dist, rank, local, world
    return None, 0, 0, 1


# ------------------------------------------------------------------------------------------------ CPU arm

def softstep_config(n, world):
    """`config` of the headline workload; both arms print exactly this."""
    return {"workload": "softstep_fused_2^26_f32", "elements_per_gpu": n, "hardness": HARDNESS,
            "sharpness": SHARPNESS, "strength": STRENGTH, "bytes_per_element": BYTES_PER_ELEM,
            "l2": "inputs (w, g: 2 x 256 MiB) exceed the 126 MB L2; no flush needed",
            "sharding": ("one shard per GPU, fp64 loss scalar all-reduced (NCCL, asynchronous: overlaps the next step, "
                         "drained inside the timed region)") if world > 1 else "single GPU"}


def host_threads():
    """Every host thread this process may run on (torchrun exports OMP_NUM_THREADS=1; the CPU arm must not inherit it)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def load_reference():
    """The reference's own Python module when its checkout is on this machine, else None."""
    import contextlib
    import io
    ref_dir = os.environ.get("TMQ_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
    if not os.path.isfile(os.path.join(ref_dir, "tmq", "tmq.py")):
        return None
    sys.path.insert(0, ref_dir)
    try:
        with contextlib.redirect_stdout(io.StringIO()), contextlib.redirect_stderr(io.StringIO()):
            import tmq as ref
    except Exception:
        return None
    finally:
        sys.path.remove(ref_dir)
    return ref


class _Ctrl:
    def __init__(self, digamma):
        self.digamma = digamma


def cpu_element_pass(ref):
    """One QAT element pass on CPU tensors: forward, loss mean, both backwards (autograd, accumulated into .grad),
    clamp - through the reference's autograd functions (tmq/tmq.py:404-493, :696-699) or their restatement."""
    if ref is None:
        from oracle import softstep_torch as OT
        return "port", OT.qat_element_pass

    def run(w, g, digamma, sharpness, strength, lo, hi):
        w = w.detach().requires_grad_(True)
        y = ref.SoftStep.apply(w, 1.0, _Ctrl(digamma))
        loss = torch.mean(ref.SoftStepDerivative.apply(w, sharpness, strength))
        torch.autograd.backward([y, loss], [g, torch.ones_like(loss)])
        with torch.no_grad():
            wc = torch.clamp(w, lo, hi)
        return y.detach(), w.grad, wc, loss.detach()
    return "reference", run


def cpu_softstep_baseline(elems, reps, warm=1):
    """The reference CPU path on all host threads; returns (GB/s at 20 B/elem, seconds per pass, kind, threads)."""
    cores = host_threads()
    kind, run = cpu_element_pass(load_reference())
    gen = torch.Generator().manual_seed(0)
    w = torch.rand(elems, generator=gen) * 3 - 1.5
    g = torch.randn(elems, generator=gen)
    for i in range(warm):
        run(w, g, HARDNESS[i % 4], SHARPNESS, STRENGTH, LO, HI)
    t0 = time.perf_counter()
    for i in range(reps):
        run(w, g, HARDNESS[i % 4], SHARPNESS, STRENGTH, LO, HI)
    dt = (time.perf_counter() - t0) / reps
    return elems * BYTES_PER_ELEM / dt / 1e9, dt, kind, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n = args.n
    gbs, dt, kind, cores = cpu_softstep_baseline(n, args.steps, warm=args.warmup)
    what = ("the reference's own tmq/tmq.py autograd functions" if kind == "reference"
            else "restatement of the reference's autograd functions (no reference checkout on this machine)")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": softstep_config(n, max(world, args.gpus)),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"every step is one full pass over {n} elements on one host process ({what}; PyTorch "
                                   f"CPU eager: forward, loss mean, both backwards through autograd, clamp)"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm

def run_ours(args):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the tmq_b200 kernels have no CPU fallback")
    dist, rank, local, world = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from tmq_b200 import ops

    n = args.n
    gen = torch.Generator(device=dev).manual_seed(rank)
    w = torch.rand(n, generator=gen, device=dev) * 3 - 1.5
    g = torch.randn(n, generator=gen, device=dev)
    out = (torch.empty_like(w), torch.empty_like(w), torch.empty_like(w),
           torch.empty((), dtype=torch.float64, device=dev))
    gq = 1.0 / n

    # multi-GPU: the loss scalar of step i is all-reduced asynchronously (NCCL's stream) while step i+1 runs; a ring of
    # four loss buffers keeps the kernel from overwriting a scalar still in flight, and the timed region ends only after
    # every outstanding all-reduce has completed
    loss_ring = [out[3]] + [torch.empty_like(out[3]) for _ in range(3)]
    pending = [None] * len(loss_ring)

    def step(i):
        slot = i % len(loss_ring)
        if pending[slot] is not None:
            pending[slot].wait()
            pending[slot] = None
        res = ops.fused_step(w, g, HARDNESS[i % 4], SHARPNESS, STRENGTH, LO, HI, gq=gq,
                             out=(out[0], out[1], out[2], loss_ring[slot]))
        if dist is not None:
            pending[slot] = dist.all_reduce(res[3], async_op=True)
        return res

    def drain():
        for slot, work in enumerate(pending):
            if work is not None:
                work.wait()
                pending[slot] = None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    drain()
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    drain()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * n * BYTES_PER_ELEM / (ms_per_step * 1e-3) / 1e9

    # kernel-only duration for the roofline (no collective in between), same launches, same stream
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for i in range(args.steps):
        ops.fused_step(w, g, HARDNESS[i % 4], SHARPNESS, STRENGTH, LO, HI, gq=gq, out=out)
    k1.record()
    torch.cuda.synchronize()
    kernel_ms = k0.elapsed_time(k1) / args.steps

    # end to end: pinned host buffers in, results out, every step
    hw, hg = w.cpu().pin_memory(), g.cpu().pin_memory()
    hy, hgw, hwc = (torch.empty(n, dtype=torch.float32).pin_memory() for _ in range(3))

    def e2e_step(i):
        # the public host-buffer call: chunks stream host -> device -> kernel -> host on three streams; synchronous
        loss = ops.fused_step_host(hw, hg, hy, hgw, hwc, HARDNESS[i % 4], SHARPNESS, STRENGTH, LO, HI, gq=gq, device=dev)
        if dist is not None:
            dist.all_reduce(torch.tensor([loss], dtype=torch.float64, device=dev))

    e2e_steps = max(1, min(args.steps, 10)) if not args.no_e2e else 0
    for i in range(2 if e2e_steps else 0):
        e2e_step(i)
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    s1.record()
    barrier()
    t = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item()) / max(e2e_steps, 1)
    e2e_value = world * n * BYTES_PER_ELEM / (e2e_ms * 1e-3) / 1e9 if e2e_steps else None

    # where the end-to-end time goes: each copy direction alone, every rank at once (the ranks share the host's memory
    # and its PCIe root complexes), max over ranks like every other multi-GPU time here
    legs = {}
    if e2e_steps:
        def leg(fn):
            fn()
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            for _ in range(3):
                fn()
            a1.record()
            barrier()
            tt = torch.tensor([a0.elapsed_time(a1) / 3], dtype=torch.float64, device=dev)
            if dist is not None:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item())
        ms_in = leg(lambda: (w.copy_(hw, non_blocking=True), g.copy_(hg, non_blocking=True)))
        ms_out = leg(lambda: (hy.copy_(out[0], non_blocking=True), hgw.copy_(out[1], non_blocking=True),
                              hwc.copy_(out[2], non_blocking=True)))
        legs = {"h2d_only_ms": ms_in, "h2d_only_GBps_aggregate": world * 2 * n * 4 / ms_in / 1e6,
                "d2h_only_ms": ms_out, "d2h_only_GBps_aggregate": world * 3 * n * 4 / ms_out / 1e6,
                "kernel_only_ms": kernel_ms,
                "reading": "the step cannot beat max(h2d_only, d2h_only): the two directions overlap, the kernel hides under both"}
    clocks = sampler.stop() if rank == 0 else None

    # the workloads that move data between GPUs (N > 1), or that complete the single-GPU picture (N = 1); every rank
    # takes part, rank 0 reports
    extra = {}
    if not args.no_extra:
        del hw, hg, hy, hgw, hwc
        del w, g, out, loss_ring
        torch.cuda.empty_cache()
        ctx = _Ctx(dist, rank, world, dev)
        xs, xw = max(3, min(args.steps, 10)), 3
        if world == 1:
            extra = ternary_sections(ctx.peaks)
            extra["resnet18_packed_inference_batch256"] = wl_resnet(ctx, "infer", xs, xw, per_layer=True)
            torch.cuda.empty_cache()
            extra["resnet18_qat_batch256"] = wl_resnet(ctx, "qat", xs, xw)
        else:
            extra["column_sharded_gemm_M8192_K8192_N28672"] = wl_gemm(ctx, xs, xw)
            torch.cuda.empty_cache()
            extra["resnet18_packed_inference_batch256"] = wl_resnet(ctx, "infer", xs, xw)
            torch.cuda.empty_cache()
            extra["resnet18_qat_batch256"] = wl_resnet(ctx, "qat", xs, xw)
        torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    achieved = n * BYTES_PER_ELEM / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": softstep_config(n, world),
        "e2e": dict({"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": 2 * n * 4, "d2h_bytes_per_step": 3 * n * 4 + 8 * 16,
                     "ms_per_step": e2e_ms, "steps": e2e_steps,
                     "call": "ops.fused_step_host: pinned host buffers, 16 chunks of 2^22 elements pipelined over three streams"},
                    **legs),
        "gpu_launches": args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES_PER_ELEM * n,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at 2^25 "
                                       "elements (623.6 MB), scaled by the element count",
                     "peak_kind": peak_kind,
                     "kernel": "softstep_kernel<FWD|BWD|QSUM|QGRAD|CLAMP>", "kernel_ms": kernel_ms,
                     "algorithmic_bytes": n * BYTES_PER_ELEM},
    }
    if extra:
        line["extra"] = extra
    if world == 1 and not args.no_cpu:
        gbs, dt, kind, cores = cpu_softstep_baseline(1 << 24, 3)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                                "sample": "3 passes over 2^24 of the 2^26 elements; the reference's PyTorch CPU eager "
                                          "sequence (tmq/tmq.py:404-493, :696-699: autograd functions, mean, backward, clamp)"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------ ternary kernels

def _time_cuda(fn, reps, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _ternary_packed(ops, N, K, seed, p=(0.3, 0.4, 0.3)):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    u = torch.rand(N, K, generator=gen, device="cuda")
    W = torch.where(u < p[0], -1.0, torch.where(u < p[0] + p[1], 0.0, 1.0))
    return ops.compactify_ternary(W)


def measure_tensor_peaks():
    """Dense 8192^3 library GEMMs on this GPU: bf16 (torch.matmul) and int8 (torch._int_mm), each as a burst (best of 10
    single launches) and sustained (one event pair around about two seconds of back-to-back launches, under the power
    cap) - the way the machine's bf16 peaks were recorded."""
    out = {}

    def sustained(fn, flops, seconds=2.0):
        n = max(10, int(seconds / (_time_cuda(fn, 3, warm=1) * 1e-3)))
        return flops / _time_cuda(fn, n, warm=0) / 1e9

    flops = 2 * 8192 ** 3
    a = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    b = torch.randn(8192, 8192, device="cuda").to(torch.bfloat16)
    best = min(_time_cuda(lambda: a @ b, 1, warm=1) for _ in range(10))
    out["bf16_tflops"] = flops / best / 1e9
    try:
        ai = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8)
        bi = torch.randint(-127, 128, (8192, 8192), device="cuda", dtype=torch.int8).t()
        best = min(_time_cuda(lambda: torch._int_mm(ai, bi), 1, warm=1) for _ in range(10))
        out["int8_tops"] = flops / best / 1e9
        out["int8_tops_sustained"] = sustained(lambda: torch._int_mm(ai, bi), flops)
    except Exception as exc:  # library path unavailable: leave the peak out rather than guess
        out["int8_tops"] = None
        out["int8_error"] = str(exc)[:120]
    out["bf16_tflops_sustained"] = sustained(lambda: a @ b, flops)
    torch.cuda.synchronize()
    time.sleep(3.0)            # let the part cool: the sections that follow are bursts
    return out


def ternary_sections(peaks):
    """Baseline configs 5 (prefill GEMM M=8192, K=8192, N=28672) and 3 (decode GEMV N=11008, K=4096, M in 1/8/32)."""
    from tmq_b200 import _lib, ops
    L = _lib.lib()
    res = {}
    lib_peaks = measure_tensor_peaks()
    res["library_peaks_this_run"] = lib_peaks
    # ---- config 5
    M, K, N = 8192, 8192, 28672
    P = _ternary_packed(ops, N, K, 0)
    scale = torch.rand(N, device="cuda") * 0.09 + 0.01
    X = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    wt = ops.prepack(P, N, ops.FMT_BF16)
    ms = _time_cuda(lambda: ops.ternary_gemm(X, wt, N, scale), 10)
    ops.check_gemm_status()
    tf = 2 * M * N * K / ms / 1e9
    res["gemm_bf16_M8192_K8192_N28672"] = {"ms": ms, "tops_equiv": tf, "peak": peaks["bf16_tflops"],
                                           "frac_of_measured_bf16_burst": tf / peaks["bf16_tflops"],
                                           "frac_of_library_bf16_this_run": tf / lib_peaks["bf16_tflops"]}
    del wt, X
    X8 = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8)
    wt8 = ops.prepack(P, N, ops.FMT_I8)
    ms = _time_cuda(lambda: ops.ternary_gemm_i8(X8, wt8, N), 10)
    ops.check_gemm_status()
    tf = 2 * M * N * K / ms / 1e9
    res["gemm_i8_M8192_K8192_N28672"] = {"ms": ms, "tops_equiv": tf, "library_int8_peak_this_run": lib_peaks["int8_tops"],
                                         "frac_of_library_int8_this_run": (tf / lib_peaks["int8_tops"])
                                         if lib_peaks["int8_tops"] else None,
                                         "frac_of_nominal_4500": tf / 4500.0}
    del wt8, X8, P
    # ---- config 3: 32 distinct matrices (352 MB > L2) back to back in one CUDA graph
    # (a few idle seconds first: the GEMMs above ran into the power cap, and these latency-bound launches should not
    # inherit their clocks)
    torch.cuda.synchronize()
    import time
    time.sleep(4.0)
    N, K, NM = 11008, 4096, 32
    wts = []
    for i in range(NM):
        wts.append(ops.prepack(_ternary_packed(ops, N, K, 100 + i), N, ops.FMT_BF16))
    scale = torch.rand(N, device="cuda") * 0.09 + 0.01
    def graph_us_per_matrix(body):
        """`body(stream_handle)` launches the whole set of NM matrices once; captured into a CUDA graph, replayed."""
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            body(stream.cuda_stream)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                body(stream.cuda_stream)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(10):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10 / NM * 1e3

    def gemv_entry(us, nbytes, Mg, protocol):
        return {"us_per_matrix": us, "gbs": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peaks["hbm_gbs"],
                "tops_equiv": 2 * Mg * N * K / us / 1e6, "algorithmic_bytes": nbytes, "protocol": protocol}

    def pointer_array(tensors):
        arr = (ctypes.c_void_p * len(tensors))()
        for i, t in enumerate(tensors):
            arr[i] = t.data_ptr()
        return arr

    status = ops.gemm_status_word(torch.device("cuda", torch.cuda.current_device()))
    for Mg in (1, 8, 16, 32):
        X = torch.randn(Mg, K, device="cuda").to(torch.bfloat16)
        Y = torch.empty(Mg, N, device="cuda", dtype=torch.bfloat16)

        def body(st):
            for i in range(NM):
                for m0 in range(0, Mg, GEMV_ROWS_PER_PASS):
                    rc = L.tmq_ternary_gemv_bf16(X.data_ptr() + m0 * K * 2, wts[i].data_ptr(), scale.data_ptr(), None,
                                                 Y.data_ptr() + m0 * N * 2, min(GEMV_ROWS_PER_PASS, Mg - m0), N, K, N, 0,
                                                 status.data_ptr(), st)
                    assert rc == 0
        nbytes = N * K // 4 + 2 * Mg * K + 2 * Mg * N + 4 * N
        res[f"gemv_bf16_M{Mg}_N11008_K4096"] = gemv_entry(
            graph_us_per_matrix(body), nbytes, Mg, "32 distinct matrices in one CUDA graph, time/32; "
            f"{(Mg + GEMV_ROWS_PER_PASS - 1) // GEMV_ROWS_PER_PASS} launch(es) per matrix")
    # batched entry point: the same 32 matrices, `group` of them per launch sharing the activation vector (2 = gate / up,
    # 4 ~ query / key / value / gate, 16 = the most one launch takes); every matrix writes its own result
    X = torch.randn(1, K, device="cuda").to(torch.bfloat16)
    Ys = [torch.empty(1, N, device="cuda", dtype=torch.bfloat16) for _ in range(NM)]
    scales = pointer_array([scale] * NM)
    for group in (2, 4, 16):
        Wp = [pointer_array(wts[i:i + group]) for i in range(0, NM, group)]
        Yp = [pointer_array(Ys[i:i + group]) for i in range(0, NM, group)]

        def body(st):
            for q in range(NM // group):
                rc = L.tmq_ternary_gemv_batched_bf16(X.data_ptr(), 0, Wp[q], scales, None, Yp[q], group, 1, N, K, N, 0,
                                                     status.data_ptr(), st)
                assert rc == 0
        nbytes = N * K // 4 + 2 * K + 2 * N + 4 * N
        res[f"gemv_batched{group}_bf16_M1_N11008_K4096"] = gemv_entry(
            graph_us_per_matrix(body), nbytes, 1,
            f"32 distinct matrices in one CUDA graph, {group} per launch (tmq_ternary_gemv_batched_bf16), time/32")
    del Ys
    # the same protocols with int8 activations (exact int32 results; byte dot products at M = 1)
    wts8 = []
    for i in range(NM):
        wts8.append(ops.prepack(_ternary_packed(ops, N, K, 100 + i), N, ops.FMT_I8))
    del wts
    for Mg in (1, 8, 16):
        X8 = torch.randint(-127, 128, (Mg, K), device="cuda", dtype=torch.int8)
        Y8 = torch.empty(Mg, N, device="cuda", dtype=torch.int32)

        def body8(st):
            for i in range(NM):
                rc = L.tmq_ternary_gemv_i8(X8.data_ptr(), wts8[i].data_ptr(), Y8.data_ptr(), Mg, N, K, N,
                                           status.data_ptr(), st)
                assert rc == 0
        nbytes = N * K // 4 + Mg * K + 4 * Mg * N
        res[f"gemv_i8_M{Mg}_N11008_K4096"] = gemv_entry(graph_us_per_matrix(body8), nbytes, Mg,
                                                       "32 distinct matrices in one CUDA graph, time/32")
    X8 = torch.randint(-127, 128, (1, K), device="cuda", dtype=torch.int8)
    Ys8 = [torch.empty(1, N, device="cuda", dtype=torch.int32) for _ in range(NM)]
    for group in (2, 4, 16):
        Wp = [pointer_array(wts8[i:i + group]) for i in range(0, NM, group)]
        Yp = [pointer_array(Ys8[i:i + group]) for i in range(0, NM, group)]

        def body8b(st):
            for q in range(NM // group):
                rc = L.tmq_ternary_gemv_batched_i8(X8.data_ptr(), 0, Wp[q], Yp[q], group, 1, N, K, N, status.data_ptr(), st)
                assert rc == 0
        nbytes = N * K // 4 + K + 4 * N
        res[f"gemv_batched{group}_i8_M1_N11008_K4096"] = gemv_entry(
            graph_us_per_matrix(body8b), nbytes, 1,
            f"32 distinct matrices in one CUDA graph, {group} per launch (tmq_ternary_gemv_batched_i8), time/32")
    del Ys8
    ops.check_gemm_status()
    del wts8
    res.update(qat_linear_sections(ops))
    res["cpu_baselines"] = ternary_cpu_baselines()
    return res


def qat_linear_sections(ops):
    """Training forward of a QAT Linear layer (soft staircase + matmul), fused kernel against the two-pass routes.
    16 distinct weight matrices (1 GB of fp32 latent weights > L2) so that every call reads its weights from HBM."""
    out = {}
    N = K = 4096
    NW = 16
    ws = [torch.rand(N, K, device="cuda") * 2.5 - 1.25 for _ in range(NW)]
    bias = torch.randn(N, device="cuda")
    for M in (64, 256, 2048):
        x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        xf = x.float()
        state = {"i": 0}

        def nxt():
            state["i"] = (state["i"] + 1) % NW
            return ws[state["i"]]
        fused = _time_cuda(lambda: ops.qat_linear_forward(x, nxt(), bias, 5.0), 32)
        two_pass_f32 = _time_cuda(lambda: torch.nn.functional.linear(xf, ops.fwd_softstep(nxt(), 5.0), bias), 32)
        two_pass_bf16 = _time_cuda(lambda: torch.nn.functional.linear(x, ops.fwd_softstep(nxt(), 5.0).to(torch.bfloat16),
                                                                      None), 32)
        out[f"qat_linear_fwd_M{M}_N4096_K4096"] = {
            "fused_us": fused * 1e3, "staircase_kernel_plus_fp32_linear_us": two_pass_f32 * 1e3,
            "staircase_kernel_plus_bf16_cast_plus_bf16_linear_us": two_pass_bf16 * 1e3,
            "fused_tflops_equiv": 2 * M * N * K / fused / 1e9,
            "weights_per_us": N * K / (fused * 1e3),
            "note": "fused = tmq_qat_linear_fwd_bf16 (bf16 activations, S(W) as two bf16 terms, fp32 out); the fp32 route "
                    "is what the reference's layer does (SoftStep.apply + F.linear)"}
    ops.check_gemm_status()
    return out


def ternary_cpu_baselines():
    """What the reference offers on the host for the inference path: un-compacted layers through PyTorch CPU eager
    (F.linear on the expanded fp32 weights) and its single-threaded packer (restated in oracle/oracle.c).  Bounded
    samples: 64 activation rows of the M=8192 K=8192 N=28672 problem; one 11008 x 4096 matrix for the packer."""
    import time
    import numpy as np
    from oracle import ternary as T
    out = {"cores": torch.get_num_threads()}
    M, K, N = 64, 8192, 28672
    gen = torch.Generator().manual_seed(0)
    W = torch.randint(-1, 2, (N, K), generator=gen).float()
    X = torch.randn(M, K, generator=gen)
    torch.nn.functional.linear(X, W)
    t0 = time.perf_counter()
    torch.nn.functional.linear(X, W)
    dt = time.perf_counter() - t0
    out["linear_f32_K8192_N28672"] = {"tops_equiv": 2 * M * N * K / dt / 1e12, "seconds": dt,
                                      "sample": "64 of 8192 activation rows, torch CPU eager F.linear on expanded weights",
                                      "kind": "port"}
    del W, X
    Wp = np.random.default_rng(0).integers(-1, 2, (11008, 4096)).astype(np.float32)
    t0 = time.perf_counter()
    T.pack(Wp)
    dt = time.perf_counter() - t0
    out["pack_11008x4096"] = {"seconds": dt, "sample": "one matrix, single-threaded C restatement of the reference packer",
                              "kind": "port", "cores": 1}
    return out


# ------------------------------------------------------------------------------------------------ other workloads

def _conv_layers(net, images):
    """(name, PackedConv or None, M, N, K, bytes) of every matrix-shaped layer of the packed ResNet-18 at 224 x 224."""
    out, size = [], 224

    def add(name, conv, size_in):
        size_out = (size_in + 2 * conv.padding[0] - conv.dilation[0] * (conv.ky - 1) - 1) // conv.stride[0] + 1
        m, n, k = images * size_out * size_out, conv.cout, conv.cin * conv.ky * conv.kx
        in_bytes = images * size_in * size_in * conv.cin * (4 if conv.cin < 64 else 2)      # the stem reads fp32 images
        out.append((name, conv, m, n, k, in_bytes + 2 * m * n + n * k / 4))
        return size_out

    size = add("conv1", net.conv1, size)
    pooled = (size + 2 - 3) // 2 + 1                     # 3 x 3 / 2 max pooling, fused into the stem's epilogue:
    name, conv, m, n, k, nbytes = out[0]                 # the stem writes the pooled map only
    out[0] = (name, conv, m, n, k, nbytes - 2 * m * n + 2 * images * pooled * pooled * n)
    size = pooled
    for i, (c1, c2, down) in enumerate(net.blocks):
        if down is not None:
            add(f"block{i}.down", down, size)
        mid = add(f"block{i}.conv1", c1, size)
        size = add(f"block{i}.conv2", c2, mid)
    out.append(("fc", None, images, net.fc_n, net.fc_k, 2 * images * (net.fc_n + net.fc_k) + net.fc_n * net.fc_k / 4))
    return out


def _resnet_layer_roofline(net, images, peaks, measured_ms):
    """Per-layer floor of the packed ResNet-18 pass on one GPU: each convolution / linear layer can be no faster than
    max(2*M*N*K / bf16 peak, (activations in + out at 2 bytes + packed weights) / HBM peak), the stem counted with the
    pooled output it writes; the sum over the layers against the measured time of the whole pass (which also holds the
    average pooling and the launch gaps)."""
    floors = [max(2.0 * m * n * k / (peaks["bf16_tflops"] * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9))
              for _, _, m, n, k, nbytes in _conv_layers(net, images)]
    ideal_ms = sum(floors) * 1e3
    return {"bound": "per layer max(tensor, hbm)", "achieved": measured_ms, "peak": ideal_ms, "unit": "ms per pass",
            "frac": ideal_ms / measured_ms, "traffic": None, "layers": len(floors)}


def _resnet_per_layer(net, x, peaks):
    """Each layer of the packed pass timed alone on its actual input (CUDA events, 5 launches after 2 warm-ups; the
    activations of one layer exceed L2 only in the early stages, so late layers read their input from L2, as they do in
    the real pass).  Reports time, TFLOP/s, share of the measured bf16 peak and of the layer's own floor."""
    captured = []
    net(x, trace=lambda name, layer, x_in, res, y: captured.append((name, layer, x_in, res)))
    shapes = {name: (m, n, k, nbytes) for name, _, m, n, k, nbytes in _conv_layers(net, x.shape[0])}
    rows = {}
    for name, layer, x_in, res in captured:
        if layer is None:
            continue
        if name == "conv1":      # the pass runs the stem with ReLU and the max pooling fused into its epilogue
            fn = (lambda: layer.from_images_pooled(x_in)) if layer.from_images_pooled(x_in) is not None \
                else (lambda: layer.from_images(x_in, defer_relu=True))
        else:
            fn = lambda: layer(x_in, residual=res)
        ms = _time_cuda(fn, 5, warm=2)
        m, n, k, nbytes = shapes[name]
        tf = 2.0 * m * n * k / ms / 1e9
        floor_ms = max(2.0 * m * n * k / (peaks["bf16_tflops"] * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
        rows[name] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 3),
                      "frac_of_layer_floor": round(floor_ms / ms, 3), "M": m, "N": n, "K": k}
    return rows


class _Ctx:
    """What every workload needs: the process group (or None), rank / world, device, peaks, and the timing helpers."""

    def __init__(self, dist, rank, world, dev):
        self.dist, self.rank, self.world, self.dev = dist, rank, world, dev
        self.peaks, self.peak_kind = measured_peaks()

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, step, steps, warmup):
        """ms per step: warm-ups, barrier, CUDA events around `steps` calls, barrier, max over ranks."""
        for i in range(max(warmup, 3)):
            step(i)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        self.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=self.dev)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item()) / steps


def wl_gemm(ctx, steps, warmup, M=8192, K=8192, N=28672, chunks=None):
    """Prefill linear, output columns sharded over the ranks, all-gather of the column blocks.  `chunks` row chunks
    pipeline the gather of one chunk under the GEMM of the next (default: 4 when sharded)."""
    from tmq_b200 import dist as tdist
    from tmq_b200 import ops
    dev, world = ctx.dev, ctx.world
    P = _ternary_packed(ops, N, K, 0)                         # same seed on every rank: the same matrix
    scale = torch.rand(N, generator=torch.Generator(device=dev).manual_seed(1), device=dev) * 0.09 + 0.01
    X = torch.randn(M, K, generator=torch.Generator(device=dev).manual_seed(2), device=dev).to(torch.bfloat16)
    lin = tdist.ColumnShardedLinear(P, N, scale, None, rank=ctx.rank, world_size=world)
    del P
    chunks = (4 if world > 1 else 1) if chunks is None else chunks
    ms = ctx.timed(lambda i: lin(X, blocked=True, chunks=chunks), steps, warmup)
    ops.check_gemm_status(dev)
    ms_local = _time_cuda(lambda: lin.local(X), max(3, steps // 2))
    ms_unchunked = ctx.timed(lambda i: lin(X, blocked=True, chunks=1), max(3, steps // 2), 3) if world > 1 else ms
    fused = {}
    if world > 1:
        # GEMM + all-gather as one kernel: the epilogue stores this rank's block into every rank's result buffer
        try:
            # mapping the buffers is a collective step: go on only if it worked on EVERY rank, or the ranks would part
            ok = torch.ones(1, dtype=torch.int32, device=dev)
            why = ""
            try:
                lin.prepare_fused(M, dev)
            except Exception as err:                       # noqa: BLE001
                ok.zero_()
                why = f" ({type(err).__name__}: {err})"
            ctx.dist.all_reduce(ok, op=ctx.dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                raise RuntimeError("peer mapping unavailable on some rank" + why)
            ms_fused = ctx.timed(lambda i: lin.fused(X), steps, warmup)
            ops.check_gemm_status(dev)
            ref = lin(X)                                   # NCCL route, row-major
            same = bool(torch.equal(ref, lin.fused(X)))
            fused = {"fused_gemm_allgather_ms": ms_fused, "fused_tops_equiv": 2 * M * N * K / ms_fused / 1e9,
                     "fused_equals_nccl_route": same, "peer_mapping": lin._peer[M][0].kind}
        except Exception as err:                           # noqa: BLE001 - reported, the NCCL route stays the record
            fused = {"fused_gemm_allgather_error": f"{type(err).__name__}: {err}"[:300]}
    route = "nccl all-gather"
    if fused.get("fused_equals_nccl_route") and fused["fused_gemm_allgather_ms"] < ms:
        # the record is the faster of the two routes; both times stay in `config`
        fused["nccl_route_ms"] = ms
        ms = fused["fused_gemm_allgather_ms"]
        route = "fused: GEMM epilogue stores into every rank's buffer over NVLink"
        chunks = 1
    value = 2 * M * N * K / ms / 1e9
    gather_bytes = M * N * 2 * (world - 1) // max(world, 1)
    peaks = ctx.peaks
    return {"metric": "ternary_gemm_bf16_TOPS_equiv", "value": value, "unit": "TOPS-equiv", "n_gpus": world,
            "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"ternary_linear_M{M}_K{K}_N{N}", "route": route,
                       "sharding": "output columns, 128-aligned; NCCL route: the GEMM epilogue writes this rank's block "
                       "into its slot of the gather buffer, all-gather in place, 4 row chunks pipelined (result left "
                       "blocked: [chunks, world, M/chunks, N/world]); fused route: one kernel, row-major result",
                       "local_gemm_ms": ms_local, "ms_per_step_unchunked": ms_unchunked,
                       "all_gather_bytes_received_per_gpu": gather_bytes,
                       "all_gather_floor_ms_at_770GBs": gather_bytes / 770e9 * 1e3, **fused,
                       "l2": "activations + output (604 MB) exceed L2"},
            "gpu_launches": steps * chunks,
            "roofline": {"bound": "tensor", "achieved": 2 * M * (N / world) * K / ms_local / 1e9,
                         "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": 2 * M * (N / world) * K / ms_local / 1e9 / peaks["bf16_tflops"], "traffic": None,
                         "peak_kind": ctx.peak_kind, "kernel": "ternary_gemm_kernel<bf16,256>"}}


def wl_resnet(ctx, kind, steps, warmup, batch=256, fused_optimizer=False, per_layer=False):
    """ResNet-18 (101 classes) on synthetic 224 x 224 images, the batch split over the ranks (strong scaling):
    kind "qat": one QAT step, data parallel; kind "infer": inference from packed weights, no collective."""
    from tmq_b200 import dist as tdist
    from tmq_b200 import ops, workloads
    import tmq_b200 as tmq
    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    b0, b1 = tdist.shard_range(batch, rank, world)
    gen = torch.Generator(device=dev).manual_seed(10 + rank)
    x = torch.randn(b1 - b0, 3, 224, 224, generator=gen, device=dev)
    y = torch.randint(0, 101, (b1 - b0,), generator=gen, device=dev)
    torch.manual_seed(0)
    extra_cfg, roof = {}, None
    if kind == "qat":
        model, ctrl = workloads.build_resnet18(101)
        model.to(dev).train()
        for e in range(1, 45):
            ctrl.step(e)
        # gradients of the last layers are all-reduced (25 MB buckets) while backward still works on the first ones
        bucket = tdist.FlatGradBucket(model.parameters(), bucket_bytes=25 << 20) if world > 1 else None
        if fused_optimizer:      # Adam + clamp as one multi-tensor launch (plus one for the unclamped parameters)
            opt = workloads.fused_optimizer(model, ctrl, lr=1e-3, bucket=bucket)
        else:
            opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        ms = ctx.timed(lambda i: workloads.qat_step(model, ctrl, opt, x, y, bucket), steps, warmup)
        metric = "resnet18_qat_images_per_s"
        sharding = "data parallel, fp32 gradients in one flat buffer, all-reduced in 25 MB buckets from gradient hooks"
        if fused_optimizer:
            sharding += "; fused multi-tensor Adam + clamp"
        if world > 1:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(3):
                ctx.dist.all_reduce(bucket.flat)
            torch.cuda.synchronize()
            extra_cfg["allreduce_alone_ms"] = (time.perf_counter() - t0) / 3 * 1e3
            extra_cfg["gradient_bytes"] = bucket.flat.numel() * 4
        # share of the step spent in this library's kernels (soft-step forward / backward of 21 layers, loss, clamp)
        w_elems = sum(n.weight.numel() for n in ctrl._registry.values())
        extra_cfg["quantized_weights"] = w_elems
    else:
        model, ctrl = workloads.build_resnet18(101, ctrl=tmq.QuantizationControl())
        with torch.no_grad():
            for node in ctrl._registry.values():
                u = torch.rand(node.weight.shape)
                node.weight.copy_(torch.where(u < 0.35, -1.0, torch.where(u < 0.65, 0.0, 1.0)))
        model.to(dev).eval()
        tmq.compressed_state_dict(model)
        net = workloads.PackedResNet18(model)
        ms = ctx.timed(lambda i: net(x), steps, warmup)
        # the same pass replayed as one CUDA graph (input copy included): what counts when the per-GPU batch is small
        try:
            graphed = workloads.GraphedInference(net, x)
            same = bool(torch.equal(graphed(x), net(x)))
            ms_graph = ctx.timed(lambda i: graphed(x), steps, warmup)
            extra_cfg["launch_by_launch_ms"] = ms
            extra_cfg["cuda_graph_ms"] = ms_graph
            extra_cfg["cuda_graph_equals_launches"] = same
            if same and ms_graph < ms:
                ms = ms_graph
                extra_cfg["timed"] = "CUDA graph replay of the whole pass, input copy included"
        except Exception as err:                               # noqa: BLE001 - the launch-by-launch number stays
            extra_cfg["cuda_graph_error"] = f"{type(err).__name__}: {err}"[:200]
        ops.check_gemm_status(dev)
        metric, sharding = "resnet18_packed_inference_images_per_s", "batch sharded, no collective"
        roof = _resnet_layer_roofline(net, b1 - b0, ctx.peaks, ms)
        if per_layer:
            roof["per_layer"] = _resnet_per_layer(net, x, ctx.peaks)
    line = {"metric": metric, "value": batch / (ms * 1e-3), "unit": "images/s", "n_gpus": world, "steps": steps,
            "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32" if kind == "qat" else "bf16", "data": "synthetic",
            "config": dict({"workload": f"resnet18_101cls_batch{batch}_224x224", "sharding": sharding,
                            "macs_per_batch": 4.643e11 * batch / 256}, **extra_cfg)}
    if roof is not None:
        line["roofline"] = roof
    return line


def run_workload(args):
    """Secondary workloads, same launch contract: --workload gemm | gemv | resnet_qat | resnet_infer | dwconv | ..."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the tmq_b200 kernels have no CPU fallback")
    dist, rank, local, world = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from tmq_b200 import ops
    ctx = _Ctx(dist, rank, world, dev)
    peaks, peak_kind, timed = ctx.peaks, ctx.peak_kind, ctx.timed

    if args.workload == "gemv":
        # decode-like config through the C ABI, distinct matrices so that L2 cannot hold them (profiling helper)
        from tmq_b200 import _lib
        Lb = _lib.lib()
        N, K, NM, Mg = 11008, 4096, args.gemv_matrices, args.gemv_rows
        wts = [ops.prepack(_ternary_packed(ops, N, K, 100 + i), N, ops.FMT_BF16) for i in range(NM)]
        scale = torch.rand(N, device=dev) * 0.09 + 0.01
        X = torch.randn(Mg, K, device=dev).to(torch.bfloat16)
        Y = torch.empty(Mg, N, device=dev, dtype=torch.bfloat16)
        status = ops.gemm_status_word(X.device)
        st = torch.cuda.current_stream().cuda_stream

        def sweep(i):
            for wt in wts:
                for m0 in range(0, Mg, GEMV_ROWS_PER_PASS):
                    rc = Lb.tmq_ternary_gemv_bf16(X.data_ptr() + m0 * K * 2, wt.data_ptr(), scale.data_ptr(), None,
                                                  Y.data_ptr() + m0 * N * 2, min(GEMV_ROWS_PER_PASS, Mg - m0), N, K, N, 0,
                                                  status.data_ptr(), st)
                    assert rc == 0
        ms = timed(sweep, args.steps, args.warmup) / NM
        nbytes = N * K // 4 + 2 * Mg * K + 2 * Mg * N + 4 * N
        line = {"metric": "ternary_gemv_bf16_GBps", "value": nbytes / ms / 1e6, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"ternary_gemv_M{Mg}_N11008_K4096", "matrices": NM,
                           "note": "stream launches (no CUDA graph): includes launch gaps; the headline GEMV number is "
                                   "the graph protocol of the default run"}}
    elif args.workload == "gemv_batched":
        # the same decode-like config through the batched entry point: --gemv-group matrices per launch, int8 or bf16
        from tmq_b200 import _lib
        Lb = _lib.lib()
        N, K, NM, Mg, G = 11008, 4096, args.gemv_matrices, args.gemv_rows, args.gemv_group
        i8 = args.gemv_dtype == "i8"
        fmt = ops.FMT_I8 if i8 else ops.FMT_BF16
        wts = [ops.prepack(_ternary_packed(ops, N, K, 100 + i), N, fmt) for i in range(NM)]
        X = torch.randint(-127, 128, (Mg, K), device=dev, dtype=torch.int8) if i8 else torch.randn(Mg, K, device=dev).to(torch.bfloat16)
        Ys = [torch.empty(Mg, N, device=dev, dtype=torch.int32 if i8 else torch.bfloat16) for _ in range(NM)]
        status = ops.gemm_status_word(X.device)
        st = torch.cuda.current_stream().cuda_stream

        def parr(ts):
            arr = (ctypes.c_void_p * len(ts))()
            for i, t in enumerate(ts):
                arr[i] = t.data_ptr()
            return arr
        groups = [(parr(wts[i:i + G]), parr(Ys[i:i + G]), len(wts[i:i + G])) for i in range(0, NM, G)]

        def sweep(i):
            for Wp, Yp, n in groups:
                if i8:
                    rc = Lb.tmq_ternary_gemv_batched_i8(X.data_ptr(), 0, Wp, Yp, n, Mg, N, K, N, status.data_ptr(), st)
                else:
                    rc = Lb.tmq_ternary_gemv_batched_bf16(X.data_ptr(), 0, Wp, None, None, Yp, n, Mg, N, K, N, 0,
                                                          status.data_ptr(), st)
                assert rc == 0
        ms = timed(sweep, args.steps, args.warmup) / NM
        nbytes = N * K // 4 + (1 if i8 else 2) * Mg * K + (4 if i8 else 2) * Mg * N
        line = {"metric": f"ternary_gemv_batched_{args.gemv_dtype}_GBps", "value": nbytes / ms / 1e6, "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.gemv_dtype,
                "data": "synthetic",
                "config": {"workload": f"ternary_gemv_batched_M{Mg}_N11008_K4096", "matrices": NM, "per_launch": G}}
    elif args.workload == "qat_linear":
        # training forward of a QAT Linear layer with the staircase fused into the operand load (profiling helper)
        N = K = 4096
        Mq = args.qat_rows
        ws = [torch.rand(N, K, device=dev) * 2.5 - 1.25 for _ in range(8)]
        x = torch.randn(Mq, K, device=dev).to(torch.bfloat16)
        ms = timed(lambda i: ops.qat_linear_forward(x, ws[i % 8], None, 5.0), args.steps, args.warmup)
        line = {"metric": "qat_linear_fwd_weights_per_us", "value": N * K / ms / 1e3, "unit": "weights/us", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"qat_linear_fwd_M{Mq}_N4096_K4096", "weights": "8 distinct fp32 matrices (537 MB)"}}
    elif args.workload in ("dwconv", "dwconvtrans"):
        # depthwise compact convolution straight from the image: MobileNet-like 3x3, fp32 NCHW, batch sharded over ranks
        Bt, C, H, W = 256 // world, 128, 56, 56
        gen = torch.Generator(device=dev).manual_seed(rank)
        Wt = torch.randint(-1, 2, (C, 1, 3, 3), generator=gen, device=dev).float()
        Pk = ops.compactify_ternary(Wt)
        sc = torch.rand(C, generator=gen, device=dev) + 0.5
        bi = torch.randn(C, generator=gen, device=dev)
        xs = [torch.randn(Bt, C, H, W, generator=gen, device=dev) for _ in range(2)]      # 2 x 411 MB > L2
        if args.workload == "dwconv":
            fn = lambda x: ops.ternary_dwconv2d(x, Pk, (3, 3), (1, 1), (1, 1), (1, 1), sc, bi)
        else:
            fn = lambda x: ops.ternary_dwconvtrans2d(x, Pk, (3, 3), (1, 1), (1, 1), (1, 1), (0, 0), sc, bi)
        y = fn(xs[0])
        ms = timed(lambda i: fn(xs[i & 1]), args.steps, args.warmup)
        nbytes = xs[0].numel() * 4 + y.numel() * 4
        line = {"metric": f"ternary_{args.workload}2d_f32_GBps", "value": world * nbytes / ms / 1e6, "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"depthwise_3x3_B{Bt * world}_C{C}_{H}x{W}", "l2": "two alternating inputs of 411 MB"},
                "gpu_launches": args.steps,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind,
                             "algorithmic_bytes_per_launch": nbytes}}
    elif args.workload == "adam":
        # fused multi-tensor Adam + clamp: 64 tensors of 2^19 elements (w, g, m, v: 537 MB > L2), 28 bytes per element
        gen = torch.Generator(device=dev).manual_seed(rank)
        params = [torch.nn.Parameter(torch.rand(1 << 19, generator=gen, device=dev) * 2.4 - 1.2) for _ in range(64)]
        opt = ops.MultiTensorAdam(params, lr=1e-3, clamp_params=params, clamp=(-1.0, 1.0))
        opt.grad.copy_(torch.randn(opt.grad.numel(), generator=gen, device=dev))
        ms = timed(lambda i: opt.step(), args.steps, args.warmup)
        nbytes = 28 * sum(p.numel() for p in params)
        line = {"metric": "fused_adam_clamp_GBps", "value": world * nbytes / ms / 1e6, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "multi_tensor_adam_clamp_64x2^19", "l2": "537 MB of state per step"},
                "gpu_launches": args.steps,
                "roofline": {"bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": nbytes / ms / 1e6 / peaks["hbm_gbs"], "traffic": None, "peak_source": peak_kind,
                             "algorithmic_bytes_per_launch": nbytes}}
    elif args.workload == "gemm":
        line = wl_gemm(ctx, args.steps, args.warmup, args.gemm_m, args.gemm_k, args.gemm_n,
                       chunks=args.gemm_chunks if args.gemm_chunks > 0 else None)
    elif args.workload in ("resnet_qat", "resnet_infer"):
        line = wl_resnet(ctx, "qat" if args.workload == "resnet_qat" else "infer", args.steps, args.warmup, args.batch,
                         args.fused_optimizer, per_layer=args.per_layer)
    else:
        raise SystemExit(f"unknown workload {args.workload}")
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n", type=int, default=1 << 26, help="elements per GPU (default: the baseline's 2^26)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the ternary GEMM / GEMV sections")
    ap.add_argument("--workload", default="softstep", choices=["softstep", "gemm", "gemv", "gemv_batched", "qat_linear", "resnet_qat", "resnet_infer", "dwconv",
                             "dwconvtrans", "adam"])
    ap.add_argument("--gemm-m", type=int, default=8192)
    ap.add_argument("--gemm-k", type=int, default=8192)
    ap.add_argument("--gemm-n", type=int, default=28672)
    ap.add_argument("--batch", type=int, default=256, help="images per step of the ResNet workloads")
    ap.add_argument("--fused-optimizer", action="store_true", help="resnet_qat: multi-tensor Adam with the clamp fused in")
    ap.add_argument("--gemm-chunks", type=int, default=0, help="row chunks of the column-sharded GEMM (0: default)")
    ap.add_argument("--per-layer", action="store_true", help="resnet_infer: time every layer alone as well")
    ap.add_argument("--gemv-rows", type=int, default=1)
    ap.add_argument("--gemv-matrices", type=int, default=32)
    ap.add_argument("--gemv-group", type=int, default=16, help="matrices per launch of --workload gemv_batched")
    ap.add_argument("--gemv-dtype", default="bf16", choices=["bf16", "i8"])
    ap.add_argument("--qat-rows", type=int, default=64, help="activation rows of --workload qat_linear")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload != "softstep":
        run_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
