#!/usr/bin/env python
"""Benchmark of the NVFP4 block-scaled matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1|c2|c3|c4]

A step is one pass of the hot path over one batch of seeded synthetic input (the leaderboard
harness that generated the reference's inputs is not part of the reference; see
nvfp4_gemm_b200/inputs.py).  At N = 1 the workload is the decode-shaped GEMM the reference's
numbers are quoted on (M=128, N=7168, K=16384, L=1).  At N > 1 the workload is the only one the
path partitions: M=8192, N=28672, K=8192 split column-parallel over N, with the fp16 column
blocks all-gathered (strong scaling: total work fixed).

Rank 0 prints ONE JSON line.  `value` is device-timed throughput with inputs resident in HBM;
`e2e` times the public `custom_kernel` call with host buffers, copies included.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    "c0": dict(m=128, n=256, k=256, l=1, bound="hbm", name="C0 CPU-runnable GEMM m128 n256 k256 l1"),
    "c1": dict(m=128, n=7168, k=16384, l=1, bound="hbm", name="C1 decode GEMM m128 n7168 k16384 l1"),
    "c2": dict(m=7168, n=1, k=16384, l=4, bound="hbm", name="C2 GEMV m7168 k16384 l4"),
    "c3": dict(m=4096, n=7168, k=7168, l=1, bound="tensor", name="C3 prefill GEMM m4096 n7168 k7168 l1"),
    "c4": dict(m=8192, n=28672, k=8192, l=1, bound="tensor", name="C4 GEMM m8192 n28672 k8192 l1 (column-parallel over N)"),
}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (one capture per kernel and workload).
NCU_DRAM_BYTES_PER_LAUNCH = {"c1": 68.3e6, "c2": 268.0e6, "c3": 132.3e6, "c4": 804.6e6}
# The reference task's other timed shapes with the speed-of-light figures its statement gives for
# them (task.yml:29-33, task_gemv.yml:29-33: max(math, DRAM) of a B200 at 1.5 GHz), reported as
# extra rows beside the headline.
LEADERBOARD = {
    "c1": dict(sol_us=8.994),
    "gemm_m128_n4096_k7168": dict(m=128, n=4096, k=7168, l=1, sol_us=2.354),
    "gemm_m128_n7168_k2048": dict(m=128, n=7168, k=2048, l=1, sol_us=1.333),
    "gemv_m7168_k16384_l1": dict(m=7168, n=1, k=16384, l=1, sol_us=8.622),
    "gemv_m4096_k7168_l8": dict(m=4096, n=1, k=7168, l=8, sol_us=17.275),
    "gemv_m7168_k2048_l4": dict(m=7168, n=1, k=2048, l=4, sol_us=4.317),
}
# Data-movement kernels beside the path, timed on one GPU against the HBM copy peak.
AUX_WORKLOADS = {
    "quantize": "NVFP4 quantiser, bf16 8192 x 28672 -> packed e2m1 + plain and permuted e4m3 scales",
    "exchange_copy": "copy kernel of the per-panel all-gather, 7 column blocks of 8192 x 3584 fp16 inside 8192 x 28672, source and destination on this GPU",
}
FP4_DENSE_PEAK_TFLOPS = 9000.0   # nominal dense FP4 tensor peak of one B200 (no measured FP4 figure exists)


def algorithmic_flops(w):
    return 2.0 * w["m"] * w["n"] * w["k"] * w["l"]


def algorithmic_bytes(w):
    m, n, k, l = w["m"], w["n"], w["k"], w["l"]
    return l * (m * k / 2 + n * k / 2 + m * k / 16 + n * k / 16 + 2 * m * n)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return dict(sm_mhz=(sm[len(sm) // 2] if sm else None), sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))


class CpuSample:
    """A bounded slice of a workload for the CPU oracle (C restatement; the reference has no CPU
    code for this path): all K, the first `rows` rows of A against the first `cols` rows of B,
    with `cols` wide enough that every host thread gets a 64-column panel of its own.  Inputs are
    generated once, outside anything that is timed."""

    def __init__(self, w, threads=0):
        from nvfp4_gemm_b200.inputs import generate_input
        from oracle import nvfp4_oracle as O
        O.build_c()
        self.O = O
        self.cores = threads or O.c_max_threads()
        k, n_full = w["k"], w["n"]
        if n_full > 1:
            self.rows = min(w["m"], 128)
            self.cols = min(n_full, max(256, 64 * self.cores))
        else:                                  # GEMV: one B row; the oracle's panels are over B rows, so one thread works
            self.rows, self.cols = min(w["m"], 2048), 1
        self.k, self.n_full = k, n_full
        self.threads_used = max(1, min(self.cores, -(-self.cols // 64)))
        data = generate_input(self.rows, self.cols, k, 1, 1111, device="cpu")
        self.args = O.tensors_to_numpy(data)
        self.flops = 2.0 * self.rows * self.cols * k

    def run_once(self, threads=None):
        t0 = time.perf_counter()
        self.O.ref_gemm_c(*self.args, threads=threads or self.cores)
        return time.perf_counter() - t0

    def describe(self, reps):
        return (f"{self.rows}x{self.cols}x{self.k} slice of the workload (all K, first {self.cols} of {self.n_full} B rows), "
                f"{reps} repeats, {self.threads_used} threads busy")


def cpu_baseline_sample(w, threads=0, budget_s=12.0):
    s = CpuSample(w, threads)
    dt = s.run_once()
    reps = int(max(1, min(20, budget_s / max(dt, 1e-3))))
    dt = sum(s.run_once() for _ in range(reps)) / reps
    return dict(tflops=s.flops / dt / 1e12, seconds=dt, cores=s.threads_used, sample=s.describe(reps))


def cpu_config0_row():
    """Config 0 (the CPU-runnable 128 x 256 x 256 GEMM) on the host: all threads and one thread."""
    s = CpuSample(WORKLOADS["c0"])
    s.run_once()
    reps = 50
    t_all = min(s.run_once() for _ in range(reps))
    t_one = min(s.run_once(threads=1) for _ in range(reps))
    return dict(us=t_all * 1e6, threads=s.threads_used, us_one_thread=t_one * 1e6, gflops=s.flops / t_all / 1e9,
                gflops_one_thread=s.flops / t_one / 1e9, kind="port", timing="best of 50, time.perf_counter around the C oracle call")


def run_reference_arm(args, w):
    """The 'reference' arm: the path's CPU implementation on the host cores.  The reference has no
    CPU code (and its harness ref_kernel is absent), so this is the oracle port.  A step is one
    pass over the bounded slice; inputs are generated before anything is timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = CpuSample(w)
    # size the sample so that warm-up + K steps end within about two minutes
    while s.run_once() * (args.steps + args.warmup) > 120.0 and s.rows > 8:
        s = CpuSample(dict(w, m=s.rows // 2))
    for _ in range(args.warmup):
        s.run_once()
    steps = args.steps
    times = [s.run_once() for _ in range(steps)]
    dt = sum(times) / len(times)
    value = s.flops / dt / 1e12
    line = dict(impl="reference", metric="nvfp4_matmul_throughput", value=value, unit="TFLOP/s", n_gpus=args.gpus,
                steps=steps, warmup=args.warmup, ms_per_step=1e3 * dt,
                higher_is_better=True, scaling="strong" if args.gpus > 1 else "weak", vs_baseline=None, dtype="e2m1 x ue4m3 -> f32 -> f16",
                data="synthetic", config=dict(workload=w["name"]),
                cpu_baseline=dict(value=value, unit="TFLOP/s", cores=s.threads_used, kind="port", sample=s.describe(steps)),
                e2e=dict(value=value, unit="TFLOP/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS) + sorted(AUX_WORKLOADS),
                    help="default: c1 on one GPU, c4 on several; 'quantize' and 'exchange_copy' time the data-movement kernels beside the path (one GPU)")
    ap.add_argument("--allgather", default="auto", choices=["auto", "fused", "push", "pull", "ce", "nccl"],
                    help="N > 1: how the column blocks are exchanged.  fused = peer stores in the GEMM epilogue; push / pull = "
                         "this library's copy kernel per row panel on a second stream; ce = copy engines; nccl = NCCL + re-layout; "
                         "auto = fused on 2 GPUs, push on more (the measured best of each)")
    ap.add_argument("--panels", type=int, default=0, help="N > 1: row panels the exchange is pipelined over (all modes but fused); 0 = the measured best")
    ap.add_argument("--copy-sms", type=int, default=-1, help="N > 1, push / pull: SMs reserved for the copy kernel (the GEMM runs on the rest); -1 = the measured best")
    ap.add_argument("--peer-tma", type=int, default=-1, help="N > 1, fused: peers served by tensor stores instead of the epilogue warps' own stores; -1 = the library default")
    ap.add_argument("--nvfp4-out", action="store_true", help="N = 1, GEMM workloads: time the re-quantising epilogue variant (NVFP4 output) instead")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary per-config table")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    wl_key = args.workload or ("c1" if args.gpus == 1 else "c4")
    if wl_key in AUX_WORKLOADS:
        bench_aux(args, wl_key)
        return
    w = WORKLOADS[wl_key]
    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    import torch
    from nvfp4_gemm_b200 import submission as S
    from nvfp4_gemm_b200.inputs import generate_input

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    if world > 1:
        bench_column_parallel(args, w, rank, world, dev)
        return

    peaks = measured_peaks()
    l2_bytes = torch.cuda.get_device_properties(dev).L2_cache_size
    set_bytes = algorithmic_bytes(w)
    n_sets = int(min(8, max(3, -(-3 * l2_bytes // int(set_bytes)))))   # rotate over > 3x L2 of inputs
    sets = [generate_input(w["m"], w["n"], w["k"], w["l"], 1111 + i, device=dev) for i in range(n_sets)]

    if args.nvfp4_out:
        # the GEMM with the re-quantising epilogue (packed e2m1 + scales instead of fp16): a variant
        # for profiling and comparison, not the default workload
        q_out = [S.gemm_epilogue(s[:6] + (None,), nvfp4_out=True) for s in sets]

        def step(i):
            return S.gemm_epilogue(sets[i % n_sets][:6] + (None,), nvfp4_out=True, out=q_out[i % n_sets])
    else:
        def step(i):
            return S.custom_kernel(sets[i % n_sets])

    for i in range(args.warmup):
        step(i)
    S.check_status()
    torch.cuda.synchronize()

    # The K timed steps are K kernel launches recorded once into a CUDA graph (the library takes
    # the capture stream like any other stream) and replayed between two events: the timed region
    # is device time of exactly K passes, free of Python call overhead.
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    launches0 = S.launch_count()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(args.steps):
                step(i)
    launches = S.launch_count() - launches0          # kernels recorded = kernels each replay launches
    torch.cuda.synchronize()
    graph.replay()                                   # untimed replay: graph upload, clocks up
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    sampler.start()
    reps = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        reps.append(e0.elapsed_time(e1))
    # keep the same load running (untimed) until the clock sampler has seen it for ~0.6 s: the timed
    # replays alone are a few milliseconds, shorter than nvidia-smi's sampling period
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 0.6:
        graph.replay()
        torch.cuda.synchronize()
    S.check_status()
    kernel_name = S.last_kernel()
    isolated_us = isolated_launch_us(lambda i: step(i), n_sets)
    reps.sort()
    total_ms = reps[len(reps) // 2]                  # median of 5 timed regions of K steps each
    per_launch_ms = [r / args.steps for r in reps]

    ms_per_step = total_ms / args.steps
    flops = algorithmic_flops(w)
    byts = algorithmic_bytes(w)
    tflops = flops / (ms_per_step * 1e-3) / 1e12
    gbs = byts / (ms_per_step * 1e-3) / 1e9

    # ---- end to end through custom_kernel with host buffers (pinned), copies inside the timed region
    def _raw(t):
        # the tensors are dense permutations of contiguous storage: view them as flat memory
        return torch.as_strided(t.view(torch.uint8) if t.element_size() == 1 else t, (t.numel(),), (1,))

    host_sets = [[_raw(t).cpu().pin_memory() for t in s[:6]] for s in sets[:2]]
    # Two device-side input/output sets and three streams: the copy-in of step i + 1 runs while
    # step i computes and its result is read back (every step still copies all its inputs in and
    # its whole result out; the steps are pipelined, as a serving loop would run them).
    dev_bufs = [[torch.empty_like(t) for t in sets[0]] for _ in range(2)]
    c_hosts = [torch.empty(sets[0][6].numel(), dtype=torch.float16).pin_memory() for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in host_sets[0])
    d2h = c_hosts[0].numel() * c_hosts[0].element_size()
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b = i % 2
        hs = host_sets[i % len(host_sets)]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[b])          # the kernel that last read this input set is done
            for j in range(6):
                _raw(dev_bufs[b][j]).copy_(hs[j], non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            s_run.wait_event(ev_out[b])         # the previous result in this output buffer has been read back
            S.custom_kernel(tuple(dev_bufs[b]))
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            c_hosts[b].copy_(_raw(dev_bufs[b][6]), non_blocking=True)
            ev_out[b].record(s_out)

    e2e_steps = max(3, min(args.steps, 20))
    for i in range(4):
        e2e_step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()                                  # on the current (default) stream, which the three streams are ordered against below
    for st in (s_in, s_run, s_out):
        st.wait_stream(torch.cuda.current_stream())
    for i in range(e2e_steps):
        e2e_step(i)
    for st in (s_in, s_run, s_out):
        torch.cuda.current_stream().wait_stream(st)
    e1.record()
    torch.cuda.synchronize()
    S.release_stream(s_run)
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks = sampler.stop()

    if w["bound"] == "hbm":
        roofline = dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"],
                        traffic=None, peak_source=peaks["source"], kernel=kernel_name)
    else:
        roofline = dict(bound="tensor", achieved=tflops, peak=FP4_DENSE_PEAK_TFLOPS, unit="TFLOP/s",
                        frac=tflops / FP4_DENSE_PEAK_TFLOPS, traffic=None, peak_source="nominal dense FP4", kernel=kernel_name)
    roofline["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(wl_key)

    line = dict(metric="nvfp4_matmul_throughput", value=tflops, unit="TFLOP/s", n_gpus=1, steps=args.steps,
                warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True, scaling="weak",
                # against the fastest time the reference project published for this shape on a B200:
                # its cuBLASLt submission, 22.6 us (out_cub.txt:16-18); its own kernels took 144 and 459 us
                vs_baseline=(tflops / (flops / 22.6e-6 / 1e12)) if wl_key == "c1" else None,
                dtype="e2m1 x ue4m3 -> f32 -> f16", data="synthetic",
                config=dict(workload=w["name"] + (" [NVFP4 output variant]" if args.nvfp4_out else ""), timing=f"CUDA events around a CUDA-graph replay of the K steps, median of 5; {n_sets} rotating input sets = {n_sets * set_bytes / 1e6:.0f} MB > L2 {l2_bytes / 1e6:.0f} MB",
                            us_per_step=ms_per_step * 1e3, us_per_step_best_of_5=per_launch_ms[0] * 1e3, gb_per_s=gbs,
                            isolated_launch_us=isolated_us,
                            isolated_launch_timing="one launch between two CUDA events, stream synchronised before each, no graph, inputs rotating (cold L2); median of 60",
                            reference_published_us={"cuBLASLt": 22.6, "cute_dsl_template": 144.0, "hand_written_tcgen05": 459.0} if wl_key == "c1" else None),
                roofline=roofline,
                e2e=dict(value=flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=e2e_ms, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                         note="every step copies its six inputs from pinned host memory and its result back; steps are pipelined over three streams and two buffer sets"),
                gpu_launches=int(launches), clocks=clocks)

    del graph
    S.release_stream(side)            # the timed graph is gone: give its stream's scratch set back
    if not args.no_extra:
        del sets, host_sets, dev_bufs
        torch.cuda.empty_cache()
        line["other_configs"] = extra_table(S, generate_input, dev, peaks, local_rank)
    if not args.no_cpu_baseline:
        cb = cpu_baseline_sample(w)
        line["cpu_baseline"] = dict(value=cb["tflops"], unit="TFLOP/s", cores=cb["cores"], kind="port", sample=cb["sample"])
        if not args.no_extra:
            line["other_configs"]["c0_cpu_128x256x256"] = cpu_config0_row()
    print(json.dumps(line), flush=True)


def bench_aux(args, key):
    """HBM-bound helper kernels (one GPU): achieved GB/s of algorithmic bytes against the measured copy peak."""
    import ctypes
    import torch
    from nvfp4_gemm_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream().cuda_stream
    peaks = measured_peaks()
    m, n = 8192, 28672
    if key == "quantize":
        xs = [torch.randn((m, n), device=dev, dtype=torch.bfloat16) for _ in range(2)]       # 2 x 470 MB > L2
        packed = torch.empty((m, n // 2), dtype=torch.uint8, device=dev)
        sf = torch.empty((m, n // 16), dtype=torch.uint8, device=dev)
        perm = torch.empty(((m // 128) * (n // 64) * 512,), dtype=torch.uint8, device=dev)
        byts = m * n * 2 + m * n // 2 + 2 * (m * n // 16)

        def step(i):
            x = xs[i % 2]
            _lib.check(lib.nvfp4_quantize(x.data_ptr(), 1, packed.data_ptr(), sf.data_ptr(), perm.data_ptr(), m, n, n, n // 2, n // 16, stream))
    else:
        g = 8
        nl = n // g
        src = [torch.randn((m, n), device=dev).half() for _ in range(2)]
        dst = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(2)]
        byts = 2 * (g - 1) * m * nl * 2

        def ptrs(t):
            return (ctypes.c_void_p * (g - 1))(*[t.data_ptr() + (b + 1) * nl * 2 for b in range(g - 1)])
        tables = [(ptrs(dst[i]), ptrs(src[i])) for i in range(2)]

        def step(i):
            d, s_ = tables[i % 2]
            _lib.check(lib.nvfp4_copy_column_blocks(d, s_, g - 1, 0, m, nl, n, 0, 0, stream))
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = lib.nvfp4_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    launches = lib.nvfp4_launch_count() - launches0
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    gbs = byts / (ms * 1e-3) / 1e9
    print(json.dumps(dict(metric="hbm_bytes_per_second", value=gbs, unit="GB/s", n_gpus=1, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
                          higher_is_better=True, scaling="weak", vs_baseline=None, dtype="u8", data="synthetic",
                          config=dict(workload=AUX_WORKLOADS[key], timing="CUDA events around K back-to-back launches, two rotating buffer sets > L2"),
                          roofline=dict(bound="hbm", achieved=gbs, peak=peaks["hbm_gbs"], unit="GB/s", frac=gbs / peaks["hbm_gbs"], traffic=None,
                                        peak_source=peaks["source"]),
                          gpu_launches=int(launches), clocks=clocks)), flush=True)


def isolated_launch_us(fn, n_sets, n=60):
    """Latency one launch sees on its own: events around a single call, the stream drained before
    each, no CUDA graph (so no overlap with a neighbouring launch), inputs rotating through more
    than L2.  Includes the launch overhead a lone call pays."""
    import torch
    ts = []
    for i in range(n + 5):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(i % n_sets)
        e1.record()
        torch.cuda.synchronize()
        if i >= 5:
            ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def extra_table(S, generate_input, dev, peaks, gpu_index):
    """Device-timed µs / TFLOPS / GB/s for the other single-GPU configurations and the same-GPU
    cuBLASLt comparator (torch._scaled_mm), reported beside the headline line.  Every row carries
    the SM clock sampled while that row's kernels ran."""
    import torch
    out = {}

    def time_fn(fn, n_sets, inner=4):
        for i in range(n_sets):
            fn(i)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for _ in range(inner):
                    for i in range(n_sets):
                        fn(i)
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(7):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / (inner * n_sets) * 1e3)
        # keep the row's load up long enough for the clock sampler (100 ms period) to see it
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < 0.35:
            g.replay()
            torch.cuda.synchronize()
        ts.sort()
        del g
        S.release_stream(side)        # the graph is gone: its stream's scratch set can serve another stream
        return ts[0], ts[len(ts) // 2]

    def flat(t):
        return torch.as_strided(t.view(torch.uint8), (t.numel(),), (1,)).view(t.dtype)

    shapes = {key: WORKLOADS[key] for key in ("c1", "c2", "c3")}
    shapes.update({key: v for key, v in LEADERBOARD.items() if "m" in v})
    shapes["c4_one_gpu"] = WORKLOADS["c4"]
    for key, w in shapes.items():
        # enough rotating input sets to exceed 3x L2 (126 MB), so every launch reads HBM
        n_sets = int(min(48, max(2 if key == "c4_one_gpu" else 3, -(-400e6 // algorithmic_bytes(w)))))
        sets = [generate_input(w["m"], w["n"], w["k"], w["l"], 2000 + i, device=dev) for i in range(n_sets)]
        sampler = ClockSampler(gpu_index)
        sampler.start()
        us, us_median = time_fn(lambda i: S.custom_kernel(sets[i % n_sets]), n_sets, inner=2 if key == "c4_one_gpu" else 4)
        clk = sampler.stop()
        rec = dict(us=us, us_median=us_median, tflops=algorithmic_flops(w) / us / 1e6, gb_per_s=algorithmic_bytes(w) / us / 1e3, kernel=S.last_kernel())
        rec["frac_hbm_measured"] = rec["gb_per_s"] / peaks["hbm_gbs"]
        rec["frac_fp4_nominal"] = rec["tflops"] / FP4_DENSE_PEAK_TFLOPS
        rec["input_sets"] = n_sets
        rec["clocks"] = dict(sm_mhz=clk.get("sm_mhz"), reasons=clk.get("reasons"), samples=clk.get("samples"))
        sol = LEADERBOARD.get(key, w).get("sol_us")
        if sol:
            rec["task_sol_us_at_1500mhz"] = sol
            rec["sol_over_measured"] = sol / us
        if key in ("c3", "c4_one_gpu"):
            # the same GEMM with the result re-quantised to NVFP4 in the epilogue (bias / activation off)
            q_out = [S.gemm_epilogue(s[:6] + (None,), nvfp4_out=True) for s in sets]
            qus, _ = time_fn(lambda i: S.gemm_epilogue(sets[i % n_sets][:6] + (None,), nvfp4_out=True, out=q_out[i % n_sets]), n_sets,
                             inner=2 if key == "c4_one_gpu" else 4)
            rec["nvfp4_output_us"] = qus
            rec["nvfp4_output_kernel"] = S.last_kernel()
            del q_out
        if w["m"] <= 128 and w["n"] > 1:
            rec["isolated_launch_us"] = isolated_launch_us(lambda i: S.custom_kernel(sets[i % n_sets]), n_sets)
        if w["n"] > 1:
            try:
                ar = [(s[0][:, :, 0], s[1][:, :, 0].t(), flat(s[4]), flat(s[5])) for s in sets]
                outs = [torch.empty((w["m"], w["n"]), dtype=torch.float16, device=dev) for _ in sets]
                cus, cus_median = time_fn(lambda i: torch._scaled_mm(*ar[i % n_sets], out_dtype=torch.float16, out=outs[i % n_sets]), n_sets,
                                          inner=2 if key == "c4_one_gpu" else 4)
                rec["cublaslt_us"] = cus
                rec["cublaslt_us_median"] = cus_median
                rec["cublaslt_tflops"] = algorithmic_flops(w) / cus / 1e6
                if w["m"] <= 128:
                    rec["cublaslt_isolated_launch_us"] = isolated_launch_us(
                        lambda i: torch._scaled_mm(*ar[i % n_sets], out_dtype=torch.float16, out=outs[i % n_sets]), n_sets)
                del ar, outs
            except Exception as e:  # noqa: BLE001
                rec["cublaslt_us"] = None
                rec["cublaslt_error"] = str(e)[:200]
        out[key] = rec
        del sets
        torch.cuda.empty_cache()
    S.check_status()
    return out


def default_exchange(world):
    """Measured-best exchange settings per GPU count (B200 / NVSwitch, the 8192 x 28672 x 8192 job):
    (mode, row panels, SMs given to the copy kernel)."""
    return {2: ("fused", 4, 0), 4: ("fused", 4, 0), 8: ("push", 4, 0)}.get(world, ("push", 4, 0))


def bench_column_parallel(args, w, rank, world, dev):
    """`bench.py --gpus N` for N > 1: strong scaling of the one partitioned workload."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from nvfp4_gemm_b200 import submission as S
    from nvfp4_gemm_b200.inputs import generate_input
    from nvfp4_gemm_b200.multi_gpu import (ColumnParallelGemm, CopyEngineAllGatherGemm, FusedAllGatherGemm, PanelAllGatherGemm,
                                           plan_shard, shard_inputs, to_device_same_layout)

    m, n, k = w["m"], w["n"], w["k"]
    shard = plan_shard(n, world, rank)
    if args.peer_tma >= 0:
        from nvfp4_gemm_b200 import _lib
        _lib.load().nvfp4_set_peer_tma_limit(args.peer_tma)
    # every rank builds the same full B from the seed and keeps its rows (inputs are synthetic)
    n_sets = 2
    sets, host_sets = [], []
    for i in range(n_sets):
        full = generate_input(m, n, k, 1, 1111 + i, device="cpu")
        local = shard_inputs(full, shard)
        host_sets.append([_flat_bytes(t).clone().pin_memory() for t in local[:6]])
        sets.append(tuple(to_device_same_layout(t, dev) for t in local[:6]) + (None,))
        del full
    mode, panels, copy_sms = default_exchange(world)
    if args.allgather != "auto":
        mode = args.allgather
    if args.panels > 0:
        panels = args.panels
    if args.copy_sms >= 0:
        copy_sms = args.copy_sms

    def build(mode, nvfp4_out=False):
        if mode == "fused":
            return FusedAllGatherGemm(m, n, k, device=dev)
        if mode == "ce":
            return CopyEngineAllGatherGemm(m, n, k, device=dev, panels=panels)
        if mode in ("pull", "push"):
            return PanelAllGatherGemm(m, n, k, device=dev, panels=panels, direction=mode, copy_sms=copy_sms, nvfp4_out=nvfp4_out)
        return None

    note = ""
    try:
        plan = build(mode)
    except Exception as e:  # symmetric memory unavailable on this box: use the NCCL path and say so
        plan, note, mode = None, f" ({mode} path unavailable: {str(e)[:120]})", "nccl"
    if plan is not None:
        c_full = plan.c_full

        def step(i):
            plan(sets[i % n_sets])
    else:
        c_full = torch.empty((1, m, n), dtype=torch.float16, device=dev).permute(1, 2, 0)
        nccl_plan = ColumnParallelGemm(m, n, k, device=dev, panels=panels)

        def step(i):
            nccl_plan(sets[i % n_sets], c_full)

    def timed(fn, steps):
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / steps

    for i in range(args.warmup):
        step(i)
    S.check_status()

    # ---- parity of the gathered result (rank 0): sampled rows x all columns against the CPU oracle
    step(0)
    torch.cuda.synchronize()
    dist.barrier()
    parity = None
    rows = np.sort(np.random.default_rng(0).choice(m, 16, replace=False))
    if rank == 0:
        from oracle import nvfp4_oracle as O
        full = generate_input(m, n, k, 1, 1111, device="cpu")
        a_np, b_np, sfa_np, sfb_np = O.tensors_to_numpy(full)
        exp = O.ref_gemm_c(a_np[rows], b_np, sfa_np[rows], sfb_np)
        got = c_full[torch.from_numpy(rows).to(dev)].cpu().numpy()
        parity = "bit-exact on 16 sampled rows x all columns" if np.array_equal(got.view(np.uint16), exp.view(np.uint16)) else "MISMATCH"
        del full
    dist.barrier()

    # ---- the timed region: K steps, device time, max over ranks
    sampler = ClockSampler(dev.index)
    sampler.start()
    launches0 = S.launch_count()
    ms_per_step = timed(step, args.steps)
    launches = S.launch_count() - launches0
    clocks = sampler.stop()
    S.check_status()

    # ---- end to end: every step copies this rank's six input tensors from pinned host memory and
    # reads its share of the gathered result (rows [rank*M/g, (rank+1)*M/g) x all N columns) back
    r0, r1 = rank * m // world, (rank + 1) * m // world
    c_host = torch.empty(((r1 - r0) * n,), dtype=torch.float16).pin_memory()
    h2d = sum(t.numel() for t in host_sets[0])
    d2h = c_host.numel() * 2

    def e2e_step(i):
        for dst, src in zip(sets[i % n_sets][:6], host_sets[i % n_sets]):
            _flat_bytes(dst).copy_(src, non_blocking=True)
        step(i)
        c_host.copy_(c_full[r0:r1, :, 0].reshape(-1), non_blocking=True)

    for i in range(2):
        e2e_step(i)
    e2e_ms = timed(e2e_step, max(3, min(args.steps, 8)))

    # ---- GEMM-only time of this rank's block, for the split of compute vs exchange
    gemm_only_c = torch.empty((1, m, shard.n_local), dtype=torch.float16, device=dev).permute(1, 2, 0)
    local = sets[0][:6] + (gemm_only_c,)
    S.custom_kernel(local)
    gemm_ms = timed(lambda i: S.custom_kernel(local), 5)
    del local, gemm_only_c

    # ---- the same exchange with the result re-quantised to NVFP4 in the GEMM's epilogue
    # (packed e2m1 + permuted scales: 0.5625 bytes per element over NVLink instead of 2)
    q_ms, q_parity = None, None
    if plan is not None and not args.no_extra:
        del plan
        try:
            qplan = PanelAllGatherGemm(m, n, k, device=dev, panels=panels, direction="push", copy_sms=copy_sms, nvfp4_out=True)
            for i in range(3):
                qplan(sets[i % n_sets])
            torch.cuda.synchronize()
            dist.barrier()
            if rank == 0:
                from oracle import nvfp4_oracle as O
                packed, perm = qplan.result()
                full = generate_input(m, n, k, 1, 1111 + 2 % n_sets, device="cpu")
                a_np, b_np, sfa_np, sfb_np = O.tensors_to_numpy(full)
                c16 = O.ref_gemm_c(a_np[rows], b_np, sfa_np[rows], sfb_np)
                exp_packed, exp_sf = O.ref_requantize(c16)
                got_packed = packed.view(torch.uint8)[torch.from_numpy(rows).to(dev)].cpu().numpy()
                perm_flat = torch.as_strided(perm.view(torch.uint8), (perm.numel(),), (1,)).cpu().numpy()
                sf_cols = n // 16
                got_sf = np.empty((len(rows), sf_cols, 1), dtype=np.uint8)
                cols = np.arange(sf_cols)
                for ri, r in enumerate(rows):
                    got_sf[ri, :, 0] = perm_flat[O.permuted_sf_offset(int(r), cols, n // 64)]
                ok = np.array_equal(got_packed, exp_packed) and np.array_equal(got_sf, exp_sf)
                q_parity = "bit-exact on 16 sampled rows (packed values and scales)" if ok else "MISMATCH"
                del full
            dist.barrier()
            q_ms = timed(lambda i: qplan(sets[i % n_sets]), max(3, min(args.steps, 10)))
            S.check_status()
            del qplan
        except Exception as e:  # noqa: BLE001
            q_parity = f"not run: {str(e)[:160]}"

    # ---- the same whole job on ONE GPU of this box (rank 0, the others idle): the strong-scaling
    # denominator, measured beside the multi-GPU number
    one_gpu_ms = None
    torch.cuda.empty_cache()
    if rank == 0:
        whole = [generate_input(m, n, k, 1, 1111 + i, device=dev) for i in range(2)]
        for d in whole:
            S.custom_kernel(d)
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for i in range(6):
            S.custom_kernel(whole[i % 2])
        g1.record()
        torch.cuda.synchronize()
        one_gpu_ms = g0.elapsed_time(g1) / 6
        del whole
    dist.barrier()

    if rank == 0:
        flops = algorithmic_flops(w)
        tflops = flops / (ms_per_step * 1e-3) / 1e12
        gather_bytes = (world - 1) / world * m * n * 2
        how = {"ce": "column blocks pushed to the peers by copy engine per row panel, overlapping the next panel's GEMM",
               "pull": f"each rank pulls the other ranks' column blocks per row panel ({panels} panels) with its own copy kernel (loads over NVLink), overlapping the next panel's GEMM",
               "push": f"each rank pushes its column block to the peers per row panel ({panels} panels) with its own copy kernel (stores over NVLink) on {copy_sms} SMs of its own, the GEMM on the rest",
               "fused": "all-gather fused into the GEMM epilogue (peer stores over NVLink)",
               "nccl": f"NCCL all-gather of fp16 blocks + re-layout, {panels} row panels{note}"}[mode]
        line = dict(metric="nvfp4_matmul_throughput", value=tflops, unit="TFLOP/s", n_gpus=world, steps=args.steps,
                    warmup=args.warmup, ms_per_step=ms_per_step, higher_is_better=True, scaling="strong", vs_baseline=None,
                    dtype="e2m1 x ue4m3 -> f32 -> f16", data="synthetic",
                    config=dict(workload=w["name"], parallelism=f"column-parallel over N on {world} GPUs; {how}",
                                timing="CUDA events, max over ranks; 2 rotating input sets per rank > L2",
                                note="the N = 1 line of this bench is a different workload (the decode GEMM): ratios of this line's value to it are not a scaling curve; "
                                     "one_gpu_same_job_ms is this job on one GPU of the same box",
                                gemm_only_ms_per_rank=gemm_ms,
                                one_gpu_same_job_ms=one_gpu_ms,
                                speedup_over_one_gpu=(one_gpu_ms / ms_per_step) if one_gpu_ms else None,
                                gemm_only_tflops_per_gpu=flops / world / (gemm_ms * 1e-3) / 1e12,
                                allgather_bytes_in_per_gpu=gather_bytes, parity_vs_oracle=parity,
                                nvlink_bound_ms=gather_bytes / 770e9 * 1e3,
                                nvfp4_output_exchange=dict(ms_per_step=q_ms, parity_vs_oracle=q_parity,
                                                           bytes_in_per_gpu=(world - 1) / world * m * n * 0.5625,
                                                           speedup_over_one_gpu=(one_gpu_ms / q_ms) if (one_gpu_ms and q_ms) else None,
                                                           what="same job, result re-quantised to NVFP4 in the GEMM epilogue and exchanged in that form (push)")),
                    roofline=dict(bound="nvlink", achieved=gather_bytes / (ms_per_step * 1e-3) / 1e9, peak=770.0, unit="GB/s",
                                  frac=gather_bytes / (ms_per_step * 1e-3) / 1e9 / 770.0, traffic=None,
                                  peak_source="measured peer copy per direction"),
                    e2e=dict(value=flops / (e2e_ms * 1e-3) / 1e12, unit="TFLOP/s", ms_per_step=e2e_ms, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                             note="per rank and step: the six input tensors from pinned host memory, and the rank's 1/g of the rows of the gathered fp16 C back to the host"),
                    gpu_launches=int(launches), clocks=clocks)
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def _flat_bytes(t):
    """A dense (possibly permuted) tensor as its flat bytes, for layout-preserving copies."""
    import torch
    raw = t.view(torch.uint8) if t.element_size() == 1 else t
    return torch.as_strided(raw, (t.numel(),), (1,), raw.storage_offset())


if __name__ == "__main__":
    main()
