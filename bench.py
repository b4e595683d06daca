"""Benchmark of the quantized GEMV/GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Workload: the Llama-7B layer sweep (W4A16, group 128, asymmetric):
(N,K) in {(12288,4096) fused QKV, (4096,4096) O, (22016,4096) gate+up, (4096,11008) down}
x M in {1,4,16}.  One step = one forward of each of the 12 (shape, M) cases.  Every case
owns its packed weights and two replicas of the whole set (632 MB, 5x the 126 MB L2) are
alternated between steps, so every launch streams its weights from HBM.

metric / value: achieved GB/s = the reference's algorithmic-bytes model
(activations + outputs + packed codes + fp16 scales + packed zeros) per step divided by
the device time per step, inputs resident in HBM, the steps replayed as CUDA graphs of
10 steps each (--steps-per-graph; the gap between two graph launches is not part of the path).
The K steps of --steps are timed as one pass with CUDA events, and the pass is repeated (at least
7 times, until 0.25 s of device time): value and ms_per_step are the MEDIAN pass, `spread` holds
the fastest and slowest one.
e2e: the same bytes over the time of calling each case through the host-buffer entry
(pinned host activations in, host result out; a step queues its 12 layers - captured once in a
CUDA graph - and waits for the stream once; copies and the wait are inside the timed region).  With N > 1 every rank runs its own replica of the sweep (the path has no
cross-rank exchange; weak scaling) and value is the sum over ranks on the slowest rank's
time.
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
sys.path.insert(0, os.path.join(ROOT, "qfactory-ae_b200"))
sys.path.insert(0, ROOT)

SHAPES = [("qkv", 12288, 4096), ("o", 4096, 4096), ("gate_up", 22016, 4096), ("down", 4096, 11008)]
BATCHES = [1, 4, 16]
BITS, GS = 4, 128
METRIC = "w4a16_g128_gemv_achieved_hbm_bandwidth"
UNIT = "GB/s"
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one launch, from profiler
# captures of the (22016,4096) case; traffic grows with the weight bytes, so the average launch
# of the sweep is scaled by the same factor
NCU_TRAFFIC_RATIO = {"qgemm_tc_kernel": 1.00592, "gemv_splitk_kernel": 1.0179, "gemv_mma_kernel": 1.008, "gemv_mma_kernel_small": 1.008}
# (N, K) of the linear layers of other model families, and squares, for --sweep
SWEEP_FAMILIES = {
    "llama2-13b": [(5120, 5120), (27648, 5120), (5120, 13824), (15360, 5120)],
    "llama2-70b": [(8192, 8192), (57344, 8192), (8192, 28672), (10240, 8192)],
    "qwen2.5-7b": [(3584, 3584), (37888, 3584), (3584, 18944), (4608, 3584)],
    "qwen2.5-32b": [(5120, 5120), (55296, 5120), (5120, 27648), (7168, 5120)],
    "qwen2.5-72b": [(8192, 8192), (59392, 8192), (8192, 29696), (10240, 8192)],
    "squares-pure": [(1024, 1024), (2048, 2048), (4096, 4096), (8192, 8192), (16384, 16384), (32768, 32768)],
}
WORKLOAD = "llama7b_layer_sweep_w4a16_g128_asym: (N,K) in {(12288,4096),(4096,4096),(22016,4096),(4096,11008)} x M in {1,4,16}"


def algorithmic_bytes(M, N, K, bits=BITS, gs=GS, sym=False):
    """Footprint model of the reference's bandwidth figures
    (reference: reproduce/fig9/plot_bandwidth_size.py:37-44)."""
    b = 2 * (M * K + M * N) + N * K * bits // 8
    if gs != -1:
        b += (K // gs) * N * 2
        if not sym:
            b += (K // gs) * N * bits // 8
    return b


def step_bytes():
    return sum(algorithmic_bytes(M, N, K) for _, N, K in SHAPES for M in BATCHES)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_tensor_peak():
    """Dense bf16 TFLOP/s of a GEMM timed alone (burst), measured on this pool, else the fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured burst"
        except Exception:
            pass
    return 1590.0, "fallback burst"


def bench_config(world):
    """The workload description both arms print (the CPU arm runs the same 12 cases)."""
    return {"workload": WORKLOAD, "bits": BITS, "group_size": GS, "cases_per_step": len(SHAPES) * len(BATCHES),
            "batches": BATCHES, "parallelism": f"replicas x{world}"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def bind_host_to_gpu(torch, local):
    """With several ranks on one node every process pins its host staging buffers; a process that runs on
    the other socket gets them from the far NUMA node and its PCIe copies cross the socket link.  Restrict
    the process to the CPUs NVML reports as local to its GPU before anything is allocated (read-only NVML
    queries; nothing of the GPU is changed).  Returns the number of CPUs kept, or 0 when nothing was done."""
    try:
        import pynvml

        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(local).uuid)
        try:
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            h = pynvml.nvmlDeviceGetHandleByIndex(local)
        ncpu = os.cpu_count() or 1
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, (ncpu + 63) // 64)
        cpus = {i for i in range(ncpu) if (mask[i // 64] >> (i % 64)) & 1} & os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return 0


def use_all_host_threads(torch):
    """The CPU arm uses every host core this process may run on (torchrun exports
    OMP_NUM_THREADS=1 to its workers, which would otherwise leave it on one thread)."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    if n > torch.get_num_threads():
        torch.set_num_threads(n)


def run_reference(args, rank, world):
    """The reference's own CPU path for this workload (dequantize, then fp16 matmul, in torch
    on the host cores), restated in oracle/qf_oracle.py.  One step = the same 12 cases as the
    GPU arm: the four layer shapes at M = 1, 4 and 16, each dequantised and multiplied."""
    if rank != 0:
        return
    import torch
    from oracle import qf_oracle as O

    use_all_host_threads(torch)
    cases = [O.make_case(M, N, K, BITS, GS, False, seed=0) for _, N, K in SHAPES for M in BATCHES]
    nbytes = step_bytes()

    def one_step():
        for x, q, s, z in cases:
            O.qlinear_fp16(x, O.dequant_effective(q, s, O.effective_zero(z.numpy(), BITS)))

    warm = max(args.warmup, 0)
    for _ in range(warm):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = (time.perf_counter() - t0) / args.steps
    val = nbytes / dt / 1e9
    cores = torch.get_num_threads()
    sample = f"the 12 cases (4 layer shapes x M in 1,4,16) per step, {args.steps} steps timed after {warm} warm-up steps"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": bench_config(world),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def cpu_baseline_sample(budget_s=12.0):
    import torch
    from oracle import qf_oracle as O

    use_all_host_threads(torch)
    cases = [O.make_case(M, N, K, BITS, GS, False, seed=0) for _, N, K in SHAPES for M in BATCHES]
    nbytes = step_bytes()
    best, t_start, passes = float("inf"), time.perf_counter(), 0
    while passes < 2 or (time.perf_counter() - t_start < budget_s and passes < 30):
        t0 = time.perf_counter()
        for x, q, s, z in cases:
            O.qlinear_fp16(x, O.dequant_effective(q, s, O.effective_zero(z.numpy(), BITS)))
        best = min(best, time.perf_counter() - t0)
        passes += 1
    return {"value": nbytes / best / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"dequant + fp16 matmul of the 12 cases (4 layer shapes x M in 1,4,16), best of {passes} passes"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--pdl", type=int, default=1,
                    help="launch with programmatic stream serialisation (weights prefetch under the previous kernel's tail)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--per-shape", type=int, default=1)
    ap.add_argument("--extras", type=int, default=1, help="also report the bit-width sweep, the tcgen05 GEMM regime and the "
                    "eager per-call host cost (one GPU only)")
    ap.add_argument("--decode", type=int, default=1,
                    help="also report decode tok/s of the Llama-2-70B-architecture decoder, tensor-parallel over the ranks")
    ap.add_argument("--decode-batch", type=int, default=1)
    ap.add_argument("--case", default="", help="profiling aid: run ONE layer NxKxM a few times (4 weight replicas in "
                    "rotation, so launches stay HBM-cold) and exit; meant to be wrapped in ncu")
    ap.add_argument("--reps", type=int, default=8)
    ap.add_argument("--decode-case", type=int, default=0, help="profiling aid: the decoder with this many layers of the "
                    "70B architecture, a 128-token prefill and 6 single-token steps launched one by one (no graph), then "
                    "exit; meant to be wrapped in a profiler's launch list")
    ap.add_argument("--force", default="", choices=["", "simt", "tensor"])
    ap.add_argument("--host-streams", type=int, default=8, help="streams the end-to-end step spreads its layers over")
    ap.add_argument("--sweep", default="", help="comma-separated sweeps instead of the benchmark, one JSON line each: "
                    "a family of SWEEP_FAMILIES (sizes at M = 1), 'bits' (2/3/4/8-bit on 8192x8192) or 'batch' "
                    "(M = 1..1024 on the Llama-70B MLP shapes)")
    ap.add_argument("--steps-per-graph", type=int, default=10, help="steps captured in one CUDA graph (a decoder's graph "
                    "holds hundreds of layer launches; a single 12-launch step per graph would time the gap between graph "
                    "launches as much as the kernels)")
    ap.add_argument("--bind-host", type=int, default=1, help="with more than one rank: keep each process on the CPUs "
                    "local to its GPU (NUMA-local pinned staging buffers); 0: leave the affinity alone")
    ap.add_argument("--graph", type=int, default=1, help="0: issue the step's launches one by one instead of "
                    "replaying a CUDA graph (for per-launch profiling; not the benchmark configuration)")
    ap.add_argument("--layout", default="auto", choices=["auto", "tile", "fragment"],
                    help="packed layout of the benchmark layers (auto: fragment for these 4-bit shapes)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from qfactory import QLinear, _native

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    _native.lib()  # fail loudly if the native library is missing
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    host_cpus = bind_host_to_gpu(torch, local) if (world > 1 and args.bind_host) else 0
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    REPL = 2
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    flags = _native.FLAG_PDL if args.pdl else 0
    if args.force:
        flags |= _native.FLAG_FORCE_SIMT if args.force == "simt" else _native.FLAG_FORCE_TENSOR

    if args.decode_case:
        from qfactory.decoder import DecoderConfig, QuantDecoder, run_decode

        model = QuantDecoder(DecoderConfig(layers=args.decode_case), device=dev, batch=args.decode_batch)
        sec, _ = run_decode(model, prompt_len=128, steps=6, use_graph=False)
        print(json.dumps({"decode_case_layers": args.decode_case, "eager_ms_per_step": sec / 6 * 1e3}))
        return

    if args.case:
        N, K, M = (int(v) for v in args.case.lower().split("x"))
        layers = []
        for _ in range(4):
            L = QLinear.empty(max(M, 16), K, N, BITS, GS, sym=False, device=dev, layout=args.layout)
            L.w.random_(-128, 127)
            L.s.uniform_(0.002, 0.02)
            L.z.random_(0, 15)
            L.flags = flags
            layers.append(L)
        x = torch.randn(M, K, device=dev).half()
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        for i in range(args.reps):
            layers[i % 4](x, out=y)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "reps": args.reps, "launch": _native.last_launch(),
                          "algorithmic_bytes": algorithmic_bytes(M, N, K)}))
        return

    # one layer alone: graph replay over >= 400 MB of rotating weight replicas, so that every
    # launch streams its weights from HBM; time per launch from events around the replays
    def time_layer(N, K, M, bits, gs, sym):
        R = max(2, min(48, (400 << 20) // (N * K * bits // 8) + 1))
        ls = []
        for _ in range(R):
            lay = args.layout
            L = QLinear.empty(M, K, N, bits, gs, sym=sym, device=dev, layout=lay)
            L.w.random_(-128, 127)
            if L.s is not None:
                L.s.uniform_(0.002, 0.02)
            if L.z is not None:
                L.z.view(torch.uint8).random_(0, (1 << bits) - 1)
            L.flags = flags
            L._prepare()
            ls.append(L)
        x = torch.randn(M, K, device=dev).half()
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            ls[0](x, out=y)
            torch.cuda.synchronize()
            launch = _native.last_launch()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=st):
                for L in ls:
                    L(x, out=y)
            for _ in range(3):
                gr.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                gr.replay()
            b.record()
            torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (10 * R)
        nb = algorithmic_bytes(M, N, K, bits, gs, sym)
        del gr, ls
        torch.cuda.empty_cache()
        return {"N": N, "K": K, "M": M, "bits": bits, "group": gs, "sym": sym, "us": round(us, 2),
                "GBps": round(nb / us / 1e3, 1), "TFLOPs": round(2.0 * M * N * K / us / 1e6, 1),
                "MB": round(nb / 1e6, 1), "kernel": launch["kernel"], "grid_x": launch["grid_x"]}

    if args.sweep:
        # Other sweeps of the reference, each layer alone, graph replay over >= 400 MB of rotating
        # weight replicas; one JSON line per sweep:
        #   <family>  bandwidth against layer size at M = 1 (reference: reproduce/fig9/plot_bandwidth_size.py,
        #             shapes of data/nkg_shapes.json)
        #   bits      2/3/4/8-bit, asymmetric and symmetric, on (8192,8192), M = 1, group 128
        #   batch     W4 g128 on the Llama-70B MLP shapes, M = 1 .. 1024 (GEMV -> tcgen05 GEMM)
        for name in args.sweep.split(","):
            if name == "bits":
                rows = [time_layer(8192, 8192, 1, b, GS, sym) for b in (2, 3, 4, 8) for sym in (False, True)]
            elif name == "batch":
                rows = [time_layer(N, K, M, BITS, GS, False) for N, K in ((28672, 8192), (8192, 28672))
                        for M in (1, 2, 4, 8, 16, 32, 64, 128, 256, 1024)]
            else:
                rows = [time_layer(N, K, 1, BITS, gs, False) for N, K in SWEEP_FAMILIES[name]
                        for gs in ((GS, -1) if name == "squares-pure" else (GS,))]
            print(json.dumps({"sweep": name, "peak_GBps": measured_peaks()[0], "rows": rows}), flush=True)
        return

    def make_layer(N, K):
        L = QLinear.empty(16, K, N, BITS, GS, sym=False, device=dev, layout=args.layout)
        L.w.copy_(torch.randint(-128, 128, L.w.shape, generator=g, dtype=torch.int8, device=dev))
        L.s.copy_((torch.rand(L.s.shape, generator=g, device=dev) * 0.018 + 0.002).half())
        L.z.copy_(torch.randint(0, 16, L.z.shape, generator=g, dtype=torch.int8, device=dev))
        L.flags = flags
        return L

    cases = []  # replica -> list of (name, M, layer, x_dev, y_dev, x_host, y_host)
    for rep in range(REPL):
        row = []
        for name, N, K in SHAPES:
            for M in BATCHES:
                layer = make_layer(N, K)
                x = torch.randn(M, K, generator=g, device=dev).half()
                y = torch.empty(M, N, dtype=torch.float16, device=dev)
                xh = x.cpu().pin_memory()
                yh = torch.empty(M, N, dtype=torch.float16).pin_memory()
                row.append((name, M, layer, x, y, xh, yh))
        cases.append(row)
    n_cases = len(cases[0])

    def run_step(rep):
        for _, _, layer, x, y, _, _ in cases[rep]:
            layer(x, out=y)

    stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        for rep in range(REPL):
            run_step(rep)  # builds descriptors / workspaces outside capture
        torch.cuda.synchronize()
        class Eager:  # --graph 0: the same launches issued one by one (profiling aid)
            def __init__(self, fn):
                self.replay = fn

        G = max(1, args.steps_per_graph) if args.graph else 1

        def capture(step_fn):
            """One single-step graph per replica, and one graph of G steps that alternate the replicas."""
            singles = []
            for rep in range(REPL):
                if not args.graph:
                    singles.append(Eager(lambda rep=rep: step_fn(rep)))
                    continue
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=stream):
                    step_fn(rep)
                singles.append(gr)
            multi = None
            if G > 1:
                multi = torch.cuda.CUDAGraph()
                with torch.cuda.graph(multi, stream=stream):
                    for j in range(G):
                        step_fn(j % REPL)
            return singles, multi

        def replay_steps(gs, n):
            singles, multi = gs
            i = 0
            if multi is not None:
                while i + G <= n:
                    multi.replay()
                    i += G
            while i < n:
                singles[i % REPL].replay()
                i += 1

        graphs = capture(run_step)

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        # which kernel serves each case, and one graph per kernel so that the dominant kernel's
        # own time can be measured with events in this same run
        # (the mma.sync GEMV has two register builds, picked by the CTA size: they show up under two
        # names in a profile, so they are told apart here as well: 4 = its build for small CTAs)
        kern_of = []
        for _, M, layer, x, y, _, _ in cases[0]:
            layer(x, out=y)
            info = _native.last_launch()
            kern_of.append(4 if info["kernel"] == 3 and info["block"] <= 128 else info["kernel"])
        torch.cuda.synchronize()
        sub_graphs = {}
        for kid in sorted(set(kern_of)):
            def sub_step(rep, kid=kid):
                for ci, (_, _, layer, x, y, _, _) in enumerate(cases[rep]):
                    if kern_of[ci] == kid:
                        layer(x, out=y)

            sub_graphs[kid] = capture(sub_step)

        replay_steps(graphs, max(args.warmup, 3))
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        # a pass = the K steps of --steps between two events; passes are repeated (>= 7, until a
        # quarter of a second of device time) and the median pass is the one reported
        pass_ms = []
        while len(pass_ms) < 7 or (sum(pass_ms) < 250.0 and len(pass_ms) < 200):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            replay_steps(graphs, args.steps)
            e1.record()
            barrier()
            t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)   # every rank counts the same passes
            pass_ms.append(float(t[0]))
        srt = sorted(pass_ms)
        ms = srt[len(srt) // 2]

        kernel_ms = {}
        for kid, gl in sub_graphs.items():
            replay_steps(gl, 3)
            torch.cuda.synchronize()
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record()
            replay_steps(gl, args.steps)
            k1.record()
            torch.cuda.synchronize()
            kernel_ms[kid] = k0.elapsed_time(k1) / args.steps

        # end to end through the host-buffer entry point
        e2e_steps = max(3, min(args.steps, 50))
        # a step queues its 12 layers (pinned x in, y out: H2D copy, kernel, D2H copy each) and waits
        # for the stream once; the queued calls of a step are captured once in a CUDA graph, as a
        # caller with a fixed set of layers would do, and the graph is replayed every step
        # (the layers are independent, so they are spread over a few streams: the small PCIe
        # copies of one layer overlap the kernels and copies of the others)
        side = [torch.cuda.Stream(device=dev) for _ in range(max(1, args.host_streams))]

        def host_step(rep):
            main = torch.cuda.current_stream(dev)
            for sd in side:
                sd.wait_stream(main)
            for i, (_, _, layer, _, _, xh, yh) in enumerate(cases[rep]):
                with torch.cuda.stream(side[i % len(side)]):
                    layer.forward_host(xh, yh, sync=False)
            for sd in side:
                main.wait_stream(sd)

        for i in range(2):
            host_step(i % REPL)  # allocates the staging buffers outside the capture
            torch.cuda.current_stream(dev).synchronize()
        host_graphs = []
        for rep in range(REPL):
            if not args.graph:
                host_graphs.append(Eager(lambda rep=rep: host_step(rep)))
                continue
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                host_step(rep)
            host_graphs.append(gr)
        for i in range(3):
            host_graphs[i % REPL].replay()
            torch.cuda.current_stream(dev).synchronize()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for i in range(e2e_steps):
            host_graphs[i % REPL].replay()
            torch.cuda.current_stream(dev).synchronize()
        f1.record()
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        clocks = sampler.stop() if rank == 0 else None

        # per-case breakdown: each case as a CUDA graph over enough weight replicas (>= 400 MB) that
        # every launch streams its weights from HBM; time per launch from events around the replays
        per_shape = []
        if args.per_shape and rank == 0:
            for ci in range(n_cases):
                name, M, layer0, x, y, _, _ = cases[0][ci]
                N, K = layer0.out_features, layer0.in_features
                R = max(2, min(48, (400 << 20) // (N * K * BITS // 8) + 1))
                reps_l = [make_layer(N, K) for _ in range(R)]
                for l in reps_l:
                    l._prepare()  # descriptor and workspace now, not inside the capture below
                st = torch.cuda.Stream(device=dev)
                with torch.cuda.stream(st):
                    reps_l[0](x, out=y)
                    torch.cuda.synchronize()
                    launch = _native.last_launch()
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=st):
                        for l in reps_l:
                            l(x, out=y)
                    for _ in range(3):
                        gr.replay()
                    torch.cuda.synchronize()
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(10):
                        gr.replay()
                    b.record()
                    torch.cuda.synchronize()
                med = a.elapsed_time(b) / (10 * R)
                del gr, reps_l
                nb = algorithmic_bytes(M, N, K)
                gbps = nb / (med * 1e-3) / 1e9
                per_shape.append({"layer": name, "N": N, "K": K, "M": M, "us": round(med * 1e3, 2), "GBps": round(gbps, 1),
                                  "frac": round(gbps / measured_peaks()[0], 3), "kernel": launch["kernel"],
                                  "grid": [launch["grid_x"], launch["grid_y"]], "block": launch["block"]})

    # free the sweep's device memory before the decoder is built
    case_meta = [(M, layer.out_features, layer.in_features) for _, M, layer, *_ in cases[0]]
    del graphs, sub_graphs, cases
    torch.cuda.empty_cache()

    # ---- one GPU only: the other stated configurations, each layer alone -------------------------
    extras = {}
    if args.extras and world == 1:
        tpeak, tkind = measured_tensor_peak()
        hpeak = measured_peaks()[0]
        try:
            # bit-width sweep on (8192,8192), M = 1, group 128, asymmetric and symmetric
            extras["bits"] = [{"bits": r["bits"], "sym": r["sym"], "us": r["us"], "GBps": r["GBps"],
                               "frac": round(r["GBps"] / hpeak, 3), "kernel": r["kernel"]}
                              for r in (time_layer(8192, 8192, 1, b, GS, sym) for b in (2, 3, 4, 8) for sym in (False, True))]
            # batch sweep on the Llama-70B MLP shapes across the GEMV -> tcgen05 GEMM boundary
            rows = []
            for N, K in ((28672, 8192), (8192, 28672)):
                for M in (16, 32, 64, 128, 256, 1024):
                    r = time_layer(N, K, M, BITS, GS, False)
                    rows.append({"N": N, "K": K, "M": M, "us": r["us"], "GBps": r["GBps"], "TFLOPs": r["TFLOPs"],
                                 "frac_tensor": round(r["TFLOPs"] / tpeak, 3), "frac_hbm": round(r["GBps"] / hpeak, 3),
                                 "kernel": r["kernel"]})
            extras["gemm"] = {"tensor_peak_TFLOPs": tpeak, "tensor_peak_kind": tkind, "rows": rows}
            # host cost of one eager call (no graph): 400 calls of the (4096,4096) layer at M = 1 issued
            # back to back, wall clock from the first call to the return of the last (the device is
            # faster than the host here, so this is the per-call host time: validation, plan lookup, launch)
            L = QLinear.empty(1, 4096, 4096, BITS, GS, sym=False, device=dev, layout=args.layout)
            L.w.random_(-128, 127)
            L.s.uniform_(0.002, 0.02)
            L.z.random_(0, 15)
            L.flags = flags
            xe = torch.randn(1, 4096, device=dev).half()
            ye = torch.empty(1, 4096, dtype=torch.float16, device=dev)
            for _ in range(20):
                L(xe, out=ye)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(400):
                L(xe, out=ye)
            host_s = time.perf_counter() - t0
            torch.cuda.synchronize()
            total_s = time.perf_counter() - t0
            # the same through the C ABI alone (ctypes, arguments prepared once): validation, plan lookup, launch
            import ctypes

            fwd, dref = _native.lib().qfb_linear_forward, ctypes.byref(L._desc)
            call_args = (dref, xe.data_ptr(), 1, ye.data_ptr(), L._ws.data_ptr(), L._ws_bytes, flags,
                         torch.cuda.current_stream(dev).cuda_stream)
            for _ in range(20):
                fwd(*call_args)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(400):
                fwd(*call_args)
            abi_s = time.perf_counter() - t0
            torch.cuda.synchronize()
            extras["eager"] = {"layer": "4096x4096 M=1", "module_host_us_per_call": round(host_s / 400 * 1e6, 2),
                               "abi_host_us_per_call": round(abi_s / 400 * 1e6, 2),
                               "us_per_call_with_device": round(total_s / 400 * 1e6, 2)}
            del L
            # same-box GPU baseline: the reference project's own kernel (its default and its scheduled
            # design point, compiled ahead of time for sm_100a) on the four layer shapes at M = 1, in the
            # reference's packed layout, timed by the same graph-replay method over rotating weights
            from oracle import ref_gpu

            if ref_gpu.available():
                rows = []
                for si, (N, K) in enumerate(ref_gpu.SHAPES):
                    R = max(2, min(48, (400 << 20) // (N * K // 2) + 1))
                    ws = [torch.randint(-128, 128, (N, K // 2), dtype=torch.int8, device=dev) for _ in range(R)]
                    sc = (torch.rand(N, K // GS, device=dev) * 0.018 + 0.002).half()
                    zz = torch.randint(-128, 128, (N, K // GS // 2), dtype=torch.int8, device=dev)
                    xr = torch.randn(1, K, device=dev).half()
                    yr = torch.empty(1, N, dtype=torch.float16, device=dev)
                    row = {"N": N, "K": K, "M": 1}
                    for sched, key in ((0, "default_us"), (1, "scheduled_us")):
                        st = torch.cuda.Stream(device=dev)
                        with torch.cuda.stream(st):
                            assert ref_gpu.launch(si, sched, xr, ws[0], yr, sc, zz, st.cuda_stream) == 0
                            torch.cuda.synchronize()
                            gr = torch.cuda.CUDAGraph()
                            with torch.cuda.graph(gr, stream=st):
                                for w in ws:
                                    ref_gpu.launch(si, sched, xr, w, yr, sc, zz, st.cuda_stream)
                            for _ in range(3):
                                gr.replay()
                            torch.cuda.synchronize()
                            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            a.record()
                            for _ in range(10):
                                gr.replay()
                            b.record()
                            torch.cuda.synchronize()
                        row[key] = round(a.elapsed_time(b) * 1e3 / (10 * R), 2)
                        del gr
                    best = min(row["default_us"], row["scheduled_us"])
                    row["GBps"] = round(algorithmic_bytes(1, N, K) / best / 1e3, 1)
                    rows.append(row)
                    del ws
                    torch.cuda.empty_cache()
                extras["ref_gpu_kernel"] = {"what": "the reference project's kernel_gptq template (BLOCK_N 1, BLOCK_SIZE 128, NUM_ELM 8, "
                                            "eager decode; default and scheduled load paths), sm_100a, same box, same timing method",
                                            "rows": rows}
        except Exception as e:
            extras["error"] = str(e)[:200]
        torch.cuda.empty_cache()

    # ---- tensor-parallel decoder: numeric check, then decode tokens/s -----------------------------
    # secondary figure: decode tokens/s of the random-init Llama-2-70B-architecture decoder,
    # all linears W4A16 g128, prompt 128 then 256 greedy steps, tensor-parallel over the ranks
    decode = None
    if args.decode and 8 % world == 0:
        try:
            from qfactory.decoder import DecoderConfig, QuantDecoder, run_decode, teacher_forced_logits, time_linears

            decode = {}
            if world > 1:
                # the SAME seeded network, sharded over the ranks (column / row shards of one set of
                # tensors) against the unsharded model on this GPU: 80 prompt tokens (more rows than the
                # peer-memory kernel takes: the process group's all-reduce), then 4 single-token steps
                # (the peer-memory kernel), same tokens fed to both
                small = DecoderConfig(layers=2, d_model=1024, n_heads=8, n_kv_heads=8, d_ff=4096, vocab=2048, max_len=128,
                                      scale_boost=40.0)
                gtok = torch.Generator(device=dev).manual_seed(7)
                toks = torch.randint(0, small.vocab, (2, 84), generator=gtok, device=dev)
                tp_model = QuantDecoder(small, world=world, rank=rank, device=dev, seed=11, batch=2, weights="seeded")
                got = teacher_forced_logits(tp_model, toks, prompt_len=80).float()
                status = tp_model.comm.read_status() if tp_model.comm is not None else 0
                coll = tp_model.collective_name()
                tp_model.close()
                one = QuantDecoder(small, world=1, rank=0, device=dev, seed=11, batch=2, weights="seeded")
                want = teacher_forced_logits(one, toks, prompt_len=80).float()
                err = torch.stack([(got - want).abs().max() / want.abs().max(), torch.tensor(float(status), device=dev)])
                dist.all_reduce(err, op=dist.ReduceOp.MAX)
                decode["tp_check"] = {"max_rel_err": float(err[0]), "ok": bool(float(err[0]) <= 2e-2 and float(err[1]) == 0),
                                      "device_status": int(err[1]), "collective": coll,
                                      "model": "2 layers, d=1024, one seeded network sharded over the ranks vs unsharded"}
                del tp_model, one
                torch.cuda.empty_cache()

            cfg = DecoderConfig()
            model = QuantDecoder(cfg, world=world, rank=rank, device=dev, batch=args.decode_batch)

            def timed_decode():
                sec, _ = run_decode(model, prompt_len=128, steps=256)
                dt = torch.tensor([sec], dtype=torch.float64, device=dev)
                if world > 1:
                    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
                return float(dt[0])

            sec = timed_decode()
            decode.update({"model": "llama2-70b-architecture random init, W4A16 g128 (output projection included)",
                           "kernels_per_layer": 7,
                           "tp": world, "batch": args.decode_batch, "prompt": 128, "steps": 256,
                           "tok_per_s": 256 * args.decode_batch / sec, "ms_per_step": sec / 256 * 1e3,
                           "collective": model.collective_name()})
            if model.comm is not None:
                decode["device_status"] = model.comm.read_status()
            # where the step's time goes: the linears alone (the step's quantized linears replayed back to
            # back from a graph), and the reductions (the step with every reduction left out, and, where
            # the peer-memory kernel is in use, the step with NCCL instead)
            decode["linears_ms_per_step"] = time_linears(model) * 1e3
            if world > 1:
                used = model.collective
                model.collective = "none"
                sec_none = timed_decode()
                decode["allreduce_ms_per_step"] = (sec - sec_none) / 256 * 1e3
                decode["ms_per_step_without_reductions"] = sec_none / 256 * 1e3
                if model.comm is not None:
                    model.collective = "nccl"
                    sec_nccl = timed_decode()
                    decode["nccl"] = {"tok_per_s": 256 * args.decode_batch / sec_nccl, "ms_per_step": sec_nccl / 256 * 1e3,
                                      "allreduce_ms_per_step": (sec_nccl - sec_none) / 256 * 1e3}
                model.collective = used
            model.close()
            del model
            torch.cuda.empty_cache()
        except Exception as e:  # the headline line must not depend on the secondary figure
            import traceback

            decode = dict(decode or {}, error=(str(e) + " | " + traceback.format_exc().strip().splitlines()[-2].strip())[:300])

    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0])

    if rank == 0:
        peak, peak_kind = measured_peaks()
        sb = step_bytes()
        value = sb * args.steps * world / (ms * 1e-3) / 1e9
        e2e_val = sb * e2e_steps * world / (e2e_ms * 1e-3) / 1e9
        launches = n_cases * args.steps
        # dominant kernel = the one with the larger share of the step's device time
        names = {1: "gemv_splitk_kernel", 2: "qgemm_tc_kernel", 3: "gemv_mma_kernel", 4: "gemv_mma_kernel_small"}
        shares = {}
        for kid, kms in kernel_ms.items():
            idx = [ci for ci in range(n_cases) if kern_of[ci] == kid]
            kb = sum(algorithmic_bytes(*case_meta[ci]) for ci in idx)
            shares[kid] = {"kernel": names.get(kid, str(kid)), "launches_per_step": len(idx), "ms_per_step": kms,
                           "bytes_per_step": kb, "GBps": kb / (kms * 1e-3) / 1e9}
        dom = max(shares, key=lambda k: shares[k]["ms_per_step"])
        per_launch_s = shares[dom]["ms_per_step"] * 1e-3 / shares[dom]["launches_per_step"]
        achieved = shares[dom]["GBps"]
        h2d = sum(2 * M * K for _, _, K in SHAPES for M in BATCHES)
        d2h = sum(2 * M * N for _, N, _ in SHAPES for M in BATCHES)
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": bench_config(world),
            "protocol": {"cache": f"inputs larger than L2: {REPL} replicas of all weights ({REPL * sb / 1e6:.0f} MB) alternated between steps",
                         "graph": bool(args.graph), "steps_per_graph": G, "pdl": bool(args.pdl), "host_cpus_bound": host_cpus, "launches_per_step": n_cases,
                         "timed": f"{len(pass_ms)} passes of {args.steps} steps, CUDA events, max over ranks per pass; value = median pass"},
            "spread": {"passes": len(pass_ms), "ms_per_step_min": srt[0] / args.steps, "ms_per_step_median": ms / args.steps,
                       "ms_per_step_max": srt[-1] / args.steps},
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": launches * world,
            "clocks": clocks,
            "kernels": list(shares.values()),
            "roofline": {"bound": "hbm", "kernel": shares[dom]["kernel"], "achieved": achieved, "peak": peak,
                         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "avg_launch_us": per_launch_s * 1e6, "traffic": None},
            "per_shape": per_shape,
            "decode": decode,
        }
        out.update(extras)
        ratio = NCU_TRAFFIC_RATIO.get(shares[dom]["kernel"])
        if ratio:
            out["roofline"]["traffic"] = int(ratio * shares[dom]["bytes_per_step"] / shares[dom]["launches_per_step"])
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_baseline_sample()
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
