"""Benchmark of the FP8 grouped-MLP hot path: forward + dgrad + wgrad on synthetic data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One process per GPU (launched under torch.distributed.run for N > 1).  A "step" is one forward +
backward of GroupedMlp over one routed batch.  Prints ONE JSON line on rank 0:

* ``value``      TFLOP/s with inputs resident in HBM (algorithmic FLOPs 18 * rows * hidden * ffn for SwiGLU,
                 true rows, padding not counted), CUDA-event timed, max over ranks;
* ``e2e``        same metric through the public module API with HOST buffers: every step copies the step's
                 inputs (x, grad_out) from pinned host memory and reads the results (out, grad_input) back;
* ``roofline``   the dominant kernel (the tcgen05 grouped GEMM, 6 launches per step): algorithmic FLOPs per
                 launch / mean launch duration from CUDA events recorded around each launch inside the timed
                 region, against 2 x the measured dense bf16 rate (dense FP8 is twice bf16 on this part);
* ``cpu_baseline`` the CPU oracle (torch per-group float8-emulated matmuls + CPU quantise/transposes)
                 timed on the host cores on a bounded sample of the same workload;
* ``pad``        (N = 1) the HBM-bound kernel families on the pad / cast microbenchmark (256 groups, rows ~ U[0, 4096],
                 K = 7168, bf16 ~ N(0, 3) with 0.1 % outliers x 100): algorithmic bytes, GB/s, fraction of the measured
                 copy bandwidth and of 8 TB/s for each op;
* ``library_gemm`` (N = 1) this package's grouped GEMM beside the per-group ``torch._scaled_mm`` loop (cuBLASLt) on the
                 six GEMM shapes of the step: a comparison leg, the library is never on the product path;
* ``fine_grained`` (N = 1) the fine-grained MoE step (64 experts, hidden 2048, ffn 1408, 49152 rows, Zipf loads);
* ``ep``         (N > 1) efficiency against the exchange-free local step, exposed waits, host time per rank, and
                 ``check``: one extra step compared bit for bit with the NCCL all-to-all transport from the same state.

``--impl reference`` times that CPU path alone (the reference has no CPU or sm_100 implementation of
its own: its GEMM is Hopper-only CUTLASS and its other GEMM path needs Transformer Engine, so the
float8-emulated per-group matmul loop of its test-suite is what can run on host cores).

Workloads (synthetic, seeded): N = 1 -> Mixtral-8x7B-shaped MLP (8 experts, hidden 4096, ffn 14336,
SwiGLU, 16384 tokens top-2 = 32768 routed rows, multinomial routing over softmax(N(0,1)) logits);
N > 1 -> expert parallelism (128 experts split over the ranks, hidden 4096, ffn 1536, 32768 tokens per
GPU top-8, all-to-all dispatch/combine over NCCL).
"""
import argparse
import datetime
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "grouped_mlp_fwd_bwd_fp8_tflops"
NOMINAL_FP8_TFLOPS = 4500.0
# DRAM bytes (read + write) per GEMM launch, averaged over the six launches of one Mixtral-shaped step, from a
# one-pass ncu capture of the six full-size launches (dram__bytes_read.sum + dram__bytes_write.sum: 17.76 GB in all).
GEMM_DRAM_BYTES_PER_LAUNCH = 2.960e9

# Expert-parallel workload (N > 1; weak scaling, the per-GPU work is fixed): 128 experts split evenly over the ranks,
# hidden 4096, ffn 1536, SwiGLU, 32768 tokens per GPU routed top-8 (softmax over N(0,1) logits, 8 distinct experts per
# token) = 262144 routed rows per GPU, delayed scaling with an amax history of 16.
EP = dict(E=128, H=4096, F=1536, tokens_per_gpu=32768, topk=8,
          name=("expert-parallel GroupedMLP (E=128 split over the ranks, hidden 4096, ffn 1536, SwiGLU, "
                "32768 tokens/GPU top-8, all-to-all dispatch/combine)"))
EP["rows_per_expert"] = EP["tokens_per_gpu"] * EP["topk"] // EP["E"]   # per source rank; sizes the CPU baseline sample


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="auto", choices=["auto", "mixtral", "ep"])
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-extras", action="store_true", help="N = 1: skip the pad / library_gemm / fine_grained legs")
    p.add_argument("--ep-transport", default="peer", choices=["peer", "nccl"],
                   help="expert-parallel leg: copy-engine pushes into peer memory pipelined with the GEMMs, or NCCL all-to-all")
    p.add_argument("--ep-bf16-dispatch", action="store_true", help="peer transport: dispatch rows as bf16 instead of FP8")
    p.add_argument("--ep-quick", action="store_true", help="N > 1: timed step, traces and the local step only (no e2e, check, tp legs)")
    p.add_argument("--ep-chunks", default="tapered", help="expert chunks of the peer-transport pipeline: a count, 'tapered', "
                   "or comma-separated expert counts per chunk")
    return p.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
def mixtral_workload(seed=0):
    E, H, F, tokens, topk = 8, 4096, 14336, 16384, 2
    g = torch.Generator().manual_seed(seed)
    probs = torch.softmax(torch.randn(tokens, E, generator=g), dim=-1)
    picks = torch.multinomial(probs, topk, replacement=False, generator=g)  # (tokens, 2) distinct experts
    sizes = torch.bincount(picks.reshape(-1), minlength=E)
    return dict(name="mixtral-8x7b-shaped GroupedMLP (E=8, hidden 4096, ffn 14336, SwiGLU, 16384 tokens top-2)",
                E=E, H=H, F=F, tokens=tokens, topk=topk, sizes=sizes, rows=int(sizes.sum()))


def fine_grained_workload(seed=3):
    """Fine-grained MoE: 64 experts, hidden 2048, ffn 1408, SwiGLU, 8192 tokens top-6 = 49152 routed rows with
    Zipf(s = 1.2) expert popularity, so many groups are small, empty or not multiples of 16."""
    E, H, F, rows = 64, 2048, 1408, 49152
    g = torch.Generator().manual_seed(seed)
    p = 1.0 / torch.arange(1, E + 1, dtype=torch.float64) ** 1.2
    idx = torch.multinomial((p / p.sum()).float(), rows, replacement=True, generator=g)
    return dict(E=E, H=H, F=F, rows=rows, sizes=torch.bincount(idx, minlength=E))


def mlp_flops(rows, H, F):
    return 18.0 * rows * H * F  # SwiGLU: fc1 is H -> 2F; fwd + dgrad + wgrad = 3 x (2*rows*H*2F + 2*rows*F*H)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi.  The sampler process starts when the object is
    created (do that before the warm-up: nvidia-smi needs a moment to come up, longer with eight GPUs); the ``with``
    block marks the timed region, and only samples stamped inside it are summarised."""

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.raw, self.samples, self.proc = index, [], [], None
        self.t0 = self.t1 = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def __enter__(self):
        self.t0 = datetime.datetime.now()
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7 and parts[1].isdigit():
                try:
                    stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                except ValueError:
                    continue
                self.raw.append((stamp, parts[1:]))

    def __exit__(self, *exc):
        self.t1 = datetime.datetime.now()
        if self.proc is not None:
            time.sleep(0.12)  # let the sample that covers the end of the region arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        slack = datetime.timedelta(milliseconds=60)
        self.samples = [v for t, v in self.raw if self.t0 - slack <= t <= self.t1 + slack]

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------------
# CPU path (oracle port) -- the baseline arm
# ------------------------------------------------------------------------------------------------
def cpu_sample_step(H, F_full, rows_per_expert, seed=0):
    """Returns (callable running one CPU step on the sample, flops of the sample, description)."""
    from oracle import oracle as O

    rows, F = max(64, rows_per_expert // 8), F_full // 8
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    dy = torch.randn(rows, H, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(1, 2 * F, H, generator=g) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(1, H, F, generator=g) * 0.02).to(torch.bfloat16)
    one = [1.0]
    scales = dict(x=one, w1=one, act=one, w2=one, dy=one, dpre=one)

    def step():
        return O.grouped_mlp_step(x, w1, w2, dy, [rows], scales, act="swiglu")

    desc = (f"1 expert, {rows} rows, hidden {H}, ffn slice {F} of {F_full} (same rows:weights ratio as the full "
            f"step), full fwd+bwd incl. quantise/transposes, torch CPU float8-emulated matmuls")
    return step, mlp_flops(rows, H, F), desc


def run_cpu(step, flops, reps, warmup):
    torch.set_num_threads(os.cpu_count() or 1)
    for _ in range(warmup):
        step()
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return flops / mean / 1e12, mean


def reference_arm(args, wl_desc, H, F, rows_per_expert):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, flops, desc = cpu_sample_step(H, F, rows_per_expert)
    tflops, mean = run_cpu(step, flops, args.steps, args.warmup)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8 (e4m3 fwd / e5m2 grad, fp32 accumulate; float8-emulated on CPU)",
        "data": "synthetic", "config": {"workload": wl_desc, "sample": desc},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm, N = 1
# ------------------------------------------------------------------------------------------------
def timed_steps(fn, steps):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3  # seconds


class E2EPipeline:
    """End-to-end loop through the public API with host buffers: every step copies its inputs from pinned host memory
    and reads its results back to pinned host memory, all inside the timed region.  Like an input pipeline with
    prefetch, the copies run on their own streams: step i+1's inputs are copied while step i computes (two sets of
    device input buffers), and step i's results are read while step i+1 computes.

    ``run_step(*device_inputs)`` returns the device tensors to read back, in the order of ``host_out``."""

    def __init__(self, run_step, host_in, host_out, dev):
        self.run_step, self.dev = run_step, dev
        self.host_in, self.host_out = list(host_in), list(host_out)
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.bufs = [[torch.empty_like(h, device=dev) for h in self.host_in] for _ in range(2)]
        self.ready = [torch.cuda.Event() for _ in range(2)]
        self.done = [None, None]
        self.keep = [None, None]   # results of the step that last used a buffer set, alive until their read-back is done
        self.h2d_bytes = sum(h.numel() * h.element_size() for h in self.host_in)
        self.d2h_bytes = sum(h.numel() * h.element_size() for h in self.host_out)

    def _prefetch(self, i):
        b = i % 2
        with torch.cuda.stream(self.h2d):
            if self.done[b] is not None:
                self.h2d.wait_event(self.done[b])     # the step that last used this buffer set has finished
            for dst, src in zip(self.bufs[b], self.host_in):
                dst.copy_(src, non_blocking=True)
            self.ready[b].record(self.h2d)

    def run(self, steps):
        cur = torch.cuda.current_stream(self.dev)
        self._prefetch(0)
        for i in range(steps):
            b = i % 2
            if i + 1 < steps:
                self._prefetch(i + 1)
            cur.wait_event(self.ready[b])
            if self.keep[b] is not None:
                # results may live in memory that is reused once they are dropped: drop them only after their copy
                cur.wait_event(self.keep[b][1])
                self.keep[b] = None
            outs = self.run_step(*self.bufs[b])
            ev = torch.cuda.Event()
            ev.record(cur)
            self.done[b] = ev
            with torch.cuda.stream(self.d2h):
                self.d2h.wait_event(ev)
                for dst, src in zip(self.host_out, outs):
                    dst.copy_(src.detach(), non_blocking=True)
                read = torch.cuda.Event()
                read.record(self.d2h)
            self.keep[b] = (outs, read)
        cur.wait_stream(self.d2h)
        cur.wait_stream(self.h2d)
        self.done = [None, None]
        self.keep = [None, None]


def run_single(args):
    import fp8_gmm_b200 as fg
    from fp8_gmm_b200 import backend

    wl = mixtral_workload()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    E, H, F, rows = wl["E"], wl["H"], wl["F"], wl["rows"]
    sizes = wl["sizes"]
    g = torch.Generator().manual_seed(1)
    x_host = torch.randn(rows, H, generator=g).to(torch.bfloat16).pin_memory()
    dy_host = torch.randn(rows, H, generator=g).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(rows, H, dtype=torch.bfloat16).pin_memory()
    gi_host = torch.empty(rows, H, dtype=torch.bfloat16).pin_memory()
    torch.manual_seed(2)
    mlp = fg.GroupedMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu")
    with torch.no_grad():
        mlp.fc1_weight.normal_(0.0, 0.02)
        mlp.fc2_weight.normal_(0.0, 0.02)
    x_dev = x_host.to(dev).requires_grad_(True)
    dy_dev = dy_host.to(dev)
    recipe = fg.DelayedScaling(amax_history_len=16)

    def step():
        mlp.fc1_weight.grad = None
        mlp.fc2_weight.grad = None
        x_dev.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = mlp(x_dev, sizes)
        out.backward(dy_dev)
        return out

    def step_on(x_buf, dy_in):
        mlp.fc1_weight.grad = None
        mlp.fc2_weight.grad = None
        x_in = x_buf.detach().requires_grad_(True)
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = mlp(x_in, sizes)
        out.backward(dy_in)
        return out, x_in.grad

    e2e = E2EPipeline(step_on, [x_host, dy_host], [out_host, gi_host], dev)

    sampler = ClockSampler(dev.index or 0)
    for _ in range(max(args.warmup, 3)):
        step()
    backend.device_status()

    flops = mlp_flops(rows, H, F)
    timings = []
    backend.set_gemm_timings(timings)
    launches0 = backend.launch_count()
    with sampler as clocks:
        secs = timed_steps(step, args.steps)
    launches = backend.launch_count() - launches0
    backend.set_gemm_timings(None)
    gemm_ms = sum(s.elapsed_time(e) for s, e, _ in timings)
    gemm_flops = flops * args.steps  # all of a step's algorithmic FLOPs are in its six GEMM launches
    n_gemm = len(timings)

    e2e.run(2)
    secs_e2e = timed_steps(lambda: e2e.run(args.steps), 1)
    backend.device_status()

    peaks = measured_peaks()
    peak_fp8 = 2.0 * peaks["bf16_sustained"]
    value = flops * args.steps / secs / 1e12
    achieved = gemm_flops / (gemm_ms / 1e3) / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8 (e4m3 fwd / e5m2 grad, fp32 accumulate in TMEM, bf16 out)", "data": "synthetic",
        "config": {"workload": wl["name"], "routed_rows": rows, "group_sizes": sizes.tolist(),
                   "l2": "operands (2.8 GB of weights + 0.8 GB of activations per step) far exceed the 126 MB L2",
                   "recipe": "delayed scaling, amax history 16"},
        "tokens_per_s": wl["tokens"] * args.steps / secs,
        "frac_of_nominal_fp8_peak": value / NOMINAL_FP8_TFLOPS,
        "clocks": clocks.summary(),
        "e2e": {"value": flops * args.steps / secs_e2e / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": e2e.h2d_bytes, "d2h_bytes_per_step": e2e.d2h_bytes,
                "ms_per_step": secs_e2e / args.steps * 1e3,
                "how": "GroupedMlp forward + backward per step; inputs copied from pinned host memory and results read "
                       "back every step on side streams (next step's inputs prefetched during this step's compute)"},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "grouped_gemm_pair_kernel (tcgen05; 6 GEMM calls per step, events around each call; the four "
                               "forward/dgrad calls add a short grouped_gemm_kernel launch for the groups' tails)", "bound": "tensor",
                     "achieved": achieved, "peak": peak_fp8, "unit": "TFLOP/s", "frac": achieved / peak_fp8,
                     "peak_source": f"2 x {peaks['source']} dense bf16 sustained ({peaks['bf16_sustained']} TFLOP/s)",
                     "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                     "launches_timed": n_gemm, "mean_launch_ms": gemm_ms / max(n_gemm, 1),
                     "flops_per_launch": gemm_flops / max(n_gemm, 1),
                     "gemm_share_of_step": (gemm_ms / 1e3) / secs,
                     "traffic": GEMM_DRAM_BYTES_PER_LAUNCH},
    }
    if not args.no_cpu_baseline:
        cstep, cflops, desc = cpu_sample_step(H, F, rows // E)
        ctf, _ = run_cpu(cstep, cflops, reps=3, warmup=1)
        line["cpu_baseline"] = {"value": ctf, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                                "sample": desc}
    if not args.no_extras:
        # the same step as a later micro-batch of a gradient-accumulation window: the FP8 weights cast by the first
        # micro-batch are reused (is_first_microbatch=False), so the 4.2 GB of weight casts per step disappear
        def cached_step():
            mlp.fc1_weight.grad = mlp.fc2_weight.grad = x_dev.grad = None
            with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
                out = mlp(x_dev, sizes, is_first_microbatch=False)
            out.backward(dy_dev)

        mlp.fc1_weight.grad = mlp.fc2_weight.grad = x_dev.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            mlp(x_dev, sizes, is_first_microbatch=True).backward(dy_dev)
        for _ in range(2):
            cached_step()
        secs_cached = timed_steps(cached_step, args.steps)
        line["weight_cache"] = {"ms_per_step": secs_cached / args.steps * 1e3, "tflops": flops * args.steps / secs_cached / 1e12,
                                "what": "micro-batches after the first of an accumulation window (is_first_microbatch=False): "
                                        "FP8 weights reused, no weight casts"}
        del cached_step
        # free the step's tensors first: the microbenchmark holds about 20 GB
        del mlp, x_dev, dy_dev, e2e, step, step_on
        torch.cuda.empty_cache()
        import bench_kernels

        line["fine_grained"] = fine_grained_leg(fg, backend, dev, args.steps)
        line["pad"] = bench_kernels.pad_suite(backend, dev)
        line["pad"]["peak_hbm_gbs"] = {"measured_copy": peaks["hbm_gbs"], "nominal": 8000.0}
        line["library_gemm"] = bench_kernels.library_gemm_suite(backend, dev, sizes.tolist())
        backend.device_status()
    print(json.dumps(line), flush=True)


def fine_grained_leg(fg, backend, dev, steps):
    """The fine-grained MoE step (small, empty and ragged groups) through GroupedMlp: ms per step and TFLOP/s."""
    wl = fine_grained_workload()
    E, H, F, rows, sizes = wl["E"], wl["H"], wl["F"], wl["rows"], wl["sizes"]
    torch.manual_seed(4)
    mlp = fg.GroupedMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu")
    with torch.no_grad():
        mlp.fc1_weight.normal_(0.0, 0.02)
        mlp.fc2_weight.normal_(0.0, 0.02)
    x = torch.randn(rows, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    recipe = fg.DelayedScaling(amax_history_len=16)

    def step():
        mlp.fc1_weight.grad = mlp.fc2_weight.grad = x.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = mlp(x, sizes)
        out.backward(dy)

    for _ in range(3):
        step()
    timings = []
    backend.set_gemm_timings(timings)
    secs = timed_steps(step, steps)
    backend.set_gemm_timings(None)
    gemm_ms = sum(s.elapsed_time(e) for s, e, _ in timings)
    flops = mlp_flops(rows, H, F)
    return {"workload": "fine-grained MoE (E=64, hidden 2048, ffn 1408, SwiGLU, 8192 tokens top-6, Zipf(1.2) loads)",
            "group_sizes_min_median_max": [int(sizes.min()), int(sizes.median()), int(sizes.max())],
            "empty_groups": int((sizes == 0).sum()), "ragged_groups": int((sizes % 16 != 0).sum()),
            "ms_per_step": secs / steps * 1e3, "tflops": flops * steps / secs / 1e12,
            "gemm_share_of_step": (gemm_ms / 1e3) / secs}


def main():
    args = parse()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    workload = args.workload
    if workload == "auto":
        workload = "mixtral" if max(world, args.gpus) == 1 else "ep"
    if args.impl == "reference":
        if workload == "mixtral":
            wl = mixtral_workload()
            reference_arm(args, wl["name"], wl["H"], wl["F"], wl["rows"] // wl["E"])
        else:
            reference_arm(args, EP["name"], EP["H"], EP["F"], EP["rows_per_expert"] * 8)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: fp8_gmm_b200 has no CPU path (use --impl reference for the CPU baseline)")
    if workload == "mixtral":
        run_single(args)
    else:
        import bench_ep

        bench_ep.run(args, METRIC, EP, measured_peaks(), ClockSampler, cpu_sample_step, run_cpu)


if __name__ == "__main__":
    main()
