"""Expert-parallel leg of bench.py: one rank per GPU, NCCL all-to-all dispatch / combine around GroupedMlp.

Workload (synthetic, seeded; BASELINE config 4): 128 experts split evenly over the ranks, hidden 4096, ffn 1536,
SwiGLU, 32768 tokens per GPU routed top-8 (softmax over N(0,1) logits, 8 distinct experts per token) = 262144
routed rows per GPU, delayed scaling with an amax history of 16.  Weak scaling: the per-GPU work is fixed.
"""
import json
import os
import time

import torch
import torch.distributed as dist

E, H, F, TOKENS_PER_GPU, TOPK = 128, 4096, 1536, 32768, 8
ROWS_PER_EXPERT = TOKENS_PER_GPU * TOPK // E  # per source rank; used to size the CPU baseline sample
WORKLOAD_NAME = ("expert-parallel GroupedMLP (E=128 split over the ranks, hidden 4096, ffn 1536, SwiGLU, "
                 "32768 tokens/GPU top-8, all-to-all dispatch/combine)")


def routed_sizes(seed):
    g = torch.Generator().manual_seed(seed)
    probs = torch.softmax(torch.randn(TOKENS_PER_GPU, E, generator=g), dim=-1)
    picks = torch.multinomial(probs, TOPK, replacement=False, generator=g)
    return torch.bincount(picks.reshape(-1), minlength=E)


def _timed(fn, steps, world):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    secs = torch.tensor([start.elapsed_time(end) / 1e3], device="cuda")
    if world > 1:
        dist.barrier()
        dist.all_reduce(secs, op=dist.ReduceOp.MAX)
    return float(secs)


def run(args, metric, peaks, ClockSampler, cpu_sample_step, run_cpu, E2EPipeline):
    import fp8_gmm_b200 as fg
    from fp8_gmm_b200 import backend, ep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    sizes = routed_sizes(1000 + rank)
    rows = int(sizes.sum())
    g = torch.Generator().manual_seed(2000 + rank)
    x_host = torch.randn(rows, H, generator=g).to(torch.bfloat16).pin_memory()
    dy_host = torch.randn(rows, H, generator=g).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(rows, H, dtype=torch.bfloat16).pin_memory()
    gi_host = torch.empty(rows, H, dtype=torch.bfloat16).pin_memory()
    torch.manual_seed(3000 + rank)
    spec = str(args.ep_chunks)
    chunks = spec if spec == "tapered" else int(spec) if spec.isdigit() else [int(v) for v in spec.split(",")]
    model = ep.ExpertParallelMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu",
                                 transport=args.ep_transport, num_chunks=chunks,
                                 fp8_dispatch=not args.ep_bf16_dispatch)
    with torch.no_grad():
        model.mlp.fc1_weight.normal_(0.0, 0.02)
        model.mlp.fc2_weight.normal_(0.0, 0.02)
    x_dev = x_host.to(dev).requires_grad_(True)
    dy_dev = dy_host.to(dev)
    recipe = fg.DelayedScaling(amax_history_len=16)

    host = {"fwd": 0.0, "bwd": 0.0, "n": 0}   # host time spent enqueueing (no synchronisation inside)

    def step():
        model.mlp.fc1_weight.grad = None
        model.mlp.fc2_weight.grad = None
        x_dev.grad = None
        t0 = time.perf_counter()
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = model(x_dev, sizes)
        t1 = time.perf_counter()
        out.backward(dy_dev)
        host["fwd"] += t1 - t0
        host["bwd"] += time.perf_counter() - t1
        host["n"] += 1
        return out

    def step_on(x_in, dy_in):
        model.mlp.fc1_weight.grad = None
        model.mlp.fc2_weight.grad = None
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = model(x_in, sizes)
        out.backward(dy_in)
        return out, x_in.grad

    e2e = E2EPipeline(step_on, x_host, dy_host, out_host, gi_host, dev)

    warmup = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    for _ in range(warmup):
        step()
    backend.device_status()

    # Timed region: K clean steps.  The per-launch GEMM events (roofline) and the events around every wait for
    # rows are taken in a second pass of the same K steps right after: with six chunks a step issues 36 GEMMs and
    # 14 waits, and two event records around each of them cost host time that the timed region should not carry.
    launches0 = backend.launch_count()
    host.update(fwd=0.0, bwd=0.0, n=0)
    with sampler as clocks:
        secs = _timed(step, args.steps, world)
    host_ms = (host["fwd"] / max(host["n"], 1) * 1e3, host["bwd"] / max(host["n"], 1) * 1e3)
    launches = backend.launch_count() - launches0

    channel = None
    if world > 1 and args.ep_transport == "peer":
        from fp8_gmm_b200 import ep_peer

        ectx = ep_peer.EpContext.get(dev, model.group)
        channel = ectx.channel
        channel.wait_events = ectx.channel_back.wait_events = []   # one shared list, in program order
    timings = []
    backend.set_gemm_timings(timings)
    _timed(step, args.steps, world)
    backend.set_gemm_timings(None)
    exposed_ms = None
    if channel is not None:
        exposed_ms = sum(s.elapsed_time(e) for s, e in channel.wait_events) / args.steps
        per_step = len(channel.wait_events) // args.steps
        last_step_waits = [round(s.elapsed_time(e), 3) for s, e in channel.wait_events[-per_step:]]
        channel.wait_events = ectx.channel_back.wait_events = None
    gemm_ms = sum(s.elapsed_time(e) for s, e, _ in timings)
    gemm_flops_local = sum(f for _, _, f in timings)

    e2e.run(2)
    secs_e2e = _timed(lambda: e2e.run(args.steps), 1, world)

    # the same local problem without the exchange (what this rank's experts compute), for the EP efficiency figure
    local_secs = None
    if world > 1:
        plan = ep.make_plan(sizes, dev)
        local_rows = int(plan.local_group_sizes.sum())
        lx = torch.randn(local_rows, H, device=dev, dtype=torch.bfloat16).requires_grad_(True)
        ldy = torch.randn(local_rows, H, device=dev, dtype=torch.bfloat16)

        def local_step():
            model.mlp.fc1_weight.grad = None
            model.mlp.fc2_weight.grad = None
            lx.grad = None
            with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
                o = model.mlp(lx, plan.local_group_sizes)
            o.backward(ldy)

        for _ in range(3):
            local_step()
        local_secs = _timed(local_step, args.steps, world)
    backend.device_status()

    total_rows = torch.tensor([float(rows)], device=dev)
    if world > 1:
        dist.all_reduce(total_rows)
    flops = 18.0 * float(total_rows) * H * F  # every routed row is processed exactly once, on the rank owning its expert
    if rank == 0:
        peak_fp8 = 2.0 * peaks["bf16_sustained"]
        value = flops * args.steps / secs / 1e12
        achieved = gemm_flops_local / (gemm_ms / 1e3) / 1e12
        line = {
            "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8 (e4m3 fwd / e5m2 grad, fp32 accumulate in TMEM, bf16 out)", "data": "synthetic",
            "config": {"workload": WORKLOAD_NAME, "parallelism": f"ep{world}", "experts_per_gpu": E // world,
                       "exchange": (f"copy-engine pushes into peer memory ({'bf16' if args.ep_bf16_dispatch else 'FP8'} dispatch, bf16 combine), "
                                    f"{args.ep_chunks} expert chunks pipelined with the GEMMs"
                                    if args.ep_transport == "peer" and world > 1 else "NCCL all-to-all" if world > 1 else "none"),
                       "routed_rows_per_gpu": TOKENS_PER_GPU * TOPK,
                       "l2": "operands (2.1 GB of activations per GPU per exchange, 0.2-2.4 GB of weights) exceed the 126 MB L2",
                       "recipe": "delayed scaling, amax history 16"},
            "tokens_per_s": TOKENS_PER_GPU * world * args.steps / secs,
            "tokens_per_s_per_gpu": TOKENS_PER_GPU * args.steps / secs,
            "frac_of_nominal_fp8_peak": value / (4500.0 * world),
            "clocks": clocks.summary(),
            "e2e": {"value": flops * args.steps / secs_e2e / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": (x_host.numel() + dy_host.numel()) * 2 * world,
                    "d2h_bytes_per_step": (out_host.numel() + gi_host.numel()) * 2 * world,
                    "ms_per_step": secs_e2e / args.steps * 1e3},
            "gpu_launches": int(launches),
            "roofline": {"kernel": "grouped_gemm kernels on rank 0 (tcgen05; per-launch CUDA events in a second pass of the same steps)", "bound": "tensor",
                         "achieved": achieved, "peak": peak_fp8, "unit": "TFLOP/s", "frac": achieved / peak_fp8,
                         "peak_source": f"2 x {peaks['source']} dense bf16 sustained ({peaks['bf16_sustained']} TFLOP/s)",
                         "frac_of_nominal_4500": achieved / 4500.0, "launches_timed": len(timings),
                         "mean_launch_ms": gemm_ms / max(len(timings), 1),
                         "flops_per_launch": gemm_flops_local / max(len(timings), 1),
                         "gemm_share_of_step": (gemm_ms / 1e3) / secs, "traffic": None},
        }
        if local_secs is not None:
            line["ep"] = {"local_ms_per_step_without_exchange": local_secs / args.steps * 1e3,
                          "efficiency_vs_local": local_secs / secs,
                          "ms_per_step_waiting_for_rows_rank0": exposed_ms}
            if exposed_ms is not None:
                line["ep"]["waits_ms_last_step_rank0"] = last_step_waits
            # forward includes the host's wait for the size exchange; backward is pure enqueue time
            line["ep"]["host_ms_per_step_rank0"] = {"forward": host_ms[0], "backward": host_ms[1]}
        if world == 1 and not args.no_cpu_baseline:
            cstep, cflops, desc = cpu_sample_step(H, F, ROWS_PER_EXPERT * 8)
            ctf, _ = run_cpu(cstep, cflops, reps=3, warmup=1)
            line["cpu_baseline"] = {"value": ctf, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
