"""Expert-parallel leg of bench.py (N > 1): one rank per GPU, dispatch / combine around GroupedMlp.

Workload: bench.EP (128 experts split evenly over the ranks, hidden 4096, ffn 1536, SwiGLU, 32768 tokens per GPU
routed top-8 = 262144 routed rows per GPU, delayed scaling with an amax history of 16).  Weak scaling: the per-GPU
work is fixed.  Legs, all CUDA-event timed, max over ranks:

* the timed step: rows already sorted by expert and resident in HBM -> ExpertParallelMlp forward + backward;
* a second pass of the same steps with events around every GEMM launch (roofline) and every wait for rows;
* the same rank's experts and rows without any exchange ("local"), for ``ep.efficiency_vs_local``;
* ``e2e``: tokens, expert ids and router weights come from pinned host memory every step, rows are sorted and
  gathered on the device (fp8_gmm_b200.routing), run through the expert-parallel MLP, scattered back with the router
  weights, and the tokens' results and input gradients are read back to the host;
* ``ep.check``: one more step from a snapshot of the FP8 state, run once over the peer-memory pipeline and once over
  the NCCL all-to-all transport around the unchanged local GroupedMlp; results, input gradients and both weight
  gradients must be bit-identical on every rank.
"""
import json
import os
import time

import torch
import torch.distributed as dist


def routed_sizes(wl, seed):
    g = torch.Generator().manual_seed(seed)
    probs = torch.softmax(torch.randn(wl["tokens_per_gpu"], wl["E"], generator=g), dim=-1)
    picks = torch.multinomial(probs, wl["topk"], replacement=False, generator=g)
    return torch.bincount(picks.reshape(-1), minlength=wl["E"]), picks, probs.gather(1, picks)


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


def _gather_floats(values, world, dev):
    """[[rank 0's values], [rank 1's], ...] on every rank."""
    t = torch.tensor(values, dtype=torch.float64, device=dev)
    if world == 1:
        return [t.tolist()]
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t)
    return [p.tolist() for p in parts]


def check_against_nccl_transport(fg, ep, model, args, wl, x_dev, dy_dev, sizes, recipe, dev, world):
    """One step from a snapshot of the FP8 state, once through the model under test and once through the NCCL
    all-to-all transport around the unchanged local GroupedMlp (same parameters, same state): "equal", or the number
    of tensors that differ summed over ranks."""
    H, F, E = wl["H"], wl["F"], wl["E"]
    other = ep.ExpertParallelMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu", transport="nccl")
    other.mlp.fc1_weight, other.mlp.fc2_weight = model.mlp.fc1_weight, model.mlp.fc2_weight
    state = model.mlp.get_extra_state()
    results = []
    for m in (model, other):
        m.mlp.set_extra_state(state)
        m.mlp.fc1_weight.grad = m.mlp.fc2_weight.grad = None
        x = x_dev.detach().requires_grad_(True)
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = m(x, sizes)
        out.backward(dy_dev)
        results.append((out.detach().clone(), x.grad.clone(), m.mlp.fc1_weight.grad.clone(), m.mlp.fc2_weight.grad.clone()))
        del out, x
    bad = sum(0 if torch.equal(a, b) else 1 for a, b in zip(*results))
    total = torch.tensor([float(bad)], device=dev)
    dist.all_reduce(total)
    del other, results
    torch.cuda.empty_cache()
    return "equal" if int(total) == 0 else f"{int(total)} tensors differ"


def tensor_parallel_leg(fg, dev, world, steps):
    """The reference's one collective at the Mixtral-shaped sizes: every rank holds a 1/world slice of the ffn
    dimension of all 8 experts (fc1 column-parallel, fc2 row-parallel) and the same 32768 routed rows, so the input
    gradient has to be summed over the ranks (GroupedMlp(..., has_tp=True)).  Timed three ways: without the sum, with
    the chunked peer-memory reduction behind the fc1 data-gradient GEMM, and with the plain NCCL all-reduce."""
    import fp8_gmm_b200.grouped_mlp as gm
    from fp8_gmm_b200 import tp

    E, H, F, rows = 8, 4096, 14336 // world, 32768
    sizes = torch.full((E,), rows // E, dtype=torch.int64)
    torch.manual_seed(5)
    mlp = fg.GroupedMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu")
    with torch.no_grad():
        mlp.fc1_weight.normal_(0.0, 0.02)
        mlp.fc2_weight.normal_(0.0, 0.02)
    x = torch.randn(rows, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    dy = torch.randn(rows, H, device=dev).to(torch.bfloat16)
    recipe = fg.DelayedScaling(amax_history_len=16)

    def make(has_tp):
        def step():
            mlp.fc1_weight.grad = mlp.fc2_weight.grad = x.grad = None
            with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
                out = mlp(x, sizes, has_tp=has_tp, tp_group=dist.group.WORLD if has_tp else None)
            out.backward(dy)
        return step

    out = {}
    saved = os.environ.get("FP8GMM_TP")
    for name, has_tp, path in (("no_sum", False, None), ("peer_memory", True, "peer"), ("nccl_all_reduce", True, "nccl")):
        if path is not None:
            os.environ["FP8GMM_TP"] = path
        step = make(has_tp)
        for _ in range(3):
            step()
        out[name + "_ms_per_step"] = _timed(step, steps, world) / steps * 1e3
    if saved is None:
        os.environ.pop("FP8GMM_TP", None)
    else:
        os.environ["FP8GMM_TP"] = saved
    out["exposed_ms_peer_memory"] = out["peer_memory_ms_per_step"] - out["no_sum_ms_per_step"]
    out["exposed_ms_nccl_all_reduce"] = out["nccl_all_reduce_ms_per_step"] - out["no_sum_ms_per_step"]
    out["workload"] = (f"Mixtral-shaped GroupedMlp, ffn 14336 split over {world} ranks, 32768 rows, grad_input "
                       f"({rows} x {H} bf16 = {rows * H * 2 / 1e6:.0f} MB) summed over the ranks; {gm.TP_CHUNKS} chunks")
    return out


def run(args, metric, wl, peaks, ClockSampler, cpu_sample_step, run_cpu):
    import fp8_gmm_b200 as fg
    from bench import E2EPipeline
    from fp8_gmm_b200 import backend, ep, routing

    E, H, F, TOPK, TOKENS = wl["E"], wl["H"], wl["F"], wl["topk"], wl["tokens_per_gpu"]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    sizes, picks, gates = routed_sizes(wl, 1000 + rank)
    rows = int(sizes.sum())
    g = torch.Generator().manual_seed(2000 + rank)
    tok_host = torch.randn(TOKENS, H, generator=g).to(torch.bfloat16).pin_memory()
    dtok_host = torch.randn(TOKENS, H, generator=g).to(torch.bfloat16).pin_memory()
    ids_host = picks.to(torch.int32).contiguous().pin_memory()
    gates_host = gates.float().contiguous().pin_memory()
    y_host = torch.empty(TOKENS, H, dtype=torch.bfloat16).pin_memory()
    gtok_host = torch.empty(TOKENS, H, dtype=torch.bfloat16).pin_memory()
    torch.manual_seed(3000 + rank)
    spec = str(args.ep_chunks)
    chunks = spec if spec == "tapered" else int(spec) if spec.isdigit() else [int(v) for v in spec.split(",")]
    model = ep.ExpertParallelMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu",
                                 transport=args.ep_transport, num_chunks=chunks,
                                 fp8_dispatch=not args.ep_bf16_dispatch)
    with torch.no_grad():
        model.mlp.fc1_weight.normal_(0.0, 0.02)
        model.mlp.fc2_weight.normal_(0.0, 0.02)
    # rows sorted by expert, resident: what the timed step consumes (built once with the router-side kernels)
    route = routing.sort_by_expert(ids_host.to(dev), E)
    x_dev = routing.gather(tok_host.to(dev), route.indices, route.bin_ids, route.bins, TOPK).detach().requires_grad_(True)
    dy_dev = routing.gather(dtok_host.to(dev), route.indices, route.bin_ids, route.bins, TOPK).detach()
    assert x_dev.shape[0] == rows and torch.equal(route.tokens_per_expert.cpu(), sizes)
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

    def step_from_tokens(tok, dtok, ids, gate_w):
        """Tokens in, tokens out: sort by expert, gather, expert-parallel MLP, weighted scatter, and back."""
        model.mlp.fc1_weight.grad = None
        model.mlp.fc2_weight.grad = None
        tok_in = tok.detach().requires_grad_(True)
        r = routing.sort_by_expert(ids, E)
        # The module takes the group sizes as a CPU tensor.  The expert ids of this leg come from the host, so the
        # histogram is taken there (0.3 ms) instead of reading the device's back, which would stall the host behind
        # the GPU every step (the reference's example does the latter: fp8_gmm/example.py:54).
        group_sizes = torch.bincount(ids_host.reshape(-1), minlength=E)
        rows_in = routing.gather(tok_in, r.indices, r.bin_ids, r.bins, TOPK)
        with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
            out = model(rows_in, group_sizes)
        y = routing.scatter(out, r.indices, r.bin_ids, gate_w, r.bins, TOPK)
        y.backward(dtok)
        return y, tok_in.grad

    e2e = E2EPipeline(step_from_tokens, [tok_host, dtok_host, ids_host, gates_host], [y_host, gtok_host], dev)

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

        ectx = ep_peer.EpContext.setup(dev, model.group)
        channel = ectx.channel
        channel.wait_events = ectx.channel_back.wait_events = []   # one shared list, in program order
        channel.round_events, ectx.channel_back.round_events = [], []
    timings = []
    backend.set_gemm_timings(timings)
    _timed(step, args.steps, world)
    backend.set_gemm_timings(None)
    exposed_ms, last_step_waits, rounds = None, [], None
    if channel is not None:
        # copy rounds of the last traced step on this rank: when each round started (ms after the first dispatch round
        # of the step began), how long it took and at what rate it moved its bytes
        def round_table(events):
            per = len(events) // args.steps
            last = events[-per:]
            return [(round(first[0].elapsed_time(s), 2), round(s.elapsed_time(e), 2), round(b / max(s.elapsed_time(e), 1e-3) / 1e6, 1))
                    for s, e, b in last]

        first = channel.round_events[-(len(channel.round_events) // args.steps)]
        rounds = {"dispatch_start_ms_dur_ms_GBps": round_table(channel.round_events),
                  "combine_start_ms_dur_ms_GBps": round_table(ectx.channel_back.round_events)}
        channel.round_events = ectx.channel_back.round_events = None
        exposed_ms = sum(s.elapsed_time(e) for s, e in channel.wait_events) / args.steps
        per_step = len(channel.wait_events) // args.steps
        last_step_waits = [round(s.elapsed_time(e), 3) for s, e in channel.wait_events[-per_step:]]
        channel.wait_events = ectx.channel_back.wait_events = None
    gemm_ms = sum(s.elapsed_time(e) for s, e, _ in timings)
    gemm_flops_local = sum(f for _, _, f in timings)

    quick = bool(getattr(args, "ep_quick", False))
    secs_e2e = float("nan")
    if not quick:
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
        del lx, ldy
    backend.device_status()
    check = None
    if world > 1 and not quick:
        check = check_against_nccl_transport(fg, ep, model, args, wl, x_dev, dy_dev, sizes, recipe, dev, world)
        backend.device_status()

    tp_line = None
    e2e_bytes = (e2e.h2d_bytes, e2e.d2h_bytes)
    if world > 1 and not quick:
        del x_dev, dy_dev, e2e
        torch.cuda.empty_cache()
        tp_line = tensor_parallel_leg(fg, dev, world, args.steps)
        backend.device_status()
    total_rows = torch.tensor([float(rows)], device=dev)
    if world > 1:
        dist.all_reduce(total_rows)
    flops = 18.0 * float(total_rows) * H * F  # every routed row is processed exactly once, on the rank owning its expert
    per_rank = _gather_floats([host_ms[0], host_ms[1], exposed_ms or 0.0] + [float(w) for w in last_step_waits], world, dev)
    if rank == 0:
        peak_fp8 = 2.0 * peaks["bf16_sustained"]
        value = flops * args.steps / secs / 1e12
        achieved = gemm_flops_local / (gemm_ms / 1e3) / 1e12
        line = {
            "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp8 (e4m3 fwd / e5m2 grad, fp32 accumulate in TMEM, bf16 out)", "data": "synthetic",
            "config": {"workload": wl["name"], "parallelism": f"ep{world}", "experts_per_gpu": E // world,
                       "exchange": (f"peer memory: {'bf16' if args.ep_bf16_dispatch else 'FP8'} dispatch pushed by the copy engines, bf16 combine "
                                    + f"stored by the fc2 / fc1-dgrad GEMM epilogues straight into the tensors of home ranks {list(ep_peer.EpContext.setup(dev, model.group).direct_homes())} (rank 0's view), "
                                    + "staged and pushed by the copy engines for the others, "
                                    + f"{args.ep_chunks} expert chunks pipelined with the GEMMs"
                                    if args.ep_transport == "peer" and world > 1 else "NCCL all-to-all" if world > 1 else "none"),
                       "routed_rows_per_gpu": TOKENS * TOPK,
                       "l2": "operands (2.1 GB of activations per GPU per exchange, 0.2-2.4 GB of weights) exceed the 126 MB L2",
                       "recipe": "delayed scaling, amax history 16"},
            "tokens_per_s": TOKENS * world * args.steps / secs,
            "tokens_per_s_per_gpu": TOKENS * args.steps / secs,
            "frac_of_nominal_fp8_peak": value / (4500.0 * world),
            "clocks": clocks.summary(),
            "e2e": {"value": flops * args.steps / secs_e2e / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": e2e_bytes[0] * world, "d2h_bytes_per_step": e2e_bytes[1] * world,
                    "ms_per_step": secs_e2e / args.steps * 1e3,
                    "how": "per step and rank: tokens, output gradients, expert ids and router weights copied from pinned host "
                           "memory; sort / gather on the device (group sizes counted on the host from the same ids), "
                           "expert-parallel MLP forward + backward, weighted scatter; token results and token gradients read "
                           "back (copies on side streams, next step prefetched)"},
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
                          "efficiency_vs_local": local_secs / secs, "check": check,
                          "check_how": "one extra step from the same FP8 state through this transport and through NCCL all-to-all "
                                       "around the unchanged GroupedMlp: out, grad_input, both weight gradients, torch.equal on every rank",
                          # forward includes the host's wait for the size exchange; backward is pure enqueue time
                          "host_ms_per_step_by_rank": {"forward": [r[0] for r in per_rank], "backward": [r[1] for r in per_rank]},
                          "ms_per_step_waiting_for_rows_by_rank": [r[2] for r in per_rank],
                          "waits_ms_last_step_by_rank": [r[3:] for r in per_rank],
                          "copy_rounds_last_step_rank0": rounds}
        if tp_line is not None:
            line["tp"] = tp_line
        if not args.no_cpu_baseline:
            cstep, cflops, desc = cpu_sample_step(H, F, wl["rows_per_expert"] * 8)
            ctf, _ = run_cpu(cstep, cflops, reps=3, warmup=1)
            line["cpu_baseline"] = {"value": ctf, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
