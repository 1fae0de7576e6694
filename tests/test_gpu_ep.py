"""GPU, 2 ranks (skipped on a single-GPU machine): ExpertParallelMlp equals, bit for bit, one GroupedMlp that holds
all experts on one GPU -- forward, backward, weight gradients and FP8 recipe state -- over two steps of delayed
scaling, for the NCCL all-to-all transport and for the peer-memory transport with FP8 and with bf16 dispatch, results
going home through the GEMM epilogue's peer stores or through staged copies (the second step reuses the receive
buffers and the result pool)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
WORLD, E, H, F = 2, 8, 256, 384


def _sizes(rank):
    g = torch.Generator().manual_seed(50 + rank)
    s = torch.randint(0, 90, (E,), generator=g)
    s[(3 * rank + 1) % E] = 0
    return s


def _worker(rank, port, errq, transport):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        if transport.startswith("peer"):
            # how results go home: stored by the GEMM epilogue into the home rank's tensor (all rows, or only the
            # rank's own with the other rank's rows staged and copied), or all staged and pushed by the copy engines
            os.environ["FP8GMM_EP_DIRECT"] = "none" if transport.endswith("staged") else "0" if transport.endswith("mixed") else "all"
            transport = transport.replace("-staged", "").replace("-mixed", "")
        # four chunks of one expert, the merged forward dispatch sending two chunks per round (FP8 dispatch only)
        chunks = 4 if transport == "peer" else 2
        os.environ["FP8GMM_EP_DISPATCH_ROUNDS"] = "2,2"
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev)
        import fp8_gmm_b200 as fg
        from fp8_gmm_b200 import ep

        g = torch.Generator().manual_seed(7)
        w1 = (torch.randn(E, 2 * F, H, generator=g) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(E, H, F, generator=g) * 0.05).to(torch.bfloat16)
        xs, dys = [], []
        for r in range(WORLD):
            gr = torch.Generator().manual_seed(70 + r)
            n = int(_sizes(r).sum())
            xs.append(torch.randn(n, H, generator=gr).to(torch.bfloat16))
            dys.append(torch.randn(n, H, generator=gr).to(torch.bfloat16))
        El = E // WORLD
        model = ep.ExpertParallelMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu",
                                     transport=transport.split("-")[0], num_chunks=chunks,
                                     fp8_dispatch=not transport.endswith("bf16"))
        with torch.no_grad():
            model.mlp.fc1_weight.copy_(w1[rank * El:(rank + 1) * El])
            model.mlp.fc2_weight.copy_(w2[rank * El:(rank + 1) * El])
        # single-GPU reference on this rank: all experts, rows of both source ranks interleaved expert-major
        ref = fg.GroupedMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu")
        with torch.no_grad():
            ref.fc1_weight.copy_(w1)
            ref.fc2_weight.copy_(w2)
        all_sizes = torch.stack([_sizes(r) for r in range(WORLD)])
        blocks_x, blocks_dy, where = [], [], []
        for e in range(E):
            for r in range(WORLD):
                lo = int(all_sizes[r, :e].sum())
                n = int(all_sizes[r, e])
                blocks_x.append(xs[r][lo:lo + n])
                blocks_dy.append(dys[r][lo:lo + n])
                where.append((r, lo, n))
        x = xs[rank].to(dev).requires_grad_(True)
        xr = torch.cat(blocks_x).to(dev).requires_grad_(True)
        dyr = torch.cat(blocks_dy).to(dev)
        recipe = fg.DelayedScaling(amax_history_len=4)
        G = E
        own = slice(rank * El, (rank + 1) * El)

        def slots(meta, per, groups, first, count):
            """Meta slots (scale / amax history columns) of experts [first, first + count) of a module with `groups`
            experts: `per` slots per GEMM, fc1's GEMMs first, then fc2's (fp8_gmm/utils.py:98-103 of the reference)."""
            idx = [per * (half * groups + first + j) + t for half in range(2) for j in range(count) for t in range(per)]
            return meta[..., idx]

        # Two steps of delayed scaling: the first runs with all scales 1, the second with scales derived from the
        # first step's amaxes (under FP8 dispatch those travel from the owners to the sources and back as partial
        # amaxes).  The design promises the bytes a single GPU would have produced, so everything is compared with
        # torch.equal: results, input gradients, both weight gradients, the amax history and the scales.
        for step in range(2):
            x.grad = xr.grad = None
            for m in (model.mlp, ref):
                m.fc1_weight.grad = m.fc2_weight.grad = None
            with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
                out = model(x, _sizes(rank))
            out.backward(dys[rank].to(dev))
            with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
                outr = ref(xr, all_sizes.sum(0))
            outr.backward(dyr)
            fg.backend.device_status()
            pos = 0
            for r, lo, n in where:
                if r == rank and n:
                    assert torch.equal(out[lo:lo + n], outr[pos:pos + n]), f"step {step}: out differs"
                    assert torch.equal(x.grad[lo:lo + n], xr.grad[pos:pos + n]), f"step {step}: grad_input differs"
                pos += n
            assert torch.equal(model.mlp.fc1_weight.grad, ref.fc1_weight.grad[own]), f"step {step}: fc1 weight gradient"
            assert torch.equal(model.mlp.fc2_weight.grad, ref.fc2_weight.grad[own]), f"step {step}: fc2 weight gradient"
            for key, per in (("scaling_fwd", 3), ("scaling_bwd", 2)):
                mine, whole = model.mlp.fp8_meta[key], ref.fp8_meta[key]
                assert torch.equal(mine.amax_history, slots(whole.amax_history, per, G, rank * El, El)), f"step {step}: {key} amax"
                assert torch.equal(mine.scale, slots(whole.scale, per, G, rank * El, El)), f"step {step}: {key} scale"
            del out, outr
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        errq.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("transport", ["nccl", "peer", "peer-bf16", "peer-staged", "peer-mixed"])
def test_expert_parallel_matches_single_gpu(cuda, transport):
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = 29900 + os.getpid() % 90 + {"nccl": 0, "peer": 100, "peer-bf16": 200, "peer-staged": 300, "peer-mixed": 400}[transport]
    procs = [ctx.Process(target=_worker, args=(r, port, errq, transport)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errors.append("a rank did not finish in time")
        elif p.exitcode != 0:
            errors.append(f"exit code {p.exitcode}")
    assert not errors, errors
