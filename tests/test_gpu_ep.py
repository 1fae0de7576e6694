"""GPU, 2 ranks (skipped on a single-GPU machine): ExpertParallelMlp over NCCL equals one GroupedMlp that holds all
experts on one GPU, forward and backward, on the first step of delayed scaling (all scales 1)."""
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
                                     transport=transport.split("-")[0], num_chunks=2,
                                     fp8_dispatch=not transport.endswith("bf16"))
        with torch.no_grad():
            model.mlp.fc1_weight.copy_(w1[rank * El:(rank + 1) * El])
            model.mlp.fc2_weight.copy_(w2[rank * El:(rank + 1) * El])
        x = xs[rank].to(dev).requires_grad_(True)
        with fg.fp8_autocast(enabled=True):
            out = model(x, _sizes(rank))
        out.backward(dys[rank].to(dev))
        fg.backend.device_status()
        if transport.startswith("peer"):
            # a second step reuses the receive buffers and the result pool: same inputs, same state -> same results
            first = (out.detach().clone(), x.grad.clone(), model.mlp.fc1_weight.grad.clone())
            del out
            x.grad, model.mlp.fc1_weight.grad, model.mlp.fc2_weight.grad = None, None, None
            model.mlp.fp8_meta_tensors_initialized = False   # restart delayed scaling so step 2 repeats step 1
            with fg.fp8_autocast(enabled=True):
                out = model(x, _sizes(rank))
            out.backward(dys[rank].to(dev))
            fg.backend.device_status()
            assert torch.equal(out, first[0]) and torch.equal(x.grad, first[1])
            assert torch.equal(model.mlp.fc1_weight.grad, first[2])
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
        xr = torch.cat(blocks_x).to(dev).requires_grad_(True)
        with fg.fp8_autocast(enabled=True):
            outr = ref(xr, all_sizes.sum(0))
        outr.backward(torch.cat(blocks_dy).to(dev))
        pos = 0
        for r, lo, n in where:
            if r == rank and n:
                assert torch.allclose(out[lo:lo + n].float(), outr[pos:pos + n].float(), rtol=2e-2, atol=2e-2)
                assert torch.allclose(x.grad[lo:lo + n].float(), xr.grad[pos:pos + n].float(), rtol=2e-2, atol=2e-2)
            pos += n
        gw = ref.fc1_weight.grad[rank * El:(rank + 1) * El].float()
        rel = (model.mlp.fc1_weight.grad.float() - gw).norm() / gw.norm()
        assert float(rel) < 1e-2, float(rel)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        errq.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("transport", ["nccl", "peer", "peer-bf16"])
def test_expert_parallel_matches_single_gpu(cuda, transport):
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = 29900 + os.getpid() % 90 + {"nccl": 0, "peer": 100, "peer-bf16": 200}[transport]
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
