"""GPU, 2 ranks (skipped on a single-GPU machine): GroupedMlp(..., has_tp=True, tp_group=...) returns the sum of the
ranks' input gradients -- the reference's only collective (fp8_gmm/grouped_mlp.py:300-303,323-324) -- through the
chunked peer-memory reduction (default on NCCL groups) and through the plain NCCL all-reduce (FP8GMM_TP=nccl)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
WORLD, E, H, F = 2, 6, 256, 384
SIZES = [70, 0, 33, 128, 5, 200]


def _worker(rank, port, errq, path):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", FP8GMM_TP=path)
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev)
        import fp8_gmm_b200 as fg

        # every rank holds its own slice of the ffn dimension (fc1 column-parallel, fc2 row-parallel) and sees the
        # same rows and the same output gradient
        gw = torch.Generator().manual_seed(100 + rank)
        w1 = (torch.randn(E, 2 * F, H, generator=gw) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn(E, H, F, generator=gw) * 0.05).to(torch.bfloat16)
        g = torch.Generator().manual_seed(5)
        rows = sum(SIZES)
        x0 = torch.randn(rows, H, generator=g).to(torch.bfloat16)
        dy = torch.randn(rows, H, generator=g).to(torch.bfloat16).to(dev)

        def run(has_tp, steps):
            mlp = fg.GroupedMlp(H, F, E, torch.bfloat16, device=dev, activation="swiglu")
            with torch.no_grad():
                mlp.fc1_weight.copy_(w1)
                mlp.fc2_weight.copy_(w2)
            res = []
            for _ in range(steps):
                x = x0.to(dev).requires_grad_(True)
                mlp.fc1_weight.grad = mlp.fc2_weight.grad = None
                with fg.fp8_autocast(enabled=True, fp8_recipe=fg.DelayedScaling(amax_history_len=4)):
                    out = mlp(x, torch.tensor(SIZES), has_tp=has_tp, tp_group=dist.group.WORLD if has_tp else None)
                out.backward(dy)
                fg.backend.device_status()
                res.append((out.detach().clone(), x.grad.clone(), mlp.fc1_weight.grad.clone(), mlp.fc2_weight.grad.clone()))
            return res

        local = run(False, 2)
        summed = run(True, 2)      # the second step reuses the staging buffer
        for step in range(2):
            parts = [torch.empty_like(local[step][1]) for _ in range(WORLD)]
            dist.all_gather(parts, local[step][1])
            want = (parts[0].float() + parts[1].float()).to(torch.bfloat16)
            got = summed[step][1]
            if path == "peer":
                assert torch.equal(got, want), f"step {step}: peer-memory sum differs from the sum of the parts"
            else:
                assert torch.allclose(got.float(), want.float(), rtol=2 ** -7, atol=1e-6)
            # every rank ends with the same bits
            both = [torch.empty_like(got) for _ in range(WORLD)]
            dist.all_gather(both, got)
            assert torch.equal(both[0], both[1])
            # nothing else depends on has_tp
            assert torch.equal(summed[step][0], local[step][0])
            assert torch.equal(summed[step][2], local[step][2]) and torch.equal(summed[step][3], local[step][3])
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        errq.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


@pytest.mark.parametrize("path", ["peer", "nccl"])
def test_tensor_parallel_input_gradient_is_the_sum_over_ranks(cuda, path):
    if torch.cuda.device_count() < WORLD:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = 29700 + os.getpid() % 90 + (0 if path == "peer" else 100)
    procs = [ctx.Process(target=_worker, args=(r, port, errq, path)) for r in range(WORLD)]
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
