"""CPU, 2 gloo ranks: the expert-parallel exchange logic (split sizes, block permutation, dispatch / combine and
their gradients) and the host-side peer-liveness check.  The local expert computation is replaced by a function
that tags rows with their global expert, so the test proves that every row reaches the rank that owns its expert,
in expert-major order, and comes back to the place it started from."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

WORLD = 2
E = 6  # global experts, 3 per rank


def _init(rank, port, timeout_s=30):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD, timeout=datetime.timedelta(seconds=timeout_s))


def _rank_sizes(rank):
    g = torch.Generator().manual_seed(100 + rank)
    sizes = torch.randint(0, 7, (E,), generator=g)
    sizes[(rank + 2) % E] = 0  # an expert that this rank sends nothing to
    return sizes


def _worker_roundtrip(rank, port, errq):
    try:
        from fp8_gmm_b200 import ep

        _init(rank, port)
        sizes = _rank_sizes(rank)
        rows = int(sizes.sum())
        expert_of_row = torch.repeat_interleave(torch.arange(E), sizes)
        # row payload: (source rank, source row, global expert)
        x = torch.stack([torch.full((rows,), float(rank)), torch.arange(rows, dtype=torch.float32), expert_of_row.float()], 1)
        x.requires_grad_(True)
        plan = ep.make_plan(sizes, torch.device("cpu"))
        all_sizes = torch.stack([_rank_sizes(r) for r in range(WORLD)])          # what every rank holds
        El = E // WORLD
        mine = all_sizes[:, rank * El:(rank + 1) * El]                            # (src, local expert)
        assert plan.send_rows == sizes.reshape(WORLD, El).sum(1).tolist()
        assert plan.recv_rows == mine.sum(1).tolist()
        assert torch.equal(plan.local_group_sizes, mine.sum(0))
        local = ep.dispatch(x, plan)
        # expert-major: all rows of local expert 0 (from src 0, then src 1), then expert 1, ...
        want_expert = torch.repeat_interleave(torch.arange(El) + rank * El, plan.local_group_sizes).float()
        assert torch.equal(local[:, 2].detach(), want_expert)
        pos = 0
        for e in range(El):
            for src in range(WORLD):
                n = int(mine[src, e])
                blk = local[pos:pos + n].detach()
                assert (blk[:, 0] == src).all()
                assert (blk[:, 1][1:] > blk[:, 1][:-1]).all()  # source order kept inside a block
                pos += n
        # stand-in for the local experts: scale every row by (global expert + 1)
        y = local * (local[:, 2:3].detach() + 1.0)
        out = ep.combine(y, plan)
        assert torch.equal(out.detach(), x.detach() * (expert_of_row.float()[:, None] + 1.0))
        w = torch.arange(1, rows * 3 + 1, dtype=torch.float32).reshape(rows, 3)
        (out * w).sum().backward()
        assert torch.equal(x.grad, w * (expert_of_row.float()[:, None] + 1.0))
        dist.barrier()
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        errq.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


def _worker_peer_loss(rank, port, store_path, errq):
    try:
        from fp8_gmm_b200 import ep

        _init(rank, port)
        store = dist.FileStore(store_path, WORLD)
        mon = ep.PeerMonitor(store, rank, WORLD, timeout_s=2.0)
        mon.check(0)  # both alive
        dist.barrier()
        if rank == 1:
            # this rank "dies" between steps: it raises on the host with nothing in flight and never reaches step 1
            dist.destroy_process_group()
            return
        try:
            mon.check(1)
            errq.put("rank 0 did not notice that its peer is gone")
        except RuntimeError as exc:
            assert "did not reach step 1" in str(exc)
        dist.destroy_process_group()
    except Exception as exc:  # noqa: BLE001
        errq.put(f"rank {rank}: {type(exc).__name__}: {exc}")
        raise


def _run(target, extra=()):
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=target, args=(r, port) + tuple(extra) + (errq,)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
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


def test_block_permutation_is_a_permutation():
    from fp8_gmm_b200 import ep

    counts = torch.tensor([[2, 0, 3], [1, 4, 0]])
    fwd, inv = ep.block_permutation(counts)
    assert sorted(fwd.tolist()) == list(range(10))
    assert torch.equal(fwd[inv], torch.arange(10)) and torch.equal(inv[fwd], torch.arange(10))
    # source-major rows: src0 e0 (0,1) e2 (2,3,4); src1 e0 (5) e1 (6..9).  expert-major: e0: 0,1,5; e1: 6..9; e2: 2,3,4
    assert fwd.tolist() == [0, 1, 5, 6, 7, 8, 9, 2, 3, 4]
    src, dst, rows, grp = ep.permutation_blocks(counts)
    assert src.tolist() == [0, 2, 2, 5, 6, 10] and rows.tolist() == [2, 0, 3, 1, 4, 0] and grp.tolist() == [0, 1, 2, 0, 1, 2]
    assert dst.tolist() == [0, 3, 7, 2, 3, 10]
    for b in range(6):  # the block table and the per-row index describe the same permutation
        for i in range(int(rows[b])):
            assert fwd[int(dst[b]) + i] == int(src[b]) + i
    empty_f, empty_i = ep.block_permutation(torch.zeros(2, 3, dtype=torch.int64))
    assert empty_f.numel() == 0 and empty_i.numel() == 0


def test_dispatch_combine_round_trip_on_two_gloo_ranks():
    _run(_worker_roundtrip)


def test_peer_loss_between_steps_is_detected_on_the_host():
    with tempfile.TemporaryDirectory() as d:
        _run(_worker_peer_loss, extra=(os.path.join(d, "store"),))
