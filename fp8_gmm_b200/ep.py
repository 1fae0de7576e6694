"""Expert parallelism around an unchanged GroupedMlp: all-to-all dispatch / combine over NCCL.

The reference is single-GPU apart from one tensor-parallel all-reduce (fp8_gmm/grouped_mlp.py:300-303); its
example does "dispatch/combine" with megablocks gather/scatter on one device (fp8_gmm/example.py:52-59,85-92).
Experts shard naturally -- each expert's weights and FP8 metas live on exactly one rank -- so this module adds
the exchange step around the local grouped MLP:

    rows sorted by global expert  --counts a2a-->  --rows a2a (dispatch)-->  source-major blocks
        --block permutation-->  expert-major rows  --GroupedMlp(local experts)-->
        --inverse permutation-->  --rows a2a (combine)-->  rows in the caller's original order

Rank r owns experts [r*E/P, (r+1)*E/P).  The caller's contract is the reference's: rows already sorted by
(global) expert and a CPU int64 tensor of group sizes.  Backward runs the same two exchanges reversed (autograd
functions below).  Remote rows always land in local HBM through NCCL before any kernel of this package reads
them; no kernel here touches peer memory.  Everything except the local MLP is device-agnostic torch code, so the
routing logic is tested on gloo CPU ranks.
"""
from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class EpPlan:
    """Split sizes and block permutations of one exchange, computed on the host from the count exchange."""

    send_rows: list          # rows this rank sends to each destination rank
    recv_rows: list          # rows this rank receives from each source rank
    local_group_sizes: torch.Tensor  # CPU int64 (E_local,): rows per local expert after the exchange
    to_expert_major: torch.Tensor    # device int64 (R,): expert-major position i reads source-major row index[i]
    to_source_major: torch.Tensor    # device int64 (R,): inverse permutation
    group: object = None
    recv_counts: torch.Tensor = None  # CPU int64 (P, E_local)

    def row_permutation(self):
        """The same permutation in the block form the fused kernels take (backend.RowPermutation): the cast reads the
        source-major blocks and writes them expert-major, the GEMM epilogues write results back source-major."""
        from .backend import RowPermutation

        src_start, dst_start, rows, group = permutation_blocks(self.recv_counts)
        return RowPermutation(src_start, dst_start, rows, group, self.to_expert_major.to(torch.int32))


def exchange_counts(group_sizes, group=None):
    """All ranks learn how many rows of each of their local experts every source rank holds.

    group_sizes: CPU int64 (E,) rows per *global* expert on this rank.  Returns CPU int64 (P, E_local):
    recv_counts[src, e] = rows of local expert e that rank src will send.  One small all-to-all."""
    world = dist.get_world_size(group)
    E = group_sizes.numel()
    assert E % world == 0, "the number of experts must be divisible by the number of ranks"
    send = group_sizes.to(torch.int64).reshape(world, E // world).contiguous()
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    send_d = send.to(dev)
    recv_d = torch.empty_like(send_d)
    dist.all_to_all_single(recv_d, send_d, group=group)
    return recv_d.cpu()


def block_permutation(recv_counts):
    """Index vectors between the source-major layout the all-to-all delivers and the expert-major layout the
    grouped MLP consumes.  recv_counts: CPU int64 (P, E_local).  Returns (to_expert_major, to_source_major)."""
    P, El = recv_counts.shape
    counts = recv_counts.reshape(-1)                                   # block (src, e), source-major order
    starts = torch.cumsum(counts, 0) - counts                          # start row of block (src, e) in source-major
    order = torch.arange(P * El).reshape(P, El).t().reshape(-1)        # blocks in expert-major order: (e, src)
    blk_counts = counts[order]
    blk_starts = starts[order]
    total = int(counts.sum())
    if total == 0:
        empty = torch.empty(0, dtype=torch.int64)
        return empty, empty
    # row i of the expert-major layout belongs to block b(i) at offset o(i): source row = blk_starts[b] + o
    blk_of_row = torch.repeat_interleave(torch.arange(P * El), blk_counts)
    dst_starts = torch.cumsum(blk_counts, 0) - blk_counts
    offset = torch.arange(total) - dst_starts[blk_of_row]
    to_expert_major = blk_starts[blk_of_row] + offset
    to_source_major = torch.empty_like(to_expert_major)
    to_source_major[to_expert_major] = torch.arange(total)
    return to_expert_major, to_source_major


def permutation_blocks(recv_counts):
    """Block table of the source-major -> expert-major permutation: one block per (source rank, local expert).
    Returns CPU int64 tensors (src_start, dst_start, rows, group), blocks listed in source-major order."""
    P, El = recv_counts.shape
    counts = recv_counts.reshape(-1)
    src_start = torch.cumsum(counts, 0) - counts
    em = recv_counts.t().contiguous().reshape(-1)                    # blocks in expert-major order (e, src)
    em_start = (torch.cumsum(em, 0) - em).reshape(El, P).t().contiguous().reshape(-1)   # back to (src, e) order
    group = torch.arange(El).repeat(P)
    return src_start, em_start, counts.clone(), group


def make_plan(group_sizes, device, group=None):
    world = dist.get_world_size(group)
    E = group_sizes.numel()
    El = E // world
    recv_counts = exchange_counts(group_sizes, group)
    send_rows = group_sizes.to(torch.int64).reshape(world, El).sum(1).tolist()
    recv_rows = recv_counts.sum(1).tolist()
    fwd, inv = block_permutation(recv_counts)
    return EpPlan(send_rows=send_rows, recv_rows=recv_rows, local_group_sizes=recv_counts.sum(0).contiguous(),
                  to_expert_major=fwd.to(device, non_blocking=True), to_source_major=inv.to(device, non_blocking=True),
                  group=group, recv_counts=recv_counts)


class _AllToAllRows(torch.autograd.Function):
    """Row exchange with uneven splits; the gradient is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, send_rows, recv_rows, group):
        ctx.send_rows, ctx.recv_rows, ctx.group = send_rows, recv_rows, group
        out = x.new_empty((sum(recv_rows),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv_rows, input_split_sizes=send_rows, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        out = grad.new_empty((sum(ctx.send_rows),) + tuple(grad.shape[1:]))
        dist.all_to_all_single(out, grad.contiguous(), output_split_sizes=ctx.send_rows, input_split_sizes=ctx.recv_rows,
                               group=ctx.group)
        return out, None, None, None


class _PermuteRows(torch.autograd.Function):
    """out[i] = x[index[i]] for a permutation; the gradient gathers with the inverse (no atomics)."""

    @staticmethod
    def forward(ctx, x, index, inverse):
        ctx.save_for_backward(inverse)
        return x.index_select(0, index)

    @staticmethod
    def backward(ctx, grad):
        (inverse,) = ctx.saved_tensors
        return grad.index_select(0, inverse), None, None


def dispatch(x, plan):
    """Rows sorted by global expert on every rank -> rows of this rank's experts, expert-major."""
    recv = _AllToAllRows.apply(x, plan.send_rows, plan.recv_rows, plan.group)
    return _PermuteRows.apply(recv, plan.to_expert_major, plan.to_source_major)


def combine(y, plan):
    """Inverse of dispatch: expert-major rows of the local experts -> back to the ranks and order they came from."""
    back = _PermuteRows.apply(y, plan.to_source_major, plan.to_expert_major)
    return _AllToAllRows.apply(back, plan.recv_rows, plan.send_rows, plan.group)


class ExpertParallelMlp(torch.nn.Module):
    """GroupedMlp over ``num_experts`` experts sharded evenly over the ranks of ``group``.

    forward(input, group_sizes): input (rows, hidden) bf16 sorted by global expert, group_sizes CPU int64
    (num_experts,) -- the reference's calling convention (fp8_gmm/grouped_mlp.py:347) with global experts.
    Returns (rows, hidden) in the same order.  ``world_size == 1`` degenerates to the plain GroupedMlp.
    """

    def __init__(self, in_features, out_features, num_experts, dtype, device="cuda", activation="gelu", group=None,
                 transport="auto", num_chunks=4, fp8_dispatch=True):
        """``transport``: "peer" = rows pushed by the copy engines into peer-mapped buffers, pipelined with the GEMMs
        in ``num_chunks`` chunks of experts (fp8_gmm_b200.ep_peer; one NVSwitch node, NCCL process group);
        "nccl" = NCCL all-to-all before and after the whole local MLP; "auto" = "peer" on an NCCL group.
        ``fp8_dispatch`` (peer transport): rows are cast to FP8 on the rank that holds them, with the owning rank's
        scale for their expert, and travel as FP8 -- the same bytes the owner would have produced, half the traffic;
        the partial amaxes travel with them and are max-merged at the owner."""
        super().__init__()
        from .grouped_mlp import GroupedMlp

        assert transport in ("auto", "peer", "nccl")
        self.transport, self.num_chunks, self.fp8_dispatch = transport, num_chunks, fp8_dispatch
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        assert num_experts % self.world == 0, "the number of experts must be divisible by the number of ranks"
        self.num_experts = num_experts
        self.local_experts = num_experts // self.world
        self.mlp = GroupedMlp(in_features, out_features, self.local_experts, dtype, device=device, activation=activation)

    def forward(self, input, group_sizes, is_first_microbatch=None):
        if not torch.is_tensor(group_sizes):
            group_sizes = torch.tensor(list(group_sizes), dtype=torch.int64)
        if self.world == 1:
            return self.mlp(input, group_sizes, is_first_microbatch=is_first_microbatch)
        transport = self.transport
        if transport == "auto":
            transport = "peer" if input.is_cuda and dist.get_backend(self.group) == "nccl" else "nccl"
        if transport == "peer":
            from . import ep_peer

            return ep_peer.forward(self, input, group_sizes, is_first_microbatch, self.num_chunks)
        plan = make_plan(group_sizes, input.device, self.group)
        # the exchange delivers rows source-major; the MLP's casts and GEMM epilogues apply the block permutation to
        # and from expert-major order themselves, so no gather / scatter pass runs on either side
        recv = _AllToAllRows.apply(input, plan.send_rows, plan.recv_rows, plan.group)
        out = self.mlp(recv, plan.local_group_sizes, is_first_microbatch=is_first_microbatch,
                       row_permutation=plan.row_permutation())
        return _AllToAllRows.apply(out, plan.recv_rows, plan.send_rows, plan.group)


class PeerMonitor:
    """Host-side liveness check between steps: every rank publishes a heartbeat for the step it is about to run and
    waits a bounded time for its peers' heartbeats before launching anything, so a rank that died or raised between
    steps surfaces as an exception here instead of as a collective that never completes."""

    def __init__(self, store, rank, world, timeout_s=5.0, prefix="fp8gmm/alive"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def check(self, step):
        import datetime

        self.store.set(f"{self.prefix}/{step}/{self.rank}", "1")
        keys = [f"{self.prefix}/{step}/{r}" for r in range(self.world) if r != self.rank]
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as exc:  # the store raises a backend-specific timeout error
            raise RuntimeError(f"rank {self.rank}: a peer did not reach step {step} within {self.timeout_s} s") from exc
