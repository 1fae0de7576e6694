"""Expert parallelism over peer memory: the dispatch / combine exchange pipelined with the grouped MLP.

Where fp8_gmm_b200.ep moves rows with NCCL all-to-all around an unchanged GroupedMlp (exchange, then compute,
then exchange), this module splits a rank's experts into chunks and overlaps the exchange of one chunk with the
GEMMs of another:

    copy engines, dispatch channel :  D0 D1 D2 D3
    copy engines, combine channel  :           C0                C1                C2       C3
    SMs                            :  w-cast [cast fc1 fc2]0   [cast fc1 fc2]1   [...]2   [...]3

``Dk`` pushes the rows of chunk k's experts from every rank straight into their place in the owner's
expert-major receive buffer (one device-to-device copy per (destination expert) block, so no permutation kernel
runs on either side); ``Ck`` pushes chunk k's results back to the rows' home ranks, into the tensor the caller
gets.  Backward runs the same schedule with the gradient.  The copies run on the copy engines (fp8_gmm_b200.peer),
so the persistent GEMM kernels keep every SM.  The reference has no counterpart (single GPU; its example permutes
on one device, reference fp8_gmm/example.py:52-59,85-92); numerics per expert are exactly GroupedMlp's.

The plan arithmetic (PeerPlan) is pure host code and is tested on CPU by simulating the copies.
"""
import copy
import os
import weakref

import numpy as np
import torch
import torch.distributed as dist

from . import backend
from .grouped_linear import cast_weight_cached
from ._lib import check, lib
from .peer import PeerBuffer, PeerChannel
from .recipe import get_fp8_te_dtype
from .utils import Fp8MetaWrapper, Fp8TensorType, MetaTensorType, cumsum_group_sizes, to_torch_dtype

_T, _M = Fp8TensorType, MetaTensorType


_TAPER = (1, 2, 4, 4, 3, 2)  # sixteenths of the local experts per chunk: small first and last rounds, which nothing hides


def chunk_bounds(experts_local, spec):
    """[(first expert, end expert)] of the pipeline's chunks.  ``spec``: an int (that many even chunks), "tapered"
    (chunks of 1/16, 1/8, 1/4, 1/4, 3/16, 1/8 of the experts: the first dispatch and the last combine round, which
    no computation overlaps, stay short), or an explicit sequence of expert counts summing to ``experts_local``."""
    El = experts_local
    if isinstance(spec, str):
        assert spec == "tapered", spec
        sizes = [max(1, round(El * f / 16)) for f in _TAPER] if El >= 6 else [1] * El
        while sum(sizes) > El:
            sizes[sizes.index(max(sizes))] -= 1
        while sum(sizes) < El:
            sizes[sizes.index(max(sizes))] += 1
    elif isinstance(spec, int):
        C = max(1, min(spec, El))
        bounds = [round(i * El / C) for i in range(C + 1)]
        sizes = [bounds[i + 1] - bounds[i] for i in range(C)]
    else:
        sizes = [int(v) for v in spec]
        assert sum(sizes) == El and min(sizes) >= 0, "chunk sizes must sum to the number of local experts"
    out, start = [], 0
    for n in sizes:
        if n > 0:
            out.append((start, start + n))
        start += n
    return out


class PeerPlan:
    """Row bookkeeping of one exchange, derived from everybody's group sizes.

    counts: CPU int64 (P, E), counts[s, e] = rows of global expert e held by rank s (sorted by expert there).
    Rank o owns experts [o*El, (o+1)*El).  At the owner rows are expert-major and, inside an expert, ordered by
    source rank.  Offsets are in rows."""

    def __init__(self, counts, rank, num_chunks):
        counts = counts.to(torch.int64)
        self.world, self.num_experts = counts.shape
        self.rank = rank
        P, E = self.world, self.num_experts
        assert E % P == 0
        El = self.experts_local = E // P
        self.counts = counts
        zero = torch.zeros(P, 1, dtype=torch.int64)
        self.send_off = torch.cat([zero, torch.cumsum(counts, 1)], 1)                    # (P, E+1)
        by_owner = counts.reshape(P, P, El).permute(1, 2, 0).contiguous()               # (owner, j, src)
        rows_local = by_owner.sum(2)                                                     # (owner, j)
        self.exp_off = torch.cat([zero, torch.cumsum(rows_local, 1)], 1)                # (owner, El+1)
        within = torch.cumsum(by_owner, 2) - by_owner                                   # exclusive over src
        self.blk_off = self.exp_off[:, :El, None] + within                              # (owner, j, src)
        self.by_owner = by_owner
        self._counts_l, self._send_off_l, self._blk_off_l = counts.tolist(), self.send_off.tolist(), self.blk_off.tolist()
        self.local_sizes = rows_local[rank].tolist()
        self.rows_local_max = int(rows_local.sum(1).max())
        self.rows_own = int(counts[rank].sum())
        self.rows_own_max = int(counts.sum(1).max())
        self.chunks = chunk_bounds(El, num_chunks)
        self._lists = {}

    def _peer_order(self):
        # staggered so that at any moment every receiver is written by a different sender
        return [(self.rank + i) % self.world for i in range(1, self.world + 1)]

    def dispatch_blocks(self, chunk):
        """(owner, dst_row at the owner, src_row here, rows) for the rows this rank sends for one chunk of experts."""
        key = ("d", chunk)
        if key not in self._lists:
            j0, j1 = chunk
            El, r = self.experts_local, self.rank
            out = []
            cnt, send, blk = self._counts_l[r], self._send_off_l[r], self._blk_off_l
            for o in self._peer_order():
                for j in range(j0, j1):
                    n = cnt[o * El + j]
                    if n:
                        out.append((o, blk[o][j][r], send[o * El + j], n))
            self._lists[key] = out
        return self._lists[key]

    def dispatch_arrays(self, chunk):
        key = ("da", chunk)
        if key not in self._lists:
            self._lists[key] = _block_arrays(self.dispatch_blocks(chunk))
        return self._lists[key]

    def combine_arrays(self, chunk):
        key = ("ca", chunk)
        if key not in self._lists:
            self._lists[key] = _block_arrays(self.combine_blocks(chunk))
        return self._lists[key]

    def staged_combine(self):
        """Layout that lets one copy per (home rank, chunk) return the results.  At the owner rows are expert-major
        (inside an expert ordered by source rank); a home rank wants the rows of a chunk's experts back to back (it
        holds them sorted by global expert).  So the GEMM epilogue that produces a chunk's result rows writes them
        *source-major inside the chunk* -- all rows of source 0 for the chunk's experts, then source 1, ... -- through
        its row map, and the rows of one (home rank, chunk) form one contiguous run on both sides.

        Returns (row_map, copies): ``row_map`` int32 numpy (rows_local,), expert-major row -> staged row, relative to
        the first row of the row's chunk; ``copies[chunk]`` = four int64 arrays (home rank, dst_row at home, staged
        src_row here, rows), peers in the staggered order."""
        key = "stage"
        if key not in self._lists:
            El, r = self.experts_local, self.rank
            by = self.by_owner[r].numpy()            # (El, P): rows of local expert j that came from source s
            exp_off = self.exp_off[r].numpy()        # (El + 1,)
            blk_off = self.blk_off[r].numpy()        # (El, P): expert-major start of block (j, s)
            send_off = self.send_off.numpy()         # (P, E + 1)
            row_map = np.empty(int(exp_off[-1]), dtype=np.int32)
            copies = {}
            order = np.asarray(self._peer_order(), dtype=np.int64)
            for (j0, j1) in self.chunks:
                r0, r1 = int(exp_off[j0]), int(exp_off[j1])
                cnt = by[j0:j1]
                per_src = cnt.sum(0)
                src_base = np.cumsum(per_src) - per_src
                staged = src_base[None, :] + (np.cumsum(cnt, 0) - cnt)      # staged start of block (j, s), chunk-relative
                delta = (staged - (blk_off[j0:j1] - r0)).reshape(-1)
                row_map[r0:r1] = np.arange(r1 - r0, dtype=np.int64) + np.repeat(delta, cnt.reshape(-1))
                copies[(j0, j1)] = (order, send_off[order, r * El + j0], r0 + src_base[order], per_src[order])
            self._lists[key] = (row_map, copies)
        return self._lists[key]

    def staged_dispatch(self, rounds=None):
        """The same source-major layout for the way in.  A rank's rows for one owner and a run of that owner's experts
        are one contiguous run at the source (rows are sorted by global expert), so with a source-major staging buffer
        at the owner one copy per (owner, round) delivers them, and the owner brings them expert-major with a local
        block permutation (fp8gmm_block_permute_rows), chunk by chunk.  ``rounds``: [(first expert, end expert)] of
        the dispatch rounds, each covering whole chunks (default: one round per chunk); fewer rounds mean fewer and
        larger copies.

        Returns (copies, perms): ``copies[round]`` = four int64 arrays (owner, dst_row in the owner's staging buffer,
        src_row here, rows), owners in the staggered order; ``perms[chunk]`` = three int64 arrays (staged start,
        expert-major start, rows) of this rank's blocks (local expert, source) of the chunk."""
        rounds = tuple(self.chunks) if rounds is None else tuple(tuple(g) for g in rounds)
        key = ("stage_in", rounds)
        if key not in self._lists:
            El, r, P = self.experts_local, self.rank, self.world
            by_all = self.by_owner.numpy()           # (owner, El, src)
            exp_off = self.exp_off.numpy()           # (owner, El + 1)
            blk_off = self.blk_off[r].numpy()        # (El, P)
            send_off = self.send_off[r].numpy()      # (E + 1,)
            order = np.asarray(self._peer_order(), dtype=np.int64)
            copies, perms = {}, {}
            for (g0, g1) in rounds:
                cnt_all = by_all[:, g0:g1, :]                                  # (owner, jc, src)
                per_src = cnt_all.sum(1)                                       # (owner, src)
                src_base = np.cumsum(per_src, 1) - per_src                     # rows of earlier sources in the round
                dst_row = exp_off[order, g0] + src_base[order, r]
                copies[(g0, g1)] = (order, dst_row, send_off[order * El + g0], per_src[order, r])
                cnt = cnt_all[r]                                               # (jc, src) at this owner
                staged = int(exp_off[r, g0]) + src_base[r][None, :] + (np.cumsum(cnt, 0) - cnt)
                inside = [c for c in self.chunks if g0 <= c[0] and c[1] <= g1]
                assert sum(c[1] - c[0] for c in inside) == g1 - g0, "a dispatch round covers whole chunks"
                for (j0, j1) in inside:
                    perms[(j0, j1)] = (np.ascontiguousarray(staged[j0 - g0:j1 - g0].reshape(-1)),
                                       np.ascontiguousarray(blk_off[j0:j1].reshape(-1)),
                                       np.ascontiguousarray(cnt[j0 - g0:j1 - g0].reshape(-1)))
            self._lists[key] = (copies, perms)
        return self._lists[key]

    def direct_row_map(self):
        """Row map for results that the GEMM epilogue stores straight into the home ranks' buffers: int32 numpy
        (rows_local,), expert-major row here -> backend.peer_row_entry(home rank, row in the home rank's result tensor).
        A home rank holds its rows sorted by global expert, so block (local expert j, source s) of this owner lands at
        row send_off[s, first expert of this owner + j] there."""
        key = "direct"
        if key not in self._lists:
            El, r, P = self.experts_local, self.rank, self.world
            assert P <= 32 and self.rows_own_max < (1 << backend.ROW_MAP_PEER_SHIFT), "row-map entries hold 5 + 26 bits"
            cnt = self.by_owner[r].numpy().reshape(-1)                          # blocks in expert-major order: (j, s)
            start = self.blk_off[r].numpy().reshape(-1)
            home_row = self.send_off.numpy()[:, r * El:(r + 1) * El].T.reshape(-1)    # (j, s) -> first row at home rank s
            src = np.tile(np.arange(P, dtype=np.int64), El)
            total = int(self.exp_off[r, -1])
            entries = np.repeat(backend.peer_row_entry(src, home_row) - start, cnt) + np.arange(total, dtype=np.int64)
            self._lists[key] = entries.astype(np.int32)
        return self._lists[key]

    def combine_map(self, direct_homes):
        """How this owner's result rows go home when the rows of the home ranks in ``direct_homes`` are stored by the
        GEMM epilogue straight into those ranks' tensors and the others are staged source-major here and pushed by the
        copy engines.  Returns (entries, copies): ``entries`` int32 numpy (rows_local,) for the epilogue -- a direct
        row names (home rank, row there), a staged row names buffer index ``world`` (the local staging buffer, last in
        the epilogue's table) and its staged row; ``copies[chunk]`` as in staged_combine, without the direct homes."""
        key = ("mix", tuple(sorted(direct_homes)))
        if key not in self._lists:
            rel, copies = self.staged_combine()
            direct = self.direct_row_map().astype(np.int64)
            exp_off = self.exp_off[self.rank].numpy()
            chunk_start = np.zeros(rel.shape[0], dtype=np.int64)
            for (j0, j1) in self.chunks:
                chunk_start[int(exp_off[j0]):int(exp_off[j1])] = int(exp_off[j0])
            homes = np.asarray(sorted(direct_homes), dtype=np.int64)
            is_direct = np.isin(direct >> backend.ROW_MAP_PEER_SHIFT, homes)
            entries = np.where(is_direct, direct, backend.peer_row_entry(self.world, chunk_start + rel)).astype(np.int32)
            kept = {}
            for chunk, arrays in copies.items():
                mask = ~np.isin(arrays[0], homes)
                kept[chunk] = tuple(np.ascontiguousarray(a[mask]) for a in arrays)
            self._lists[key] = (entries, kept)
        return self._lists[key]

    def combine_map_dev(self, device, direct_homes):
        key = ("mix_dev", device.index, tuple(sorted(direct_homes)))
        if key not in self._lists:
            self._lists[key] = torch.from_numpy(self.combine_map(direct_homes)[0]).to(device)
        return self._lists[key]

    def staged_row_map(self, device):
        """The staged row map on the device (uploaded once per plan)."""
        key = ("stage_dev", device.index)
        if key not in self._lists:
            self._lists[key] = torch.from_numpy(self.staged_combine()[0]).to(device)
        return self._lists[key]

    def combine_blocks(self, chunk):
        """(home rank, dst_row at home, src_row here, rows) for the result rows this rank returns for one chunk."""
        key = ("c", chunk)
        if key not in self._lists:
            j0, j1 = chunk
            El, r = self.experts_local, self.rank
            out = []
            cnt, send, blk = self._counts_l, self._send_off_l, self._blk_off_l[r]
            for s in self._peer_order():
                for j in range(j0, j1):
                    n = cnt[s][r * El + j]
                    if n:
                        out.append((s, send[s][r * El + j], blk[j][s], n))
            self._lists[key] = out
        return self._lists[key]


def _block_arrays(blocks):
    """(peer, dst_row, src_row, rows) tuples -> four int64 numpy arrays."""
    a = np.asarray(blocks, dtype=np.int64).reshape(-1, 4)
    return a[:, 0].copy(), a[:, 1].copy(), a[:, 2].copy(), a[:, 3].copy()


def _copy_blocks(peer_ptrs, arrays, src_ptr, row_bytes, extra=None):
    """Copy-block array for one round: rows `src_row..` at `src_ptr` go to row `dst_row` of peer `peer`'s buffer."""
    peer, dst_row, src_row, rows = arrays
    n = len(peer) + (0 if extra is None else len(extra))
    out = np.empty(n, dtype=PeerChannel._BLOCK)
    m = len(peer)
    out["dst"][:m] = peer_ptrs[peer] + (dst_row * row_bytes).astype(np.uint64)
    out["src"][:m] = np.uint64(src_ptr) + (src_row * row_bytes).astype(np.uint64)
    out["bytes"][:m] = (rows * row_bytes).astype(np.uint64)
    if extra is not None:
        out[m:] = extra
    return out


class _Pool:
    """Receive buffers for combined results.  A buffer is handed to the caller as a tensor and comes back when that
    tensor dies.  Buffers are allocated collectively, so index i names the same allocation round on every rank."""

    def __init__(self, device, group):
        self.device, self.group = device, group
        self.buffers, self.free = [], []

    def pick(self, nbytes):
        for i in self.free:
            if self.buffers[i].nbytes >= nbytes:
                self.free.remove(i)
                return i
        return -1

    def grow(self, nbytes):
        self.buffers.append(PeerBuffer(nbytes, self.device, self.group))
        return len(self.buffers) - 1

    def release(self, i):
        self.free.append(i)


def resolve_result_buffers(picks, buffers_before):
    """picks: per rank [out_id, grad_id] as each rank chose from its own free list (-1 = none free, -2 = not wanted).
    Every rank allocates ``missing`` new buffers (as many as the neediest rank lacks), numbered from
    ``buffers_before`` on every rank alike, and a rank that lacked buffers takes the new ones in order.  Returns
    (missing, per-rank [out_id, grad_id] with the -1 entries resolved).  Pure function of what the all-gather
    delivered, so all ranks reach the same answer."""
    missing = max((sum(1 for i in pair if i == -1) for pair in picks), default=0)
    resolved = []
    for pair in picks:
        fresh = iter(range(buffers_before, buffers_before + missing))
        resolved.append([next(fresh) if i == -1 else i for i in pair])
    return missing, resolved


def dispatch_rounds_for(spec, chunks):
    """Expert ranges [(first, end)] of the forward dispatch rounds for FP8GMM_EP_DISPATCH_ROUNDS = ``spec``: "chunks" or
    "auto" (one round per chunk) or a comma-separated list of chunk counts per round ("2,4": the first two chunks travel
    together, then the next four; the last round takes what is left)."""
    chunks = list(chunks)
    if spec in ("chunks", "auto") or len(chunks) <= 2:
        return chunks
    counts = [int(v) for v in spec.split(",")]
    out, i = [], 0
    for n in counts:
        if i >= len(chunks) or n <= 0:
            continue
        part = chunks[i:i + n]
        out.append((part[0][0], part[-1][1]))
        i += n
    if i < len(chunks):
        out.append((chunks[i][0], chunks[-1][1]))
    return out


def direct_homes_for(spec, rank, world):
    """Home ranks served by the GEMM epilogue's peer stores for FP8GMM_EP_DIRECT = ``spec``: "all", "none", "auto" (all
    in a group of two, none in larger groups) or a number k (this rank and the k ranks after it)."""
    if spec == "auto":
        spec = "all" if world <= 2 else "none"
    if spec == "none":
        return ()
    k = world - 1 if spec == "all" else min(int(spec), world - 1)
    return tuple(sorted((rank + i) % world for i in range(k + 1)))


class EpContext:
    """Per (device, group) transport state shared by all ExpertParallelMlp modules: the channel (side stream and
    sequence numbers), the receive buffer for dispatched rows and the pool of result buffers.

    Creating it is collective: every rank of ``group`` exchanges IPC handles, and with ``group=None`` and no
    ``host_group`` a gloo group over ALL ranks of the job is created.  Call ``EpContext.setup`` on every rank at a
    point all of them reach (the first forward does it implicitly, which is only safe when every rank of the group
    -- of the whole job for ``group=None`` -- runs that forward).  In a job where only some ranks hold an
    ExpertParallelMlp, pass the expert-parallel ``group`` and a gloo ``host_group`` over the same ranks.
    ``close()`` (collective as well) unmaps and frees the buffers."""

    _instances = {}

    @classmethod
    def setup(cls, device, group=None, host_group=None):
        key = (device.index, id(group))
        if key not in cls._instances:
            cls._instances[key] = cls(device, group, host_group)
        return cls._instances[key]

    get = setup

    def close(self):
        """Frees this context's peer buffers.  Collective: every rank calls it, with no exchange in flight."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for buf in [self.recv, self.recv_stage, self._amax_stage] + self.pool.buffers:
            if buf is not None:
                buf.close()
        for ch in (self.channel, self.channel_back, self.ready):
            ch.close()
        self.recv = self._amax_stage = self._amax_view = None
        self.pool.buffers, self.pool.free = [], []
        self._ptr_tables, self._stage_out = {}, None
        self._instances.pop((self.device.index, id(self.group)), None)

    def __init__(self, device, group, host_group=None):
        self.device, self.group = device, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        # Bounded waits that ran out (a peer more than fp8gmm_set_wait_limits late) are noticed one step later,
        # without a synchronisation: the step ends with an asynchronous copy of the device status word, the next
        # step begins by looking at it and refuses to go on with rows that never arrived.
        self.status = backend.StatusWatch()
        self.failed = False
        self._last_plan = None
        # two channels = two side streams: dispatch and combine copies run on different copy engines at the same time
        # (four copy lanes each: blocks of 8-16 MiB moved 8-9 % faster than over one lane in a 4-GPU all-to-all pattern)
        self.channel = PeerChannel(device, group, copy_streams=4)          # dispatch rounds
        self.channel_back = PeerChannel(device, group, copy_streams=4)     # combine rounds
        # Dispatch rounds issued ahead of the chunk being computed (default: all of them at once -- the rows are ready).
        # Measured at 8 GPUs: with every round queued up front the first combine round sits behind them on the copy
        # engines (3.3 ms for 117 MB), but a look-ahead of 1 or 2 rounds is no faster overall (20.3 / 21.0 ms per step
        # against 19.9): dispatch and combine share the rank's NVLink egress, which the copy engines fill to
        # 350-450 GB/s in this all-to-all pattern whatever the order.
        self.dispatch_ahead = int(os.environ.get("FP8GMM_EP_DISPATCH_AHEAD", "1000"))
        # "My buffers are free" announcements (signals only, no copies) and a host-side group for the size exchange:
        # together they replace a device all-gather + host synchronisation per step, so the host may run a step ahead
        # of the GPU and a late host on one rank does not stall the others' GPUs.  A sub-group keeps the device gather
        # (creating a gloo group is collective over all ranks of the job).
        self.ready = PeerChannel(device, group)
        self.host_group = host_group if host_group is not None else (dist.new_group(backend="gloo") if group is None else None)
        self.pool = _Pool(device, group)
        self.recv = None
        self.recv_stage = None   # forward FP8 dispatch: source-major staging (one copy per sender and chunk lands here)
        # FP8GMM_EP_DISPATCH=blocks keeps one copy per (owner, expert) straight into expert-major place in forward too
        self.merged_dispatch = os.environ.get("FP8GMM_EP_DISPATCH", "merged") != "blocks"
        # Rounds of the merged forward dispatch (dispatch_rounds_for): the copy engines pay a fixed 15-20 us per copy
        # and work through a rank's copies one after the other (8 MiB copies reach 290 GB/s, 32 MiB 540, 128 MiB 700),
        # so the rows of several chunks may travel as one copy per owner.  One round per chunk stays the default: at
        # 4 GPUs "2,1,3" cut the ranks' waits from 1.8-3.6 to 2.2-2.6 ms per step but the step (19.4 ms) stayed inside
        # the run-to-run spread, and a chunk that waits for a large round leaves the SMs idle.
        self.dispatch_rounds_spec = os.environ.get("FP8GMM_EP_DISPATCH_ROUNDS", "auto")
        self._amax_stage = None
        self._amax_view = None
        # How results go home.  The fc2 (forward) and fc1 data-gradient (backward) epilogues can store a row straight
        # into its home rank's result tensor through the peer mapping (no copy, the exchange is part of the GEMM), or
        # write it into a local source-major staging buffer from which the copy engines take one block per (home
        # rank, chunk) home.  Peer stores stall the epilogue once the link is the bottleneck, staged rows cost the
        # copy engines' time: FP8GMM_EP_DIRECT picks the home ranks served by peer stores -- "all", "none", a number
        # k (this rank and the k ranks after it) or "auto": all in a group of two, where the rows of one GEMM cross the
        # link faster than the GEMM computes them (17.1 against 18.4 ms per step); none in larger groups, where 3/4 and
        # more of the rows leave (4 GPUs, one box: all 21.1 ms per step against 19.0 staged; own rows only 18.5-19.8,
        # own + next rank 18.5, none 18.8-18.9: no gain outside the run-to-run spread; 8 GPUs: none 19.9, own + next rank
        # 20.9, own + next two 20.6 -- the waits shrink but the epilogues stall on the link for longer than that).
        self.direct_spec = os.environ.get("FP8GMM_EP_DIRECT", "auto")
        self._ptr_tables = {}
        self._stage_out = None

    def direct_homes(self):
        """Home ranks whose rows the GEMM epilogues store directly (see __init__)."""
        return direct_homes_for(self.direct_spec, self.rank, self.world)

    def stage_out(self, nbytes):
        """Local staging buffer for result rows that travel by copy (kept across steps: its address is part of the
        epilogue's buffer table; a step's copies out of it are complete before the step's last wait returns)."""
        if self._stage_out is None or self._stage_out.numel() < nbytes:
            self._stage_out = torch.empty(int(nbytes * 1.25) + 256, dtype=torch.uint8, device=self.device)
            self._ptr_tables = {}
        return self._stage_out

    def result_ptr_table(self, buf_ids):
        """Device int64 vector for the epilogue: address, in this rank's address space, of rank r's result buffer
        buf_ids[r], and the local staging buffer as entry ``world``."""
        key = tuple(buf_ids)
        if key not in self._ptr_tables:
            ptrs = [self.pool.buffers[b].ptrs[r] for r, b in enumerate(buf_ids)] + [self._stage_out.data_ptr()]
            self._ptr_tables[key] = torch.tensor(ptrs, dtype=torch.int64).to(self.device)
        return self._ptr_tables[key]

    def wait_buffers_free(self, plan):
        """The compute stream waits until every rank has announced that its buffers of the step before are free (the
        announcement plan() sent): needed before a kernel of this stream stores into other ranks' result tensors."""
        check(lib.fp8gmm_peer_wait(self.ready.flags.local, self.world, plan.free_seq,
                                   torch.cuda.current_stream(self.device).cuda_stream), "peer_wait")

    def amax_stage(self, experts_local):
        """(world x experts_local) fp32 in every rank's memory: row s = rank s's partial amaxes of my experts."""
        need = self.world * experts_local * 4
        if self._amax_stage is None or self._amax_stage.nbytes < need:
            self._amax_stage = PeerBuffer(max(need, 4096), self.device, self.group)
            self._amax_view = None
        return self._amax_stage

    def amax_stage_tensor(self, experts_local):
        """The local staging rows as a (world, experts_local) fp32 tensor (built once: a view over foreign memory)."""
        stage = self.amax_stage(experts_local)
        if self._amax_view is None or self._amax_view.shape[1] != experts_local:
            self._amax_view = stage.tensor((self.world, experts_local), torch.float32)
        return self._amax_view

    def plan(self, group_sizes, row_bytes, num_chunks, want_grad_buffer):
        """One small all-gather (host side): everybody's group sizes plus the result buffers each rank picked."""
        E = group_sizes.numel()
        own_bytes = int(group_sizes.sum()) * row_bytes
        pool = self.pool
        out_id = pool.pick(own_bytes)
        gi_id = pool.pick(own_bytes) if want_grad_buffer else -2
        meta = torch.cat([group_sizes.to(torch.int64), torch.tensor([out_id, gi_id], dtype=torch.int64)])
        if self.host_group is not None:
            parts = [torch.empty_like(meta) for _ in range(self.world)]
            dist.all_gather(parts, meta, group=self.host_group)      # host to host: the GPU is not waited for
            gathered = torch.stack(parts)
        else:
            mine = meta.to(self.device, non_blocking=True)
            gathered = torch.empty(self.world, E + 2, dtype=torch.int64, device=self.device)
            dist.all_gather_into_tensor(gathered, mine, group=self.group)
            gathered = gathered.cpu()
        # Device-side ordering of this step's pushes after every rank's previous use of the buffers they land in:
        # each rank announces, after all the work its compute stream holds so far, that its buffers are free; both
        # copy streams wait for everybody's announcement before their next copy.
        free_seq = self.ready.push_arrays(np.empty(0, dtype=PeerChannel._BLOCK))
        for ch in (self.channel, self.channel_back):
            check(lib.fp8gmm_peer_wait(self.ready.flags.local, self.world, free_seq, ch.stream.cuda_stream), "peer_wait")
        counts = gathered[:, :E].contiguous()
        last = self._last_plan
        if last is not None and last[1] == repr(num_chunks) and torch.equal(last[0].counts, counts):
            plan = copy.copy(last[0])   # same routing as the step before: offsets and copy lists are shared, buffer ids are not
        else:
            plan = PeerPlan(counts, self.rank, num_chunks)
            self._last_plan = (plan, repr(num_chunks))
        # collective growth: everybody allocates as many new result buffers as the neediest rank asked for
        picks = gathered[:, E:].tolist()
        n_before = len(pool.buffers)
        missing, resolved = resolve_result_buffers(picks, n_before)
        new_ids = [pool.grow(int(plan.rows_own_max * 1.25) * row_bytes + 256) for _ in range(missing)]
        mine = resolved[self.rank]
        for i in new_ids:
            if i not in mine:
                pool.release(i)
        plan.out_ids, plan.gi_ids = [r[0] for r in resolved], [r[1] for r in resolved]
        plan.free_seq = free_seq
        need = plan.rows_local_max * row_bytes
        if self.recv is None or self.recv.nbytes < need:
            # every rank sees the same sizes, so all of them take this branch together
            if self.recv is not None:
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
                self.recv.close()
            self.recv = PeerBuffer(int(plan.rows_local_max * 1.25) * row_bytes + 256, self.device, self.group)
            if self.recv_stage is not None:
                self.recv_stage.close()
            # FP8 rows: half the bytes of the bf16-sized receive buffer
            self.recv_stage = PeerBuffer(int(plan.rows_local_max * 1.25) * (row_bytes // 2) + 256, self.device, self.group)
        return plan

    def result_tensor(self, buf_id, rows, cols):
        buf = self.pool.buffers[buf_id]
        pool = weakref.ref(self.pool)

        def back():
            p = pool()
            if p is not None:
                p.release(buf_id)

        return buf.tensor((rows, cols), torch.bfloat16, on_release=back)


def _strided_rows(spec, count):
    """The ``count`` slots of a (tensor, stride) meta view as a strided 1-D tensor view."""
    t, stride = spec
    return t[: (count - 1) * stride + 1: stride] if count > 0 else t[:0]


def _gather_scales(spec, experts_local, group):
    """Every owner's per-expert scales -> one device vector indexed by global expert (no host involvement)."""
    local = _strided_rows(spec, experts_local).contiguous()
    out = torch.empty(dist.get_world_size(group) * experts_local, dtype=torch.float32, device=local.device)
    dist.all_gather_into_tensor(out, local, group=group)
    return out


def _quantize_at_source(ectx, plan, rows_bf16, scales_all, fp8_dtype):
    """FP8 dispatch, source side: this rank's rows (sorted by global expert) are cast with the *owner's* scale of each
    expert, so the bytes that travel are exactly the bytes the owner would have produced, and half as many.  Returns
    (fp8 rows, per-global-expert amax of the rows held here)."""
    E = plan.num_experts
    q = torch.empty(rows_bf16.shape, dtype=fp8_dtype, device=rows_bf16.device)
    amax_part = torch.zeros(E, dtype=torch.float32, device=rows_bf16.device)
    backend.grouped_cast_transpose(rows_bf16, plan._send_off_l[plan.rank], q, None, None, (scales_all, 1), (amax_part, 1))
    return q, amax_part


def _amax_blocks(ectx, plan, amax_part, chunk):
    """Copies that hand this rank's partial amaxes of one chunk of experts to their owners' staging rows."""
    j0, j1 = chunk
    El, r = plan.experts_local, plan.rank
    stage = ectx.amax_stage(El)
    out = np.empty(plan.world, dtype=PeerChannel._BLOCK)
    owners = np.arange(plan.world, dtype=np.uint64)
    out["dst"] = np.asarray(stage.ptrs, dtype=np.uint64) + np.uint64((r * El + j0) * 4)
    out["src"] = np.uint64(amax_part.data_ptr()) + (owners * np.uint64(El) + np.uint64(j0)) * np.uint64(4)
    out["bytes"] = np.uint64((j1 - j0) * 4)
    return out


def _merge_amax(ectx, plan, spec, chunk):
    """Owner side: max-merge the sources' partial amaxes of a chunk into the recipe's amax slots."""
    j0, j1 = chunk
    El = plan.experts_local
    stage = ectx.amax_stage_tensor(El)
    view = _strided_rows(spec, j1 - j0)
    torch.maximum(view, stage[:, j0:j1].amax(dim=0), out=view)


def _rel(offsets, j0, j1):
    base = offsets[j0]
    return [o - base for o in offsets[j0:j1 + 1]]


class _PeerEpMlp(torch.autograd.Function):
    """fc1 -> activation -> fc2 over this rank's experts with the row exchange pipelined chunk by chunk."""

    @staticmethod
    def forward(ctx, x, fc1_weight, fc2_weight, st):
        mlp, plan, ectx = st["mlp"], st["plan"], st["ctx"]
        ch, ch_back = ectx.channel, ectx.channel_back
        fp8_meta, activation = mlp.fp8_meta, mlp.activation
        grad_on = st["grad_enabled"]
        need_wgrad = grad_on and fc1_weight.requires_grad
        need_dgrad = grad_on and x.requires_grad
        El = plan.experts_local
        need_t = need_wgrad and not backend.WGRAD_ROWMAJOR   # padded transposes only for the reference's wgrad dataflow
        _, padded, cumsums, padded_cumsums = cumsum_group_sizes(plan.local_sizes, need_padding=need_t)
        offs = padded_cumsums if padded else cumsums
        rows = cumsums[-1]
        metas = Fp8MetaWrapper(El, fp8_meta)
        fdt = to_torch_dtype(get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=True))
        x = x.contiguous()
        hidden = x.shape[1]
        row_bytes = hidden * 2
        fc1_out = fc1_weight.shape[1]
        ffn = fc1_out // 2 if activation == "swiglu" else fc1_out
        dev = x.device
        sizes_cpu = torch.tensor(plan.local_sizes, dtype=torch.int64)

        recv_ptrs = ectx.recv.ptrs
        fp8d = st["fp8_dispatch"]
        ms = metas.get_meta_strided
        if fp8d:
            src, amax_part = _quantize_at_source(ectx, plan, x, st["x_scales"], fdt)
            ectx.amax_stage(El)            # collective on first use: before any push refers to it
            d_bytes = hidden               # bytes per dispatched row
        else:
            src, amax_part, d_bytes = x, None, row_bytes
        x_ptr = src.data_ptr()
        recv_np = np.asarray(recv_ptrs, dtype=np.uint64)

        # FP8 forward dispatch: one copy per (owner, chunk) into the owner's source-major staging buffer; the owner's
        # block permutation (which is also the copy that keeps the rows for the fc1 weight gradient) puts them
        # expert-major.  16-64 MiB copies instead of one 8 MiB copy per (owner, expert).
        merged = fp8d and ectx.merged_dispatch
        chunks = plan.chunks
        # dispatch rounds: one per chunk, or -- merged -- fewer rounds that each carry the rows of several chunks
        rounds = dispatch_rounds_for(ectx.dispatch_rounds_spec, chunks) if merged else chunks
        round_of = [next(i for i, (g0, g1) in enumerate(rounds) if g0 <= j0 and j1 <= g1) for (j0, j1) in chunks]
        if merged:
            stage_np = np.asarray(ectx.recv_stage.ptrs, dtype=np.uint64)
            in_copies, in_perms = plan.staged_dispatch(rounds)

        def dispatch(experts, first):
            extra = _amax_blocks(ectx, plan, amax_part, experts) if fp8d else None
            blocks = (_copy_blocks(stage_np, in_copies[experts], x_ptr, d_bytes, extra) if merged else
                      _copy_blocks(recv_np, plan.dispatch_arrays(experts), x_ptr, d_bytes, extra))
            # later rounds do not wait for the compute stream: the rows they carry were ready before the first round
            return ch.push_arrays(blocks, after_compute=first)

        # The first rounds are queued now (the rows are ready), the rest as the chunks before them are reached, so
        # that the copy engines see dispatch and combine rounds interleaved (EpContext.dispatch_ahead).
        ahead = max(1, ectx.dispatch_ahead)
        seq = []

        def push_until(n):
            while len(seq) < min(n, len(rounds)):
                seq.append(dispatch(rounds[len(seq)], not seq))

        push_until(ahead)
        waited = -1
        # the fc2 weight cast runs while the first rows are on their way
        cache, reuse = st["weight_cache"], st["reuse_weights"]
        fc1_w_fp8, fc1_w_t = st["fc1_fp8"]   # cast before the size exchange, so the GPU had work during the host sync
        kn = backend.DGRAD_KN   # dgrad multiplies by the forward FP8 weights as they are: no weight transposes
        fc2_w_fp8, fc2_w_t = cast_weight_cached(fc2_weight, fdt, (need_dgrad or need_wgrad) and not kn, ms(_T.kWeightGroup2, _M.kScale),
                                                ms(_T.kWeightGroup2, _M.kAmax), cache, "fc2", reuse)
        keep_rows = need_wgrad and not need_t     # the row-major FP8 input is the fc1 wgrad operand: it must outlive forward
        if merged:
            recv = None
            staged_in = ectx.recv_stage.tensor((rows, hidden), fdt)
            input_fp8 = torch.empty(rows, hidden, dtype=fdt, device=dev)     # expert-major, filled chunk by chunk
            input_keep = input_fp8 if keep_rows else None
        elif fp8d:
            # the received bytes are the GEMM operand as they lie in the receive buffer
            recv = None
            input_fp8 = ectx.recv.tensor((rows, hidden), fdt)
            input_keep = torch.empty(rows, hidden, dtype=fdt, device=dev) if keep_rows else None
        else:
            recv = ectx.recv.tensor((rows, hidden), torch.bfloat16)
            input_fp8 = torch.empty(rows, hidden, dtype=fdt, device=dev)
            input_keep = input_fp8 if keep_rows else None
        input_t_fp8 = torch.empty(offs[-1], hidden, dtype=fdt, device=dev) if need_t else None
        pre_act = torch.empty(rows, fc1_out, dtype=torch.bfloat16, device=dev)
        act_fp8 = torch.empty(rows, ffn, dtype=fdt, device=dev)
        out = ectx.result_tensor(plan.out_ids[plan.rank], plan.rows_own, hidden)
        # Results go home from the fc2 epilogue: rows of the home ranks in `homes` by stores into those ranks' `out`
        # tensors, the others source-major into the staging buffer, from which one copy per (home rank, chunk) takes them
        # (blocks of tens of MiB instead of one block per expert: the copy engines run faster on them).
        homes = ectx.direct_homes()
        out_np = np.asarray([ectx.pool.buffers[plan.out_ids[r]].ptrs[r] for r in range(plan.world)], dtype=np.uint64)
        stage_ptr = ectx.stage_out(rows * row_bytes).data_ptr()
        if homes:
            home_map, stage_copies = plan.combine_map_dev(dev, homes), plan.combine_map(homes)[1]
            home_ptrs = ectx.result_ptr_table(plan.out_ids)
            freed = all(h == plan.rank for h in homes)      # this rank's own tensor needs no announcement from anybody
        else:
            out_local = ectx.stage_out(rows * row_bytes)[:rows * row_bytes].view(torch.bfloat16).view(rows, hidden)
            stage_map, stage_copies = plan.staged_row_map(dev), plan.staged_combine()[1]
        last = None
        for c, (j0, j1) in enumerate(chunks):
            u = round_of[c]
            push_until(u + ahead + 1)
            if u != waited:
                ch.wait(seq[u])
                waited = u
            r0, r1 = cumsums[j0], cumsums[j1]
            if fp8d:
                _merge_amax(ectx, plan, ms(_T.kInputGroup1, _M.kAmax, j0), (j0, j1))
            if r1 > r0:
                if merged:
                    backend.block_permute_rows(staged_in, input_fp8, *in_perms[(j0, j1)])
                if not fp8d:
                    backend.grouped_cast_transpose(
                        recv[r0:r1], _rel(cumsums, j0, j1), input_fp8[r0:r1],
                        input_t_fp8[offs[j0]:offs[j1]] if need_t else None, _rel(offs, j0, j1),
                        ms(_T.kInputGroup1, _M.kScale, j0), ms(_T.kInputGroup1, _M.kAmax, j0))
                elif need_t:
                    backend.grouped_cast_transpose(input_fp8[r0:r1], _rel(cumsums, j0, j1), None,
                                                   input_t_fp8[offs[j0]:offs[j1]], _rel(offs, j0, j1), None, None)
                elif keep_rows and not merged:
                    # the receive buffer is reused by the next exchange: keep the rows for the fc1 weight gradient
                    input_keep[r0:r1].copy_(input_fp8[r0:r1])
                backend.fp8_gmm(
                    input_fp8[r0:r1], fc1_w_fp8[j0:j1], sizes_cpu[j0:j1],
                    ms(_T.kInputGroup1, _M.kScaleInv, j0), ms(_T.kWeightGroup1, _M.kScaleInv, j0),
                    c=act_fp8[r0:r1], pre_gelu_out=pre_act[r0:r1],
                    c_scales=ms(_T.kInputGroup2, _M.kScale, j0), c_amaxes=ms(_T.kInputGroup2, _M.kAmax, j0),
                    backward=False, activation=activation)
                if homes and not freed:
                    ectx.wait_buffers_free(plan)
                    freed = True
                backend.fp8_gmm(
                    act_fp8[r0:r1], fc2_w_fp8[j0:j1], sizes_cpu[j0:j1],
                    ms(_T.kInputGroup2, _M.kScaleInv, j0), ms(_T.kWeightGroup2, _M.kScaleInv, j0),
                    c=None if homes else out_local[r0:r1], backward=False,
                    c_row_map=home_map[r0:r1] if homes else stage_map[r0:r1], c_peers=home_ptrs if homes else None)
            last = ch_back.push_arrays(_copy_blocks(out_np, stage_copies[(j0, j1)], stage_ptr, row_bytes))
        ch_back.wait(last)
        if grad_on:
            # reserved now so that every rank knows where to push gradients; returns to the pool with ctx if
            # backward never runs
            ctx.gi = ectx.result_tensor(plan.gi_ids[plan.rank], plan.rows_own, hidden) if need_dgrad else None
            ctx.save_for_backward(input_t_fp8 if need_t else input_keep, (fc1_w_fp8 if need_dgrad else None) if kn else fc1_w_t,
                                  fc2_w_fp8 if kn else fc2_w_t, pre_act, act_fp8 if need_wgrad else None)
            ctx.need_t, ctx.kn = need_t, kn
            metas.set_forward_scale_inv_cloned()
            ctx.metas, ctx.st = metas, st
            ctx.cumsums, ctx.offs, ctx.sizes_cpu = cumsums, offs, sizes_cpu
            ctx.fc1_shape, ctx.fc2_shape = fc1_weight.shape, fc2_weight.shape
            ctx.need_wgrad, ctx.need_dgrad = need_wgrad, need_dgrad
        else:
            ectx.status.record()
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input_t_fp8, fc1_w_t, fc2_w_t, pre_act, act_fp8 = ctx.saved_tensors
        st, metas, cumsums, offs, sizes_cpu = ctx.st, ctx.metas, ctx.cumsums, ctx.offs, ctx.sizes_cpu
        mlp, plan, ectx = st["mlp"], st["plan"], st["ctx"]
        ch, ch_back = ectx.channel, ectx.channel_back
        fp8_meta, activation = mlp.fp8_meta, mlp.activation
        fp8_meta["prepare_backward"]()
        gdt = to_torch_dtype(get_fp8_te_dtype(fp8_meta["recipe"], fprop_tensor=False))
        dy = grad_out.contiguous()
        El, fc1_out, hidden = ctx.fc1_shape
        ffn = ctx.fc2_shape[2]
        row_bytes = hidden * 2
        rows = cumsums[-1]
        dev = dy.device
        wgrad, dgrad = ctx.need_wgrad, ctx.need_dgrad
        need_t = wgrad and ctx.need_t
        ms = metas.get_meta_strided

        recv_ptrs = ectx.recv.ptrs
        fp8d = st["fp8_dispatch"]
        if fp8d:
            # the owners' gradient scales were refreshed by prepare_backward just above: hand them round on the device
            dy_scales = _gather_scales(ms(_T.kGradOutputGroup1, _M.kScale), El, ectx.group)
            src, amax_part = _quantize_at_source(ectx, plan, dy, dy_scales, gdt)
            d_bytes = hidden
        else:
            src, amax_part, d_bytes = dy, None, row_bytes
        dy_ptr = src.data_ptr()
        recv_np = np.asarray(recv_ptrs, dtype=np.uint64)

        def dispatch(chunk, first):
            extra = _amax_blocks(ectx, plan, amax_part, chunk) if fp8d else None
            return ch.push_arrays(_copy_blocks(recv_np, plan.dispatch_arrays(chunk), dy_ptr, d_bytes, extra), after_compute=first)

        chunks = plan.chunks
        ahead = max(1, ectx.dispatch_ahead)
        seq = [dispatch(chunk, i == 0) for i, chunk in enumerate(chunks[:ahead])]   # look-ahead as in forward
        if fp8d:
            recv = None
            grad_out_fp8 = ectx.recv.tensor((rows, hidden), gdt)
        else:
            recv = ectx.recv.tensor((rows, hidden), torch.bfloat16)
            grad_out_fp8 = torch.empty(rows, hidden, dtype=gdt, device=dev)
        grad_out_t = torch.empty(offs[-1], hidden, dtype=gdt, device=dev) if need_t else None
        act_t = torch.empty(offs[-1], ffn, dtype=act_fp8.dtype, device=dev) if need_t else None
        grad_pre_fp8 = torch.empty(rows, fc1_out, dtype=gdt, device=dev)
        grad_pre_t = torch.empty(offs[-1], fc1_out, dtype=gdt, device=dev) if need_t else None
        grad_fc1 = torch.empty(ctx.fc1_shape, dtype=torch.bfloat16, device=dev) if wgrad else None
        grad_fc2 = torch.empty(ctx.fc2_shape, dtype=torch.bfloat16, device=dev) if wgrad else None
        gi = ctx.gi
        ctx.gi = None
        homes = ectx.direct_homes()
        if dgrad:
            assert min(plan.gi_ids) >= 0, "input.requires_grad must agree on all ranks"
            gi_np = np.asarray([ectx.pool.buffers[plan.gi_ids[r]].ptrs[r] for r in range(plan.world)], dtype=np.uint64)
            stage_ptr = ectx.stage_out(rows * row_bytes).data_ptr()
            if homes:
                # the gradient buffers were reserved (and announced free) together with the forward results: the
                # compute stream has waited for that announcement in forward
                home_map, stage_copies = plan.combine_map_dev(dev, homes), plan.combine_map(homes)[1]
                home_ptrs = ectx.result_ptr_table(plan.gi_ids)
            else:
                gi_local = ectx.stage_out(rows * row_bytes)[:rows * row_bytes].view(torch.bfloat16).view(rows, hidden)
                stage_map, stage_copies = plan.staged_row_map(dev), plan.staged_combine()[1]
        last = None
        for c, (j0, j1) in enumerate(chunks):
            r0, r1 = cumsums[j0], cumsums[j1]
            t0, t1 = offs[j0], offs[j1]
            live = r1 > r0
            if live and need_t:
                # needs no gradient rows: runs while they are still on their way
                backend.grouped_cast_transpose(act_fp8[r0:r1], _rel(cumsums, j0, j1), None, act_t[t0:t1], _rel(offs, j0, j1),
                                               None, None)
            if c + ahead < len(chunks):
                seq.append(dispatch(chunks[c + ahead], False))
            ch.wait(seq[c])
            if fp8d:
                _merge_amax(ectx, plan, ms(_T.kGradOutputGroup1, _M.kAmax, j0), (j0, j1))
            if live:
                if not fp8d:
                    backend.grouped_cast_transpose(
                        recv[r0:r1], _rel(cumsums, j0, j1), grad_out_fp8[r0:r1], grad_out_t[t0:t1] if need_t else None,
                        _rel(offs, j0, j1), ms(_T.kGradOutputGroup1, _M.kScale, j0), ms(_T.kGradOutputGroup1, _M.kAmax, j0))
                elif need_t:
                    backend.grouped_cast_transpose(grad_out_fp8[r0:r1], _rel(cumsums, j0, j1), None, grad_out_t[t0:t1],
                                                   _rel(offs, j0, j1), None, None)
                dy_si = ms(_T.kGradOutputGroup1, _M.kScaleInv, j0)
                if need_t:
                    backend.grouped_wgrad(grad_out_t[t0:t1], act_t[t0:t1], _rel(offs, j0, j1), hidden, ffn, dy_si,
                                          ms(_T.kForwardInputGroup2, _M.kScaleInv, j0), c=grad_fc2[j0:j1])
                elif wgrad:
                    backend.grouped_wgrad_rowmajor(grad_out_fp8[r0:r1], act_fp8[r0:r1], _rel(cumsums, j0, j1), dy_si,
                                                   ms(_T.kForwardInputGroup2, _M.kScaleInv, j0), c=grad_fc2[j0:j1])
                if activation == "swiglu" and not need_t and backend.FUSED_DSWIGLU:
                    backend.fp8_gmm_dswiglu(grad_out_fp8[r0:r1], fc2_w_t[j0:j1], sizes_cpu[j0:j1], dy_si,
                                            ms(_T.kForwardWeightGroup2, _M.kScaleInv, j0), pre_act[r0:r1], grad_pre_fp8[r0:r1],
                                            ms(_T.kGradOutputGroup2, _M.kScale, j0), ms(_T.kGradOutputGroup2, _M.kAmax, j0),
                                            b_is_kn=ctx.kn)
                else:
                    grad_act = backend.fp8_gmm(grad_out_fp8[r0:r1], fc2_w_t[j0:j1], sizes_cpu[j0:j1], dy_si,
                                               ms(_T.kForwardWeightGroup2, _M.kScaleInv, j0), backward=True, b_is_kn=ctx.kn)
                    backend.grouped_cast_transpose(
                        grad_act, _rel(cumsums, j0, j1), grad_pre_fp8[r0:r1], grad_pre_t[t0:t1] if need_t else None,
                        _rel(offs, j0, j1), ms(_T.kGradOutputGroup2, _M.kScale, j0), ms(_T.kGradOutputGroup2, _M.kAmax, j0),
                        in2=pre_act[r0:r1], activation=activation)
                dpre_si = ms(_T.kGradOutputGroup2, _M.kScaleInv, j0)
                if dgrad:
                    backend.fp8_gmm(grad_pre_fp8[r0:r1], fc1_w_t[j0:j1], sizes_cpu[j0:j1], dpre_si,
                                    ms(_T.kForwardWeightGroup1, _M.kScaleInv, j0), c=None if homes else gi_local[r0:r1],
                                    backward=True, b_is_kn=ctx.kn, c_row_map=home_map[r0:r1] if homes else stage_map[r0:r1],
                                    c_peers=home_ptrs if homes else None)
            elif wgrad:
                grad_fc1[j0:j1].zero_()
                grad_fc2[j0:j1].zero_()
            if dgrad:
                last = ch_back.push_arrays(_copy_blocks(gi_np, stage_copies[(j0, j1)], stage_ptr, row_bytes))
            else:
                last = ch_back.push([])
            if live and need_t:
                backend.grouped_wgrad(grad_pre_t[t0:t1], input_t_fp8[t0:t1], _rel(offs, j0, j1), fc1_out, hidden, dpre_si,
                                      ms(_T.kForwardInputGroup1, _M.kScaleInv, j0), c=grad_fc1[j0:j1])
            elif live and wgrad:
                # `input_t_fp8` holds the row-major FP8 input here
                backend.grouped_wgrad_rowmajor(grad_pre_fp8[r0:r1], input_t_fp8[r0:r1], _rel(cumsums, j0, j1), dpre_si,
                                               ms(_T.kForwardInputGroup1, _M.kScaleInv, j0), c=grad_fc1[j0:j1])
        ch_back.wait(last)
        ectx.status.record()
        return gi, grad_fc1, grad_fc2, None


def forward(module, input, group_sizes, is_first_microbatch, num_chunks):
    """ExpertParallelMlp.forward over the peer-memory transport."""
    mlp = module.mlp
    ectx = EpContext.setup(input.device, module.group)
    if not ectx.failed:
        try:
            ectx.status.check()
        except RuntimeError:
            ectx.failed = True     # no further pushes into buffers whose state is unknown
            raise
    if ectx.failed:
        raise RuntimeError("fp8_gmm_b200: the expert-parallel exchange was abandoned after a device-side timeout; "
                           "rebuild the process group and the modules")
    grad_on = torch.is_grad_enabled()
    want_gi = grad_on and input.requires_grad
    mlp.get_fp8_weights_scratchpad(is_first_microbatch)
    cache = None if is_first_microbatch is None else mlp._fp8_weights
    reuse = is_first_microbatch is False
    with mlp.prepare_forward(input, is_first_microbatch, mlp.num_groups * 2):
        # The fc1 weight cast needs nothing from the other ranks: it is enqueued first and keeps the GPU busy
        # while the host waits for the all-gather of the group sizes.
        metas = Fp8MetaWrapper(mlp.num_groups, mlp.fp8_meta)
        fdt = to_torch_dtype(get_fp8_te_dtype(mlp.fp8_meta["recipe"], fprop_tensor=True))
        fc1 = cast_weight_cached(mlp.fc1_weight, fdt, want_gi and not backend.DGRAD_KN, metas.get_meta_strided(_T.kWeightGroup1, _M.kScale),
                                 metas.get_meta_strided(_T.kWeightGroup1, _M.kAmax), cache, "fc1", reuse)
        fp8d = bool(getattr(module, "fp8_dispatch", True))
        x_scales = _gather_scales(metas.get_meta_strided(_T.kInputGroup1, _M.kScale), mlp.num_groups, module.group) if fp8d else None
        plan = ectx.plan(group_sizes, input.shape[1] * 2, num_chunks, want_gi)
        st = {"mlp": mlp, "plan": plan, "ctx": ectx, "grad_enabled": grad_on, "weight_cache": cache,
              "reuse_weights": reuse, "fc1_fp8": fc1, "fp8_dispatch": fp8d, "x_scales": x_scales}
        if grad_on:
            return _PeerEpMlp.apply(input, mlp.fc1_weight, mlp.fc2_weight, st)
        return _PeerEpMlp.forward(None, input, mlp.fc1_weight, mlp.fc2_weight, st)
