"""Tensor-parallel sum of the MLP's input gradient over peer memory, overlapped with the GEMMs that produce it.

The reference's only collective is an asynchronous NCCL all-reduce of ``grad_input`` over ``tp_group``, started after
the fc1 data-gradient GEMM and awaited after the fc1 weight-gradient loop (reference
fp8_gmm/grouped_mlp.py:300-303,323-324).  On one NVSwitch node this module replaces it: the fc1 data-gradient GEMM
runs in a few chunks of experts and writes its partial rows into a peer-mapped staging buffer; as soon as a chunk
is written on every rank, two light kernels (fp8gmm_peer_reduce_scatter_bf16 / fp8gmm_peer_all_gather_bf16, plain
peer loads, a few dozen CTAs on a side stream) finish that chunk's sum while the next chunk's GEMM and the fc1
weight gradient run on the tensor cores.  Every element is summed once, by one rank, in ascending rank order in fp32
with one rounding, so all ranks end with identical bits.

    SMs, compute stream :  dgrad chunk 0 | dgrad chunk 1 | dgrad chunk 2 | dgrad chunk 3 | fc1 wgrad ........ | wait
    side stream         :                  sum chunk 0     sum chunk 1     sum chunk 2     sum chunk 3

Ordering between ranks uses three sets of sequence numbers in a peer-mapped flag page: "my partial rows of chunk n
are written", "my slice of chunk n is summed", "I have finished reading round m" (the last one lets the next round
overwrite the staging buffer).  All waits are bounded on the device (see fp8gmm_peer_wait).
"""
import ctypes

import torch
import torch.distributed as dist

from ._lib import check, lib
from .peer import PeerBuffer

_READY, _REDUCED, _RELEASED = 0, 1, 2
_WORDS = 64   # sequence numbers per set (one per sender; fp8gmm_peer_wait handles at most 64)


def chunk_groups(cumsums, num_chunks):
    """[(first group, end group)] cutting the groups into at most ``num_chunks`` runs of about equal row counts.
    ``cumsums``: prefix sums of the group sizes (len = groups + 1).  Pure host arithmetic."""
    G = len(cumsums) - 1
    total = cumsums[-1]
    if G == 0:
        return []
    num_chunks = max(1, min(num_chunks, G))
    bounds = [0]
    for c in range(1, num_chunks):
        target = total * c / num_chunks
        j = min(range(bounds[-1], G + 1), key=lambda g: abs(cumsums[g] - target))
        bounds.append(max(j, bounds[-1]))
    bounds.append(G)
    return [(a, b) for a, b in zip(bounds[:-1], bounds[1:]) if b > a]


class TpReducer:
    """Per (device, tensor-parallel group) state: staging buffer, flag page, side stream, sequence counters.
    Creating it (and growing the staging buffer) is collective over the group; all ranks of a tensor-parallel group
    run the same shapes, so they take those steps together."""

    _instances = {}

    @classmethod
    def setup(cls, device, group):
        key = (device.index, id(group))
        if key not in cls._instances:
            cls._instances[key] = cls(device, group)
        return cls._instances[key]

    def __init__(self, device, group):
        self.device, self.group = device, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= _WORDS
        self.flags = PeerBuffer(4096, device, group)
        self.stage = None
        self.stream = torch.cuda.Stream(device=device)
        self.chunk_seq = 0
        self.round = 0
        self.max_ctas = 48
        self._targets = []
        for s in range(3):
            arr = (ctypes.c_void_p * self.world)()
            for r in range(self.world):
                arr[r] = self.flags.ptrs[r] + 4 * (s * _WORDS + self.rank)     # my word of set s in rank r's page
            self._targets.append(arr)
        self._bufs = None

    def close(self):
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        if self.stage is not None:
            self.stage.close()
        self.flags.close()
        self._instances.pop((self.device.index, id(self.group)), None)

    # ---- signalling ------------------------------------------------------------------------------
    def _signal(self, which, value, stream):
        check(lib.fp8gmm_peer_signal(self._targets[which], self.world, value & 0xFFFFFFFF, stream.cuda_stream), "peer_signal")

    def _wait(self, which, value, stream):
        check(lib.fp8gmm_peer_wait(self.flags.local + 4 * which * _WORDS, self.world, value & 0xFFFFFFFF, stream.cuda_stream),
              "peer_wait")

    # ---- one backward pass -----------------------------------------------------------------------
    def begin(self, rows, cols):
        """Staging tensor (rows, cols) bf16 for the partial sums of this pass.  The compute stream first waits until
        every rank has finished reading the previous pass's staging data."""
        nbytes = rows * cols * 2
        if self.stage is None or self.stage.nbytes < nbytes:
            if self.stage is not None:
                torch.cuda.synchronize(self.device)
                dist.barrier(group=self.group)
                self.stage.close()
            self.stage = PeerBuffer(int(nbytes * 1.25) + 256, self.device, self.group)
            arr = (ctypes.c_void_p * self.world)()
            for r in range(self.world):
                arr[r] = self.stage.ptrs[r]
            self._bufs = arr
        cur = torch.cuda.current_stream(self.device)
        if self.round > 0:
            self._wait(_RELEASED, self.round, cur)
        return self.stage.tensor((rows, cols), torch.bfloat16)

    def reduce_rows(self, out, row0, row1):
        """Sum rows [row0, row1) of the staging tensor over the group into ``out`` (a local (rows, cols) bf16 tensor),
        on the side stream, after everything the compute stream holds so far (the GEMM that wrote those rows)."""
        cols = out.shape[1]
        assert cols % 8 == 0, "the feature width must be a multiple of 8"
        self.chunk_seq += 1
        seq = self.chunk_seq
        side = self.stream
        side.wait_stream(torch.cuda.current_stream(self.device))
        offset, numel = row0 * cols, (row1 - row0) * cols
        self._signal(_READY, seq, side)
        self._wait(_READY, seq, side)
        check(lib.fp8gmm_peer_reduce_scatter_bf16(self._bufs, self.world, self.rank, offset, numel, self.max_ctas,
                                                  side.cuda_stream), "peer_reduce_scatter_bf16")
        self._signal(_REDUCED, seq, side)
        self._wait(_REDUCED, seq, side)
        check(lib.fp8gmm_peer_all_gather_bf16(self._bufs, self.world, self.rank, offset, numel, out.data_ptr(), self.max_ctas,
                                              side.cuda_stream), "peer_all_gather_bf16")

    def finish(self):
        """Compute stream waits for the sums; peers learn that this rank no longer reads their staging buffers."""
        self.round += 1
        self._signal(_RELEASED, self.round, self.stream)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)


PEER_REDUCTION_MAX_RANKS = 4


def use_peer_reduction(tp_group):
    """The peer-memory path serves NCCL groups (one process per GPU on one node) of up to PEER_REDUCTION_MAX_RANKS
    ranks; other backends and larger groups keep the plain ``torch.distributed.all_reduce`` of the reference.
    Measured on the Mixtral-shaped MLP (268 MB of grad_input): at 2 ranks the chunked peer-memory sum exposes 0.21 ms
    against 0.84 ms for the NCCL all-reduce; at 8 ranks each rank's GEMM share is too short to hide 470 MB of peer
    loads (2.8 ms exposed) while NCCL reduces inside the switch (0.8 ms).  FP8GMM_TP=nccl / FP8GMM_TP=peer force one."""
    import os

    choice = os.environ.get("FP8GMM_TP", "auto")
    if choice == "nccl" or not dist.is_initialized() or dist.get_backend(tp_group) != "nccl":
        return False
    world = dist.get_world_size(tp_group)
    return world <= _WORDS if choice == "peer" else world <= PEER_REDUCTION_MAX_RANKS
