"""Peer-memory transport between the ranks of one NVSwitch node (one process per GPU).

Used by fp8_gmm_b200.ep for the dispatch / combine row exchange; the reference has nothing comparable (it is
single-GPU apart from one all-reduce, reference fp8_gmm/grouped_mlp.py:300-303).  Every rank allocates receive
buffers through the C ABI (cudaMalloc + CUDA IPC export), all ranks map each other's buffers once, and from then
on rows move as device-to-device copies on a side stream: the copy engines push them over NVLink while the SMs
keep running GEMMs.  A 32-bit sequence number per (receiver, sender) pair, written after the sender's copies
and awaited by a one-warp kernel on the receiver's compute stream, says when a round of copies has landed.
``torch.distributed`` is used only at set-up (to hand the IPC handles round) -- nothing on the data path.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from ._lib import CopyBlock, check, lib

_HANDLE_BYTES = 64


class _Span:
    """Minimal __cuda_array_interface__ holder so torch can view foreign device memory without copying.
    ``on_release`` runs when the last tensor made from it is gone."""

    def __init__(self, ptr, nbytes, on_release=None):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._on_release = on_release

    def __del__(self):
        if self._on_release is not None:
            try:
                self._on_release()
            except Exception:  # interpreter shutdown
                pass


def as_tensor(ptr, shape, dtype, device, on_release=None):
    """Torch tensor over ``ptr`` (device memory not owned by torch's allocator)."""
    numel = 1
    for s in shape:
        numel *= int(s)
    nbytes = numel * torch.empty((), dtype=dtype).element_size()
    if nbytes == 0:
        if on_release is not None:
            on_release()
        return torch.empty(shape, dtype=dtype, device=device)
    flat = torch.as_tensor(_Span(ptr, nbytes, on_release), device=device)
    return flat.view(dtype).view(*shape)


class PeerBuffer:
    """One device buffer per rank, each mapped by every other rank.  Collective: all ranks of ``group`` must
    create their buffers in the same order.  ``ptrs[r]`` is rank r's buffer as seen from this process."""

    def __init__(self, nbytes, device, group=None):
        self.group, self.device, self.nbytes = group, device, int(nbytes)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(_HANDLE_BYTES)
        with torch.cuda.device(device):
            check(lib.fp8gmm_peer_alloc(self.nbytes, ctypes.byref(ptr), handle), "peer_alloc")
        self.local = ptr.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            p = ctypes.c_void_p()
            with torch.cuda.device(device):
                check(lib.fp8gmm_peer_open(ctypes.create_string_buffer(h, _HANDLE_BYTES), ctypes.byref(p)), "peer_open")
            self.ptrs.append(p.value)
        self._closed = False

    def tensor(self, shape, dtype, byte_offset=0, on_release=None):
        return as_tensor(self.local + byte_offset, shape, dtype, self.device, on_release)

    def close(self):
        """Unmaps the peers' buffers and frees the local one.  Collective in spirit: call it on every rank once
        no rank still copies into these buffers (e.g. after a barrier)."""
        if self._closed:
            return
        self._closed = True
        with torch.cuda.device(self.device):
            for r, p in enumerate(self.ptrs):
                if r != self.rank:
                    lib.fp8gmm_peer_close(p)
            lib.fp8gmm_peer_free(self.local)


class PeerChannel:
    """Side stream + sequence numbers of one group of ranks.

    ``push(blocks)`` enqueues copies on the side stream (after whatever the compute stream has enqueued so far)
    and then announces a new sequence number to every rank; ``wait(seq)`` makes the compute stream wait until every
    rank's copies up to ``seq`` have landed here.  All ranks must call ``push`` the same number of times in the
    same order -- a rank with nothing to send still pushes an empty round."""

    def __init__(self, device, group=None, copy_streams=1):
        self.group, self.device = group, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        assert self.world <= 64
        self.flags = PeerBuffer(4096, device, group)          # word s of rank r's page: rounds completed by sender s
        self.stream = torch.cuda.Stream(device=device)
        # optionally a round's copies are dealt over a few streams ("lanes"): no gain between two GPUs (575-600 GB/s
        # per direction for 16 MiB blocks either way), 8-9 % with four lanes when four GPUs push to each other
        self.side = [torch.cuda.Stream(device=device) for _ in range(max(copy_streams, 1) - 1)]
        self.seq = 0
        self.wait_events = None   # a list here collects (start, end) CUDA events around every wait (benchmarks)
        self.round_events = None  # a list here collects (start, end, bytes) per round of copies on the copy stream
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.flags.ptrs[r] + 4 * self.rank       # my word in rank r's page
        self._signal_targets = arr

    _BLOCK = np.dtype([("dst", np.uint64), ("src", np.uint64), ("bytes", np.uint64)])   # layout of fp8gmm_copy_block

    def push(self, blocks, after_compute=True):
        """blocks: iterable of (dst_ptr, src_ptr, nbytes).  Returns the sequence number of this round."""
        blocks = [b for b in blocks if b[2] > 0]
        arr = np.empty(len(blocks), dtype=self._BLOCK)
        if blocks:
            arr["dst"], arr["src"], arr["bytes"] = zip(*blocks)
        return self.push_arrays(arr, after_compute)

    def push_arrays(self, arr, after_compute=True):
        """As push, for a numpy array of copy blocks (dtype ``PeerChannel._BLOCK``; zero-byte entries are skipped by
        the library): no per-block Python work, which matters when a step issues a few hundred copies."""
        arr = np.ascontiguousarray(arr)
        n = len(arr)
        self.seq = (self.seq + 1) & 0xFFFFFFFF
        if after_compute:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
        base = arr.ctypes.data
        lanes = 1 + len(self.side) if n >= 2 * (1 + len(self.side)) else 1
        trace = self.round_events
        if trace is not None:
            t_start = torch.cuda.Event(enable_timing=True)
            t_start.record(self.stream)
        as_blocks = ctypes.POINTER(CopyBlock)
        if lanes == 1:
            check(lib.fp8gmm_peer_copy_blocks(ctypes.cast(base, as_blocks), n, self.stream.cuda_stream), "peer_copy_blocks")
        else:
            # consecutive blocks usually go to the same peer: deal them out in runs, so that the lanes work on
            # different peers at the same time
            streams = [self.stream] + self.side
            for st in self.side:
                st.wait_stream(self.stream)
            run = -(-n // lanes)
            for k, st in enumerate(streams):
                lo, hi = k * run, min((k + 1) * run, n)
                if hi > lo:
                    check(lib.fp8gmm_peer_copy_blocks(ctypes.cast(base + lo * self._BLOCK.itemsize, as_blocks), hi - lo,
                                                      st.cuda_stream), "peer_copy_blocks")
            for st in self.side:
                self.stream.wait_stream(st)
        if trace is not None:
            t_end = torch.cuda.Event(enable_timing=True)
            t_end.record(self.stream)
            trace.append((t_start, t_end, int(arr["bytes"].sum()) if n else 0))
        check(lib.fp8gmm_peer_signal(self._signal_targets, self.world, self.seq, self.stream.cuda_stream), "peer_signal")
        return self.seq

    def wait(self, seq):
        """Compute stream waits for round ``seq`` of every sender (bounded on the device; see fp8gmm_peer_wait)."""
        trace = self.wait_events
        if trace is not None:
            start = torch.cuda.Event(enable_timing=True)
            start.record()
        check(lib.fp8gmm_peer_wait(self.flags.local, self.world, seq, torch.cuda.current_stream(self.device).cuda_stream),
              "peer_wait")
        if trace is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            trace.append((start, end))

    def close(self):
        self.flags.close()
