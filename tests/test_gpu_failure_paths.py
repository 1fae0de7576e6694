"""GPU: the failure paths that can be exercised without faulting or hanging anything.

Every wait inside this package's kernels is bounded: when it runs out the kernel records a code in the device
status word and returns, and the host finds out through fp8gmm_device_status (blocking) or
fp8gmm_device_status_async (a copy into page-locked memory that a training loop looks at one step later).  The
test below makes such a wait run out on purpose in the only way that needs no broken kernel: fp8gmm_peer_wait on a
sequence number that nobody ever signals, with the limit lowered to 50 ms.  The kernel must come back by itself,
the status must say FP8GMM_DEVICE_TIMEOUT once and be clear afterwards, and the context must stay usable.
(The GEMM kernel's mbarrier waits share the mechanism, but they can only run out if a TMA copy or an MMA never
completes, which no valid launch produces; they are not provoked here.)
"""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_wait_gives_up_and_reports_a_timeout(cuda):
    from fp8_gmm_b200 import _lib, backend

    lib = _lib.lib
    flags = torch.zeros(64, dtype=torch.int32, device=cuda)     # sequence numbers: nobody will ever write 1 here
    stream = torch.cuda.current_stream().cuda_stream
    backend.device_status()                                      # starts clean
    watch = backend.StatusWatch()
    backend.set_wait_limits(peer_wait_s=0.05)
    try:
        t0 = time.perf_counter()
        assert lib.fp8gmm_peer_wait(flags.data_ptr(), 2, 1, stream) == 0
        watch.record()
        torch.cuda.synchronize()
        waited = time.perf_counter() - t0
        assert 0.04 <= waited < 1.0, f"the wait should give up after about 50 ms, took {waited:.3f} s"
        with pytest.raises(RuntimeError, match="bounded wait"):
            watch.check()                                        # the non-blocking view saw it
        assert lib.fp8gmm_device_status(stream) == 4             # FP8GMM_DEVICE_TIMEOUT, and the word is cleared
        assert b"bounded wait" in lib.fp8gmm_last_error()
        assert lib.fp8gmm_device_status(stream) == 0
        # a wait whose numbers are already there returns at once and reports nothing
        flags.fill_(7)
        assert lib.fp8gmm_peer_wait(flags.data_ptr(), 2, 7, stream) == 0
        assert lib.fp8gmm_peer_wait(flags.data_ptr(), 2, 5, stream) == 0   # older rounds count as reached
        backend.device_status()
    finally:
        backend.set_wait_limits(peer_wait_s=2.0)
    # the context is alive: a kernel of the library still runs
    x = torch.randn(64, 64, device=cuda).to(torch.bfloat16)
    q = torch.empty(64, 64, dtype=torch.float8_e4m3fn, device=cuda)
    backend.multi_quantize([x], [q], [torch.ones(1, device=cuda)], [torch.zeros(1, device=cuda)])
    backend.device_status()


def test_wgrad_entry_points_refuse_a_capturing_stream(cuda):
    """The three weight-gradient entry points stage their descriptors from short-lived host memory; on a stream that
    is being captured they must refuse (FP8GMM_UNSUPPORTED) instead of recording a copy from a dead buffer."""
    from fp8_gmm_b200 import backend

    n = k = 64
    dy = torch.zeros(32, n, dtype=torch.uint8, device=cuda).view(torch.float8_e5m2)
    x = torch.zeros(32, k, dtype=torch.uint8, device=cuda).view(torch.float8_e4m3fn)
    ones = torch.ones(1, device=cuda)
    c = torch.empty(1, n, k, dtype=torch.bfloat16, device=cuda)
    backend.grouped_wgrad_rowmajor(dy, x, [0, 32], ones, ones, c=c)   # warm: workspace exists, nothing allocates below
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        graph.capture_begin()
        try:
            with pytest.raises(RuntimeError, match="captured"):
                backend.grouped_wgrad_rowmajor(dy, x, [0, 32], ones, ones, c=c)
        finally:
            graph.capture_end()
    torch.cuda.synchronize()
    backend.grouped_wgrad_rowmajor(dy, x, [0, 32], ones, ones, c=c)
    backend.device_status()
    assert (c == 0).all()
