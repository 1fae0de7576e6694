"""GPU: the allocation-free weight-gradient entry point, fp8gmm_grouped_wgrad_static.

Some hosts of this library cannot give it a device workspace and cannot allocate one either (a framework
that has reserved the whole GPU for its own pool, a runtime that forbids plug-ins to allocate once it is
running).  For them the weight-gradient GEMM exists in a form that keeps its per-group TMA descriptors in
a fixed array inside the library.  This test calls that entry point directly through the C ABI, twice in a
row with different group layouts (a call must not be disturbed by what the one before left in the shared
array, also when it uses fewer slots), and requires the same bits as the workspace-taking entry point produces
and <= 4e-3 relative Frobenius error against the CPU oracle.  The size limit is checked too.

The file name sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def _operands(sizes, n, k, seed, dev):
    from fp8_gmm_b200.utils import cumsum_group_sizes

    G, padded, cums, pcs = cumsum_group_sizes(sizes, need_padding=True)
    offs = pcs if padded else cums
    g = torch.Generator().manual_seed(seed)
    # random FP8 bytes with moderate magnitudes (exponent field below its top values: no NaN/Inf encodings)
    a = torch.randint(0, 256, (offs[-1] * n,), generator=g, dtype=torch.uint8)
    b = torch.randint(0, 256, (offs[-1] * k,), generator=g, dtype=torch.uint8)
    a = torch.where((a & 0x7F) >= 0x70, (a & 0x8F) | 0x30, a)
    b = torch.where((b & 0x7F) >= 0x70, (b & 0x8F) | 0x30, b)
    sa = torch.rand(G, generator=g) * 0.01 + 0.001
    sb = torch.rand(G, generator=g) * 0.01 + 0.001
    return offs, a.view(E5).to(dev), b.view(E4).to(dev), sa.to(dev), sb.to(dev)


def _call_static(lib_mod, a_t, b_t, offs, n, k, sa, sb, c):
    args = lib_mod.WgradArgs()
    args.a_t, args.b_t, args.c = a_t.data_ptr(), b_t.data_ptr(), c.data_ptr()
    arr = (ctypes.c_int64 * len(offs))(*offs)
    args.t_offsets = ctypes.cast(arr, ctypes.POINTER(ctypes.c_int64))
    args.num_groups, args.n, args.k = len(offs) - 1, n, k
    args.a_format, args.b_format = 1, 0
    args.a_scale_inv, args.a_scale_inv_stride = sa.data_ptr(), 1
    args.b_scale_inv, args.b_scale_inv_stride = sb.data_ptr(), 1
    args.workspace, args.workspace_bytes = None, 0  # ignored by this entry point
    return lib_mod.lib.fp8gmm_grouped_wgrad_static(ctypes.byref(args), torch.cuda.current_stream().cuda_stream)


def _oracle_wgrad(a_t, b_t, offs, n, k, sa, sb):
    """The CPU oracle on the same padded-transposed blocks."""
    from oracle import oracle as O

    a8, b8 = a_t.cpu().view(torch.uint8), b_t.cpu().view(torch.uint8)
    G = len(offs) - 1
    blocks_a = [a8[offs[g] * n:offs[g + 1] * n].reshape(n, offs[g + 1] - offs[g]).view(E5) for g in range(G)]
    blocks_b = [b8[offs[g] * k:offs[g + 1] * k].reshape(k, offs[g + 1] - offs[g]).view(E4) for g in range(G)]
    return O, O.grouped_wgrad(blocks_a, blocks_b, sa.cpu(), sb.cpu())


def test_static_wgrad_matches_workspace_wgrad_and_the_oracle_on_calls_in_a_row(cuda):
    from fp8_gmm_b200 import _lib, backend

    # three calls back to back; the third has fewer groups than the one before, so descriptor slots of the shared
    # array that the second call filled are stale during the third and must not be read
    cases = [([128, 0, 37, 300, 16, 1], 272, 144, 11), ([64, 200, 5], 512, 256, 12), ([48, 7], 512, 256, 13)]
    for sizes, n, k, seed in cases:
        offs, a_t, b_t, sa, sb = _operands(sizes, n, k, seed, cuda)
        G = len(sizes)
        want = backend.grouped_wgrad(a_t, b_t, offs, n, k, sa, sb)
        got = torch.full((G, n, k), float("nan"), dtype=torch.bfloat16, device=cuda)
        rc = _call_static(_lib, a_t, b_t, offs, n, k, sa, sb, got)
        assert rc == 0, _lib.lib.fp8gmm_last_error()
        backend.device_status()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        O, ref = _oracle_wgrad(a_t, b_t, offs, n, k, sa, sb)
        assert O.rel_frobenius(got.cpu(), ref) <= 4e-3
        for g, m in enumerate(sizes):
            if m == 0:
                assert (got[g] == 0).all()


def test_static_wgrad_rejects_more_groups_than_its_array_holds(cuda):
    from fp8_gmm_b200 import _lib

    G = 129
    offs = [16 * i for i in range(G + 1)]
    a_t = torch.zeros(offs[-1] * 32, dtype=torch.uint8, device=cuda).view(E5)
    b_t = torch.zeros(offs[-1] * 32, dtype=torch.uint8, device=cuda).view(E4)
    s = torch.ones(G, device=cuda)
    c = torch.empty(G, 32, 32, dtype=torch.bfloat16, device=cuda)
    rc = _call_static(_lib, a_t, b_t, offs, 32, 32, s, s, c)
    assert rc == 3  # FP8GMM_UNSUPPORTED
    assert b"128" in _lib.lib.fp8gmm_last_error()
