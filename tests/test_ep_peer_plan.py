"""CPU: the row bookkeeping of the peer-memory exchange (fp8_gmm_b200.ep_peer.PeerPlan).  The device copies are
simulated with numpy: every rank's dispatch blocks are applied to per-rank receive arrays, the "experts" tag the
rows, and the combine blocks must bring every row back to where it started."""
import numpy as np
import pytest
import torch

from fp8_gmm_b200.backend import ROW_MAP_PEER_SHIFT
from fp8_gmm_b200.ep_peer import PeerPlan, chunk_bounds, direct_homes_for, dispatch_rounds_for, resolve_result_buffers


def _counts(P, E, seed, zeros=True):
    g = torch.Generator().manual_seed(seed)
    c = torch.randint(0, 9, (P, E), generator=g)
    if zeros:
        c[0, 1] = 0
        c[:, E - 1] = 0  # an expert nobody routes to
    return c


@pytest.mark.parametrize("P,E,chunks", [(2, 6, 3), (4, 8, 2), (8, 16, 4), (2, 2, 4), (3, 9, 1)])
def test_dispatch_then_combine_is_the_identity(P, E, chunks):
    counts = _counts(P, E, seed=P * 100 + E)
    plans = [PeerPlan(counts, r, chunks) for r in range(P)]
    El = E // P
    # payload of a row: (home rank, home row, global expert)
    x = []
    for s in range(P):
        expert = np.repeat(np.arange(E), counts[s].numpy())
        x.append(np.stack([np.full(expert.shape, s), np.arange(expert.size), expert], 1))
    recv = [np.full((int(sum(plans[o].local_sizes)), 3), -1) for o in range(P)]
    for chunk_index in range(len(plans[0].chunks)):
        for s in range(P):
            for o, d, src, n in plans[s].dispatch_blocks(plans[s].chunks[chunk_index]):
                assert (recv[o][d:d + n] == -1).all(), "two blocks overlap at the owner"
                recv[o][d:d + n] = x[s][src:src + n]
    for o in range(P):
        assert (recv[o] != -1).all(), "a row of the receive buffer was never written"
        # expert-major, and inside an expert ordered by source rank then source row
        local_expert = recv[o][:, 2] - o * El
        assert ((local_expert >= 0) & (local_expert < El)).all()
        key = local_expert * 10**8 + recv[o][:, 0] * 10**5 + recv[o][:, 1]
        assert (np.diff(key) > 0).all()
        assert np.bincount(local_expert, minlength=El).tolist() == plans[o].local_sizes
    back = [np.full_like(x[s], -1) for s in range(P)]
    for o in range(P):
        for chunk in plans[o].chunks:
            for s, d, src, n in plans[o].combine_blocks(chunk):
                back[s][d:d + n] = recv[o][src:src + n]
    for s in range(P):
        assert (back[s] == x[s]).all()
    # The staged form of the combine: the producing GEMM writes a chunk's rows source-major through its row map and
    # one copy per (home rank, chunk) takes them home.  Must be the same permutation.
    back2 = [np.full_like(x[s], -1) for s in range(P)]
    for o in range(P):
        row_map, copies = plans[o].staged_combine()
        assert row_map.dtype == np.int32 and row_map.shape == (recv[o].shape[0],)
        staged = np.full_like(recv[o], -1)
        off = np.concatenate([[0], np.cumsum(plans[o].local_sizes)])
        for j0, j1 in plans[o].chunks:
            r0, r1 = int(off[j0]), int(off[j1])
            rel = row_map[r0:r1]
            assert sorted(rel.tolist()) == list(range(r1 - r0)), "the map permutes the rows of its chunk"
            staged[r0 + rel] = recv[o][r0:r1]
            homes, dst, src, n = copies[(j0, j1)]
            assert sorted(homes.tolist()) == list(range(P)), "one copy per home rank and chunk"
            for s, d, a, k in zip(homes.tolist(), dst.tolist(), src.tolist(), n.tolist()):
                back2[s][d:d + k] = staged[a:a + k]
        assert (staged != -1).all()
    for s in range(P):
        assert (back2[s] == x[s]).all()
    # The direct form: the producing GEMM's epilogue stores every row into its home rank's buffer through a row map
    # whose entries name (home rank, row there).  Must be the same permutation again.
    back3 = [np.full_like(x[s], -1) for s in range(P)]
    for o in range(P):
        entries = plans[o].direct_row_map()
        assert entries.dtype == np.int32 and entries.shape == (recv[o].shape[0],) and (entries >= 0).all()
        home, row = entries >> ROW_MAP_PEER_SHIFT, entries & ((1 << ROW_MAP_PEER_SHIFT) - 1)
        for q in range(entries.size):
            assert (back3[home[q]][row[q]] == -1).all(), "two rows land on the same home row"
            back3[home[q]][row[q]] = recv[o][q]
    for s in range(P):
        assert (back3[s] == x[s]).all()
    # Mixed: some home ranks are served by epilogue stores, the rest through the staging buffer (named as buffer P in
    # the entries) and one copy per (home rank, chunk).
    for direct_homes in [(), (0,), tuple(range(0, P, 2)), tuple(range(P))]:
        back4 = [np.full_like(x[s], -1) for s in range(P)]
        for o in range(P):
            entries, copies = plans[o].combine_map(direct_homes)
            buf, row = entries >> ROW_MAP_PEER_SHIFT, entries & ((1 << ROW_MAP_PEER_SHIFT) - 1)
            staged = np.full_like(recv[o], -1)
            for q in range(entries.size):
                if buf[q] == P:
                    assert (staged[row[q]] == -1).all()
                    staged[row[q]] = recv[o][q]
                else:
                    assert buf[q] in direct_homes
                    back4[buf[q]][row[q]] = recv[o][q]
            for chunk in plans[o].chunks:
                homes, dst, src, n = copies[chunk]
                assert not set(homes.tolist()) & set(direct_homes)
                for s, d, a, k in zip(homes.tolist(), dst.tolist(), src.tolist(), n.tolist()):
                    assert (staged[a:a + k] != -1).all() or k == 0
                    back4[s][d:d + k] = staged[a:a + k]
        for s in range(P):
            assert (back4[s] == x[s]).all(), direct_homes


def test_chunks_cover_the_local_experts_once():
    counts = _counts(4, 20, seed=1, zeros=False)
    for chunks in (1, 2, 3, 5, 8):
        plan = PeerPlan(counts, 1, chunks)
        covered = [j for j0, j1 in plan.chunks for j in range(j0, j1)]
        assert covered == list(range(5))
        assert len(plan.chunks) == min(chunks, 5)


def test_staggered_peer_order():
    counts = _counts(4, 8, seed=3, zeros=False)
    firsts = [PeerPlan(counts, r, 1).dispatch_blocks((0, 2))[0][0] for r in range(4)]
    assert sorted(firsts) == [0, 1, 2, 3], "every rank must start with a different destination"


@pytest.mark.parametrize("El", [1, 2, 5, 6, 16, 32, 64])
def test_tapered_and_explicit_chunks_partition_the_experts(El):
    for spec in ("tapered", 3, [El]):
        chunks = chunk_bounds(El, spec)
        assert [j for a, b in chunks for j in range(a, b)] == list(range(El))
    if El >= 16:
        sizes = [b - a for a, b in chunk_bounds(El, "tapered")]
        assert sizes[0] < max(sizes) and sizes[-1] < max(sizes)


def test_result_buffer_resolution_is_the_same_on_every_rank():
    # rank 0 has both buffers, rank 1 lacks the gradient buffer, rank 2 lacks both, rank 3 wants no gradient buffer
    picks = [[0, 1], [2, -1], [-1, -1], [1, -2]]
    missing, resolved = resolve_result_buffers(picks, buffers_before=3)
    assert missing == 2
    assert resolved == [[0, 1], [2, 3], [3, 4], [1, -2]]
    assert resolve_result_buffers([[0, 1], [1, 0]], 2) == (0, [[0, 1], [1, 0]])
    assert resolve_result_buffers([[-1, -2]], 0) == (1, [[0, -2]])


def test_home_ranks_served_by_epilogue_stores():
    assert direct_homes_for("auto", 1, 2) == (0, 1)
    assert direct_homes_for("auto", 5, 8) == ()
    assert direct_homes_for("none", 3, 4) == ()
    assert direct_homes_for("all", 3, 4) == (0, 1, 2, 3)
    assert direct_homes_for("2", 7, 8) == (0, 1, 7)
    assert direct_homes_for("9", 1, 4) == (0, 1, 2, 3)


@pytest.mark.parametrize("P,E,chunks,spec", [(2, 8, 4, "chunks"), (4, 16, 4, "2,2"), (8, 32, "tapered", "2,4"),
                                             (4, 32, "tapered", "1,2,3"), (2, 12, 3, "2,2")])
def test_merged_dispatch_rounds_then_block_permutation_is_the_expert_major_layout(P, E, chunks, spec):
    """Forward dispatch through the source-major staging buffer: one copy per (owner, round), a round carrying the rows
    of one or several chunks, then the owner's block permutation chunk by chunk -- must leave exactly what the
    per-expert copies straight into expert-major place leave."""
    counts = _counts(P, E, seed=P * 10 + E)
    plans = [PeerPlan(counts, r, chunks) for r in range(P)]
    x = []
    for s in range(P):
        expert = np.repeat(np.arange(E), counts[s].numpy())
        x.append(np.stack([np.full(expert.shape, s), np.arange(expert.size), expert], 1))
    want = [np.full((int(sum(plans[o].local_sizes)), 3), -1) for o in range(P)]
    for s in range(P):
        for chunk in plans[s].chunks:
            for o, d, src, n in plans[s].dispatch_blocks(chunk):
                want[o][d:d + n] = x[s][src:src + n]
    rounds = dispatch_rounds_for(spec, plans[0].chunks)
    assert rounds[0][0] == 0 and rounds[-1][1] == E // P and all(a[1] == b[0] for a, b in zip(rounds, rounds[1:]))
    staging = [np.full_like(want[o], -1) for o in range(P)]
    for s in range(P):
        copies, _ = plans[s].staged_dispatch(rounds)
        assert sorted(copies) == sorted(rounds)
        for rnd in rounds:
            owners, dst, src, n = copies[rnd]
            assert sorted(owners.tolist()) == list(range(P)), "one copy per owner and round"
            for o, d, a, k in zip(owners.tolist(), dst.tolist(), src.tolist(), n.tolist()):
                assert (staging[o][d:d + k] == -1).all(), "two copies overlap in the staging buffer"
                staging[o][d:d + k] = x[s][a:a + k]
    for o in range(P):
        got = np.full_like(want[o], -1)
        _, perms = plans[o].staged_dispatch(rounds)
        assert sorted(perms) == sorted(plans[o].chunks)
        for chunk in plans[o].chunks:
            for a, d, k in zip(*[v.tolist() for v in perms[chunk]]):
                got[d:d + k] = staging[o][a:a + k]
        assert (got == want[o]).all()


def test_dispatch_round_specs():
    chunks = chunk_bounds(16, "tapered")
    assert dispatch_rounds_for("chunks", chunks) == chunks
    assert dispatch_rounds_for("auto", chunks) == chunks
    assert dispatch_rounds_for("2,4", chunks) == [(0, 3), (3, 16)]
    assert dispatch_rounds_for("1,2,3", chunks) == [(0, 1), (1, 7), (7, 16)]
    assert dispatch_rounds_for("2,2", chunks) == [(0, 3), (3, 11), (11, 16)]     # the last round takes what is left
    assert dispatch_rounds_for("2,4", chunk_bounds(4, 2)) == [(0, 2), (2, 4)]    # two chunks: nothing to merge
