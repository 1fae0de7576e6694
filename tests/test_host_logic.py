"""CPU: host-side bookkeeping that defines layouts and meta slots (reference fp8_gmm/utils.py)."""
import torch

from fp8_gmm_b200 import recipe, utils
from oracle import oracle as O


def test_cumsum_group_sizes_matches_reference_semantics():
    # reference fp8_gmm/utils.py:48-62
    assert utils.cumsum_group_sizes([128, 96, 160, 128], need_padding=True) == (4, False, [0, 128, 224, 384, 512], [0, 128, 224, 384, 512])
    assert utils.cumsum_group_sizes([5, 0, 33], need_padding=True) == (3, True, [0, 5, 5, 38], [0, 16, 16, 64])
    assert utils.cumsum_group_sizes([5, 0, 33]) == (3, False, [0, 5, 5, 38], None)
    assert utils.cumsum_group_sizes([]) == (0, False, [0], None)
    for sizes in ([1, 2, 3], [16, 32], [0, 0], [4095, 17, 1]):
        assert utils.cumsum_group_sizes(sizes, True) == O.cumsum_group_sizes(sizes, True)


class _Meta:
    def __init__(self, n, hist=2):
        self.scale = torch.arange(n, dtype=torch.float32)
        self.scale_inv = torch.arange(n, dtype=torch.float32) + 100
        self.amax_history = torch.arange(hist * n, dtype=torch.float32).reshape(hist, n) + 1000


def test_meta_slots():
    # reference fp8_gmm/utils.py:98-103: slot = (group_offset + i) * stage + type
    G = 3
    meta = {"scaling_fwd": _Meta(3 * 2 * G), "scaling_bwd": _Meta(2 * 2 * G)}
    w = utils.Fp8MetaWrapper(G, meta)
    T, M = utils.Fp8TensorType, utils.MetaTensorType
    get = lambda t, m: [float(v) for v in w.get_meta_tensors(t, m)]  # noqa: E731
    assert get(T.kInputGroup1, M.kScale) == [0, 3, 6]
    assert get(T.kWeightGroup1, M.kScale) == [1, 4, 7]
    assert get(T.kInputGroup2, M.kScale) == [9, 12, 15]
    assert get(T.kWeightGroup2, M.kScaleInv) == [110, 113, 116]
    assert get(T.kGradOutputGroup1, M.kScale) == [0, 2, 4]
    assert get(T.kGradOutputGroup2, M.kAmax) == [1006, 1008, 1010]
    w.set_forward_scale_inv_cloned()
    meta["scaling_fwd"].scale_inv += 1  # later updates must not leak into the snapshot
    assert get(T.kForwardInputGroup1, M.kScaleInv) == [100, 103, 106]
    assert get(T.kForwardWeightGroup2, M.kScaleInv) == [110, 113, 116]
    # strided form addresses the same slots
    for t, m in [(T.kInputGroup2, M.kScale), (T.kGradOutputGroup2, M.kAmax), (T.kForwardWeightGroup1, M.kScaleInv)]:
        base, stride = w.get_meta_strided(t, m)
        assert [float(base[i * stride]) for i in range(G)] == get(t, m)


def test_dtype_maps_and_recipe_formats():
    assert utils.to_torch_dtype(utils.to_tex_dtype(torch.float8_e5m2)) == torch.float8_e5m2
    r = recipe.DelayedScaling(fp8_format=recipe.Format.HYBRID)
    assert recipe.get_fp8_te_dtype(r, True) == utils.DType.kFloat8E4M3
    assert recipe.get_fp8_te_dtype(r, False) == utils.DType.kFloat8E5M2
    assert recipe.get_fp8_te_dtype(recipe.DelayedScaling(fp8_format=recipe.Format.E4M3), False) == utils.DType.kFloat8E4M3
    with recipe.fp8_autocast(enabled=True, fp8_recipe=recipe.DelayedScaling(amax_history_len=16)):
        assert recipe.is_fp8_enabled() and recipe.get_fp8_recipe().amax_history_len == 16
    assert not recipe.is_fp8_enabled()


def test_router_oracle_round_trip():
    """oracle.moe_sort / moe_gather / moe_scatter: gathering and scattering with unit weights and top_k = 1 is the
    identity; with top_k > 1 every token gets the sum of its copies."""
    from oracle import oracle as O

    g = torch.Generator().manual_seed(0)
    tokens, top_k, E, H = 50, 3, 7, 16
    ids = torch.randint(0, E, (tokens * top_k,), generator=g)
    indices, bin_ids, bins, hist, inverse = O.moe_sort(ids, E)
    assert torch.equal(bin_ids, ids[indices]) and (bin_ids[1:] >= bin_ids[:-1]).all()
    assert int(bins[-1]) == tokens * top_k and torch.equal(hist, torch.bincount(ids, minlength=E))
    x = torch.randn(tokens, H, generator=g).to(torch.bfloat16)
    rows = O.moe_gather(x, indices, top_k)
    assert torch.equal(rows[inverse].reshape(tokens, top_k, H)[:, 0], x)
    out = O.moe_scatter(rows, inverse, top_k)
    assert torch.allclose(out.float(), 3 * x.float(), rtol=1e-2, atol=1e-2)


def test_tensor_parallel_chunks_cover_all_groups_in_order():
    """Chunk bookkeeping of the tensor-parallel reduction: contiguous runs of groups, every group in exactly one
    chunk, about equal row counts, empty groups and fewer groups than chunks handled."""
    from fp8_gmm_b200.tp import chunk_groups

    for sizes, chunks in [([4122, 4066, 4022, 4015, 4148, 4194, 4168, 4033], 4), ([5, 0, 0, 900, 1], 4), ([7], 4), ([0, 0, 0], 2),
                          ([10] * 64, 4), ([], 4), ([1000, 1, 1, 1, 1, 1, 1, 1000], 3)]:
        cums = [0]
        for s in sizes:
            cums.append(cums[-1] + s)
        out = chunk_groups(cums, chunks)
        assert len(out) <= max(chunks, 1)
        flat = [g for a, b in out for g in range(a, b)]
        assert flat == list(range(len(sizes)))
        assert all(b > a for a, b in out)
    even = chunk_groups([0, 100, 200, 300, 400, 500, 600, 700, 800], 4)
    assert even == [(0, 2), (2, 4), (4, 6), (6, 8)]


def test_fp8_state_survives_torch_save_and_default_torch_load(tmp_path):
    """The FP8 recipe state is part of state_dict and holds tensors / numbers / strings only, so a checkpoint written
    with torch.save loads with torch.load's default arguments (weights_only=True) and restores scales, amax history,
    step counters and the recipe; a Transformer-Engine-style dictionary of meta tensors is accepted as well."""
    import torch

    import fp8_gmm_b200 as fg
    from fp8_gmm_b200.recipe import Format

    recipe = fg.DelayedScaling(margin=1, interval=2, fp8_format=Format.HYBRID, amax_history_len=5, amax_compute_algo="most_recent")
    a = fg.GroupedMlp(32, 64, 3, torch.bfloat16, device="cpu", activation="swiglu")
    with fg.fp8_autocast(enabled=True, fp8_recipe=recipe):
        a._init_fp8_meta(6, torch.device("cpu"))
    g = torch.Generator().manual_seed(0)
    for key in ("scaling_fwd", "scaling_bwd"):
        meta = a.fp8_meta[key]
        meta.scale.copy_(torch.rand(meta.scale.shape, generator=g) + 0.5)
        meta.scale_inv.copy_(1.0 / meta.scale)
        meta.amax_history.copy_(torch.rand(meta.amax_history.shape, generator=g))
    a.fp8_meta["step_fwd"], a.fp8_meta["step_bwd"] = 7, 6
    a.fp8_meta["update_amax_and_scale_fwd"] = True
    path = tmp_path / "ckpt.pt"
    torch.save(a.state_dict(), path)
    loaded = torch.load(path)                       # default arguments: weights_only=True
    b = fg.GroupedMlp(32, 64, 3, torch.bfloat16, device="cpu", activation="swiglu")
    b.load_state_dict(loaded)
    assert torch.equal(a.fc1_weight, b.fc1_weight)
    for key in ("scaling_fwd", "scaling_bwd"):
        for field in ("scale", "scale_inv", "amax_history"):
            assert torch.equal(getattr(a.fp8_meta[key], field), getattr(b.fp8_meta[key], field))
    assert b.fp8_meta["recipe"] == recipe and b.fp8_meta["step_fwd"] == 7 and b.fp8_meta["step_bwd"] == 6
    assert b.fp8_meta["update_amax_and_scale_fwd"] is True
    # Transformer Engine's key layout
    te_style = {f"{name}_{d}": getattr(a.fp8_meta[f"scaling_{d}"], name).clone() for d in ("fwd", "bwd")
                for name in ("scale", "scale_inv", "amax_history")}
    c = fg.GroupedMlp(32, 64, 3, torch.bfloat16, device="cpu", activation="swiglu")
    c.set_extra_state(te_style)
    assert c.fp8_meta["num_gemms"] == 6 and torch.equal(c.fp8_meta["scaling_bwd"].scale, a.fp8_meta["scaling_bwd"].scale)
    assert c.fp8_meta["recipe"].amax_history_len == 5
