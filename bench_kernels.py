"""Per-kernel microbenchmarks (CUDA-event timed) for the three kernel families of fp8_gmm_b200.

    python bench_kernels.py gemm  [--groups G --rows R --n N --k K --act none|gelu|swiglu --a-format e4m3|e5m2]
    python bench_kernels.py wgrad [--groups G --rows R --n N --k K]
    python bench_kernels.py step-gemms            # the six GEMMs of the Mixtral-shaped step, one by one
    python bench_kernels.py scaled-mm [--groups G --rows R --n N --k K]   # library baseline: torch._scaled_mm per group
    python bench_kernels.py library-step          # this package vs the per-group library loop on the six step GEMMs
    python bench_kernels.py pad   [--groups G --max-rows M --cols K --mode cast|amax+cast|transpose|quantize|dswiglu|dswiglu+transpose]
                                                  # default = the pad-fusion microbenchmark: 256 groups, rows ~ U[0,4096],
                                                  # K = 7168, bf16 ~ N(0,3) with 0.1 % outliers x100
    common: [--iters I --warmup W]

Every sub-command prints one JSON line.  GEMMs report TFLOP/s (algorithmic FLOPs, true rows) and the
fraction of 2 x the measured dense bf16 rate; the HBM-bound kernels report GB/s (algorithmic bytes:
cast + padded transpose = 2mn read + mn + Mpad*n written; quantise = 3 bytes per element; fp8 transpose =
mn + Mpad*n) and the fraction of the measured copy bandwidth and of the nominal 8 TB/s.  Working sets
exceed the 126 MB L2 in the default configurations.  These are also the small cases used for ncu captures.
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

E4, E5 = torch.float8_e4m3fn, torch.float8_e5m2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


LAST_CLOCKS = None


def time_ms(fn, iters, warmup):
    """Mean milliseconds per call over `iters` back-to-back calls; SM clocks are sampled meanwhile."""
    global LAST_CLOCKS
    from bench import ClockSampler

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
    LAST_CLOCKS = clocks.summary()
    return s.elapsed_time(e) / iters


def rand_fp8(shape, dtype, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    b = torch.randint(0, 256, shape, generator=g, dtype=torch.uint8, device=dev)
    b = torch.where((b & 0x7F) >= 0x70, b & 0x8F | 0x30, b)  # moderate magnitudes, no NaN/Inf encodings
    return b.view(dtype)


def even_sizes(groups, rows):
    base = rows // groups
    sizes = [base] * groups
    sizes[-1] += rows - base * groups
    return sizes


def gemm_case(backend, dev, sizes, n, k, act, a_dtype, iters, warmup, label, b_is_kn=False, buffers=0):
    """b_is_kn: B is (G, K, N) and read MN-major (how dgrad consumes the forward weights by default).
    buffers > 0: the epilogue stores its rows into that many result buffers named by a row map (the expert-parallel
    combine; here all buffers are in this GPU's memory): runs of 1000 rows go to the buffers in turn."""
    G, m = len(sizes), sum(sizes)
    a = rand_fp8((m, k), a_dtype, dev, 1)
    b = rand_fp8((G, k, n) if b_is_kn else (G, n, k), E4, dev, 2)
    ones = torch.ones(G, device=dev)
    ms_sizes = torch.tensor(sizes)
    if act == "none" and buffers > 0:
        rows = torch.arange(m, dtype=torch.int64)
        run = rows // 1000
        buf = run % buffers
        row_in_buf = (run // buffers) * 1000 + rows % 1000
        entries = backend.peer_row_entry(buf, row_in_buf).to(torch.int32).to(dev)
        outs = [torch.empty(int(row_in_buf[buf == r].max()) + 1, n, dtype=torch.bfloat16, device=dev) for r in range(buffers)]
        table = torch.tensor([t.data_ptr() for t in outs], dtype=torch.int64).to(dev)
        fn = lambda: backend.fp8_gmm(a, b, ms_sizes, ones, ones, c_row_map=entries, c_peers=table, b_is_kn=b_is_kn)  # noqa: E731
        label += f", rows stored into {buffers} buffers through the row map"
    elif act == "none":
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: backend.fp8_gmm(a, b, ms_sizes, ones, ones, c=c, b_is_kn=b_is_kn)  # noqa: E731
    else:
        n_act = n // 2 if act == "swiglu" else n
        pre = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        c = torch.empty(m, n_act, dtype=E4, device=dev)
        amax = torch.zeros(G, device=dev)
        fn = lambda: backend.fp8_gmm(a, b, ms_sizes, ones, ones, c=c, pre_gelu_out=pre, c_scales=ones, c_amaxes=amax,  # noqa: E731
                                     activation=act)
    ms = time_ms(fn, iters, warmup)
    backend.device_status()
    _, bf16, src = peaks()
    tf = 2.0 * m * n * k / ms / 1e9
    return {"kernel": "grouped_gemm" + (" (B read MN-major)" if b_is_kn else ""), "case": label, "groups": G, "rows": m, "n": n, "k": k, "act": act,
            "a_format": "e4m3" if a_dtype == E4 else "e5m2", "ms": ms, "tflops": tf, "clocks": LAST_CLOCKS,
            "frac_of_2x_bf16_" + src: tf / (2 * bf16), "frac_of_nominal_4500": tf / 4500.0}


def wgrad_case(backend, dev, sizes, n, k, iters, warmup, label, rowmajor=False):
    """rowmajor: operands are the row-major activations (read MN-major, the default dataflow); else the reference's
    padded transposes."""
    from fp8_gmm_b200.utils import cumsum_group_sizes

    G, padded, cums, pcs = cumsum_group_sizes(sizes, need_padding=True)
    offs = pcs if padded else cums
    ones = torch.ones(G, device=dev)
    c = torch.empty(G, n, k, dtype=torch.bfloat16, device=dev)
    if rowmajor:
        dy = rand_fp8((cums[-1], n), E5, dev, 3)
        x = rand_fp8((cums[-1], k), E4, dev, 4)
        fn = lambda: backend.grouped_wgrad_rowmajor(dy, x, cums, ones, ones, c=c)  # noqa: E731
    else:
        a_t = rand_fp8((offs[-1] * n,), E5, dev, 3)
        b_t = rand_fp8((offs[-1] * k,), E4, dev, 4)
        fn = lambda: backend.grouped_wgrad(a_t, b_t, offs, n, k, ones, ones, c=c)  # noqa: E731
    ms = time_ms(fn, iters, warmup)
    backend.device_status()
    _, bf16, src = peaks()
    tf = 2.0 * sum(sizes) * n * k / ms / 1e9
    return {"kernel": "grouped_gemm(wgrad, " + ("row-major operands" if rowmajor else "padded transposes") + ")", "case": label, "groups": G, "rows": sum(sizes), "n": n, "k": k, "ms": ms,
            "tflops": tf, "clocks": LAST_CLOCKS, "frac_of_2x_bf16_" + src: tf / (2 * bf16), "frac_of_nominal_4500": tf / 4500.0}


def scaled_mm_case(dev, sizes, n, k, iters, warmup, label, kind="fwd"):
    """Library comparison (never on the product path): the per-group cuBLASLt FP8 loop, ``torch._scaled_mm`` once per
    group, which is what the reference's Transformer-Engine path amounts to on this GPU (reference
    fp8_gmm/backend.py:84-96, wgrad fp8_gmm/grouped_linear.py:165-182).  Operands are laid out the way the reference
    prepares them, outside the timed region: forward / dgrad multiply row slices by a (N, K) weight (for dgrad the
    reference's per-expert weight transpose), wgrad multiplies the padded transposes (N x L_g) (K x L_g)^T.  All
    operands e4m3 (same rate as e5m2 x e4m3).  C_g (m_g x n) with contraction k; for kind="wgrad" C_g is (n x k) with
    contraction m_g rounded up to 16."""
    G, m = len(sizes), sum(sizes)
    one = torch.ones((), device=dev)
    if kind == "wgrad":
        pads = [(s_ + 15) // 16 * 16 for s_ in sizes]
        a_t = [rand_fp8((n, L), E4, dev, 10 + g) for g, L in enumerate(pads)]
        b_t = [rand_fp8((k, L), E4, dev, 50 + g) for g, L in enumerate(pads)]
        c = torch.empty(G, n, k, dtype=torch.bfloat16, device=dev)

        def fn():
            for g in range(G):
                torch._scaled_mm(a_t[g], b_t[g].t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=c[g])
    else:
        a = rand_fp8((m, k), E4, dev, 1)
        b = rand_fp8((G, n, k), E4, dev, 2)
        c = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        offs = [0]
        for s_ in sizes:
            offs.append(offs[-1] + s_)

        def fn():
            for g in range(G):
                torch._scaled_mm(a[offs[g]:offs[g + 1]], b[g].t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16,
                                 out=c[offs[g]:offs[g + 1]])

    ms = time_ms(fn, iters, warmup)
    _, bf16, src = peaks()
    tf = 2.0 * m * n * k / ms / 1e9
    return {"kernel": "torch._scaled_mm per group (cuBLASLt, library baseline)", "case": label, "groups": G, "rows": m,
            "n": n, "k": k, "ms": ms, "tflops": tf, "clocks": LAST_CLOCKS, "frac_of_2x_bf16_" + src: tf / (2 * bf16)}


def step_shapes(H=4096, F=14336):
    """(label, kind, N, K, activation, A format) of the six GEMMs of one Mixtral-shaped SwiGLU step."""
    return [("fc1_fwd", "fwd", 2 * F, H, "swiglu", E4), ("fc2_fwd", "fwd", H, F, "none", E4),
            ("fc2_dgrad", "dgrad", F, H, "none", E5), ("fc1_dgrad", "dgrad", H, 2 * F, "none", E5),
            ("fc2_wgrad", "wgrad", H, F, "none", E5), ("fc1_wgrad", "wgrad", 2 * F, H, "none", E5)]


def library_gemm_suite(backend, dev, sizes, iters=5, warmup=2, H=4096, F=14336):
    """This package's grouped GEMM and the per-group library loop side by side on the six shapes of the step, timed
    the same way (back-to-back launches, CUDA events).  Returns {label: {"ours_tflops", "library_tflops", ...}}."""
    out = {}
    for label, kind, n, k, act, a_dt in step_shapes(H, F):
        if kind == "wgrad":
            ours = wgrad_case(backend, dev, sizes, n, k, iters, warmup, label, rowmajor=True)
        else:
            ours = gemm_case(backend, dev, sizes, n, k, act, a_dt, iters, warmup, label, b_is_kn=kind == "dgrad")
        torch.cuda.empty_cache()
        lib_ = scaled_mm_case(dev, sizes, n, k, iters, warmup, label, kind="wgrad" if kind == "wgrad" else "fwd")
        torch.cuda.empty_cache()
        out[label] = {"ours_tflops": ours["tflops"], "library_tflops": lib_["tflops"], "ours_ms": ours["ms"],
                      "library_ms": lib_["ms"], "ours_sm_mhz": (ours["clocks"] or {}).get("sm_mhz"),
                      "library_sm_mhz": (lib_["clocks"] or {}).get("sm_mhz")}
    return out


def pad_inputs(dev, groups, max_rows, cols, seed=0):
    """The pad / cast microbenchmark's inputs: `groups` row blocks with rows ~ U[0, max_rows] (seeded), `cols` wide,
    bf16 ~ N(0, 3) with 0.1 % of the elements multiplied by 100.  Generated on the device in slabs."""
    g = torch.Generator().manual_seed(seed)
    rows = torch.randint(0, max_rows + 1, (groups,), generator=g).tolist()
    m = sum(rows)
    gd = torch.Generator(device=dev).manual_seed(seed + 1)
    x = torch.empty(m, cols, dtype=torch.bfloat16, device=dev)
    for r0 in range(0, m, 32768):
        r1 = min(m, r0 + 32768)
        v = torch.randn(r1 - r0, cols, generator=gd, device=dev) * 3.0
        x[r0:r1] = torch.where(torch.rand(r1 - r0, cols, generator=gd, device=dev) < 1e-3, v * 100.0, v).to(torch.bfloat16)
    return rows, x


PAD_MODES = ["cast", "amax+cast", "transpose", "quantize", "dswiglu", "dswiglu+transpose"]


def pad_case(backend, dev, groups, max_rows, cols, mode, iters, warmup):
    """One HBM-bound kernel family on the pad microbenchmark's data.  Algorithmic bytes per op:
    cast (bf16 -> e4m3 row-major + padded transpose + amax) 2mn + mn + Mpad*n; amax+cast (current scaling: amax pass,
    scale, then cast) 2mn more; transpose (fp8 -> padded fp8) mn + Mpad*n; quantize (flat cast + amax) 3mn;
    dswiglu (d-activation fused with the e5m2 cast; dy (m, n/2), pre-activation (m, n) -> (m, n)) mn + 2mn + mn,
    + Mpad*n with the padded transpose."""
    from fp8_gmm_b200.utils import cumsum_group_sizes

    rows, x = pad_inputs(dev, groups, max_rows, cols)
    G, padded, cums, pcs = cumsum_group_sizes(rows, need_padding=True)
    m, k = cums[-1], cols
    scale = torch.ones(G, device=dev)
    amax = torch.zeros(G, device=dev)
    hbm, _, src = peaks()
    if mode.startswith("dswiglu"):
        half = k // 2
        gd = torch.Generator(device=dev).manual_seed(7)
        dy = torch.randn(m, half, generator=gd, device=dev).to(torch.bfloat16)
        out = torch.empty(m, k, dtype=E5, device=dev)
        out_t = torch.empty(pcs[-1], k, dtype=E5, device=dev) if mode.endswith("transpose") else None
        fn = lambda: backend.grouped_cast_transpose(dy, cums, out, out_t, pcs, (scale, 1), (amax, 1), in2=x, activation="swiglu")  # noqa: E731
        nbytes = 2 * m * half + 2 * m * k + m * k + (pcs[-1] * k if out_t is not None else 0)
    else:
        out = torch.empty(m, k, dtype=E4, device=dev)
        out_t = torch.empty(pcs[-1], k, dtype=E4, device=dev) if mode != "quantize" else None
        if mode == "cast":
            fn = lambda: backend.grouped_cast_transpose(x, cums, out, out_t, pcs, (scale, 1), (amax, 1))  # noqa: E731
            nbytes = 2 * m * k + m * k + pcs[-1] * k
        elif mode == "amax+cast":
            views = [x[cums[i]:cums[i + 1]] for i in range(G)]
            am = [amax[i] for i in range(G)]

            def fn():
                amax.zero_()
                backend.multi_amax(views, am)
                torch.div(448.0, torch.clamp(amax, min=1e-30), out=scale)
                backend.grouped_cast_transpose(x, cums, out, out_t, pcs, (scale, 1), None)

            nbytes = 2 * m * k + 2 * m * k + m * k + pcs[-1] * k
        elif mode == "transpose":
            fn = lambda: backend.grouped_cast_transpose(out, cums, None, out_t, pcs, None, None)  # noqa: E731
            nbytes = m * k + pcs[-1] * k
        else:
            views = [x[cums[i]:cums[i + 1]] for i in range(G)]
            outs = [out[cums[i]:cums[i + 1]] for i in range(G)]
            sc, am = [scale[i] for i in range(G)], [amax[i] for i in range(G)]
            fn = lambda: backend.multi_quantize(views, outs, sc, am)  # noqa: E731
            nbytes = 3 * m * k
    ms = time_ms(fn, iters, warmup)
    backend.device_status()
    gbs = nbytes / ms / 1e6
    return {"kernel": "multi_pad/" + mode, "clocks": LAST_CLOCKS, "groups": G, "rows": m, "padded_rows": pcs[-1], "cols": k, "ms": ms,
            "algorithmic_bytes": nbytes, "GBps": gbs, "frac_of_hbm_" + src: gbs / hbm, "frac_of_nominal_8000": gbs / 8000.0}


def pad_suite(backend, dev, groups=256, max_rows=4096, cols=7168, iters=5, warmup=2):
    """Every HBM-bound kernel family on the pad microbenchmark (256 groups, rows ~ U[0, 4096], K = 7168): one entry
    per op with its algorithmic bytes, GB/s and the fractions of the measured copy bandwidth and of 8 TB/s."""
    out = {}
    for mode in PAD_MODES:
        r = pad_case(backend, dev, groups, max_rows, cols, mode, iters, warmup)
        torch.cuda.empty_cache()
        out[mode] = {key: r[key] for key in r if key not in ("kernel", "clocks", "groups", "cols")}
    return out


def main():
    p = argparse.ArgumentParser()
    p.add_argument("what", choices=["gemm", "wgrad", "step-gemms", "pad", "scaled-mm", "library-step"])
    p.add_argument("--groups", type=int, default=None)
    p.add_argument("--rows", type=int, default=32768)
    p.add_argument("--n", type=int, default=4096)
    p.add_argument("--k", type=int, default=4096)
    p.add_argument("--act", default="none", choices=["none", "gelu", "swiglu"])
    p.add_argument("--a-format", default="e4m3", choices=["e4m3", "e5m2"])
    p.add_argument("--buffers", type=int, default=0, help="gemm: store the rows into this many buffers through a row map")
    p.add_argument("--max-rows", type=int, default=4096)
    p.add_argument("--cols", type=int, default=7168)
    p.add_argument("--mode", default="cast", choices=PAD_MODES)
    p.add_argument("--dataflow", default="native", choices=["native", "reference"],
                   help="step-gemms / wgrad: operands as the modules use them by default (forward weights for dgrad, "
                        "row-major activations for wgrad) or the reference's transposes")
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--warmup", type=int, default=3)
    args = p.parse_args()
    from fp8_gmm_b200 import backend

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if args.what == "gemm":
        sizes = even_sizes(args.groups or 8, args.rows)
        print(json.dumps(gemm_case(backend, dev, sizes, args.n, args.k, args.act, E4 if args.a_format == "e4m3" else E5,
                                   args.iters, args.warmup, "custom", buffers=args.buffers)))
    elif args.what == "scaled-mm":
        sizes = even_sizes(args.groups or 8, args.rows)
        print(json.dumps(scaled_mm_case(dev, sizes, args.n, args.k, args.iters, args.warmup, "custom")))
    elif args.what == "library-step":
        print(json.dumps(library_gemm_suite(backend, dev, even_sizes(8, 32768), args.iters, args.warmup)))
    elif args.what == "wgrad":
        sizes = even_sizes(args.groups or 8, args.rows)
        print(json.dumps(wgrad_case(backend, dev, sizes, args.n, args.k, args.iters, args.warmup, "custom",
                                    rowmajor=args.dataflow == "native")))
    elif args.what == "step-gemms":
        sizes, H, F = even_sizes(8, 32768), 4096, 14336
        nat = args.dataflow == "native"
        for label, fn in [
            ("fc1 fwd + SwiGLU epilogue", lambda: gemm_case(backend, dev, sizes, 2 * F, H, "swiglu", E4, args.iters, args.warmup, "fc1_fwd")),
            ("fc2 fwd", lambda: gemm_case(backend, dev, sizes, H, F, "none", E4, args.iters, args.warmup, "fc2_fwd")),
            ("fc2 dgrad", lambda: gemm_case(backend, dev, sizes, F, H, "none", E5, args.iters, args.warmup, "fc2_dgrad", nat)),
            ("fc1 dgrad", lambda: gemm_case(backend, dev, sizes, H, 2 * F, "none", E5, args.iters, args.warmup, "fc1_dgrad", nat)),
            ("fc2 wgrad", lambda: wgrad_case(backend, dev, sizes, H, F, args.iters, args.warmup, "fc2_wgrad", nat)),
            ("fc1 wgrad", lambda: wgrad_case(backend, dev, sizes, 2 * F, H, args.iters, args.warmup, "fc1_wgrad", nat)),
        ]:
            print(json.dumps(fn()), flush=True)
            torch.cuda.empty_cache()
    else:
        print(json.dumps(pad_case(backend, dev, args.groups or 256, args.max_rows, args.cols, args.mode, args.iters, args.warmup)))


if __name__ == "__main__":
    main()
