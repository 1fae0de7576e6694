"""Generate golden vectors from the reference's own CUDA kernels (run on a machine with a B200).

    python oracle/build_ref_kernels.py            # where the reference checkout is available
    python tests/golden/make_golden.py OUT_DIR    # on the GPU machine; copy OUT_DIR/*.npz to tests/golden/

Each file holds one small seeded case: the bf16 inputs (as uint16 bit patterns), the scale, and the bytes
the reference kernels produced for quantise, cast + padded transpose (+ amax), fp8 transpose, scale-mul
and the dGELU-fused cast (reference csrc/multi_pointwise.cu, csrc/multi_pad_fusion.cu compiled for
sm_100a by oracle/build_ref_kernels.py).  tests/test_oracle_pins.py checks the CPU oracle against them.
"""
import importlib.util
import glob
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

CASES = [  # (rows, cols, fp8 format, scale, seed); the committed fixtures are the cases below 100 KB
    (8, 8, 0, 1.0, 0), (33, 40, 0, 3.25, 1), (120, 208, 1, 0.4375, 2), (1, 321, 0, 17.0, 3),
    (233, 1, 1, 2.5, 4), (256, 256, 0, 61.7, 5), (148, 67, 1, 911.0, 6),
]


def load_ref():
    cands = glob.glob(os.path.join(ROOT, "oracle", "_ref", "ref_fp8_gmm_kernels*.so"))
    if not cands:
        raise SystemExit("oracle/_ref/ref_fp8_gmm_kernels*.so not found: run oracle/build_ref_kernels.py first")
    spec = importlib.util.spec_from_file_location("ref_fp8_gmm_kernels", cands[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__))
    os.makedirs(out_dir, exist_ok=True)
    ref = load_ref()
    dev = torch.device("cuda:0")
    u16 = lambda t: t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    u8 = lambda t: t.cpu().contiguous().view(torch.uint8).numpy()  # noqa: E731
    for rows, cols, fmt, scale, seed in CASES:
        dt = torch.float8_e4m3fn if fmt == 0 else torch.float8_e5m2
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(rows, cols, generator=g).mul(2.0).to(torch.bfloat16)
        pre = torch.randn(rows, cols, generator=g).to(torch.bfloat16)
        pr = (rows + 15) // 16 * 16
        dx, dpre = x.to(dev), pre.to(dev)
        sc = torch.tensor([scale], device=dev)
        quant = torch.empty(rows, cols, dtype=dt, device=dev)
        am_q = torch.zeros(1, device=dev)
        ref.multi_quantize([dx], [quant], [sc], [am_q])
        cast = torch.empty(rows, cols, dtype=dt, device=dev)
        cast_t = torch.empty(cols, pr, dtype=dt, device=dev)
        am = torch.zeros(1, device=dev)
        ref.multi_pad_cast_transpose([dx], [cast], [cast_t], [sc], [am])
        tr = torch.empty(cols, pr, dtype=dt, device=dev)
        ref.multi_pad_transpose([cast], [tr])
        sm = dx.clone()
        s1, s2 = torch.tensor([0.37], device=dev), torch.tensor([1.0 / scale], device=dev)
        ref.multi_scale_mul([sm], [s1], [s2])
        dg = torch.empty(rows, cols, dtype=dt, device=dev)
        dg_t = torch.empty(cols, pr, dtype=dt, device=dev)
        am_g = torch.zeros(1, device=dev)
        ref.multi_pad_cast_transpose_dgelu([dx], [dpre], [dg], [dg_t], [sc], [am_g])
        torch.cuda.synchronize()
        assert float(am_q) == float(am)
        np.savez_compressed(
            os.path.join(out_dir, f"ref_kernels_{rows}x{cols}_f{fmt}.npz"),
            x=u16(x), pre=u16(pre), scale=np.float32(scale), fmt=np.int32(fmt), padded_rows=np.int32(pr),
            quant=u8(quant), cast=u8(cast), cast_t=u8(cast_t), amax=np.float32(float(am)), transpose=u8(tr),
            s1=np.float32(0.37), s2=np.float32(float(s2)), scale_mul=u16(sm),
            dgelu_cast=u8(dg), dgelu_cast_t=u8(dg_t), dgelu_amax=np.float32(float(am_g)))
    print("wrote", len(CASES), "golden files to", out_dir)


if __name__ == "__main__":
    main()
