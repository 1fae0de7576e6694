"""Shared fixtures for the parity tests: shapes of the reference's own tests and seeded inputs."""
import torch

# reference fp8_gmm/test.py:10-21: five tile-aligned and five ragged shapes
REF_SHAPES = [
    (2048, 12288), (768, 1024), (256, 65536), (65536, 128), (256, 256),
    (120, 2080), (8, 8), (1, 3221), (2333, 1), (1481, 677),
]
SMALL_SHAPES = [(768, 1024), (256, 256), (120, 2080), (8, 8), (1, 3221), (2333, 1), (1481, 677), (16, 16), (33, 40)]
FP8_DTYPES = [torch.float8_e4m3fn, torch.float8_e5m2]


def padded_rows(rows, padded):
    """reference fp8_gmm/test.py:23-30: last dim of the transpose rounded up to 16 when `padded`."""
    return rows + (16 - rows % 16) % 16 if padded else rows


def randn_bf16(shape, seed, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).to(torch.bfloat16)


def u8(t):
    return t.contiguous().view(torch.uint8)


def routed_group_sizes(num_groups, rows, seed, zipf_s=None):
    """Group sizes of a routed batch: multinomial over softmax(N(0,1)) logits, or Zipf(s) popularity."""
    g = torch.Generator().manual_seed(seed)
    if zipf_s is None:
        p = torch.softmax(torch.randn(num_groups, generator=g), 0)
    else:
        p = 1.0 / torch.arange(1, num_groups + 1, dtype=torch.float64) ** zipf_s
        p = (p / p.sum()).float()
    idx = torch.multinomial(p, rows, replacement=True, generator=g)
    return torch.bincount(idx, minlength=num_groups).tolist()


def fp8_steps(a, b):
    """Distance in representable FP8 steps between two byte tensors (sign-magnitude order, -0 == +0).

    The activation-fused kernels can produce a zero of either sign where the CPU evaluates the
    activation derivative to a zero of the other sign; as numbers they are identical."""
    def ordered(t):
        t = t.contiguous().view(torch.uint8).int()
        mag = t & 0x7F
        return torch.where(t >= 0x80, -mag, mag)
    return (ordered(a) - ordered(b)).abs()
