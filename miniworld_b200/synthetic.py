"""Seeded synthetic inputs for the triangle-multiplication forward path.

The reference benchmarks this module on ``randn`` pair tensors with synthetic token masks
(``scripts/benchmark_engine_h100.py:148-151`` in the reference project); no dataset is involved.
Every tensor is drawn on the CPU in fp32 from one ``torch.Generator`` in a fixed order, then
rounded to bf16 once where the workload is a bf16 one, so the CPU checker and the GPU kernels see
the same bytes.

Draw order (one generator): ln_pair.weight, ln_pair.bias, to_left, to_left_gate, to_right,
to_right_gate, ln_out.weight, ln_out.bias, to_gate, to_out, then per-channel scale (workload
"crop768" only), z, then mask randomness.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

D_PAIR = 128
D_HIDDEN = 128


@dataclass
class Workload:
    name: str
    z: torch.Tensor  # [B,N,N,C] bf16 (fp32 for the fp32 workload)
    mask: Optional[torch.Tensor]  # Bool[B,N] or None
    params: dict  # reference state_dict keys -> tensors (bf16 linears, fp32 LN affine)
    directions: tuple  # ("outgoing",) or ("outgoing", "incoming")
    B: int
    N: int


def make_params(gen: torch.Generator, c: int = D_PAIR, h: int = D_HIDDEN, dtype=torch.bfloat16) -> dict:
    """LayerNorm gamma = 1 + 0.1 N(0,1), beta = 0.02 N(0,1); linear weights ~ N(0, 1/fan_in)."""

    def rn(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32)

    p = {}
    p["ln_pair.weight"] = 1.0 + 0.1 * rn(c)
    p["ln_pair.bias"] = 0.02 * rn(c)
    p["to_left.weight"] = (rn(h, c) * c**-0.5).to(dtype)
    p["to_left_gate.weight"] = (rn(h, c) * c**-0.5).to(dtype)
    p["to_right.weight"] = (rn(h, c) * c**-0.5).to(dtype)
    p["to_right_gate.weight"] = (rn(h, c) * c**-0.5).to(dtype)
    p["ln_out.weight"] = 1.0 + 0.1 * rn(h)
    p["ln_out.bias"] = 0.02 * rn(h)
    p["to_gate.weight"] = (rn(c, c) * c**-0.5).to(dtype)
    p["to_out.weight"] = (rn(c, h) * h**-0.5).to(dtype)
    return p


WORKLOADS = {
    # name: (B, N, dtype, directions)
    "cpu128": (1, 128, torch.float32, ("outgoing",)),
    "n384": (1, 384, torch.bfloat16, ("outgoing", "incoming")),
    "crop768": (1, 768, torch.bfloat16, ("outgoing", "incoming")),
    "batch8x256": (8, 256, torch.bfloat16, ("outgoing", "incoming")),
    "complex2048": (1, 2048, torch.bfloat16, ("outgoing", "incoming")),
}


def make_workload(name: str, seed: int = 0, n_override: Optional[int] = None, b_override: Optional[int] = None) -> Workload:
    """Build one of the five benchmark workloads (optionally at a smaller N for CPU tests).

    cpu128       B1 N128 fp32, all-ones mask, outgoing only
    n384         B1 N384 bf16, last 38 tokens padded (10 %)
    crop768      B1 N768 bf16, z scaled per channel by U(0.5,2), each token masked w.p. 0.1
    batch8x256   B8 N256 bf16, per-sample valid length U{160..256}, tail padded
    complex2048  B1 N2048 bf16, 4 chains of N/4 tokens, 5 % of tokens masked
    """
    B, N, dtype, directions = WORKLOADS[name]
    if n_override is not None:
        N = int(n_override)
    if b_override is not None:
        B = int(b_override)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(seed)
    params = make_params(gen, dtype=dtype)
    C = D_PAIR
    scale = None
    if name == "crop768":
        scale = 0.5 + 1.5 * torch.rand(C, generator=gen, dtype=torch.float32)
    z = torch.randn(B, N, N, C, generator=gen, dtype=torch.float32)
    if scale is not None:
        z = z * scale
    z = z.to(dtype)

    if name == "cpu128":
        mask = torch.ones(B, N, dtype=torch.bool)
    elif name == "n384":
        mask = torch.ones(B, N, dtype=torch.bool)
        pad = max(1, round(N * 38 / 384))
        mask[:, N - pad :] = False
    elif name == "crop768":
        mask = torch.rand(B, N, generator=gen) >= 0.1
    elif name == "batch8x256":
        lo = max(1, round(N * 160 / 256))
        lengths = torch.randint(lo, N + 1, (B,), generator=gen)
        mask = torch.arange(N)[None, :] < lengths[:, None]
    elif name == "complex2048":
        mask = torch.rand(B, N, generator=gen) >= 0.05
    else:  # pragma: no cover
        raise KeyError(name)
    return Workload(name=name, z=z, mask=mask, params=params, directions=directions, B=B, N=N)


def cells(w: Workload) -> int:
    """Pair cells of one forward: B * N^2."""
    return w.B * w.N * w.N


def flops(B: int, N: int, c: int = D_PAIR, h: int = D_HIDDEN) -> dict:
    """Algorithmic FLOPs of one direction: contraction 2 B N^3 H, projections 2 B N^2 (4CH + C^2 + HC)."""
    contr = 2.0 * B * N**3 * h
    proj = 2.0 * B * N * N * (4 * c * h + c * c + h * c)
    return {"contraction": contr, "projection": proj, "total": contr + proj}


def pass_bytes(B: int, N: int, c: int = D_PAIR) -> int:
    """Bytes of one bf16 pair-tensor pass, P = B N^2 C 2."""
    return B * N * N * c * 2
