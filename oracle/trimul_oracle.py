"""CPU oracle for the triangle multiplicative update forward pass (TEST INFRASTRUCTURE ONLY).

This file is a checker. Only the tests, the smoke entry point and the CPU-baseline leg of the
benchmark may import it; the product package never does, and it is never the thing shipped or
measured on the GPU.

PARITY UNPINNED.  The arithmetic of the reference module lives in an un-vendored dependency of
MiniWorld (``miniworld-engine==2.4.4``, ``pyproject.toml:105``; class
``miniworld_engine.modules.triangle_multiplication.TriangleMultiplication``) whose source is not
in the reference tree and which cannot be installed offline.  The reference tree also stores no
tensors for this path.  This restatement therefore follows the published algorithm and the
reference's own descriptions of it, and is pinned only by the identities the reference tests
assert (all-invalid mask returns the input bit-exactly; the output gate is not masked) and by an
independent double-precision C restatement (``oracle/trimul_ref.c``).

What each step follows (paths inside the reference project):

* algorithm: ``docs/paper/supplement.tex:100-117`` (AF3 Alg. 12/13) and the maths block of
  ``docs/archive/trimul-fusion/history/initial-triton.py:11-26`` ("matches the PYTORCH ref");
* einsum strings: ``docs/archive/trimul-fusion/history/initial-triton.py:96-97``;
* mask: token mask ``m[b,i] & m[b,k]`` multiplies left/right only
  (``initial-triton.py:87-93``); the output gate uses the *unmasked* normalised input and the
  output is not masked (``docs/archive/trimul-fusion/f567-config/split_reference.py:17-18``);
* residual owned by the module: ``src/miniworld/blocks/msa_module.py:116-117`` (no external add);
* parameter set, all linears bias-free: ``benchmarks/protenix_finetune/patch_engine.py:25-29,51``;
* LayerNorm eps default 1e-5, fp32 affine: ``src/miniworld/layers/primitives.py:86-109``.

Optional biases (``None`` = the reference layout) exist because the benchmark configuration names
an OpenFold-style "gate biases = 1, projection biases = 0" variant.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

PARAM_KEYS = (
    "ln_pair.weight",
    "ln_pair.bias",
    "to_left.weight",
    "to_left_gate.weight",
    "to_right.weight",
    "to_right_gate.weight",
    "ln_out.weight",
    "ln_out.bias",
    "to_gate.weight",
    "to_out.weight",
)

BIAS_KEYS = ("to_left", "to_left_gate", "to_right", "to_right_gate", "to_gate", "to_out")


@dataclass
class Stages:
    """Intermediate tensors of one forward, channel-last, fp32."""

    x_hat: torch.Tensor  # LN_in(z)             [B,N,N,C]
    left: torch.Tensor  # masked left operand  [B,N,N,H]
    right: torch.Tensor  # masked right operand [B,N,N,H]
    tri: torch.Tensor  # contraction          [B,N,N,H]
    update: torch.Tensor  # gate * proj          [B,N,N,C]
    out: torch.Tensor  # z + update (or update when residual=False)


def _lin(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    return F.linear(x, w, b)


def pair_valid(
    mask: Optional[torch.Tensor], pair_mask: Optional[torch.Tensor], B: int, N: int
) -> Optional[torch.Tensor]:
    """Boolean [B,N,N] validity of each pair cell, or None when nothing is masked."""
    valid = None
    if mask is not None:
        m = mask.to(torch.bool)
        valid = m[:, :, None] & m[:, None, :]
    if pair_mask is not None:
        pm = pair_mask != 0
        valid = pm if valid is None else (valid & pm)
    return valid


def trimul_forward_stages(
    z: torch.Tensor,
    params: dict,
    mask: Optional[torch.Tensor] = None,
    *,
    outgoing: bool = True,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    pair_mask: Optional[torch.Tensor] = None,
    residual: bool = True,
    biases: Optional[dict] = None,
    round_intermediates: bool = False,
    k_chunk: int = 0,
    drop_scale: Optional[torch.Tensor] = None,
    differentiable: bool = False,
) -> Stages:
    """fp32 forward of TriangleMultiplication, returning every stage.

    ``differentiable`` keeps ``z`` and ``params`` attached to the autograd graph (they must then be fp32 leaves), so
    that ``out.backward(dy)`` gives the oracle's gradients: autograd through this restatement is the backward oracle,
    as the reference validates its backward against autograd through its PyTorch module
    (``docs/archive/engine2-validation-20260923/validate_bidir_reference.py:30-34``).

    ``z`` [B,N,N,C] (any float dtype; computed in fp32), ``mask`` Bool[B,N] or None, ``pair_mask``
    [B,N,N] (non-zero = valid) or None.  ``params`` uses the reference's state_dict keys.
    ``round_intermediates`` rounds left/right/tri to bf16 where the GPU pipeline stores them
    (used only to attribute error, never as the parity target).
    ``drop_scale`` [B,1,N,C] (row-shared dropout, keep-mask / (1 - p)) multiplies the update before the
    residual is added, as the training path does (``scripts/check_trimul_module_reference.py:43,114-116``
    in the reference project: a zero scale returns the input exactly).
    """
    keep = (lambda v: v.to(torch.float32)) if differentiable else (lambda v: v.detach().to(torch.float32))
    p = {k: keep(v) for k, v in params.items()}
    bz = {k: None for k in BIAS_KEYS}
    if biases:
        for k, v in biases.items():
            bz[k] = None if v is None else v.detach().to(torch.float32)
    zf = keep(z)
    B, N, N2, C = zf.shape
    assert N == N2
    H = p["to_left.weight"].shape[0]

    x = F.layer_norm(zf, (C,), p["ln_pair.weight"], p["ln_pair.bias"], eps_in)
    left = torch.sigmoid(_lin(x, p["to_left_gate.weight"], bz["to_left_gate"])) * _lin(
        x, p["to_left.weight"], bz["to_left"]
    )
    right = torch.sigmoid(_lin(x, p["to_right_gate.weight"], bz["to_right_gate"])) * _lin(
        x, p["to_right.weight"], bz["to_right"]
    )
    if round_intermediates:
        left = left.to(torch.bfloat16).to(torch.float32)
        right = right.to(torch.bfloat16).to(torch.float32)
    valid = pair_valid(mask, pair_mask, B, N)
    if valid is not None:
        m = valid[..., None].to(torch.float32)
        left = left * m
        right = right * m

    eq = "bikd,bjkd->bijd" if outgoing else "bkid,bkjd->bijd"
    if k_chunk and k_chunk < H:
        tri = torch.empty(B, N, N, H, dtype=torch.float32)
        for c0 in range(0, H, k_chunk):
            sl = slice(c0, min(H, c0 + k_chunk))
            tri[..., sl] = torch.einsum(eq, left[..., sl], right[..., sl])
    else:
        tri = torch.einsum(eq, left, right)
    if round_intermediates:
        tri = tri.to(torch.bfloat16).to(torch.float32)

    tn = F.layer_norm(tri, (H,), p["ln_out.weight"], p["ln_out.bias"], eps_out)
    proj = _lin(tn, p["to_out.weight"], bz["to_out"])
    gate = torch.sigmoid(_lin(x, p["to_gate.weight"], bz["to_gate"]))
    update = gate * proj
    if drop_scale is not None:
        update = update * drop_scale.detach().to(torch.float32)
    out = zf + update if residual else update
    return Stages(x_hat=x, left=left, right=right, tri=tri, update=update, out=out)


def trimul_forward(z, params, mask=None, **kw) -> torch.Tensor:
    """fp32 module output (``z + update`` by default); see :func:`trimul_forward_stages`."""
    return trimul_forward_stages(z, params, mask, **kw).out


def rel_frobenius(a: torch.Tensor, b: torch.Tensor) -> float:
    """||a - b||_F / ||b||_F in fp64 (the reference's metric, ``tests/test_engine_h100_masks.py:46-53``)."""
    a = a.detach().to(torch.float64)
    b = b.detach().to(torch.float64)
    return float((a - b).norm() / b.norm().clamp_min(1e-12))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.detach().to(torch.float64) - b.detach().to(torch.float64)).abs().max())


def trimul_forward_rows(
    z: torch.Tensor,
    params: dict,
    mask: Optional[torch.Tensor],
    rows,
    *,
    outgoing: bool = True,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    residual: bool = True,
    row_chunk: int = 64,
) -> torch.Tensor:
    """Module output for a few pair rows ``rows`` of a large problem (B = 1), fp32, without forming the whole
    contraction: left/right are built for every cell (O(N^2)) in row chunks, the O(N^3) step only for ``rows``.

    Same arithmetic as :func:`trimul_forward_stages`; used to check the N = 2048 workload at full size.
    Returns ``[len(rows), N, C]``.
    """
    p = {k: v.detach().to(torch.float32) for k, v in params.items()}
    assert z.shape[0] == 1
    N, C = z.shape[1], z.shape[3]
    H = p["to_left.weight"].shape[0]
    m = None if mask is None else mask[0].to(torch.bool)
    left = torch.empty(N, N, H, dtype=torch.float32)
    right = torch.empty(N, N, H, dtype=torch.float32)
    for r0 in range(0, N, row_chunk):
        zf = z[0, r0 : r0 + row_chunk].to(torch.float32)
        x = F.layer_norm(zf, (C,), p["ln_pair.weight"], p["ln_pair.bias"], eps_in)
        l = torch.sigmoid(x @ p["to_left_gate.weight"].T) * (x @ p["to_left.weight"].T)
        r = torch.sigmoid(x @ p["to_right_gate.weight"].T) * (x @ p["to_right.weight"].T)
        if m is not None:
            v = (m[r0 : r0 + row_chunk, None] & m[None, :])[..., None].to(torch.float32)
            l, r = l * v, r * v
        left[r0 : r0 + row_chunk] = l
        right[r0 : r0 + row_chunk] = r
    out = []
    for i in rows:
        if outgoing:
            tri = torch.einsum("kd,jkd->jd", left[i], right)  # t[i,j,d] = sum_k left[i,k,d] right[j,k,d]
        else:
            tri = torch.einsum("kd,kjd->jd", left[:, i], right)  # t[i,j,d] = sum_k left[k,i,d] right[k,j,d]
        zf = z[0, i].to(torch.float32)
        x = F.layer_norm(zf, (C,), p["ln_pair.weight"], p["ln_pair.bias"], eps_in)
        tn = F.layer_norm(tri, (H,), p["ln_out.weight"], p["ln_out.bias"], eps_out)
        upd = torch.sigmoid(x @ p["to_gate.weight"].T) * (tn @ p["to_out.weight"].T)
        out.append(zf + upd if residual else upd)
    return torch.stack(out)


def bidir_forward_stages(
    z: torch.Tensor,
    params: dict,
    mask: Optional[torch.Tensor] = None,
    *,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    pair_mask: Optional[torch.Tensor] = None,
    residual: bool = True,
    drop_scale: Optional[torch.Tensor] = None,
    differentiable: bool = False,
) -> Stages:
    """fp32 forward of BidirectionalTriangleMultiplication (``docs/paper/supplement.tex:125-136`` of the
    reference project; the module MiniWorld's trunk builds, ``src/miniworld/modules/mini_pairformer.py:76-80``).

    One input LayerNorm; ``to_left`` / ``to_left_gate`` / ``to_right`` / ``to_right_gate`` are [2h, C] and give
    l, r in R^{2h}; the first h channels are contracted outgoing (sum_k l_ik r_jk), the last h incoming
    (sum_k l_ki r_kj); one LayerNorm over the concatenated 2h channels, ``to_out`` [C, 2h], one gate
    ``to_gate`` [C, C] on the normalised input, residual included. Mask semantics as in the unidirectional
    module: the pair validity multiplies l and r only.
    """
    keep = (lambda v: v.to(torch.float32)) if differentiable else (lambda v: v.detach().to(torch.float32))
    p = {k: keep(v) for k, v in params.items()}
    zf = keep(z)  # differentiable: z and params stay attached to the autograd graph (the backward oracle)
    B, N, N2, C = zf.shape
    assert N == N2
    H2 = p["to_left.weight"].shape[0]
    assert H2 % 2 == 0
    h = H2 // 2
    x = F.layer_norm(zf, (C,), p["ln_pair.weight"], p["ln_pair.bias"], eps_in)
    left = torch.sigmoid(F.linear(x, p["to_left_gate.weight"])) * F.linear(x, p["to_left.weight"])
    right = torch.sigmoid(F.linear(x, p["to_right_gate.weight"])) * F.linear(x, p["to_right.weight"])
    valid = pair_valid(mask, pair_mask, B, N)
    if valid is not None:
        m = valid[..., None].to(torch.float32)
        left = left * m
        right = right * m
    tri_out = torch.einsum("bikd,bjkd->bijd", left[..., :h], right[..., :h])
    tri_in = torch.einsum("bkid,bkjd->bijd", left[..., h:], right[..., h:])
    tri = torch.cat([tri_out, tri_in], dim=-1)
    tn = F.layer_norm(tri, (H2,), p["ln_out.weight"], p["ln_out.bias"], eps_out)
    update = torch.sigmoid(F.linear(x, p["to_gate.weight"])) * F.linear(tn, p["to_out.weight"])
    if drop_scale is not None:
        update = update * drop_scale.detach().to(torch.float32)
    out = zf + update if residual else update
    return Stages(x_hat=x, left=left, right=right, tri=tri, update=update, out=out)


def bidir_forward(z, params, mask=None, **kw) -> torch.Tensor:
    return bidir_forward_stages(z, params, mask, **kw).out


TRANSITION_KEYS = ("ln_in.weight", "ln_in.bias", "expand_a.weight", "expand_b.weight", "squeeze.weight")


def transition_forward(x: torch.Tensor, params: dict, *, eps: float = 1e-5, residual: bool = True,
                       differentiable: bool = False) -> torch.Tensor:
    """fp32 forward of the pair Transition that follows the triangle update in every block
    (``src/miniworld/modules/mini_pairformer.py:81-84,108`` of the reference project):

        y = x + squeeze( SiLU(expand_a(LN(x))) * expand_b(LN(x)) )

    with ``expand_a`` / ``expand_b`` [n*C, C], ``squeeze`` [C, n*C], all bias-free, n = 4 (parameter names and the
    OpenFold/Protenix mapping layernorm1 / linear_no_bias_a / linear_no_bias_b / linear_no_bias:
    ``benchmarks/protenix_finetune/patch_engine.py:35-37``; the SwiGLU form h = SiLU(a) * b and the module-owned
    residual: ``scripts/render_transition_fusion.py:218,262`` and ``docs/h100-kernel-upgrade.md:14``). PARITY
    UNPINNED like the rest of this file: the module's source is in the same un-vendored wheel.
    """
    keep = (lambda v: v.to(torch.float32)) if differentiable else (lambda v: v.detach().to(torch.float32))
    p = {k: keep(v) for k, v in params.items()}
    xf = keep(x)  # differentiable: autograd through this restatement is the backward oracle
    C = xf.shape[-1]
    xn = F.layer_norm(xf, (C,), p["ln_in.weight"], p["ln_in.bias"], eps)
    hdn = F.silu(F.linear(xn, p["expand_a.weight"])) * F.linear(xn, p["expand_b.weight"])
    upd = F.linear(hdn, p["squeeze.weight"])
    return xf + upd if residual else upd
