"""Training path of the triangle update (every width and direction the forward serves): forward on the
library's kernels with the stage tensors kept, backward for the input and all ten parameters through
``b200_trimul_backward``.

The reference's backward is stages B1-B12 of ``docs/kernels/trimul/TRIMUL_STATUS.md:43-52`` (reference project): its
LayerNorm / projection gradients are CUDA kernels and its contraction gradients cuBLAS calls. Here all of it runs on
this library's kernels: the epilogue's backward, the four contraction-gradient products on the stage-2 kernels, the
prologue's backward per side, and the parameter-gradient reduction.

Saved for the backward: the input, the masks, the dropout scale and the forward's workspace (``left``, ``right``, ``tri``
as the stages wrote them); the normalised input, the projections and the gates are recomputed, as the reference does
(``docs/kernels/trimul/TRIMUL_STATUS.md:40-41``).
"""

from __future__ import annotations

from typing import Optional

import torch

from . import functional as F_

D = F_.D
_PARAM_KEYS = (
    "ln_pair.weight", "ln_pair.bias", "to_left.weight", "to_left_gate.weight", "to_right.weight", "to_right_gate.weight",
    "ln_out.weight", "ln_out.bias", "to_gate.weight", "to_out.weight",
)


class TriMulFunction(torch.autograd.Function):
    """``y = TriMulFunction.apply(z, token_mask, pair_mask, drop_scale, cfg, *params)``; ``cfg`` is a dict with
    ``outgoing``, ``eps_in``, ``eps_out``, ``residual``, ``biases``, ``check``; ``params`` in ``_PARAM_KEYS`` order."""

    @staticmethod
    def forward(ctx, z, token_mask, pair_mask, drop_scale, cfg, *params):
        B, N = int(z.shape[0]), int(z.shape[1])
        p = {k: v.detach() for k, v in zip(_PARAM_KEYS, params)}
        ws = F_.aligned_empty(F_.workspace_bytes(B, N, cfg["outgoing"], int(z.shape[3])), z.device)  # kept until the backward
        y = F_.trimul_forward(
            z.detach(), p, token_mask, outgoing=cfg["outgoing"], eps_in=cfg["eps_in"], eps_out=cfg["eps_out"],
            pair_mask=pair_mask, residual=cfg["residual"], biases=cfg["biases"], workspace=ws, check=cfg["check"],
            drop_scale=drop_scale,
        )
        ctx.save_for_backward(z, *params)
        ctx.ws, ctx.cfg = ws, cfg
        ctx.token_mask, ctx.pair_mask, ctx.drop_scale = token_mask, pair_mask, drop_scale
        return y

    @staticmethod
    @torch.no_grad()
    def backward(ctx, dy):
        z, *params = ctx.saved_tensors
        cfg = ctx.cfg
        if ctx.ws is None:
            raise RuntimeError("the forward's stage tensors were released by the first backward of this call "
                               "(a second backward through the same forward is not supported)")
        B, N = int(z.shape[0]), int(z.shape[1])
        dz, grads = F_.trimul_backward(
            dy.to(torch.bfloat16), z.detach(), {k: v.detach() for k, v in zip(_PARAM_KEYS, params)}, ctx.ws, ctx.token_mask,
            outgoing=cfg["outgoing"], eps_in=cfg["eps_in"], eps_out=cfg["eps_out"], pair_mask=ctx.pair_mask,
            residual=cfg["residual"], biases=cfg["biases"], drop_scale=ctx.drop_scale, check=cfg["check"],
        )
        ctx.ws = None
        out = [dz.to(z.dtype) if ctx.needs_input_grad[0] else None, None, None, None, None]
        for i, (k, prm) in enumerate(zip(_PARAM_KEYS, params)):
            out.append(grads[k].to(prm.dtype) if ctx.needs_input_grad[5 + i] else None)
        return tuple(out)


def trimul_train(z: torch.Tensor, params: dict, token_mask: Optional[torch.Tensor] = None, *,
                 outgoing: Optional[bool] = True,
                 eps_in: float = 1e-5, eps_out: float = 1e-5, pair_mask: Optional[torch.Tensor] = None,
                 residual: bool = True, biases: Optional[dict] = None, drop_scale: Optional[torch.Tensor] = None,
                 check: bool = False) -> torch.Tensor:
    """Differentiable forward: ``z`` [B, N, N, 128] bf16 (N a multiple of 8) and the ten parameters may require grad;
    ``outgoing=None`` is the bidirectional module (parameters of its wider shapes)."""
    cfg = {"outgoing": None if outgoing is None else bool(outgoing), "eps_in": float(eps_in), "eps_out": float(eps_out), "residual": bool(residual),
           "biases": biases, "check": bool(check)}
    return TriMulFunction.apply(z, token_mask, pair_mask, drop_scale, cfg, *[params[k] for k in _PARAM_KEYS])


_TRANSITION_KEYS = ("ln_in.weight", "ln_in.bias", "expand_a.weight", "expand_b.weight", "squeeze.weight")


class TransitionFunction(torch.autograd.Function):
    """``y = TransitionFunction.apply(x, cfg, *params)`` for the pair Transition; ``cfg``: ``eps``, ``residual``,
    ``check``; ``params`` in ``_TRANSITION_KEYS`` order. Nothing but the input is kept for the backward (the hidden
    activations are recomputed)."""

    @staticmethod
    def forward(ctx, x, cfg, *params):
        p = {k: v.detach() for k, v in zip(_TRANSITION_KEYS, params)}
        packed = F_.aligned_empty(F_.transition_packed_bytes(), x.device)
        status = torch.zeros(16, dtype=torch.int32, device=x.device)
        F_.transition_pack_weights(p, packed)
        y = F_.transition_forward(x.detach(), packed, status, eps=cfg["eps"], residual=cfg["residual"])
        if cfg["check"]:
            F_.check_status(status, "b200_transition_forward")
        ctx.save_for_backward(x, *params)
        ctx.cfg = cfg
        return y

    @staticmethod
    @torch.no_grad()
    def backward(ctx, dy):
        x, *params = ctx.saved_tensors
        cfg = ctx.cfg
        dx, grads = F_.transition_backward(dy.to(torch.bfloat16).contiguous(), x.detach(),
                                           {k: v.detach() for k, v in zip(_TRANSITION_KEYS, params)}, eps=cfg["eps"],
                                           residual=cfg["residual"], check=cfg["check"])
        out = [dx if ctx.needs_input_grad[0] else None, None]
        for i, (k, prm) in enumerate(zip(_TRANSITION_KEYS, params)):
            out.append(grads[k].to(prm.dtype) if ctx.needs_input_grad[2 + i] else None)
        return tuple(out)


def transition_train(x: torch.Tensor, params: dict, *, eps: float = 1e-5, residual: bool = True, check: bool = False):
    """Differentiable pair Transition: ``x`` [..., 128] bf16 contiguous and the five parameters may require grad."""
    cfg = {"eps": float(eps), "residual": bool(residual), "check": bool(check)}
    return TransitionFunction.apply(x, cfg, *[params[k] for k in _TRANSITION_KEYS])
