"""Training path of the unidirectional triangle update: forward on the library's kernels with the stage tensors
kept, backward for the input and all ten parameters.

What runs where in the backward (the reference's split is the mirror image: its contraction gradients are cuBLAS calls
and its LayerNorm / projection gradients are CUDA kernels, ``docs/kernels/trimul/TRIMUL_STATUS.md:43-52`` in the
reference project):

* the four products of the contraction gradients (the dominant cost, 4 N^3 C multiply-adds) run on this library's
  stage-2 kernels (``b200_trimul_contract_backward``);
* the gradients through the two LayerNorms, the six linears, the sigmoid gates, the mask and the dropout scale are
  torch tensor expressions in fp32 on the GPU (library GEMMs and elementwise kernels), written out below.

Saved for the backward: the input, the masks, the dropout scale and the forward's workspace (``left``, ``right``, ``tri``
as the stages wrote them); the normalised input, the projections and the gates are recomputed, as the reference does
(``docs/kernels/trimul/TRIMUL_STATUS.md:40-41``).
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as tF

from . import _lib
from . import functional as F_

D = F_.D
_PARAM_KEYS = (
    "ln_pair.weight", "ln_pair.bias", "to_left.weight", "to_left_gate.weight", "to_right.weight", "to_right_gate.weight",
    "ln_out.weight", "ln_out.bias", "to_gate.weight", "to_out.weight",
)
_TRI_SCALE = 0.0625  # every contraction output of the library is stored times 2^-4


def _workspace_views(ws: torch.Tensor, B: int, N: int):
    """status, left, right, tri views of a forward workspace (``b200_trimul_workspace_layout``)."""
    arr = (ctypes.c_size_t * 5)()
    _lib.check(_lib.load().b200_trimul_workspace_layout(B, N, arr), "b200_trimul_workspace_layout")
    off = list(arr)
    nbytes = B * N * D * N * 2

    def plane(o):
        return ws[o : o + nbytes].view(torch.float16).view(B, N, D, N)

    return ws[off[0] : off[0] + 64].view(torch.int32), plane(off[2]), plane(off[3]), plane(off[4])


def _valid(token_mask, pair_mask, B, N, device):
    v = None
    if token_mask is not None:
        t = token_mask.to(device) != 0
        v = t[:, :, None] & t[:, None, :]
    if pair_mask is not None:
        pm = pair_mask.to(device) != 0
        v = pm if v is None else (v & pm)
    return v


def _ln_backward(dxh: torch.Tensor, xh: torch.Tensor, rstd: torch.Tensor) -> torch.Tensor:
    """Gradient through x_hat = (x - mean) * rstd over the last dimension, given d loss / d x_hat."""
    m1 = dxh.mean(-1, keepdim=True)
    m2 = (dxh * xh).mean(-1, keepdim=True)
    return rstd * (dxh - m1 - xh * m2)


def _normalise(x: torch.Tensor, eps: float):
    mean = x.mean(-1, keepdim=True)
    var = x.var(-1, unbiased=False, keepdim=True)
    rstd = torch.rsqrt(var + eps)
    return (x - mean) * rstd, rstd


class TriMulFunction(torch.autograd.Function):
    """``y = TriMulFunction.apply(z, token_mask, pair_mask, drop_scale, cfg, *params)``; ``cfg`` is a dict with
    ``outgoing``, ``eps_in``, ``eps_out``, ``residual``, ``biases``, ``check``; ``params`` in ``_PARAM_KEYS`` order."""

    @staticmethod
    def forward(ctx, z, token_mask, pair_mask, drop_scale, cfg, *params):
        if z.shape[3] != D:
            raise NotImplementedError("the backward is implemented for d_pair = d_hidden = 128")
        B, N = int(z.shape[0]), int(z.shape[1])
        p = {k: v.detach() for k, v in zip(_PARAM_KEYS, params)}
        ws = F_.aligned_empty(F_.workspace_bytes(B, N, cfg["outgoing"]), z.device)  # kept until the backward has run
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
        B, N = int(z.shape[0]), int(z.shape[1])
        status, left, right, tri = _workspace_views(ctx.ws, B, N)

        def contract_grad(dtri):
            dleft = torch.empty_like(left)
            dright = torch.empty_like(right)
            F_.contract_backward(dtri, left, right, dleft, dright, status, B, N, cfg["outgoing"])
            if cfg["check"]:
                F_.check_status(status, "contract_backward")
            return dleft, dright

        dz, grads = backward_core(z, params, cfg, ctx.token_mask, ctx.pair_mask, ctx.drop_scale, tri, dy, contract_grad)
        ctx.ws = None
        out = [dz.to(z.dtype) if ctx.needs_input_grad[0] else None, None, None, None, None]
        for i, (k, prm) in enumerate(zip(_PARAM_KEYS, params)):
            out.append(grads[k].to(prm.dtype) if ctx.needs_input_grad[5 + i] else None)
        return tuple(out)


def backward_core(z, params, cfg, token_mask, pair_mask, drop_scale, tri, dy, contract_grad):
    """The backward as tensor expressions around ``contract_grad(dtri fp16 [B,N,128,N]) -> (dleft, dright)`` (fp16,
    the sums times 2^-4). ``tri`` is the forward's stage-2 output (fp16, times 2^-4). Returns d loss / d z (fp32) and
    a dict of fp32 parameter gradients."""
    B, N = int(z.shape[0]), int(z.shape[1])
    dev = z.device
    f32 = torch.float32
    P = {k: v.detach().to(f32) for k, v in zip(_PARAM_KEYS, params)}
    bias = {k: v.detach().to(device=dev, dtype=f32) for k, v in (cfg["biases"] or {}).items()}

    # ---- recompute the epilogue's inputs
    xh, rstd_in = _normalise(z.to(f32), cfg["eps_in"])
    xn = xh * P["ln_pair.weight"] + P["ln_pair.bias"]
    t = tri.to(f32).permute(0, 1, 3, 2) * (1.0 / _TRI_SCALE)  # [B, i, j, h]
    th, rstd_out = _normalise(t, cfg["eps_out"])
    tn = th * P["ln_out.weight"] + P["ln_out.bias"]
    proj = tF.linear(tn, P["to_out.weight"], bias.get("to_out"))
    gate = torch.sigmoid(tF.linear(xn, P["to_gate.weight"], bias.get("to_gate")))
    du = dy.to(f32)
    if drop_scale is not None:
        du = du * drop_scale.to(f32).reshape(B, 1, N, D)
    # ---- epilogue gradients
    dproj = du * gate
    dgate = du * proj * gate * (1.0 - gate)
    flat = lambda a: a.reshape(-1, a.shape[-1])  # noqa: E731
    g_out = flat(dproj).t() @ flat(tn)
    g_gate = flat(dgate).t() @ flat(xn)
    dtn = dproj @ P["to_out.weight"]
    g_ln_out_w = (dtn * th).sum((0, 1, 2))
    g_ln_out_b = dtn.sum((0, 1, 2))
    dt = _ln_backward(dtn * P["ln_out.weight"], th, rstd_out)
    dxn = dgate @ P["to_gate.weight"]
    del proj, dproj, dgate, dtn, tn, th, t
    # ---- contraction gradients on the library's kernels: fp16 operands, so dt is brought to a power-of-two scale
    # that puts its largest magnitude near 64 (no host synchronisation: the scale stays on the device)
    amax = dt.abs().amax().clamp_min(1e-30)
    c = torch.exp2(torch.floor(torch.log2(64.0 / amax)))
    dtri = (dt * c).permute(0, 1, 3, 2).to(torch.float16).contiguous()
    del dt
    dleft, dright = contract_grad(dtri)
    unscale = (1.0 / _TRI_SCALE) / c
    dl = dleft.to(f32).permute(0, 1, 3, 2) * unscale  # [B, i, k, h]
    dr = dright.to(f32).permute(0, 1, 3, 2) * unscale
    del dtri, dleft, dright
    # ---- prologue gradients (projections and gates recomputed)
    valid = _valid(token_mask, pair_mask, B, N, dev)
    grads = {}
    for side, dside in (("left", dl), ("right", dr)):
        v = tF.linear(xn, P[f"to_{side}.weight"], bias.get(f"to_{side}"))
        s = torch.sigmoid(tF.linear(xn, P[f"to_{side}_gate.weight"], bias.get(f"to_{side}_gate")))
        if valid is not None:
            dside = dside * valid[..., None].to(f32)
        dv = dside * s
        dg = dside * v * s * (1.0 - s)
        grads[f"to_{side}.weight"] = flat(dv).t() @ flat(xn)
        grads[f"to_{side}_gate.weight"] = flat(dg).t() @ flat(xn)
        dxn = dxn + dv @ P[f"to_{side}.weight"] + dg @ P[f"to_{side}_gate.weight"]
        del v, s, dv, dg
    grads["ln_pair.weight"] = (dxn * xh).sum((0, 1, 2))
    grads["ln_pair.bias"] = dxn.sum((0, 1, 2))
    dz = _ln_backward(dxn * P["ln_pair.weight"], xh, rstd_in)
    if cfg["residual"]:
        dz = dz + dy.to(f32)
    grads["ln_out.weight"], grads["ln_out.bias"] = g_ln_out_w, g_ln_out_b
    grads["to_gate.weight"], grads["to_out.weight"] = g_gate, g_out
    return dz, grads


def trimul_train(z: torch.Tensor, params: dict, token_mask: Optional[torch.Tensor] = None, *, outgoing: bool = True,
                 eps_in: float = 1e-5, eps_out: float = 1e-5, pair_mask: Optional[torch.Tensor] = None,
                 residual: bool = True, biases: Optional[dict] = None, drop_scale: Optional[torch.Tensor] = None,
                 check: bool = False) -> torch.Tensor:
    """Differentiable forward: ``z`` [B, N, N, 128] bf16 (N a multiple of 8) and the ten parameters may require grad."""
    cfg = {"outgoing": bool(outgoing), "eps_in": float(eps_in), "eps_out": float(eps_out), "residual": bool(residual),
           "biases": biases, "check": bool(check)}
    return TriMulFunction.apply(z, token_mask, pair_mask, drop_scale, cfg, *[params[k] for k in _PARAM_KEYS])
