"""Host-side mirror of the reference module interface for the triangle multiplicative update.

``TriangleMultiplication`` keeps the constructor, ``forward(pair, mask)`` signature, parameter names and
``state_dict`` layout of ``miniworld_engine.modules.TriangleMultiplication`` as MiniWorld uses it
(``src/miniworld/blocks/msa_module.py:60-71,116-117``, ``src/miniworld/blocks/template.py:41-52,84-85``
in the reference project): parameters ``ln_pair.{weight,bias}``, ``to_left``, ``to_left_gate``,
``to_right``, ``to_right_gate``, ``ln_out.{weight,bias}``, ``to_gate``, ``to_out`` (all linears
bias-free, ``benchmarks/protenix_finetune/patch_engine.py:25-29,51``); the module returns
``pair + update`` (it owns the residual).  ``TriangleMultiplicationOutgoing`` / ``...Incoming`` are the
OpenFold-style names with ``forward(z, pair_mask)``.

``BidirectionalTriangleMultiplication`` is the single operator MiniWorld's own trunk builds
(``src/miniworld/modules/mini_pairformer.py:76-80``, ``src/miniworld/modules/mini_msa_module.py:104``): one input
LayerNorm, left / right of width 2h whose halves are contracted outgoing and incoming, one LayerNorm over the 2h
contracted channels, one gate, one residual (``docs/paper/supplement.tex:125-136``); same parameter names, wider
shapes.

In training mode with ``p_drop > 0`` the forward applies the row-shared dropout of the reference
(``x + drop_row(f(x))``: one keep-mask per (batch, column, channel), shared by all rows,
``src/miniworld/blocks/template.py:38-40``). Every module here is differentiable (:mod:`miniworld_b200.training`): the triangle updates (input and all ten
parameters) and the pair Transition (input and its five parameters).
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from . import functional as F_

D_SUPPORTED = 128

# reference name -> OpenFold / Protenix name (benchmarks/protenix_finetune/patch_engine.py:25-29)
OPENFOLD_ALIASES = {
    "ln_pair": "layer_norm_in",
    "to_left": "linear_a_p",
    "to_left_gate": "linear_a_g",
    "to_right": "linear_b_p",
    "to_right_gate": "linear_b_g",
    "ln_out": "layer_norm_out",
    "to_gate": "linear_g",
    "to_out": "linear_z",
}

_ACCEPTED_IMPLEMENTATIONS = {None, "b200", "miniworld", "miniworld_engine", "engine", "cuda"}


def to_openfold_state_dict(sd: dict) -> dict:
    """Rename reference keys (``to_left.weight`` ...) to OpenFold keys (``linear_a_p.weight`` ...)."""
    out = {}
    for k, v in sd.items():
        head, _, tail = k.partition(".")
        out[f"{OPENFOLD_ALIASES.get(head, head)}.{tail}"] = v
    return out


def from_openfold_state_dict(sd: dict) -> dict:
    """Inverse of :func:`to_openfold_state_dict`; OpenFold bias entries of the linears are rejected."""
    inv = {v: k for k, v in OPENFOLD_ALIASES.items()}
    out = {}
    for k, v in sd.items():
        head, _, tail = k.partition(".")
        name = inv.get(head, head)
        if tail == "bias" and not name.startswith("ln_"):
            raise KeyError(f"{k}: the reference layout has bias-free linears; pass biases explicitly via set_biases()")
        out[f"{name}.{tail}"] = v
    return out


class Fp32LayerNorm(nn.LayerNorm):
    """LayerNorm parameter holder whose affine parameters are pinned to fp32: ``module.to(torch.bfloat16)`` moves them
    between devices but never changes (or rounds) their values, like the reference's fp32-pinned LayerNorm
    (``src/miniworld/layers/primitives.py:86-88``). Only ``weight``, ``bias`` and ``eps`` are used; the
    normalisation itself runs inside the fused kernels."""

    def _apply(self, fn, recurse=True):
        def pinned(t):
            out = fn(t)
            if t.is_floating_point() and out.dtype != t.dtype:
                return t.to(device=out.device)  # follow the device, keep the fp32 values bit for bit
            return out

        return super()._apply(pinned, recurse)


class TriangleMultiplication(nn.Module):
    """Triangle multiplicative update on B200 kernels (forward and backward).

    ``forward(pair [B,N,N,d_pair] bf16, mask Bool[B,N] | None) -> pair + update`` (bf16).
    Linear weights may be bf16 or fp32 masters; LayerNorm affine parameters are kept in fp32 whatever
    ``.to(dtype)`` is applied to the module (``src/miniworld/layers/primitives.py:86-88``).
    ``ln_pair.eps`` / ``ln_out.eps`` are read at call time.
    """

    _bidirectional = False

    def __init__(
        self,
        d_pair: int,
        d_hidden: Optional[int] = None,
        outgoing: bool = True,
        implementation=None,
        p_drop: float = 0.0,
        residual: bool = True,
        check_status: bool = False,
    ):
        super().__init__()
        wide = 2 if self._bidirectional else 1
        d_hidden = d_pair if d_hidden is None else d_hidden
        # the kernels contract 128 channels per call of the contraction stage and take 128 or 64 input channels:
        #   d_pair 128, d_hidden 128 (either module);  d_pair 64 with d_hidden 128 (one direction: the template
        #   blocks of the Protenix harness, benchmarks/protenix_finetune/patch_engine.py:283-295);  d_pair 64 with
        #   d_hidden 64 (bidirectional: the (L, D) = (384, 64) case of the reference's validation,
        #   docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11)
        ok = (d_pair, d_hidden) == (D_SUPPORTED, D_SUPPORTED) or (d_pair, wide * d_hidden) == (64, D_SUPPORTED)
        if not ok:
            raise NotImplementedError(
                f"implemented widths: d_pair = d_hidden = {D_SUPPORTED}; d_pair = 64 with d_hidden = 128 (one direction) or "
                f"64 (bidirectional); got d_pair = {d_pair}, d_hidden = {d_hidden}"
            )
        if d_pair != D_SUPPORTED and p_drop > 0.0:
            raise NotImplementedError("the row-shared dropout of the training forward is only implemented for d_pair = 128")
        impl = getattr(implementation, "value", implementation)
        impl = impl.lower() if isinstance(impl, str) else impl
        if impl not in _ACCEPTED_IMPLEMENTATIONS:
            raise ValueError(f"implementation={implementation!r}: this module has exactly one backend (B200 CUDA kernels)")
        self.d_pair = d_pair
        self.d_hidden = d_hidden
        self.outgoing = bool(outgoing)
        self.p_drop = float(p_drop)
        self.residual = bool(residual)
        self.check_status = bool(check_status)
        self.ln_pair = Fp32LayerNorm(d_pair, eps=1e-5)
        self.to_left = nn.Linear(d_pair, wide * d_hidden, bias=False)
        self.to_left_gate = nn.Linear(d_pair, wide * d_hidden, bias=False)
        self.to_right = nn.Linear(d_pair, wide * d_hidden, bias=False)
        self.to_right_gate = nn.Linear(d_pair, wide * d_hidden, bias=False)
        self.ln_out = Fp32LayerNorm(wide * d_hidden, eps=1e-5)
        self.to_gate = nn.Linear(d_pair, d_pair, bias=False)
        self.to_out = nn.Linear(wide * d_hidden, d_pair, bias=False)
        # the reference initialises the two output linears to zero ("init='zero'")
        nn.init.zeros_(self.to_gate.weight)
        nn.init.zeros_(self.to_out.weight)
        self._biases: Optional[dict] = None
        self._workspace: Optional[torch.Tensor] = None
        self._wcache = None  # (key, validated parameter pointers); the values themselves are re-read every call

    # ------------------------------------------------------------------ dtype handling
    def _apply(self, fn, recurse=True):
        super()._apply(fn, recurse)  # the LayerNorm affine parameters stay fp32 (Fp32LayerNorm)
        self._workspace = None
        self._wcache = None
        return self

    def set_biases(self, biases: Optional[dict]) -> None:
        """Optional fp32[d] biases for the linears, keys ``to_left`` ... ``to_out`` (None = reference layout).

        They are not parameters and are not part of the ``state_dict`` (the reference module has none).
        """
        self._biases = None if not biases else dict(biases)
        self._wcache = None

    def _weights(self, device: torch.device):
        """Validated parameter pointers, rebuilt only when a parameter tensor was replaced, moved or re-typed."""
        params = self._params()
        key = tuple((v.data_ptr(), v.dtype, v.device, v.is_contiguous()) for v in params.values()) + (device,)
        if self._wcache is None or self._wcache[0] != key:
            self._wcache = (key, F_._Weights(params, self._biases, device, bidirectional=self._bidirectional,
                                             d_pair=self.d_pair))
        return self._wcache[1]

    def _params(self) -> dict:
        return {
            "ln_pair.weight": self.ln_pair.weight,
            "ln_pair.bias": self.ln_pair.bias,
            "to_left.weight": self.to_left.weight,
            "to_left_gate.weight": self.to_left_gate.weight,
            "to_right.weight": self.to_right.weight,
            "to_right_gate.weight": self.to_right_gate.weight,
            "ln_out.weight": self.ln_out.weight,
            "ln_out.bias": self.ln_out.bias,
            "to_gate.weight": self.to_gate.weight,
            "to_out.weight": self.to_out.weight,
        }

    def load_openfold_state_dict(self, sd: dict, strict: bool = True):
        return self.load_state_dict(from_openfold_state_dict(sd), strict=strict)

    def device_status(self) -> int:
        """Synchronise and return the device status word of the last forward: 0, or the 1xx code of a device-side wait
        that gave up (:func:`miniworld_b200.functional.check_status` raises on it)."""
        if self._workspace is None:
            return 0
        return F_.read_status(self._workspace[:64].view(torch.int32))

    def _direction(self):
        return None if self._bidirectional else self.outgoing

    def _make_drop_row_scale(self, pair: torch.Tensor, p: float) -> torch.Tensor:
        """Row-shared dropout scale [B, 1, N, C]: keep-mask / (1 - p), one draw per (batch, column, channel), shared by
        all rows (the reference's hook of the same name, ``scripts/check_trimul_module_reference.py:43,100-103``;
        tests replace it to fix the mask)."""
        B, N, C = pair.shape[0], pair.shape[2], pair.shape[3]
        keep = torch.rand(B, 1, N, C, device=pair.device) >= p
        return keep.to(torch.bfloat16) / (1.0 - p)

    def _get_workspace(self, B: int, N: int, device: torch.device) -> torch.Tensor:
        need = F_.workspace_bytes(B, N, self._direction(), self.d_pair)
        ws = self._workspace
        if ws is None or ws.device != device or ws.numel() < need:
            ws = F_.aligned_empty(need, device)
            self._workspace = ws
        return ws

    def _backward_supported(self) -> bool:
        return True  # every width the constructor accepts has a backward

    def _run(self, pair: torch.Tensor, token_mask, pair_mask) -> torch.Tensor:
        # the differentiable path is taken when the input requires grad, or in training mode when a parameter does
        train = torch.is_grad_enabled() and (
            pair.requires_grad or (self.training and any(q.requires_grad for q in self.parameters()))
        )
        if train and not self._backward_supported():
            if pair.requires_grad:
                raise NotImplementedError(
                    "backward is implemented for d_pair = d_hidden = 128 only: call under "
                    "torch.no_grad() or with an input that does not require grad"
                )
            train = False
        if pair.dim() != 4 or pair.shape[1] != pair.shape[2] or pair.shape[3] != self.d_pair:
            raise RuntimeError(f"pair must be [B, N, N, {self.d_pair}], got {tuple(pair.shape)}")
        if not pair.is_cuda:
            raise RuntimeError("pair must be a CUDA tensor: this module has no CPU implementation")
        in_dtype = pair.dtype
        if train:
            return self._run_train(pair, token_mask, pair_mask)
        z = pair.detach()
        if z.dtype != torch.bfloat16:
            z = z.to(torch.bfloat16)
        z = z.contiguous()
        B, N = int(z.shape[0]), int(z.shape[1])
        pad = (-N) % 8
        scale = None
        if self.training and self.p_drop > 0.0:
            scale = self._make_drop_row_scale(z, self.p_drop).to(device=z.device, dtype=torch.bfloat16)
            if pad:
                sp = scale.new_zeros(B, 1, N + pad, self.d_pair)
                sp[:, :, :N] = scale
                scale = sp
        if pad:
            # pad with masked tokens: masked rows/columns of left/right are zero, so the crop is exact
            zp = z.new_zeros(B, N + pad, N + pad, self.d_pair)
            zp[:, :N, :N] = z
            tm = torch.ones(B, N, dtype=torch.bool, device=z.device) if token_mask is None else token_mask.to(z.device) != 0
            tmp = torch.zeros(B, N + pad, dtype=torch.bool, device=z.device)
            tmp[:, :N] = tm
            pmp = None
            if pair_mask is not None:
                pmp = torch.zeros(B, N + pad, N + pad, dtype=torch.bool, device=z.device)
                pmp[:, :N, :N] = pair_mask.to(z.device) != 0
            z, token_mask, pair_mask = zp, tmp, pmp
        Np = N + pad
        with torch.no_grad():
            y = F_.trimul_forward(
                z,
                self._params(),
                token_mask,
                outgoing=self._direction(),
                eps_in=float(self.ln_pair.eps),
                eps_out=float(self.ln_out.eps),
                pair_mask=pair_mask,
                residual=self.residual,
                biases=self._biases,
                workspace=self._get_workspace(B, Np, z.device),
                check=self.check_status,
                weights=self._weights(z.device),
                drop_scale=scale,
            )
        if pad:
            y = y[:, :N, :N].contiguous()
        return y if in_dtype == torch.bfloat16 else y.to(in_dtype)

    def _run_train(self, pair: torch.Tensor, token_mask, pair_mask) -> torch.Tensor:
        """Differentiable forward (:mod:`miniworld_b200.training`): the stage tensors of this call are kept for the
        backward in a workspace of their own; padding, cropping and dtype casts are ordinary differentiable ops."""
        from .training import trimul_train

        in_dtype = pair.dtype
        z = pair if pair.dtype == torch.bfloat16 else pair.to(torch.bfloat16)
        z = z.contiguous()
        B, N = int(z.shape[0]), int(z.shape[1])
        pad = (-N) % 8
        scale = None
        if self.training and self.p_drop > 0.0:
            scale = self._make_drop_row_scale(z, self.p_drop).to(device=z.device, dtype=torch.bfloat16)
            if pad:
                scale = nn.functional.pad(scale, (0, 0, 0, pad))
            scale = scale.contiguous()
        if pad:
            z = nn.functional.pad(z, (0, 0, 0, pad, 0, pad))
            tm = torch.ones(B, N, dtype=torch.bool, device=z.device) if token_mask is None else token_mask.to(z.device) != 0
            token_mask = nn.functional.pad(tm, (0, pad))
            if pair_mask is not None:
                pair_mask = nn.functional.pad(pair_mask.to(z.device) != 0, (0, pad, 0, pad))
        y = trimul_train(
            z, self._params(), token_mask, outgoing=self._direction(), eps_in=float(self.ln_pair.eps),
            eps_out=float(self.ln_out.eps), pair_mask=pair_mask, residual=self.residual, biases=self._biases,
            drop_scale=scale, check=self.check_status,
        )
        if pad:
            y = y[:, :N, :N]
        return y if in_dtype == torch.bfloat16 else y.to(in_dtype)

    def forward(self, pair: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if mask is not None and mask.dim() != 2:
            raise RuntimeError(f"mask must be a token mask [B, N], got {tuple(mask.shape)}")
        return self._run(pair, mask, None)


class _OpenFoldStyle(TriangleMultiplication):
    """``forward(z, pair_mask)`` where ``pair_mask`` is None, a token mask [B,N] or a pair mask [B,N,N]."""

    _outgoing = True

    def __init__(self, d_pair: int = D_SUPPORTED, d_hidden: Optional[int] = None, residual: bool = True, **kw):
        kw.pop("outgoing", None)
        super().__init__(d_pair, d_hidden, outgoing=self._outgoing, residual=residual, **kw)

    def forward(self, z: torch.Tensor, pair_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if pair_mask is None or pair_mask.dim() == 2:
            return self._run(z, pair_mask, None)
        if pair_mask.dim() == 3:
            return self._run(z, None, pair_mask)
        raise RuntimeError(f"pair_mask must be [B,N] or [B,N,N], got {tuple(pair_mask.shape)}")


class TriangleMultiplicationOutgoing(_OpenFoldStyle):
    _outgoing = True


class TriangleMultiplicationIncoming(_OpenFoldStyle):
    _outgoing = False


class BidirectionalTriangleMultiplication(TriangleMultiplication):
    """Both directions in one operator: ``forward(pair [B,N,N,128] bf16, mask Bool[B,N] | None) -> pair + update``.

    Constructor as in the reference (``BidirectionalTriangleMultiplication(d_pair, implementation=..., p_drop=...)``,
    ``src/miniworld/modules/mini_pairformer.py:76-80``). Parameters: ``ln_pair`` [128]; ``to_left``, ``to_left_gate``,
    ``to_right``, ``to_right_gate`` [256, 128] (rows 0-127: outgoing half, rows 128-255: incoming half); ``ln_out``
    [256]; ``to_gate`` [128, 128]; ``to_out`` [128, 256].
    """

    _bidirectional = True

    def __init__(self, d_pair: int = D_SUPPORTED, d_hidden: Optional[int] = None, implementation=None, p_drop: float = 0.0,
                 residual: bool = True, check_status: bool = False):
        super().__init__(d_pair, d_hidden, outgoing=True, implementation=implementation, p_drop=p_drop,
                         residual=residual, check_status=check_status)


class Transition(nn.Module):
    """Pair transition ``x + squeeze(SiLU(expand_a(LN x)) * expand_b(LN x))`` on the B200 kernels (forward and backward).

    Mirrors ``miniworld_engine.modules.Transition(d, n=4, implementation=...)`` as MiniWorld's blocks build it
    (``src/miniworld/modules/mini_pairformer.py:81-84``; it owns its residual, ``:108``): parameters ``ln_in`` [d],
    ``expand_a`` / ``expand_b`` [n d, d], ``squeeze`` [d, n d], all linears bias-free
    (``benchmarks/protenix_finetune/patch_engine.py:35-37``). d = 128 and n = 4 are what the kernel takes.
    """

    def __init__(self, d: int = D_SUPPORTED, n: int = 4, implementation=None, residual: bool = True, check_status: bool = False):
        super().__init__()
        if d != D_SUPPORTED or n != 4:
            raise NotImplementedError(f"only d = {D_SUPPORTED}, n = 4 is implemented on this path (got d = {d}, n = {n})")
        impl = getattr(implementation, "value", implementation)
        impl = impl.lower() if isinstance(impl, str) else impl
        if impl not in _ACCEPTED_IMPLEMENTATIONS:
            raise ValueError(f"implementation={implementation!r}: this module has exactly one backend (B200 CUDA kernels)")
        self.d, self.n = d, n
        self.residual = bool(residual)
        self.check_status = bool(check_status)
        self.ln_in = Fp32LayerNorm(d, eps=1e-5)
        self.expand_a = nn.Linear(d, n * d, bias=False)
        self.expand_b = nn.Linear(d, n * d, bias=False)
        self.squeeze = nn.Linear(n * d, d, bias=False)
        nn.init.zeros_(self.squeeze.weight)  # the reference's final linears start at zero
        self._scratch = None

    def _apply(self, fn, recurse=True):
        super()._apply(fn, recurse)
        self._scratch = None
        return self

    def device_status(self) -> int:
        return 0 if self._scratch is None else F_.read_status(self._scratch[1])

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("input must be a CUDA tensor: this module has no CPU implementation")
        if x.shape[-1] != self.d:
            raise RuntimeError(f"input must be [..., {self.d}], got {tuple(x.shape)}")
        in_dtype = x.dtype
        # the differentiable path is taken when the input requires grad, or in training mode when a parameter does
        if torch.is_grad_enabled() and (x.requires_grad or (self.training and any(q.requires_grad for q in self.parameters()))):
            from .training import transition_train

            xb = (x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)).contiguous()
            params = {"ln_in.weight": self.ln_in.weight, "ln_in.bias": self.ln_in.bias, "expand_a.weight": self.expand_a.weight,
                      "expand_b.weight": self.expand_b.weight, "squeeze.weight": self.squeeze.weight}
            y = transition_train(xb, params, eps=float(self.ln_in.eps), residual=self.residual, check=self.check_status)
            return y if in_dtype == torch.bfloat16 else y.to(in_dtype)
        xb = x.detach()
        if xb.dtype != torch.bfloat16:
            xb = xb.to(torch.bfloat16)
        xb = xb.contiguous()
        if self._scratch is None or self._scratch[0].device != xb.device:
            self._scratch = (F_.aligned_empty(F_.transition_packed_bytes(), xb.device),
                             torch.zeros(16, dtype=torch.int32, device=xb.device))
        packed, status = self._scratch
        params = {"ln_in.weight": self.ln_in.weight, "ln_in.bias": self.ln_in.bias, "expand_a.weight": self.expand_a.weight,
                  "expand_b.weight": self.expand_b.weight, "squeeze.weight": self.squeeze.weight}
        with torch.no_grad():
            F_.transition_pack_weights(params, packed)  # packed in every call: a captured graph replays current weights
            y = F_.transition_forward(xb, packed, status, eps=float(self.ln_in.eps), residual=self.residual)
        if self.check_status:
            F_.check_status(status, "b200_transition_forward")
        return y if in_dtype == torch.bfloat16 else y.to(in_dtype)
