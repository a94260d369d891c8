"""Functional entry points: torch tensors in, C-ABI kernels on the current CUDA stream, torch tensors out.

PyTorch is used only for device memory and streams. Every function raises ``RuntimeError`` when the
CUDA library is missing or a call fails; nothing here falls back to PyTorch arithmetic.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_size_t, c_void_p
from typing import Optional, Sequence

import torch

from . import _lib

D = 128  # d_pair = d_hidden supported by the kernels

WEIGHT_KEYS = ("to_left.weight", "to_left_gate.weight", "to_right.weight", "to_right_gate.weight", "to_gate.weight", "to_out.weight")
LN_KEYS = ("ln_pair.weight", "ln_pair.bias", "ln_out.weight", "ln_out.bias")
BIAS_ORDER = ("to_left", "to_left_gate", "to_right", "to_right_gate", "to_gate", "to_out")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this path has no CPU implementation")


def aligned_empty(nbytes: int, device: torch.device, align: int = 1024) -> torch.Tensor:
    """uint8 buffer of ``nbytes`` whose data pointer is ``align``-byte aligned."""
    raw = torch.empty(nbytes + align, dtype=torch.uint8, device=device)
    off = (-raw.data_ptr()) % align
    return raw[off : off + nbytes]


def _direction(outgoing: Optional[bool]) -> int:
    """True -> outgoing, False -> incoming, None -> the bidirectional module."""
    if outgoing is None:
        return _lib.BIDIRECTIONAL
    return _lib.OUTGOING if outgoing else _lib.INCOMING


def workspace_bytes(B: int, N: int, outgoing: Optional[bool] = True, d_pair: int = D) -> int:
    out = c_size_t(0)
    d_hidden = D if (d_pair == D or outgoing is not None) else 64
    rc = _lib.load().b200_trimul_workspace_bytes(B, N, d_pair, d_hidden, _direction(outgoing), ctypes.byref(out))
    _lib.check(rc, "b200_trimul_workspace_bytes")
    return int(out.value)


def workspace_layout(B: int, N: int) -> list[int]:
    arr = (c_size_t * 5)()
    rc = _lib.load().b200_trimul_workspace_layout(B, N, arr)
    _lib.check(rc, "b200_trimul_workspace_layout")
    return [int(v) for v in arr]


def packed_bytes() -> int:
    return int(_lib.load().b200_trimul_packed_bytes())


def as_mask_u8(mask: Optional[torch.Tensor], device: torch.device) -> Optional[torch.Tensor]:
    """Bool / integer / float mask -> contiguous uint8 (non-zero = valid) on ``device``."""
    if mask is None:
        return None
    m = mask.to(device)
    if m.dtype == torch.bool:
        return m.contiguous().view(torch.uint8)
    return (m != 0).contiguous().view(torch.uint8)


class _Weights:
    """Validated pointers of one parameter set (all weights in one dtype, LN affine fp32)."""

    def __init__(self, params: dict, biases: Optional[dict], device: torch.device, bidirectional: bool = False,
                 d_pair: int = D):
        self.bidirectional = bool(bidirectional)
        if d_pair not in (D, 64):
            raise RuntimeError(f"d_pair must be {D} or 64, got {d_pair}")
        self.d_pair = C = int(d_pair)
        # contracted channels in total: 128, except the 128-wide bidirectional module (128 per direction). With
        # d_pair = 64 that is d_hidden = 128 for one direction, or 64 per direction for the bidirectional module.
        wide = 2 * D if (bidirectional and C == D) else D
        self.d_hidden = D if (C == D or not bidirectional) else 64
        shapes = {"to_left.weight": (wide, C), "to_left_gate.weight": (wide, C), "to_right.weight": (wide, C),
                  "to_right_gate.weight": (wide, C), "to_gate.weight": (C, C), "to_out.weight": (C, wide),
                  "ln_pair.weight": (C,), "ln_pair.bias": (C,), "ln_out.weight": (wide,), "ln_out.bias": (wide,)}
        bias_len = {"to_left": wide, "to_left_gate": wide, "to_right": wide, "to_right_gate": wide, "to_gate": C, "to_out": C}
        ws = [params[k] for k in WEIGHT_KEYS]
        dt = ws[0].dtype
        if dt not in (torch.bfloat16, torch.float32):
            raise RuntimeError(f"linear weights must be bf16 or fp32, got {dt}")
        keep = []
        for k, w in zip(WEIGHT_KEYS, ws):
            _require_cuda(w, k)
            if w.dtype != dt:
                raise RuntimeError("all six linear weights must share one dtype")
            if tuple(w.shape) != shapes[k]:
                raise RuntimeError(f"{k}: expected shape {shapes[k]}, got {tuple(w.shape)} (d_pair = {C}, "
                                   f"{'bidirectional' if bidirectional else 'one direction'})")
            if not w.is_contiguous():
                # a silent .contiguous() copy would be cached by the caller and go stale after an in-place update
                raise RuntimeError(f"{k} must be contiguous (the kernels read the parameter's own storage on every call)")
            keep.append(w.detach())
        lns = []
        for k in LN_KEYS:
            v = params[k]
            _require_cuda(v, k)
            if tuple(v.shape) != shapes[k]:
                raise RuntimeError(f"{k}: expected shape {shapes[k]}, got {tuple(v.shape)}")
            if v.dtype != torch.float32 or not v.is_contiguous():
                raise RuntimeError(f"{k} must be a contiguous fp32 tensor (LayerNorm affine parameters stay fp32), got {v.dtype}")
            lns.append(v.detach())
        self.weights = keep
        self.lns = lns
        self.dtype_code = _lib.DTYPE_BF16 if dt == torch.bfloat16 else _lib.DTYPE_F32
        self.bias_tensors = None
        self.bias_array = None
        if biases:
            bt = []
            arr = (c_void_p * 6)()
            for i, k in enumerate(BIAS_ORDER):
                b = biases.get(k)
                if b is None:
                    bt.append(None)
                    arr[i] = None
                else:
                    bb = b.detach().to(device=device, dtype=torch.float32).contiguous()
                    if tuple(bb.shape) != (bias_len[k],):
                        raise RuntimeError(f"bias {k}: expected shape ({bias_len[k]},)")
                    bt.append(bb)
                    arr[i] = bb.data_ptr()
            self.bias_tensors = bt
            self.bias_array = arr


def _check_z(z: torch.Tensor, widths=(D,)) -> tuple[int, int]:
    _require_cuda(z, "pair tensor")
    if z.dtype != torch.bfloat16:
        raise RuntimeError(f"pair tensor must be bf16, got {z.dtype}")
    if z.dim() != 4 or z.shape[3] not in widths:
        raise RuntimeError(f"pair tensor must be [B, rows, N, {' or '.join(str(w) for w in widths)}], got {tuple(z.shape)}")
    if not z.is_contiguous():
        raise RuntimeError("pair tensor must be contiguous")
    return int(z.shape[0]), int(z.shape[2])


def pack_weights(params: dict, packed: torch.Tensor, biases: Optional[dict] = None) -> None:
    w = _Weights(params, biases, packed.device)
    with torch.cuda.device(packed.device):
        rc = _lib.load().b200_trimul_pack_weights(
            *[_ptr(t) for t in w.weights[:4]],
            _ptr(w.weights[4]),
            _ptr(w.weights[5]),
            w.dtype_code,
            *[_ptr(t) for t in w.lns],
            w.bias_array,
            _ptr(packed),
            _stream(packed.device),
        )
    _lib.check(rc, "b200_trimul_pack_weights")


def pack_weights_bidir(params: dict, packed_out: torch.Tensor, packed_in: torch.Tensor, biases: Optional[dict] = None) -> None:
    """Pack the bidirectional module's parameters into the two blocks stage 1 (per direction) and stage 3 read."""
    w = _Weights(params, biases, packed_out.device, bidirectional=True)
    with torch.cuda.device(packed_out.device):
        rc = _lib.load().b200_trimul_pack_weights_bidir(
            *[_ptr(t) for t in w.weights[:4]], _ptr(w.weights[4]), _ptr(w.weights[5]), w.dtype_code,
            *[_ptr(t) for t in w.lns], w.bias_array, _ptr(packed_out), _ptr(packed_in), _stream(packed_out.device),
        )
    _lib.check(rc, "b200_trimul_pack_weights_bidir")


def epilogue_wide(
    tri: torch.Tensor,
    tri_in: Optional[torch.Tensor],
    z: torch.Tensor,
    packed: torch.Tensor,
    packed_in: Optional[torch.Tensor],
    y: torch.Tensor,
    status: torch.Tensor,
    drop_scale: Optional[torch.Tensor] = None,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    residual: bool = True,
) -> None:
    """Stage 3, general form: LayerNorm over [tri] (128 channels) or [tri, tri_in] (256), optional dropout scale."""
    B, N = _check_z(z)
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_epilogue_wide(
            _ptr(tri), _ptr(tri_in), _ptr(z), _ptr(packed), _ptr(packed_in), _ptr(drop_scale), _ptr(y), B, N,
            int(z.shape[1]), float(eps_in), float(eps_out), int(bool(residual)), _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_epilogue_wide")


def prologue(
    z: torch.Tensor,
    packed: torch.Tensor,
    left: torch.Tensor,
    right: torch.Tensor,
    status: torch.Tensor,
    token_mask: Optional[torch.Tensor] = None,
    pair_mask: Optional[torch.Tensor] = None,
    row_begin: int = 0,
    eps_in: float = 1e-5,
    has_bias: bool = False,
) -> None:
    """``z`` holds pair rows row_begin .. row_begin+rows-1: [B, rows, N, 128]; writes left/right [B, rows, 128, N]."""
    B, N = _check_z(z)
    rows = int(z.shape[1])
    tm = as_mask_u8(token_mask, z.device)
    pm = as_mask_u8(pair_mask, z.device)
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_prologue(
            _ptr(z), _ptr(packed), _ptr(tm), _ptr(pm), _ptr(left), _ptr(right), B, N, row_begin, rows, float(eps_in),
            int(bool(has_bias)), _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_prologue")


def _ptr_array(tensors):
    arr = (ctypes.c_void_p * max(len(tensors), 1))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


def prologue_push(
    z: torch.Tensor,
    packed: torch.Tensor,
    left: torch.Tensor,
    right_all: torch.Tensor,
    right_all_peers: list,
    status: torch.Tensor,
    token_mask: Optional[torch.Tensor] = None,
    row_begin: int = 0,
    eps_in: float = 1e-5,
    has_bias: bool = False,
) -> None:
    """Stage 1 for the rows ``z`` [1, rows, N, 128] of one GPU of a row-sharded run: ``left`` [1, rows, 128, N] stays
    local, ``right`` goes to rows row_begin.. of ``right_all`` [1, N, 128, N] and of every tensor in
    ``right_all_peers`` (the other GPUs' gathered copies, mapped into this process)."""
    B, N = _check_z(z)
    if B != 1:
        raise RuntimeError("prologue_push is the row-sharded form: B must be 1")
    rows = int(z.shape[1])
    tm = as_mask_u8(token_mask, z.device)
    peers = _ptr_array(right_all_peers)
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_prologue_push(
            _ptr(z), _ptr(packed), _ptr(tm), None, _ptr(left), _ptr(right_all), peers, len(right_all_peers), N, row_begin,
            rows, float(eps_in), int(bool(has_bias)), _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_prologue_push")


def reduce_partials(tri: torch.Tensor, partials: list, N: int, row_begin: int, rows: int) -> None:
    """``tri`` [1, rows, 128, N] = sum of rows row_begin.. of every ``partials[s]`` [1, N, 128, N] (local or peer memory)."""
    srcs = _ptr_array(partials)
    with torch.cuda.device(tri.device):
        rc = _lib.load().b200_trimul_reduce_partials(_ptr(tri), srcs, len(partials), N, row_begin, rows, _stream(tri.device))
    _lib.check(rc, "b200_trimul_reduce_partials")


def contract(
    left: torch.Tensor,
    right: torch.Tensor,
    tri: torch.Tensor,
    status: torch.Tensor,
    B: int,
    N: int,
    row_begin: int,
    rows: int,
    outgoing: bool,
) -> None:
    with torch.cuda.device(tri.device):
        rc = _lib.load().b200_trimul_contract(
            _ptr(left), _ptr(right), _ptr(tri), B, N, row_begin, rows, _lib.OUTGOING if outgoing else _lib.INCOMING,
            _ptr(status), _stream(tri.device),
        )
    _lib.check(rc, "b200_trimul_contract")


def contract_backward(
    dtri: torch.Tensor, left: torch.Tensor, right: torch.Tensor, dleft: torch.Tensor, dright: torch.Tensor,
    status: torch.Tensor, B: int, N: int, outgoing: bool,
) -> None:
    """Gradients of the contraction with respect to ``left`` and ``right`` (all [B, N, 128, N] fp16): ``dleft`` and
    ``dright`` receive the sums times 2^-4, saturated, in whatever scale ``dtri`` carries."""
    for name, t in (("dtri", dtri), ("left", left), ("right", right), ("dleft", dleft), ("dright", dright)):
        _require_cuda(t, name)
        if t.dtype != torch.float16 or tuple(t.shape) != (B, N, D, N) or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous fp16 [B, N, {D}, N] tensor, got {t.dtype} {tuple(t.shape)}")
    with torch.cuda.device(dtri.device):
        rc = _lib.load().b200_trimul_contract_backward(
            _ptr(dtri), _ptr(left), _ptr(right), _ptr(dleft), _ptr(dright), B, N,
            _lib.OUTGOING if outgoing else _lib.INCOMING, _ptr(status), _stream(dtri.device),
        )
    _lib.check(rc, "b200_trimul_contract_backward")


def contract_partial(
    left: torch.Tensor, right: torch.Tensor, tri_partial: torch.Tensor, status: torch.Tensor, B: int, N: int, k_rows: int
) -> None:
    """Incoming-direction partial sum over the ``k_rows`` pair rows held in ``left`` / ``right`` ([B, k_rows, 128, N]):
    ``tri_partial`` [B, N, 128, N] covers every (i, j); the partials of all row slabs add up to the full ``tri``."""
    with torch.cuda.device(tri_partial.device):
        rc = _lib.load().b200_trimul_contract_partial(
            _ptr(left), _ptr(right), _ptr(tri_partial), B, N, k_rows, _ptr(status), _stream(tri_partial.device)
        )
    _lib.check(rc, "b200_trimul_contract_partial")


def epilogue(
    tri: torch.Tensor,
    z: torch.Tensor,
    packed: torch.Tensor,
    y: torch.Tensor,
    status: torch.Tensor,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    residual: bool = True,
) -> None:
    B, N = _check_z(z)
    rows = int(z.shape[1])
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_epilogue(
            _ptr(tri), _ptr(z), _ptr(packed), _ptr(y), B, N, rows, float(eps_in), float(eps_out), int(bool(residual)),
            _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_epilogue")


def prologue_channels(
    z: torch.Tensor,
    packed: torch.Tensor,
    left_groups: list,
    right_groups: list,
    status: torch.Tensor,
    token_mask: Optional[torch.Tensor] = None,
    row_begin: int = 0,
    eps_in: float = 1e-5,
    has_bias: bool = False,
) -> None:
    """Stage 1 of the channel-sharded form for the rows ``z`` [1, rows, N, 128]: channel group g of ``left`` / ``right``
    goes to rows row_begin.. of ``left_groups[g]`` / ``right_groups[g]`` ([1, N, 128/P, N], on the GPU that contracts
    group g; peer memory for the other GPUs)."""
    B, N = _check_z(z)
    if B != 1 or len(left_groups) != len(right_groups):
        raise RuntimeError("prologue_channels: B must be 1 and both outputs need one buffer per channel group")
    tm = as_mask_u8(token_mask, z.device)
    lg, rg = _ptr_array(left_groups), _ptr_array(right_groups)
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_prologue_channels(
            _ptr(z), _ptr(packed), _ptr(tm), lg, rg, len(left_groups), N, row_begin, int(z.shape[1]), float(eps_in),
            int(bool(has_bias)), _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_prologue_channels")


def contract_channels(
    left_group: torch.Tensor, right_group: torch.Tensor, tri_owners: list, group: int, status: torch.Tensor, N: int,
    outgoing: bool,
) -> None:
    """Stage 2 of the channel-sharded form on the GPU that owns channel group ``group``: ``left_group`` /
    ``right_group`` [1, N, 128/P, N]; rows s*N/P.. of the result go to slab ``group`` of ``tri_owners[s]``
    ([P, N/P, 128/P, N] on GPU s)."""
    owners = _ptr_array(tri_owners)
    with torch.cuda.device(left_group.device):
        rc = _lib.load().b200_trimul_contract_channels(
            _ptr(left_group), _ptr(right_group), owners, len(tri_owners), group, N,
            _lib.OUTGOING if outgoing else _lib.INCOMING, _ptr(status), _stream(left_group.device),
        )
    _lib.check(rc, "b200_trimul_contract_channels")


def epilogue_groups(
    tri_groups: torch.Tensor,
    z: torch.Tensor,
    packed: torch.Tensor,
    y: torch.Tensor,
    status: torch.Tensor,
    groups: int,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    residual: bool = True,
) -> None:
    """Stage 3 of the channel-sharded form: ``tri_groups`` [P, rows, 128/P, N] holds this GPU's rows, one slab per
    channel group."""
    B, N = _check_z(z)
    with torch.cuda.device(z.device):
        rc = _lib.load().b200_trimul_epilogue_groups(
            _ptr(tri_groups), _ptr(z), _ptr(packed), _ptr(y), N, int(z.shape[1]), groups, float(eps_in), float(eps_out),
            int(bool(residual)), _ptr(status), _stream(z.device),
        )
    _lib.check(rc, "b200_trimul_epilogue_groups")


def peer_barrier(flags: list, rank: int, epoch: int, status: torch.Tensor, timeout_ms: int = 2000) -> None:
    """Stream-ordered barrier between the GPUs of a run: ``flags[r]`` is GPU r's int32[8] flag array as mapped into this
    process (zeroed once), ``epoch`` grows by one per barrier. A wait that runs out records device code 106 in
    ``status`` (see :func:`check_status`) instead of hanging."""
    arr = _ptr_array(flags)
    dev = flags[rank].device
    with torch.cuda.device(dev):
        rc = _lib.load().b200_trimul_peer_barrier(arr, rank, len(flags), epoch, int(timeout_ms), _ptr(status), _stream(dev))
    _lib.check(rc, "b200_trimul_peer_barrier")


def read_status(status: torch.Tensor) -> int:
    """Synchronise the current stream and return the device status word (0 = ok)."""
    out = c_int(0)
    with torch.cuda.device(status.device):
        rc = _lib.load().b200_trimul_read_status(_ptr(status), _stream(status.device), ctypes.byref(out))
    _lib.check(rc, "b200_trimul_read_status")
    return int(out.value)


def check_status(status: torch.Tensor, what: str = "trimul") -> None:
    code = read_status(status)
    if code != 0:
        raise RuntimeError(f"{what}: {_lib.strerror(code)} [{code}]")


def trimul_forward(
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
    workspace: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    check: bool = False,
    weights: Optional["_Weights"] = None,
    drop_scale: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One module forward on one GPU. ``z`` [B,N,N,128] bf16; ``mask`` Bool[B,N] or None; returns ``out``.

    ``outgoing=None`` selects the bidirectional module (parameters of the wider shapes, see
    ``b200_trimul_forward_ex`` in the header). ``drop_scale`` [B,1,N,128] (or [B,N,128]) bf16 is the row-shared
    dropout scale of the training path: ``out = z + drop_scale * update``.

    ``workspace`` (uint8, 1024-aligned, at least :func:`workspace_bytes`) is allocated when not given.
    ``check=True`` synchronises and raises if a device-side wait gave up. ``weights`` is an already validated
    :class:`_Weights` of the same parameters (it only holds pointers: the values are packed on the GPU in every call).
    """
    B, N = _check_z(z, widths=(D, 64))
    if z.shape[1] != N:
        raise RuntimeError(f"pair tensor must be square in its token dims, got {tuple(z.shape)}")
    dev = z.device
    C = int(z.shape[3])
    w = weights if weights is not None else _Weights(params, biases, dev, bidirectional=outgoing is None, d_pair=C)
    if w.bidirectional != (outgoing is None) or w.d_pair != C:
        raise RuntimeError("the validated weights belong to another module kind (direction or width)")
    if C != D and drop_scale is not None:
        raise RuntimeError("the row-shared dropout scale is only implemented for d_pair = 128")
    ds = None
    if drop_scale is not None:
        _require_cuda(drop_scale, "drop_scale")
        if drop_scale.numel() != B * N * D or drop_scale.shape[-1] != D or drop_scale.shape[0] != B:  # d_pair = 128 here
            raise RuntimeError(f"drop_scale must be [B, 1, N, {D}] = ({B}, 1, {N}, {D}), got {tuple(drop_scale.shape)}")
        ds = drop_scale.detach().to(torch.bfloat16).contiguous()
    need = workspace_bytes(B, N, outgoing, C)
    if workspace is None:
        workspace = aligned_empty(need, dev)
    elif workspace.numel() * workspace.element_size() < need:
        raise RuntimeError(f"workspace too small: {workspace.numel() * workspace.element_size()} < {need}")
    if out is None:
        out = torch.empty_like(z)
    tm = as_mask_u8(mask, dev)
    pm = as_mask_u8(pair_mask, dev)
    if tm is not None and tuple(tm.shape) != (B, N):
        raise RuntimeError(f"token mask must be [B, N] = ({B}, {N}), got {tuple(tm.shape)}")
    if pm is not None and tuple(pm.shape) != (B, N, N):
        raise RuntimeError(f"pair mask must be [B, N, N], got {tuple(pm.shape)}")
    with torch.cuda.device(dev):
        rc = _lib.load().b200_trimul_forward_ex(
            _ptr(z),
            *[_ptr(t) for t in w.weights],
            w.dtype_code,
            *[_ptr(t) for t in w.lns],
            w.bias_array,
            _ptr(tm),
            _ptr(pm),
            _ptr(ds),
            _ptr(out),
            _ptr(workspace),
            workspace.numel() * workspace.element_size(),
            B,
            N,
            C,
            w.d_hidden,
            _direction(outgoing),
            float(eps_in),
            float(eps_out),
            int(bool(residual)),
            _stream(dev),
        )
    _lib.check(rc, "b200_trimul_forward_ex")
    if check:
        check_status(workspace[:4].view(torch.int32), "b200_trimul_forward")
    return out


def backward_workspace_bytes(B: int, N: int, outgoing: Optional[bool] = True) -> int:
    out = c_size_t(0)
    _lib.check(_lib.load().b200_trimul_backward_workspace_bytes(B, N, _direction(outgoing), ctypes.byref(out)),
               "b200_trimul_backward_workspace_bytes")
    return int(out.value)


def trimul_backward(
    dy: torch.Tensor,
    z: torch.Tensor,
    params: dict,
    forward_workspace: torch.Tensor,
    mask: Optional[torch.Tensor] = None,
    *,
    outgoing: Optional[bool] = True,
    eps_in: float = 1e-5,
    eps_out: float = 1e-5,
    pair_mask: Optional[torch.Tensor] = None,
    residual: bool = True,
    biases: Optional[dict] = None,
    drop_scale: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    check: bool = False,
):
    """Backward of :func:`trimul_forward` (``b200_trimul_backward``) for every width the forward takes;
    ``outgoing=None`` is the bidirectional module.

    ``forward_workspace`` is the workspace the forward call used for the same inputs (it holds the stage tensors).
    Returns ``(dz bf16, the input's shape, grads)`` with ``grads`` a dict of fp32 tensors of the parameters' shapes under the
    parameter keys.
    """
    B, N = _check_z(z, widths=(D, 64))
    C = int(z.shape[3])
    if z.shape[1] != N:
        raise RuntimeError(f"pair tensor must be square in its token dims, got {tuple(z.shape)}")
    dev = z.device
    _require_cuda(dy, "dy")
    if dy.dtype != torch.bfloat16 or tuple(dy.shape) != tuple(z.shape):
        raise RuntimeError(f"dy must be bf16 of the input's shape {tuple(z.shape)}, got {dy.dtype} {tuple(dy.shape)}")
    dy = dy.contiguous()
    if not z.is_contiguous():
        raise RuntimeError("the pair tensor must be contiguous")
    bidir = outgoing is None
    w = _Weights(params, biases, dev, bidirectional=bidir, d_pair=C)
    if C != D and drop_scale is not None:
        raise RuntimeError("the row-shared dropout scale is only implemented for d_pair = 128")
    ds = None
    if drop_scale is not None:
        if drop_scale.numel() != B * N * D or drop_scale.shape[-1] != D or drop_scale.shape[0] != B:
            raise RuntimeError(f"drop_scale must be [B, 1, N, {D}], got {tuple(drop_scale.shape)}")
        ds = drop_scale.detach().to(device=dev, dtype=torch.bfloat16).contiguous()
    need = backward_workspace_bytes(B, N, outgoing)
    if workspace is None:
        workspace = aligned_empty(need, dev)
    elif workspace.numel() * workspace.element_size() < need:
        raise RuntimeError(f"workspace too small: {workspace.numel() * workspace.element_size()} < {need}")
    if forward_workspace.numel() * forward_workspace.element_size() < workspace_bytes(B, N, outgoing, C):
        raise RuntimeError("forward_workspace is smaller than the forward's workspace for this shape")
    tm = as_mask_u8(mask, dev)
    pm = as_mask_u8(pair_mask, dev)
    dz = torch.empty_like(z)
    wide = 2 * D if (bidir and C == D) else D  # contracted channels in total
    shapes = [(wide, C)] * 4 + [(C, C), (C, wide)]
    dws = [torch.empty(sh, dtype=torch.float32, device=dev) for sh in shapes]
    dln = [torch.empty(n, dtype=torch.float32, device=dev) for n in (C, C, wide, wide)]
    dw_arr = (c_void_p * 6)(*[t.data_ptr() for t in dws])
    with torch.cuda.device(dev):
        rc = _lib.load().b200_trimul_backward(
            _ptr(dy), _ptr(z), *[_ptr(t) for t in w.weights], w.dtype_code, *[_ptr(t) for t in w.lns], w.bias_array,
            _ptr(tm), _ptr(pm), _ptr(ds), _ptr(forward_workspace), _ptr(dz), dw_arr, *[_ptr(t) for t in dln],
            _ptr(workspace), workspace.numel() * workspace.element_size(), B, N, C, w.d_hidden, _direction(outgoing), float(eps_in),
            float(eps_out), int(bool(residual)), _stream(dev),
        )
    _lib.check(rc, "b200_trimul_backward")
    if check:
        check_status(workspace[:4].view(torch.int32), "b200_trimul_backward")
    grads = dict(zip(WEIGHT_KEYS, dws))
    grads.update(zip(LN_KEYS, dln))
    return dz, grads


# ------------------------------------------------------------------------------------------ pair Transition
TRANSITION_KEYS = ("ln_in.weight", "ln_in.bias", "expand_a.weight", "expand_b.weight", "squeeze.weight")


def transition_packed_bytes() -> int:
    return int(_lib.load().b200_transition_packed_bytes())


def transition_pack_weights(params: dict, packed: torch.Tensor) -> None:
    """Pack ``expand_a`` / ``expand_b`` [512, 128], ``squeeze`` [128, 512] (bf16 or fp32) and the fp32 LayerNorm
    affine into the block the transition kernel reads."""
    wa, wb, wsq = params["expand_a.weight"], params["expand_b.weight"], params["squeeze.weight"]
    g, b = params["ln_in.weight"], params["ln_in.bias"]
    dt = wa.dtype
    if dt not in (torch.bfloat16, torch.float32) or wb.dtype != dt or wsq.dtype != dt:
        raise RuntimeError("the three transition weights must share one dtype, bf16 or fp32")
    if tuple(wa.shape) != (4 * D, D) or tuple(wb.shape) != (4 * D, D) or tuple(wsq.shape) != (D, 4 * D):
        raise RuntimeError(f"transition weights must be [{4 * D},{D}], [{4 * D},{D}], [{D},{4 * D}] (d = {D}, n = 4 only)")
    for name, t in (("expand_a.weight", wa), ("expand_b.weight", wb), ("squeeze.weight", wsq), ("ln_in.weight", g), ("ln_in.bias", b)):
        _require_cuda(t, name)
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if g.dtype != torch.float32 or b.dtype != torch.float32 or tuple(g.shape) != (D,) or tuple(b.shape) != (D,):
        raise RuntimeError(f"ln_in.weight / ln_in.bias must be fp32[{D}]")
    with torch.cuda.device(packed.device):
        rc = _lib.load().b200_transition_pack_weights(
            _ptr(wa.detach()), _ptr(wb.detach()), _ptr(wsq.detach()), _lib.DTYPE_BF16 if dt == torch.bfloat16 else _lib.DTYPE_F32,
            _ptr(g.detach()), _ptr(b.detach()), _ptr(packed), _stream(packed.device),
        )
    _lib.check(rc, "b200_transition_pack_weights")


def transition_forward(x: torch.Tensor, packed: torch.Tensor, status: torch.Tensor, out: Optional[torch.Tensor] = None,
                       eps: float = 1e-5, residual: bool = True) -> torch.Tensor:
    """``y = x + squeeze(SiLU(expand_a(LN x)) * expand_b(LN x))`` for ``x`` [..., 128] bf16 (contiguous)."""
    _require_cuda(x, "transition input")
    if x.dtype != torch.bfloat16 or x.shape[-1] != D or not x.is_contiguous():
        raise RuntimeError(f"transition input must be a contiguous bf16 tensor [..., {D}], got {x.dtype} {tuple(x.shape)}")
    if out is None:
        out = torch.empty_like(x)
    positions = x.numel() // D
    with torch.cuda.device(x.device):
        rc = _lib.load().b200_transition_forward(_ptr(x), _ptr(packed), _ptr(out), positions, D, 4, float(eps),
                                                 int(bool(residual)), _ptr(status), _stream(x.device))
    _lib.check(rc, "b200_transition_forward")
    return out


def transition_backward(dy: torch.Tensor, x: torch.Tensor, params: dict, *, eps: float = 1e-5, residual: bool = True,
                        workspace: Optional[torch.Tensor] = None, check: bool = False):
    """Backward of the pair Transition (``b200_transition_backward``): ``dy``, ``x`` [..., 128] bf16 contiguous, ``params``
    under ``TRANSITION_KEYS``. Returns ``(dx bf16, grads)`` with fp32 gradients of the parameters' shapes."""
    for name, t in (("dy", dy), ("x", x)):
        _require_cuda(t, name)
        if t.dtype != torch.bfloat16 or t.shape[-1] != D or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous bf16 tensor [..., {D}], got {t.dtype} {tuple(t.shape)}")
    if tuple(dy.shape) != tuple(x.shape):
        raise RuntimeError("dy must have the input's shape")
    wa, wb, wsq = params["expand_a.weight"], params["expand_b.weight"], params["squeeze.weight"]
    g, b = params["ln_in.weight"], params["ln_in.bias"]
    dt = wa.dtype
    if dt not in (torch.bfloat16, torch.float32) or wb.dtype != dt or wsq.dtype != dt:
        raise RuntimeError("the three transition weights must share one dtype, bf16 or fp32")
    if tuple(wa.shape) != (4 * D, D) or tuple(wb.shape) != (4 * D, D) or tuple(wsq.shape) != (D, 4 * D):
        raise RuntimeError(f"transition weights must be [{4 * D},{D}], [{4 * D},{D}], [{D},{4 * D}] (d = {D}, n = 4 only)")
    for name, t in (("expand_a.weight", wa), ("expand_b.weight", wb), ("squeeze.weight", wsq), ("ln_in.weight", g), ("ln_in.bias", b)):
        _require_cuda(t, name)
        if not t.is_contiguous():
            raise RuntimeError(f"{name} must be contiguous")
    if g.dtype != torch.float32 or b.dtype != torch.float32:
        raise RuntimeError("the LayerNorm affine parameters must be fp32")
    dev = x.device
    positions = x.numel() // D
    need = c_size_t(0)
    _lib.check(_lib.load().b200_transition_backward_workspace_bytes(positions, ctypes.byref(need)),
               "b200_transition_backward_workspace_bytes")
    if workspace is None:
        workspace = aligned_empty(int(need.value), dev)
    elif workspace.numel() * workspace.element_size() < need.value:
        raise RuntimeError("workspace too small")
    dx = torch.empty_like(x)
    f32 = dict(dtype=torch.float32, device=dev)
    d_wa, d_wb, d_ws = torch.empty(4 * D, D, **f32), torch.empty(4 * D, D, **f32), torch.empty(D, 4 * D, **f32)
    d_g, d_b = torch.empty(D, **f32), torch.empty(D, **f32)
    with torch.cuda.device(dev):
        rc = _lib.load().b200_transition_backward(
            _ptr(dy), _ptr(x), _ptr(wa.detach()), _ptr(wb.detach()), _ptr(wsq.detach()),
            _lib.DTYPE_BF16 if dt == torch.bfloat16 else _lib.DTYPE_F32, _ptr(g.detach()), _ptr(b.detach()), _ptr(dx),
            _ptr(d_wa), _ptr(d_wb), _ptr(d_ws), _ptr(d_g), _ptr(d_b), _ptr(workspace),
            workspace.numel() * workspace.element_size(), positions, D, 4, float(eps), int(bool(residual)), _stream(dev),
        )
    _lib.check(rc, "b200_transition_backward")
    if check:
        check_status(workspace[:4].view(torch.int32), "b200_transition_backward")
    return dx, {"ln_in.weight": d_g, "ln_in.bias": d_b, "expand_a.weight": d_wa, "expand_b.weight": d_wb,
                "squeeze.weight": d_ws}
