"""Shared helpers of the parity tests (the oracle is used only here, as the checker)."""

import torch

from oracle import trimul_oracle as oracle

REL_FRO_TOL = 5e-3  # relative Frobenius error of the module output, bf16 I/O
MAX_ABS_TOL = 3e-2  # max abs error of the module output, bf16 I/O
UPDATE_REL_TOL = 1.2e-2  # the update alone (y - z) is held to a looser, separately stated bound


def to_row_plane(x_bnnh: torch.Tensor) -> torch.Tensor:
    """[B, N, N, H] channel-last -> [B, N, H, N] row-plane (the GPU intermediate layout)."""
    return x_bnnh.permute(0, 1, 3, 2).contiguous()


def from_row_plane(x_bnhn: torch.Tensor) -> torch.Tensor:
    return x_bnhn.permute(0, 1, 3, 2).contiguous()


def params_to(params: dict, device) -> dict:
    return {k: v.to(device) for k, v in params.items()}


def rand_params(seed: int, dtype=torch.bfloat16, c: int = 128, ln_bias_scale: float = 0.02) -> dict:
    from miniworld_b200.synthetic import make_params

    g = torch.Generator().manual_seed(seed)
    p = make_params(g, c, c, dtype)
    if ln_bias_scale != 0.02:
        p["ln_pair.bias"] = p["ln_pair.bias"] * (ln_bias_scale / 0.02)
        p["ln_out.bias"] = p["ln_out.bias"] * (ln_bias_scale / 0.02)
    return p


def max_abs_split(y: torch.Tensor, ref: torch.Tensor) -> tuple[float, float]:
    """Worst absolute error where |ref| < 8 (the 3e-2 bound applies as stated) and where |ref| >= 8 (bf16 spacing of
    the reference value itself is 2^-4 or more there, so rounding alone costs up to 3.1e-2)."""
    err = (y - ref).abs()
    small = ref.abs() < 8.0
    lo = float(err[small].max()) if bool(small.any()) else 0.0
    hi = float(err[~small].max()) if bool((~small).any()) else 0.0
    return lo, hi


def assert_module_parity(y_gpu: torch.Tensor, y_ref: torch.Tensor, z: torch.Tensor, what: str = "", check_update: bool = True) -> None:
    y = y_gpu.detach().float().cpu()
    ref = y_ref.detach().float().cpu()
    zf = z.detach().float().cpu()
    assert torch.isfinite(y).all(), what
    rel = oracle.rel_frobenius(y, ref)
    upd = oracle.rel_frobenius(y - zf, ref - zf)
    lo, hi = max_abs_split(y, ref)
    print(f"[parity] {what}: rel_frobenius={rel:.3e} update_rel={upd:.3e} max_abs(|y|<8)={lo:.3e} max_abs(|y|>=8)={hi:.3e}")
    assert rel <= REL_FRO_TOL, (what, "rel_frobenius", rel)
    # max abs <= 3e-2. A bf16 output cannot meet that where the spacing of the reference value itself is
    # 2^-4 (|y| >= 8: rounding alone costs up to 3.1e-2); there the bound is 3/4 of the spacing.
    err = (y - ref).abs()
    spacing = torch.exp2(torch.floor(torch.log2(ref.abs().clamp_min(1e-30))) - 7.0)
    limit = torch.maximum(torch.full_like(err, MAX_ABS_TOL), 0.75 * spacing)
    worst = float((err - limit).max())
    assert worst <= 0.0, (what, "max_abs", float(err.max()), "excess over limit", worst)
    if check_update:  # meaningless where the update is smaller than the bf16 spacing of the output it is added to
        assert upd <= UPDATE_REL_TOL, (what, "update rel_frobenius", upd)
