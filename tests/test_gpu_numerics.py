"""Numerical corner cases of the CUDA path against the fp32 oracle on the same rounded inputs.

* Both LayerNorms are computed in ways that could cancel when the mean is far larger than the spread (the input
  one with a subtract-the-mean second pass, the output one and the output gate folded around their GEMMs as
  rstd * (v W'^T - mean * rowsum(W')) + d): inputs with a large common offset and with large per-channel offsets.
* The intermediates left / right / tri are fp16: heavy-tailed activations with enlarged weights must neither
  produce infinities nor NaN (the packs saturate), and must stay within the stated bounds while the values fit.
* Tiny output weights (fp16 subnormal range after the 0.5 pre-scale), as right after a zero initialisation.
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from oracle import trimul_oracle as oracle
from tests.helpers import assert_module_parity, max_abs_split, params_to, rand_params

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _module(params, outgoing):
    m = mw.TriangleMultiplication(128, outgoing=outgoing, check_status=True)
    m.load_state_dict({k: v.clone() for k, v in params.items()})
    return m.to(DEV).to(torch.bfloat16).eval()


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("kind", ["common_offset_20", "channel_offsets_30", "channel_scales"])
def test_layernorm_folding_survives_large_means(kind, outgoing):
    N = 128
    g = torch.Generator().manual_seed(401)
    p = rand_params(41, ln_bias_scale=0.2)
    z = torch.randn(1, N, N, 128, generator=g)
    if kind == "common_offset_20":
        z = z + 20.0  # |mean| = 20 sigma for every position
    elif kind == "channel_offsets_30":
        z = z + (torch.rand(128, generator=g) * 60.0 - 30.0)  # per-channel offsets up to +-30: large spread AND mean
    else:
        z = z * (0.5 + 1.5 * torch.rand(128, generator=g)) * 8.0
    z = z.to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.1
    ref = oracle.trimul_forward_stages(z, p, mask, outgoing=outgoing)
    m = _module(p, outgoing)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    # z itself is large here (|z| up to ~30 -> bf16 spacing 2^-3), so the comparison that matters is the update
    got_upd = y.float().cpu() - z.float()
    ref_upd = ref.update
    assert torch.isfinite(y.float()).all()
    # y = bf16(z + u): the rounding of the sum hides u below the spacing of z; compare through the oracle's own
    # bf16-rounded output and, for the update, in units of that spacing
    ref_y = ref.out
    spacing = torch.exp2(torch.floor(torch.log2(ref_y.abs().clamp_min(1e-30))) - 7.0)
    err = (y.float().cpu() - ref_y).abs()
    worst = float((err / torch.maximum(spacing, torch.full_like(spacing, 3e-2 / 0.75))).max())
    print(f"[numerics] {kind} outgoing={outgoing}: rel={oracle.rel_frobenius(y.float().cpu(), ref_y):.3e} "
          f"worst error / max(bf16 spacing, 4e-2) = {worst:.3f}; update rel = {oracle.rel_frobenius(got_upd, ref_upd):.3e}")
    assert oracle.rel_frobenius(y.float().cpu(), ref_y) <= 5e-3
    assert worst <= 0.75  # three quarters of the output spacing (half from the final rounding)
    # the residual-free output isolates the update: same module, residual off
    m.residual = False
    with torch.no_grad():
        u = m(z.to(DEV), mask.to(DEV))
    rel_u = oracle.rel_frobenius(u.float().cpu(), ref_upd)
    lo, hi = max_abs_split(u.float().cpu(), ref_upd)
    print(f"[numerics] {kind} outgoing={outgoing}: update alone rel={rel_u:.3e} max_abs={max(lo, hi):.3e}")
    assert rel_u <= 1.2e-2, rel_u
    assert max(lo, hi) <= 3e-2


@pytest.mark.parametrize("outgoing", [True, False])
def test_heavy_tailed_activations_stay_finite_and_in_bounds(outgoing):
    """1 % of the entries of z are 30 x larger and the left / right projection weights are 128 x larger than the usual
    initialisation: |left|, |right| reach several hundred and |t| a few 1e5, i.e. t * 2^-4 uses about a third of
    the fp16 range - close to but inside it, where fp16 keeps its full relative precision."""
    N = 128
    g = torch.Generator().manual_seed(402)
    p = rand_params(42)
    for k in ("to_left.weight", "to_right.weight"):
        p[k] = (p[k].float() * 128.0).to(torch.bfloat16)
    z = torch.randn(1, N, N, 128, generator=g)
    spikes = torch.rand(1, N, N, 128, generator=g) < 0.01
    z = torch.where(spikes, z * 30.0, z).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.1
    ref = oracle.trimul_forward_stages(z, p, mask, outgoing=outgoing)
    print(f"[numerics] heavy tail: max|left|={float(ref.left.abs().max()):.1f} max|tri|={float(ref.tri.abs().max()):.1f}")
    m = _module(p, outgoing)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert 1e5 < float(ref.tri.abs().max()) < 1.0e6, "the case is meant to come close to the fp16 range of t * 2^-4"
    assert_module_parity(y, ref.out, z, f"heavy tail outgoing={outgoing}")


@pytest.mark.parametrize("outgoing", [True, False])
def test_out_of_range_intermediates_saturate_instead_of_poisoning(outgoing):
    """Weights 20000 x larger than usual push sigmoid(g) * p past 65504 in places. The reference's bf16 pipeline keeps
    such values; this path saturates them at +-65504 (documented in the header), and what matters is that no
    infinity or NaN appears: inf * 0 against a masked zero would turn whole rows and columns into NaN."""
    N = 64
    g = torch.Generator().manual_seed(403)
    p = rand_params(43)
    for k in ("to_left.weight", "to_right.weight"):
        p[k] = (p[k].float() * 20000.0).to(torch.bfloat16)
    z = (torch.randn(1, N, N, 128, generator=g) * 8.0).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.3
    ref = oracle.trimul_forward_stages(z, p, mask, outgoing=outgoing)
    assert float(ref.left.abs().max()) > 65504.0, "the case must actually leave the fp16 range"
    packed = F_.aligned_empty(F_.packed_bytes(), torch.device(DEV))
    F_.pack_weights(params_to(p, DEV), packed)
    left = torch.full((1, N, 128, N), float("nan"), dtype=torch.float16, device=DEV)
    right = torch.full_like(left, float("nan"))
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    F_.prologue(z.to(DEV), packed, left, right, st, token_mask=mask)
    F_.check_status(st, "prologue")
    assert torch.isfinite(left.float()).all() and torch.isfinite(right.float()).all()
    assert float(left.float().abs().max()) == 65504.0  # saturated, not infinite
    m = _module(p, outgoing)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert torch.isfinite(y.float()).all()


@pytest.mark.parametrize("scale", [1e-3, 1e-5])
def test_tiny_output_weights(scale):
    """to_out / to_gate entries of 1e-3 .. 1e-5 of the usual size (the module's two output linears start at zero, so
    early fine-tuning sees such values). fp16(0.5 W gamma) is then subnormal: the update is tiny and its absolute
    error must stay far below the output's bf16 spacing; the relative error of the update is reported."""
    N = 64
    g = torch.Generator().manual_seed(404)
    p = rand_params(44)
    for k in ("to_out.weight", "to_gate.weight"):
        p[k] = (p[k].float() * scale).to(torch.bfloat16)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    ref = oracle.trimul_forward_stages(z, p, None, outgoing=True)
    m = _module(p, True)
    m.residual = False
    with torch.no_grad():
        u = m(z.to(DEV), None)
    got = u.float().cpu()
    rel = oracle.rel_frobenius(got, ref.update)
    print(f"[numerics] tiny output weights x{scale:g}: |update| max {float(ref.update.abs().max()):.3e}, rel {rel:.3e}, "
          f"max abs err {oracle.max_abs(got, ref.update):.3e}")
    assert torch.isfinite(got).all()
    assert oracle.max_abs(got, ref.update) <= 1e-3 * max(scale / 1e-3, 1.0) * 3e-2
    if scale >= 1e-3:
        assert rel <= 2e-2
