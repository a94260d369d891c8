"""BidirectionalTriangleMultiplication (the operator MiniWorld's trunk builds) and the row-shared dropout of the
training forward, against the fp32 CPU oracle on the same bf16-rounded inputs and weights.

Shapes, initialisation and the zero-gamma case follow the reference's own validation of this module
(docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11-38 in the reference project: L in
{384, 768}, weights N(0, 1/D), gamma = 1 + 0.1 N(0,1), every third gamma zero, random token mask, fixed dropout
scale); its tolerance there is 3e-2 relative L2, here the module bounds (5e-3 / 3e-2) apply.
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from oracle import trimul_oracle as oracle
from tests.helpers import assert_module_parity, rand_params

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bidir_params(seed, beta_scale=0.05):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return {
        "ln_pair.weight": 1.0 + 0.1 * rn(128), "ln_pair.bias": beta_scale * rn(128),
        "to_left.weight": (rn(256, 128) * 128**-0.5).to(torch.bfloat16),
        "to_left_gate.weight": (rn(256, 128) * 128**-0.5).to(torch.bfloat16),
        "to_right.weight": (rn(256, 128) * 128**-0.5).to(torch.bfloat16),
        "to_right_gate.weight": (rn(256, 128) * 128**-0.5).to(torch.bfloat16),
        "ln_out.weight": 1.0 + 0.1 * rn(256), "ln_out.bias": beta_scale * rn(256),
        "to_gate.weight": (rn(128, 128) * 128**-0.5).to(torch.bfloat16),
        "to_out.weight": (rn(128, 256) * 256**-0.5).to(torch.bfloat16),
    }


def _module(p, **kw):
    m = mw.BidirectionalTriangleMultiplication(128, check_status=True, **kw)
    m.load_state_dict({k: v.clone() for k, v in p.items()})
    return m.to(DEV).to(torch.bfloat16).eval()


def test_state_dict_layout():
    m = mw.BidirectionalTriangleMultiplication(128)
    sd = m.state_dict()
    assert list(sd) == ["ln_pair.weight", "ln_pair.bias", "to_left.weight", "to_left_gate.weight", "to_right.weight",
                        "to_right_gate.weight", "ln_out.weight", "ln_out.bias", "to_gate.weight", "to_out.weight"]
    assert sd["to_left.weight"].shape == (256, 128) and sd["to_out.weight"].shape == (128, 256)
    assert sd["ln_out.weight"].shape == (256,) and sd["to_gate.weight"].shape == (128, 128)


@pytest.mark.parametrize("N,mask_kind", [(64, "none"), (128, "holes"), (200, "random"), (384, "random")])
def test_bidirectional_matches_oracle(N, mask_kind):
    p = bidir_params(300 + N)
    g = torch.Generator().manual_seed(301 + N)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    mask = None
    if mask_kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    elif mask_kind == "random":
        mask = torch.rand(1, N, generator=g) > 0.2
    ref = oracle.bidir_forward(z, p, mask)
    with torch.no_grad():
        y = _module(p)(z.to(DEV), None if mask is None else mask.to(DEV))
    assert y.dtype == torch.bfloat16 and y.shape == z.shape
    assert_module_parity(y, ref, z, f"bidirectional N={N} mask={mask_kind}")


def test_bidirectional_large_crop_zero_gamma_and_batch():
    """L = 768 with every third gamma of both LayerNorms zero (the reference's hardest validation case), and a batch of
    two samples with different masks equal to the per-sample loop bit for bit."""
    p = bidir_params(310)
    p["ln_pair.weight"][::3] = 0
    p["ln_out.weight"][::3] = 0
    g = torch.Generator().manual_seed(311)
    N = 768
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.2
    ref = oracle.bidir_forward(z, p, mask)
    m = _module(p)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert_module_parity(y, ref, z, "bidirectional L=768 zero gamma")
    zb = torch.randn(2, 136, 136, 128, generator=g).to(torch.bfloat16).to(DEV)
    mb = (torch.rand(2, 136, generator=g) > 0.2).to(DEV)
    with torch.no_grad():
        yb = m(zb, mb)
        loop = torch.cat([m(zb[b : b + 1].contiguous(), mb[b : b + 1].contiguous()) for b in range(2)])
    assert torch.equal(yb, loop)


def test_bidirectional_identities_and_pair_mask_free_gate():
    """All tokens masked and beta_out = 0 returns the input exactly; the gate is not masked (non-zero beta_out shows an
    update at masked cells); mask None equals an all-true mask."""
    p = bidir_params(320, beta_scale=0.3)
    N = 64
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(321)).to(torch.bfloat16).to(DEV)
    m = _module(p)
    with torch.no_grad():
        a = m(z, None)
        b = m(z, torch.ones(1, N, dtype=torch.bool, device=DEV))
        masked = m(z, torch.zeros(1, N, dtype=torch.bool, device=DEV))
    assert torch.equal(a, b)
    assert float((masked.float() - z.float()).abs().max()) > 1e-3
    p0 = dict(p)
    p0["ln_out.bias"] = torch.zeros(256)
    with torch.no_grad():
        y0 = _module(p0)(z, torch.zeros(1, N, dtype=torch.bool, device=DEV))
    assert torch.equal(y0, z)


def test_direction_zero_through_the_c_abi_with_fp32_masters_and_biases():
    """`b200_trimul_forward` itself takes direction 0 (the engine's numbering) with fp32 master weights and biases of
    the wide shapes."""
    p = {k: (v.float() if k.startswith("to_") else v) for k, v in bidir_params(330).items()}
    N = 72
    g = torch.Generator().manual_seed(331)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.2
    biases = {"to_left_gate": torch.ones(256), "to_right_gate": torch.linspace(-1, 1, 256), "to_out": 0.1 * torch.randn(128, generator=g)}
    pf = {k: v.float() for k, v in p.items()}
    x = torch.nn.functional.layer_norm(z.float(), (128,), pf["ln_pair.weight"], pf["ln_pair.bias"], 1e-5)
    left = torch.sigmoid(x @ pf["to_left_gate.weight"].T + biases["to_left_gate"]) * (x @ pf["to_left.weight"].T)
    right = torch.sigmoid(x @ pf["to_right_gate.weight"].T + biases["to_right_gate"]) * (x @ pf["to_right.weight"].T)
    v = (mask[:, :, None] & mask[:, None, :])[..., None].float()
    left, right = left * v, right * v
    tri = torch.cat([torch.einsum("bikd,bjkd->bijd", left[..., :128], right[..., :128]),
                     torch.einsum("bkid,bkjd->bijd", left[..., 128:], right[..., 128:])], -1)
    tn = torch.nn.functional.layer_norm(tri, (256,), pf["ln_out.weight"], pf["ln_out.bias"], 1e-5)
    ref = z.float() + torch.sigmoid(x @ pf["to_gate.weight"].T) * (tn @ pf["to_out.weight"].T + biases["to_out"])
    y = F_.trimul_forward(z.to(DEV), {k: v.to(DEV) for k, v in p.items()}, mask.to(DEV), outgoing=None,
                          biases={k: v.to(DEV) for k, v in biases.items()}, check=True)
    assert_module_parity(y, ref, z, "direction 0, fp32 masters, biases")


@pytest.mark.parametrize("bidirectional", [False, True])
def test_training_forward_applies_row_shared_dropout(bidirectional):
    """Training mode with p_drop > 0: y = x + scale * update with one scale per (batch, column, channel) shared by all
    rows; a fixed scale is compared with the oracle, a zero scale returns the input exactly
    (scripts/check_trimul_module_reference.py:43,114-116 in the reference project), and there is no backward."""
    N = 104
    g = torch.Generator().manual_seed(340)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.2
    scale = ((torch.rand(2, 1, N, 128, generator=g) > 0.25).float() / 0.75).to(torch.bfloat16)
    if bidirectional:
        p = bidir_params(341)
        m = _module(p, p_drop=0.25)
        ref = oracle.bidir_forward(z, p, mask, drop_scale=scale)
    else:
        p = rand_params(342)
        m = mw.TriangleMultiplication(128, outgoing=False, p_drop=0.25, check_status=True)
        m.load_state_dict(p)
        m = m.to(DEV).to(torch.bfloat16)
        ref = oracle.trimul_forward(z, p, mask, outgoing=False, drop_scale=scale)
    m.train()
    m._make_drop_row_scale = lambda pair, pdrop: scale.to(DEV)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert_module_parity(y, ref, z, f"dropout forward bidirectional={bidirectional}")
    dropped = (scale == 0)[:, 0]  # [B, N, C]
    got_upd = (y.float().cpu() - z.float())
    assert bool((got_upd.permute(0, 2, 3, 1)[dropped] == 0).all()), "a dropped (column, channel) keeps the input in every row"
    m._make_drop_row_scale = lambda pair, pdrop: torch.zeros(2, 1, N, 128, dtype=torch.bfloat16, device=DEV)
    with torch.no_grad():
        y0 = m(z.to(DEV), mask.to(DEV))
    assert torch.equal(y0.cpu(), z)
    # the module's own draw: keep probability 1 - p, values 0 or 1 / (1 - p)
    del m._make_drop_row_scale
    s = m._make_drop_row_scale(z.to(DEV), 0.25)
    assert s.shape == (2, 1, N, 128)
    vals = torch.unique(s.float().cpu())
    keep_value = float(torch.tensor(1 / 0.75).to(torch.bfloat16))  # the scale is held in bf16
    assert set(vals.tolist()) <= {0.0, keep_value} and 0.6 < float((s != 0).float().mean()) < 0.9
    m.eval()
    with torch.no_grad():
        y_eval = m(z.to(DEV), mask.to(DEV))
    ref_eval = (oracle.bidir_forward if bidirectional else lambda *a, **k: oracle.trimul_forward(*a, outgoing=False, **k))(z, p, mask)
    assert_module_parity(y_eval, ref_eval, z, "eval mode ignores p_drop")


@pytest.mark.parametrize("B,N", [(1, 64), (2, 136), (1, 384)])
def test_wide_epilogue_on_one_tensor_agrees_with_the_epilogue_kernel(B, N):
    """The chunked epilogue kernel run on a single 128-channel tensor computes what `epilogue_kernel` computes; the
    two differ only in how the output statistics are split over threads, i.e. by rounding (at most one bf16 step on
    a small fraction of the outputs)."""
    p = rand_params(350, ln_bias_scale=0.2)
    g = torch.Generator().manual_seed(351 + N)
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    tri = ((torch.randn(B, N, 128, N, generator=g) * 3.0 + 0.7) * 0.0625).to(torch.float16).to(DEV)
    packed = F_.aligned_empty(F_.packed_bytes(), torch.device(DEV))
    F_.pack_weights({k: v.to(DEV) for k, v in p.items()}, packed)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    y_ref = torch.full_like(z, float("nan"))
    y_new = torch.full_like(z, float("nan"))
    F_.epilogue(tri, z, packed, y_ref, st, eps_in=0.03, eps_out=0.07)
    F_.epilogue_wide(tri, None, z, packed, None, y_new, st, eps_in=0.03, eps_out=0.07)
    F_.check_status(st, "epilogues")
    assert torch.isfinite(y_new.float()).all()
    diff = (y_new.float() - y_ref.float()).abs()
    # one bf16 step of the output where it is of order one (the update's own error is far below that)
    spacing = torch.exp2(torch.floor(torch.log2(y_ref.float().abs().clamp_min(1.0))) - 7.0)
    assert bool((diff <= spacing * 1.001).all()), float((diff / spacing).max())
    assert float((diff > 0).float().mean()) < 0.02
    assert oracle.rel_frobenius(y_new.float().cpu(), y_ref.float().cpu()) < 3e-4
