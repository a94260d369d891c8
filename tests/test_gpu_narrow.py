"""The 64-wide pair stacks: `TriangleMultiplication(64, d_hidden=128)` (the template blocks of the Protenix harness,
benchmarks/protenix_finetune/patch_engine.py:283-295 in the reference project) and
`BidirectionalTriangleMultiplication(64)` (the (L, D) = (384, 64) case of the reference's validation,
docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11), against the fp32 CPU oracle on the same
bf16-rounded inputs and weights. Initialisation as in that validation: weights N(0, 1/D), gamma = 1 + 0.1 N(0,1).
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from oracle import trimul_oracle as oracle
from tests.helpers import assert_module_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def narrow_params(seed, beta_scale=0.05):
    """Shapes shared by both 64-wide forms: 128 contracted channels in total."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    bf = torch.bfloat16
    return {
        "ln_pair.weight": 1.0 + 0.1 * rn(64), "ln_pair.bias": beta_scale * rn(64),
        "to_left.weight": (rn(128, 64) * 64**-0.5).to(bf), "to_left_gate.weight": (rn(128, 64) * 64**-0.5).to(bf),
        "to_right.weight": (rn(128, 64) * 64**-0.5).to(bf), "to_right_gate.weight": (rn(128, 64) * 64**-0.5).to(bf),
        "ln_out.weight": 1.0 + 0.1 * rn(128), "ln_out.bias": beta_scale * rn(128),
        "to_gate.weight": (rn(64, 64) * 64**-0.5).to(bf), "to_out.weight": (rn(64, 128) * 128**-0.5).to(bf),
    }


def _module(p, kind, **kw):
    if kind == "bidirectional":
        m = mw.BidirectionalTriangleMultiplication(64, check_status=True, **kw)
    else:
        m = mw.TriangleMultiplication(64, d_hidden=128, outgoing=kind == "outgoing", check_status=True, **kw)
    m.load_state_dict({k: v.clone() for k, v in p.items()})
    return m.to(DEV).to(torch.bfloat16).eval()


def _oracle(z, p, mask, kind, **kw):
    if kind == "bidirectional":
        return oracle.bidir_forward(z, p, mask, **kw)
    return oracle.trimul_forward(z, p, mask, outgoing=kind == "outgoing", **kw)


def _mask(kind, N, g):
    if kind == "none":
        return None
    if kind == "holes":
        m = torch.ones(1, N, dtype=torch.bool)
        m[:, ::3] = False
        return m
    return torch.rand(1, N, generator=g) > 0.2


@pytest.mark.parametrize("kind", ["outgoing", "incoming", "bidirectional"])
@pytest.mark.parametrize("N,mask_kind", [(64, "none"), (136, "holes"), (200, "random"), (384, "random")])
def test_narrow_matches_oracle(kind, N, mask_kind):
    p = narrow_params(400 + N)
    g = torch.Generator().manual_seed(401 + N)
    z = torch.randn(1, N, N, 64, generator=g).to(torch.bfloat16)
    mask = _mask(mask_kind, N, g)
    ref = _oracle(z, p, mask, kind)
    with torch.no_grad():
        y = _module(p, kind)(z.to(DEV), None if mask is None else mask.to(DEV))
    assert y.dtype == torch.bfloat16 and y.shape == z.shape
    assert_module_parity(y, ref, z, f"d_pair 64 {kind} N={N} mask={mask_kind}")


@pytest.mark.parametrize("kind", ["incoming", "bidirectional"])
def test_narrow_zero_gamma_batch_and_padding(kind):
    """Every third gamma of both LayerNorms zero (the reference's hardest validation case) at L = 384; a batch of two
    samples with different masks equals the per-sample loop bit for bit; N not a multiple of 8 goes through the
    module's padding."""
    p = narrow_params(410)
    p["ln_pair.weight"][::3] = 0
    p["ln_out.weight"][::3] = 0
    g = torch.Generator().manual_seed(411)
    N = 384
    z = torch.randn(1, N, N, 64, generator=g).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.2
    m = _module(p, kind)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert_module_parity(y, _oracle(z, p, mask, kind), z, f"d_pair 64 {kind} zero gamma")
    zb = torch.randn(2, 136, 136, 64, generator=g).to(torch.bfloat16).to(DEV)
    mb = (torch.rand(2, 136, generator=g) > 0.2).to(DEV)
    with torch.no_grad():
        yb = m(zb, mb)
        loop = torch.cat([m(zb[b : b + 1].contiguous(), mb[b : b + 1].contiguous()) for b in range(2)])
    assert torch.equal(yb, loop)
    zo = torch.randn(1, 77, 77, 64, generator=g).to(torch.bfloat16)
    mo = torch.rand(1, 77, generator=g) > 0.2
    with torch.no_grad():
        yo = m(zo.to(DEV), mo.to(DEV))
    assert_module_parity(yo, _oracle(zo, p, mo, kind), zo, f"d_pair 64 {kind} N=77 (padded)")


def test_narrow_identities_biases_and_loud_errors():
    """All tokens masked with beta_out = 0 returns the input exactly; fp32 master weights with gate / output biases
    through the functional entry point; the dropout scale and mismatched weights raise."""
    p = narrow_params(420, beta_scale=0.3)
    N = 72
    g = torch.Generator().manual_seed(421)
    z = torch.randn(2, N, N, 64, generator=g).to(torch.bfloat16)
    p0 = dict(p)
    p0["ln_out.bias"] = torch.zeros(128)
    with torch.no_grad():
        y0 = _module(p0, "bidirectional")(z.to(DEV), torch.zeros(2, N, dtype=torch.bool, device=DEV))
    assert torch.equal(y0.cpu(), z)
    mask = torch.rand(2, N, generator=g) > 0.2
    pf = {k: v.float() for k, v in p.items()}
    biases = {"to_left_gate": torch.ones(128), "to_right_gate": torch.linspace(-1, 1, 128),
              "to_gate": 0.2 * torch.randn(64, generator=g), "to_out": 0.1 * torch.randn(64, generator=g)}
    x = torch.nn.functional.layer_norm(z.float(), (64,), pf["ln_pair.weight"], pf["ln_pair.bias"], 1e-5)
    left = torch.sigmoid(x @ pf["to_left_gate.weight"].T + biases["to_left_gate"]) * (x @ pf["to_left.weight"].T)
    right = torch.sigmoid(x @ pf["to_right_gate.weight"].T + biases["to_right_gate"]) * (x @ pf["to_right.weight"].T)
    v = (mask[:, :, None] & mask[:, None, :])[..., None].float()
    tri = torch.einsum("bkid,bkjd->bijd", left * v, right * v)
    tn = torch.nn.functional.layer_norm(tri, (128,), pf["ln_out.weight"], pf["ln_out.bias"], 1e-5)
    ref = z.float() + torch.sigmoid(x @ pf["to_gate.weight"].T + biases["to_gate"]) * (tn @ pf["to_out.weight"].T + biases["to_out"])
    dev = lambda d: {k: t.to(DEV) for k, t in d.items()}  # noqa: E731
    y = F_.trimul_forward(z.to(DEV), dev(pf), mask.to(DEV), outgoing=False, biases=dev(biases), check=True)
    assert_module_parity(y, ref, z, "d_pair 64 incoming, fp32 masters, biases")
    with pytest.raises(RuntimeError, match="dropout"):
        F_.trimul_forward(z.to(DEV), dev(p), mask.to(DEV), outgoing=False,
                          drop_scale=torch.ones(2, 1, N, 64, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(RuntimeError):
        F_.trimul_forward(torch.zeros(1, N, N, 128, dtype=torch.bfloat16, device=DEV), dev(p))  # 64-wide weights, 128-wide pair


def test_narrow_workspace_is_reused_and_smaller_than_the_wide_bidirectional_one():
    assert F_.workspace_bytes(1, 384, None, 64) == F_.workspace_bytes(1, 384, True, 64) == F_.workspace_bytes(1, 384, True)
    assert F_.workspace_bytes(1, 384, None, 64) < F_.workspace_bytes(1, 384, None)
