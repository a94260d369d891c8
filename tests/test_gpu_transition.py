"""Pair Transition on the B200 kernel against the fp32 CPU oracle on the same bf16-rounded input and weights.

Bounds as for the triangle update (bf16 I/O): relative Frobenius <= 5e-3 and max abs <= 3e-2 on the module output,
and the update alone (residual off) within 1.2e-2 relative Frobenius. The reference's own Transition checks compare
bf16 against fp32 PyTorch at a few 1e-3 relative L2 (docs/engine2-training-connection.md:121 in the reference project).
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from oracle import trimul_oracle as oracle
from tests.helpers import assert_module_parity

pytestmark = pytest.mark.gpu
DEV = "cuda"


def transition_params(seed, dtype=torch.bfloat16, beta_scale=0.05):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return {
        "ln_in.weight": 1.0 + 0.1 * rn(128), "ln_in.bias": beta_scale * rn(128),
        "expand_a.weight": (rn(512, 128) * 128**-0.5).to(dtype), "expand_b.weight": (rn(512, 128) * 128**-0.5).to(dtype),
        "squeeze.weight": (rn(128, 512) * 512**-0.5).to(dtype),
    }


def _module(p, dtype=torch.bfloat16, **kw):
    m = mw.Transition(128, check_status=True, **kw)
    m.load_state_dict({k: v.clone() for k, v in p.items()})
    return m.to(DEV).to(dtype).eval()


def test_state_dict_layout():
    sd = mw.Transition(128).state_dict()
    assert list(sd) == ["ln_in.weight", "ln_in.bias", "expand_a.weight", "expand_b.weight", "squeeze.weight"]
    assert sd["expand_a.weight"].shape == (512, 128) and sd["squeeze.weight"].shape == (128, 512)
    with pytest.raises(NotImplementedError):
        mw.Transition(64)
    with pytest.raises(NotImplementedError):
        mw.Transition(128, n=2)


@pytest.mark.parametrize("shape", [(1, 16, 16), (1, 40, 40), (2, 128, 128), (1, 200, 200), (1, 384, 384), (777,)])
def test_transition_matches_oracle(shape):
    """From one partial tile (256 positions of the 256-position tile), through ragged position counts, to 147 456
    positions (several tiles per CTA pair)."""
    p = transition_params(500 + len(shape) + shape[-1])
    g = torch.Generator().manual_seed(501 + shape[-1])
    x = torch.randn(*shape, 128, generator=g).to(torch.bfloat16)
    ref = oracle.transition_forward(x, p)
    out = torch.full_like(x, float("nan")).to(DEV)
    packed = F_.aligned_empty(F_.transition_packed_bytes(), torch.device(DEV))
    F_.transition_pack_weights({k: v.to(DEV) for k, v in p.items()}, packed)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    F_.transition_forward(x.to(DEV), packed, st, out=out)
    F_.check_status(st, "transition")
    assert_module_parity(out, ref, x, f"transition {shape}")
    with torch.no_grad():
        y = _module(p)(x.to(DEV))
    assert torch.equal(y, out)


def test_transition_update_alone_custom_eps_zero_gamma_and_fp32_masters():
    p = transition_params(510, dtype=torch.float32, beta_scale=0.3)
    p["ln_in.weight"][::3] = 0
    x = (torch.randn(1, 96, 96, 128, generator=torch.Generator().manual_seed(511)) * 2.0 + 0.5).to(torch.bfloat16)
    m = _module(p, dtype=torch.float32, residual=False)
    assert m.expand_a.weight.dtype == torch.float32 and m.ln_in.weight.dtype == torch.float32
    m.ln_in.eps = 0.03
    ref = oracle.transition_forward(x, p, eps=0.03, residual=False)
    with torch.no_grad():
        u = m(x.to(DEV))
    got = u.float().cpu()
    assert torch.isfinite(got).all()
    rel = oracle.rel_frobenius(got, ref)
    print(f"[parity] transition update alone: rel_frobenius={rel:.3e} max_abs={oracle.max_abs(got, ref):.3e}")
    assert rel <= 1.2e-2 and oracle.max_abs(got, ref) <= 3e-2


def test_transition_is_deterministic_and_in_place_capable():
    p = transition_params(520)
    x = torch.randn(1, 256, 256, 128, generator=torch.Generator().manual_seed(521)).to(torch.bfloat16).to(DEV)
    m = _module(p)
    with torch.no_grad():
        first = m(x)
        for _ in range(20):
            assert torch.equal(m(x), first)
    # y may alias x: every tile is read into shared memory (and re-read for the residual) before its y is stored
    packed = F_.aligned_empty(F_.transition_packed_bytes(), torch.device(DEV))
    F_.transition_pack_weights({k: v.to(DEV) for k, v in p.items()}, packed)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    xi = x.clone()
    F_.transition_forward(xi, packed, st, out=xi)
    F_.check_status(st, "transition in place")
    assert torch.equal(xi, first)


def test_transition_large_offsets_and_saturation():
    """A large common offset of the input (LayerNorm cancellation) stays within the bounds; enlarged weights push the
    hidden activations past the fp16 range, where they saturate instead of producing infinities."""
    p = transition_params(530)
    g = torch.Generator().manual_seed(531)
    x = (torch.randn(1, 64, 64, 128, generator=g) + 20.0).to(torch.bfloat16)
    ref = oracle.transition_forward(x, p, residual=False)
    with torch.no_grad():
        u = _module(p, residual=False)(x.to(DEV))
    assert oracle.rel_frobenius(u.float().cpu(), ref) <= 1.2e-2
    for k in ("expand_a.weight", "expand_b.weight"):
        p[k] = (p[k].float() * 300.0).to(torch.bfloat16)
    with torch.no_grad():
        y = _module(p)(x.to(DEV))
    assert torch.isfinite(y.float()).all()


def _oracle_grads(x, p, dy, **kw):
    xf = x.detach().float().requires_grad_(True)
    pf = {k: v.detach().clone().float().requires_grad_(True) for k, v in p.items()}
    y = oracle.transition_forward(xf, pf, differentiable=True, **kw)
    y.backward(dy.float())
    return y.detach(), xf.grad, {k: v.grad for k, v in pf.items()}


def _rel(a, b):
    return oracle.rel_frobenius(a.detach().float().cpu(), b.detach().float().cpu())


@pytest.mark.parametrize("shape,residual,dtype", [((1, 64, 64, 128), True, torch.bfloat16), ((2, 77, 77, 128), True, torch.bfloat16),
                                                  ((1, 200, 136, 128), False, torch.float32), ((1, 384, 384, 128), True, torch.bfloat16)])
def test_transition_gradients_match_the_oracle(shape, residual, dtype):
    """Backward of the pair Transition: gradients of the input and the five parameters against autograd through the
    fp32 oracle (relative L2 below 1e-2 each; the reference's bound for its fused transition is a few 1e-3 against fp32
    PyTorch, docs/engine2-training-connection.md:121 in the reference project), bit-identical on repetition."""
    p = transition_params(900 + shape[1], dtype=dtype)
    g = torch.Generator().manual_seed(901 + shape[1])
    x = torch.randn(*shape, generator=g).to(torch.bfloat16)
    dy = (torch.randn(*shape, generator=g) * 0.01).to(torch.bfloat16)
    y_ref, dx_ref, gp_ref = _oracle_grads(x, p, dy, residual=residual)
    m = mw.Transition(128, residual=residual, check_status=True)
    m.load_state_dict({k: v.clone() for k, v in p.items()})
    m = m.to(DEV).to(dtype).train()
    runs = []
    for _ in range(2):
        m.zero_grad()
        xd = x.to(DEV).requires_grad_(True)
        y = m(xd)
        y.backward(dy.to(DEV))
        runs.append((xd.grad.clone(), {k: v.grad.clone() for k, v in m.named_parameters()}))
    assert _rel(y, y_ref) <= 5e-3
    errs = {"dx": _rel(runs[0][0], dx_ref)}
    for k in gp_ref:
        assert runs[0][1][k].shape == gp_ref[k].shape
        errs[k] = _rel(runs[0][1][k], gp_ref[k])
        assert torch.equal(runs[0][1][k], runs[1][1][k]), k
    assert torch.equal(runs[0][0], runs[1][0])
    print("[transition grads]", {k: f"{v:.2e}" for k, v in errs.items()})
    assert max(errs.values()) <= 1e-2, errs
    y_eval = m.eval()(x.to(DEV))
    assert not y_eval.requires_grad


def test_transition_backward_soak_is_bit_identical():
    """Forty backward calls of the pair Transition (147 456 positions: more tiles than CTAs, so every CTA loops and
    prefetches) give the first call's bits for the input gradient and the five parameter gradients."""
    from miniworld_b200 import functional as F_

    p = {k: v.to(DEV) for k, v in transition_params(930).items()}
    g = torch.Generator().manual_seed(931)
    x = torch.randn(1, 384, 384, 128, generator=g).to(torch.bfloat16).to(DEV)
    dy = (torch.randn(1, 384, 384, 128, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    first = None
    for it in range(40):
        dx, grads = F_.transition_backward(dy, x, p, check=True)
        cur = [dx] + [grads[k] for k in sorted(grads)]
        assert all(torch.isfinite(t.float()).all() for t in cur)
        if first is None:
            first = [t.clone() for t in cur]
        else:
            for a, b in zip(first, cur):
                assert torch.equal(a, b), it
