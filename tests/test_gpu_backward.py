"""Backward of the unidirectional triangle update: gradients for the input and all ten parameters against autograd
through the fp32 CPU oracle on the same bf16-rounded input, weights and upstream gradient.

The measure and the bound are the reference's own for its backward (relative L2 of every gradient below 3e-2,
docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11-38 in the reference project; its kernel-level
tests use 4e-3 against fp32 torch, tests/test_engine_trimul_backward_fusion.py:31-71). Here every gradient has to meet
1e-2: the operands of the contraction gradients are fp16 and the input / output tensors bf16.
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200.training import _PARAM_KEYS, trimul_train
from oracle import trimul_oracle as oracle
from tests.helpers import rand_params

pytestmark = pytest.mark.gpu
DEV = "cuda"
GRAD_REL_TOL = 1e-2


def _oracle_grads(z, p, mask, dy, outgoing, **kw):
    zf = z.detach().float().requires_grad_(True)
    pf = {k: v.detach().clone().float().requires_grad_(True) for k, v in p.items()}
    y = oracle.trimul_forward(zf, pf, mask, outgoing=outgoing, differentiable=True, **kw)
    y.backward(dy.float())
    return y.detach(), zf.grad, {k: v.grad for k, v in pf.items()}


def _check(name, got, ref, tol=GRAD_REL_TOL):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    assert torch.isfinite(got).all(), name
    rel = oracle.rel_frobenius(got, ref)
    print(f"[grad] {name}: rel_l2={rel:.3e}")
    assert rel <= tol, (name, rel)


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("N,mask_kind", [(64, "none"), (136, "random"), (200, "holes"), (256, "random")])
def test_gradients_match_the_oracle(N, mask_kind, outgoing):
    p = rand_params(500 + N)
    # the reference initialises to_gate / to_out to zero; draw them so that every gradient is exercised
    g = torch.Generator().manual_seed(501 + N)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(1, N, N, 128, generator=g) * 0.01).to(torch.bfloat16)
    mask = None
    if mask_kind == "random":
        mask = torch.rand(1, N, generator=g) > 0.2
    elif mask_kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, outgoing)
    zd = z.to(DEV).requires_grad_(True)
    pd = {k: v.detach().to(DEV).requires_grad_(True) for k, v in p.items()}
    y = trimul_train(zd, pd, None if mask is None else mask.to(DEV), outgoing=outgoing, check=True)
    assert y.requires_grad
    y.backward(dy.to(DEV))
    _check("y", y, y_ref, 5e-3)
    _check("dz", zd.grad, dz_ref)
    for k in _PARAM_KEYS:
        assert pd[k].grad is not None and pd[k].grad.dtype == pd[k].dtype, k
        _check(k, pd[k].grad, gp_ref[k])


def test_module_training_step_with_dropout_padding_and_no_residual():
    """The module in training mode: N not a multiple of 8 (padding and cropping are differentiable), a fixed row-shared
    dropout scale, no residual, fp32 LayerNorm parameters and bf16 weights; gradients land on the parameters."""
    N = 77
    p = rand_params(520)
    g = torch.Generator().manual_seed(521)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(2, N, N, 128, generator=g) * 0.02).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.2
    scale = ((torch.rand(2, 1, N, 128, generator=g) > 0.25).float() / 0.75).to(torch.bfloat16)
    y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, False, residual=False, drop_scale=scale)
    m = mw.TriangleMultiplication(128, outgoing=False, p_drop=0.25, residual=False, check_status=True)
    m.load_state_dict(p)
    m = m.to(DEV).to(torch.bfloat16).train()
    m._make_drop_row_scale = lambda pair, pdrop: scale.to(DEV)
    zd = z.to(DEV).requires_grad_(True)
    y = m(zd, mask.to(DEV))
    y.backward(dy.to(DEV))
    _check("y", y, y_ref, 5e-3)
    _check("dz", zd.grad, dz_ref)
    sd = dict(m.named_parameters())
    for k in _PARAM_KEYS:
        assert sd[k].grad is not None, k
        _check(k, sd[k].grad, gp_ref[k])
    # parameters only (the input does not require grad): still differentiable in training mode
    m.zero_grad()
    y2 = m(z.to(DEV), mask.to(DEV))
    assert y2.requires_grad and torch.equal(y2.detach(), y.detach())
    # evaluation mode with an input that does not require grad: the plain forward, nothing kept
    y3 = m.eval()(z.to(DEV), mask.to(DEV))
    assert not y3.requires_grad
