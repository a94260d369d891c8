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
    with pytest.raises(RuntimeError):
        y.backward(dy.to(DEV))  # the stage tensors are released after the first backward
    # parameters only (the input does not require grad): still differentiable in training mode
    m.zero_grad()
    y2 = m(z.to(DEV), mask.to(DEV))
    assert y2.requires_grad and torch.equal(y2.detach(), y.detach())
    # evaluation mode with an input that does not require grad: the plain forward, nothing kept
    y3 = m.eval()(z.to(DEV), mask.to(DEV))
    assert not y3.requires_grad


def test_biases_pair_mask_fp32_masters_and_determinism():
    """fp32 master weights, gate / output / projection biases (constants: no gradient), a pair mask on top of the token
    mask, through the functional entry point; a second backward on the same inputs is bit-identical (fixed summation
    order, no atomics)."""
    from miniworld_b200 import functional as F_

    N = 104
    p = {k: v.float() for k, v in rand_params(530).items()}
    g = torch.Generator().manual_seed(531)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(2, N, N, 128, generator=g) * 3.0).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.15
    pmask = torch.rand(2, N, N, generator=g) > 0.1
    biases = {"to_left_gate": torch.ones(128), "to_right": 0.1 * torch.randn(128, generator=g),
              "to_gate": 0.2 * torch.randn(128, generator=g), "to_out": 0.1 * torch.randn(128, generator=g)}
    y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, True, pair_mask=pmask, biases=biases)
    dev = lambda d: {k: t.to(DEV) for k, t in d.items()}  # noqa: E731
    zd, pd = z.to(DEV), dev(p)
    ws = F_.aligned_empty(F_.workspace_bytes(2, N, True), torch.device(DEV))
    y = F_.trimul_forward(zd, pd, mask.to(DEV), outgoing=True, pair_mask=pmask.to(DEV), biases=dev(biases), workspace=ws, check=True)
    _check("y", y, y_ref, 5e-3)
    runs = []
    for _ in range(2):
        dz, grads = F_.trimul_backward(dy.to(DEV), zd, pd, ws, mask.to(DEV), outgoing=True, pair_mask=pmask.to(DEV),
                                       biases=dev(biases), check=True)
        runs.append((dz, grads))
    _check("dz", runs[0][0], dz_ref)
    for k in _PARAM_KEYS:
        assert runs[0][1][k].dtype == torch.float32
        _check(k, runs[0][1][k], gp_ref[k], 4e-3)  # fp32 gradients: no bf16 rounding of the result
        assert torch.equal(runs[0][1][k], runs[1][1][k]), k
    assert torch.equal(runs[0][0], runs[1][0])


def test_gradient_scale_invariance_and_zero_gradient():
    """The power-of-two scale the fp16 gradient tiles carry is invisible: dy and 2^-20 dy give gradients that differ by
    exactly that factor; dy = 0 gives zeros (not NaN)."""
    from miniworld_b200 import functional as F_

    N = 72
    p = rand_params(540)
    g = torch.Generator().manual_seed(541)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    dy = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    pd = {k: v.to(DEV) for k, v in p.items()}
    ws = F_.aligned_empty(F_.workspace_bytes(1, N, False), torch.device(DEV))
    F_.trimul_forward(z, pd, None, outgoing=False, workspace=ws, check=True)
    dz1, g1 = F_.trimul_backward(dy, z, pd, ws, None, outgoing=False, residual=False, check=True)
    dz2, g2 = F_.trimul_backward((dy.float() * 2.0**-20).to(torch.bfloat16), z, pd, ws, None, outgoing=False, residual=False, check=True)
    assert torch.equal(dz1.float() * 2.0**-20, dz2.float())
    for k in _PARAM_KEYS:
        assert torch.equal(g1[k] * 2.0**-20, g2[k]), k
    dz0, g0 = F_.trimul_backward(torch.zeros_like(dy), z, pd, ws, None, outgoing=False, residual=False, check=True)
    assert not dz0.float().any() and all(not v.any() for v in g0.values())


def test_gradients_at_crop_384():
    """L = 384 (the reference's validation length), both LayerNorms with every third gamma zero."""
    N = 384
    p = rand_params(550)
    p["ln_pair.weight"][::3] = 0
    p["ln_out.weight"][::3] = 0
    g = torch.Generator().manual_seed(551)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(1, N, N, 128, generator=g) * 0.01).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.2
    y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, False)
    zd = z.to(DEV).requires_grad_(True)
    pd = {k: v.detach().to(DEV).requires_grad_(True) for k, v in p.items()}
    y = trimul_train(zd, pd, mask.to(DEV), outgoing=False, check=True)
    y.backward(dy.to(DEV))
    _check("y", y, y_ref, 5e-3)
    _check("dz", zd.grad, dz_ref)
    for k in _PARAM_KEYS:
        _check(k, pd[k].grad, gp_ref[k])


def _bidir_params(seed, beta_scale=0.05):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *sh: torch.randn(*sh, generator=g)  # noqa: E731
    bf = torch.bfloat16
    return {
        "ln_pair.weight": 1.0 + 0.1 * rn(128), "ln_pair.bias": beta_scale * rn(128),
        "to_left.weight": (rn(256, 128) * 128**-0.5).to(bf), "to_left_gate.weight": (rn(256, 128) * 128**-0.5).to(bf),
        "to_right.weight": (rn(256, 128) * 128**-0.5).to(bf), "to_right_gate.weight": (rn(256, 128) * 128**-0.5).to(bf),
        "ln_out.weight": 1.0 + 0.1 * rn(256), "ln_out.bias": beta_scale * rn(256),
        "to_gate.weight": (rn(128, 128) * 128**-0.5).to(bf), "to_out.weight": (rn(128, 256) * 256**-0.5).to(bf),
    }


def _bidir_oracle_grads(z, p, mask, dy, **kw):
    zf = z.detach().float().requires_grad_(True)
    pf = {k: v.detach().clone().float().requires_grad_(True) for k, v in p.items()}
    y = oracle.bidir_forward(zf, pf, mask, differentiable=True, **kw)
    y.backward(dy.float())
    return y.detach(), zf.grad, {k: v.grad for k, v in pf.items()}


@pytest.mark.parametrize("N,mask_kind", [(64, "none"), (136, "random"), (200, "holes"), (384, "random")])
def test_bidirectional_gradients_match_the_oracle(N, mask_kind):
    """The module MiniWorld's trunk builds (256 contracted channels, one LayerNorm over them): gradients for the input
    and all ten parameters of the wide shapes, as the reference validates its own backward
    (docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11-38 in the reference project: L = 384,
    random token mask, relative L2 of every gradient)."""
    p = _bidir_params(600 + N)
    g = torch.Generator().manual_seed(601 + N)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(1, N, N, 128, generator=g) * 0.01).to(torch.bfloat16)
    mask = None
    if mask_kind == "random":
        mask = torch.rand(1, N, generator=g) > 0.2
    elif mask_kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    y_ref, dz_ref, gp_ref = _bidir_oracle_grads(z, p, mask, dy)
    zd = z.to(DEV).requires_grad_(True)
    pd = {k: v.detach().to(DEV).requires_grad_(True) for k, v in p.items()}
    y = trimul_train(zd, pd, None if mask is None else mask.to(DEV), outgoing=None, check=True)
    y.backward(dy.to(DEV))
    _check("y", y, y_ref, 5e-3)
    _check("dz", zd.grad, dz_ref)
    for k in _PARAM_KEYS:
        assert pd[k].grad is not None and pd[k].grad.shape == pd[k].shape, k
        _check(k, pd[k].grad, gp_ref[k])


def test_bidirectional_module_training_step_dropout_zero_gamma_and_determinism():
    """`BidirectionalTriangleMultiplication` in training mode: every third gamma of both LayerNorms zero, a fixed
    row-shared dropout scale, N not a multiple of 8, a batch of two; two backward passes are bit-identical."""
    N = 77
    p = _bidir_params(620)
    p["ln_pair.weight"][::3] = 0
    p["ln_out.weight"][::3] = 0
    g = torch.Generator().manual_seed(621)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    dy = (torch.randn(2, N, N, 128, generator=g) * 0.5).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.2
    scale = ((torch.rand(2, 1, N, 128, generator=g) > 0.25).float() / 0.75).to(torch.bfloat16)
    y_ref, dz_ref, gp_ref = _bidir_oracle_grads(z, p, mask, dy, drop_scale=scale)
    m = mw.BidirectionalTriangleMultiplication(128, p_drop=0.25, check_status=True)
    m.load_state_dict(p)
    m = m.to(DEV).to(torch.bfloat16).train()
    m._make_drop_row_scale = lambda pair, pdrop: scale.to(DEV)
    grads = []
    for _ in range(2):
        m.zero_grad()
        zd = z.to(DEV).requires_grad_(True)
        y = m(zd, mask.to(DEV))
        y.backward(dy.to(DEV))
        grads.append((zd.grad.clone(), {k: v.grad.clone() for k, v in m.named_parameters()}))
    _check("y", y, y_ref, 5e-3)
    _check("dz", grads[0][0], dz_ref)
    for k in _PARAM_KEYS:
        _check(k, grads[0][1][k], gp_ref[k])
        assert torch.equal(grads[0][1][k], grads[1][1][k]), k
    assert torch.equal(grads[0][0], grads[1][0])


def _narrow_params(seed, beta_scale=0.05):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *sh: torch.randn(*sh, generator=g)  # noqa: E731
    bf = torch.bfloat16
    return {
        "ln_pair.weight": 1.0 + 0.1 * rn(64), "ln_pair.bias": beta_scale * rn(64),
        "to_left.weight": (rn(128, 64) * 64**-0.5).to(bf), "to_left_gate.weight": (rn(128, 64) * 64**-0.5).to(bf),
        "to_right.weight": (rn(128, 64) * 64**-0.5).to(bf), "to_right_gate.weight": (rn(128, 64) * 64**-0.5).to(bf),
        "ln_out.weight": 1.0 + 0.1 * rn(128), "ln_out.bias": beta_scale * rn(128),
        "to_gate.weight": (rn(64, 64) * 64**-0.5).to(bf), "to_out.weight": (rn(64, 128) * 128**-0.5).to(bf),
    }


@pytest.mark.parametrize("kind", ["outgoing", "incoming", "bidirectional"])
@pytest.mark.parametrize("N,mask_kind", [(64, "none"), (136, "random"), (200, "holes"), (384, "random")])
def test_narrow_gradients_match_the_oracle(kind, N, mask_kind):
    """The 64-wide pair stacks: `TriangleMultiplication(64, d_hidden=128)` (the template blocks of the fine-tuning
    harness, benchmarks/protenix_finetune/patch_engine.py:283-295 in the reference project) and
    `BidirectionalTriangleMultiplication(64)` (the (L, D) = (384, 64) case of the reference's backward validation,
    docs/archive/engine2-validation-20260923/validate_bidir_reference.py:11)."""
    p = _narrow_params(700 + N)
    g = torch.Generator().manual_seed(701 + N)
    z = torch.randn(1, N, N, 64, generator=g).to(torch.bfloat16)
    dy = (torch.randn(1, N, N, 64, generator=g) * 0.01).to(torch.bfloat16)
    mask = None
    if mask_kind == "random":
        mask = torch.rand(1, N, generator=g) > 0.2
    elif mask_kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    if kind == "bidirectional":
        y_ref, dz_ref, gp_ref = _bidir_oracle_grads(z, p, mask, dy)
        m = mw.BidirectionalTriangleMultiplication(64, check_status=True)
    else:
        y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, kind == "outgoing")
        m = mw.TriangleMultiplication(64, d_hidden=128, outgoing=kind == "outgoing", check_status=True)
    m.load_state_dict(p)
    m = m.to(DEV).to(torch.bfloat16).train()
    zd = z.to(DEV).requires_grad_(True)
    y = m(zd, None if mask is None else mask.to(DEV))
    y.backward(dy.to(DEV))
    _check("y", y, y_ref, 5e-3)
    _check("dz", zd.grad, dz_ref)
    sd = dict(m.named_parameters())
    for k in _PARAM_KEYS:
        assert sd[k].grad is not None and sd[k].grad.shape == sd[k].shape, k
        _check(k, sd[k].grad, gp_ref[k])


def test_training_step_replays_from_a_cuda_graph():
    """Forward (stage tensors kept) and backward are asynchronous on the stream with no host synchronisation, so one
    training step can be captured once and replayed: the replay with a new upstream gradient equals the eager call bit
    for bit."""
    from miniworld_b200 import functional as F_

    N = 136
    p = {k: v.to(DEV) for k, v in rand_params(560).items()}
    g = torch.Generator().manual_seed(561)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    mask = (torch.rand(1, N, generator=g) > 0.2).to(DEV)
    dy_a = (torch.randn(1, N, N, 128, generator=g) * 0.01).to(torch.bfloat16).to(DEV)
    dy_b = (torch.randn(1, N, N, 128, generator=g) * 3.0).to(torch.bfloat16).to(DEV)
    dev = torch.device(DEV)
    ws = F_.aligned_empty(F_.workspace_bytes(1, N, False), dev)
    bws = F_.aligned_empty(F_.backward_workspace_bytes(1, N, False), dev)
    y = torch.empty_like(z)
    dy = dy_a.clone()

    def step():
        F_.trimul_forward(z, p, mask, outgoing=False, workspace=ws, out=y)
        return F_.trimul_backward(dy, z, p, ws, mask, outgoing=False, workspace=bws)

    step()  # warm-up outside the capture (kernel attributes, tensor maps' driver entry point)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        dz_g, grads_g = step()
    for src in (dy_b, dy_a):
        dy.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        dz_r, grads_r = dz_g.clone(), {k: v.clone() for k, v in grads_g.items()}
        dz_e, grads_e = step()
        torch.cuda.synchronize()
        assert torch.equal(dz_r, dz_e)
        for k in _PARAM_KEYS:
            assert torch.equal(grads_r[k], grads_e[k]), k
    F_.check_status(bws[:64].view(torch.int32), "b200_trimul_backward")


@pytest.mark.parametrize("kind", ["common_offset_20", "heavy_tail"])
def test_backward_numerical_corners(kind):
    """The backward on the inputs of the forward's numerical corner cases: a common offset of 20 on z (|mean| = 20 sigma
    at every position), and heavy-tailed z with 128 x larger projection weights (|t| of a few 1e5, a third of the fp16
    range of the stored t): gradients stay finite and keep the usual accuracy (measured 2e-3 in both cases)."""
    N = 128
    g = torch.Generator().manual_seed(570)
    p = rand_params(571, ln_bias_scale=0.2)
    z = torch.randn(1, N, N, 128, generator=g)
    tol = GRAD_REL_TOL
    if kind == "common_offset_20":
        z = z + 20.0
    else:
        for k in ("to_left.weight", "to_right.weight"):
            p[k] = (p[k].float() * 128.0).to(torch.bfloat16)
        spikes = torch.rand(1, N, N, 128, generator=g) < 0.01
        z = torch.where(spikes, z * 30.0, z)
    z = z.to(torch.bfloat16)
    dy = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(1, N, generator=g) > 0.1
    y_ref, dz_ref, gp_ref = _oracle_grads(z, p, mask, dy, True)
    zd = z.to(DEV).requires_grad_(True)
    pd = {k: v.detach().to(DEV).requires_grad_(True) for k, v in p.items()}
    y = trimul_train(zd, pd, mask.to(DEV), outgoing=True, check=True)
    y.backward(dy.to(DEV))
    _check("dz", zd.grad, dz_ref, tol)
    for k in _PARAM_KEYS:
        _check(k, pd[k].grad, gp_ref[k], tol)


def test_backward_soak_is_bit_identical():
    """The backward kernels synchronise through per-thread waits on mbarriers with few CTA-wide barriers; a missing
    order would show as run-to-run differences. Forty backward calls (N = 384: three 128-wide
    column blocks per row, ragged masks, both directions, plus the bidirectional module) must give the first call's bits
    for the input gradient and every parameter gradient."""
    from miniworld_b200 import functional as F_
    from tests.test_gpu_bidirectional import bidir_params

    B, N = 1, 384
    g = torch.Generator().manual_seed(4242)
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    dy = (torch.randn(B, N, N, 128, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    mask = (torch.rand(B, N, generator=g) > 0.15).to(DEV)
    for outgoing in (True, False, None):
        p = bidir_params(77) if outgoing is None else rand_params(76)
        p = {k: v.to(DEV) for k, v in p.items()}
        ws = F_.aligned_empty(F_.workspace_bytes(B, N, outgoing), torch.device(DEV))
        F_.trimul_forward(z, p, mask, outgoing=outgoing, workspace=ws)
        first = None
        for it in range(40 if outgoing is not None else 15):
            dz, grads = F_.trimul_backward(dy, z, p, ws, mask, outgoing=outgoing, check=True)
            cur = [dz] + [grads[k] for k in sorted(grads)]
            assert all(torch.isfinite(t.float()).all() for t in cur)
            if first is None:
                first = [t.clone() for t in cur]
            else:
                for a, b in zip(first, cur):
                    assert torch.equal(a, b), (outgoing, it)
