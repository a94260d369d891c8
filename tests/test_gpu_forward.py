"""End-to-end parity of the module forward against the fp32 CPU oracle, plus the reference's identities.

Tolerances (bf16 I/O, fp32 oracle on the same bf16-rounded inputs and weights): relative Frobenius
<= 5e-3 and max abs <= 3e-2 on the module output; the update alone (y - z) is additionally held to
1.2e-2 relative Frobenius.
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from miniworld_b200.synthetic import make_workload
from oracle import trimul_oracle as oracle
from tests.helpers import assert_module_parity, params_to, rand_params

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _module(params, outgoing=True, dtype=torch.bfloat16, cls=None, **kw):
    m = (cls(128, **kw) if cls else mw.TriangleMultiplication(128, outgoing=outgoing, check_status=True, **kw))
    m.load_state_dict({k: v.clone() for k, v in params.items()})
    m = m.to(DEV).to(dtype).eval()
    return m


def _holes(B, N):
    mask = torch.ones(B, N, dtype=torch.bool)
    mask[:, ::3] = False  # the reference's every-third-token mask (tests/test_engine_h100_masks.py:74)
    return mask


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("N", [128, 384])
@pytest.mark.parametrize("mask_kind", ["none", "all_valid", "holes"])
def test_module_matches_oracle(N, outgoing, mask_kind):
    torch.manual_seed(62)
    p = rand_params(21)
    z = torch.randn(1, N, N, 128).to(torch.bfloat16)
    mask = None if mask_kind == "none" else torch.ones(1, N, dtype=torch.bool)
    if mask_kind == "holes":
        mask = _holes(1, N)
    ref = oracle.trimul_forward(z, p, mask, outgoing=outgoing)
    m = _module(p, outgoing)
    with torch.no_grad():
        y = m(z.to(DEV), None if mask is None else mask.to(DEV))
    assert y.dtype == torch.bfloat16 and y.shape == z.shape
    assert_module_parity(y, ref, z, f"N={N} outgoing={outgoing} mask={mask_kind}")


@pytest.mark.parametrize("outgoing", [True, False])
def test_mask_none_equals_all_true(outgoing):
    p = rand_params(22)
    z = torch.randn(1, 64, 64, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    m = _module(p, outgoing)
    with torch.no_grad():
        a = m(z, None)
        b = m(z, torch.ones(1, 64, dtype=torch.bool, device=DEV))
    assert torch.equal(a, b)


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("N", [128, 384])
def test_all_invalid_mask_returns_input_bit_exact(N, outgoing):
    """Reference identity: all tokens masked and ln_out.bias = 0 => y == x exactly (tests/test_engine_h100_masks.py:89-91)."""
    p = rand_params(23)
    p["ln_out.bias"] = torch.zeros(128)
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    m = _module(p, outgoing)
    with torch.no_grad():
        y = m(z, torch.zeros(1, N, dtype=torch.bool, device=DEV))
    torch.testing.assert_close(y, z, rtol=0, atol=0)


@pytest.mark.parametrize("outgoing", [True, False])
def test_mask_keeps_output_gate_and_custom_eps(outgoing):
    """Non-zero LN biases expose masking the gate input by mistake; eps is read from the LN sub-modules
    at call time (tests/test_engine_h100_masks.py:117-133)."""
    p = rand_params(24)
    p["ln_pair.bias"] = torch.full((128,), 0.2)
    p["ln_out.bias"] = torch.full((128,), 0.4)
    N = 128
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    mask = _holes(1, N)
    m = _module(p, outgoing)
    m.ln_pair.eps = 0.03
    m.ln_out.eps = 0.07
    ref = oracle.trimul_forward(z, p, mask, outgoing=outgoing, eps_in=0.03, eps_out=0.07)
    with torch.no_grad():
        y = m(z.to(DEV), mask.to(DEV))
    assert_module_parity(y, ref, z, "custom eps")
    # masked cells still receive sigmoid(gate) * (beta_out W_o^T): the update there is not zero
    upd = (y.float().cpu() - z.float())[0, 0, 0]
    assert float(upd.abs().max()) > 1e-3


@pytest.mark.parametrize("outgoing", [True, False])
def test_batched_forward_equals_the_per_sample_loop_and_is_deterministic(outgoing):
    """Samples of a batch are independent (the reference checks batched templates against the per-template loop,
    tests/test_template_embedder_batching.py:92-104): the batched forward equals the loop bit for bit, and a
    second call gives the same bits."""
    p = rand_params(33)
    m = _module(p, outgoing)
    g = torch.Generator().manual_seed(34)
    B, N = 3, 136
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    mask = (torch.rand(B, N, generator=g) > 0.2).to(DEV)
    with torch.no_grad():
        y = m(z, mask)
        again = m(z, mask)
        loop = torch.cat([m(z[b : b + 1].contiguous(), mask[b : b + 1].contiguous()) for b in range(B)])
    assert torch.equal(y, again)
    assert torch.equal(y, loop)


def test_zero_gamma_rows():
    """Every third LayerNorm gamma = 0 (docs/archive/engine2-validation-20260923/validate_bidir_reference.py:20-22)."""
    p = rand_params(25)
    p["ln_pair.weight"][::3] = 0
    p["ln_out.weight"][::3] = 0
    N = 64
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16)
    ref = oracle.trimul_forward(z, p, None)
    with torch.no_grad():
        y = _module(p)(z.to(DEV), None)
    assert_module_parity(y, ref, z, "zero gamma")


@pytest.mark.parametrize("N", [20, 52])
def test_odd_lengths_are_padded_and_cropped(N):
    p = rand_params(26)
    g = torch.Generator().manual_seed(5)
    z = torch.randn(2, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(2, N, generator=g) > 0.2
    for outgoing in (True, False):
        ref = oracle.trimul_forward(z, p, mask, outgoing=outgoing)
        with torch.no_grad():
            y = _module(p, outgoing)(z.to(DEV), mask.to(DEV))
        assert y.shape == z.shape
        assert_module_parity(y, ref, z, f"N={N}")


def test_fp32_master_weights_and_biases():
    p = rand_params(27, dtype=torch.float32)
    N = 64
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(6)).to(torch.bfloat16)
    biases = {"to_left_gate": torch.ones(128), "to_right_gate": torch.ones(128), "to_gate": torch.ones(128)}
    ref = oracle.trimul_forward(z, p, None, biases=biases)
    m = _module(p, dtype=torch.float32)
    assert m.to_left.weight.dtype == torch.float32
    m.set_biases({k: v.to(DEV) for k, v in biases.items()})
    with torch.no_grad():
        y = m(z.to(DEV), None)
    assert_module_parity(y, ref, z, "fp32 masters + biases")


def test_openfold_style_classes_and_pair_mask():
    p = rand_params(28)
    N = 64
    g = torch.Generator().manual_seed(7)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    tok = torch.rand(1, N, generator=g) > 0.2
    pair = tok[:, :, None] & tok[:, None, :]
    for cls, outgoing in ((mw.TriangleMultiplicationOutgoing, True), (mw.TriangleMultiplicationIncoming, False)):
        m = cls(128, residual=False, check_status=True)
        m.load_openfold_state_dict(mw.to_openfold_state_dict(p))
        m = m.to(DEV).to(torch.bfloat16).eval()
        with torch.no_grad():
            y_tok = m(z.to(DEV), tok.to(DEV))
            y_pair = m(z.to(DEV), pair.to(DEV))
        assert torch.equal(y_tok, y_pair)  # a token-derived pair mask is the same mask
        ref = oracle.trimul_forward(z, p, tok, outgoing=outgoing, residual=False)
        got = y_tok.float().cpu()
        assert oracle.rel_frobenius(got, ref) < 1.2e-2
        # an arbitrary pair mask
        pm = torch.rand(1, N, N, generator=g) > 0.4
        ref2 = oracle.trimul_forward(z, p, None, outgoing=outgoing, pair_mask=pm, residual=False)
        with torch.no_grad():
            y2 = m(z.to(DEV), pm.to(DEV))
        assert oracle.rel_frobenius(y2.float().cpu(), ref2) < 1.2e-2


@pytest.mark.parametrize("name,n", [("n384", None), ("crop768", None), ("batch8x256", None)])
def test_benchmark_workloads_match_oracle(name, n):
    w = make_workload(name, seed=0, n_override=n)
    for direction in w.directions:
        outgoing = direction == "outgoing"
        ref = oracle.trimul_forward(w.z, w.params, w.mask, outgoing=outgoing, k_chunk=32)
        m = _module(w.params, outgoing)
        with torch.no_grad():
            y = m(w.z.to(DEV), w.mask.to(DEV))
        assert_module_parity(y, ref, w.z, f"{name} {direction}")


def test_graph_capture_sees_weight_updates():
    """Weights are packed inside every call, so a captured graph replays with the current values
    (the reference hit stale packed weights after capture, docs/repositories.md:218)."""
    p = rand_params(29)
    N = 64
    z = torch.randn(1, N, N, 128, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16).to(DEV)
    m = _module(p)
    m.check_status = False
    with torch.no_grad():
        m(z, None)  # warm-up allocates the workspace
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y = m(z, None)
        graph.replay()
        torch.cuda.synchronize()
        before = y.clone()
        m.to_out.weight.mul_(2.0)
        graph.replay()
        torch.cuda.synchronize()
        eager = m(z, None)
    assert torch.equal(y, eager)
    assert not torch.equal(y, before)


def test_errors_are_loud():
    p = rand_params(30)
    m = _module(p)
    with pytest.raises(RuntimeError):
        m(torch.zeros(1, 16, 16, 128, dtype=torch.bfloat16), None)  # CPU tensor: no fallback
    with pytest.raises(RuntimeError):
        F_.trimul_forward(torch.zeros(1, 12, 12, 128, dtype=torch.bfloat16, device=DEV), params_to(p, DEV))  # N % 8
    with pytest.raises(NotImplementedError):
        mw.TriangleMultiplication(64)  # 64 contracted channels in one direction is not a shape the kernels take
    zz = torch.zeros(1, 16, 16, 128, dtype=torch.bfloat16, device=DEV, requires_grad=True)
    with pytest.raises(NotImplementedError):  # widths the kernels do not take
        mw.Transition(64)


def test_large_complex_workload_full_size_rows():
    """The large-complex workload (B = 1, N = 2048, 4 chains, 5 % of tokens masked) at full size: a sample of pair rows is
    compared with the oracle (which forms the O(N^3) contraction only for those rows), both directions; plus the
    size-independent identity that an all-invalid mask returns the input."""
    w = make_workload("complex2048", seed=0)
    rows = [0, 511, 512, 1300, 2047]
    zd, md = w.z.to(DEV), w.mask.to(DEV)
    for direction in w.directions:
        outgoing = direction == "outgoing"
        m = _module(w.params, outgoing)
        with torch.no_grad():
            y = m(zd, md)
        ref = oracle.trimul_forward_rows(w.z, w.params, w.mask, rows, outgoing=outgoing)
        got = y[0, rows].float().cpu()
        assert torch.isfinite(y.float()).all()
        assert_module_parity(got, ref, w.z[0, rows], f"complex2048 {direction} rows")
        del y
    p0 = dict(w.params)
    p0["ln_out.bias"] = torch.zeros(128)
    m = _module(p0, True)
    with torch.no_grad():
        y = m(zd, torch.zeros_like(md))
    assert torch.equal(y, zd)


def test_fp32_workload_is_served_through_bf16():
    """The fp32 workload (N = 128, all-ones mask, outgoing) is a CPU configuration of the reference; the
    module takes the fp32 tensor, rounds it to bf16 once, and returns fp32. Checked against the oracle evaluated on
    the same rounded input and weights."""
    w = make_workload("cpu128", seed=0)
    p16 = {k: (v.to(torch.bfloat16) if k.startswith("to_") else v) for k, v in w.params.items()}
    z16 = w.z.to(torch.bfloat16)
    ref = oracle.trimul_forward(z16, p16, w.mask, outgoing=True)
    m = _module(p16, True)
    with torch.no_grad():
        y = m(w.z.to(DEV), w.mask.to(DEV))
    assert y.dtype == torch.float32
    assert_module_parity(y, ref, z16, "cpu128")
