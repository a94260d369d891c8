"""CPU tests of the checker itself: the torch oracle against the committed vectors, against the
independent C restatement, and against the identities the reference's own tests assert."""

import ctypes
import importlib.util
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import trimul_oracle as oracle
from tests.helpers import rand_params

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


def _golden_module():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name", sorted(_golden_module().CASES))
def test_oracle_reproduces_golden_vectors(name):
    mg = _golden_module()
    case = mg.make_case(name)
    data = np.load(os.path.join(GOLDEN, name + ".npz"))
    assert str(data["digest"]) == mg.input_digest(case), "seeded inputs changed"
    st = mg.run_oracle(case)
    np.testing.assert_allclose(st.out.numpy(), data["out"], rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(st.tri[0, : data["tri_sample"].shape[0]].numpy(), data["tri_sample"], rtol=1e-5, atol=1e-5)


def _c_ref():
    lib_path = os.path.join(ROOT, "oracle", "_build", "libtrimul_ref.so")
    if not os.path.exists(lib_path):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    lib = ctypes.CDLL(lib_path)
    dp = ctypes.POINTER(ctypes.c_double)
    lib.trimul_ref_forward.restype = ctypes.c_int
    lib.trimul_ref_forward.argtypes = [dp, ctypes.c_void_p] + [dp] * 10 + [ctypes.c_int] * 4 + [ctypes.c_double] * 2 + [ctypes.c_int, dp]
    return lib


def _as_dp(t):
    a = np.ascontiguousarray(t.detach().to(torch.float64).numpy())
    return a, a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("mask_kind", ["none", "holes", "pair"])
def test_oracle_matches_c_restatement(outgoing, mask_kind):
    lib = _c_ref()
    N = 12
    p = rand_params(41, ln_bias_scale=0.2)
    g = torch.Generator().manual_seed(9)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    mask = pair_mask = None
    if mask_kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    if mask_kind == "pair":
        pair_mask = torch.rand(1, N, N, generator=g) > 0.3
    ref = oracle.trimul_forward(z, p, mask, outgoing=outgoing, pair_mask=pair_mask, eps_in=0.03, eps_out=0.07)
    valid = oracle.pair_valid(mask, pair_mask, 1, N)
    keep = []
    ptrs = []
    for t in (z[0], p["ln_pair.weight"], p["ln_pair.bias"], p["to_left.weight"], p["to_left_gate.weight"], p["to_right.weight"],
              p["to_right_gate.weight"], p["ln_out.weight"], p["ln_out.bias"], p["to_gate.weight"], p["to_out.weight"]):
        a, ptr = _as_dp(t)
        keep.append(a)
        ptrs.append(ptr)
    out = np.zeros((N, N, 128), dtype=np.float64)
    vm = None
    vptr = None
    if valid is not None:
        vm = np.ascontiguousarray(valid[0].numpy().astype(np.uint8))
        vptr = vm.ctypes.data_as(ctypes.c_void_p)
    rc = lib.trimul_ref_forward(ptrs[0], vptr, *ptrs[1:], N, 128, 128, int(outgoing), 0.03, 0.07, 1,
                                out.ctypes.data_as(ctypes.POINTER(ctypes.c_double)))
    assert rc == 0
    np.testing.assert_allclose(ref[0].numpy(), out, rtol=2e-4, atol=2e-4)


@pytest.mark.parametrize("outgoing", [True, False])
def test_all_invalid_mask_is_identity(outgoing):
    """ln_out.bias = 0 and every token masked => y == x exactly (reference: tests/test_engine_h100_masks.py:89-91)."""
    p = rand_params(42)
    p["ln_out.bias"] = torch.zeros(128)
    z = torch.randn(1, 16, 16, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    y = oracle.trimul_forward(z, p, torch.zeros(1, 16, dtype=torch.bool), outgoing=outgoing)
    assert torch.equal(y, z.float())


def test_mask_none_equals_all_true_and_gate_unmasked():
    p = rand_params(43, ln_bias_scale=0.4)
    z = torch.randn(1, 16, 16, 128, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    a = oracle.trimul_forward(z, p, None)
    b = oracle.trimul_forward(z, p, torch.ones(1, 16, dtype=torch.bool))
    assert torch.equal(a, b)
    mask = torch.ones(1, 16, dtype=torch.bool)
    mask[:, ::3] = False
    st = oracle.trimul_forward_stages(z, p, mask)
    # masked cells: left/right are zero, the update is sigmoid(gate) * (beta_out W_o^T) and not zero
    assert bool((st.left[0, 0] == 0).all()) and bool((st.right[0, :, 0] == 0).all())
    assert float(st.update[0, 0, 0].abs().max()) > 1e-3


def test_token_mask_equals_derived_pair_mask_and_einsum_directions():
    p = rand_params(44)
    g = torch.Generator().manual_seed(3)
    z = torch.randn(2, 10, 10, 128, generator=g).to(torch.bfloat16)
    tok = torch.rand(2, 10, generator=g) > 0.3
    pm = tok[:, :, None] & tok[:, None, :]
    for outgoing in (True, False):
        a = oracle.trimul_forward(z, p, tok, outgoing=outgoing)
        b = oracle.trimul_forward(z, p, None, outgoing=outgoing, pair_mask=pm)
        assert torch.equal(a, b)
    # incoming contraction of z == outgoing contraction of the transposed pair tensor (no mask)
    zt = z.transpose(1, 2).contiguous()
    st_in = oracle.trimul_forward_stages(z, p, None, outgoing=False)
    st_out_t = oracle.trimul_forward_stages(zt, p, None, outgoing=True)
    torch.testing.assert_close(st_in.tri, st_out_t.tri, rtol=1e-5, atol=1e-5)
    # channel-chunked contraction is the same contraction
    c = oracle.trimul_forward(z, p, tok, k_chunk=32)
    torch.testing.assert_close(c, oracle.trimul_forward(z, p, tok), rtol=1e-6, atol=1e-6)


def _bidir_params(seed):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return {
        "ln_pair.weight": 1.0 + 0.1 * rn(128), "ln_pair.bias": 0.2 * rn(128),
        "to_left.weight": rn(64, 128) * 128**-0.5, "to_left_gate.weight": rn(64, 128) * 128**-0.5,
        "to_right.weight": rn(64, 128) * 128**-0.5, "to_right_gate.weight": rn(64, 128) * 128**-0.5,
        "ln_out.weight": 1.0 + 0.1 * rn(64), "ln_out.bias": 0.2 * rn(64),
        "to_gate.weight": rn(128, 128) * 128**-0.5, "to_out.weight": rn(128, 64) * 64**-0.5,
    }


@pytest.mark.parametrize("with_scale", [False, True])
def test_bidirectional_oracle_matches_c_restatement(with_scale):
    """The torch restatement of the bidirectional module against the independent C one (h = 32 here: the split of the
    2h channels into an outgoing and an incoming half, the LayerNorm over all 2h, the dropout scale)."""
    lib = _c_ref()
    dp = ctypes.POINTER(ctypes.c_double)
    lib.trimul_ref_bidir_forward.restype = ctypes.c_int
    lib.trimul_ref_bidir_forward.argtypes = [dp, ctypes.c_void_p] + [dp] * 10 + [ctypes.c_void_p] + [ctypes.c_int] * 3 + [ctypes.c_double] * 2 + [ctypes.c_int, dp]
    N = 10
    p = _bidir_params(51)
    g = torch.Generator().manual_seed(52)
    z = torch.randn(1, N, N, 128, generator=g)
    mask = torch.rand(1, N, generator=g) > 0.3
    scale = (torch.rand(1, 1, N, 128, generator=g) > 0.25).float() / 0.75 if with_scale else None
    ref = oracle.bidir_forward(z, p, mask, eps_in=0.03, eps_out=0.07, drop_scale=scale)
    valid = oracle.pair_valid(mask, None, 1, N)
    keep, ptrs = [], []
    for t in (z[0], p["ln_pair.weight"], p["ln_pair.bias"], p["to_left.weight"], p["to_left_gate.weight"], p["to_right.weight"],
              p["to_right_gate.weight"], p["ln_out.weight"], p["ln_out.bias"], p["to_gate.weight"], p["to_out.weight"]):
        a, ptr = _as_dp(t)
        keep.append(a)
        ptrs.append(ptr)
    vm = np.ascontiguousarray(valid[0].numpy().astype(np.uint8))
    sc = None
    sptr = None
    if scale is not None:
        sc = np.ascontiguousarray(scale[0, 0].double().numpy())
        sptr = sc.ctypes.data_as(ctypes.c_void_p)
    out = np.zeros((N, N, 128), dtype=np.float64)
    rc = lib.trimul_ref_bidir_forward(ptrs[0], vm.ctypes.data_as(ctypes.c_void_p), *ptrs[1:], sptr, N, 128, 32, 0.03, 0.07, 1,
                                      out.ctypes.data_as(dp))
    assert rc == 0
    np.testing.assert_allclose(ref[0].numpy(), out, rtol=2e-4, atol=2e-4)
    # the halves really are contracted in different directions: swapping them changes the result
    st = oracle.bidir_forward_stages(z, p, mask)
    h = 32
    assert not torch.allclose(st.tri[..., :h], st.tri[..., h:])
    # zero dropout scale returns the input exactly (reference: scripts/check_trimul_module_reference.py:114-116)
    y0 = oracle.bidir_forward(z, p, mask, drop_scale=torch.zeros(1, 1, N, 128))
    assert torch.equal(y0, z)


def test_bidirectional_oracle_halves_equal_the_unidirectional_contractions():
    p = _bidir_params(53)
    g = torch.Generator().manual_seed(54)
    z = torch.randn(1, 9, 9, 128, generator=g)
    mask = torch.rand(1, 9, generator=g) > 0.3
    st = oracle.bidir_forward_stages(z, p, mask)
    for sl, outgoing in ((slice(0, 32), True), (slice(32, 64), False)):
        q = {k: v for k, v in p.items()}
        for k in ("to_left.weight", "to_left_gate.weight", "to_right.weight", "to_right_gate.weight"):
            q[k] = p[k][sl]
        q["ln_out.weight"], q["ln_out.bias"], q["to_out.weight"] = p["ln_out.weight"][sl], p["ln_out.bias"][sl], p["to_out.weight"][:, sl]
        uni = oracle.trimul_forward_stages(z, q, mask, outgoing=outgoing)
        torch.testing.assert_close(st.tri[..., sl], uni.tri, rtol=1e-5, atol=1e-5)


def test_transition_oracle_matches_c_restatement():
    lib = _c_ref()
    dp = ctypes.POINTER(ctypes.c_double)
    lib.transition_ref_forward.restype = ctypes.c_int
    lib.transition_ref_forward.argtypes = [dp] * 6 + [ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_int, dp]
    g = torch.Generator().manual_seed(61)
    C, n = 128, 4
    p = {"ln_in.weight": 1.0 + 0.1 * torch.randn(C, generator=g), "ln_in.bias": 0.2 * torch.randn(C, generator=g),
         "expand_a.weight": torch.randn(n * C, C, generator=g) * C**-0.5, "expand_b.weight": torch.randn(n * C, C, generator=g) * C**-0.5,
         "squeeze.weight": torch.randn(C, n * C, generator=g) * (n * C) ** -0.5}
    x = torch.randn(2, 5, 5, C, generator=g)
    ref = oracle.transition_forward(x, p, eps=0.02)
    keep, ptrs = [], []
    for t in (x.reshape(-1, C), p["ln_in.weight"], p["ln_in.bias"], p["expand_a.weight"], p["expand_b.weight"], p["squeeze.weight"]):
        a, ptr = _as_dp(t)
        keep.append(a)
        ptrs.append(ptr)
    out = np.zeros((50, C), dtype=np.float64)
    rc = lib.transition_ref_forward(*ptrs, 50, C, n * C, 0.02, 1, out.ctypes.data_as(dp))
    assert rc == 0
    np.testing.assert_allclose(ref.reshape(50, C).numpy(), out, rtol=2e-4, atol=2e-4)
    upd = oracle.transition_forward(x, p, eps=0.02, residual=False)
    torch.testing.assert_close(upd + x, ref)
