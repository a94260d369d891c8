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
