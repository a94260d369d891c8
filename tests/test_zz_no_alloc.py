"""The allocation-free forward (`b200_trimul_forward_static`) against the ordinary entry point.

Some users of the library may not allocate device memory (their pool owns the whole GPU, or their host
forbids allocation after start-up), so this entry point keeps its scratch in a fixed array inside the
library. The test drives it through the C ABI with ctypes, twice in a row with different inputs and
directions, and requires the same bytes as `b200_trimul_forward` with a caller-owned workspace: both run
the same kernels, and the shared scratch must not leak one call's contents into the next. It is collected
last so that a run which stops at the first failure has already run everything else.
"""

import ctypes

import pytest
import torch

from miniworld_b200 import _lib
from miniworld_b200 import functional as F_
from tests.helpers import params_to, rand_params

pytestmark = pytest.mark.gpu
DEV = "cuda"
E_TOO_LARGE = -8


def _call_static(z, p, mask, outgoing, residual=True, pair_mask=None, biases=None):
    lib = _lib.load()
    w = F_._Weights(p, biases, z.device)
    y = torch.full_like(z, float("nan"))
    tm = F_.as_mask_u8(mask, z.device)
    pm = F_.as_mask_u8(pair_mask, z.device)
    status_ptr = ctypes.c_void_p(0)
    B, N = int(z.shape[0]), int(z.shape[1])
    rc = lib.b200_trimul_forward_static(
        z.data_ptr(), *[t.data_ptr() for t in w.weights], w.dtype_code, *[t.data_ptr() for t in w.lns], w.bias_array,
        None if tm is None else tm.data_ptr(), None if pm is None else pm.data_ptr(), y.data_ptr(), B, N, 128, 128,
        _lib.OUTGOING if outgoing else _lib.INCOMING, 1e-5, 1e-5, int(residual), ctypes.byref(status_ptr),
        torch.cuda.current_stream().cuda_stream,
    )
    return rc, y, status_ptr


def _device_status(status_ptr):
    out = ctypes.c_int(-1)
    rc = _lib.load().b200_trimul_read_status(status_ptr, torch.cuda.current_stream().cuda_stream, ctypes.byref(out))
    assert rc == 0
    return out.value


def test_static_scratch_forward_matches_workspace_forward_twice_in_a_row():
    p = params_to(rand_params(51), DEV)
    g = torch.Generator().manual_seed(52)
    cases = [
        (torch.randn(1, 128, 128, 128, generator=g).to(torch.bfloat16), torch.rand(1, 128, generator=g) > 0.2, True),
        (torch.randn(4, 64, 64, 128, generator=g).to(torch.bfloat16), torch.rand(4, 64, generator=g) > 0.3, False),
    ]
    for z, mask, outgoing in cases:  # two calls in a row on the shared scratch
        z, mask = z.to(DEV), mask.to(DEV)
        want = F_.trimul_forward(z, p, mask, outgoing=outgoing, check=True)
        rc, got, status_ptr = _call_static(z, p, mask, outgoing)
        assert rc == 0, _lib.strerror(rc)
        assert status_ptr.value, "the status address must be reported"
        assert _device_status(status_ptr) == 0
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want), float((got.float() - want.float()).abs().max())


def test_static_scratch_forward_with_pair_mask_biases_and_no_residual():
    """The remaining arguments of the entry point: an arbitrary pair mask, gate biases, and the update alone
    (residual off) - again two calls in a row against the workspace entry point, same bytes required."""
    p = params_to(rand_params(54), DEV)
    g = torch.Generator().manual_seed(55)
    biases = {"to_left_gate": torch.ones(128, device=DEV), "to_right_gate": torch.ones(128, device=DEV),
              "to_gate": torch.linspace(-1, 1, 128).to(DEV)}
    for outgoing in (True, False):
        z = torch.randn(2, 88, 88, 128, generator=g).to(torch.bfloat16).to(DEV)
        pm = (torch.rand(2, 88, 88, generator=g) > 0.3).to(DEV)
        want = F_.trimul_forward(z, p, None, outgoing=outgoing, pair_mask=pm, residual=False, biases=biases, check=True)
        rc, got, status_ptr = _call_static(z, p, None, outgoing, residual=False, pair_mask=pm, biases=biases)
        assert rc == 0, _lib.strerror(rc)
        assert _device_status(status_ptr) == 0
        assert torch.equal(got, want), float((got.float() - want.float()).abs().max())


def test_static_scratch_forward_rejects_what_does_not_fit():
    p = params_to(rand_params(53), DEV)
    z = torch.zeros(1, 136, 136, 128, dtype=torch.bfloat16, device=DEV)  # 18496 cells > 16384
    rc, y, _ = _call_static(z, p, None, True)
    assert rc == E_TOO_LARGE
    assert "16384" in _lib.strerror(rc)
    torch.cuda.synchronize()
    assert bool(torch.isnan(y.float()).all()), "nothing may have been launched"
    z2 = torch.zeros(2, 128, 128, 128, dtype=torch.bfloat16, device=DEV)  # batch pushes it over the limit
    assert _call_static(z2, p, None, False)[0] == E_TOO_LARGE
