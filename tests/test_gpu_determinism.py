"""Bit-exact repeatability of the forward and of the prologue alone over many launches.

The prologue and the contraction run as pairs of CTAs that hand work to each other through shared-memory
barriers in the partner CTA. A lost ordering between the two CTAs would show as an output that differs from one
launch to the next, so every launch is compared bit for bit with the first, on the two largest benchmark shapes
with random masks. Nothing here can hang: all device-side waits are bounded.
"""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from miniworld_b200.synthetic import make_workload

pytestmark = pytest.mark.gpu
DEV = "cuda"
REPEATS = 200


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("name", ["crop768", "batch8x256"])
def test_forward_is_bit_identical_over_many_launches(name, outgoing):
    w = make_workload(name, seed=5)
    g = torch.Generator().manual_seed(55)
    mask = (torch.rand(w.B, w.N, generator=g) > 0.2).to(DEV)
    z = w.z.to(DEV)
    m = mw.TriangleMultiplication(128, outgoing=outgoing)
    m.load_state_dict(w.params)
    m = m.to(DEV).to(torch.bfloat16).eval()
    with torch.no_grad():
        first = m(z, mask).clone()
        mismatches = torch.zeros((), dtype=torch.int64, device=DEV)
        for _ in range(REPEATS):
            y = m(z, mask)
            mismatches += (y.view(torch.int16) != first.view(torch.int16)).sum()
    assert m.device_status() == 0
    assert int(mismatches) == 0, f"{int(mismatches)} differing elements over {REPEATS} launches"


@pytest.mark.parametrize("name", ["crop768", "batch8x256"])
def test_prologue_alone_is_bit_identical_over_many_launches(name):
    """Stage 1 on NaN-poisoned outputs, every launch: an element that one launch fails to write, or writes
    differently, is caught."""
    w = make_workload(name, seed=6)
    g = torch.Generator().manual_seed(66)
    B, N = w.B, w.N
    mask = (torch.rand(B, N, generator=g) > 0.2).to(DEV)
    z = w.z.to(DEV)
    packed = F_.aligned_empty(F_.packed_bytes(), torch.device(DEV))
    F_.pack_weights({k: v.to(DEV) for k, v in w.params.items()}, packed)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    left = torch.empty(B, N, 128, N, dtype=torch.float16, device=DEV)
    right = torch.empty_like(left)
    first = None
    mismatches = torch.zeros((), dtype=torch.int64, device=DEV)
    for _ in range(REPEATS):
        left.fill_(float("nan"))
        right.fill_(float("nan"))
        F_.prologue(z, packed, left, right, st, token_mask=mask)
        if first is None:
            first = (left.clone(), right.clone())
            assert torch.isfinite(left.float()).all() and torch.isfinite(right.float()).all()
        else:
            mismatches += (left.view(torch.int16) != first[0].view(torch.int16)).sum()
            mismatches += (right.view(torch.int16) != first[1].view(torch.int16)).sum()
    F_.check_status(st, "prologue soak")
    assert int(mismatches) == 0, f"{int(mismatches)} differing elements over {REPEATS} launches"
