"""The committed vectors under tests/golden/ as fixed targets for the CUDA path.

Each case re-draws its inputs from the recorded seed (verified by the stored checksum), runs the module through
the C ABI on the GPU and holds the output to the stated bounds against the stored fp32 output: relative Frobenius
<= 5e-3, max abs <= 3e-2 (bf16 I/O). The all-invalid case must return the input bit for bit.
"""

import os
import sys

import numpy as np
import pytest
import torch

import miniworld_b200 as mw
from tests.helpers import assert_module_parity

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, HERE)
import make_golden  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_module_output_matches_golden_vector(name):
    case = make_golden.make_case(name)
    stored = np.load(os.path.join(HERE, name + ".npz"))
    assert str(stored["digest"]) == make_golden.input_digest(case), "inputs re-drawn from the seed differ from the recorded ones"
    want = torch.from_numpy(stored["out"])
    # the token-mask cases go through the reference-named class, the pair-mask case through the OpenFold-style
    # class whose second argument may be a [B, N, N] mask
    if case["pair_mask"] is not None:
        cls = mw.TriangleMultiplicationOutgoing if case["outgoing"] else mw.TriangleMultiplicationIncoming
        m = cls(128, check_status=True)
        arg = case["pair_mask"]
    else:
        m = mw.TriangleMultiplication(128, outgoing=case["outgoing"], check_status=True)
        arg = case["mask"]
    m.load_state_dict(case["params"])
    m = m.to(DEV).to(torch.bfloat16).eval()
    m.ln_pair.eps, m.ln_out.eps = case["eps_in"], case["eps_out"]
    with torch.no_grad():
        y = m(case["z"].to(DEV), None if arg is None else arg.to(DEV))
    # all tokens masked: the update is sigmoid(g) * (W_o beta_out), about 1e-2, below the bf16 spacing of z + update,
    # so its relative error says nothing; the output itself is still held to the bounds
    assert_module_parity(y, want, case["z"], name, check_update=(name != "out_n16_allinvalid"))
    if name == "out_n16_allinvalid":
        # every token masked: left = right = 0, t = 0, LN_out(0) = beta_out; the update is sigmoid(g) * (W_o beta_out),
        # and the stored output pins it. With beta_out = 0 the module returns its input exactly.
        p0 = dict(case["params"])
        p0["ln_out.bias"] = torch.zeros(128)
        m.load_state_dict(p0)
        with torch.no_grad():
            y0 = m(case["z"].to(DEV), case["mask"].to(DEV))
        assert torch.equal(y0.cpu(), case["z"])
