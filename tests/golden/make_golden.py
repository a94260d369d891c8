"""Regenerates tests/golden/*.npz: seeded inputs -> oracle outputs for small cases.

Run from the repository root:  python tests/golden/make_golden.py

The reference module itself cannot be imported (its arithmetic is in the un-vendored wheel
``miniworld-engine==2.4.4``), so these vectors come from ``oracle/trimul_oracle.py`` and were checked
against the independent C restatement ``oracle/trimul_ref.c`` when they were made. They freeze the
oracle (a regression pin) and give the GPU tests fixed targets; they are not outputs of the reference.
Inputs are not stored: they are re-drawn from the recorded seeds and verified by checksum.
"""

import hashlib
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from miniworld_b200.synthetic import make_params  # noqa: E402
from oracle import trimul_oracle as oracle  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# name: (N, outgoing, mask kind, seed, eps_in, eps_out)
CASES = {
    "out_n16_nomask": (16, True, "none", 101, 1e-5, 1e-5),
    "in_n16_holes": (16, False, "holes", 102, 1e-5, 1e-5),
    "out_n24_tail_eps": (24, True, "tail", 103, 0.03, 0.07),
    "in_n16_pairmask": (16, False, "pair", 104, 1e-5, 1e-5),
    "out_n16_allinvalid": (16, True, "all_invalid", 105, 1e-5, 1e-5),
}


def make_case(name):
    N, outgoing, kind, seed, eps_in, eps_out = CASES[name]
    g = torch.Generator().manual_seed(seed)
    params = make_params(g, 128, 128, torch.bfloat16)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
    mask = pair_mask = None
    if kind == "holes":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, ::3] = False
    elif kind == "tail":
        mask = torch.ones(1, N, dtype=torch.bool)
        mask[:, N - 3 :] = False
    elif kind == "all_invalid":
        mask = torch.zeros(1, N, dtype=torch.bool)
    elif kind == "pair":
        pair_mask = torch.rand(1, N, N, generator=g) > 0.3
    return dict(N=N, outgoing=outgoing, params=params, z=z, mask=mask, pair_mask=pair_mask, eps_in=eps_in, eps_out=eps_out)


def input_digest(case) -> str:
    h = hashlib.sha256()
    h.update(case["z"].view(torch.int16).numpy().tobytes())
    for k in oracle.PARAM_KEYS:
        v = case["params"][k]
        h.update((v.view(torch.int16) if v.dtype == torch.bfloat16 else v).numpy().tobytes())
    for k in ("mask", "pair_mask"):
        if case[k] is not None:
            h.update(case[k].numpy().tobytes())
    return h.hexdigest()


def run_oracle(case):
    st = oracle.trimul_forward_stages(
        case["z"], case["params"], case["mask"], outgoing=case["outgoing"], eps_in=case["eps_in"], eps_out=case["eps_out"],
        pair_mask=case["pair_mask"],
    )
    return st


def main():
    for name in CASES:
        case = make_case(name)
        st = run_oracle(case)
        np.savez(
            os.path.join(HERE, name + ".npz"),
            out=st.out.numpy().astype(np.float32),
            tri_sample=st.tri[0, : min(4, case["N"])].numpy().astype(np.float32),
            digest=np.array(input_digest(case)),
        )
        print(name, "written", float(st.out.abs().mean()))


if __name__ == "__main__":
    main()
