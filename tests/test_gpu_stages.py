"""Per-stage parity of the CUDA kernels through the C ABI (pack, prologue, contraction, epilogue).

Each stage is fed seeded inputs and compared with an fp32 torch evaluation of the same stage; outputs
and scratch are NaN-poisoned first (the reference's trick, tests/test_engine_trimul_f567_config.py:103
in the reference project) so that an unwritten element cannot pass.
"""

import pytest
import torch

from miniworld_b200 import functional as F_
from oracle import trimul_oracle as oracle
from tests.helpers import from_row_plane, params_to, rand_params, to_row_plane

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _status(dev=DEV):
    return torch.zeros(16, dtype=torch.int32, device=dev)


def _packed(params, biases=None):
    packed = F_.aligned_empty(F_.packed_bytes(), torch.device(DEV))
    packed.fill_(0xFF)
    F_.pack_weights(params_to(params, DEV), packed, biases)
    torch.cuda.synchronize()
    return packed


def _nan_bf16(*shape):
    return torch.full(shape, float("nan"), dtype=torch.bfloat16, device=DEV)


def _nan_f16(*shape):
    """NaN-poisoned fp16 buffer (the intermediates left / right / tri are fp16; tri is scaled by 2^-4)."""
    return torch.full(shape, float("nan"), dtype=torch.float16, device=DEV)


TRI_SCALE = 0.0625


@pytest.mark.parametrize("wdtype", [torch.bfloat16, torch.float32])
def test_pack_weights(wdtype):
    p = rand_params(3, dtype=wdtype)
    biases = {"to_left_gate": torch.full((128,), 1.0), "to_gate": torch.linspace(-1, 1, 128)}
    packed = _packed(p, {k: v.to(DEV) for k, v in biases.items()})
    mats = torch.cat([
        packed[: 5 * 32768].view(torch.float16).view(5, 128, 128).float().cpu(),  # fp16: meet fp16 activations
        packed[5 * 32768 : 6 * 32768].view(torch.bfloat16).view(1, 128, 128).float().cpu(),  # gate: meets bf16 z
    ])
    d1 = packed[6 * 32768 : 6 * 32768 + 2048].view(torch.float32).view(4, 128).cpu()
    c3 = packed[6 * 32768 + 2048 : 6 * 32768 + 4096].view(torch.float32).view(128, 4).cpu()
    ln = packed[6 * 32768 + 4096 : 6 * 32768 + 5120].view(torch.float32).view(2, 128).cpu()
    assert torch.equal(ln[0], p["ln_pair.weight"]) and torch.equal(ln[1], p["ln_pair.bias"])
    names = ["to_left", "to_left_gate", "to_right", "to_right_gate", "to_out", "to_gate"]
    for m, name in enumerate(names):
        w = p[name + ".weight"].float()
        gamma = p["ln_out.weight"] if name == "to_out" else p["ln_pair.weight"]
        beta = p["ln_out.bias"] if name == "to_out" else p["ln_pair.bias"]
        folded = m >= 4  # the prologue applies the input LayerNorm affine itself
        want = (0.5 * w * gamma[None, :]).to(torch.bfloat16 if name == "to_gate" else torch.float16).float() if folded else (0.5 * w).to(torch.float16).float()
        assert torch.equal(mats[m], want), name
        d = 0.5 * ((w @ beta if folded else 0.0) + biases.get(name, torch.zeros(128)))
        s = want.sum(1)
        if m < 4:
            torch.testing.assert_close(d1[m], d, rtol=1e-5, atol=1e-6)
        elif name == "to_gate":
            torch.testing.assert_close(c3[:, 0], s, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(c3[:, 1], d, rtol=1e-5, atol=1e-6)
        else:
            torch.testing.assert_close(c3[:, 2], s, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(c3[:, 3], d, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("B,N", [(1, 16), (2, 64), (1, 136), (1, 256), (1, 384), (1, 200), (1, 512), (1, 768)])
def test_contract_matches_einsum(B, N, outgoing):
    g = torch.Generator().manual_seed(100 + N)
    left = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    right = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    tri = _nan_f16(B, N, 128, N)
    st = _status()
    F_.contract(left, right, tri, st, B, N, 0, N, outgoing)
    F_.check_status(st, "contract")
    lf, rf = left.float(), right.float()
    # row-plane [b, row, h, col]
    ref = torch.einsum("bihk,bjhk->bihj", lf, rf) if outgoing else torch.einsum("bkhi,bkhj->bihj", lf, rf)
    got = tri.float() / TRI_SCALE
    assert torch.isfinite(got).all()
    rel = oracle.rel_frobenius(got.cpu(), ref.cpu())
    assert rel < 4e-4, rel  # fp16 rounding of the stored result
    # elementwise: within one fp16 ulp of the fp32 result
    err = (got - ref).abs()
    tol = ref.abs() * 2**-10 + 2e-3
    assert bool((err <= tol).all()), float((err - tol).max())


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("B,N", [(2, 64), (1, 136), (1, 200), (1, 384), (1, 512)])
def test_contract_backward_matches_einsum(B, N, outgoing):
    """Gradients of the contraction with respect to both operands (one product with a K-major and an MN-major operand,
    one in the other direction's form) against fp32 einsums, which is what autograd gives for the forward einsum."""
    g = torch.Generator().manual_seed(150 + N)
    left = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    right = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    dtri = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    dleft, dright = _nan_f16(B, N, 128, N), _nan_f16(B, N, 128, N)
    st = _status()
    F_.contract_backward(dtri, left, right, dleft, dright, st, B, N, outgoing)
    F_.check_status(st, "contract_backward")
    lf, rf, df = left.float(), right.float(), dtri.float()
    if outgoing:  # t[b,i,h,j] = sum_k l[b,i,h,k] r[b,j,h,k]
        ref_l = torch.einsum("bihj,bjhk->bihk", df, rf)
        ref_r = torch.einsum("bihj,bihk->bjhk", df, lf)
    else:  # t[b,i,h,j] = sum_k l[b,k,h,i] r[b,k,h,j]
        ref_l = torch.einsum("bihj,bkhj->bkhi", df, rf)
        ref_r = torch.einsum("bihj,bkhi->bkhj", df, lf)
    for name, got16, ref in (("dleft", dleft, ref_l), ("dright", dright, ref_r)):
        got = got16.float() / TRI_SCALE
        assert torch.isfinite(got).all(), name
        assert oracle.rel_frobenius(got.cpu(), ref.cpu()) < 4e-4, name
        err = (got - ref).abs()
        tol = ref.abs() * 2**-10 + 2e-3
        assert bool((err <= tol).all()), (name, float((err - tol).max()))


@pytest.mark.parametrize("outgoing", [True, False])
def test_contract_row_range(outgoing):
    """A row range of the output (what one rank of a row-sharded run computes) equals the slice of the full result."""
    B, N, r0, rows = 1, 192, 64, 72
    g = torch.Generator().manual_seed(7)
    left = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    right = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    full = _nan_f16(B, N, 128, N)
    st = _status()
    F_.contract(left, right, full, st, B, N, 0, N, outgoing)
    part = _nan_f16(B, rows, 128, N)
    a_in = left[:, r0 : r0 + rows].contiguous() if outgoing else left
    F_.contract(a_in, right, part, st, B, N, r0, rows, outgoing)
    F_.check_status(st, "contract")
    assert torch.equal(part, full[:, r0 : r0 + rows])


@pytest.mark.parametrize("N,slabs", [(192, [(0, 96), (96, 96)]), (200, [(0, 72), (72, 40), (112, 88)]), (384, [(0, 384)])])
def test_contract_partial_sums_to_full(N, slabs):
    """Incoming partial sums over slabs of the pair rows k (what the ranks of a k-sharded run compute) add up to the
    full contraction; a single slab covering every k is bit-identical to it."""
    B = 1
    g = torch.Generator().manual_seed(11 + N)
    left = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    right = torch.randn(B, N, 128, N, generator=g).to(torch.float16).to(DEV)
    st = _status()
    full = _nan_f16(B, N, 128, N)
    F_.contract(left, right, full, st, B, N, 0, N, False)
    acc = torch.zeros(B, N, 128, N, dtype=torch.float32, device=DEV)
    for k0, kr in slabs:
        part = _nan_f16(B, N, 128, N)
        F_.contract_partial(left[:, k0 : k0 + kr].contiguous(), right[:, k0 : k0 + kr].contiguous(), part, st, B, N, kr)
        assert torch.isfinite(part.float()).all()
        ref = torch.einsum("bkhi,bkhj->bihj", left[:, k0 : k0 + kr].float(), right[:, k0 : k0 + kr].float())
        err = (part.float() / TRI_SCALE - ref).abs()
        tol = ref.abs() * 2**-10 + 2e-3
        assert bool((err <= tol).all()), float((err - tol).max())
        acc += part.float()
    F_.check_status(st, "contract_partial")
    if len(slabs) == 1:
        assert torch.equal(part, full)
    else:
        rel = oracle.rel_frobenius(acc.cpu(), full.float().cpu())
        assert rel < 6e-4, rel  # one fp16 rounding per slab


@pytest.mark.parametrize("mask_kind", ["none", "tail", "holes", "all_invalid", "pair"])
@pytest.mark.parametrize("B,N", [(1, 16), (2, 40), (1, 128), (1, 200)])
def test_prologue_matches_oracle(B, N, mask_kind):
    p = rand_params(11)
    g = torch.Generator().manual_seed(200 + N)
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16)
    mask = pair_mask = None
    if mask_kind == "tail":
        mask = torch.ones(B, N, dtype=torch.bool)
        mask[:, N - max(1, N // 10) :] = False
    elif mask_kind == "holes":
        mask = torch.ones(B, N, dtype=torch.bool)
        mask[:, ::3] = False
    elif mask_kind == "all_invalid":
        mask = torch.zeros(B, N, dtype=torch.bool)
    elif mask_kind == "pair":
        pair_mask = torch.rand(B, N, N, generator=g) > 0.3
    st_ref = oracle.trimul_forward_stages(z, p, mask, pair_mask=pair_mask)
    packed = _packed(p)
    zd = z.to(DEV)
    left, right = _nan_f16(B, N, 128, N), _nan_f16(B, N, 128, N)
    st = _status()
    F_.prologue(zd, packed, left, right, st, token_mask=mask, pair_mask=pair_mask, row_begin=0, eps_in=1e-5)
    F_.check_status(st, "prologue")
    for name, got, ref in (("left", left, st_ref.left), ("right", right, st_ref.right)):
        got = from_row_plane(got.float().cpu())
        assert torch.isfinite(got).all(), name
        valid = oracle.pair_valid(mask, pair_mask, B, N)
        if valid is not None:
            assert bool((got[~valid] == 0).all()), name + ": masked cells must be exactly zero"
        if mask_kind == "all_invalid":
            assert bool((got == 0).all())
            continue
        rel = oracle.rel_frobenius(got, ref)
        assert rel < 1.5e-3, (name, rel)  # fp16 x_hat / weights / output, tanh.approx gate
        assert oracle.max_abs(got, ref) < 1e-2, name


def test_prologue_row_range_and_eps():
    """Rows 8..23 of a 32-token problem with a custom eps equal the same rows of the full run."""
    B, N, r0, rows = 2, 32, 8, 16
    p = rand_params(12)
    g = torch.Generator().manual_seed(5)
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16)
    mask = torch.rand(B, N, generator=g) > 0.25
    packed = _packed(p)
    st = _status()
    full_l, full_r = _nan_f16(B, N, 128, N), _nan_f16(B, N, 128, N)
    F_.prologue(z.to(DEV), packed, full_l, full_r, st, token_mask=mask, eps_in=0.03)
    part_l, part_r = _nan_f16(B, rows, 128, N), _nan_f16(B, rows, 128, N)
    F_.prologue(z[:, r0 : r0 + rows].contiguous().to(DEV), packed, part_l, part_r, st, token_mask=mask, row_begin=r0, eps_in=0.03)
    F_.check_status(st, "prologue")
    assert torch.equal(part_l, full_l[:, r0 : r0 + rows])
    assert torch.equal(part_r, full_r[:, r0 : r0 + rows])
    ref = oracle.trimul_forward_stages(z, p, mask, eps_in=0.03)
    assert oracle.rel_frobenius(from_row_plane(full_l.float().cpu()), ref.left) < 1.5e-3


@pytest.mark.parametrize("residual", [True, False])
@pytest.mark.parametrize("B,N", [(1, 16), (2, 40), (1, 128), (1, 200)])
def test_epilogue_matches_torch(B, N, residual):
    p = rand_params(13, ln_bias_scale=0.2)
    g = torch.Generator().manual_seed(300 + N)
    z = torch.randn(B, N, N, 128, generator=g).to(torch.bfloat16)
    # contraction-like magnitudes with a non-zero mean across channels
    tri = (torch.randn(B, N, N, 128, generator=g) * 3.0 + 0.7).to(torch.bfloat16)
    eps_in, eps_out = 0.03, 0.07
    pf = {k: v.float() for k, v in p.items()}
    x = torch.nn.functional.layer_norm(z.float(), (128,), pf["ln_pair.weight"], pf["ln_pair.bias"], eps_in)
    tn = torch.nn.functional.layer_norm(tri.float(), (128,), pf["ln_out.weight"], pf["ln_out.bias"], eps_out)
    upd = torch.sigmoid(x @ pf["to_gate.weight"].T) * (tn @ pf["to_out.weight"].T)
    ref = z.float() + upd if residual else upd
    packed = _packed(p)
    y = _nan_bf16(B, N, N, 128)
    st = _status()
    tri_dev = (to_row_plane(tri).float() * TRI_SCALE).to(torch.float16).to(DEV)  # what the contraction stores
    F_.epilogue(tri_dev, z.to(DEV), packed, y, st, eps_in=eps_in, eps_out=eps_out, residual=residual)
    F_.check_status(st, "epilogue")
    got = y.float().cpu()
    assert torch.isfinite(got).all()
    assert oracle.rel_frobenius(got, ref) < 5e-3
    assert oracle.max_abs(got, ref) < 3e-2
