"""Host-side logic that needs no GPU: module surface (constructor, state_dict, aliases, dtype policy, loud errors),
synthetic workloads, shard planning, and the row-sharded collective schedule on two gloo ranks."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import miniworld_b200 as mw
from miniworld_b200 import sharded, synthetic
from oracle import trimul_oracle as oracle
from tests.helpers import rand_params

REFERENCE_KEYS = [
    "ln_pair.weight", "ln_pair.bias", "to_left.weight", "to_left_gate.weight", "to_right.weight",
    "to_right_gate.weight", "ln_out.weight", "ln_out.bias", "to_gate.weight", "to_out.weight",
]


def test_state_dict_layout_matches_the_reference_module():
    m = mw.TriangleMultiplication(128)
    assert list(m.state_dict().keys()) == REFERENCE_KEYS
    assert all(v.shape == (128, 128) for k, v in m.state_dict().items() if k.startswith("to_"))
    # the reference zero-initialises the two output linears
    assert float(m.to_gate.weight.abs().max()) == 0.0 and float(m.to_out.weight.abs().max()) == 0.0
    m.load_state_dict(rand_params(1))
    m2 = mw.TriangleMultiplication(128, outgoing=False, implementation="miniworld", p_drop=0.25)
    m2.load_state_dict(m.state_dict())
    assert not m2.outgoing and m2.p_drop == 0.25


def test_layernorm_affine_stays_fp32_and_linears_follow_the_module_dtype():
    p = rand_params(3)
    m = mw.TriangleMultiplication(128)
    m.load_state_dict(p)
    m = m.to(torch.bfloat16)
    assert m.ln_pair.weight.dtype == torch.float32 and m.ln_out.bias.dtype == torch.float32
    assert m.to_left.weight.dtype == torch.bfloat16
    # pinned, not converted there and back: the fp32 values survive the module-wide cast bit for bit
    for k in ("ln_pair.weight", "ln_pair.bias", "ln_out.weight", "ln_out.bias"):
        assert torch.equal(m.state_dict()[k], p[k]), k
    m.ln_pair.eps = 0.03  # mutable attribute read at call time
    assert m.ln_pair.eps == 0.03


def test_openfold_alias_round_trip():
    p = rand_params(2)
    of = mw.to_openfold_state_dict(p)
    assert set(of) == {
        "layer_norm_in.weight", "layer_norm_in.bias", "linear_a_p.weight", "linear_a_g.weight", "linear_b_p.weight",
        "linear_b_g.weight", "layer_norm_out.weight", "layer_norm_out.bias", "linear_g.weight", "linear_z.weight",
    }
    back = mw.from_openfold_state_dict(of)
    assert list(back) == list(p) and all(torch.equal(back[k], p[k]) for k in p)
    of["linear_g.bias"] = torch.ones(128)
    with pytest.raises(KeyError):
        mw.from_openfold_state_dict(of)
    m = mw.TriangleMultiplicationIncoming(128, residual=False)
    assert not m.outgoing and not m.residual


def test_unsupported_configurations_raise():
    with pytest.raises(NotImplementedError):
        mw.TriangleMultiplication(64)  # 64 contracted channels in one direction
    with pytest.raises(NotImplementedError):
        mw.TriangleMultiplication(128, d_hidden=256)
    with pytest.raises(NotImplementedError):
        mw.BidirectionalTriangleMultiplication(64, d_hidden=128)
    with pytest.raises(NotImplementedError):
        mw.TriangleMultiplication(64, d_hidden=128, p_drop=0.25)
    m64 = mw.TriangleMultiplication(64, d_hidden=128)  # the template blocks' shape
    assert m64.to_left.weight.shape == (128, 64) and m64.to_out.weight.shape == (64, 128) and m64.ln_out.weight.shape == (128,)
    b64 = mw.BidirectionalTriangleMultiplication(64)
    assert b64.to_left.weight.shape == (128, 64) and b64.to_gate.weight.shape == (64, 64) and b64.ln_out.weight.shape == (128,)
    with pytest.raises(ValueError):
        mw.TriangleMultiplication(128, implementation="cuequivariance")
    m = mw.TriangleMultiplication(128)
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16))  # no CPU implementation, no fallback
    with pytest.raises(RuntimeError, match="CUDA"):  # the differentiable path has no CPU implementation either
        m(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16, requires_grad=True))
    with pytest.raises(RuntimeError, match="CUDA"):
        mw.BidirectionalTriangleMultiplication(64)(torch.zeros(1, 8, 8, 64, dtype=torch.bfloat16, requires_grad=True))
    with pytest.raises(RuntimeError, match="CUDA"):
        mw.Transition(128)(torch.zeros(1, 8, 8, 128, dtype=torch.bfloat16, requires_grad=True))
    with pytest.raises(RuntimeError):
        mw.TriangleMultiplication(128).eval()(torch.zeros(1, 8, 8, 128), torch.ones(1, 8, 8, dtype=torch.bool))


def test_synthetic_workloads_are_deterministic_and_shaped():
    a = synthetic.make_workload("n384", seed=3, n_override=32)
    b = synthetic.make_workload("n384", seed=3, n_override=32)
    assert torch.equal(a.z, b.z) and torch.equal(a.mask, b.mask)
    assert a.z.dtype == torch.bfloat16 and a.z.shape == (1, 32, 32, 128)
    assert int((~a.mask).sum()) == 3  # last ~10 % of the tokens padded
    c = synthetic.make_workload("batch8x256", seed=0, n_override=16)
    assert c.z.shape[0] == 8 and bool(c.mask[:, 0].all())  # tails padded, heads valid
    d = synthetic.make_workload("cpu128", seed=0, n_override=8)
    assert d.z.dtype == torch.float32 and d.directions == ("outgoing",)
    f = synthetic.flops(1, 768)
    assert abs(f["contraction"] - 115.96e9) < 1e8 and abs(f["projection"] - 115.96e9) < 1e8
    assert synthetic.pass_bytes(1, 768) == 150994944


def test_shard_planning():
    assert [sharded.row_range(768, 4, r) for r in range(4)] == [(0, 192), (192, 192), (384, 192), (576, 192)]
    with pytest.raises(ValueError):
        sharded.row_range(100, 8, 0)
    with pytest.raises(ValueError):
        sharded.row_range(768, 4, 4)
    parts = [sharded.shard_batch(8, 3, r) for r in range(3)]
    assert parts == [(0, 3), (3, 3), (6, 2)]
    assert sum(c for _, c in parts) == 8


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_contraction_scheme_choice():
    # the channel scheme needs P | 128, N/P a multiple of 32 and an N the CTA-pair contraction handles
    assert sharded.channels_feasible(768, 8) and sharded.channels_feasible(768, 2) and sharded.channels_feasible(2048, 8)
    assert not sharded.channels_feasible(384, 8)      # 48 rows per rank
    assert not sharded.channels_feasible(384, 4)      # 384 rows pad to 512: more than a quarter
    assert not sharded.channels_feasible(768, 3) and not sharded.channels_feasible(128, 2)
    # fewer bytes per rank from four GPUs on
    assert sharded.choose_contraction(768, 2) == "rows" and sharded.choose_contraction(768, 4) == "channels"
    assert sharded.choose_contraction(768, 8) == "channels" and sharded.choose_contraction(384, 8) == "rows"
    with pytest.raises(ValueError):
        sharded.RowShardedTriangleMultiplication(128, contraction="channels", transport="nccl")


def _row_sharded_worker(rank, world, port, scheme, ret):
    outgoing = scheme in ("outgoing", "channels_outgoing")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N = 16
        p = rand_params(5)
        g = torch.Generator().manual_seed(11)
        z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16)
        mask = torch.rand(1, N, generator=g) > 0.2
        begin, rows = sharded.row_range(N, world, rank)
        # the schedule of RowShardedTriangleMultiplication.forward with the oracle's stages standing in for
        # the three kernels: local prologue -> all-gather of the contracted operand(s) -> local contraction, or
        # (incoming, "reduce") local partial contraction over the rank's rows k -> reduce-scatter over i
        full = oracle.trimul_forward_stages(z, p, mask, outgoing=outgoing)
        left_loc = full.left[:, begin : begin + rows].permute(0, 1, 3, 2).contiguous()   # row-plane [1, rows, H, N]
        right_loc = full.right[:, begin : begin + rows].permute(0, 1, 3, 2).contiguous()
        right_all = torch.empty(1, N, 128, N)
        if scheme.startswith("channels"):
            # channel-sharded contraction; all-to-alls stand in for the stores into the destination GPUs' buffers.
            # stage 1: channel group g of this rank's rows -> rank g, which ends up with [N, 128/P, N] (rows rank-major)
            cg = 128 // world
            ops = []
            for loc in (left_loc, right_loc):
                send = loc.view(rows, world, cg, N).permute(1, 0, 2, 3).contiguous()  # [group][rows][cg][N]
                recv = torch.empty(world, rows, cg, N)
                dist.all_to_all_single(recv, send)
                ops.append(recv.view(1, N, cg, N))
            lg, rg = ops
            # stage 2 on this rank's channel group for ALL rows; row block s of the result -> slab `rank` of rank s
            tri_c = torch.einsum("bihk,bjhk->bihj", lg, rg) if outgoing else torch.einsum("bkhi,bkhj->bihj", lg, rg)
            slabs = torch.empty(world, rows, cg, N)
            dist.all_to_all_single(slabs, tri_c.view(world, rows, cg, N).contiguous())
            # stage 3 reads [P, rows, 128/P, N]: slab g holds channel group g of this rank's rows
            tri = slabs.permute(1, 0, 2, 3).reshape(1, rows, 128, N)
        elif scheme == "incoming_reduce":
            partial = torch.einsum("bkhi,bkhj->bihj", left_loc, right_loc).contiguous()  # all (i, j), own k
            tri = torch.empty(1, rows, 128, N)
            dist.reduce_scatter_tensor(tri.view(rows, 128, N), partial.view(N, 128, N))
        elif outgoing:
            dist.all_gather_into_tensor(right_all.view(N, 128, N), right_loc.view(rows, 128, N))
            tri = torch.einsum("bihk,bjhk->bihj", left_loc, right_all)
        else:
            dist.all_gather_into_tensor(right_all.view(N, 128, N), right_loc.view(rows, 128, N))
            left_all = torch.empty(1, N, 128, N)
            dist.all_gather_into_tensor(left_all.view(N, 128, N), left_loc.view(rows, 128, N))
            tri = torch.einsum("bkhi,bkhj->bihj", left_all[..., begin : begin + rows], right_all)
        want = full.tri[:, begin : begin + rows].permute(0, 1, 3, 2)
        ret[rank] = float((tri - want).abs().max())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scheme", ["outgoing", "incoming_gather", "incoming_reduce", "channels_outgoing",
                                    "channels_incoming"])
def test_row_sharded_schedule_on_two_gloo_ranks(scheme):
    """The gathered row-plane tensor is the full operand with no repacking, the partial-sum tensor splits into the
    ranks' row blocks the same way, the channel-group buffers [N, 128/P, N] and [P, rows, 128/P, N] of the
    channel-sharded form hold what stages 2 and 3 expect, and each rank's rows of the contraction equal the
    unsharded result (world_size 2, gloo, CPU)."""
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_row_sharded_worker, args=(world, port, scheme, ret), nprocs=world, join=True)
        assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)


class _FakeSymmMem:
    """Stand-in for torch's symmetric-memory module on CPU: ``empty`` fails on the ranks listed in ``fail_on``."""

    def __init__(self, rank, fail_on):
        self.rank, self.fail_on = rank, fail_on

    def empty(self, numel, dtype, device):
        if self.rank in self.fail_on:
            raise RuntimeError("out of memory (injected)")
        return torch.empty(numel, dtype=dtype, device=device)

    def rendezvous(self, t, group):
        raise AssertionError("handles must not be exchanged unless every rank holds all of its buffers")


def _symmetric_failure_worker(rank, world, port, explicit, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import warnings

        sharded._symm_mem = lambda: _FakeSymmMem(rank, fail_on={1})
        m = sharded.RowShardedTriangleMultiplication(128, transport="p2p" if explicit else "auto")
        dev = torch.device("cpu")
        try:
            with warnings.catch_warnings(record=True) as caught:
                warnings.simplefilter("always")
                out = m._symmetric(256, world, dev)
            ret[rank] = ("fallback", out is None, m.transport, m.contraction, len(caught))
        except RuntimeError as exc:
            ret[rank] = ("raised", "p2p" in str(exc))
        # both ranks are still in step: one more collective completes
        t = torch.ones(1)
        dist.all_reduce(t)
        assert float(t) == world
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("explicit", [True, False])
def test_symmetric_setup_failure_on_one_rank_does_not_split_the_ranks(explicit):
    """One rank cannot allocate its symmetric buffers: every rank still runs the same collectives, then all of them
    raise (transport asked for by name) or all of them fall back to NCCL with a warning (world_size 2, gloo, CPU)."""
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_symmetric_failure_worker, args=(world, port, explicit, ret), nprocs=world, join=True)
        assert len(ret) == world
        for rank in range(world):
            if explicit:
                assert ret[rank] == ("raised", True), dict(ret)
            else:
                assert ret[rank] == ("fallback", True, "nccl", "rows", 1), dict(ret)
