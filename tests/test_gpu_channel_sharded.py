"""Channel-sharded multi-GPU form, emulated on ONE GPU: the P "GPUs" are run one after the other and their buffers
are ordinary local tensors, which exercises the destination lists of stage 1, the per-owner stores of stage 2 and
the grouped load of stage 3 exactly as P processes would (the kernels never wait on one another). The result must be
bit-identical to the single-GPU forward: the same kernels, the same k order, only the destinations differ."""

import pytest
import torch

import miniworld_b200 as mw
from miniworld_b200 import functional as F_
from tests.helpers import rand_params

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


@pytest.mark.parametrize("outgoing", [True, False])
@pytest.mark.parametrize("N,P", [(256, 2), (256, 4), (768, 8), (512, 4), (1024, 2), (2048, 8)])
def test_channel_sharded_emulation_equals_single_gpu(N, P, outgoing):
    p = rand_params(71)
    g = torch.Generator().manual_seed(72 + N)
    z = torch.randn(1, N, N, 128, generator=g).to(torch.bfloat16).to(DEV)
    mask = (torch.rand(1, N, generator=g) > 0.15).to(DEV)
    full = mw.TriangleMultiplication(128, outgoing=outgoing, check_status=True)
    full.load_state_dict(p)
    full = full.to(DEV).to(torch.bfloat16).eval()
    with torch.no_grad():
        want = full(z, mask)

    cg, rows = 128 // P, N // P
    nan = lambda *shape: torch.full(shape, float("nan"), dtype=torch.float16, device=DEV)  # noqa: E731
    left_g = [nan(1, N, cg, N) for _ in range(P)]   # buffer of "GPU" g: channel group g, all rows
    right_g = [nan(1, N, cg, N) for _ in range(P)]
    tri_o = [nan(P, rows, cg, N) for _ in range(P)]  # buffer of "GPU" s: its rows, one slab per channel group
    packed = F_.aligned_empty(F_.packed_bytes(), DEV)
    F_.pack_weights({k: v.to(DEV) for k, v in full._params().items()}, packed)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    for r in range(P):  # stage 1 on every "GPU"
        zr = z[:, r * rows : (r + 1) * rows].contiguous()
        F_.prologue_channels(zr, packed, left_g, right_g, st, token_mask=mask, row_begin=r * rows)
    for grp in range(P):  # stage 2
        F_.contract_channels(left_g[grp], right_g[grp], tri_o, grp, st, N, outgoing)
    got = torch.empty_like(z)
    for r in range(P):  # stage 3
        zr = z[:, r * rows : (r + 1) * rows].contiguous()
        yr = torch.empty_like(zr)
        F_.epilogue_groups(tri_o[r], zr, packed, yr, st, P)
        got[:, r * rows : (r + 1) * rows] = yr
    F_.check_status(st, "channel-sharded emulation")
    assert all(torch.isfinite(t.float()).all() for t in left_g + right_g + tri_o)
    assert torch.equal(got, want), float((got.float() - want.float()).abs().max())


def test_channel_sharded_shape_errors():
    t = torch.zeros(1, 256, 64, 256, dtype=torch.float16, device=DEV)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError):  # 3 does not divide 128
        F_.contract_channels(t, t, [t, t, t], 0, st, 256, True)
    with pytest.raises(RuntimeError):  # N / P = 40 is not a multiple of 32
        F_.contract_channels(t, t, [t] * 8, 0, st, 320, True)


def test_peer_barrier_passes_when_the_peer_has_arrived_and_times_out_otherwise():
    """The barrier between GPUs, with local arrays standing in for the peer's: it publishes this GPU's epoch, returns
    at once when the peer's epoch is already there, and a wait that nothing ends runs out after the given limit
    with device code 106 in the status word - the context stays usable."""
    mine = torch.zeros(8, dtype=torch.int32, device=DEV)
    peer = torch.zeros(8, dtype=torch.int32, device=DEV)
    st = torch.zeros(16, dtype=torch.int32, device=DEV)
    mine[1] = 3  # the "peer" (rank 1) reached epoch 3 earlier
    F_.peer_barrier([mine, peer], 0, 3, st, timeout_ms=1000)
    assert F_.read_status(st) == 0
    assert int(peer[0]) == 3  # this GPU's arrival, written into the peer's array
    F_.peer_barrier([mine, peer], 0, 4, st, timeout_ms=5)  # nobody writes epoch 4 into mine[1]
    assert F_.read_status(st) == 106
    with pytest.raises(RuntimeError, match="barrier between GPUs"):
        F_.check_status(st, "peer barrier")
    st.zero_()
    x = torch.ones(4, device=DEV) * 2  # the context still works
    assert float(x.sum()) == 8.0
