"""Multi-GPU forms of the triangle multiplicative update (one process per GPU, ``torch.distributed``).

Two schemes, neither present in the reference (it only has data-parallel training):

* :class:`RowShardedTriangleMultiplication` - the pair tensor is sharded by rows ``i`` (B = 1). The prologue
  and the epilogue are local to the rows a rank owns. The contraction needs the other ranks' rows of the
  contracted operand(s), which are all-gathered into local HBM (NCCL) and then read by local TMA loads; no
  kernel ever loads from a peer's memory.
    outgoing  t[i in I_r, j] = sum_k a[i,k] b[j,k]     -> all-gather of ``right`` (rows j)
    incoming  t[i, j] = sum_r sum_{k in I_r} a[k,i] b[k,j] -> every rank sums over the rows k it owns, for ALL
                                                           (i, j), and a reduce-scatter over i adds the partial
                                                           sums (one tensor crosses the links instead of two).
                                                           ``incoming="gather"`` selects the older scheme, an
                                                           all-gather of ``left`` and ``right`` (rows k), which is
                                                           bit-identical to the single-GPU forward.
  The row-plane layout [rows, H, N] makes the gathered tensor [P, N/P, H, N] == [N, H, N] with no repacking, and
  the partial-sum tensor [N, H, N] splits into the ranks' row blocks the same way.

  Two transports move those tensors. ``"nccl"``: ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` between the
  kernels. ``"p2p"``: the kernels themselves use the other GPUs' memory (buffers from torch's symmetric memory,
  mapped into every process) - the prologue's TMA stores write each tile of ``right`` into every GPU's gathered
  copy as it is produced, and a reduce kernel reads the peers' partial sums with plain loads; the only collective
  left is a one-element all-reduce that orders "my kernel has finished" before "the peers read / I read". No
  kernel waits on another GPU, and no load is a multicast load. Two buffers alternate between calls, so a rank
  that runs ahead writes the buffer its peers are not reading.
* :func:`shard_batch` - plain batch data parallelism for B > 1: samples are independent, no collective.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import functional as F_
from .modules import TriangleMultiplication

D = 128


def row_range(n_rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [begin, begin+count) owned by ``rank``: equal contiguous blocks; N must divide evenly."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad world/rank {world}/{rank}")
    if n_rows % world != 0:
        raise ValueError(f"row sharding needs N divisible by the world size (N={n_rows}, world={world})")
    count = n_rows // world
    return rank * count, count


def shard_batch(batch: int, world: int, rank: int) -> tuple[int, int]:
    """Samples [begin, begin+count) of a batch owned by ``rank`` (contiguous, remainder to the first ranks)."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad world/rank {world}/{rank}")
    base, rem = divmod(batch, world)
    count = base + (1 if rank < rem else 0)
    begin = rank * base + min(rank, rem)
    return begin, count


class RowShardedTriangleMultiplication(TriangleMultiplication):
    """Same parameters and state_dict as :class:`TriangleMultiplication`; ``forward`` takes the local rows.

    ``forward(pair_rows [1, N/P, N, 128] bf16, mask Bool[1, N] | None) -> [1, N/P, N, 128]``: the rows
    ``rank*N/P ...`` of ``pair + update``. Every rank must call it (it contains a collective).
    """

    def __init__(self, d_pair: int = D, d_hidden: Optional[int] = None, outgoing: bool = True, group=None,
                 incoming: str = "reduce", transport: str = "auto", **kw):
        super().__init__(d_pair, d_hidden, outgoing=outgoing, **kw)
        if incoming not in ("reduce", "gather"):
            raise ValueError(f"incoming must be 'reduce' or 'gather', got {incoming!r}")
        if transport not in ("auto", "p2p", "nccl"):
            raise ValueError(f"transport must be 'auto', 'p2p' or 'nccl', got {transport!r}")
        self.group = group
        self.incoming_scheme = incoming
        self.transport = "nccl" if (not outgoing and incoming == "gather") else transport
        self._bufs = None
        self._sym = None
        self._calls = 0

    def _symmetric(self, N: int, device: torch.device):
        """Two [1, N, 128, N] fp16 buffers in symmetric memory with every rank's view of them, or None (NCCL path).

        Collective: every rank allocates and exchanges handles on the first call for a given N."""
        if self.transport == "nccl":
            return None
        if self._sym is not None and self._sym[0] == (N, device):
            return self._sym[1]
        import torch.distributed._symmetric_memory as symm_mem

        group = self.group if self.group is not None else dist.group.WORLD
        world = dist.get_world_size(group)
        ok = torch.ones(1, device=device)
        views, owners = [], []
        try:
            for _ in range(2):
                t = symm_mem.empty(N * D * N, dtype=torch.float16, device=device)
                hdl = symm_mem.rendezvous(t, group)
                owners.append((t, hdl))  # the views below do not keep the allocation alive
                views.append([hdl.get_buffer(r, (1, N, D, N), torch.float16) for r in range(world)])
        except Exception as exc:  # no peer access between the GPUs, or no symmetric memory in this build
            if self.transport == "p2p":
                raise RuntimeError(f"transport='p2p' needs torch symmetric memory between the ranks: {exc!r}") from exc
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)  # all ranks take the same path
        if float(ok.item()) == 0.0:
            self.transport = "nccl"
            self._sym = None
            return None
        self.transport = "p2p"
        self._sym = ((N, device), views, owners)
        return views

    def _scratch(self, N: int, rows: int, device: torch.device):
        key = (N, rows, device)
        if self._bufs is None or self._bufs[0] != key:
            plane = lambda r: torch.empty(1, r, D, N, dtype=torch.float16, device=device)  # noqa: E731
            nccl = self.transport == "nccl"
            gather = nccl and (self.outgoing or self.incoming_scheme == "gather")
            bufs = dict(
                flag=torch.zeros(1, device=device),
                packed=F_.aligned_empty(F_.packed_bytes(), device),
                status=torch.zeros(16, dtype=torch.int32, device=device),
                left=plane(rows),
                right=plane(rows),
                right_all=plane(N) if gather else None,
                left_all=plane(N) if gather and not self.outgoing else None,
                tri_partial=plane(N) if nccl and not gather else None,
                tri=plane(rows),
            )
            self._bufs = (key, bufs)
        return self._bufs[1]

    def forward(self, pair_rows: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if torch.is_grad_enabled() and pair_rows.requires_grad:
            raise NotImplementedError("backward is not implemented")
        if not pair_rows.is_cuda:
            raise RuntimeError("pair rows must be a CUDA tensor: this module has no CPU implementation")
        world = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        if pair_rows.dim() != 4 or pair_rows.shape[0] != 1 or pair_rows.shape[3] != D:
            raise RuntimeError(f"pair rows must be [1, N/P, N, {D}], got {tuple(pair_rows.shape)}")
        rows, N = int(pair_rows.shape[1]), int(pair_rows.shape[2])
        begin, count = row_range(N, world, rank)
        if count != rows:
            raise RuntimeError(f"rank {rank} of {world} owns {count} rows of N={N}, got {rows}")
        z = pair_rows.detach().to(torch.bfloat16).contiguous()
        dev = z.device
        sym = self._symmetric(N, dev)  # settles the transport before the scratch buffers are sized
        b = self._scratch(N, rows, dev)
        F_.pack_weights(self._params(), b["packed"], self._biases)
        b["status"].zero_()
        has_bias = bool(self._biases) and any(self._biases.get(k) is not None for k in F_.BIAS_ORDER[:4])
        pro = dict(token_mask=mask, row_begin=begin, eps_in=float(self.ln_pair.eps), has_bias=has_bias)
        if sym is not None:
            self._tri_p2p(z, b, sym, pro, N, begin, rows, world, rank)
        else:
            self._tri_nccl(z, b, pro, N, begin, rows)
        y = torch.empty_like(z)
        F_.epilogue(b["tri"], z, b["packed"], y, b["status"], eps_in=float(self.ln_pair.eps),
                    eps_out=float(self.ln_out.eps), residual=self.residual)
        if self.check_status:
            F_.check_status(b["status"], "row-sharded trimul")
        return y

    def _tri_p2p(self, z, b, sym, pro, N, begin, rows, world, rank) -> None:
        """Stages 1 and 2 with the kernels writing to / reading from the peers' memory."""
        views = sym[self._calls & 1]  # every rank makes the same number of calls, so all pick the same buffer
        self._calls += 1
        mine = views[rank]
        if self.outgoing:
            peers = [views[r] for r in range(world) if r != rank]
            F_.prologue_push(z, b["packed"], b["left"], mine, peers, b["status"], **pro)
            dist.all_reduce(b["flag"], group=self.group)  # every rank's stores have landed in every copy
            F_.contract(b["left"], mine, b["tri"], b["status"], 1, N, begin, rows, True)
        else:
            F_.prologue(z, b["packed"], b["left"], b["right"], b["status"], **pro)
            F_.contract_partial(b["left"], b["right"], mine, b["status"], 1, N, rows)
            dist.all_reduce(b["flag"], group=self.group)  # every rank's partial sums are complete
            F_.reduce_partials(b["tri"], views, N, begin, rows)  # rank order: the same sum on every run

    def _tri_nccl(self, z, b, pro, N, begin, rows) -> None:
        """Stages 1 and 2 with NCCL collectives between the kernels (B = 1: the collectives work on [rows, 128, N]
        views, so that the rank-major concatenation is the row dimension)."""
        F_.prologue(z, b["packed"], b["left"], b["right"], b["status"], **pro)
        if self.outgoing:
            dist.all_gather_into_tensor(b["right_all"].view(N, D, N), b["right"].view(rows, D, N), group=self.group)
            F_.contract(b["left"], b["right_all"], b["tri"], b["status"], 1, N, begin, rows, True)
        elif self.incoming_scheme == "gather":
            dist.all_gather_into_tensor(b["right_all"].view(N, D, N), b["right"].view(rows, D, N), group=self.group)
            dist.all_gather_into_tensor(b["left_all"].view(N, D, N), b["left"].view(rows, D, N), group=self.group)
            F_.contract(b["left_all"], b["right_all"], b["tri"], b["status"], 1, N, begin, rows, False)
        else:
            # partial sum over this rank's rows k for every (i, j), then the ranks' partials are added row block
            # by row block (fp16 sums of values already scaled by 2^-4)
            F_.contract_partial(b["left"], b["right"], b["tri_partial"], b["status"], 1, N, rows)
            dist.reduce_scatter_tensor(b["tri"].view(rows, D, N), b["tri_partial"].view(N, D, N), group=self.group)
