"""Multi-GPU forms of the triangle multiplicative update (one process per GPU, ``torch.distributed``).

Neither is present in the reference (it only has data-parallel training):

* :class:`RowShardedTriangleMultiplication` - the pair tensor is sharded by rows ``i`` (B = 1): every rank passes
  and gets back its rows. The prologue and the epilogue are local to those rows; the contraction in between needs
  data of the other ranks, and there are two ways to split it:

  ``contraction="rows"`` - each rank contracts for its own output rows.
    outgoing  t[i in I_r, j] = sum_k a[i,k] b[j,k]          -> every rank needs all rows j of ``right``
    incoming  t[i, j] = sum_r sum_{k in I_r} a[k,i] b[k,j]  -> every rank sums over the rows k it owns, for ALL
                                                               (i, j), and the partial sums are added per row
                                                               block (one tensor crosses the links, not two).
                                                               ``incoming="gather"`` selects the older scheme, an
                                                               all-gather of ``left`` and ``right`` (rows k), which
                                                               is bit-identical to the single-GPU forward.
    Per direction every rank sends or receives (P-1)/P of one [N, 128, N] tensor.

  ``contraction="channels"`` - rank g contracts the 128/P channels of group g for ALL rows (channels play the role
    the heads play in sequence-parallel attention). Each rank sends (P-1)/P of its own 1/P of ``left`` and ``right``
    and receives as much, then sends (P-1)/P of its 1/P of the result: about 3/P of a tensor per direction, less
    than the row scheme from P = 4 on, and bit-identical to the single-GPU forward.

  Two transports. ``"p2p"``: the kernels themselves use the other GPUs' memory (buffers from torch's symmetric
  memory, mapped into every process) - the prologue's and the contraction's TMA stores write each tile into the
  buffer of the GPU that needs it as the tile is produced, and (row scheme, incoming) a reduce kernel reads the
  peers' partial sums with plain loads; between the stages a one-thread-per-peer barrier kernel exchanges epoch
  flags through the same peer memory (bounded wait: it reports through the status word instead of hanging) to
  order "my kernel has finished" before "the peers read / I read". No compute kernel waits on another GPU, and no
  load is a multicast load. Two sets of buffers alternate between calls, so a rank that runs ahead writes the set its peers are not
  reading. ``"nccl"`` (row scheme only): ``all_gather_into_tensor`` / ``reduce_scatter_tensor`` between the
  kernels; the row-plane layout [rows, H, N] makes the gathered tensor [P, N/P, H, N] == [N, H, N] with no
  repacking, and the partial-sum tensor splits into the ranks' row blocks the same way.
* :func:`shard_batch` - plain batch data parallelism for B > 1: samples are independent, no collective.
"""

from __future__ import annotations

from typing import Optional

import warnings

import torch
import torch.distributed as dist

from . import functional as F_
from .modules import TriangleMultiplication

D = 128


def _symm_mem():
    """torch's symmetric-memory module (imported late: it needs a CUDA build of torch)."""
    import torch.distributed._symmetric_memory as symm_mem

    return symm_mem


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


def channels_feasible(n: int, world: int) -> bool:
    """Whether the channel-sharded contraction can run: P divides 128 into groups of at least 8 channels, every
    32-row slice of the result has one owner, and the CTA-pair contraction kernel (the one that stores per owner)
    is the kernel chosen for N rows (N >= 256 padded to 256-row tiles by at most a quarter)."""
    if world < 2 or D % world != 0 or D // world < 8 or n % world != 0 or (n // world) % 32 != 0:
        return False
    return n >= 256 and ((-n) % 256) * 4 <= n


def choose_contraction(n: int, world: int) -> str:
    """Fewer bytes per rank: the row scheme moves (P-1)/P of a tensor per direction, the channel scheme 3(P-1)/P^2."""
    return "channels" if world >= 4 and channels_feasible(n, world) else "rows"


class RowShardedTriangleMultiplication(TriangleMultiplication):
    """Same parameters and state_dict as :class:`TriangleMultiplication`; ``forward`` takes the local rows.

    ``forward(pair_rows [1, N/P, N, 128] bf16, mask Bool[1, N] | None) -> [1, N/P, N, 128]``: the rows
    ``rank*N/P ...`` of ``pair + update``. Every rank must call it (it contains a collective).
    """

    def __init__(self, d_pair: int = D, d_hidden: Optional[int] = None, outgoing: bool = True, group=None,
                 incoming: str = "reduce", transport: str = "auto", contraction: str = "auto", **kw):
        super().__init__(d_pair, d_hidden, outgoing=outgoing, **kw)
        if incoming not in ("reduce", "gather"):
            raise ValueError(f"incoming must be 'reduce' or 'gather', got {incoming!r}")
        if transport not in ("auto", "p2p", "nccl"):
            raise ValueError(f"transport must be 'auto', 'p2p' or 'nccl', got {transport!r}")
        if contraction not in ("auto", "rows", "channels"):
            raise ValueError(f"contraction must be 'auto', 'rows' or 'channels', got {contraction!r}")
        if contraction == "channels" and transport == "nccl":
            raise ValueError("the channel-sharded contraction stores into peer memory: it needs transport 'p2p'")
        self.group = group
        self.incoming_scheme = incoming
        self.transport = "nccl" if (contraction != "channels" and not outgoing and incoming == "gather") else transport
        self.contraction = contraction
        self._explicit = transport == "p2p" or contraction == "channels"  # asked for by name: no silent fallback
        self._bufs = None
        self._sym = None
        self._calls = 0
        self._epoch = 0
        self.barrier_timeout_ms = 2000

    # ------------------------------------------------------------------ buffers
    def _symmetric(self, N: int, world: int, device: torch.device):
        """Two sets of fp16 buffers in symmetric memory, each entry the list of every rank's view of one buffer, or
        None (NCCL path). Settles ``self.transport`` and ``self.contraction``.

        Collective: every rank allocates and exchanges handles on the first call for a given N."""
        if self.contraction == "auto":
            self.contraction = choose_contraction(N, world) if self.transport != "nccl" else "rows"
        if self.contraction == "channels" and not channels_feasible(N, world):
            raise RuntimeError(f"the channel-sharded contraction cannot run for N={N} on {world} GPUs")
        if self.transport == "nccl":
            return None
        if self._sym is not None and self._sym[0] == (N, device):
            return self._sym[1]
        group = self.group if self.group is not None else dist.group.WORLD
        rows, cg = N // world, D // world
        if self.contraction == "channels":
            shapes = {"left": (1, N, cg, N), "right": (1, N, cg, N), "tri": (world, rows, cg, N)}
        else:
            shapes = {"full": (1, N, D, N)}  # gathered `right` (outgoing) or the partial sums (incoming)

        # Two phases, each closed by the same all-reduce on every rank whatever happened locally, so that a failure
        # on one rank (out of memory, no peer mapping) can never leave the others waiting inside a collective:
        # phase 1 allocates everything locally (no communication), phase 2 exchanges the handles (a collective per
        # buffer, entered only when every rank holds all of its buffers).
        allocs, err = [], None
        try:
            symm_mem = _symm_mem()
            t = symm_mem.empty(8, dtype=torch.int32, device=device)
            t.zero_()
            allocs.append(("flags", None, t))
            for _ in range(2):
                for name, shape in shapes.items():
                    numel = 1
                    for d in shape:
                        numel *= d
                    allocs.append((name, shape, symm_mem.empty(numel, dtype=torch.float16, device=device)))
        except Exception as exc:  # no symmetric memory in this build, or the allocation failed on this rank
            err = exc
        if not self._agree(err is None, device):
            return self._no_p2p(err, "allocating symmetric memory failed on at least one rank")
        sets, owners, flags = [], [], None
        try:
            for name, shape, t in allocs:
                hdl = symm_mem.rendezvous(t, group)
                owners.append((t, hdl))  # the views below do not keep the allocation alive
                if name == "flags":
                    flags = [hdl.get_buffer(r, (8,), torch.int32) for r in range(world)]
                    continue
                if not sets or name in sets[-1]:
                    sets.append({})
                sets[-1][name] = [hdl.get_buffer(r, shape, torch.float16) for r in range(world)]
        except Exception as exc:  # no peer access between the GPUs
            err = exc
        if not self._agree(err is None, device):
            return self._no_p2p(err, "mapping the peers' symmetric memory failed on at least one rank")
        # (the all-reduce above also orders every rank's zeroing of its flags before any peer's first barrier)
        self.transport = "p2p"
        self._flags = flags
        self._epoch = 0
        self._sym = ((N, device), sets, owners)
        return sets

    def _agree(self, ok: bool, device: torch.device) -> bool:
        """True iff ``ok`` holds on every rank (one all-reduce, issued by every rank on every path)."""
        t = torch.full((1,), 1.0 if ok else 0.0, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return float(t.item()) != 0.0

    def _no_p2p(self, err, what: str):
        """Every rank arrives here together. Asked for by name: raise everywhere; otherwise warn once and use NCCL."""
        if self._explicit:
            raise RuntimeError(f"transport 'p2p' needs torch symmetric memory between the ranks: {what}"
                               + (f" (this rank: {err!r})" if err is not None else ""))
        warnings.warn(f"RowShardedTriangleMultiplication: {what}; using NCCL collectives and the row scheme instead"
                      + (f" (this rank: {err!r})" if err is not None else ""), RuntimeWarning, stacklevel=3)
        self.transport = "nccl"
        self.contraction = "rows"
        self._sym = None
        return None

    def _barrier(self, rank: int, status: torch.Tensor) -> None:
        """Everything enqueued so far has finished on every GPU before anything enqueued next starts."""
        self._epoch += 1
        F_.peer_barrier(self._flags, rank, self._epoch, status, self.barrier_timeout_ms)

    def _scratch(self, N: int, rows: int, device: torch.device):
        key = (N, rows, device)
        if self._bufs is None or self._bufs[0] != key:
            plane = lambda r: torch.empty(1, r, D, N, dtype=torch.float16, device=device)  # noqa: E731
            nccl = self.transport == "nccl"
            channels = self.contraction == "channels"
            gather = nccl and (self.outgoing or self.incoming_scheme == "gather")
            bufs = dict(
                packed=F_.aligned_empty(F_.packed_bytes(), device),
                status=torch.zeros(16, dtype=torch.int32, device=device),
                left=None if channels else plane(rows),
                right=None if channels else plane(rows),
                right_all=plane(N) if gather else None,
                left_all=plane(N) if gather and not self.outgoing else None,
                tri_partial=plane(N) if nccl and not gather else None,
                tri=None if channels else plane(rows),
            )
            self._bufs = (key, bufs)
        return self._bufs[1]

    def device_status(self) -> int:
        """Synchronise and return the device status word of the last forward (0, or a 1xx code: 106 = the barrier
        between GPUs gave up waiting for a peer)."""
        return 0 if self._bufs is None else F_.read_status(self._bufs[1]["status"])

    # ------------------------------------------------------------------ forward
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
        sym = self._symmetric(N, world, dev)  # settles transport and contraction before the scratch is sized
        b = self._scratch(N, rows, dev)
        F_.pack_weights(self._params(), b["packed"], self._biases)
        b["status"].zero_()
        has_bias = bool(self._biases) and any(self._biases.get(k) is not None for k in F_.BIAS_ORDER[:4])
        pro = dict(token_mask=mask, row_begin=begin, eps_in=float(self.ln_pair.eps), has_bias=has_bias)
        epi = dict(eps_in=float(self.ln_pair.eps), eps_out=float(self.ln_out.eps), residual=self.residual)
        y = torch.empty_like(z)
        if sym is None:
            self._tri_nccl(z, b, pro, N, begin, rows)
            F_.epilogue(b["tri"], z, b["packed"], y, b["status"], **epi)
        else:
            bufs = sym[self._calls & 1]  # every rank makes the same number of calls, so all pick the same set
            self._calls += 1
            if self.contraction == "channels":
                F_.prologue_channels(z, b["packed"], bufs["left"], bufs["right"], b["status"], **pro)
                self._barrier(rank, b["status"])  # every rank's rows have landed in every group's operands
                F_.contract_channels(bufs["left"][rank], bufs["right"][rank], bufs["tri"], rank, b["status"], N,
                                     self.outgoing)
                self._barrier(rank, b["status"])  # every group's result has landed at the row owners
                F_.epilogue_groups(bufs["tri"][rank], z, b["packed"], y, b["status"], world, **epi)
            else:
                self._tri_p2p(z, b, bufs["full"], pro, N, begin, rows, world, rank)
                F_.epilogue(b["tri"], z, b["packed"], y, b["status"], **epi)
        if self.check_status:
            F_.check_status(b["status"], "row-sharded trimul")
        return y

    def _tri_p2p(self, z, b, views, pro, N, begin, rows, world, rank) -> None:
        """Stages 1 and 2 of the row scheme with the kernels writing to / reading from the peers' memory."""
        mine = views[rank]
        if self.outgoing:
            peers = [views[r] for r in range(world) if r != rank]
            F_.prologue_push(z, b["packed"], b["left"], mine, peers, b["status"], **pro)
            self._barrier(rank, b["status"])  # every rank's stores have landed in every copy
            F_.contract(b["left"], mine, b["tri"], b["status"], 1, N, begin, rows, True)
        else:
            F_.prologue(z, b["packed"], b["left"], b["right"], b["status"], **pro)
            F_.contract_partial(b["left"], b["right"], mine, b["status"], 1, N, rows)
            self._barrier(rank, b["status"])  # every rank's partial sums are complete
            F_.reduce_partials(b["tri"], views, N, begin, rows)  # rank order: the same sum on every run

    def _tri_nccl(self, z, b, pro, N, begin, rows) -> None:
        """Stages 1 and 2 of the row scheme with NCCL collectives between the kernels (B = 1: the collectives work on
        [rows, 128, N] views, so that the rank-major concatenation is the row dimension)."""
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
