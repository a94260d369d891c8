"""Benchmark of the triangle multiplicative update forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Metric: pair cells per second through a TriMul module forward (B*N^2 cells per forward). One step is one
outgoing forward followed by one incoming forward of the same seeded pair tensor (two module forwards,
2*B*N^2 cells). At one GPU the workload is the N = 768 inference crop; at N > 1 GPUs (torchrun, one rank per
GPU) the same pair tensor is sharded by rows over the ranks (the kernels store into the other GPUs' buffers
through peer memory; NCCL collectives only where peer memory cannot be mapped), so scaling is strong; a batched
workload (`--workload batch8x256`) is split by samples instead. Every multi-GPU line carries `parity`: each rank's
rows compared with the single-GPU forward of the whole tensor. `extra` holds shorter runs of the other benchmark
workloads. Rank 0 prints ONE JSON line.

`--impl reference` times the CPU restatement of the reference module (the reference's own implementation
lives in an un-vendored wheel and cannot be installed offline) on the host cores, on the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from miniworld_b200 import synthetic  # noqa: E402

METRIC = "trimul_fwd_pair_cells_per_s"
UNIT = "pair-cells/s"


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_forward_pair(w, threads: int):
    """One outgoing + one incoming forward of the CPU oracle; returns seconds."""
    from oracle import trimul_oracle as oracle

    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    with torch.no_grad():
        for outgoing in (True, False):
            oracle.trimul_forward(w.z, w.params, w.mask, outgoing=outgoing, k_chunk=32)
    return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # under torchrun only rank 0 measures the CPU arm
    threads = os.cpu_count() or 1
    w = synthetic.make_workload(args.workload, seed=0)
    # every step is the full workload once (outgoing + incoming); steps bounded so the run stays in minutes
    steps = max(1, min(args.steps, 3))
    warm = 1 if args.warmup > 0 else 0
    for _ in range(warm):
        cpu_forward_pair(w, threads)
    times = [cpu_forward_pair(w, threads) for _ in range(steps)]
    t = statistics.median(times)
    value = 2.0 * synthetic.cells(w) / t
    sample = f"{steps} x (outgoing + incoming forward) of the full {args.workload} workload, median"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": w.B, "N": w.N, "d_pair": 128, "d_hidden": 128,
                   "step": "outgoing + incoming forward", "cells_per_step": 2 * synthetic.cells(w)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample,
                         "torch": torch.__version__},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU restatement of the reference module (fp32 PyTorch); the reference's own module is in the "
                "un-vendored miniworld-engine wheel and cannot be installed offline",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
def time_events(fn, steps: int, stream, before_end=None) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the launching stream, sync on both sides."""
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(steps):
        fn()
    if before_end is not None:
        before_end()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end)


def graph_ms(fn, steps: int, stream, dev):
    """Median milliseconds per call of fn replayed from a CUDA graph of one call (device-paced launches), or None
    when the call cannot be captured here."""
    try:
        side = torch.cuda.Stream(dev)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            fn()
        stream.wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        return statistics.median(sorted(time_events(graph.replay, steps, stream) / steps for _ in range(REPEATS)))
    except RuntimeError:
        return None


class HostPipeline:
    """End-to-end step with host buffers: pinned z -> device (copy stream), two module forwards (current
    stream), y -> pinned host (second copy stream). Two device input buffers, so the copies of one step overlap
    the kernels of its neighbours; every step still moves its own input and its own result."""

    def __init__(self, z_host, y_host, forward_pair, dev):
        self.z_host, self.y_host, self.forward_pair, self.dev = z_host, y_host, forward_pair, dev
        self.s_in = torch.cuda.Stream(dev)
        self.s_out = torch.cuda.Stream(dev)
        self.zd = [torch.empty(z_host.shape, dtype=z_host.dtype, device=dev) for _ in range(2)]
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_free = [None, None]
        self.k = 0

    def step(self):
        b = self.k & 1
        cur = torch.cuda.current_stream(self.dev)
        with torch.cuda.stream(self.s_in):
            if self.ev_free[b] is not None:
                self.s_in.wait_event(self.ev_free[b])  # the forwards that read this buffer two steps ago are done
            self.zd[b].copy_(self.z_host, non_blocking=True)
            self.ev_in[b].record(self.s_in)
        cur.wait_event(self.ev_in[b])
        y = self.forward_pair(self.zd[b])
        done = torch.cuda.Event()
        done.record(cur)
        self.ev_free[b] = done
        y.record_stream(self.s_out)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            self.y_host.copy_(y, non_blocking=True)
        self.k += 1

    def drain(self):
        """Make the current stream wait for the last device->host copy (so that the closing event covers it)."""
        ev = torch.cuda.Event()
        ev.record(self.s_out)
        torch.cuda.current_stream(self.dev).wait_event(ev)


REPEATS = 5  # every timed K-step region is measured this many times; the median is reported, min and max beside it


def _stats(ms_list, steps):
    per = sorted(m / steps for m in ms_list)
    return {"median": statistics.median(per), "min": per[0], "max": per[-1], "repeats": len(per)}


class Runner:
    """One workload set up on this rank: the modules, the resident input and the two step functions."""

    def __init__(self, name, world, rank, dev, contraction="auto", on_device=False):
        import miniworld_b200 as mw
        from miniworld_b200 import sharded

        self.name, self.world, self.rank, self.dev = name, world, rank, dev
        if on_device:
            # large extra workloads: drawn on the device from a fixed seed (the same values on every rank); they are
            # only compared between this repository's own single-GPU and multi-GPU forwards, never with the CPU oracle
            B, N, _, _ = synthetic.WORKLOADS[name]
            gen = torch.Generator(device=dev).manual_seed(1234)
            cpu_gen = torch.Generator().manual_seed(1234)
            params = synthetic.make_params(cpu_gen)
            z_full = torch.randn(B, N, N, 128, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
            mask = torch.rand(B, N, generator=gen, device=dev) >= 0.05
            self.w = synthetic.Workload(name=name, z=z_full, mask=mask, params=params, directions=("outgoing", "incoming"), B=B, N=N)
        else:
            self.w = synthetic.make_workload(name, seed=0)
        w = self.w
        self.B, self.N = w.B, w.N
        self.cells_per_step = 2 * synthetic.cells(w)
        self.mods = {}
        if world == 1:
            self.kind = "single"
            self.parallelism = "single GPU"
            sl = (slice(None), slice(None))
        elif w.B > 1:
            # batch data parallelism: samples are independent, so every rank runs its own samples with the ordinary
            # module and nothing crosses the links
            self.kind = "batch"
            b0, cnt = sharded.shard_batch(w.B, world, rank)
            self.parallelism = f"batch of {w.B} samples split over {world} GPUs (replicas, no collective)"
            sl = (slice(b0, b0 + cnt), slice(None))
            self.local_samples = cnt
        else:
            self.kind = "rows"
            begin, rows = sharded.row_range(w.N, world, rank)
            sl = (slice(None), slice(begin, begin + rows))
            self.begin, self.rows = begin, rows
        for direction in ("outgoing", "incoming"):
            if self.kind == "rows":
                m = sharded.RowShardedTriangleMultiplication(128, outgoing=(direction == "outgoing"), contraction=contraction)
            else:
                m = mw.TriangleMultiplication(128, outgoing=(direction == "outgoing"))
            m.load_state_dict(w.params)
            self.mods[direction] = m.to(dev).to(torch.bfloat16).eval()
        z_local = w.z[sl[0], sl[1]].contiguous()
        self.mask = (w.mask if self.kind != "batch" else w.mask[sl[0]]).to(dev)
        self.empty = z_local.shape[0] == 0
        if on_device:
            self.z_host = None
            self.z = z_local
        else:
            self.z_host = z_local.pin_memory()
            self.z = self.z_host.to(dev, non_blocking=True)
        torch.cuda.synchronize()

    def step(self):
        if self.empty:
            return None
        with torch.no_grad():
            self.mods["outgoing"](self.z, self.mask)
            return self.mods["incoming"](self.z, self.mask)

    def forward_pair(self, zd):
        with torch.no_grad():
            self.mods["outgoing"](zd, self.mask)
            return self.mods["incoming"](zd, self.mask)

    def check_status(self):
        for name, m in self.mods.items():  # a device-side wait that gave up (bounded waits) must not pass as a result
            code = m.device_status()
            if code != 0:
                raise SystemExit(f"{self.name}: {name} forward reported device status {code}")

    def describe(self):
        if self.kind == "rows":
            return describe_sharding(self.world, self.mods["outgoing"])
        return self.parallelism

    def launches_per_step(self):
        """This repository's kernels per step: (pack, prologue, contraction, epilogue) x 2 directions; on several GPUs
        the barrier kernels between the stages and, row scheme, the reduce kernel of the incoming direction."""
        if self.kind != "rows":
            return 8
        m = self.mods["outgoing"]
        if m.transport != "p2p":
            return 8
        return 8 + 4 if m.contraction == "channels" else 8 + 2 + 1

    def parity(self):
        """Several GPUs, pair rows sharded: this rank's rows of the sharded forward against the same rows of the
        single-GPU forward of the whole tensor, run here on this GPU. Returns {direction: (bit_identical, max_abs,
        max error in bf16 steps of the single-GPU value)}."""
        import miniworld_b200 as mw

        out = {}
        w = self.w
        zf = w.z.to(self.dev)
        mf = w.mask.to(self.dev)
        for direction in ("outgoing", "incoming"):
            full = mw.TriangleMultiplication(128, outgoing=(direction == "outgoing"))
            full.load_state_dict(w.params)
            full = full.to(self.dev).to(torch.bfloat16).eval()
            with torch.no_grad():
                want = full(zf, mf)[:, self.begin : self.begin + self.rows]
                got = self.mods[direction](self.z, self.mask)
            torch.cuda.synchronize()
            same = bool(torch.equal(got, want))
            diff = (got.float() - want.float()).abs()
            err = float(diff.max())
            # in units of the bf16 spacing of the single-GPU value (values below 1 are measured against the spacing at 1)
            steps = float((diff / torch.exp2(torch.floor(torch.log2(want.float().abs().clamp_min(1.0))) - 7.0)).max())
            del full, want, got, diff
            out[direction] = (same, err, steps)
        return out


def run_b200(args):
    import torch.distributed as dist

    from miniworld_b200 import functional as F_

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback for the product path)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, before_end=None):
        """REPEATS measurements of `steps` calls of fn: barrier + synchronize on both sides, CUDA events on the
        launching stream, the maximum over the ranks for each measurement."""
        out = []
        for _ in range(REPEATS):
            barrier()
            ms = time_events(fn, steps, stream, before_end=before_end)
            barrier()
            out.append(max_over_ranks(ms))
        return out

    def measure(r: Runner, steps: int, warmup: int, with_graph: bool):
        for _ in range(max(warmup, 3)):
            r.step()
        eager = _stats(timed(r.step, steps), steps)
        res = {"eager": eager, "ms_per_step": eager["median"], "launch": "eager launches from the module's forward"}
        if with_graph and not r.empty:
            # the same K steps replayed from a CUDA graph of one step (same kernels, same arguments): the gaps between
            # the launches of a step shrink from host-paced to device-paced
            try:
                side = torch.cuda.Stream(dev)
                side.wait_stream(stream)
                with torch.cuda.stream(side):
                    r.step()
                stream.wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    r.step()
                for _ in range(3):
                    graph.replay()
                g = _stats(timed(graph.replay, steps), steps)
                res["graph"] = g
                if g["median"] < res["ms_per_step"]:
                    res["ms_per_step"], res["launch"] = g["median"], "CUDA graph replay of one step (two module forwards)"
            except RuntimeError as exc:  # capture not possible in this set-up: keep the eager figure
                res["launch"] += f" (graph capture failed: {type(exc).__name__})"
        r.check_status()
        return res

    def parity_line(r: Runner):
        """Multi-GPU output parity against the single-GPU forward, agreed over the ranks; raises on a violation."""
        if r.kind != "rows":
            return None
        par = r.parity()
        line = {}
        for direction, (same, err, steps) in par.items():
            t = torch.tensor([0.0 if same else 1.0, err, steps], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            all_same, worst, worst_steps = t[0].item() == 0.0, float(t[1].item()), float(t[2].item())
            m = r.mods[direction]
            # same kernels and k order -> bit-identical, except the row scheme's incoming direction, whose partial sums
            # are rounded to fp16 once per GPU: two bf16 steps of the output at most
            exact_expected = direction == "outgoing" or m.contraction == "channels" or m.incoming_scheme == "gather"
            line[direction] = "bit-identical" if all_same else {"max_abs": worst, "max_bf16_steps": worst_steps}
            if (exact_expected and not all_same) or worst_steps > 2.0:
                raise SystemExit(f"{r.name}: multi-GPU {direction} output differs from the single-GPU forward "
                                 f"(max abs {worst}, bit-identical expected: {exact_expected})")
        return line

    def link_evidence(r: Runner):
        """Several GPUs, p2p transport: CUDA-event time of stage 1 (the kernel that stores its output tiles into the
        peers' memory over NVLink) with the peers as destinations and with local buffers of the same shapes instead;
        the bytes it sends to peers; and the rate that follows if the difference is the links' time."""
        from miniworld_b200 import functional as F_

        if r.kind != "rows":
            return None
        m = r.mods["outgoing"]
        if m.transport != "p2p" or m._sym is None or m._bufs is None:
            return None
        sets, b = m._sym[1], m._bufs[1]
        z, N, rows = r.z, r.N, r.rows
        pro = dict(token_mask=r.mask, row_begin=r.begin, eps_in=float(m.ln_pair.eps), has_bias=False)
        f16 = dict(dtype=torch.float16, device=dev)
        if m.contraction == "channels":
            cg = 128 // world
            local_l = [torch.empty(1, N, cg, N, **f16) for _ in range(world)]
            local_r = [torch.empty(1, N, cg, N, **f16) for _ in range(world)]
            peer = lambda: F_.prologue_channels(z, b["packed"], sets[0]["left"], sets[0]["right"], b["status"], **pro)  # noqa: E731
            local = lambda: F_.prologue_channels(z, b["packed"], local_l, local_r, b["status"], **pro)  # noqa: E731
            sent = 2 * rows * (128 - cg) * N * 2  # left and right, the channel groups of the other GPUs
            stage = "prologue_channels"
        else:
            views = sets[0]["full"]
            left = torch.empty(1, rows, 128, N, **f16)
            local_copies = [torch.empty(1, N, 128, N, **f16) for _ in range(world)]
            peers = [views[q] for q in range(world) if q != rank]
            peer = lambda: F_.prologue_push(z, b["packed"], left, views[rank], peers, b["status"], **pro)  # noqa: E731
            local = lambda: F_.prologue_push(z, b["packed"], left, local_copies[rank],  # noqa: E731
                                             [local_copies[q] for q in range(world) if q != rank], b["status"], **pro)
            sent = rows * 128 * N * 2 * (world - 1)  # `right` to every other GPU
            stage = "prologue_push"
        out = {"stage": stage, "bytes_to_peers_per_gpu": sent}
        for name, fn in (("peer_ms", peer), ("local_ms", local)):
            for _ in range(3):
                fn()
            barrier()
            ms = sorted(time_events(fn, 10, stream) / 10 for _ in range(3))
            out[name] = max_over_ranks(ms[1])
            barrier()
        out["peer_gbs_lower_bound"] = sent / (out["peer_ms"] * 1e-3) / 1e9
        if out["peer_ms"] > out["local_ms"]:
            out["link_gbs_if_difference_is_link_time"] = sent / ((out["peer_ms"] - out["local_ms"]) * 1e-3) / 1e9
        out["how"] = ("stage 1 alone, ten launches per sample, median of three, max over ranks; the peers' buffers are the "
                      "symmetric-memory views the forward uses, the local run stores the same tiles into this GPU's memory")
        r.check_status()
        return out

    # ---- headline workload
    r = Runner(args.workload, world, rank, dev, contraction=args.contraction)
    B, N = r.B, r.N
    for _ in range(max(args.warmup, 3)):
        r.step()
    barrier()
    sampler = ClockSampler(local_rank)  # samples clocks and throttle reasons over the timed regions that follow
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    res = measure(r, args.steps, args.warmup, with_graph=(world == 1))
    # ---- end-to-end timing: host pinned input -> device -> two forwards -> host pinned output, every step
    y_host = torch.empty_like(r.z_host).pin_memory()
    pipe = HostPipeline(r.z_host, y_host, r.forward_pair, dev)
    for _ in range(2):
        pipe.step()
    e2e = _stats(timed(pipe.step, args.steps, before_end=pipe.drain), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    r.check_status()
    h2d = r.z_host.numel() * 2
    d2h = y_host.numel() * 2
    parity = parity_line(r) if world > 1 else None
    link = link_evidence(r) if world > 1 else None

    # ---- per-stage timing for the roofline (single GPU only: a second K-step loop with events per stage)
    roofline = None
    stages_ms = None
    if world == 1:
        stages_ms, roofline = stage_roofline(r, args.steps, stream, traffic=422.9e6 if args.workload == "crop768" else None)

    # ---- the other benchmark workloads, shorter runs (the headline stays the workload the metric is quoted on)
    extra = {}
    if not args.no_extra:
        names = [n for n in ("n384", "batch8x256", "complex2048") if n != args.workload]
        for name in names:
            B2, N2, _, _ = synthetic.WORKLOADS[name]
            if world > 1 and B2 == 1 and N2 % world != 0:
                continue
            if world > 1 and name == "n384":
                continue  # 48-row slabs at 8 GPUs: below what the sharded kernels take; a single-GPU workload
            steps2 = max(3, min(args.steps, 10 if name != "complex2048" else 5))
            r2 = Runner(name, world, rank, dev, contraction=args.contraction, on_device=(name == "complex2048"))
            m2 = measure(r2, steps2, 3, with_graph=(world == 1))
            entry = {"B": r2.B, "N": r2.N, "ms_per_step": m2["ms_per_step"], "launch": m2["launch"], "eager": m2["eager"],
                     "value": r2.cells_per_step / (m2["ms_per_step"] * 1e-3), "unit": UNIT, "steps": steps2,
                     "parallelism": r2.describe(),
                     "data": "synthetic, drawn on the device" if name == "complex2048" else "synthetic"}
            if "graph" in m2:
                entry["graph"] = m2["graph"]
            if world == 1:
                st2, rf2 = stage_roofline(r2, steps2, stream, traffic=None)
                entry["stages_ms"], entry["roofline"] = st2, rf2
            else:
                p2 = parity_line(r2)
                l2 = link_evidence(r2)
                if l2 is not None:
                    entry["nvlink"] = l2
                if p2 is not None:
                    entry["parity"] = p2
            extra[name] = entry
            del r2
            torch.cuda.empty_cache()

    # ---- the two neighbouring operators of a Pairformer block, single GPU, on the headline shape: the bidirectional
    # triangle update MiniWorld's trunk builds and the pair Transition that follows it
    if world == 1 and not args.no_extra:
        extra.update(block_operators(r, max(3, min(args.steps, 10)), stream, dev))

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        t = cpu_forward_pair(r.w, threads)
        cpu_baseline = {"value": r.cells_per_step / t, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"1 x (outgoing + incoming forward) of the full {args.workload} workload, fp32 PyTorch oracle",
                        "seconds": t, "torch": torch.__version__}

    if rank == 0:
        t_step = res["ms_per_step"]
        t_e2e = e2e["median"]
        line = {
            "metric": METRIC, "value": r.cells_per_step / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t_step,
            "ms_per_step_eager": res["eager"]["median"], "launch": res["launch"],
            "timing": {"repeats": REPEATS, "eager": res["eager"], "graph": res.get("graph"),
                       "how": "each figure is the median of `repeats` measurements of K steps (CUDA events, barrier and "
                              "synchronize on both sides, maximum over the ranks per measurement)"},
            "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "N": N, "d_pair": 128, "d_hidden": 128,
                       "step": "outgoing forward + incoming forward (2 module forwards)",
                       "cells_per_step": r.cells_per_step,
                       "parallelism": r.describe(),
                       "l2": "inputs and intermediates (604 MB at N=768) exceed the 126 MB L2; no flush"},
            "e2e": {"value": r.cells_per_step / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "min": e2e["min"], "max": e2e["max"], "repeats": REPEATS,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "pinned host z -> device, two module forwards, y -> pinned host, every step; two device "
                           "input buffers so copies overlap the neighbouring steps' kernels; median of the repeats"},
            "gpu_launches": r.launches_per_step() * args.steps,
            "clocks": clocks,
        }
        if parity is not None:
            line["parity"] = parity
        if link is not None:
            line["nvlink"] = link
        if stages_ms is not None:
            line["stages_ms"] = stages_ms
        if roofline is not None:
            line["roofline"] = roofline
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        if extra:
            line["extra"] = extra
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def block_operators(r: "Runner", steps: int, stream, dev) -> dict:
    """CUDA-event times of BidirectionalTriangleMultiplication and Transition forwards on the headline input."""
    import miniworld_b200 as mw

    out = {}
    peaks = measured_peaks()
    gen = torch.Generator().manual_seed(77)

    def rn(*shape):
        return torch.randn(*shape, generator=gen)

    bid = mw.BidirectionalTriangleMultiplication(128)
    bid.load_state_dict({
        "ln_pair.weight": 1.0 + 0.1 * rn(128), "ln_pair.bias": 0.02 * rn(128),
        "to_left.weight": rn(256, 128) * 128**-0.5, "to_left_gate.weight": rn(256, 128) * 128**-0.5,
        "to_right.weight": rn(256, 128) * 128**-0.5, "to_right_gate.weight": rn(256, 128) * 128**-0.5,
        "ln_out.weight": 1.0 + 0.1 * rn(256), "ln_out.bias": 0.02 * rn(256),
        "to_gate.weight": rn(128, 128) * 128**-0.5, "to_out.weight": rn(128, 256) * 256**-0.5})
    bid = bid.to(dev).to(torch.bfloat16).eval()
    tr = mw.Transition(128)
    tr.load_state_dict({"ln_in.weight": 1.0 + 0.1 * rn(128), "ln_in.bias": 0.02 * rn(128),
                        "expand_a.weight": rn(512, 128) * 128**-0.5, "expand_b.weight": rn(512, 128) * 128**-0.5,
                        "squeeze.weight": rn(128, 512) * 512**-0.5})
    tr = tr.to(dev).to(torch.bfloat16).eval()
    cells = synthetic.cells(r.w)
    with torch.no_grad():
        for name, fn in (("bidirectional", lambda: bid(r.z, r.mask)), ("transition", lambda: tr(r.z))):
            for _ in range(3):
                fn()
            ms = sorted(time_events(fn, steps, stream) / steps for _ in range(REPEATS))
            entry = {"workload": r.name, "ms_per_forward": statistics.median(ms), "min": ms[0], "max": ms[-1],
                     "value": cells / (statistics.median(ms) * 1e-3), "unit": UNIT}
            if name == "transition":
                fl = cells * 393216.0  # 2 * (2 * 128 * 512 + 512 * 128) FLOP per position
                entry["roofline"] = {"kernel": "transition_kernel", "bound": "tensor", "flops_per_launch": fl,
                                     "achieved": fl / (entry["ms_per_forward"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                                     "peak": peaks["bf16_tflops"],
                                     "frac": fl / (entry["ms_per_forward"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}
            else:
                entry["note"] = ("one operator = both directions: compare with ms_per_step of the headline, which is one "
                                 "outgoing and one incoming module forward")
            out[name] = entry
    if bid.device_status() != 0 or tr.device_status() != 0:
        raise SystemExit("bidirectional / transition forward reported a device status")
    out["training"] = training_step(r, steps, stream, dev, bid)
    # the Transition's training step on the same input
    params = {k: v.detach() for k, v in tr.state_dict().items()}
    dy = (torch.randn(r.z.shape, generator=torch.Generator(device=dev).manual_seed(79), device=dev) * 0.01).to(torch.bfloat16)
    from miniworld_b200 import functional as F_

    def tr_bwd():
        F_.transition_backward(dy, r.z, params)

    for _ in range(3):
        tr_bwd()
    ms = sorted(time_events(tr_bwd, steps, stream) / steps for _ in range(REPEATS))
    out["training"]["transition"] = {"ms_forward": out["transition"]["ms_per_forward"], "ms_backward": statistics.median(ms),
                                     "backward_over_forward": statistics.median(ms) / out["transition"]["ms_per_forward"]}
    g = graph_ms(tr_bwd, steps, stream, dev)
    if g is not None:
        out["training"]["transition"]["ms_backward_graph"] = g
    return out


def training_step(r: "Runner", steps: int, stream, dev, bid) -> dict:
    """CUDA-event times of one training step on the headline input, for the two unidirectional modules and for the
    bidirectional one: the forward with its stage tensors kept, and ``b200_trimul_backward`` (gradients of the input and
    all ten parameters)."""
    from miniworld_b200 import functional as F_

    B, N, z, mask = r.B, r.N, r.z, r.mask
    gen = torch.Generator(device=dev).manual_seed(78)
    dy = (torch.randn(z.shape, generator=gen, device=dev) * 0.01).to(torch.bfloat16)
    res = {"workload": r.name}
    for direction in tuple(r.w.directions) + ("bidirectional",):
        outgoing = None if direction == "bidirectional" else direction == "outgoing"
        mod = bid if outgoing is None else r.mods[direction]
        params = {k: v.detach() for k, v in mod._params().items()}
        ws = F_.aligned_empty(F_.workspace_bytes(B, N, outgoing), dev)
        bws = F_.aligned_empty(F_.backward_workspace_bytes(B, N, outgoing), dev)
        y = torch.empty_like(z)

        def fwd():
            F_.trimul_forward(z, params, mask, outgoing=outgoing, workspace=ws, out=y)

        def bwd():
            F_.trimul_backward(dy, z, params, ws, mask, outgoing=outgoing, workspace=bws)

        entry = {}
        for name, fn in (("forward", fwd), ("backward", bwd)):
            for _ in range(3):
                fn()
            ms = sorted(time_events(fn, steps, stream) / steps for _ in range(REPEATS))
            entry[f"ms_{name}"] = statistics.median(ms)
        g = graph_ms(bwd, steps, stream, dev)  # the same call with device-paced launches
        if g is not None:
            entry["ms_backward_graph"] = g
        F_.check_status(bws[:64].view(torch.int32), "b200_trimul_backward")
        entry["backward_over_forward"] = entry["ms_backward"] / entry["ms_forward"]
        res[direction] = entry
    return res


def stage_roofline(r: Runner, steps: int, stream, traffic):
    """Single GPU: K steps with CUDA events around each stage (called through the staged C-ABI entry points with
    pointers prepared once), and the roofline figures that follow from the stage times."""
    from miniworld_b200 import functional as F_

    B, N, dev, z, mask = r.B, r.N, r.dev, r.z, r.mask
    layout = F_.workspace_layout(B, N)
    ws = F_.aligned_empty(F_.workspace_bytes(B, N), dev)
    plane = B * N * 128 * N
    status = ws[:64].view(torch.int32)
    packed = ws[layout[1] : layout[1] + F_.packed_bytes()]
    left = ws[layout[2] : layout[2] + plane * 2].view(torch.float16).view(B, N, 128, N)
    right = ws[layout[3] : layout[3] + plane * 2].view(torch.float16).view(B, N, 128, N)
    tri = ws[layout[4] : layout[4] + plane * 2].view(torch.float16).view(B, N, 128, N)
    y = torch.empty_like(z)
    params = r.mods["outgoing"]._params()
    names = ("pack", "prologue", "contract_outgoing", "contract_incoming", "epilogue")
    acc = {n: 0.0 for n in names}
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    status.zero_()
    for it in range(3 + steps):
        evs[0].record(stream)
        F_.pack_weights(params, packed)
        evs[1].record(stream)
        F_.prologue(z, packed, left, right, status, token_mask=mask)
        evs[2].record(stream)
        F_.contract(left, right, tri, status, B, N, 0, N, True)
        evs[3].record(stream)
        F_.contract(left, right, tri, status, B, N, 0, N, False)
        evs[4].record(stream)
        F_.epilogue(tri, z, packed, y, status)
        evs[5].record(stream)
        torch.cuda.synchronize()
        if it >= 3:
            for i, n in enumerate(names):
                acc[n] += evs[i].elapsed_time(evs[i + 1])
    F_.check_status(status, "bench stages")
    stages_ms = {n: v / steps for n, v in acc.items()}
    stages_ms["note"] = ("each stage is launched by its own Python call between two events, so a stage shorter than the "
                         "call's host cost (about 30 us: pack) shows the host cost, not the kernel")
    peaks = measured_peaks()
    fl = synthetic.flops(B, N)
    t_contract = 0.5 * (stages_ms["contract_outgoing"] + stages_ms["contract_incoming"])
    achieved = fl["contraction"] / (t_contract * 1e-3) / 1e12
    P = synthetic.pass_bytes(B, N)
    roofline = {
        "kernel": "contract_pair_kernel" if N >= 256 else "contract_kernel", "bound": "tensor", "achieved": achieved,
        "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
        "peak_source": peaks["source"] + " (burst)",
        "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
        "flops_per_launch": fl["contraction"],
        # dram__bytes_read.sum + dram__bytes_write.sum of one contraction launch, from the ncu capture of the crop768
        # workload summarised under profiles/; not captured for the other workloads
        "traffic": traffic,
        "timed": "separate loop of K steps, CUDA events around each stage on the launching stream",
        "other_kernels": {
            "prologue_kernel": {"bound": "hbm", "algorithmic_bytes": 3 * P,
                                "achieved_gbs": 3 * P / (stages_ms["prologue"] * 1e-3) / 1e9,
                                "frac": 3 * P / (stages_ms["prologue"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "epilogue_kernel": {"bound": "hbm", "algorithmic_bytes": 3 * P,
                                "achieved_gbs": 3 * P / (stages_ms["epilogue"] * 1e-3) / 1e9,
                                "frac": 3 * P / (stages_ms["epilogue"] * 1e-3) / 1e9 / peaks["hbm_gbs"]},
        },
    }
    return stages_ms, roofline


def describe_sharding(world: int, module) -> str:
    """One line for `config.parallelism`: what the sharded module settled on."""
    head = f"pair rows sharded over {world} GPUs, transport {module.transport}, contraction by {module.contraction}: "
    if module.contraction == "channels":
        return head + ("prologue and contraction store each tile into the GPU that needs it (channel groups out, "
                       "row blocks back)")
    if module.transport == "p2p":
        return head + ("outgoing = prologue writes `right` into every GPU's copy, incoming = partial sums over the "
                       "local rows k + reduce kernel reading the peers")
    return head + "outgoing = all-gather of `right`, incoming = partial sums + reduce-scatter"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--workload", default="crop768", choices=sorted(synthetic.WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the shorter runs of the other benchmark workloads")
    ap.add_argument("--operators-only", action="store_true",
                    help="run only the bidirectional and transition forwards on the workload (for profiler captures)")
    ap.add_argument("--contraction", choices=["auto", "rows", "channels"], default="auto",
                    help="several GPUs: how the contraction is split (auto: channels from 4 GPUs on)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.operators_only:
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        r = Runner(args.workload, 1, 0, dev)
        print(json.dumps({"operators": block_operators(r, args.steps, torch.cuda.current_stream(dev), dev)}), flush=True)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
