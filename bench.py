"""Benchmark of the triangle multiplicative update forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Metric: pair cells per second through a TriMul module forward (B*N^2 cells per forward). One step is one
outgoing forward followed by one incoming forward of the same seeded pair tensor (two module forwards,
2*B*N^2 cells). At one GPU the workload is the N = 768 inference crop; at N > 1 GPUs (torchrun, one rank per
GPU) the same pair tensor is row-sharded over the ranks with NCCL all-gathers of the contracted operands, so
scaling is strong. Rank 0 prints ONE JSON line.

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
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None,
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


def run_b200(args):
    import torch.distributed as dist

    import miniworld_b200 as mw
    from miniworld_b200 import functional as F_
    from miniworld_b200 import sharded

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

    w = synthetic.make_workload(args.workload, seed=0)
    B, N = w.B, w.N
    cells_per_step = 2 * synthetic.cells(w)
    stream = torch.cuda.current_stream(dev)

    if world == 1:
        mods = {}
        for direction in ("outgoing", "incoming"):
            m = mw.TriangleMultiplication(128, outgoing=(direction == "outgoing"))
            m.load_state_dict(w.params)
            mods[direction] = m.to(dev).to(torch.bfloat16).eval()
        z_host = w.z.contiguous().pin_memory()
        mask = w.mask.to(dev)
        z = z_host.to(dev, non_blocking=True)
        y_host = torch.empty_like(z_host).pin_memory()
        torch.cuda.synchronize()

        def step():
            with torch.no_grad():
                mods["outgoing"](z, mask)
                return mods["incoming"](z, mask)

        def forward_pair(zd):
            with torch.no_grad():
                mods["outgoing"](zd, mask)
                return mods["incoming"](zd, mask)

        pipe = HostPipeline(z_host, y_host, forward_pair, dev)
        step_e2e = pipe.step

        h2d = z_host.numel() * 2
        d2h = y_host.numel() * 2
    else:
        begin, rows = sharded.row_range(N, world, rank)
        mods = {}
        for direction in ("outgoing", "incoming"):
            m = sharded.RowShardedTriangleMultiplication(128, outgoing=(direction == "outgoing"),
                                                         contraction=args.contraction)
            m.load_state_dict(w.params)
            mods[direction] = m.to(dev).to(torch.bfloat16).eval()
        z_host = w.z[:, begin : begin + rows].contiguous().pin_memory()
        mask = w.mask.to(dev)
        z = z_host.to(dev, non_blocking=True)
        y_host = torch.empty_like(z_host).pin_memory()
        torch.cuda.synchronize()

        def step():
            with torch.no_grad():
                mods["outgoing"](z, mask)
                return mods["incoming"](z, mask)

        def forward_pair(zd):
            with torch.no_grad():
                mods["outgoing"](zd, mask)
                return mods["incoming"](zd, mask)

        pipe = HostPipeline(z_host, y_host, forward_pair, dev)
        step_e2e = pipe.step

        h2d = z_host.numel() * 2
        d2h = y_host.numel() * 2

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

    # ---- kernel-resident timing (inputs already in HBM)
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    ms = time_events(step, args.steps, stream)
    barrier()
    ms = max_over_ranks(ms)
    ms_eager = ms
    launch = "eager launches from the module's forward"
    if world == 1:
        # the same K steps replayed from a CUDA graph of one step (same kernels, same arguments): the gaps between the
        # eight launches of a step shrink from host-paced to device-paced
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                step()
            stream.wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            for _ in range(3):
                graph.replay()
            ms_graph = time_events(graph.replay, args.steps, stream)
            if ms_graph < ms:
                ms, launch = ms_graph, "CUDA graph replay of one step (two module forwards)"
        except RuntimeError as exc:  # capture not possible in this set-up: keep the eager figure
            launch += f" (graph capture failed: {type(exc).__name__})"
    # ---- end-to-end timing: host pinned input -> device -> two forwards -> host pinned output, every step
    for _ in range(2):
        step_e2e()
    barrier()
    ms_e2e = max_over_ranks(time_events(step_e2e, args.steps, stream, before_end=pipe.drain))
    clocks = sampler.stop() if rank == 0 else None
    for name, m in mods.items():  # a device-side wait that gave up (bounded waits) must not pass as a result
        code = m.device_status()
        if code != 0:
            raise SystemExit(f"{name} forward reported device status {code}")

    # ---- per-stage timing for the roofline (single GPU only: a second K-step loop with events per stage)
    roofline = None
    stages_ms = None
    if world == 1:
        layout = F_.workspace_layout(B, N)
        ws = F_.aligned_empty(F_.workspace_bytes(B, N), dev)
        plane = B * N * 128 * N
        status = ws[:64].view(torch.int32)
        packed = ws[layout[1] : layout[1] + F_.packed_bytes()]
        left = ws[layout[2] : layout[2] + plane * 2].view(torch.float16).view(B, N, 128, N)
        right = ws[layout[3] : layout[3] + plane * 2].view(torch.float16).view(B, N, 128, N)
        tri = ws[layout[4] : layout[4] + plane * 2].view(torch.float16).view(B, N, 128, N)
        y = torch.empty_like(z)
        params = mods["outgoing"]._params()
        names = ("pack", "prologue", "contract_outgoing", "contract_incoming", "epilogue")
        acc = {n: 0.0 for n in names}
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
        for it in range(3 + args.steps):
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
        stages_ms = {n: v / args.steps for n, v in acc.items()}
        peaks = measured_peaks()
        fl = synthetic.flops(B, N)
        t_contract = 0.5 * (stages_ms["contract_outgoing"] + stages_ms["contract_incoming"])
        achieved = fl["contraction"] / (t_contract * 1e-3) / 1e12
        P = synthetic.pass_bytes(B, N)
        roofline = {
            "kernel": "contract_pair_kernel" if N >= 256 else "contract_kernel", "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
            "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"] + " (burst)",
            "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"] if peaks["bf16_tflops_sustained"] else None,
            "flops_per_launch": fl["contraction"],
            # dram__bytes_read.sum + dram__bytes_write.sum of one contraction launch, from the ncu capture of this
            # workload summarised under profiles/; not captured for the other workloads
            "traffic": 422.9e6 if args.workload == "crop768" else None,
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

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        t = cpu_forward_pair(w, threads)
        cpu_baseline = {"value": cells_per_step / t, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"1 x (outgoing + incoming forward) of the full {args.workload} workload, fp32 PyTorch oracle",
                        "seconds": t, "torch": torch.__version__}

    if rank == 0:
        t_step = ms / args.steps
        t_e2e = ms_e2e / args.steps
        line = {
            "metric": METRIC, "value": cells_per_step / (t_step * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t_step,
            "ms_per_step_eager": ms_eager / args.steps, "launch": launch, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "B": B, "N": N, "d_pair": 128, "d_hidden": 128,
                       "step": "outgoing forward + incoming forward (2 module forwards)",
                       "cells_per_step": cells_per_step,
                       "parallelism": "single GPU" if world == 1 else describe_sharding(world, mods["outgoing"]),
                       "l2": "inputs and intermediates (604 MB at N=768) exceed the 126 MB L2; no flush"},
            "e2e": {"value": cells_per_step / (t_e2e * 1e-3), "unit": UNIT, "ms_per_step": t_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "pinned host z -> device, two module forwards, y -> pinned host, every step; two device "
                           "input buffers so copies overlap the neighbouring steps' kernels"},
            # this repository's kernels per step: (pack, prologue, contraction, epilogue) x 2 directions, plus the
            # peer-reading reduce kernel of the incoming direction on the p2p transport
            "gpu_launches": (9 if world > 1 and mods["outgoing"].transport == "p2p"
                             and mods["outgoing"].contraction == "rows" else 8) * args.steps,
            "clocks": clocks,
        }
        if stages_ms is not None:
            line["stages_ms"] = stages_ms
        if roofline is not None:
            line["roofline"] = roofline
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


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
    ap.add_argument("--contraction", choices=["auto", "rows", "channels"], default="auto",
                    help="several GPUs: how the contraction is split (auto: channels from 4 GPUs on)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
