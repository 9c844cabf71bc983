"""Benchmark of the muse_bf16_proj hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--case layer:m] [--no-table]

Metric: microseconds per call (CUDA-graph replay, cold L2) and achieved HBM GB/s. One STEP is one
replay of a CUDA graph holding the qkv_gate projection [12288, 4096] at m = 1, 2, 4, 8, 16, 32 -- six
calls, each on its own copy of the weight, so every call streams its 100.7 MB from HBM (600 MB of
distinct weights per step against a 126 MB L2; no flush kernel sits inside the timed region). K steps
are timed back to back between two CUDA events on the replaying stream, bracketed by a barrier and
a device synchronize; `value` = that time / (6 K). Prints ONE JSON line.

Beside the headline the line carries: `cases` (every configuration of the benchmark, each timed
the same way on rotating weight copies), `roofline` for the dominant kernel, `e2e` (the same calls
through kernel_fn() from pinned host buffers, copies inside the timed region), `cpu_baseline` (the
reference's torch CPU path on this host), and the SM clocks sampled while timing.

With --gpus N > 1 (launched by torchrun, one rank per GPU) the weight is sharded by output rows,
each call is the local kernel followed by an NCCL all-gather inside the same graph, and the time
is the maximum over ranks.

--impl reference times the reference's own CPU implementation of the path (its torch x @ W.T /
hi-lo router, restated in oracle/ because the reference checkout does not travel) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = {"qkv_gate": (12288, 4096), "o": (4096, 4096), "pooler": (1024, 4096), "unpooler": (4096, 1024),
          "router": (256, 4096)}
FP32_LAYERS = {"router"}
WORKLOAD_LAYER = "qkv_gate"
WORKLOAD_TOKENS = (1, 2, 4, 8, 16, 32)
# the table: the workload's calls, then the other configurations the benchmark names (qkv_gate and o at
# m = 128, 256 belong to its column-parallel sweep)
CASES = {"qkv_gate": WORKLOAD_TOKENS + (128, 256), "o": (1, 8, 32, 128, 256), "router": (1, 8, 32, 128, 256),
         "pooler": (1, 32, 64, 128, 256), "unpooler": (1, 32, 64, 128, 256)}
WEIGHT_STD = 0.02
SEED = 5151
ROTATE_BYTES = 640 << 20      # distinct weight bytes a per-case graph cycles through (5x the L2)
MAX_COPIES = 160
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
METRIC = "us/call (CUDA-graph, cold L2)"
# one description of the workload for both arms, so that their `config.workload` strings are equal
WORKLOAD_TEXT = (f"{WORKLOAD_LAYER} projection: x [m,4096] bf16 ~N(0,1), W [12288,4096] bf16 ~N(0,0.02), "
                 f"m in {list(WORKLOAD_TOKENS)}; value = mean time of the six calls")
L2_TEXT = "cold: every call reads a weight copy that is not in cache (604 MB of distinct weights per pass vs 126 MB L2)"
# Column-parallel calls compared before any timing (layer, m): each exchange protocol and kernel family.
PARITY_CASES = (("qkv_gate", 1), ("qkv_gate", 8), ("qkv_gate", 16), ("qkv_gate", 32), ("qkv_gate", 64), ("qkv_gate", 256),
                ("o", 1), ("o", 8), ("o", 32), ("o", 128), ("router", 1), ("router", 8), ("router", 128))
# DRAM bytes (read + write) per launch from one ncu capture per kernel on ONE GPU (profiles/*.md); a static
# figure the line carries for comparison with `bytes_per_launch`, not something measured in this run.
NCU_TRAFFIC = {
    "fewtok_xreg<32,4,false> qkv_gate m=8": 104474368,
    "fewtok_xreg<16,8,true> qkv_gate m=16": 104567808,
    "gemm_tc qkv_gate m=32": 104101632,
    "gemm_tc qkv_gate m=128": 105473280,
    "gemm_tc qkv_gate m=256": 109367808,
    "gemv1_rows o m=1": 33578496,
    "skinny_tc router m=128": 5302016,
    "fewtok_xreg_f32<16,8> router m=32": 4471040,
}


def algorithmic_bytes(layer: str, m: int, n: int, k: int) -> int:
    wb = 4 if layer in FP32_LAYERS else 2
    return n * k * wb + m * k * 2 + m * n * wb


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:  # noqa: BLE001
            pass
    return FALLBACK_HBM_GBS, "fallback"


def make_weight(layer: str, device, seed: int, rows: slice | None = None) -> torch.Tensor:
    n, k = LAYERS[layer]
    g = torch.Generator(device=device).manual_seed(seed)
    w = torch.randn((n, k), generator=g, device=device) * WEIGHT_STD
    w = w.to(torch.float32 if layer in FP32_LAYERS else torch.bfloat16)
    return w if rows is None else w[rows].clone()


def make_x(layer: str, m: int, device, seed: int) -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn((m, LAYERS[layer][1]), generator=g, device=device).to(torch.bfloat16)


class ClockSampler:
    """Polls NVML (read-only) for SM clock and throttle reasons while the timed regions run."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._busy = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._thread = threading.Thread(target=self._run, args=(period_s,), daemon=True)
            self._thread.start()
        except Exception:  # noqa: BLE001
            self._nv = None

    def _run(self, period_s: float):
        nv = self._nv
        while not self._stop.is_set():
            if self._busy.is_set():
                try:
                    self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                    self.reasons |= {name for bit, name in self.REASONS.items() if mask & bit}
                except Exception:  # noqa: BLE001
                    pass
            time.sleep(period_s)

    def __enter__(self):
        self._busy.set()
        return self

    def __exit__(self, *exc):
        self._busy.clear()

    def summary(self) -> dict:
        self._stop.set()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:  # noqa: BLE001
            return local
    return local


# --------------------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# --------------------------------------------------------------------------------------------------

def cpu_path_us(tokens, layer: str, reps: int, warmup: int) -> tuple[float, dict]:
    """Mean over `tokens` of the median wall time of the reference's CPU kernel_fn, in microseconds."""
    from oracle import muse_proj_oracle as oracle  # the timed CPU baseline; never on the product path

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = oracle.target_weights(SEED, device="cpu", only={layer})
    state = oracle.cpu_prepare(w)
    per = {}
    for m in tokens:
        data = oracle.target_input(m, layer, 1000 + m, device="cpu")
        for _ in range(warmup):
            oracle.cpu_kernel_fn(data, state)
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            oracle.cpu_kernel_fn(data, state)
            ts.append((time.perf_counter() - t0) * 1e6)
        per[m] = statistics.median(ts)
    return sum(per.values()) / len(per), {"cores": cores, "per_m_us": {str(k): round(v, 1) for k, v in per.items()}}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    us, info = cpu_path_us(WORKLOAD_TOKENS, WORKLOAD_LAYER, reps=max(1, args.steps), warmup=max(1, args.warmup))
    sample = (f"{WORKLOAD_LAYER} [12288,4096] bf16, m in {list(WORKLOAD_TOKENS)}: every call of the workload, "
              f"{max(1, args.steps)} timed repetitions each, torch CPU x @ W.T (oracle port of bf16_proj/baseline.py)")
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": "us/call", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": us * len(WORKLOAD_TOKENS) / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT, "l2": L2_TEXT, "arm": "reference CPU path on the host cores (no L2 control)"},
        "cpu_baseline": {"value": us, "unit": "us/call", "cores": info["cores"], "kind": "port", "sample": sample,
                         "per_m_us": info["per_m_us"]},
        "e2e": {"value": us, "unit": "us/call", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------

class Harness:
    def __init__(self, device, world: int, rank: int):
        from llm_inference_engine_b200 import muse_bf16_proj as proj
        from llm_inference_engine_b200.graph_timer import ColdReplayTimer

        self.proj = proj
        self.device = device
        self.world, self.rank = world, rank
        self.timer = ColdReplayTimer(device, flush_bytes=1 << 20)
        self.cp = None
        if world > 1:
            import torch.distributed as dist

            from llm_inference_engine_b200 import tp

            self.dist = dist
            self.cp = tp.ColumnParallelProjection(proj.prepare, proj.kernel_fn)
            self.cp.rows = {k: v[0] for k, v in LAYERS.items()}
            self.fused = None
            self.fused_error = None
            if not os.environ.get("MUSE_BENCH_NO_FUSED"):
                try:   # the all-gather inside the kernel (peer stores); NCCL stays as the comparison
                    self.fused = tp.FusedColumnParallel(proj.prepare, proj.kernel_fn)
                    self.fused.rows = dict(self.cp.rows)
                    for name, (n, _k) in LAYERS.items():
                        self.fused._ensure_layer(name, n, torch.float32 if name in FP32_LAYERS else torch.bfloat16, device)
                except Exception as e:  # noqa: BLE001
                    self.fused, self.fused_error = None, f"{type(e).__name__}: {e}"

    def shard(self, layer: str) -> slice | None:
        if self.world == 1:
            return None
        per = LAYERS[layer][0] // self.world
        return slice(self.rank * per, (self.rank + 1) * per)

    def states(self, layer: str, copies: int):
        """`copies` independent prepared weights of one layer (each its own tensor in HBM)."""
        out = []
        for i in range(copies):
            w = make_weight(layer, self.device, SEED + 17 * i, self.shard(layer))
            out.append(self.proj.prepare({layer: w}, warmup=(i == 0)))
        return out

    def call(self, layer: str, x: torch.Tensor, state, mode: str = "best") -> torch.Tensor:
        """mode: "best" (fused exchange when available, else NCCL), "nccl", or "local" (this rank's slice only)."""
        n, k = LAYERS[layer]
        data = {"x": x, "config": {"m": x.shape[0], "n": n, "k": k, "layer": layer}}
        if self.cp is None:
            return self.proj.kernel_fn(data, state)
        if mode == "best" and self.fused is not None:
            return self.fused.kernel_fn(data, state)
        part = self.cp.kernel_fn_local(data, state)
        return part if mode == "local" else self.cp.gather(part)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.device)

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = torch.tensor([v], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def time_graph(self, fn, steps: int, warmup: int) -> float:
        """Milliseconds per replay: `steps` replays between one pair of events, after `warmup` replays."""
        graph = self.timer.capture(fn)
        stream = self.timer.stream
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                graph.replay()
            self.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(steps):
                graph.replay()
            b.record(stream)
            self.barrier()
        return self.max_over_ranks(a.elapsed_time(b) / steps)


def copies_for(layer: str, world: int) -> int:
    n, k = LAYERS[layer]
    by = n * k * (4 if layer in FP32_LAYERS else 2) // world
    return max(6, min(MAX_COPIES, -(-ROTATE_BYTES // by)))


def kernel_family(h: Harness, state, layer: str, m: int, n_local: int, k: int) -> str:
    """Which of the library's kernels the planner gives this call (the name the ncu summaries use)."""
    from llm_inference_engine_b200.plan import FewTokPlan, GemmPlan, GemvPlan

    plan = h.proj.plan_for(state, layer, m, n_local, k, fused=h.world > 1 and h.fused is not None)
    if isinstance(plan, GemvPlan):
        return "gemv1_rows" if plan.persistent else "gemv1"
    if isinstance(plan, FewTokPlan) and layer in FP32_LAYERS:
        return f"fewtok_xreg_f32<{plan.warps},{plan.unroll}>"
    if isinstance(plan, FewTokPlan):
        name = "fewtok_xreg" if plan.warps * plan.unroll * 32 >= k else "fewtok_mma"
        return f"{name}<{plan.warps},{plan.unroll},{'true' if m > 8 * plan.tok_split else 'false'}>"
    return "gemm_tc" if isinstance(plan, GemmPlan) else "skinny_tc"


def case_table(h: Harness, layers, steps: int, warmup: int, peak: float, only=None) -> list[dict]:
    rows = []
    for layer in layers:
        copies = copies_for(layer, h.world)
        states = h.states(layer, copies)
        n, k = LAYERS[layer]
        for m in CASES[layer]:
            if only and (layer, m) != only:
                continue
            x = make_x(layer, m, h.device, 1000 + m)
            row = {"layer": layer, "m": m, "n": n, "k": k, "copies": copies}
            for key, mode in (("us", "best"), ("nccl_us", "nccl"), ("kernel_us", "local")):
                if key != "us" and h.world == 1:
                    continue
                if key == "nccl_us" and h.fused is None:
                    continue
                keep = []

                def fn(mode=mode, keep=keep):
                    keep.clear()
                    for s in states:
                        keep.append(h.call(layer, x, s, mode))

                row[key] = 1e3 * h.time_graph(fn, steps, warmup) / copies
            row["kernel"] = kernel_family(h, states[0], layer, m, n // h.world, k)
            by = algorithmic_bytes(layer, m, n // h.world, k)
            kus = row.get("kernel_us", row["us"])
            row.update({"bytes": by, "gbs": by / kus / 1e3, "frac_of_measured": by / kus / 1e3 / peak,
                        "frac_of_8tbs": by / kus / 1e3 / NOMINAL_HBM_GBS})
            rows.append(row)
        for s in states:
            h.proj.check_status(s)
        del states
        torch.cuda.empty_cache()
    return rows


def gather_check(h: Harness) -> dict:
    """Column-parallel only, before any timing: every PARITY_CASES call through the fused exchange and through
    kernel + NCCL all-gather, both against an FP32 product of the FULL weight on this rank (BF16: rtol 1e-2 /
    atol 1e-2; router: relative L2 <= 1e-5), and against each other bit for bit where both run the same
    deterministic plan. Every rank checks its own gathered copy; the verdicts are combined; a mismatch
    ends the run."""
    dist = h.dist
    bad: list[str] = []
    n_cases = 0
    worst = 0.0
    for layer in dict.fromkeys(c[0] for c in PARITY_CASES):
        n, k = LAYERS[layer]
        full = make_weight(layer, h.device, SEED).float()
        state = h.states(layer, 1)[0]
        for m in (c[1] for c in PARITY_CASES if c[0] == layer):
            x = make_x(layer, m, h.device, 4000 + m)
            want = x.float() @ full.T
            outs = {}
            if h.fused is not None:
                outs["fused"] = h.call(layer, x, state, "best").clone()
            outs["nccl"] = h.call(layer, x, state, "nccl")
            for tag, got in outs.items():
                n_cases += 1
                if layer in FP32_LAYERS:
                    err = float((got.double() - want.double()).norm() / want.double().norm())
                    ok = err <= 1e-5
                else:
                    err = float((got.float() - want).abs().max())
                    ok = bool(torch.allclose(got.float(), want, rtol=1e-2, atol=1e-2))
                worst = max(worst, err) if layer not in FP32_LAYERS else worst
                if not ok:
                    bad.append(f"{tag} {layer} m={m}: error {err:.3e}")
            if len(outs) == 2:
                local = (n // h.world, k)
                plan = h.proj.plan_for(state, layer, m, *local)
                if plan == h.proj.plan_for(state, layer, m, *local, fused=True) and getattr(plan, "groups", 1) == 1:
                    n_cases += 1
                    if not torch.equal(outs["fused"], outs["nccl"]):
                        bad.append(f"fused != nccl bitwise: {layer} m={m}")
        h.proj.check_status(state)
        del state, full
        torch.cuda.empty_cache()
    flag = torch.tensor([len(bad)], device=h.device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.SUM)
    for line in bad:
        print(f"[bench] rank {h.rank}: parity: {line}", file=sys.stderr, flush=True)
    return {"cases": n_cases, "ok": int(flag.item()) == 0, "ranks": h.world, "max_abs_err_bf16": worst,
            "what": "fused exchange and kernel + NCCL all-gather vs FP32 x @ W_full.T on every rank, and vs each other "
                    "bitwise where the plan is the same"}


def rowpar_table(h: Harness, steps: int, warmup: int) -> dict:
    """Column-parallel runs only: the `o` projection in its row-parallel layout (K sharded, the reference's real
    tensor-parallel layout, bf16_proj/reference.py:17) at m = 1 and 8: checked against an FP32 product of the
    full weight, then timed three ways on rotating cold copies: all-reduce inside the kernel (fused), kernel +
    NCCL all-reduce, and the local kernel alone."""
    from llm_inference_engine_b200 import tp

    proj, dist = h.proj, h.dist
    n, k = LAYERS["o"]
    k_loc = k // h.world
    nccl = tp.RowParallelProjection(proj.prepare, proj.kernel_fn)
    nccl.cols = {"o": k}
    fused = tp.FusedRowParallel(proj.prepare, proj.kernel_fn)
    fused.cols = {"o": k}
    fused._ensure_layer("o", n, h.device)
    copies = max(6, min(MAX_COPIES, -(-ROTATE_BYTES // (n * k_loc * 2))))
    states, fulls = [], []
    for i in range(copies):
        w = make_weight("o", h.device, SEED + 17 * i)
        if i == 0:
            fulls.append(w.float())
        states.append(proj.prepare({"o": w[:, h.rank * k_loc:(h.rank + 1) * k_loc].contiguous()}, warmup=(i == 0)))
        del w
    rows, bad = [], 0
    for m in (1, 8):
        x = make_x("o", m, h.device, 3000 + m)
        xl = x[:, h.rank * k_loc:(h.rank + 1) * k_loc].contiguous()
        data = {"x": xl, "config": {"m": m, "n": n, "k": k, "layer": "o"}}
        want = x.float() @ fulls[0].T
        for impl in (fused, nccl):
            got = impl.kernel_fn(data, states[0])
            tight = impl is fused
            bad += int(not torch.allclose(got.float(), want, rtol=1e-2 if tight else 2e-2, atol=1e-2 if tight else 5e-2))
        row = {"layer": "o (row-parallel)", "m": m, "n": n, "k_per_gpu": k_loc, "copies": copies}
        for key, fn_one in (("us", lambda st: fused.kernel_fn(data, st)), ("nccl_us", lambda st: nccl.kernel_fn(data, st)),
                            ("kernel_us", lambda st: nccl.kernel_fn_local(data, st))):
            keep = []

            def fn(fn_one=fn_one, keep=keep):
                keep.clear()
                for st in states:
                    keep.append(fn_one(st))

            row[key] = round(1e3 * h.time_graph(fn, steps, warmup) / copies, 3)
        rows.append(row)
    for st in states:
        proj.check_status(st)
    flag = torch.tensor([bad], device=h.device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.SUM)
    del states, fulls
    torch.cuda.empty_cache()
    return {"rows": rows, "parity_ok": int(flag.item()) == 0,
            "what": "o [4096,4096] with K sharded over the GPUs: us = all-reduce inside the kernel (FP32 partials, one NVLink flight), "
                    "nccl_us = kernel + NCCL all-reduce of BF16 partials, kernel_us = local kernel alone"}


def boundary_table(h: Harness, steps: int, warmup: int, only_m: int | None = None, only: str = "one_launch") -> list[dict]:
    """The path's first caller beyond the five projections (one GPU): the decode layer's post-attention boundary
    feeding the pooler and, up to 8 tokens in FP32, the router. Per token count, one graph per variant over
    rotating cold weight copies: the boundary as a kernel of its own in front of the two projections, and the
    boundary fused into both as their prologue; each with the router after the pooler on one stream and with
    the router forked to a side stream as the reference's layer does; and all three as one launch
    (muse_boundary_pooler_router)."""
    proj = h.proj
    layers = ("pooler", "router")
    copies = 80
    gate = torch.randn(LAYERS["pooler"][1], device=h.device, generator=torch.Generator(device=h.device).manual_seed(3)) * 0.3
    norm_w = (torch.randn(LAYERS["pooler"][1], device=h.device, generator=torch.Generator(device=h.device).manual_seed(4)) * 0.1).bfloat16()
    states = []
    for i in range(copies):
        st = proj.prepare({name: make_weight(name, h.device, SEED + 31 * i + j) for j, name in enumerate(layers)}, warmup=(i == 0))
        proj.prepare_boundary(st, gate, norm_w)
        states.append(st)
    side = torch.cuda.Stream(h.device)
    rows = []
    for m in (1, 4, 8):
        if only_m is not None and m != only_m:   # one case, one form (`only`): the command ncu wraps
            continue
        k = LAYERS["pooler"][1]
        g = torch.Generator(device=h.device).manual_seed(50 + m)
        stream_in = torch.randn((m, k), device=h.device, generator=g)
        attn_out = (torch.randn((m, k), device=h.device, generator=g) * 0.5).bfloat16()
        cfgs = {name: {"m": m, "n": LAYERS[name][0], "k": k, "layer": name} for name in layers}
        s1 = torch.empty_like(stream_in)
        row = {"m": m, "copies": copies}
        for fused in (False, True):
            for fork in (False, True):
                if only_m is not None and (fork or only != ("fused" if fused else "separate")):
                    continue
                keep = []

                def fn(fused=fused, fork=fork, keep=keep):
                    keep.clear()
                    for st in states:
                        if fused:
                            if fork:
                                side.wait_stream(torch.cuda.current_stream(h.device))
                            keep.append(proj.kernel_fn_boundary({"stream": stream_in, "attn_out": attn_out, "config": cfgs["pooler"]}, st, stream1=s1))
                            with torch.cuda.stream(side if fork else torch.cuda.current_stream(h.device)):
                                keep.append(proj.kernel_fn_boundary({"stream": stream_in, "attn_out": attn_out, "config": cfgs["router"]}, st))
                        else:
                            _, hb, hf = proj.attn_boundary(stream_in, attn_out, st)
                            if fork:
                                side.wait_stream(torch.cuda.current_stream(h.device))
                            keep.append(proj.kernel_fn({"x": hb, "config": cfgs["pooler"]}, st))
                            with torch.cuda.stream(side if fork else torch.cuda.current_stream(h.device)):
                                keep.append(proj.kernel_fn({"x": hf, "config": cfgs["router"]}, st))
                        if fork:
                            torch.cuda.current_stream(h.device).wait_stream(side)

                row[("fused" if fused else "separate") + ("_fork_us" if fork else "_us")] = 1e3 * h.time_graph(fn, steps, warmup) / copies

        def one(keep=[]):
            keep.clear()
            for st in states:
                keep.append(proj.boundary_pooler_router({"stream": stream_in, "attn_out": attn_out}, st, stream1=s1))

        if only_m is None or only == "one_launch":
            row["one_launch_us"] = 1e3 * h.time_graph(one, steps, warmup) / copies
        rows.append(row)
    for st in states:
        proj.check_status(st)
    del states
    torch.cuda.empty_cache()
    return rows


def ffn_boundary_table(h: Harness, steps: int, warmup: int, only_m: int | None = None) -> list[dict]:
    """The other caller-side step (one GPU): the unpooler's 1024-row slice followed by the post-FFN boundary, as two
    kernels (projection, boundary) and as one launch (muse_unpooler_ffn_boundary), per token count over rotating
    cold weight copies."""
    proj = h.proj
    n, k = LAYERS["unpooler"]
    nf = 1024                                   # this GPU's slice of the unpooler's rows up to 8 tokens
    copies = 80
    gen = lambda seed: torch.Generator(device=h.device).manual_seed(seed)  # noqa: E731
    gate = torch.randn(n, device=h.device, generator=gen(5)) * 0.3
    post_w = (torch.randn(n, device=h.device, generator=gen(6)) * 0.1).bfloat16()
    next_w = (torch.randn(n, device=h.device, generator=gen(7)) * 0.1).bfloat16()
    states = []
    for i in range(copies):
        st = proj.prepare({"unpooler": make_weight("unpooler", h.device, SEED + 13 * i)}, warmup=(i == 0))
        proj.prepare_ffn_boundary(st, gate, post_w, next_w)
        states.append(st)
    rows = []
    for m in (1, 4, 8):
        if only_m is not None and m != only_m:
            continue
        x = make_x("unpooler", m, h.device, 400 + m)
        stream1 = torch.randn((m, n), device=h.device, generator=gen(80 + m))
        cfg = {"m": m, "n": nf, "k": k, "layer": "unpooler"}
        row = {"m": m, "nf": nf, "copies": copies}
        keep = []

        def two(keep=keep):
            keep.clear()
            for st in states:
                f = proj.kernel_fn({"x": x, "config": cfg}, st)
                keep.append(proj.ffn_boundary(stream1, f, st))

        def one(keep=keep):
            keep.clear()
            for st in states:
                keep.append(proj.unpooler_ffn_boundary({"x": x, "stream1": stream1, "config": cfg}, st))

        row["separate_us"] = 1e3 * h.time_graph(two, steps, warmup) / copies
        row["one_launch_us"] = 1e3 * h.time_graph(one, steps, warmup) / copies
        rows.append(row)
    for st in states:
        proj.check_status(st)
    del states
    torch.cuda.empty_cache()
    return rows


def zip12_table(h: Harness, steps: int, warmup: int, only=None) -> list[dict]:
    """The lossless 12-bit weight form beside the plain walk (one GPU): us per call over rotating cold copies of
    qkv_gate and o at 1 and 8 tokens, and the bytes each reads."""
    proj = h.proj
    rows = []
    for layer in ("qkv_gate", "o"):
        if only and only[0] != layer:
            continue
        n, k = LAYERS[layer]
        copies = max(6, min(40, -(-(640 << 20) // (n * k * 2))))
        states = []
        for i in range(copies):
            st = proj.prepare({layer: make_weight(layer, h.device, SEED + 17 * i)}, warmup=(i == 0))
            proj.prepare_zip12(st)
            states.append(st)
        z = states[0]["_zip12"][layer]
        for m in (1, 8):
            if only and only[1] != m:
                continue
            data = {"x": make_x(layer, m, h.device, 300 + m), "config": {"m": m, "n": n, "k": k, "layer": layer}}
            row = {"layer": layer, "m": m, "copies": copies, "plain_bytes": n * k * 2, "zip12_bytes": z.nbytes,
                   "outside_window": z.exceptions / (n * k)}
            for name, fn in (("plain_us", proj.kernel_fn), ("zip12_us", proj.kernel_fn_zip12)):
                keep = []

                def body(fn=fn, keep=keep):
                    keep.clear()
                    for st in states:
                        keep.append(fn(data, st))

                row[name] = 1e3 * h.time_graph(body, steps, warmup) / copies
            rows.append(row)
        for st in states:
            proj.check_status(st)
        del states
        torch.cuda.empty_cache()
    return rows


def run_e2e(h: Harness, states, steps: int, warmup: int) -> dict:
    """The same six calls through the public API from HOST buffers: per call, x is copied from pinned
    host memory, the projection runs, and the result is copied back to pinned host memory and waited
    for. On one GPU that is kernel_fn_host() (staging copies and launch through the C ABI); column-parallel
    it is torch copies around the group's kernel_fn()."""
    n, k = LAYERS[WORKLOAD_LAYER]
    xs_host = [make_x(WORKLOAD_LAYER, m, "cpu", 1000 + m).pin_memory() for m in WORKLOAD_TOKENS]
    outs_host = [torch.empty((m, n), dtype=torch.bfloat16).pin_memory() for m in WORKLOAD_TOKENS]
    stream = h.timer.stream
    h2d = sum(x.numel() * 2 for x in xs_host)
    d2h = sum(o.numel() * 2 for o in outs_host)

    cfgs = [{"m": m, "n": n, "k": k, "layer": WORKLOAD_LAYER} for m in WORKLOAD_TOKENS]

    # Column-parallel: the recorded host round trip is used only if its first call worked on EVERY rank
    # (a rank that cannot record it must not leave the others waiting in a fused kernel).
    fused_host = h.world > 1 and h.fused is not None
    if fused_host:
        import torch.distributed as dist

        ok = 1
        try:
            with torch.cuda.stream(stream):
                h.fused.kernel_fn_host({"x": xs_host[0], "config": cfgs[0]}, states[0], outs_host[0])
        except Exception as e:  # noqa: BLE001
            print(f"[bench] rank {h.rank}: fused host round trip unavailable: {type(e).__name__}: {e}", file=sys.stderr)
            ok = 0
        flag = torch.tensor([ok], device=h.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        fused_host = bool(flag.item())

    def one_step():
        for j, (xh, oh) in enumerate(zip(xs_host, outs_host)):
            if h.world == 1:
                h.proj.kernel_fn_host({"x": xh, "config": cfgs[j]}, states[j], out=oh)
                continue
            if fused_host:
                h.fused.kernel_fn_host({"x": xh, "config": cfgs[j]}, states[j], oh)
                continue
            xd = xh.to(h.device, non_blocking=True)
            out = h.call(WORKLOAD_LAYER, xd, states[j])
            oh.copy_(out, non_blocking=True)
            stream.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(warmup):
            one_step()
        h.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            one_step()
        h.barrier()
        dt = time.perf_counter() - t0
    us = h.max_over_ranks(dt * 1e6 / (steps * len(WORKLOAD_TOKENS)))
    return {"value": us, "unit": "us/call", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "how": "wall clock around pinned-host x -> device, the projection, result -> pinned host, stream sync, per call; "
                   + ("kernel_fn_host(): copy-in, launch and copy-out recorded once per buffer pair as a CUDA graph, replayed and "
                      "synchronised every call; x comes in through a fetch kernel, and up to 8 tokens the projection kernel writes "
                      "the pinned output itself" if h.world == 1 else
                      "FusedColumnParallel.kernel_fn_host(): fetch kernel, column-parallel kernel with its exchange, copy kernel, "
                      "recorded as a CUDA graph per buffer pair" if fused_host else
                      "torch copies around the column-parallel kernel_fn()")}


def run_ours(args) -> None:
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line there.
    real_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj) -> None:
        os.write(real_stdout, (json.dumps(obj) + "\n").encode())

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    h = Harness(device, world, rank)
    if args.no_programmatic_launch:
        from llm_inference_engine_b200 import _capi

        _capi.load().muse_set_programmatic_launch(0)
    peak, peak_kind = measured_peak()
    sampler = ClockSampler(physical_gpu_index(local))
    n, k = LAYERS[WORKLOAD_LAYER]

    if args.boundary_only:
        with sampler:
            table = boundary_table(h, max(5, min(args.steps, 20)), args.warmup)
            ffn = ffn_boundary_table(h, max(5, min(args.steps, 20)), args.warmup)
        if rank == 0:
            emit({"boundary_pooler_router": table, "unpooler_ffn_boundary": ffn, "clocks": sampler.summary()})
        return

    if args.case:  # single case, few launches: the command ncu wraps
        layer, m = args.case.split(":")
        with sampler:
            if layer == "boundary_pooler_router":        # the one-launch boundary + pooler + router at m tokens
                rows = boundary_table(h, args.steps, args.warmup, only_m=int(m))
            elif layer in ("boundary_separate", "boundary_fused"):   # boundary kernel + two projections / the prologue form
                rows = boundary_table(h, args.steps, args.warmup, only_m=int(m), only=layer[9:])
            elif layer == "unpooler_ffn_boundary":       # unpooler slice + post-FFN boundary: two kernels, and one launch
                rows = ffn_boundary_table(h, args.steps, args.warmup, only_m=int(m))
            elif layer.startswith("zip12_"):             # zip12_qkv_gate:8, zip12_o:1: plain walk and 12-bit walk
                rows = zip12_table(h, args.steps, args.warmup, only=(layer[6:], int(m)))
            else:
                rows = case_table(h, [layer], args.steps, args.warmup, peak, only=(layer, int(m)))
        if rank == 0:
            emit({"case": rows[0], "clocks": sampler.summary()})
        return

    parity = None
    if world > 1:
        parity = gather_check(h)
        if not parity["ok"]:
            if rank == 0:
                emit({"error": "column-parallel output mismatch before timing", "parity_checked": parity})
            dist.destroy_process_group()
            raise SystemExit(3)

    # ---- headline: K steps of the six-call graph
    states = h.states(WORKLOAD_LAYER, len(WORKLOAD_TOKENS))
    xs = [make_x(WORKLOAD_LAYER, m, device, 1000 + m) for m in WORKLOAD_TOKENS]
    keep = []

    def step():
        keep.clear()
        for x, s in zip(xs, states):
            keep.append(h.call(WORKLOAD_LAYER, x, s))

    with sampler:
        ms_per_step = h.time_graph(step, args.steps, args.warmup)
        e2e = run_e2e(h, states, max(3, min(args.steps, 50)), args.warmup)
        nop_us = h.timer.nop_us()
        # The same step with every launch an ordinary one, reported beside `value`: how much of it is the overlap of
        # a call's launch and ramp with the previous call's tail (on every rank alike: the exchange kernels too).
        ordinary_us = None
        if not args.no_programmatic_launch:
            from llm_inference_engine_b200 import _capi

            lib = _capi.load()
            lib.muse_set_programmatic_launch(0)
            try:
                ordinary_us = 1e3 * h.time_graph(step, max(3, min(args.steps, 20)), args.warmup) / len(WORKLOAD_TOKENS)
            finally:
                lib.muse_set_programmatic_launch(1)
    for s in states:
        h.proj.check_status(s)
    del states, keep
    torch.cuda.empty_cache()
    value = 1e3 * ms_per_step / len(WORKLOAD_TOKENS)

    rows = []
    boundary_rows = []
    zip_rows = []
    ffn_rows = []
    rowpar = None
    if not args.no_table:
        with sampler:
            rows = case_table(h, list(CASES), max(5, min(args.steps, 20)), args.warmup, peak)
            if world == 1:
                boundary_rows = boundary_table(h, max(5, min(args.steps, 20)), args.warmup)
                ffn_rows = ffn_boundary_table(h, max(5, min(args.steps, 20)), args.warmup)
                zip_rows = zip12_table(h, max(5, min(args.steps, 20)), args.warmup)
            elif h.fused is not None:
                rowpar = rowpar_table(h, max(5, min(args.steps, 20)), args.warmup)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        us, info = cpu_path_us(WORKLOAD_TOKENS, WORKLOAD_LAYER, reps=100, warmup=3)
        cpu = {"value": us, "unit": "us/call", "cores": info["cores"], "kind": "port",
               "sample": f"all six calls of the workload ({WORKLOAD_LAYER} [12288,4096], m in {list(WORKLOAD_TOKENS)}), "
                         "100 timed repetitions each after 3 warm-ups, torch CPU x @ W.T with all host threads",
               "per_m_us": info["per_m_us"]}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # roofline of the dominant kernel: the kernel family with the largest share of the step's time, at the
    # largest m it serves in the workload
    work = [r for r in rows if r["layer"] == WORKLOAD_LAYER and r["m"] in WORKLOAD_TOKENS]
    share: dict[str, float] = {}
    for r in work:
        share[r["kernel"]] = share.get(r["kernel"], 0.0) + r.get("kernel_us", r["us"])
    dom = max((r for r in work if r["kernel"] == max(share, key=share.get)), key=lambda r: r["m"]) if work else None
    traffic = NCU_TRAFFIC
    if dom is not None:
        dur_us = dom.get("kernel_us", dom["us"])
        achieved = dom["bytes"] / dur_us / 1e3
        tr = traffic.get(f"{dom['kernel']} {WORKLOAD_LAYER} m={dom['m']}")
        roofline = {"bound": "hbm", "kernel": f"{dom['kernel']} ({WORKLOAD_LAYER} shard [{n // world},{k}], m={dom['m']})",
                    "share_of_step": {kf: round(v / sum(share.values()), 3) for kf, v in share.items()},
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                    "peak_kind": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                    "traffic": (tr / world if tr else None),
                    "traffic_kind": "static: ncu dram bytes of one 1-GPU launch of this kernel (profiles/), divided by the world size",
                    "bytes_per_launch": dom["bytes"], "us_per_launch": dur_us,
                    "frac_of_8tbs": achieved / NOMINAL_HBM_GBS}
    else:
        by = sum(algorithmic_bytes(WORKLOAD_LAYER, m, n // world, k) for m in WORKLOAD_TOKENS) / len(WORKLOAD_TOKENS)
        achieved = by / value / 1e3
        roofline = {"bound": "hbm", "kernel": "mean over the six calls of the step", "achieved": achieved,
                    "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": None}

    line = {
        "metric": METRIC, "value": value, "unit": "us/call", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT, "l2": L2_TEXT,
                   "arm": "one step = the six calls in one CUDA graph, each on its own weight copy; no flush in the timed region",
                   "parallelism": ("single GPU" if world == 1 else
                                   f"column-parallel x{world} (rows sharded), all-gather fused into the kernel (peer stores over NVLink)"
                                   if h.fused is not None else
                                   f"column-parallel x{world} (rows sharded) + NCCL all-gather in-graph (fused exchange unavailable: {h.fused_error})"),
                   "launch": ("every launch an ordinary one (--no-programmatic-launch)" if args.no_programmatic_launch else
                              "programmatic dependent launch: a call may become resident under the previous call's tail and reads only "
                              "weights until its grid-dependency wait"),
                   "timing": "CUDA events around K graph replays on the replaying stream, max over ranks"},
        "gpu_launches": args.steps * len(WORKLOAD_TOKENS),
        "nop_graph_replay_us": nop_us,
        "value_ordinary_launches": ordinary_us,
        "e2e": e2e,
        "roofline": roofline,
        "clocks": sampler.summary(),
        "cases": [{k2: (round(v, 4) if isinstance(v, float) else v) for k2, v in r.items()} for r in rows],
    }
    if boundary_rows:
        line["boundary_pooler_router"] = {
            "what": "us per (post-attention boundary -> pooler + router) of the decode layer, cold weights: boundary as its own "
                    "kernel (separate), as the prologue of both projections (fused), or all three as one launch (one_launch: muse_boundary_pooler_router); _fork = router on a side stream",
            "rows": [{k2: (round(v, 3) if isinstance(v, float) else v) for k2, v in r.items()} for r in boundary_rows]}
    if ffn_rows:
        line["unpooler_ffn_boundary"] = {
            "what": "us per (unpooler slice of 1024 rows -> post-FFN boundary) of the decode layer, cold weights: projection and "
                    "boundary as two kernels (separate) or as one launch (one_launch: muse_unpooler_ffn_boundary)",
            "rows": [{k2: (round(v, 3) if isinstance(v, float) else v) for k2, v in r.items()} for r in ffn_rows]}
    if zip_rows:
        line["zip12"] = {"what": "us per call, cold weights: the plain register-MMA walk and the same walk over the lossless 12-bit "
                                 "weight form (muse_fewtok_zip; not selected by the planner)",
                         "rows": [{k2: (round(v, 5) if isinstance(v, float) else v) for k2, v in r.items()} for r in zip_rows]}
    if rowpar is not None:
        line["row_parallel_o"] = rowpar
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if parity is not None:
        line["parity_checked"] = parity
    emit(line)
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--case", default=None, help="layer:m -- time one case only (the command ncu wraps)")
    ap.add_argument("--no-table", action="store_true", help="skip the per-case table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-programmatic-launch", action="store_true",
                    help="launch every kernel the ordinary way (no start under the previous kernel's tail): the A/B of that feature")
    ap.add_argument("--boundary-only", action="store_true", help="time only the boundary -> pooler + router table")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
