"""Per-call timing the way the path is deployed and the way the reference was judged: the call is
captured once in a CUDA graph and replayed from a cold L2, each replay bracketed by CUDA events on
the replaying stream (protocol of the reference's bench(), bf16_proj/tune.py:79-98). Between replays
a buffer several times the L2 size is overwritten so that no weight byte survives in cache.
"""

from __future__ import annotations

import statistics

import torch

from . import _capi

FLUSH_BYTES = 1 << 30  # 1 GiB written between replays; B200's L2 is 126 MB


class ColdReplayTimer:
    def __init__(self, device, flush_bytes: int = FLUSH_BYTES):
        self.device = torch.device(device)
        self.flush = torch.empty(flush_bytes, device=self.device, dtype=torch.uint8)
        self.stream = torch.cuda.Stream(self.device)
        self._nop_us: float | None = None

    def capture(self, fn) -> torch.cuda.CUDAGraph:
        """Run `fn` once eagerly on the timing stream (configures anything lazy), then capture it."""
        with torch.cuda.stream(self.stream):
            fn()
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                fn()
        return graph

    def time(self, graph: torch.cuda.CUDAGraph, reps: int, warmup: int = 3, cold: bool = True) -> list[float]:
        """Microseconds of each of `reps` replays (after `warmup` untimed ones)."""
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
        stops = [torch.cuda.Event(enable_timing=True) for _ in range(reps)]
        with torch.cuda.stream(self.stream):
            for i in range(-warmup, reps):
                if cold:
                    self.flush.fill_(i & 0xFF)
                if i < 0:
                    graph.replay()
                    continue
                starts[i].record(self.stream)
                graph.replay()
                stops[i].record(self.stream)
            self.stream.synchronize()
        return [1e3 * a.elapsed_time(b) for a, b in zip(starts, stops)]

    def nop_us(self, reps: int = 200) -> float:
        """Median replay time of a graph holding one empty kernel: the floor under every number."""
        if self._nop_us is None:
            lib = _capi.load()
            graph = self.capture(lambda: _capi.check(lib.muse_nop(torch.cuda.current_stream(self.device).cuda_stream), "muse_nop"))
            self._nop_us = statistics.median(self.time(graph, reps))
        return self._nop_us


def summarize(us: list[float]) -> dict:
    s = sorted(us)
    n = len(s)
    return {"median_us": statistics.median(s), "p10_us": s[n // 10], "p90_us": s[(9 * n) // 10], "min_us": s[0],
            "mean_us": sum(s) / n, "reps": n}
