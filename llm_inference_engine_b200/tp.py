"""Column-parallel projections: each rank holds a contiguous block of W's output rows, computes its
slice of `out` with the single-GPU kernels, and the slices are all-gathered (NCCL over NVLink on
GPUs) into the full [m, N] on every rank.

The reference runs on one GPU and only carries the per-GPU shapes of such a split ("the sliced
unpooler's all-gather is not run", bf16_proj/baseline.py:11); this is the exchange step it leaves out.
One process per GPU, `torch.distributed` for the plumbing. The local compute is injected so that
the sharding / gather / layout logic can be exercised with CPU ranks over gloo.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [start, stop) of an N-row weight owned by `rank`; equal blocks (all-gather needs them)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of world {world}")
    if n % world:
        raise ValueError(f"N={n} does not split into {world} equal row blocks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weights(weights: dict[str, torch.Tensor], world: int, rank: int) -> dict[str, torch.Tensor]:
    """This rank's row block of every weight, as an independent tensor (the full weight can be freed)."""
    out = {}
    for name, w in weights.items():
        a, b = shard_bounds(w.shape[0], world, rank)
        out[name] = w[a:b].clone()
    return out


class ColumnParallelProjection:
    """prepare()/kernel_fn() with the same meaning as the single-GPU entry points, over a group.

    `local_prepare(weights) -> state` and `local_kernel_fn(data, state) -> Tensor` are the
    single-device implementation (llm_inference_engine_b200.muse_bf16_proj on GPUs).
    """

    def __init__(self, local_prepare: Callable, local_kernel_fn: Callable, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._prepare = local_prepare
        self._kernel_fn = local_kernel_fn
        self.rows: dict[str, int] = {}

    def prepare(self, weights: dict[str, torch.Tensor], already_sharded: bool = False):
        if already_sharded:
            shards = weights
            self.rows = {k: v.shape[0] * self.world for k, v in weights.items()}
        else:
            shards = shard_weights(weights, self.world, self.rank)
            self.rows = {k: v.shape[0] for k, v in weights.items()}
        return self._prepare(shards)

    def local_config(self, cfg: dict) -> dict:
        n = int(cfg["n"])
        if n != self.rows[cfg["layer"]]:
            raise ValueError(f"column-parallel calls take the whole weight: n={n} != {self.rows[cfg['layer']]}")
        return dict(cfg, n=n // self.world)

    def kernel_fn_local(self, data: dict, state) -> torch.Tensor:
        """This rank's [m, N / world] slice only (what the roofline of one GPU is measured on)."""
        return self._kernel_fn({"x": data["x"], "config": self.local_config(data["config"])}, state)

    def gather(self, part: torch.Tensor) -> torch.Tensor:
        """[m, N/world] per rank -> [m, N] on every rank, rank r's block at columns r*N/world."""
        m, n_loc = part.shape
        buf = torch.empty((self.world * m, n_loc), device=part.device, dtype=part.dtype)
        dist.all_gather_into_tensor(buf, part.contiguous(), group=self.group)
        if m == 1:
            return buf.reshape(1, self.world * n_loc)  # already in place: no copy
        return buf.view(self.world, m, n_loc).permute(1, 0, 2).reshape(m, self.world * n_loc)

    def kernel_fn(self, data: dict, state) -> torch.Tensor:
        return self.gather(self.kernel_fn_local(data, state))


def shard_columns(weights: dict[str, torch.Tensor], world: int, rank: int) -> dict[str, torch.Tensor]:
    """This rank's block of every weight's K columns (the reduction dimension), as an independent tensor."""
    out = {}
    for name, w in weights.items():
        a, b = shard_bounds(w.shape[1], world, rank)
        out[name] = w[:, a:b].contiguous()
    return out


class RowParallelProjection:
    """Row-parallel projections: each rank holds a block of W's K columns and the matching slice of x (in the
    reference's model the `o` projection, whose input, the attention output, is already split by heads:
    bf16_proj/reference.py:17), computes a partial [m, N] with the single-GPU kernels, and the partials are
    summed over the group. This class is the baseline: the local kernel (BF16 partials, as a stock tensor-
    parallel stack exchanges them) followed by an NCCL all-reduce. The local compute is injected so that the
    sharding and reduction logic runs with CPU ranks over gloo."""

    def __init__(self, local_prepare: Callable, local_kernel_fn: Callable, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._prepare = local_prepare
        self._kernel_fn = local_kernel_fn
        self.cols: dict[str, int] = {}

    def prepare(self, weights: dict[str, torch.Tensor], already_sharded: bool = False):
        if already_sharded:
            shards = weights
            self.cols = {k: v.shape[1] * self.world for k, v in weights.items()}
        else:
            shards = shard_columns(weights, self.world, self.rank)
            self.cols = {k: v.shape[1] for k, v in weights.items()}
        return self._prepare(shards)

    def local_x(self, x: torch.Tensor) -> torch.Tensor:
        """The slice of a full [m, K] activation this rank multiplies (callers that already hold the slice skip this)."""
        a, b = shard_bounds(x.shape[1], self.world, self.rank)
        return x[:, a:b]

    def local_config(self, cfg: dict) -> dict:
        k = int(cfg["k"])
        if k != self.cols[cfg["layer"]]:
            raise ValueError(f"row-parallel calls name the whole reduction dimension: k={k} != {self.cols[cfg['layer']]}")
        return dict(cfg, k=k // self.world)

    def kernel_fn_local(self, data: dict, state) -> torch.Tensor:
        """This rank's partial [m, N]; data["x"] is the local [m, K / world] slice."""
        return self._kernel_fn({"x": data["x"], "config": self.local_config(data["config"])}, state)

    def kernel_fn(self, data: dict, state) -> torch.Tensor:
        part = self.kernel_fn_local(data, state)
        dist.all_reduce(part, group=self.group)
        return part


class FusedRowParallel(RowParallelProjection):
    """Row-parallel projections whose all-reduce is part of the kernel (GPUs of one node, up to 8 tokens):
    muse_fewtok_rowpar sends FP32 partial sums to every rank's staging in symmetric memory as self-validating
    lines and adds up all ranks' lines itself, so the result is FP32-accumulated across ranks, identical on
    every rank, and needs one NVLink flight and no collective call. More tokens take the baseline route."""

    def __init__(self, local_prepare: Callable, local_kernel_fn: Callable, group=None):
        super().__init__(local_prepare, local_kernel_fn, group)
        from . import _capi

        if self.world > _capi.MAX_WORLD:
            raise ValueError(f"world {self.world} > {_capi.MAX_WORLD}")
        self._capi = _capi
        self._ll: dict[str, torch.Tensor] = {}
        self._peers: dict[str, object] = {}
        self._handles: list = []
        self._flags = None
        self._flag_ptrs = None

    def _rendezvous(self, t: torch.Tensor):
        import torch.distributed._symmetric_memory as symm

        hdl = symm.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        self._handles.append(hdl)
        off = int(getattr(hdl, "offset", 0) or 0)
        return [int(p) + off for p in hdl.buffer_ptrs]

    def _ensure_layer(self, name: str, rows: int, device) -> None:
        if name in self._peers:
            return
        import torch.distributed._symmetric_memory as symm

        if self._flags is None:
            self._flags = symm.empty((32,), dtype=torch.int32, device=device)
            self._flags.zero_()
            self._flag_ptrs = self._rendezvous(self._flags)
        # 2 halves x sending rank x token x output row, 8 bytes each (an FP32 partial sum and its call number)
        ll = symm.empty((2, self.world, self._capi.RP_TOKENS, rows, 2), dtype=torch.int32, device=device)
        ll.zero_()
        ll_ptrs = self._rendezvous(ll)
        ps = self._capi.PeerSync()
        ps.world, ps.rank, ps.col0 = self.world, self.rank, 0
        for p in range(self.world):
            ps.flags[p] = self._flag_ptrs[p]
            ps.ll[p] = ll_ptrs[p]
        self._ll[name], self._peers[name] = ll, ps
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)   # every rank's staging is zero and mapped before anyone launches

    def prepare(self, weights: dict[str, torch.Tensor], already_sharded: bool = False):
        state = super().prepare(weights, already_sharded)
        for name, w in weights.items():
            if w.dtype == torch.bfloat16:
                self._ensure_layer(name, w.shape[0], w.device)
        return state

    def kernel_fn(self, data: dict, state) -> torch.Tensor:
        import ctypes

        x, cfg = data["x"], self.local_config(data["config"])
        layer, n, k_loc = cfg["layer"], int(cfg["n"]), int(cfg["k"])
        m = x.shape[0]
        w = state[layer]
        if (layer not in self._peers or m > self._capi.RP_TOKENS or k_loc % 32 or k_loc > 4096 or n != w.shape[0] or n % 8
                or x.dtype != torch.bfloat16):
            return super().kernel_fn(data, state)
        if tuple(x.shape) != (m, k_loc) or not x.is_cuda:
            raise ValueError(f"{layer}: x must be this rank's CUDA [m, {k_loc}] slice, got {tuple(x.shape)} on {x.device}")
        if x.stride(1) != 1 or x.data_ptr() % 16 or (m > 1 and (x.stride(0) % 8 or x.stride(0) < k_loc)):
            x = x.contiguous().clone()
        out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
        self._capi.check(self._capi.load().muse_fewtok_rowpar(
            w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n, k_loc, x.stride(0) if m > 1 else k_loc, n,
            state["_status"].data_ptr(), ctypes.addressof(self._peers[layer]), torch.cuda.current_stream(x.device).cuda_stream),
            f"muse_fewtok_rowpar({layer}, m={m}, n={n}, k={k_loc})")
        return out


class FusedColumnParallel(ColumnParallelProjection):
    """Column-parallel projections whose all-gather is part of the kernel (GPUs of one node).

    Every rank owns, per layer, a gathered output buffer [max_tokens, N] in symmetric (peer-mapped)
    memory. A call runs the single-GPU kernel with a muse_peer_sync_t descriptor: the epilogue stores
    this rank's [m, N / world] slice at its columns of EVERY rank's buffer with plain stores over
    NVLink, and two rounds of peer-mapped flags (entered / done) order the ranks, so when the kernel
    completes the local buffer holds the whole [m, N]: no NCCL call, no re-layout copy.

    The returned tensor is a view of that buffer; it is overwritten by the layer's next call, so
    consume it in stream order before calling the layer again (every rank must make the same
    sequence of calls). `torch.distributed._symmetric_memory` provides the peer mapping.
    """

    def __init__(self, local_prepare: Callable, local_kernel_fn: Callable, group=None, max_tokens: int = 256):
        super().__init__(local_prepare, local_kernel_fn, group)
        from . import _capi

        if self.world > _capi.MAX_WORLD:
            raise ValueError(f"world {self.world} > {_capi.MAX_WORLD}")
        self.max_tokens = max_tokens
        self._capi = _capi
        self._bufs: dict[str, torch.Tensor] = {}
        self._ll: dict[str, torch.Tensor] = {}
        self._host_graphs: dict = {}
        self._peers: dict[str, object] = {}
        self._handles: list = []
        self._flags = None
        self._flag_ptrs = None

    def _rendezvous(self, t: torch.Tensor):
        import torch.distributed._symmetric_memory as symm

        hdl = symm.rendezvous(t, self.group if self.group is not None else dist.group.WORLD)
        self._handles.append(hdl)
        off = int(getattr(hdl, "offset", 0) or 0)
        return [int(p) + off for p in hdl.buffer_ptrs]

    def _symm_empty(self, shape, dtype, device):
        import torch.distributed._symmetric_memory as symm

        return symm.empty(shape, dtype=dtype, device=device)

    def _ensure_layer(self, name: str, rows: int, dtype: torch.dtype, device) -> None:
        if name in self._bufs:
            return
        if self._flags is None:
            self._flags = self._symm_empty((32,), torch.int32, device)
            self._flags.zero_()
            self._flag_ptrs = self._rendezvous(self._flags)
        buf = self._symm_empty((self.max_tokens, rows), dtype, device)
        ptrs = self._rendezvous(buf)
        # staging of the register-MMA kernel's exchange: 2 halves x sending rank x token x slice column, 4 bytes each
        ll = self._symm_empty((2, self.world, self._capi.LL_TOKENS, rows // self.world), torch.int32, device)
        ll.zero_()
        ll_ptrs = self._rendezvous(ll)
        ps = self._capi.PeerSync()
        ps.world, ps.rank, ps.col0 = self.world, self.rank, self.rank * (rows // self.world)
        for p in range(self.world):
            ps.out[p] = ptrs[p]
            ps.flags[p] = self._flag_ptrs[p]
            ps.ll[p] = ll_ptrs[p]
        self._bufs[name], self._peers[name] = buf, ps
        self._ll[name] = ll
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)   # every rank's flags are zero and mapped before anyone launches

    def prepare(self, weights: dict[str, torch.Tensor], already_sharded: bool = False):
        state = super().prepare(weights, already_sharded)
        for name, w in weights.items():
            dtype = torch.float32 if w.dtype == torch.float32 else torch.bfloat16
            self._ensure_layer(name, self.rows[name], dtype, w.device)
        return state

    def kernel_fn(self, data: dict, state) -> torch.Tensor:
        layer = data["config"]["layer"]
        m = data["x"].shape[0]
        if m > self.max_tokens:
            raise ValueError(f"m={m} exceeds the gathered buffers ({self.max_tokens} tokens)")
        out = self._bufs[layer][:m]
        local = {"x": data["x"], "config": self.local_config(data["config"])}
        return self._kernel_fn(local, state, out=out, peers=self._peers[layer])

    HOST_GRAPH_SLOTS = 64   # recorded round trips kept (oldest dropped first)

    def kernel_fn_host(self, data: dict, state, out: torch.Tensor) -> torch.Tensor:
        """kernel_fn for activations in page-locked HOST memory: x [m, K] BF16 comes in through a small
        fetch kernel, the column-parallel kernel runs (exchange included), and the gathered [m, N] is
        copied into `out` (page-locked, contiguous) by the same small kernel; the three launches are
        recorded once per (state, layer, m, x, out) as a CUDA graph, replayed and synchronised on every call.

        Every rank must make the same calls in the same order, as for kernel_fn. A call runs exactly one
        exchange whether it finds its recording or not: the first call of a buffer pair runs the three
        launches in the open and then records them WITHOUT replaying, so a rank that alone lost its
        entry (say it re-pinned a buffer) stays in step with its peers. Time-outs of the exchange are
        reported through muse_bf16_proj.check_status(state), which the caller polls outside the hot loop."""
        x = data["x"]
        layer = data["config"]["layer"]
        m, k = x.shape
        key = (id(state), layer, m, int(data["config"]["n"]), x.data_ptr(), out.data_ptr())
        entry = self._host_graphs.get(key)
        if entry is None:
            n = self.rows[layer]
            if (x.is_cuda or out.is_cuda or not x.is_pinned() or not out.is_pinned() or not x.is_contiguous()
                    or not out.is_contiguous() or tuple(out.shape) != (m, n) or x.dtype != torch.bfloat16
                    or out.dtype != self._bufs[layer].dtype or m > self.max_tokens):
                raise ValueError("x and out must be contiguous page-locked CPU tensors, x BF16 [m, K], out [m, N] in the layer's output type")
            device = self._bufs[layer].device
            x_dev = torch.empty((m, k), device=device, dtype=torch.bfloat16)
            lib = self._capi.load()
            cfg = dict(data["config"])

            def body(stream: int) -> None:
                self._capi.check(lib.muse_fetch_host(x_dev.data_ptr(), x.data_ptr(), m * k * 2, stream), "muse_fetch_host")
                gathered = self.kernel_fn({"x": x_dev, "config": cfg}, state)
                self._capi.check(lib.muse_fetch_host(out.data_ptr(), gathered.data_ptr(), out.numel() * out.element_size(), stream),
                                 "muse_fetch_host (copy-out)")

            cur = torch.cuda.current_stream(device)
            body(cur.cuda_stream)          # this call's result; every lazily created resource exists afterwards
            cur.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):  # recorded for the next calls, not run now
                body(torch.cuda.current_stream(device).cuda_stream)
            if len(self._host_graphs) >= self.HOST_GRAPH_SLOTS:
                self._host_graphs.pop(next(iter(self._host_graphs)))
            # the state and the tensors stay alive as long as their addresses are baked in
            self._host_graphs[key] = (graph, x, out, x_dev, device, state)
            return out
        entry[0].replay()
        torch.cuda.current_stream(entry[4]).synchronize()
        return out
