"""Drop-in for the reference's `muse_bf16_proj` submission: `prepare(weights)` once, then
`kernel_fn(data, state)` per call, same tensors, same meaning (best_submissions/muse_bf16_proj.py:340-390).

    out = x @ W[:n].T      BF16 for qkv_gate / o / pooler / unpooler, FP32 for the router

`weights` maps layer name -> [N, K] tensor on a CUDA device (BF16; FP32 for "router"); `data` is
`{"x": BF16 [m, K], "config": {"m", "n", "k", "layer"}}`; the result is a new [m, n] tensor. `n` may be
smaller than W's row count (the unpooler's per-GPU slice at up to 8 tokens, bf16_proj/reference.py:37-41).

Dispatch (shape-only: plan.py; a call is CUDA-graph capturable and replays identically):
  m == 1          streaming GEMV (csrc/gemv1.cu); the router reads its FP32 weights as they are
                  (the tall qkv_gate weight takes the register-MMA walk at m = 1 too)
  few tokens      persistent register-MMA walk over the weight (csrc/fewtok_mma.cu): up to 16 tokens on
                  the big weights, up to 64 on the small ones, up to 32 for the FP32 router (hi + lo
                  split in registers)
  everything else swap-AB split-K TMA + tcgen05 kernel (csrc/skinny_tc.cu), K slices reduced inside
                  thread-block clusters through distributed shared memory; the router runs its BF16
                  hi + lo pair (split once here, as the reference does at :346-349) into one FP32
                  accumulator
Every path is hand-written sm_100a CUDA reached through the C ABI (include/muse_proj.h); there is no
cuBLAS, Triton, PyTorch-matmul or CPU fallback: a non-CUDA tensor or a missing library raises.
"""

from __future__ import annotations

from typing import TypedDict

import ctypes

import torch

from . import _capi
from .plan import (FEWTOK_BUCKETS, GEMM_MIN_TOKENS, DeviceFacts, FewTokPlan, GemmPlan, GemvPlan, SkinnyPlan, fewtok_fused_plan,
                   fewtok_plan, gemm_plan, gemv_plan, gemv_valid, skinny_plan)

FP32_LAYERS = {"router"}
# Workspace rule: sized once in prepare() so that every layer at up to this many tokens can split K;
# beyond it a shape runs with a single K slice rather than allocating during a call.
WS_MAX_TOKENS = 256
CNT_INTS = 4096
WARMUP_TOKENS = (1, 2, 16, 32, 64, 128, 256)


class Config(TypedDict):
    m: int
    n: int
    k: int
    layer: str


class Inputs(TypedDict):
    x: torch.Tensor
    config: Config


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} is on {t.device}: this path runs on a CUDA device only (no CPU fallback)")


def split_hi_lo(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """FP32 -> BF16 hi + BF16 lo with hi = bf16(w), lo = bf16(w - fp32(hi)); hi + lo carries ~16
    mantissa bits of w (best_submissions/muse_bf16_proj.py:346-349; bf16_proj/baseline.py:49-50)."""
    hi = w.to(torch.bfloat16)
    lo = (w - hi.float()).to(torch.bfloat16)
    return hi.contiguous(), lo.contiguous()


def _stream_workspace(state, device) -> tuple[torch.Tensor, torch.Tensor]:
    """The split-K workspace of the current stream. A workspace is mid-reduction while a call runs,
    so calls that may overlap on the GPU (different streams) must not share one; the reference's
    decode layer keeps a second one for its side-stream router for this reason
    (best_submissions/muse_decode_layer.py:226-233)."""
    key = torch.cuda.current_stream(device).cuda_stream
    pool = state["_ws_by_stream"]
    if key not in pool:
        pool[key] = (torch.zeros(state["_ws_floats"], device=device, dtype=torch.float32),
                     torch.zeros(CNT_INTS, device=device, dtype=torch.int32))
    return pool[key]


def prepare(weights: dict[str, torch.Tensor], warmup: bool = True):
    """Weights as given (kept alive, never modified), the router's BF16 hi + lo halves, a zeroed
    split-K workspace with its tile counters, a device status word, and every kernel variant
    launched once so that no call configures anything later (mirrors
    best_submissions/muse_bf16_proj.py:340-366)."""
    lib = _capi.load()
    state: dict = {}
    device = None
    for name, w in weights.items():
        _require_cuda(w, f"weights[{name!r}]")
        if w.dim() != 2:
            raise ValueError(f"weights[{name!r}] must be [N, K], got {tuple(w.shape)}")
        want = torch.float32 if name in FP32_LAYERS else torch.bfloat16
        if w.dtype != want:
            raise TypeError(f"weights[{name!r}] must be {want}, got {w.dtype}")
        state[name] = w.contiguous()
        device = w.device
    if device is None:
        raise ValueError("prepare() needs at least one weight")
    with torch.cuda.device(device):
        cc = lib.muse_query(2)
        if cc < 100:
            raise RuntimeError(f"compute capability {cc / 10:.1f}: these kernels are sm_100a only")
        state["_dev"] = DeviceFacts(sms=lib.muse_query(0), smem_optin=lib.muse_query(1))
        for name in FP32_LAYERS & set(weights):
            hi, lo = split_hi_lo(state[name])
            state[f"_{name}_hi"], state[f"_{name}_lo"] = hi, lo
        n_max = max(-(-w.shape[0] // 128) * 128 for w in weights.values())
        # muse_skinny_tc with groups > 1 needs n x tokens floats; muse_gemm_tc with `split` slices meeting in the
        # workspace (split - 1) times that: room for four slices of the tallest weight, and never less than 16 MB.
        state["_ws_floats"] = max(3 * n_max * WS_MAX_TOKENS, 4 << 20)
        state["_ws_by_stream"] = {}
        state["_status"] = torch.zeros(1, device=device, dtype=torch.int32)
        state["_tmaps"] = {}
        state["_plans"] = {}
        state["_override"] = {}
        _stream_workspace(state, device)
        # The kernels read weights before they wait for the work ahead of them in the stream (they may start under
        # the previous kernel's tail): whatever produced these tensors must have completed before the first call.
        torch.cuda.synchronize(device)
        if warmup:
            for layer, w in weights.items():
                n, k = w.shape
                for m in WARMUP_TOKENS:
                    x = torch.zeros((m, k), device=device, dtype=torch.bfloat16)
                    kernel_fn({"x": x, "config": {"m": m, "n": n, "k": k, "layer": layer}}, state)
            check_status(state)
    return state


def _peer_ptr(peers):
    return None if peers is None else ctypes.addressof(peers)


def check_status(state) -> None:
    """Synchronise and raise if any kernel since the last check gave up on one of its bounded waits.
    Not for use inside a stream capture."""
    word = int(state["_status"].item())
    if word:
        state["_status"].zero_()
        raise _capi.MuseError(f"a kernel reported a timed-out wait: status bits {word:#x} (see MUSE_ST_* in muse_proj.h)")


def _weight_maps(state, layer: str, n: int, box_rows: int = 128):
    """TMA maps of W[:n] (hi and lo for FP32 layers) delivering boxes of `box_rows` rows, encoded once per key."""
    key = (layer, n, box_rows)
    maps = state["_tmaps"].get(key)
    if maps is None:
        if layer in FP32_LAYERS:
            srcs = (state[f"_{layer}_hi"], state[f"_{layer}_lo"])
        else:
            srcs = (state[layer],)
        maps = tuple(_capi.TensorMap.for_matrix(t.data_ptr(), n, t.shape[1], t.stride(0) * 2, box_rows) for t in srcs)
        state["_tmaps"][key] = maps
    return maps


def plan_for(state, layer: str, m: int, n: int, k: int, fused: bool = False) -> GemvPlan | FewTokPlan | SkinnyPlan | GemmPlan:
    """The (cached) launch plan of a shape; `state["_override"][(layer, m)]` = dict(cluster=, groups=, stages=),
    dict(wpr=, unroll=), dict(warps=, unroll=) or dict(pair=, cluster=, stages=) forces values for tuning
    sweeps. `fused` = the call carries a peer descriptor."""
    key = (layer, m, n, k, fused)
    ov = state["_override"].get((layer, m))
    if ov is None and key in state["_plans"]:
        return state["_plans"][key]
    f32 = layer in FP32_LAYERS
    dev = state["_dev"]
    few = None
    if ov and "warps" in ov:
        few = FewTokPlan(**ov)
    elif ov is None and fused:
        few = fewtok_fused_plan(m, n, k, f32)
    elif ov is None and m <= FEWTOK_BUCKETS[-1]:
        few = fewtok_plan(m, n, k, f32, dev)
    gemm = None
    from .plan import GEMM_BUCKETS, TUNED_GEMM   # fewer tokens take this kernel only where the table has measured it

    tabled = m < GEMM_MIN_TOKENS and any((n, k, b) in TUNED_GEMM for b in GEMM_BUCKETS if -(-m // 16) * 16 <= b < GEMM_MIN_TOKENS)
    if few is None and not f32 and (ov is None or "pair" in ov) and (m >= GEMM_MIN_TOKENS or ov or tabled):
        lib = _capi.load()
        fit = lambda ntok, pair, stages, cluster, m_, wgs: lib.muse_gemm_tc_max_clusters(ntok, int(pair), stages, cluster, m_, wgs, 128, 1)
        if fused and tabled:
            tabled = False   # the table holds whole-weight shapes; a rank's slice is planned by the rules
        gemm = gemm_plan(m, n, k, dev, max_clusters=fit, ws_floats_cap=state["_ws_floats"], cnt_cap=CNT_INTS, **(ov or {}))
    if few is not None:
        plan = few
    elif gemm is not None:
        plan = gemm
    elif m == 1 and any(gemv_valid(k, f32, w) for w in (1, 2, 4, 8)):
        plan = GemvPlan(**ov) if ov else gemv_plan(n, k, f32, dev)
    else:
        lib = _capi.load()
        fit = lambda ntok, hilo, m_, stages, cluster: lib.muse_skinny_max_clusters(ntok, int(hilo), m_, stages, cluster)
        plan = skinny_plan(m, n, k, f32, dev, ws_floats_cap=state["_ws_floats"], cnt_cap=CNT_INTS, max_clusters=fit,
                           **(ov or {}))
    if ov is None:
        state["_plans"][key] = plan
    return plan


def kernel_fn(data: Inputs, state, out: torch.Tensor | None = None, peers=None) -> torch.Tensor:
    """x @ W[:n].T as a new tensor: BF16, or FP32 for the router. `out` (optional, beyond the
    reference's signature) is a preallocated [m, >= n] destination whose row stride is honoured.
    `peers` (optional, column-parallel use: see tp.FusedColumnParallel) is a ctypes muse_peer_sync_t:
    the kernel then writes its slice into every rank's gathered output and `out` must be this
    rank's gathered [m, N] tensor, which is returned.

    The FP32 layers (the router) also take an FP32 x of up to 32 tokens: the FP32-input mode of the
    reference's decode layer (X_F32, best_submissions/muse_decode_layer.py:165-200, x split into
    BF16 hi + lo like the weight: out = x_hi (hi + lo) + x_lo hi)."""
    x, cfg = data["x"], data["config"]
    layer, n = cfg["layer"], int(cfg["n"])
    if layer not in state or layer.startswith("_"):
        raise KeyError(f"unknown layer {layer!r}")
    _require_cuda(x, "x")
    w = state[layer]
    if x.dim() == 2 and x.dtype == torch.float32 and layer in FP32_LAYERS:
        return _kernel_fn_f32_input(x, n, layer, state, out, peers)
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise TypeError(f"x must be BF16 [m, K], got {x.dtype} {tuple(x.shape)}")
    m, k = x.shape
    if k != w.shape[1] or not 0 < n <= w.shape[0] or m < 1:
        raise ValueError(f"{layer}: x {tuple(x.shape)} / n={n} do not fit W {tuple(w.shape)}")
    if x.stride(1) != 1 or x.data_ptr() % 16 or (m > 1 and (x.stride(0) % 8 or x.stride(0) < k)):
        x = x.contiguous().clone()  # same rule as the reference (:373-374)
    f32 = layer in FP32_LAYERS
    if out is None:
        out = torch.empty((m, n), device=x.device, dtype=torch.float32 if f32 else torch.bfloat16)
    elif out.shape[0] != m or out.shape[1] < n + (peers.col0 if peers is not None else 0) or out.stride(1) != 1 or out.dtype != (torch.float32 if f32 else torch.bfloat16):
        raise ValueError("out must be [m, >= n], unit column stride, BF16 (FP32 for the router)")
    stream = torch.cuda.current_stream(x.device).cuda_stream
    plan = plan_for(state, layer, m, n, k, fused=peers is not None)
    _launch(state, layer, plan, m, n, k, x.data_ptr(), x.stride(0) if m > 1 else k, out.data_ptr(), out.stride(0), peers,
            stream, x.device)
    return out


F32_INPUT_MAX_TOKENS = 32


def _kernel_fn_f32_input(x: torch.Tensor, n: int, layer: str, state, out, peers) -> torch.Tensor:
    """The router with FP32 activations: only the register-MMA kernel has this mode (up to 32 tokens,
    K <= 4096 in whole 32-element pieces, one GPU)."""
    w = state[layer]
    m, k = x.shape
    if k != w.shape[1] or not 0 < n <= w.shape[0] or m < 1:
        raise ValueError(f"{layer}: x {tuple(x.shape)} / n={n} do not fit W {tuple(w.shape)}")
    if peers is not None or m > F32_INPUT_MAX_TOKENS or k % 32 or k // 32 > 128:
        raise TypeError(f"{layer}: FP32 x is supported on one GPU for m <= {F32_INPUT_MAX_TOKENS}, K % 32 == 0, K <= 4096; "
                        f"got m={m}, K={k}")
    if x.stride(1) != 1 or x.data_ptr() % 16 or (m > 1 and (x.stride(0) % 8 or x.stride(0) < k)):
        x = x.contiguous().clone()
    if out is None:
        out = torch.empty((m, n), device=x.device, dtype=torch.float32)
    elif out.shape[0] != m or out.shape[1] < n or out.stride(1) != 1 or out.dtype != torch.float32:
        raise ValueError("out must be [m, >= n], unit column stride, FP32")
    kblocks = k // 32
    unroll = 2 if kblocks <= 32 else 4 if kblocks <= 64 else 8
    _capi.check(_capi.load().muse_fewtok_f32(w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n, k, x.stride(0) if m > 1 else k,
                                             out.stride(0), unroll, -(-m // 8), 1, torch.cuda.current_stream(x.device).cuda_stream),
                f"muse_fewtok_f32({layer}, m={m}, n={n}, k={k}, FP32 x)")
    return out


def _launch(state, layer: str, plan, m: int, n: int, k: int, x_ptr: int, ld_x: int, out_ptr: int, ld_out: int, peers,
            stream: int, device) -> None:
    """One C-ABI call: the kernel `plan` names, on validated arguments."""
    lib = _capi.load()
    f32 = layer in FP32_LAYERS
    w = state[layer]
    status = state["_status"].data_ptr()
    if isinstance(plan, FewTokPlan) and f32:
        _capi.check(lib.muse_fewtok_f32(w.data_ptr(), x_ptr, out_ptr, m, n, k, ld_x, ld_out, plan.unroll, plan.tok_split, 0, stream),
                    f"muse_fewtok_f32({layer}, m={m}, n={n}, k={k}, {plan})")
        return
    if isinstance(plan, FewTokPlan):
        _capi.check(lib.muse_fewtok_mma(w.data_ptr(), x_ptr, out_ptr, m, n, k, ld_x, ld_out, plan.warps, plan.unroll,
                                        plan.tok_split, status, _peer_ptr(peers), stream),
                    f"muse_fewtok_mma({layer}, m={m}, n={n}, k={k}, {plan})")
        return
    if isinstance(plan, GemvPlan):
        _capi.check(lib.muse_gemv1(w.data_ptr(), x_ptr, out_ptr, n, k, int(f32), plan.wpr, plan.unroll,
                                   int(plan.persistent), status, _peer_ptr(peers), stream), f"muse_gemv1({layer}, n={n}, k={k})")
        return
    maps = _weight_maps(state, layer, n, plan.tile_rows if isinstance(plan, GemmPlan) and not plan.pair else 128)
    if isinstance(plan, GemmPlan):
        ws_ptr = cnt_ptr = None
        if plan.split > 1:
            ws, cnt = _stream_workspace(state, device)
            ws_ptr, cnt_ptr = ws.data_ptr(), cnt.data_ptr()
        _capi.check(lib.muse_gemm_tc(maps[0].ptr, x_ptr, out_ptr, ws_ptr, cnt_ptr, status, m, n, k, ld_x, ld_out, plan.ntok,
                                     int(plan.pair), plan.cluster, plan.split, plan.stages, plan.warpgroups, plan.tile_rows,
                                     plan.k_atoms, _peer_ptr(peers), stream),
                    f"muse_gemm_tc({layer}, m={m}, n={n}, k={k}, {plan})")
        return
    ws_ptr = cnt_ptr = None
    if plan.groups > 1:
        ws, cnt = _stream_workspace(state, device)
        ws_ptr, cnt_ptr = ws.data_ptr(), cnt.data_ptr()
    _capi.check(lib.muse_skinny_tc(maps[0].ptr, maps[1].ptr if f32 else None, x_ptr, out_ptr, ws_ptr, cnt_ptr, status, m, n, k,
                                   ld_x, ld_out, plan.ntok, plan.cluster, plan.groups, plan.stages, int(f32),
                                   _peer_ptr(peers), stream),
                f"muse_skinny_tc({layer}, m={m}, n={n}, k={k}, {plan})")


# ---- the post-attention boundary in front of the pooler and the router ------------------------------------
RESIDUAL_TEMPERATURE = 0.3
RESIDUAL_GATE_EPS = 1e-3
BOUNDARY_FUSED_MAX_TOKENS = 8
ROUTER_FP32_INPUT_MAX_TOKENS = 8


def prepare_boundary(state, attn_residual_gate: torch.Tensor, pre_ffn_norm: torch.Tensor) -> None:
    """Once per layer: the residual coefficients of the gate, alpha and beta as FP32 vectors
    (decode_layer/reference.py:339-344; `_residual_coefficients` of best_submissions/muse_decode_layer.py), and
    the BF16 norm weight, kept in `state` for attn_boundary() and kernel_fn_boundary()."""
    _require_cuda(attn_residual_gate, "attn_residual_gate")
    _require_cuda(pre_ffn_norm, "pre_ffn_norm")
    w = attn_residual_gate.float() / RESIDUAL_TEMPERATURE
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=RESIDUAL_GATE_EPS))
    state["_boundary"] = (alpha.contiguous(), beta.contiguous(), pre_ffn_norm.to(torch.bfloat16).contiguous())


def _boundary_args(state, stream_in: torch.Tensor, attn_out: torch.Tensor, stream1, h, h_f32) -> _capi.Boundary:
    if "_boundary" not in state:
        raise RuntimeError("prepare_boundary(state, attn_residual_gate, pre_ffn_norm) has not been called")
    alpha, beta, norm_w = state["_boundary"]
    _require_cuda(stream_in, "stream")
    _require_cuda(attn_out, "attn_out")
    m, d = stream_in.shape
    if (stream_in.dtype != torch.float32 or attn_out.dtype != torch.bfloat16 or tuple(attn_out.shape) != (m, d)
            or not stream_in.is_contiguous() or not attn_out.is_contiguous() or alpha.numel() != d or d % 8):
        raise TypeError("stream must be contiguous FP32 [m, D] and attn_out contiguous BF16 [m, D], D as prepared and a multiple of 8")
    bd = _capi.Boundary()
    bd.stream, bd.attn_out, bd.alpha, bd.beta, bd.norm_w = (stream_in.data_ptr(), attn_out.data_ptr(), alpha.data_ptr(),
                                                            beta.data_ptr(), norm_w.data_ptr())
    for name, t, dt in (("stream1", stream1, torch.float32), ("h", h, torch.bfloat16), ("h_f32", h_f32, torch.float32)):
        if t is not None:
            if not t.is_cuda or t.dtype != dt or tuple(t.shape) != (m, d) or not t.is_contiguous():
                raise TypeError(f"{name} must be a contiguous CUDA {dt} [m, D] tensor")
            setattr(bd, name, t.data_ptr())
    return bd


def attn_boundary(stream_in: torch.Tensor, attn_out: torch.Tensor, state):
    """The boundary as a kernel of its own (any m, D <= 8192): returns (stream1 FP32, h BF16, h FP32 or None);
    the FP32 copy of h is made up to 8 tokens, where the router takes FP32 activations
    (best_submissions/muse_decode_layer.py:694-712 and its call at :855-858)."""
    m, d = stream_in.shape
    stream1 = torch.empty_like(stream_in)
    h = torch.empty((m, d), device=stream_in.device, dtype=torch.bfloat16)
    h_f32 = torch.empty_like(stream_in) if m <= ROUTER_FP32_INPUT_MAX_TOKENS else None
    bd = _boundary_args(state, stream_in, attn_out, stream1, h, h_f32)
    _capi.check(_capi.load().muse_attn_boundary(ctypes.addressof(bd), m, d, torch.cuda.current_stream(stream_in.device).cuda_stream),
                f"muse_attn_boundary(m={m}, d={d})")
    return stream1, h, h_f32


def kernel_fn_boundary(data, state, stream1: torch.Tensor | None = None, h: torch.Tensor | None = None,
                       h_f32: torch.Tensor | None = None) -> torch.Tensor:
    """kernel_fn for the pooler or the router with the post-attention boundary fused in as the projection's
    prologue: data = {"stream": FP32 [m, K], "attn_out": BF16 [m, K], "config": {"layer", "m", "n", "k"}} with
    m <= 8 and K <= 4096; returns h @ W[:n].T (BF16; FP32 for the router, which takes h in FP32). `stream1`,
    `h`, `h_f32` (optional, preallocated) are filled with the boundary's own outputs, which the rest of the
    layer needs. Larger m or K: attn_boundary() followed by kernel_fn()."""
    cfg = data["config"]
    layer, n = cfg["layer"], int(cfg["n"])
    if layer not in state or layer.startswith("_"):
        raise KeyError(f"unknown layer {layer!r}")
    w = state[layer]
    stream_in, attn_out = data["stream"], data["attn_out"]
    m, k = stream_in.shape
    if k != w.shape[1] or not 0 < n <= w.shape[0]:
        raise ValueError(f"{layer}: stream {tuple(stream_in.shape)} / n={n} do not fit W {tuple(w.shape)}")
    if m > BOUNDARY_FUSED_MAX_TOKENS or k > 4096 or k % 32 or -(-n // 8) < m:
        raise ValueError(f"the fused boundary serves m <= {BOUNDARY_FUSED_MAX_TOKENS}, K <= 4096 in whole 32-element pieces "
                         f"and n >= 8 m; got m={m}, K={k}, n={n}")
    f32 = layer in FP32_LAYERS
    out = torch.empty((m, n), device=stream_in.device, dtype=torch.float32 if f32 else torch.bfloat16)
    bd = _boundary_args(state, stream_in, attn_out, stream1, h, h_f32)
    _capi.check(_capi.load().muse_fewtok_boundary(w.data_ptr(), int(f32), ctypes.addressof(bd), out.data_ptr(), m, n, k, n,
                                                  state["_status"].data_ptr(), torch.cuda.current_stream(stream_in.device).cuda_stream),
                f"muse_fewtok_boundary({layer}, m={m}, n={n}, k={k})")
    return out


def boundary_pooler_router(data, state, stream1: torch.Tensor | None = None, h: torch.Tensor | None = None,
                           h_f32: torch.Tensor | None = None):
    """The boundary, the pooler and the router as one launch (three launches on two streams in the reference:
    best_submissions/muse_decode_layer.py:855-869): data = {"stream": FP32 [m, K], "attn_out": BF16 [m, K]} with
    m <= 8 and K <= 4096; returns (pooler output BF16 [m, n_pooler], router logits FP32 [m, n_router]), the same
    values as attn_boundary() followed by kernel_fn() gives for each layer. `stream1`, `h`, `h_f32` as there."""
    wp, wr = state["pooler"], state["router"]
    stream_in, attn_out = data["stream"], data["attn_out"]
    m, k = stream_in.shape
    if k != wp.shape[1] or k != wr.shape[1]:
        raise ValueError(f"stream {tuple(stream_in.shape)} does not fit the pooler {tuple(wp.shape)} / router {tuple(wr.shape)}")
    if m > BOUNDARY_FUSED_MAX_TOKENS or k > 4096 or k % 32 or -(-wp.shape[0] // 8) < m:
        raise ValueError(f"the fused boundary serves m <= {BOUNDARY_FUSED_MAX_TOKENS}, K <= 4096 in whole 32-element pieces "
                         f"and n >= 8 m; got m={m}, K={k}")
    dev = stream_in.device
    out_p = torch.empty((m, wp.shape[0]), device=dev, dtype=torch.bfloat16)
    out_r = torch.empty((m, wr.shape[0]), device=dev, dtype=torch.float32)
    if h is None:            # the kernel's CTAs hand h to one another through this and a scratch for its low half
        h = torch.empty((m, k), device=dev, dtype=torch.bfloat16)
    h_lo = torch.empty((m, k), device=dev, dtype=torch.bfloat16)
    bd = _boundary_args(state, stream_in, attn_out, stream1, h, h_f32)
    _, cnt = _stream_workspace(state, dev)
    _capi.check(_capi.load().muse_boundary_pooler_router(wp.data_ptr(), state["_router_hi"].data_ptr(), state["_router_lo"].data_ptr(),
                                                         ctypes.addressof(bd), h_lo.data_ptr(), out_p.data_ptr(), out_r.data_ptr(), m,
                                                         wp.shape[0], wr.shape[0], k, wp.shape[0], wr.shape[0], cnt.data_ptr(),
                                                         state["_status"].data_ptr(), torch.cuda.current_stream(dev).cuda_stream),
                f"muse_boundary_pooler_router(m={m}, k={k})")
    return out_p, out_r


def prepare_ffn_boundary(state, ffn_residual_gate: torch.Tensor, post_ffn_norm: torch.Tensor, next_pre_attn_norm: torch.Tensor) -> None:
    """Once per layer: the residual coefficients of the FFN gate as FP32 vectors and the two BF16 norm weights
    (decode_layer/reference.py:473-476), kept in `state` for ffn_boundary() and unpooler_ffn_boundary()."""
    for name, t in (("ffn_residual_gate", ffn_residual_gate), ("post_ffn_norm", post_ffn_norm), ("next_pre_attn_norm", next_pre_attn_norm)):
        _require_cuda(t, name)
    w = ffn_residual_gate.float() / RESIDUAL_TEMPERATURE
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=RESIDUAL_GATE_EPS))
    state["_ffn_boundary"] = (alpha.contiguous(), beta.contiguous(), post_ffn_norm.to(torch.bfloat16).contiguous(),
                              next_pre_attn_norm.to(torch.bfloat16).contiguous())


def _ffn_boundary_args(state, stream1: torch.Tensor, stream2, hidden: torch.Tensor) -> _capi.FfnBoundary:
    if "_ffn_boundary" not in state:
        raise RuntimeError("prepare_ffn_boundary(state, ffn_residual_gate, post_ffn_norm, next_pre_attn_norm) has not been called")
    alpha, beta, post_w, next_w = state["_ffn_boundary"]
    _require_cuda(stream1, "stream1")
    m, d = stream1.shape
    if stream1.dtype != torch.float32 or not stream1.is_contiguous() or alpha.numel() != d or d % 8 or d > 8192:
        raise TypeError("stream1 must be contiguous FP32 [m, D], D as prepared, a multiple of 8 and at most 8192")
    bd = _capi.FfnBoundary()
    bd.stream1, bd.alpha, bd.beta, bd.post_w, bd.next_w = (stream1.data_ptr(), alpha.data_ptr(), beta.data_ptr(), post_w.data_ptr(),
                                                           next_w.data_ptr())
    for name, t, dt in (("stream2", stream2, torch.float32), ("hidden", hidden, torch.bfloat16)):
        if t is not None:
            if not t.is_cuda or t.dtype != dt or tuple(t.shape) != (m, d) or not t.is_contiguous():
                raise TypeError(f"{name} must be a contiguous CUDA {dt} [m, D] tensor")
            setattr(bd, name, t.data_ptr())
    return bd


def ffn_boundary(stream1: torch.Tensor, f: torch.Tensor, state):
    """The post-FFN boundary as a kernel of its own (any m): f = the unpooler's BF16 output [m, nf], nf the hidden
    width or this GPU's slice of it (the other columns count as zero). Returns (stream2 FP32, the next layer's
    attention input BF16) (best_submissions/muse_decode_layer.py:715-730 and its call at :874-877)."""
    m, d = stream1.shape
    _require_cuda(f, "f")
    if f.dtype != torch.bfloat16 or f.dim() != 2 or f.shape[0] != m or not f.is_contiguous() or f.shape[1] % 8 or f.shape[1] > d:
        raise TypeError("f must be contiguous BF16 [m, nf] with nf a multiple of 8 and at most D")
    stream2 = torch.empty_like(stream1)
    hidden = torch.empty((m, d), device=stream1.device, dtype=torch.bfloat16)
    bd = _ffn_boundary_args(state, stream1, stream2, hidden)
    _capi.check(_capi.load().muse_ffn_boundary(ctypes.addressof(bd), f.data_ptr(), m, d, f.shape[1],
                                               torch.cuda.current_stream(stream1.device).cuda_stream),
                f"muse_ffn_boundary(m={m}, d={d}, nf={f.shape[1]})")
    return stream2, hidden


def unpooler_ffn_boundary(data, state):
    """The unpooler projection and the post-FFN boundary as one launch (two in the reference's layer,
    best_submissions/muse_decode_layer.py:869-877): data = {"x": BF16 [m, K] (the experts' output), "stream1":
    FP32 [m, D], "config": {"layer": "unpooler", "n": nf, ...}} with m <= 8; nf rows of the unpooler weight are
    used (the whole weight, or this GPU's slice). Returns (stream2 FP32, next attention input BF16); f itself
    stays in an FP32 scratch (it is not rounded to BF16 on the way, unlike the two-kernel route)."""
    cfg = data["config"]
    layer, nf = cfg.get("layer", "unpooler"), int(cfg["n"])
    w = state[layer]
    x, stream1 = data["x"], data["stream1"]
    _require_cuda(x, "x")
    m, k = x.shape
    d = stream1.shape[1]
    if x.dtype != torch.bfloat16 or k != w.shape[1] or x.stride(1) != 1 or stream1.shape[0] != m:
        raise ValueError(f"{layer}: x {tuple(x.shape)} {x.dtype} / stream1 {tuple(stream1.shape)} do not fit W {tuple(w.shape)}")
    if m > BOUNDARY_FUSED_MAX_TOKENS or k > 4096 or k % 32 or nf % 8 or not 8 * m <= nf <= min(w.shape[0], d):
        raise ValueError(f"the fused form serves m <= {BOUNDARY_FUSED_MAX_TOKENS}, K <= 4096 in whole 32-element pieces and "
                         f"8 m <= nf <= min(N, D) in multiples of 8; got m={m}, K={k}, nf={nf}")
    dev = x.device
    stream2 = torch.empty_like(stream1)
    hidden = torch.empty((m, d), device=dev, dtype=torch.bfloat16)
    scratch = torch.empty((m, nf), device=dev, dtype=torch.float32)
    bd = _ffn_boundary_args(state, stream1, stream2, hidden)
    _, cnt = _stream_workspace(state, dev)
    _capi.check(_capi.load().muse_unpooler_ffn_boundary(w.data_ptr(), x.data_ptr(), scratch.data_ptr(), ctypes.addressof(bd), m, nf, k,
                                                        x.stride(0), d, cnt[16:].data_ptr(), state["_status"].data_ptr(),
                                                        torch.cuda.current_stream(dev).cuda_stream),
                f"muse_unpooler_ffn_boundary(m={m}, nf={nf}, k={k}, d={d})")
    return stream2, hidden


def prepare_zip12(state, layers=None) -> dict:
    """The lossless 12-bit form (zip12.encode) of the BF16 weights named in `layers` (default: all of them), kept in
    `state` beside the weights for kernel_fn_zip12(). Returns {layer: exceptions / weights}; a layer the form does
    not cover (K not a multiple of 128, too many weights outside the window in one row group) is left out."""
    from . import zip12

    done = {}
    for name in (layers if layers is not None else [k for k in state if not k.startswith("_") and k not in FP32_LAYERS]):
        w = state[name]
        if w.dtype != torch.bfloat16:
            raise TypeError(f"{name}: the 12-bit form is for BF16 weights")
        z = zip12.encode(w)
        if z is not None:
            state.setdefault("_zip12", {})[name] = z
            done[name] = z.exceptions / w.numel()
    if done:
        torch.cuda.synchronize(next(iter(state["_zip12"].values())).low.device)   # the planes are weights: complete before the first call
    return done


ZIP12_PLANS = ((4096, 32, 4), (2048, 16, 4))      # K up to -> (warps, unroll)


def kernel_fn_zip12(data, state) -> torch.Tensor:
    """kernel_fn through the 12-bit form of the weight (1..8 tokens, the whole weight: n = N): the same values as
    the plain register-MMA walk gives, from 25 % fewer bytes. Not what kernel_fn() selects: on B200 it is no
    faster than the plain walk (18.1-18.4 us against 18.1-18.4 us on qkv_gate, 8.9 against 8.3 on o)."""
    cfg = data["config"]
    layer, n = cfg["layer"], int(cfg["n"])
    z = state.get("_zip12", {}).get(layer)
    if z is None:
        raise KeyError(f"{layer}: prepare_zip12() has not made a 12-bit form of this layer")
    x = data["x"]
    _require_cuda(x, "x")
    m, k = x.shape
    if x.dtype != torch.bfloat16 or k != z.k or n != z.n or not 1 <= m <= 8 or x.stride(1) != 1:
        raise ValueError(f"{layer}: the 12-bit path takes BF16 x [1..8, {z.k}] and n = {z.n}; got {tuple(x.shape)} {x.dtype}, n={n}")
    plan = next(((w, u) for kmax, w, u in ZIP12_PLANS[::-1] if k <= kmax), None)
    if plan is None:
        raise ValueError(f"{layer}: K = {k} is wider than the 12-bit kernel's 4096")
    out = torch.empty((m, n), device=x.device, dtype=torch.bfloat16)
    _capi.check(_capi.load().muse_fewtok_zip(z.low.data_ptr(), z.code.data_ptr(), z.table.data_ptr() if z.cap else None, z.cap, z.base,
                                             x.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), n, plan[0], plan[1], 1,
                                             torch.cuda.current_stream(x.device).cuda_stream),
                f"muse_fewtok_zip({layer}, m={m}, n={n}, k={k})")
    return out


FETCH_X_BY_KERNEL = True
STORE_OUT_BY_KERNEL = True   # the copy-out of the larger calls by the same small kernel (786 KB: 5 us less than the copy engine)
FETCH_MAX_TOKENS = 32       # x up to 256 KB: the fetch kernel beats the copy engine at every size measured
DIRECT_OUT_MAX_TOKENS = 8   # beyond: 16-byte PCIe writes cost more than the copy-out they replace
DIRECT_OUT_GEMM_MAX_TOKENS = 32   # the many-token GEMM writes 176 contiguous bytes per token and CTA: measured 56 vs 59.5 us at m = 32, no gain at 64
HOST_GRAPH_SLOTS = 64   # recorded round trips kept per state (oldest dropped first)
_EMPTY: dict = {}


def kernel_fn_host(data: Inputs, state, out: torch.Tensor | None = None, record: bool = True) -> torch.Tensor:
    """kernel_fn for a caller whose activations live in HOST memory: `data["x"]` is a contiguous BF16
    [m, K] CPU tensor (page-locked for an asynchronous copy), the result is a CPU tensor (`out` if
    given: contiguous [m, n], page-locked), complete when the call returns. x is staged into a device
    buffer kept per (layer, m, n), the projection runs on the current stream, and the result is copied
    back and waited for. When the caller passes the same x and out tensors again (the normal case: its
    own pinned buffers), the copy-in, launch and copy-out are recorded once as a CUDA graph and replayed;
    x comes in through muse_fetch_host up to 32 tokens, and up to 8 tokens the projection kernel writes
    the pinned output itself (no copy nodes at all). `record=False` keeps the plain form: one C-ABI
    call for the register-MMA plans, three otherwise.
    Beyond the reference, whose harness owns the transfers (best_submissions/muse_bf16_proj.py:369-372)."""
    x, cfg = data["x"], data["config"]
    layer, n = cfg["layer"], int(cfg["n"])
    if record and out is not None:   # a recorded round trip of exactly these buffers: nothing left to check
        entry = state.get("_host_graphs", _EMPTY).get((layer, x.shape[0], n, x.data_ptr(), out.data_ptr()))
        if entry is not None:
            entry[0].replay()
            torch.cuda.current_stream(entry[3]).synchronize()
            return out
    if layer not in state or layer.startswith("_"):
        raise KeyError(f"unknown layer {layer!r}")
    w = state[layer]
    if x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous():
        raise TypeError("x must be a contiguous BF16 [m, K] CPU tensor")
    m, k = x.shape
    if k != w.shape[1] or not 0 < n <= w.shape[0] or m < 1:
        raise ValueError(f"{layer}: x {tuple(x.shape)} / n={n} do not fit W {tuple(w.shape)}")
    f32 = layer in FP32_LAYERS
    odt = torch.float32 if f32 else torch.bfloat16
    key = (layer, m, n)
    slot = state.setdefault("_host_slots", {}).get(key)
    if slot is None:
        slot = (torch.empty((m, k), device=w.device, dtype=torch.bfloat16), torch.empty((m, n), device=w.device, dtype=odt),
                plan_for(state, layer, m, n, k))
        state["_host_slots"][key] = slot
    x_dev, out_dev, plan = slot
    fresh_out = out is None
    if fresh_out:
        out = torch.empty((m, n), dtype=odt, pin_memory=True)
    elif out.is_cuda or out.dtype != odt or tuple(out.shape) != (m, n) or not out.is_contiguous():
        raise ValueError("out must be a contiguous CPU [m, n] tensor, BF16 (FP32 for the router)")
    lib = _capi.load()
    cur = torch.cuda.current_stream(w.device)
    stream = cur.cuda_stream
    if record and not fresh_out and x.is_pinned() and out.is_pinned():
        graphs = state.setdefault("_host_graphs", {})
        # The plain form once (it also warms every lazily created resource), then the recording.
        kernel_fn_host(data, state, out=out, record=False)
        # The register-MMA kernel stores its output as 16-byte vectors, one PCIe write each when the
        # destination is page-locked host memory (device-addressable under unified addressing): it then
        # writes the caller's buffer itself while it streams the weights, and the copy-out disappears.
        direct = (isinstance(plan, FewTokPlan) and not f32 and n % 8 == 0 and out.data_ptr() % 16 == 0
                  and m <= DIRECT_OUT_MAX_TOKENS)
        # The many-token GEMM stores a token's rows of one CTA as neighbouring 16-byte vectors (176 contiguous bytes
        # per token with 88-row tiles), which the PCIe link takes as large writes.
        direct = direct or (isinstance(plan, GemmPlan) and n % 8 == 0 and out.data_ptr() % 16 == 0
                            and m <= DIRECT_OUT_GEMM_MAX_TOKENS)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            rec = torch.cuda.current_stream(w.device).cuda_stream
            if FETCH_X_BY_KERNEL and m <= FETCH_MAX_TOKENS and x.data_ptr() % 16 == 0:   # x comes in by a small kernel
                _capi.check(lib.muse_fetch_host(x_dev.data_ptr(), x.data_ptr(), m * k * 2, rec), "muse_fetch_host")
            else:
                x_dev.copy_(x, non_blocking=True)
            _launch(state, layer, plan, m, n, k, x_dev.data_ptr(), k, out.data_ptr() if direct else out_dev.data_ptr(), n, None,
                    rec, w.device)
            if not direct and STORE_OUT_BY_KERNEL and out.data_ptr() % 16 == 0 and (out.numel() * out.element_size()) % 16 == 0:
                _capi.check(lib.muse_fetch_host(out.data_ptr(), out_dev.data_ptr(), out.numel() * out.element_size(), rec),
                            "muse_fetch_host (copy-out)")
            elif not direct:
                out.copy_(out_dev, non_blocking=True)
        if len(graphs) >= HOST_GRAPH_SLOTS:
            graphs.pop(next(iter(graphs)))
        # the tensors stay alive as long as their addresses are baked in
        graphs[(layer, m, n, x.data_ptr(), out.data_ptr())] = (graph, x, out, w.device)
        graph.replay()
        cur.synchronize()
        return out
    if isinstance(plan, FewTokPlan) and not f32:   # the whole round trip in one C call
        _capi.check(lib.muse_fewtok_mma_host(w.data_ptr(), x.data_ptr(), x_dev.data_ptr(), out_dev.data_ptr(), out.data_ptr(), m, n,
                                             k, plan.warps, plan.unroll, plan.tok_split, state["_status"].data_ptr(), stream),
                    f"muse_fewtok_mma_host({layer}, m={m}, n={n}, k={k}, {plan})")
        return out
    _capi.check(lib.muse_copy_h2d_async(x_dev.data_ptr(), x.data_ptr(), m * k * 2, stream), "muse_copy_h2d_async")
    _launch(state, layer, plan, m, n, k, x_dev.data_ptr(), k, out_dev.data_ptr(), n, None, stream, w.device)
    _capi.check(lib.muse_copy_d2h_sync(out.data_ptr(), out_dev.data_ptr(), out.numel() * out.element_size(), stream),
                "muse_copy_d2h_sync")
    return out
