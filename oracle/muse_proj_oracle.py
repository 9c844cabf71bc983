"""CPU oracle for the `muse_bf16_proj` path. TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline / reference arm may import this
module, and only as the checker or the timed CPU baseline. The product package never imports it.

It restates, in plain PyTorch on the CPU, the reference's problem definition and check:
  bf16_proj/reference.py   shapes (LAYERS :15-21), the unpooler slice rule (:37-41), seeded weight and
                           input generators with probe rows and outlier channels (:44-69), the FP64
                           reference product (:72-76), the check (:84-99), the speed-of-light floor (:102-107)
  bf16_proj/checks.py      compare(): whole-output and per-row relative L2 (:31-55)
  bf16_proj/baseline.py    what the reference is timed against (:46-65), restated without sglang:
                           BF16 layers are a plain x @ W.T; the router is F.linear in FP32 up to 8
                           tokens and two products on the BF16 hi/lo halves above
  decode_layer/reference.py  the post-attention boundary that produces the pooler's and the router's input
                           (_rms :189-191, residual_coefficients :339-344, ref_front :452-454)
Parity is PINNED: tests/test_oracle_golden.py checks every function here against vectors produced
by importing the reference itself (tests/golden/make_golden.py and make_boundary_golden.py wrote them).

Beside the reference's own geometry (per-GPU TP8 slices of an 8192-hidden model) this module
carries the 4096-hidden geometry the benchmark is quoted on (TARGET_LAYERS) with its own input
distributions: weights ~ N(0, 0.02), x ~ N(0, 1), no probe rows.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

# ---- the reference's geometry (bf16_proj/reference.py:15-34) -------------------------------------
REFERENCE_LAYERS = {
    "qkv_gate": (2304, 8192),
    "o": (8192, 1024),
    "pooler": (4096, 8192),
    "unpooler": (8192, 4096),
    "router": (256, 8192),
}
UNPOOL_SLICE_ROWS = 1024
SLICE_UP_TO_TOKENS = 8
FP32_LAYERS = frozenset({"router"})
WEIGHTS_SEED = 5151
BF16_REL_L2_TOL = 1e-2
ROUTER_REL_L2_TOL = 1e-4
PROBE_ONE_IN = 8
PROBE_REL_TOL = 1e-3
# bf16_proj/checks.py:14-17
ROW_TOL_FACTOR = 5.0
ROW_NORM_FLOOR_FRACTION = 0.1
# bf16_proj/baseline.py:43
ROUTER_FP32_UP_TO_TOKENS = 8

# ---- the geometry the benchmark is quoted on ------------------------------------------------------
TARGET_LAYERS = {
    "qkv_gate": (12288, 4096),
    "o": (4096, 4096),
    "pooler": (1024, 4096),
    "unpooler": (4096, 1024),
    "router": (256, 4096),
}
TARGET_WEIGHT_STD = 0.02
TARGET_TOKENS = {
    "qkv_gate": (1, 2, 4, 8, 16, 32),
    "o": (1,),
    "router": (1, 8, 32, 128, 256),
    "pooler": (1, 32, 64, 128, 256),
    "unpooler": (1, 32, 64, 128, 256),
}
TARGET_BF16_RTOL = 1e-2
TARGET_BF16_ATOL = 1e-2
TARGET_ROUTER_REL = 1e-5


def out_features(layer: str, m: int, layers=REFERENCE_LAYERS) -> int:
    """Rows of W one call computes; reference.py:37-41: the unpooler is sliced at up to 8 tokens."""
    full = layers[layer][0]
    if layers is REFERENCE_LAYERS and layer == "unpooler" and m <= SLICE_UP_TO_TOKENS:
        return UNPOOL_SLICE_ROWS
    return full


def _dtype_of(layer: str) -> torch.dtype:
    return torch.float32 if layer in FP32_LAYERS else torch.bfloat16


def generate_weights(seed: int = WEIGHTS_SEED, device: str = "cpu", layers=REFERENCE_LAYERS):
    """reference.py:44-49: one generator, layers in table order, randn / sqrt(K), cast per layer."""
    g = torch.Generator(device=device).manual_seed(seed)
    weights = {}
    for name, (n, k) in layers.items():
        w = torch.randn((n, k), generator=g, device=device) / math.sqrt(k)
        weights[name] = w.to(_dtype_of(name))
    return weights


def generate_input(m: int, layer: str, seed: int, dist: str = "normal", device: str = "cpu",
                   layers=REFERENCE_LAYERS):
    """reference.py:52-69. The draw order matters for bit-equality with the reference: x, (outlier
    permutation), probe mask, (forced probe row), spike columns, signs, powers."""
    g = torch.Generator(device=device).manual_seed(seed)
    k = layers[layer][1]
    x = torch.randn((m, k), generator=g, device=device)
    if dist == "outliers":
        hot = torch.randperm(k, generator=g, device=device)[: max(1, k // 100)]
        x[:, hot] *= 30
    is_probe = torch.rand((m,), generator=g, device=device) < 1 / PROBE_ONE_IN
    if m >= PROBE_ONE_IN:
        is_probe[torch.randint(m, (1,), generator=g, device=device)] = True
    col = torch.randint(k, (m,), generator=g, device=device)
    sign = torch.randint(2, (m,), generator=g, device=device) * 2 - 1
    power = torch.randint(3, 8, (m,), generator=g, device=device)
    value = (sign * 2.0 ** power).float()
    one_hot = torch.zeros_like(x).scatter_(1, col[:, None], value[:, None])
    x = torch.where(is_probe[:, None], one_hot, x)
    cfg = {"m": m, "n": out_features(layer, m, layers), "k": k, "layer": layer}
    return {"x": x.to(torch.bfloat16), "config": cfg}


def ref_kernel(data, weights) -> torch.Tensor:
    """reference.py:72-76: FP64 product, rounded once to the layer's output type."""
    layer, n = data["config"]["layer"], data["config"]["n"]
    exact = data["x"].double() @ weights[layer][:n].double().T
    return exact.to(_dtype_of(layer))


def probe_rows(x: torch.Tensor) -> torch.Tensor:
    """reference.py:79-81: rows with exactly one non-zero entry."""
    return ((x != 0).sum(-1) == 1).nonzero().flatten()


def relative_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """checks.py:20-22."""
    return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))


def compare(output, ref: torch.Tensor, tol: float) -> tuple[bool, str]:
    """checks.py:31-55, messages included (the golden test compares them verbatim)."""
    if not isinstance(output, torch.Tensor):
        return False, f"expected a tensor, got {type(output).__name__}"
    if output.shape != ref.shape or output.dtype != ref.dtype:
        return False, f"expected {tuple(ref.shape)} {ref.dtype}, got {tuple(output.shape)} {output.dtype}"
    got = output.float()
    if not torch.isfinite(got).all():
        return False, "output contains NaN or Inf"
    want = ref.float()
    delta = got - want
    err = float(delta.norm() / want.norm().clamp(min=1e-12))
    if err > tol:
        return False, f"relative L2 error {err:.3e} > {tol:g}"
    width = want.shape[-1]
    d_rows = delta.reshape(-1, width).norm(dim=-1)
    w_rows = want.reshape(-1, width).norm(dim=-1)
    floor = (ROW_NORM_FLOOR_FRACTION * w_rows.mean()).clamp(min=1e-12)
    row_err = d_rows / torch.maximum(w_rows, floor)
    worst = int(row_err.argmax())
    worst_err = float(row_err[worst])
    if worst_err > ROW_TOL_FACTOR * tol:
        where = (tuple(int(i) for i in torch.unravel_index(torch.tensor(worst), want.shape[:-1]))
                 if want.dim() > 1 else ())
        return False, (f"relative L2 error {err:.3e}, but row {where} is off by {worst_err:.3e}"
                       f" > {ROW_TOL_FACTOR:g} x {tol:g}")
    return True, f"relative L2 error {err:.3e} (worst row {worst_err:.3e})"


def check_implementation(data, output, weights) -> tuple[bool, str]:
    """reference.py:84-99: compare() at the layer's tolerance, then every probe row within 1e-3."""
    layer = data["config"]["layer"]
    tol = ROUTER_REL_L2_TOL if layer in FP32_LAYERS else BF16_REL_L2_TOL
    ref = ref_kernel(data, weights)
    ok, msg = compare(output, ref, tol)
    rows = probe_rows(data["x"])
    if not ok or not len(rows):
        return ok, msg
    want = ref[rows].double()
    off = (output[rows].double() - want).norm(dim=-1) / want.norm(dim=-1).clamp(min=1e-30)
    worst = int(off.argmax())
    if float(off[worst]) > PROBE_REL_TOL:
        return False, (f"{msg}, but probe row {int(rows[worst])} (one nonzero input, so a weight column, exact"
                       f" with the weights as given) is off by {float(off[worst]):.2e} > {PROBE_REL_TOL:g}: are the weights"
                       " used at their own precision?")
    return True, f"{msg}; {len(rows)} probe rows exact to {float(off.max()):.1e}"


def algorithmic_bytes(m: int, n: int, k: int, layer: str) -> int:
    """Bytes a call must move: weights once, x once, out once (the byte term of reference.py:102-107)."""
    wb = 4 if layer in FP32_LAYERS else 2
    return n * k * wb + m * k * 2 + m * n * wb


def speed_of_light_ns(m: int, layer: str, hw: dict, layers=REFERENCE_LAYERS) -> float:
    """reference.py:102-107: the slower of bytes / HBM rate and flops / dense BF16 rate."""
    n, k = out_features(layer, m, layers), layers[layer][1]
    by = algorithmic_bytes(m, n, k, layer)
    return 1e9 * max(by / hw["hbm_bytes_per_s"], 2.0 * m * n * k / hw["bf16_dense_flops_per_s"])


# ---- the reference's timed counterpart, runnable on CPU (bf16_proj/baseline.py:46-65) ------------

def cpu_prepare(weights):
    """baseline.py:46-53 without the transposed copies (they only serve cuBLAS's layout)."""
    state = {name: w.contiguous() for name, w in weights.items()}
    if "router" in weights:
        hi = weights["router"].to(torch.bfloat16)
        state["router_hi"] = hi
        state["router_lo"] = (weights["router"] - hi.float()).to(torch.bfloat16)
    return state


def cpu_kernel_fn(data, state) -> torch.Tensor:
    """baseline.py:56-65 as torch CPU ops. `_bf16_gemm_dispatch_impl` is a cuBLAS BF16 GEMM, i.e.
    x @ W.T; `torch.mm(out_dtype=float32)` does not exist on CPU, so the hi/lo products are taken
    in FP32 (the same sums: BF16 products are exact in FP32)."""
    x, layer, n = data["x"], data["config"]["layer"], data["config"]["n"]
    if layer not in FP32_LAYERS:
        return x @ state[layer][:n].T
    if x.shape[0] <= ROUTER_FP32_UP_TO_TOKENS:
        return F.linear(x.float(), state["router"][:n])
    xf = x.float()
    return xf @ state["router_hi"][:n].float().T + xf @ state["router_lo"][:n].float().T


# ---- the decode layer's FP32-input router mode (the path's first "next" caller) --------------------

def router_f32_input_model(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The arithmetic of `_router_kernel(..., X_F32=True)` (best_submissions/muse_decode_layer.py:165-200;
    math in README.md:192-194): x and W are FP32, each split into BF16 hi = bf16(v) and lo = bf16(v - hi),
    and out = x_hi (W_hi + W_lo)^T + x_lo W_hi^T with FP32 accumulation (the x_lo W_lo term, ~2^-32
    relative, is dropped). Taken in FP64 here, so this is the value the kernel should reach up to FP32
    summation error. Parity unpinned by a golden vector: the reference checkout holds no stored outputs
    of this mode and its Triton kernel does not run on CPU; the FP64 product of the unsplit inputs
    (`router_f32_input_reference`) bounds it, "FP32-accurate to ~2^-16" in the reference's words."""
    xh = x.to(torch.bfloat16)
    xl = (x - xh.float()).to(torch.bfloat16)
    wh = w.to(torch.bfloat16)
    wl = (w - wh.float()).to(torch.bfloat16)
    return (xh.double() @ (wh.double() + wl.double()).T + xl.double() @ wh.double().T).float()


def router_f32_input_reference(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """FP64 product of the FP32 inputs as given: the yardstick of the mode above."""
    return (x.double() @ w.double().T)


# ---- the post-attention boundary, the producer of the pooler's and the router's input ----------------------
# decode_layer/reference.py: RMS_EPS :39, POST_NORM_EPS :40, RESIDUAL_TEMPERATURE :54, RESIDUAL_GATE_EPS :55.
RMS_EPS = 1e-5
POST_NORM_EPS = 1e-8
RESIDUAL_TEMPERATURE = 0.3
RESIDUAL_GATE_EPS = 1e-3
ROUTER_FP32_INPUT_UP_TO_TOKENS = 8   # best_submissions/muse_decode_layer.py: ROUTER_FP32_MAX_TOKENS


def rms(x: torch.Tensor, eps: float = RMS_EPS) -> torch.Tensor:
    """decode_layer/reference.py:189-191."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def residual_coefficients(gate: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """decode_layer/reference.py:339-344 (the norm-preserving residual): new = alpha * stream + beta * branch."""
    w = gate.float() / RESIDUAL_TEMPERATURE
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=RESIDUAL_GATE_EPS))
    return alpha, beta


def attn_boundary(stream: torch.Tensor, attn_out: torch.Tensor, gate: torch.Tensor, pre_ffn_norm: torch.Tensor):
    """decode_layer/reference.py:452-454 (ref_front after the `o` projection): the residual stream after the
    attention block and the normalised input of the pooler and the router, both FP32:
        stream1 = alpha * stream + beta * rms(attn_out, 1e-8);  h = rms(stream1, 1e-5) * (1 + pre_ffn_norm).
    The submission's kernel for it (best_submissions/muse_decode_layer.py:694-712) takes attn_out in BF16 (the
    projection's output type) and writes h as BF16 and, up to 8 tokens, as FP32 for the router."""
    alpha, beta = residual_coefficients(gate)
    stream1 = alpha * stream.float() + beta * rms(attn_out, POST_NORM_EPS)
    h = rms(stream1) * (1.0 + pre_ffn_norm.float())
    return stream1, h


def ffn_boundary(stream1: torch.Tensor, f: torch.Tensor, gate: torch.Tensor, post_ffn_norm: torch.Tensor,
                 next_pre_attn_norm: torch.Tensor):
    """decode_layer/reference.py:466-476 (the tail of ref_back): the unpooler's output f [m, nf] (nf = the hidden
    width, or this GPU's first UNPOOL_SLICE columns up to 8 tokens, the other columns being the all-gather's
    zeros) scaled by (1 + post_ffn_norm), joined to the residual stream, and the next layer's pre-attention norm:
        f' = pad(f) * (1 + post_ffn_norm);  stream2 = alpha * stream1 + beta * rms(f', 1e-8);
        hidden = rms(stream2, 1e-5) * (1 + next_pre_attn_norm)           (both returned in FP32).
    The submission's kernel for it is best_submissions/muse_decode_layer.py:715-730."""
    m, d = stream1.shape
    full = torch.zeros((m, d), dtype=torch.float32, device=stream1.device)
    full[:, : f.shape[1]] = f.float()
    full = full * (1.0 + post_ffn_norm.float())
    alpha, beta = residual_coefficients(gate)
    stream2 = alpha * stream1.float() + beta * rms(full, POST_NORM_EPS)
    hidden = rms(stream2) * (1.0 + next_pre_attn_norm.float())
    return stream2, hidden


def ffn_boundary_inputs(m: int, d: int, nf: int, seed: int, device: str = "cpu"):
    """Seeded inputs of the post-FFN boundary: FP32 stream1 with a shared mean direction, the unpooler output
    f [m, nf] in BF16, a residual gate ~ N(0, 0.3) and the two norm weights ~ N(0, 0.1) in BF16."""
    g = torch.Generator(device=device).manual_seed(seed)
    mean = torch.randn((d,), generator=g, device=device)
    stream1 = 0.7 * mean + torch.randn((m, d), generator=g, device=device)
    f = (0.4 * torch.randn((m, nf), generator=g, device=device)).to(torch.bfloat16)
    gate = 0.3 * torch.randn((d,), generator=g, device=device)
    post_w = (0.1 * torch.randn((d,), generator=g, device=device)).to(torch.bfloat16)
    next_w = (0.1 * torch.randn((d,), generator=g, device=device)).to(torch.bfloat16)
    return stream1, f, gate, post_w, next_w


def boundary_inputs(m: int, d: int, seed: int, device: str = "cpu"):
    """Seeded inputs of the boundary in the shapes and types the decode layer hands over: FP32 stream with a
    shared mean direction (rows are far from zero-mean, as in decode_layer/reference.py:132-137), BF16
    attention output, a residual gate ~ N(0, 0.3) and a norm weight ~ N(0, 0.1) in BF16."""
    g = torch.Generator(device=device).manual_seed(seed)
    mean = torch.randn((d,), generator=g, device=device)
    stream = 0.7 * mean + torch.randn((m, d), generator=g, device=device)
    attn_out = (0.5 * torch.randn((m, d), generator=g, device=device)).to(torch.bfloat16)
    gate = 0.3 * torch.randn((d,), generator=g, device=device)
    norm_w = (0.1 * torch.randn((d,), generator=g, device=device)).to(torch.bfloat16)
    return stream, attn_out, gate, norm_w


# ---- the benchmark's own synthetic data and acceptance rule ---------------------------------------

def target_weights(seed: int = WEIGHTS_SEED, device: str = "cpu", layers=TARGET_LAYERS, only=None):
    """W ~ N(0, 0.02): BF16, FP32 for the router. One generator per layer (seed + index) so that a
    single layer can be produced without drawing the others."""
    out = {}
    for i, (name, (n, k)) in enumerate(layers.items()):
        if only is not None and name not in only:
            continue
        g = torch.Generator(device=device).manual_seed(seed + i)
        out[name] = (torch.randn((n, k), generator=g, device=device) * TARGET_WEIGHT_STD).to(_dtype_of(name))
    return out


def target_input(m: int, layer: str, seed: int, device: str = "cpu", layers=TARGET_LAYERS):
    """x ~ N(0, 1) BF16 [m, K] with the reference's config dict."""
    n, k = layers[layer]
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((m, k), generator=g, device=device).to(torch.bfloat16)
    return {"x": x, "config": {"m": m, "n": n, "k": k, "layer": layer}}


def fp32_reference(data, weights) -> torch.Tensor:
    """The acceptance reference of the benchmark: FP32-accumulated x @ W[:n].T, unrounded."""
    layer, n = data["config"]["layer"], data["config"]["n"]
    return data["x"].float() @ weights[layer][:n].float().T


def target_check(data, output, weights) -> tuple[bool, str]:
    """BF16 layers: |out - ref| <= 1e-2 + 1e-2 |ref| elementwise against the FP32-accumulated
    reference. Router: relative L2 error <= 1e-5 against the FP64 product of the FP32 weights."""
    layer, n = data["config"]["layer"], data["config"]["n"]
    want_dtype = _dtype_of(layer)
    if tuple(output.shape) != (data["x"].shape[0], n) or output.dtype != want_dtype:
        return False, f"expected {(data['x'].shape[0], n)} {want_dtype}, got {tuple(output.shape)} {output.dtype}"
    if not torch.isfinite(output.float()).all():
        return False, "output contains NaN or Inf"
    if layer in FP32_LAYERS:
        exact = data["x"].double() @ weights[layer][:n].double().T
        err = float((output.double() - exact).norm() / exact.norm().clamp(min=1e-30))
        return err <= TARGET_ROUTER_REL, f"router relative L2 error {err:.3e} (limit {TARGET_ROUTER_REL:g})"
    ref = fp32_reference(data, weights)
    excess = (output.float() - ref).abs() - (TARGET_BF16_ATOL + TARGET_BF16_RTOL * ref.abs())
    worst = float(excess.max())
    return worst <= 0, f"worst |out-ref| - (atol + rtol|ref|) = {worst:.3e} (must be <= 0)"


def zip12_decode(low: torch.Tensor, code: torch.Tensor, table: torch.Tensor, base: int) -> torch.Tensor:
    """The BF16 matrix a 12-bit form stands for (the inverse of the reference's `_zip`,
    bf16_proj/probe18.py:332-362, for the lane-major layouts the CUDA kernel reads): raw low byte, high byte =
    sign << 7 | base + index from the 4-bit code, and the table's true values put back where the code could not
    hold them. Plain index arithmetic, no shared code with the encoder's permutes."""
    n, k = low.shape
    low, code = low.cpu().to(torch.int32), code.cpu().to(torch.int32)
    rows = torch.arange(n).view(n, 1).expand(n, k)
    col = torch.arange(k).view(1, k).expand(n, k)
    piece, within = col // 32, col % 32
    q, j = within // 8, within % 8                                   # lane of the piece, weight of the lane
    low_at = (piece // 2) * 64 + q * 16 + (piece % 2) * 8 + j
    code_at = (piece // 4) * 64 + q * 16 + (piece % 4) * 4 + (j % 4)
    lo = torch.gather(low, 1, low_at)
    nb = torch.gather(code, 1, code_at)
    c = torch.where(j < 4, nb & 15, nb >> 4)
    hi = ((c & 8) << 4) | ((c & 7) + base)
    bits = (hi << 8) | lo
    out = (bits - ((bits >= 32768).to(torch.int32) << 16)).to(torch.int16).view(torch.bfloat16).clone()   # 16-bit pattern -> BF16
    t = table.cpu()
    if t.numel():
        grp, slot = (t[:, :, 0] >= 0).nonzero(as_tuple=True)
        rc = t[grp, slot, 0]
        vals = t[grp, slot, 1].contiguous().view(torch.float32)
        out[grp * 8 + (rc >> 16), rc & 0xFFFF] = vals.to(torch.bfloat16)
    return out
