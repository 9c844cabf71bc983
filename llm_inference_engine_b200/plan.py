"""Shape-only launch planning for the projection kernels.

A plan depends on (n, k, m, weight type) and on device facts (SM count, shared memory), never on
tensor values, so a call captured in a CUDA graph takes the same path when replayed. The
reference hard-codes its plans per layer for one H200 (best_submissions/muse_bf16_proj.py:56-62
GEMV_CONFIGS, :205-212 BF16_CONFIGS, :290-299 _router_config); here they are derived, with a small
table of measured overrides for the shapes that were swept on a B200.
"""

from __future__ import annotations

from dataclasses import dataclass

TILE_ROWS = 128          # weight rows per CTA of the tensor-core kernel (MMA M)
BK = 64                  # K elements per pipeline stage
MAX_STAGES = 12
NTOK_CHOICES = (16, 32, 64, 128, 256)
SMEM_PER_SM = 228 * 1024     # B200: shared memory per SM
SMEM_PER_CTA_MAX = 227 * 1024
CTA_RESERVED = 1024 + 1024 + 512   # per-CTA driver reservation + 1 KB alignment slack + static shared memory


@dataclass(frozen=True)
class DeviceFacts:
    sms: int = 148
    smem_optin: int = SMEM_PER_CTA_MAX


@dataclass(frozen=True)
class GemvPlan:
    wpr: int      # warps sharing one weight row
    unroll: int   # 16-byte loads in flight per lane per batch


@dataclass(frozen=True)
class SkinnyPlan:
    ntok: int     # tokens per tile (MMA N)
    split: int    # K slices per weight-row tile
    stages: int   # shared-memory pipeline depth
    tiles: int    # weight-row tiles x token tiles
    ws_floats: int  # workspace floats needed when split > 1 (0 otherwise)

    @property
    def ctas(self) -> int:
        return self.tiles * self.split


# Measured on B200 (CUDA-graph replay, cold L2): (n, k, w_is_f32) -> (wpr, unroll).
TUNED_GEMV: dict[tuple[int, int, bool], tuple[int, int]] = {}
# (n, k, hilo, ntok) -> (split, stages).
TUNED_SKINNY: dict[tuple[int, int, bool, int], tuple[int, int]] = {}


def _pow2_floor(v: int) -> int:
    return 1 << (max(1, v).bit_length() - 1)


def gemv_valid(k: int, w_is_f32: bool, wpr: int) -> bool:
    epv = 4 if w_is_f32 else 8
    return k % 8 == 0 and k % wpr == 0 and (k // wpr) % epv == 0


def gemv_plan(n: int, k: int, w_is_f32: bool, dev: DeviceFacts = DeviceFacts()) -> GemvPlan:
    """Enough CTAs to give every SM several (8 / wpr rows each), the longest K segment that allows."""
    if k % 8 != 0:
        raise ValueError(f"K={k}: the kernels need K % 8 == 0 (16-byte aligned weight rows)")
    tuned = TUNED_GEMV.get((n, k, w_is_f32))
    if tuned and gemv_valid(k, w_is_f32, tuned[0]):
        return GemvPlan(*tuned)
    epv = 4 if w_is_f32 else 8
    valid = [w for w in (1, 2, 4, 8) if gemv_valid(k, w_is_f32, w)]
    if not valid:
        raise ValueError(f"K={k}: no warp split leaves whole 16-byte vectors per segment")
    want = 4 * dev.sms
    wpr = next((w for w in valid if -(-n // (8 // w)) >= want), valid[-1])
    vec_per_lane = max(1, (k // wpr // epv + 31) // 32)
    return GemvPlan(wpr=wpr, unroll=min(4, _pow2_floor(vec_per_lane)))


def pick_ntok(m: int) -> int:
    return next((t for t in NTOK_CHOICES if t >= m), NTOK_CHOICES[-1])


def stage_bytes(ntok: int, hilo: bool) -> int:
    return TILE_ROWS * BK * 2 * (2 if hilo else 1) + ntok * BK * 2


def skinny_plan(m: int, n: int, k: int, hilo: bool, dev: DeviceFacts = DeviceFacts(),
                ws_floats_cap: int = 1 << 62, cnt_cap: int = 1 << 30,
                split: int | None = None, stages: int | None = None) -> SkinnyPlan:
    """Units (row tile x K slice x token tile) sized to fill the SMs in one wave.

    Two CTAs share an SM when four stages of each fit in half its shared memory (more loads in
    flight while the other CTA is in its prologue or epilogue); otherwise one CTA takes the SM.
    `split` / `stages` override the derived values (tuning sweeps).
    """
    if k % 8 != 0:
        raise ValueError(f"K={k}: the kernels need K % 8 == 0 (16-byte aligned rows for TMA)")
    ntok = pick_ntok(m)
    sb = stage_bytes(ntok, hilo)
    tiles = -(-n // TILE_ROWS) * -(-m // ntok)
    chunks = -(-k // BK)
    half = SMEM_PER_SM // 2 - CTA_RESERVED
    per_sm = 2 if 4 * sb <= half else 1
    budget = min(dev.smem_optin, SMEM_PER_SM // per_sm) - CTA_RESERVED
    tuned = TUNED_SKINNY.get((n, k, hilo, ntok))
    if split is None:
        if tuned:
            split = tuned[0]
        else:
            split = max(1, (dev.sms * per_sm) // tiles)
    split = max(1, min(split, chunks))
    ws_floats = tiles * TILE_ROWS * ntok if split > 1 else 0
    if split > 1 and (ws_floats > ws_floats_cap or tiles > cnt_cap):
        split, ws_floats = 1, 0   # never allocate behind the caller's back: fall back to one slice
    if stages is None:
        stages = tuned[1] if tuned else budget // sb
    longest = -(-chunks // split)
    stages = max(1, min(stages, MAX_STAGES, longest, (SMEM_PER_CTA_MAX - 1024 - 512) // sb))
    return SkinnyPlan(ntok=ntok, split=split, stages=stages, tiles=tiles, ws_floats=ws_floats)
