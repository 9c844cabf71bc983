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
MAX_CLUSTER = 16         # 8 is the portable limit; 9..16 need the non-portable opt-in (set by the library)
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
    persistent: bool = False   # whole rows per warp on a grid that is resident all at once (wpr == 1)


@dataclass(frozen=True)
class FewTokPlan:
    """Up to 16 tokens streamed through register-level MMAs (muse_fewtok_mma)."""
    warps: int    # per CTA: 16 or 32
    unroll: int   # 16-byte loads in flight per lane per batch
    tok_split: int = 1   # interleaved copies of the walk, each with its own block of 8 or 16 tokens


@dataclass(frozen=True)
class SkinnyPlan:
    ntok: int       # tokens per tile (MMA N)
    cluster: int    # K slices reduced on chip (CTAs per thread-block cluster)
    groups: int     # clusters per tile; > 1 means their sums meet in the global workspace
    stages: int     # shared-memory pipeline depth
    tiles: int      # weight-row tiles x token tiles
    ws_floats: int  # workspace floats needed when groups > 1 (0 otherwise)

    @property
    def split(self) -> int:
        return self.cluster * self.groups

    @property
    def ctas(self) -> int:
        return self.tiles * self.split


@dataclass(frozen=True)
class GemmPlan:
    """Many tokens through muse_gemm_tc: one token tile as wide as the call, K split so that the CTAs fill the SMs."""
    ntok: int       # tokens per tile (MMA N): a multiple of 16 up to 256
    pair: bool      # two 128-row weight tiles per CTA sharing each x chunk
    cluster: int    # K slices as one thread-block cluster, reduced through distributed shared memory
    split: int      # K slices as independent CTAs, reduced through the global workspace (one of the two is 1)
    stages: int     # shared-memory pipeline depth
    warpgroups: int = 4   # CTA size / 128 threads; all of them work in the epilogue
    tile_rows: int = 128  # weight rows per CTA without `pair`: a multiple of 8; short tiles fill the SMs without a K split
    k_atoms: int = 1      # 64-wide pieces of K per pipeline stage

    @property
    def slices(self) -> int:
        return self.cluster * self.split


GEMM_MAX_STAGES = 12
GEMM_MAX_SPLIT = 64
GEMM_SUB = 16                 # owner blocks of the K-slice reduction are multiples of this many tokens
GEMM_MIN_SMEM = 116 * 1024    # one CTA per SM (mirrors the C side)
GEMM_MIN_TOKENS = 33          # below: the register-MMA walk and muse_skinny_tc
GEMM_WARPGROUPS = 4
GEMM_BUCKETS = (32, 48, 64, 128, 256)


def _gemm_owner_block(mpad: int, slices: int) -> int:
    return -(-(-(-mpad // slices)) // GEMM_SUB) * GEMM_SUB


def gemm_smem_bytes(ntok: int, pair: bool, stages: int, cluster: int, m: int, warpgroups: int = GEMM_WARPGROUPS,
                    tile_rows: int = TILE_ROWS, k_atoms: int = 1) -> int:
    """Dynamic shared memory of a muse_gemm_tc launch (mirrors muse_gemm_tc_smem_bytes); `cluster` = the slices
    that meet in distributed shared memory (slices that meet in the global workspace need no receive area)."""
    rows = TILE_ROWS * (2 if pair else 1)
    mpad = -(-min(m, ntok) // GEMM_SUB) * GEMM_SUB
    t = _gemm_owner_block(mpad, cluster) if cluster > 1 else mpad
    rx = (cluster - 1) * rows * t * 4 if cluster > 1 else 0
    after = rx + warpgroups * GEMM_SUB * rows * 4
    own = 2 * TILE_ROWS if pair else tile_rows
    ring = stages * k_atoms * (own * BK * 2 + ntok * BK * 2) + (0 if pair else (TILE_ROWS - tile_rows) * BK * 2)
    return max(max(ring, after) + 1024, GEMM_MIN_SMEM)


def gemm_ws_floats(m: int, n: int, ntok: int, pair: bool, split: int, tile_rows: int = TILE_ROWS) -> int:
    """Workspace floats of a launch whose `split` slices meet in global memory (mirrors muse_gemm_tc_ws_floats)."""
    if split <= 1:
        return 0
    rows = TILE_ROWS * (2 if pair else 1)
    units = -(-n // (rows if pair else tile_rows)) * -(-m // ntok)
    mpad = -(-min(m, ntok) // GEMM_SUB) * GEMM_SUB
    return units * split * (split - 1) * rows * _gemm_owner_block(mpad, split)


def gemm_ntok(m: int) -> int:
    """Equal token tiles, as few as 256 tokens each allow, rounded up to the MMA's multiple of 16."""
    tiles = -(-m // 256)
    return -(-(-(-m // tiles)) // 16) * 16


def gemm_plan(m: int, n: int, k: int, dev: DeviceFacts = DeviceFacts(), max_clusters=None, ws_floats_cap: int = 0,
              cnt_cap: int = 0, ntok: int | None = None, pair: bool | None = None, cluster: int | None = None,
              split: int | None = None, stages: int | None = None, tile_rows: int | None = None,
              k_atoms: int | None = None) -> GemmPlan | None:
    """(Row units x K slices x token tiles) CTAs filling the SMs in one wave, one CTA per SM.

    Shapes that were swept on a B200 take their measured best (TUNED_GEMM). Otherwise one weight tile per CTA
    (pairs pay only on the tallest weight) and: up to 128 tokens the slices form one cluster of about a hundred
    CTAs in all (`max_clusters(ntok, pair, stages, cluster, m, warpgroups)`, the device's occupancy query, caps
    it: clusters pack into GPCs, so fewer CTAs fit than there are SMs); above, they meet in the global
    workspace, one CTA per SM, where the workspace (`ws_floats_cap`, `cnt_cap`) allows it. Explicit ntok / pair /
    cluster / split / stages override (tuning sweeps). None: the shape cannot run here."""
    if k % 8 != 0 or m < 1:
        return None
    forced = (ntok is not None or pair is not None or cluster is not None or split is not None or tile_rows is not None
              or k_atoms is not None)
    if ntok is None:
        ntok = gemm_ntok(m)
    if ntok % 16 or not 16 <= ntok <= 256:
        raise ValueError(f"ntok={ntok}: a multiple of 16 up to 256")
    chunks = -(-k // BK)
    tok_tiles = -(-m // ntok)
    limit = dev.smem_optin - 512
    if not forced:
        # the first measured bucket that holds the token tile
        tuned = next((TUNED_GEMM[(n, k, b)] for b in GEMM_BUCKETS if b >= ntok and (n, k, b) in TUNED_GEMM), None) \
            if tok_tiles == 1 else None
        if tuned:
            pair, cluster, split = tuned[0], tuned[1], tuned[2]
            tile_rows, k_atoms = (tuned[4], tuned[5]) if len(tuned) > 4 else (TILE_ROWS, 1)
            if stages is None:
                stages = tuned[3]
            units = -(-n // (2 * TILE_ROWS if pair else tile_rows))
            if split > 1 and (units * split > dev.sms or gemm_ws_floats(m, n, ntok, pair, split, tile_rows) > ws_floats_cap
                              or 2 * units > cnt_cap):
                pair = cluster = split = tile_rows = k_atoms = None   # the workspace route is closed here: plan a cluster instead
            elif cluster > 1 and (units * cluster > dev.sms or (
                    max_clusters is not None and max_clusters(ntok, pair, stages, cluster, m, GEMM_WARPGROUPS) < units)):
                pair = cluster = split = tile_rows = k_atoms = None   # this device does not hold the measured launch in one wave
            elif units > dev.sms and tile_rows != TILE_ROWS:
                tile_rows = k_atoms = None   # short tiles are sized for one wave on the device they were measured on

    if tile_rows is None:
        tile_rows = TILE_ROWS
    if k_atoms is None:
        k_atoms = 1
    if tile_rows % 8 or not 8 <= tile_rows <= TILE_ROWS or not 1 <= k_atoms <= 8:
        raise ValueError(f"tile_rows={tile_rows} (a multiple of 8 up to 128), k_atoms={k_atoms} (1..8)")
    steps = -(-chunks // k_atoms)   # K slices are whole pipeline steps

    def deepest(pr: bool, cl: int) -> int:
        best = 0
        for st in range(1, GEMM_MAX_STAGES + 1):
            if gemm_smem_bytes(ntok, pr, st, cl, m, GEMM_WARPGROUPS, TILE_ROWS if pr else tile_rows, k_atoms) <= limit:
                best = st
        return best

    def cluster_for(pr: bool) -> int:
        """About a hundred CTAs (measured on the per-GPU shard shapes: beyond that the wider reduction costs more
        than the idle SMs), at least four chunks of K per slice, and no more clusters than the device holds."""
        units = -(-n // (TILE_ROWS * 2 if pr else tile_rows)) * tok_tiles
        cl = max(1, min(100 // max(units, 1), 12, steps // 4, dev.sms // max(units, 1)))
        while cl > 1 and (deepest(pr, cl) < 2 or (max_clusters is not None and
                                                  max_clusters(ntok, pr, min(deepest(pr, cl), 4), cl, m, GEMM_WARPGROUPS) < units)):
            cl -= 1
        return cl

    if pair is None:
        pair = cluster is not None or (split or 1) > 1   # a forced slice count alone means pairs (tuning sweeps)
    if split is None:
        split = 1
        if cluster is None and ntok > 128 and tok_tiles == 1:
            # Wide token tiles: the slices of a tile meet in the workspace (no GPC packing, so every SM can
            # take one), as long as the workspace holds them.
            units = -(-n // (TILE_ROWS * 2 if pair else tile_rows))
            want = min(dev.sms // units, steps // 6 if steps >= 48 else steps // 4)
            while want > 1 and (gemm_ws_floats(m, n, ntok, pair, want, tile_rows) > ws_floats_cap or 2 * units > cnt_cap):
                want -= 1
            split = max(1, want)
    if cluster is None:
        cluster = 1 if split > 1 else cluster_for(pair)
    if pair:
        tile_rows = TILE_ROWS
    cluster = max(1, min(cluster, MAX_CLUSTER, steps))
    split = max(1, min(split, GEMM_MAX_SPLIT, steps))
    if cluster > 1 and split > 1:
        raise ValueError("muse_gemm_tc reduces its K slices either in a cluster or through the workspace, not both")
    most = deepest(pair, cluster)
    if most < 1:
        return None
    longest = -(-steps // (cluster * split))
    stages = max(1, min(stages if stages is not None else 6, most, longest))
    return GemmPlan(ntok=ntok, pair=bool(pair), cluster=cluster, split=split, stages=stages, tile_rows=tile_rows, k_atoms=k_atoms)


# Measured on B200 (CUDA-graph replay, cold L2, in-stream): (n, k, token bucket) -> (pair, cluster, split, stages[,
# tile_rows, k_atoms]). The figure after the slash is what the shape took before this kernel (muse_skinny_tc, or the
# register-MMA walk).
TUNED_GEMM: dict[tuple[int, int, int], tuple] = {
    (12288, 4096, 32): (False, 1, 1, 3, 88, 4),   # qkv_gate 21.7 us / 22.4: 140 short tiles, no K split
    (12288, 4096, 48): (False, 1, 1, 4, 128, 2),  # 23.0
    (12288, 4096, 64): (False, 1, 1, 4, 128, 2),  # 23.0 / 26.5
    (12288, 4096, 128): (False, 1, 1, 3, 128, 2),  # 24.5 / 25.6 (pairs in clusters of two: 25.4)
    (12288, 4096, 256): (False, 1, 1, 4),   # 30.4 / 31.1
    (4096, 4096, 48): (False, 4, 1, 4, 128, 2),     # o 12.0
    (4096, 4096, 64): (False, 4, 1, 4, 128, 2),     # 12.0 / 15.5
    (4096, 4096, 128): (False, 4, 1, 6),    # 13.9 / 18.5
    (4096, 4096, 256): (False, 1, 4, 4),    # 16.5 / 23.9
    (1024, 4096, 128): (False, 8, 1, 3, 128, 2),    # pooler 10.0 / 11.4
    (1024, 4096, 256): (False, 1, 16, 4),   # 12.6 / 17.3
    (4096, 1024, 64): (False, 4, 1, 2, 128, 2),     # unpooler 7.8 / 9.1
    (4096, 1024, 128): (False, 2, 1, 3, 128, 2),    # 8.7 / 9.35
    (4096, 1024, 256): (False, 2, 1, 4),    # 11.0 / 10.6
}

# Measured on B200 (CUDA-graph replay, cold L2, in-stream): (n, k, w_is_f32) -> (wpr, unroll, persistent).
TUNED_GEMV: dict[tuple[int, int, bool], tuple[int, int, bool]] = {
    (12288, 4096, False): (1, 4, True),    # qkv_gate 18.3 us (19.8 non-persistent)
    (4096, 4096, False): (1, 4, True),     # o 8.0 us (8.8)
    (1024, 4096, False): (4, 4, False),    # pooler 3.7 us
    (4096, 1024, False): (1, 4, False),    # unpooler 3.5 us
    (256, 4096, True): (8, 4, False),      # router 2.8 us
}
# Same protocol: (n, k, token bucket) -> (warps, unroll[, tok_split]) where the register-MMA walk beats the
# alternative (the figure after the slash: the GEMV in bucket 1, else the TMEM kernel). warps * unroll
# >= K / 32 selects its variant that keeps x in registers; tok_split copies of that walk share W through
# L2, which pays for the small weights only.
FEWTOK_BUCKETS = (1, 8, 16, 32, 64)
TUNED_FEWTOK: dict[tuple[int, int, int], tuple[int, ...]] = {
    (12288, 4096, 1): (32, 4),    # qkv_gate 17.6 us / 18.1
    (12288, 4096, 8): (32, 4),    # 18.1-18.4 / 20.1-20.4
    (12288, 4096, 16): (16, 8),   # 19.8 / 21.4
    (4096, 4096, 8): (32, 4),     # o 8.1-8.2 / 9.8-10.0
    (4096, 4096, 16): (16, 8),    # 9.7 / 10.1
    (1024, 4096, 8): (32, 4),     # pooler 4.2-4.5 / 6.8-7.0
    (1024, 4096, 16): (32, 4),    # 4.5 / 7.1
    (1024, 4096, 32): (16, 8, 2),  # 6.1 / 7.5
    (1024, 4096, 64): (16, 8, 4),  # 7.8 / 8.6
    (4096, 1024, 8): (16, 2),     # unpooler 3.9 / 6.1-6.2
    (4096, 1024, 16): (16, 2),    # 4.2 / 6.4
    (4096, 1024, 32): (16, 2, 2),  # 5.4 / 7.0
}
# FP32 weights (the router), split to BF16 hi + lo in registers: (n, k, token bucket) -> (unroll, tok_split);
# 16 warps, up to 8 tokens per copy of the walk.
TUNED_FEWTOK_F32: dict[tuple[int, int, int], tuple[int, int]] = {
    (256, 4096, 8): (8, 1),     # router 5.4-5.9 us / 6.4-6.5
    (256, 4096, 16): (8, 2),    # 6.1 / 6.8
    (256, 4096, 32): (8, 4),    # 6.2 / 7.0
}
FEWTOK_X_PAD = 64
# Same protocol: (n, k, hilo, token bucket) -> (ntok, cluster, groups, stages). The bucket is the
# smallest of NTOK_CHOICES holding m; ntok may be smaller (several token tiles: small weights gain
# more from extra tiles than they lose re-reading W through L2).
TUNED_SKINNY: dict[tuple[int, int, bool, int], tuple[int, int, int, int]] = {
    (12288, 4096, False, 16): (16, 3, 1, 3),     # qkv_gate 20.1 us
    (12288, 4096, False, 32): (32, 2, 1, 4),     # 23.0
    (12288, 4096, False, 64): (64, 1, 1, 6),     # 26.5
    (12288, 4096, False, 128): (128, 1, 1, 6),   # 27.7
    (12288, 4096, False, 256): (256, 1, 1, 4),   # 32.4
    (4096, 4096, False, 16): (16, 8, 1, 3),      # o 9.9
    (4096, 4096, False, 32): (32, 8, 1, 4),      # 10.5
    (4096, 4096, False, 64): (64, 4, 1, 6),      # 15.5
    (4096, 4096, False, 128): (64, 2, 1, 4),     # 19.4
    (4096, 4096, False, 256): (128, 2, 1, 4),    # 24.7
    (1024, 4096, False, 16): (16, 16, 1, 4),     # pooler 6.9
    (1024, 4096, False, 32): (32, 16, 1, 3),     # 7.4
    (1024, 4096, False, 64): (64, 16, 1, 3),     # 9.0
    (1024, 4096, False, 128): (64, 6, 1, 4),     # 11.8
    (1024, 4096, False, 256): (128, 6, 1, 4),    # 17.2
    (4096, 1024, False, 16): (16, 6, 1, 4),      # unpooler 6.2
    (4096, 1024, False, 32): (32, 8, 1, 2),      # 7.3
    (4096, 1024, False, 64): (64, 1, 1, 4),      # 9.6
    (4096, 1024, False, 128): (64, 1, 1, 4),     # 9.7
    (4096, 1024, False, 256): (128, 1, 1, 4),    # 10.8
    (256, 4096, True, 16): (16, 16, 1, 3),       # router 6.6
    (256, 4096, True, 32): (32, 16, 1, 3),       # 7.0
    (256, 4096, True, 64): (64, 16, 1, 3),       # 8.1
    (256, 4096, True, 128): (64, 16, 1, 4),      # 8.0
    (256, 4096, True, 256): (64, 8, 1, 4),       # 10.6 (four token tiles; 16-wide clusters of 8 tiles do not fit in one wave)
}


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
    # Tall weights (several rows per resident warp slot) drain more evenly on the persistent grid.
    persistent = wpr == 1 and n >= 16 * dev.sms and k * 2 <= 64 * 1024
    return GemvPlan(wpr=wpr, unroll=min(4, _pow2_floor(vec_per_lane)), persistent=persistent)


def fewtok_smem_bytes(m: int, k: int, warps: int) -> int:
    """Shared memory of muse_fewtok_mma: m padded x rows + two reduction buffers (mirrors the C side)."""
    tok = 16 if m > 8 else 8
    return m * (k * 2 + FEWTOK_X_PAD) + 2 * warps * tok * 8 * 4


LL_TOKENS = 32   # most tokens of a column-parallel register-MMA call (MUSE_LL_TOKENS)


def fewtok_fused_plan(m: int, n: int, k: int, w_is_f32: bool) -> FewTokPlan | None:
    """Column-parallel calls (n = this rank's slice): the register-MMA kernel's exchange costs one NVLink
    flight where the other kernels' costs a fence and two, so it is taken whenever it applies: BF16,
    m <= LL_TOKENS, whole 8-row groups, x in registers (K <= 4096)."""
    kblocks = k // 32
    if w_is_f32 or not 1 <= m <= LL_TOKENS or k % 32 or n % 8 or n < 128 or kblocks > 128:
        return None
    if m > 8:   # 16 tokens per CTA; beyond that two interleaved walks that share W through L2
        return FewTokPlan(16, 1 if kblocks <= 16 else 2 if kblocks <= 32 else 4 if kblocks <= 64 else 8, 2 if m > 16 else 1)
    return FewTokPlan(*((16, 1) if kblocks <= 16 else (16, 2) if kblocks <= 32 else (16, 4) if kblocks <= 64 else (32, 4)))


def fewtok_plan(m: int, n: int, k: int, w_is_f32: bool, dev: DeviceFacts = DeviceFacts()) -> FewTokPlan | None:
    """The register-MMA plan of a shape that gains from it, else None (TMEM kernel). Tuned shapes come
    from the table; others take it at m <= 8 when the weight has enough 8-row groups to occupy most SMs."""
    if not 1 <= m <= FEWTOK_BUCKETS[-1] or k % 32:
        return None
    if w_is_f32:
        tuned = TUNED_FEWTOK_F32.get((n, k, next(b for b in FEWTOK_BUCKETS if b >= m))) if m > 1 else None
        return FewTokPlan(16, tuned[0], tuned[1]) if tuned else None
    tuned = TUNED_FEWTOK.get((n, k, next(b for b in FEWTOK_BUCKETS if b >= m)))
    if tuned is None:
        if m == 1 or m > 8 or (n + 7) // 8 < dev.sms * 3 // 4:
            return None
        kblocks = k // 32   # a whole row per batch (x stays in registers) whenever 32 warps x 4 loads reach
        tuned = (16, 1) if kblocks <= 16 else (16, 2) if kblocks <= 32 else (16, 4) if kblocks <= 64 else (32, 4)
    if tuned[0] * tuned[1] < k // 32 and fewtok_smem_bytes(m, k, tuned[0]) > dev.smem_optin:
        return None
    return FewTokPlan(*tuned)


def pick_ntok(m: int) -> int:
    return next((t for t in NTOK_CHOICES if t >= m), NTOK_CHOICES[-1])


def stage_bytes(ntok: int, hilo: bool) -> int:
    return TILE_ROWS * BK * 2 * (2 if hilo else 1) + ntok * BK * 2


def owner_block(mvalid: int, cluster: int) -> int:
    """Tokens per owner CTA when a tile's tokens are dealt to the CTAs of a cluster (whole fours)."""
    return (-(-mvalid // cluster) + 3) & ~3


def smem_bytes(ntok: int, hilo: bool, stages: int, cluster: int = 1, m: int | None = None) -> int:
    """Dynamic shared memory of a launch: the ring, the receive slots of a clustered launch, 1 KB slack."""
    mvalid = ntok if m is None else min(m, ntok)
    rx = cluster * TILE_ROWS * owner_block(mvalid, cluster) * 4 if cluster > 1 else 0
    ring = stages * stage_bytes(ntok, hilo)
    staged_tokens = owner_block(mvalid, cluster) if cluster > 1 else (mvalid + 3) & ~3
    staged = staged_tokens * TILE_ROWS * 4 if staged_tokens > 16 else 0   # vector-store staging overlays the ring
    return max(ring, staged) + rx + 1024


def skinny_plan(m: int, n: int, k: int, hilo: bool, dev: DeviceFacts = DeviceFacts(),
                ws_floats_cap: int = 1 << 62, cnt_cap: int = 1 << 30,
                ntok: int | None = None, cluster: int | None = None, groups: int | None = None,
                stages: int | None = None, max_clusters=None) -> SkinnyPlan:
    """Units (row tile x K slice x token tile) sized to fill the SMs in one wave.

    Shapes that were swept on a B200 take their measured best (TUNED_SKINNY). Otherwise: the K slices
    of a tile form one cluster of up to 8 CTAs (16 when there are few tiles) that reduces on chip,
    sized so that all CTAs are resident at once with two CTAs per SM; small weights at many tokens
    use half-size token tiles to get more units. `max_clusters(ntok, hilo, m, stages, cluster)`, when
    given (the device's occupancy query), shrinks the cluster until the launch fits in one wave.
    `ntok` / `cluster` / `groups` / `stages` override everything (tuning sweeps).
    """
    if k % 8 != 0:
        raise ValueError(f"K={k}: the kernels need K % 8 == 0 (16-byte aligned rows for TMA)")
    chunks = -(-k // BK)
    n_tiles = -(-n // TILE_ROWS)
    bucket = pick_ntok(m)
    forced = ntok is not None or cluster is not None or groups is not None
    tuned = None if forced else TUNED_SKINNY.get((n, k, hilo, bucket))
    if tuned:
        ntok, cluster, groups = tuned[0], tuned[1], tuned[2]
        if stages is None:
            stages = tuned[3]
    if ntok is None:
        ntok = bucket
        if m > 64 and n_tiles * -(-m // ntok) * 4 <= dev.sms:
            ntok = max(64, ntok // 2)
    if ntok not in NTOK_CHOICES:
        raise ValueError(f"ntok={ntok}: must be one of {NTOK_CHOICES}")
    sb = stage_bytes(ntok, hilo)
    tiles = n_tiles * -(-m // ntok)
    limit = SMEM_PER_CTA_MAX - 512

    def deepest(cap: int, cl: int) -> int:
        """Most stages whose launch fits in `cap` bytes of dynamic shared memory (0: not even one)."""
        best = 0
        for st in range(1, MAX_STAGES + 1):
            if smem_bytes(ntok, hilo, st, cl, m) <= cap:
                best = st
        return best

    if cluster is None:
        want = max(1, min((dev.sms * 2) // tiles, chunks))
        cluster = min(want, 16 if tiles <= 16 else 8)
    if groups is None:
        groups = 1
    cluster = max(1, min(cluster, MAX_CLUSTER, chunks))
    while cluster > 1 and deepest(limit, cluster) < 2:
        cluster -= 1   # the receive slots must leave room for at least a two-stage ring
    groups = max(1, min(groups, chunks // cluster))
    longest = -(-chunks // (cluster * groups))
    if stages is None:
        two_per_sm = SMEM_PER_SM // 2 - 1024 - 512
        want_two = tiles * cluster * groups > dev.sms
        shared = deepest(two_per_sm, cluster) if want_two else 0
        stages = min(6, shared if shared >= 3 else deepest(limit, cluster))
    stages = max(1, min(stages, longest, deepest(limit, cluster)))
    if max_clusters is not None and not forced and not tuned:
        while cluster > 1:
            per_sm = max(1, SMEM_PER_SM // (smem_bytes(ntok, hilo, stages, cluster, m) + 1024 + 512))
            fit = max_clusters(ntok, hilo, m, stages, cluster)
            if fit <= 0 or tiles * groups <= fit * per_sm:
                break
            cluster -= 1
            stages = max(1, min(stages, deepest(limit, cluster)))
    ws_floats = tiles * TILE_ROWS * ntok if groups > 1 else 0
    if groups > 1 and (ws_floats > ws_floats_cap or tiles > cnt_cap):
        groups, ws_floats = 1, 0   # never allocate behind the caller's back: one cluster per tile instead
    return SkinnyPlan(ntok=ntok, cluster=cluster, groups=groups, stages=stages, tiles=tiles, ws_floats=ws_floats)
