"""Host-side logic that needs no GPU: launch planning, the hi/lo split, shard bounds, and a CPU
model of the tensor-core kernel's tiling + split-K + hi/lo arithmetic checked against the oracle."""

from __future__ import annotations

import pytest
import torch

from llm_inference_engine_b200 import plan, tp
from llm_inference_engine_b200.muse_bf16_proj import split_hi_lo

SHAPES = {"qkv_gate": (12288, 4096, False), "o": (4096, 4096, False), "pooler": (1024, 4096, False),
          "unpooler": (4096, 1024, False), "router": (256, 4096, True),
          "ref_qkv": (2304, 8192, False), "ref_o": (8192, 1024, False), "ref_router": (256, 8192, True)}


@pytest.mark.parametrize("name", SHAPES)
def test_gemv_plan_is_launchable(name):
    n, k, f32 = SHAPES[name]
    p = plan.gemv_plan(n, k, f32)
    assert p.wpr in (1, 2, 4, 8) and p.unroll in (1, 2, 4, 8)
    assert plan.gemv_valid(k, f32, p.wpr)


def test_gemv_plan_rejects_unaligned_k():
    with pytest.raises(ValueError):
        plan.gemv_plan(128, 100, False)


@pytest.mark.parametrize("name", SHAPES)
@pytest.mark.parametrize("m", [2, 5, 16, 17, 32, 33, 64, 100, 128, 256, 257, 1000])
def test_skinny_plan_respects_every_kernel_limit(name, m):
    n, k, hilo = SHAPES[name]
    cap = 12288 * 256
    p = plan.skinny_plan(m, n, k, hilo, ws_floats_cap=cap, cnt_cap=4096)
    chunks = -(-k // plan.BK)
    assert p.ntok in plan.NTOK_CHOICES
    assert 1 <= p.split <= chunks and p.split == p.cluster * p.groups
    assert 1 <= p.cluster <= plan.MAX_CLUSTER
    assert 1 <= p.stages <= plan.MAX_STAGES
    assert plan.smem_bytes(p.ntok, hilo, p.stages, p.cluster, m) + 512 <= plan.SMEM_PER_CTA_MAX
    assert p.tiles == -(-n // 128) * -(-m // p.ntok)
    if p.groups > 1:
        assert p.ws_floats == p.tiles * 128 * p.ntok <= cap and p.tiles <= 4096
    else:
        assert p.ws_floats == 0
    # every K slice is non-empty under the kernel's balanced split
    bounds = [s * chunks // p.split for s in range(p.split + 1)]
    assert all(b > a for a, b in zip(bounds, bounds[1:]))


def test_skinny_plan_never_outgrows_the_workspace():
    p = plan.skinny_plan(32, 256, 4096, True, cluster=2, groups=8, ws_floats_cap=1000, cnt_cap=4096)
    assert p.groups == 1 and p.ws_floats == 0
    p = plan.skinny_plan(32, 256, 4096, True, cluster=2, groups=8, ws_floats_cap=1 << 40, cnt_cap=1)
    assert p.groups == 1
    p = plan.skinny_plan(32, 256, 4096, True, cluster=2, groups=8)
    assert p.groups == 8 and p.ws_floats == p.tiles * 128 * 32


def test_plan_overrides_are_clamped():
    p = plan.skinny_plan(8, 1024, 4096, False, cluster=1000, groups=1000, stages=99)
    assert p.cluster == 16 and p.groups == 4 and p.stages == 1
    p = plan.skinny_plan(200, 1024, 4096, False, ntok=64, cluster=2)
    assert p.ntok == 64 and p.tiles == 8 * 4 and p.cluster == 2 and p.groups == 1


def test_tuned_entries_are_launchable():
    for (n, k, hilo, bucket), (ntok, cluster, groups, stages) in plan.TUNED_SKINNY.items():
        assert bucket in plan.NTOK_CHOICES and ntok in plan.NTOK_CHOICES and ntok <= bucket
        assert cluster * groups <= -(-k // plan.BK) and 1 <= cluster <= plan.MAX_CLUSTER
        assert plan.smem_bytes(ntok, hilo, stages, cluster, bucket) + 512 <= plan.SMEM_PER_CTA_MAX
        p = plan.skinny_plan(bucket, n, k, hilo)
        longest = -(-(-(-k // plan.BK)) // (cluster * groups))   # no more stages than chunks in a K slice
        assert (p.ntok, p.cluster, p.groups, p.stages) == (ntok, cluster, groups, min(stages, longest))
    for (n, k, f32), (wpr, unroll, persistent) in plan.TUNED_GEMV.items():
        assert plan.gemv_valid(k, f32, wpr) and unroll in (1, 2, 4, 8) and (wpr == 1 or not persistent)
    for (n, k, bucket), tuned in plan.TUNED_FEWTOK.items():
        warps, unroll, tok_split = (*tuned, 1)[:3]
        assert bucket in plan.FEWTOK_BUCKETS and warps in (16, 32) and unroll in (1, 2, 4, 8) and k % 32 == 0
        assert unroll < 8 or (warps == 16 and k // 32 <= 128)   # 8 loads per lane exist only with x in registers
        assert bucket <= 16 * tok_split
        if tok_split > 1 or bucket > 8:   # these need x in registers: a whole row per batch
            assert warps * unroll >= k // 32 or bucket <= 16
        assert plan.fewtok_plan(bucket, n, k, False) == plan.FewTokPlan(warps, unroll, tok_split)


@pytest.mark.parametrize("name", [k for k, v in SHAPES.items() if not v[2]])
@pytest.mark.parametrize("m", [33, 48, 64, 100, 128, 256, 257, 300, 1000])
def test_gemm_plan_respects_every_kernel_limit(name, m):
    n, k, _ = SHAPES[name]
    dev = plan.DeviceFacts()
    p = plan.gemm_plan(m, n, k, dev, ws_floats_cap=3 * 12288 * 256, cnt_cap=4096)
    chunks = -(-k // plan.BK)
    assert p.ntok % 16 == 0 and 16 <= p.ntok <= 256 and -(-m // p.ntok) == -(-m // 256)   # as few token tiles as possible
    chunks = -(-chunks // p.k_atoms)   # K slices are whole pipeline steps
    assert (p.cluster == 1 or p.split == 1) and 1 <= p.cluster <= plan.MAX_CLUSTER and 1 <= p.slices <= chunks
    assert 1 <= p.stages <= plan.GEMM_MAX_STAGES and 1 <= p.warpgroups <= 4
    assert plan.gemm_smem_bytes(p.ntok, p.pair, p.stages, p.cluster, m, p.warpgroups, p.tile_rows, p.k_atoms) + 512 <= plan.SMEM_PER_CTA_MAX
    units = -(-n // (256 if p.pair else p.tile_rows)) * -(-m // p.ntok)
    if p.slices > 1:   # one wave, one CTA per SM: K slices wait for one another
        assert units * p.slices <= dev.sms
    if p.split > 1:
        assert plan.gemm_ws_floats(m, n, p.ntok, p.pair, p.split, p.tile_rows) <= 3 * 12288 * 256 and 2 * units <= 4096
    bounds = [s * chunks // p.slices for s in range(p.slices + 1)]
    assert all(b > a for a, b in zip(bounds, bounds[1:]))


def test_gemm_plan_falls_back_to_a_cluster_without_workspace_room():
    tuned = plan.gemm_plan(256, 4096, 4096, ws_floats_cap=1 << 30, cnt_cap=4096)
    assert tuned.split == 4 and tuned.cluster == 1
    small = plan.gemm_plan(256, 4096, 4096, ws_floats_cap=1000, cnt_cap=4096)
    assert small.split == 1 and small.cluster >= 1
    fewer = plan.gemm_plan(256, 4096, 4096, plan.DeviceFacts(sms=100), ws_floats_cap=1 << 30, cnt_cap=4096)
    assert fewer.split == 3 and 32 * fewer.split <= 100     # the measured split does not fit 100 SMs: the rule's own choice
    untuned = plan.gemm_plan(256, 2048, 4096, ws_floats_cap=1 << 30, cnt_cap=4096)
    assert untuned.split == 9 and not untuned.pair and plan.gemm_plan(128, 2048, 4096).cluster == 6
    capped = plan.gemm_plan(128, 4096, 4096, max_clusters=lambda *a: 0)     # a device that holds no cluster of this shape
    assert capped.cluster == 1 and capped.split == 1
    with pytest.raises(ValueError):
        plan.gemm_plan(128, 4096, 4096, cluster=2, split=2)


def test_gemm_tuned_entries_are_launchable():
    for (n, k, bucket), tuned in plan.TUNED_GEMM.items():
        pair, cluster, split, stages = tuned[:4]
        tile_rows, k_atoms = tuned[4:] if len(tuned) > 4 else (128, 1)
        assert bucket in plan.GEMM_BUCKETS and (cluster == 1 or split == 1) and tile_rows % 8 == 0 and (not pair or tile_rows == 128)
        p = plan.gemm_plan(bucket, n, k, ws_floats_cap=3 * 12288 * 256, cnt_cap=4096)
        steps = -(-(-(-k // plan.BK)) // k_atoms)
        longest = -(-steps // (cluster * split))
        assert (p.pair, p.cluster, p.split, p.stages, p.tile_rows, p.k_atoms) == (pair, cluster, split, min(stages, longest), tile_rows, k_atoms)
        assert -(-n // (256 if pair else tile_rows)) * cluster * split <= 148
        assert plan.gemm_smem_bytes(p.ntok, pair, p.stages, cluster, bucket, p.warpgroups, tile_rows, k_atoms) + 512 <= plan.SMEM_PER_CTA_MAX


def test_fewtok_f32_table_is_consistent():
    for (n, k, bucket), (unroll, tok_split) in plan.TUNED_FEWTOK_F32.items():
        assert bucket in plan.FEWTOK_BUCKETS and unroll in (2, 4, 8) and k % 32 == 0 and k // 32 <= 16 * unroll
        assert bucket <= 8 * tok_split <= 32
        assert plan.fewtok_plan(bucket, n, k, True) == plan.FewTokPlan(16, unroll, tok_split)
    assert plan.fewtok_plan(1, 256, 4096, True) is None    # one token: the GEMV
    assert plan.fewtok_plan(64, 256, 4096, True) is None


def test_fewtok_fused_plan_covers_what_the_exchange_supports():
    assert plan.fewtok_fused_plan(1, 1536, 4096, False) == plan.FewTokPlan(32, 4)
    assert plan.fewtok_fused_plan(8, 6144, 4096, False) == plan.FewTokPlan(32, 4)
    assert plan.fewtok_fused_plan(16, 1536, 4096, False) == plan.FewTokPlan(16, 8)
    assert plan.fewtok_fused_plan(12, 512, 1024, False) == plan.FewTokPlan(16, 2)
    assert plan.fewtok_fused_plan(32, 1536, 4096, False) == plan.FewTokPlan(16, 8, 2)
    assert plan.fewtok_fused_plan(33, 1536, 4096, False) is None      # staging holds 32 tokens
    assert plan.fewtok_fused_plan(4, 1532, 4096, False) is None       # ragged last group
    assert plan.fewtok_fused_plan(4, 32, 4096, True) is None          # FP32 router
    assert plan.fewtok_fused_plan(4, 1536, 8192, False) is None       # x would not stay in registers
    assert plan.LL_TOKENS == 32


def test_fewtok_plan_only_where_it_applies():
    assert plan.fewtok_plan(1, 4096, 4096, False) is None            # one token, untuned: the GEMV
    assert plan.fewtok_plan(8, 512, 4096, True) is None              # FP32 weights, untuned shape
    assert plan.fewtok_plan(17, 4096, 4096, False) is None           # more than one MMA of tokens, untuned
    assert plan.fewtok_plan(65, 1024, 4096, False) is None
    assert plan.fewtok_plan(4, 12288, 4100, False) is None           # K not in whole 32-element pieces
    assert plan.fewtok_plan(16, 8192, 4096, False) is None           # untuned above 8 tokens: TMEM kernel
    assert plan.fewtok_plan(4, 512, 4096, False) is None             # too few row groups to occupy the SMs
    assert plan.fewtok_plan(4, 8192, 2048, False) == plan.FewTokPlan(16, 4)
    assert plan.fewtok_plan(4, 8192, 512, False) == plan.FewTokPlan(16, 1)
    assert plan.fewtok_plan(4, 8192, 8192, False) == plan.FewTokPlan(32, 4)    # two batches per row: x in shared memory
    assert plan.fewtok_plan(8, 8192, 32768, False) is None           # 8 rows of x exceed shared memory
    assert plan.fewtok_smem_bytes(8, 4096, 16) == 8 * (8192 + 64) + 2 * 16 * 64 * 4
    assert plan.fewtok_smem_bytes(3, 4096, 32) == 3 * (8192 + 64) + 2 * 32 * 64 * 4


def test_hi_lo_split_recovers_fp32_weights_to_16_bits():
    g = torch.Generator().manual_seed(0)
    w = torch.randn((256, 512), generator=g) * 0.02
    hi, lo = split_hi_lo(w)
    assert hi.dtype == lo.dtype == torch.bfloat16
    assert torch.equal(hi, w.to(torch.bfloat16))
    assert torch.equal(lo, (w - hi.float()).to(torch.bfloat16))
    rel = ((hi.double() + lo.double()) - w.double()).abs() / w.double().abs().clamp(min=1e-30)
    assert float(rel.max()) < 2.0 ** -16


def _tile_model(x, mats, ntok, split):
    """What the tensor-core kernel computes, in torch on the CPU: 128-row tiles, 64-wide K chunks
    split into balanced slices, FP32 accumulation per slice (all matrices into one accumulator),
    FP32 sum of the slices."""
    m, k = x.shape
    n = mats[0].shape[0]
    chunks = -(-k // 64)
    out = torch.zeros((m, n), dtype=torch.float32)
    for t0 in range(0, m, ntok):
        xs = x[t0:t0 + ntok].float()
        for r0 in range(0, n, 128):
            acc = torch.zeros((xs.shape[0], min(128, n - r0)), dtype=torch.float32)
            for s in range(split):
                c0, c1 = s * chunks // split, (s + 1) * chunks // split
                part = torch.zeros_like(acc)
                for mat in mats:
                    part += xs[:, c0 * 64:c1 * 64] @ mat[r0:r0 + 128, c0 * 64:c1 * 64].float().T
                acc += part
            out[t0:t0 + ntok, r0:r0 + 128] = acc
    return out


@pytest.mark.parametrize("m,layer,split", [(5, "o", 3), (16, "qkv_gate", 7), (33, "unpooler", 2), (8, "router", 16),
                                           (32, "router", 33)])
def test_tiling_and_split_k_model_meets_the_reference_check(oracle, m, layer, split):
    small = {"qkv_gate": (384, 1024), "o": (256, 512), "unpooler": (200, 768), "router": (256, 1024)}
    w = oracle.generate_weights(7, layers=small)
    data = oracle.generate_input(m, layer, 100 + m, layers=small)
    data["config"]["n"] = small[layer][0]
    ntok = plan.pick_ntok(m)
    if layer == "router":
        got = _tile_model(data["x"], split_hi_lo(w[layer]), ntok, split)
    else:
        got = _tile_model(data["x"], (w[layer],), ntok, split).to(torch.bfloat16)
    ok, msg = oracle.check_implementation(data, got, w)
    assert ok, msg


def test_shard_bounds_partition_the_rows():
    for n, world in ((12288, 8), (4096, 4), (256, 2), (1024, 1)):
        spans = [tp.shard_bounds(n, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert len({b - a for a, b in spans}) == 1
    with pytest.raises(ValueError):
        tp.shard_bounds(1000, 3, 0)
    with pytest.raises(ValueError):
        tp.shard_bounds(1024, 4, 4)


def test_oracle_model_of_the_fp32_input_router_mode():
    """The three-term split (x_hi W_hi + x_hi W_lo + x_lo W_hi) sits within the router's 1e-5 of the
    FP64 product of the unsplit FP32 inputs, three orders of magnitude closer than rounding x to BF16."""
    from oracle import muse_proj_oracle as oracle

    g = torch.Generator().manual_seed(1)
    x = torch.randn((8, 4096), generator=g)
    w = torch.randn((256, 4096), generator=g) * 0.02
    ref = oracle.router_f32_input_reference(x, w)
    rel = lambda a: float((a.double() - ref).norm() / ref.norm())
    assert rel(oracle.router_f32_input_model(x, w)) < 1e-5
    assert rel(x.to(torch.bfloat16).double() @ w.double().T) > 1e-3
