"""GPU parity: the CUDA path (through prepare()/kernel_fn() and the C ABI) against the CPU oracle on
the same seeded inputs. Mirrors the reference's own check (bf16_proj/reference.py:84-99: rel-L2 <=
1e-2 BF16 / 1e-4 router, every row <= 5x that, probe rows <= 1e-3) on the reference's shapes, and the
benchmark's acceptance rule (BF16: rtol 1e-2 / atol 1e-2 against an FP32-accumulated product;
router: 1e-5 relative L2) on the 4096-hidden shapes it is quoted on.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def proj():
    from llm_inference_engine_b200 import muse_bf16_proj

    return muse_bf16_proj


@pytest.fixture(scope="module")
def ref_setup(oracle, proj, dev):
    """Reference geometry: weights generated on the CPU (the oracle's stream), copied to the GPU."""
    w_cpu = oracle.generate_weights(oracle.WEIGHTS_SEED, device="cpu")
    state = proj.prepare({k: v.to(dev) for k, v in w_cpu.items()})
    return w_cpu, state


@pytest.fixture(scope="module")
def target_setup(oracle, proj, dev):
    w_cpu = oracle.target_weights(device="cpu")
    state = proj.prepare({k: v.to(dev) for k, v in w_cpu.items()})
    return w_cpu, state


def _run(proj, state, data, dev):
    gpu_data = {"x": data["x"].to(dev), "config": data["config"]}
    out = proj.kernel_fn(gpu_data, state)
    proj.check_status(state)
    return out.cpu()


REF_TOKENS = (1, 2, 3, 5, 7, 8, 9, 13, 16, 27, 32, 33, 64, 100, 128, 256)


@pytest.mark.parametrize("layer", ["qkv_gate", "o", "pooler", "unpooler", "router"])
@pytest.mark.parametrize("dist", ["normal", "outliers"])
def test_reference_shapes_pass_reference_check(oracle, proj, dev, ref_setup, layer, dist):
    w_cpu, state = ref_setup
    for i, m in enumerate(REF_TOKENS):
        data = oracle.generate_input(m, layer, 9000 + 31 * i + (7 if dist == "outliers" else 0), dist, device="cpu")
        out = _run(proj, state, data, dev)
        ok, msg = oracle.check_implementation(data, out, w_cpu)
        assert ok, f"{layer} m={m} {dist}: {msg}"


@pytest.mark.parametrize("layer", ["qkv_gate", "o", "pooler", "unpooler", "router"])
def test_target_shapes_meet_benchmark_tolerance(oracle, proj, dev, target_setup, layer):
    w_cpu, state = target_setup
    tokens = sorted(set(oracle.TARGET_TOKENS[layer]) | {1, 8, 32, 128, 256})
    for m in tokens:
        data = oracle.target_input(m, layer, 1000 + m, device="cpu")
        out = _run(proj, state, data, dev)
        ok, msg = oracle.target_check(data, out, w_cpu)
        assert ok, f"{layer} m={m}: {msg}"
        # and the reference's own relative-L2 rule on the same output
        want = oracle.ref_kernel(data, w_cpu)
        tol = oracle.ROUTER_REL_L2_TOL if layer in oracle.FP32_LAYERS else oracle.BF16_REL_L2_TOL
        ok, msg = oracle.compare(out, want, tol)
        assert ok, f"{layer} m={m}: {msg}"


def test_large_and_ragged_token_counts(oracle, proj, dev, target_setup):
    """m beyond one token tile (the reference warms up to m = 1000, muse_bf16_proj.py:360)."""
    w_cpu, state = target_setup
    for layer, m in (("pooler", 257), ("unpooler", 513), ("router", 1000), ("o", 300)):
        data = oracle.target_input(m, layer, 77 + m, device="cpu")
        out = _run(proj, state, data, dev)
        ok, msg = oracle.target_check(data, out, w_cpu)
        assert ok, f"{layer} m={m}: {msg}"


def test_row_slices_of_a_weight(oracle, proj, dev, target_setup):
    """n < W rows, including n that is not a multiple of the 128-row tile (slice rule reference.py:37-41)."""
    w_cpu, state = target_setup
    for layer, m, n in (("unpooler", 8, 1024), ("unpooler", 1, 1000), ("qkv_gate", 4, 200), ("router", 16, 64),
                        ("pooler", 32, 130)):
        data = oracle.target_input(m, layer, 5 + m, device="cpu")
        data["config"]["n"] = n
        out = _run(proj, state, data, dev)
        assert out.shape == (m, n)
        ok, msg = oracle.target_check(data, out, w_cpu)
        assert ok, f"{layer} m={m} n={n}: {msg}"


def test_strided_and_misaligned_x(oracle, proj, dev, target_setup):
    """x that is not unit-stride / 16-byte aligned must still work (muse_bf16_proj.py:373-374)."""
    w_cpu, state = target_setup
    data = oracle.target_input(8, "pooler", 321, device="cpu")
    k = data["config"]["k"]
    want = _run(proj, state, data, dev)
    xg = data["x"].to(dev)
    wide = torch.zeros((8, k + 8), device=dev, dtype=torch.bfloat16)
    wide[:, 3:k + 3] = xg                      # misaligned start, padded rows
    transposed = xg.t().contiguous().t()       # column-major view
    padded = torch.zeros((8, k + 64), device=dev, dtype=torch.bfloat16)
    padded[:, :k] = xg                         # aligned, row stride != K: used in place through the tensor map
    for view in (wide[:, 3:k + 3], transposed, padded[:, :k]):
        out = proj.kernel_fn({"x": view, "config": data["config"]}, state).cpu()
        # split-K sums arrive in a different order each launch: equal up to one BF16 rounding step
        assert torch.allclose(out.float(), want.float(), rtol=1e-2, atol=1e-3)


def test_gemv_is_bit_identical_across_row_slices(oracle, proj, dev, target_setup):
    """A row's dot product does not depend on which other rows are computed: sharding by output rows
    reproduces the single-GPU GEMV bit for bit."""
    w_cpu, state = target_setup
    data = oracle.target_input(1, "o", 99, device="cpu")
    half = dict(data, config=dict(data["config"], n=2048))
    for pinned in (dict(wpr=1, unroll=4, persistent=True), dict(wpr=2, unroll=2, persistent=False)):
        state["_override"][("o", 1)] = pinned   # same K split and batch order on both sides
        try:
            full = _run(proj, state, data, dev)
            assert torch.equal(_run(proj, state, half, dev), full[:, :2048])
        finally:
            del state["_override"][("o", 1)]


def test_linearity_at_full_size(oracle, proj, dev, target_setup):
    """Size-independent property at the benchmark's largest shape: f(x1) + f(x2) == f(x1 + x2) up to
    BF16 rounding of inputs/outputs (x1, x2 chosen so that x1 + x2 is exact in BF16)."""
    _, state = target_setup
    g = torch.Generator(device="cpu").manual_seed(4)
    x1 = torch.randint(-4, 5, (32, 4096), generator=g).to(torch.bfloat16)
    x2 = torch.randint(-4, 5, (32, 4096), generator=g).to(torch.bfloat16)
    cfg = {"m": 32, "n": 12288, "k": 4096, "layer": "qkv_gate"}
    outs = [proj.kernel_fn({"x": x.to(dev), "config": cfg}, state).float().cpu() for x in (x1, x2, x1 + x2)]
    proj.check_status(state)
    err = (outs[0] + outs[1] - outs[2]).norm() / outs[2].norm()
    assert float(err) < 8e-3


# (layer, m, forced plan or None for the planner's own choice). The forced plans cover what the planner
# rarely picks on its own: sums meeting in the global workspace (groups > 1), with and without clusters.
REPLAY_CASES = [
    ("qkv_gate", 32, None), ("pooler", 8, None), ("router", 32, None), ("router", 256, None), ("unpooler", 128, None),
    ("qkv_gate", 4, None), ("unpooler", 16, None), ("o", 7, dict(warps=32, unroll=2)),
    ("qkv_gate", 32, dict(cluster=1, groups=3, stages=4)),
    ("pooler", 8, dict(cluster=2, groups=9, stages=3)),
    ("pooler", 100, dict(ntok=128, cluster=4, groups=2, stages=3)),
    ("router", 32, dict(cluster=1, groups=37, stages=2)),
    ("router", 16, dict(cluster=8, groups=8, stages=1)),
    ("o", 5, dict(cluster=16, groups=1, stages=3)),
    # muse_gemm_tc: the planner's choices (cluster of four; four slices through the workspace; sixteen of them)
    # and forced ones (pairs of tiles with a cluster of two / three slices through the workspace; a ragged token tile)
    ("o", 128, None), ("o", 256, None), ("pooler", 256, None), ("qkv_gate", 64, None),
    ("qkv_gate", 256, dict(pair=True, cluster=2, stages=3)),
    ("qkv_gate", 100, dict(pair=True, split=3, stages=4)),
    ("unpooler", 200, dict(pair=False, split=4, stages=2)),
]
REPLAYS = 300
REPLAYS_WORKSPACE = 1500   # plans whose K slices meet in global memory: the depth of bf16_proj/stress.py:125


@pytest.mark.parametrize("layer,m,forced", REPLAY_CASES, ids=lambda v: str(v).replace(" ", ""))
def test_graph_replays_are_stable_and_leave_workspace_clean(oracle, proj, dev, target_setup, layer, m, forced):
    """The split-K hand-off under replay (the reference's stress pattern, bf16_proj/stress.py:122-169):
    many cold-L2 replays, no bad output, workspace and counters back to zero afterwards; plans without
    the global workspace (groups == 1) must also reproduce their output bit for bit."""
    from llm_inference_engine_b200.graph_timer import ColdReplayTimer

    w_cpu, state = target_setup
    timer = ColdReplayTimer(dev, flush_bytes=256 << 20)
    data = oracle.target_input(m, layer, 4242 + m, device="cpu")
    x = data["x"].to(dev)
    ref = (data["x"].double() @ w_cpu[layer].double().T).to(dev)
    rn = ref.norm(dim=1).clamp(min=1e-6)
    holder = {}
    if forced:
        state["_override"][(layer, m)] = forced
    try:
        plan = proj.plan_for(state, layer, m, *w_cpu[layer].shape)
        with torch.cuda.stream(timer.stream):
            graph = timer.capture(lambda: holder.__setitem__("out", proj.kernel_fn({"x": x, "config": data["config"]}, state)))
            bad = torch.zeros((), device=dev, dtype=torch.int32)
            changed = torch.zeros((), device=dev, dtype=torch.int32)
            limit = 2e-5 if layer == "router" else 5e-3
            first = None
            from llm_inference_engine_b200.plan import GemmPlan
            uses_ws = getattr(plan, "groups", 1) > 1 or (isinstance(plan, GemmPlan) and plan.split > 1)
            replays = REPLAYS_WORKSPACE if uses_ws else REPLAYS
            for i in range(replays):
                if i % 2 == 0:
                    timer.flush.fill_(i & 0xFF)
                graph.replay()
                err = ((holder["out"].double() - ref).norm(dim=1) / rn).max()
                bad += (err > limit).int()
                if first is None:
                    first = holder["out"].clone()
                else:
                    changed += (holder["out"] != first).any().int()
            timer.stream.synchronize()
            assert int(bad) == 0, f"{layer} m={m} {plan}: {int(bad)}/{replays} bad replays"
            groups = getattr(plan, "groups", 1)   # the register-MMA plans have no global workspace either
            if groups == 1:   # (muse_gemm_tc sums its slices in a fixed order whichever way they meet)
                assert int(changed) == 0, f"{layer} m={m} {plan}: output changed between replays"
            if uses_ws:   # only these plans touch (and therefore create) the stream's workspace
                ws, cnt = state["_ws_by_stream"][timer.stream.cuda_stream]
                assert int(cnt.abs().max()) == 0
                if groups > 1:   # muse_skinny_tc accumulates into it and must leave zeros; muse_gemm_tc only overwrites
                    assert float(ws.abs().max()) == 0.0
    finally:
        state["_override"].pop((layer, m), None)
    proj.check_status(state)


def test_rejects_what_it_cannot_run(proj, dev, target_setup):
    _, state = target_setup
    cfg = {"m": 1, "n": 1024, "k": 4096, "layer": "pooler"}
    with pytest.raises(RuntimeError):
        proj.kernel_fn({"x": torch.zeros((1, 4096), dtype=torch.bfloat16), "config": cfg}, state)  # CPU tensor
    with pytest.raises(ValueError):
        proj.kernel_fn({"x": torch.zeros((1, 4000), dtype=torch.bfloat16, device=dev), "config": cfg}, state)
    with pytest.raises(TypeError):
        proj.kernel_fn({"x": torch.zeros((1, 4096), dtype=torch.float16, device=dev), "config": cfg}, state)
    with pytest.raises(ValueError):
        proj.kernel_fn({"x": torch.zeros((1, 4096), dtype=torch.bfloat16, device=dev), "config": dict(cfg, n=2048)}, state)


GEMM_CASES = [  # (m, n, k, ntok, pair, cluster, split, stages, warpgroups[, tile_rows[, k_atoms]])
    (16, 128, 64, 16, False, 1, 1, 1, 1), (16, 256, 128, 16, True, 1, 1, 2, 4), (64, 512, 1024, 64, True, 4, 1, 2, 4),
    (100, 1000, 2048, 112, True, 3, 1, 3, 2), (256, 1024, 4096, 256, False, 4, 1, 4, 4), (128, 12288, 4096, 128, True, 2, 1, 4, 4),
    (256, 12288, 4096, 256, False, 1, 1, 4, 4), (128, 4096, 4096, 128, False, 4, 1, 6, 4), (300, 4096, 1024, 160, True, 4, 1, 3, 4),
    (33, 1030, 4096, 48, False, 8, 1, 4, 3), (1000, 777, 512, 256, True, 2, 1, 2, 4),
    (64, 512, 1024, 64, True, 1, 4, 2, 4), (100, 1000, 2048, 112, True, 1, 3, 3, 1), (256, 12288, 4096, 256, True, 1, 3, 3, 4),
    (256, 4096, 4096, 256, False, 1, 4, 4, 4), (256, 1024, 4096, 256, False, 1, 16, 4, 4), (40, 700, 4096, 48, False, 1, 20, 3, 2),
    # short tiles: every SM takes a slab of rows, no K split
    (32, 12288, 4096, 32, False, 1, 1, 12, 4, 88), (16, 4096, 4096, 16, False, 1, 1, 10, 2, 32), (5, 1001, 1024, 16, False, 1, 1, 6, 4, 8),
    (64, 4096, 4096, 64, False, 2, 1, 8, 4, 56), (48, 2304, 8192, 48, False, 1, 2, 6, 4, 40),
    # several 64-wide K atoms per stage (K = 2080 is 32.5 atoms: the last step is partly past the end of K)
    (32, 12288, 4096, 32, False, 1, 1, 3, 4, 88, 4), (128, 4096, 4096, 128, False, 4, 1, 3, 4, 128, 2), (100, 1000, 2080, 112, True, 3, 1, 2, 2, 128, 2),
    (16, 4096, 4096, 16, False, 1, 1, 2, 1, 32, 8), (256, 2048, 4096, 256, False, 1, 3, 2, 4, 128, 2),
]


@pytest.mark.parametrize("case", GEMM_CASES, ids=lambda c: "m{}_n{}_k{}_t{}_p{}_c{}_s{}".format(c[0], c[1], c[2], c[3], int(c[4]), c[5], c[6]))
def test_gemm_entry_point_matches_oracle_and_is_bit_stable(dev, case):
    """muse_gemm_tc (the m > 32 GEMM: pairs of weight tiles, K slices meeting in a cluster or in the workspace)
    through the C ABI: FP64 product within the BF16 tolerance, ragged N and m, strided x and out, columns
    beyond n untouched, identical bits on repeated calls, counters back to zero, and no dependence on what the
    workspace held before (it is filled with NaN)."""
    from llm_inference_engine_b200 import _capi
    from llm_inference_engine_b200._capi import TensorMap

    m, n, k, ntok, pair, cluster, split, stages, wgs = case[:9]
    tile_rows = case[9] if len(case) > 9 else 128
    k_atoms = case[10] if len(case) > 10 else 1
    lib = _capi.load()
    g = torch.Generator(device=dev).manual_seed(m * 13 + n)
    w = (torch.randn((n, k), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn((m, k + 24), generator=g, device=dev).to(torch.bfloat16)[:, :k]
    ref = x.double() @ w.double().T
    tm = TensorMap.for_matrix(w.data_ptr(), n, k, k * 2, tile_rows)
    ws = torch.full((max(1, lib.muse_gemm_tc_ws_floats(m, n, ntok, int(pair), split, tile_rows)),), float("nan"), device=dev)
    cnt = torch.zeros(max(1, lib.muse_gemm_tc_cnt_ints(m, n, ntok, int(pair), split, tile_rows)), device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    if cluster > 1 and lib.muse_gemm_tc_max_clusters(ntok, int(pair), stages, cluster, m, wgs, tile_rows, k_atoms) < 1:
        pytest.skip("this cluster shape does not fit the device")
    outs = []
    for _ in range(3):
        out = torch.full((m, n + 8), 3.0, device=dev, dtype=torch.bfloat16)
        _capi.check(lib.muse_gemm_tc(tm.ptr, x.data_ptr(), out.data_ptr(), ws.data_ptr(), cnt.data_ptr(), status.data_ptr(), m, n, k,
                                     x.stride(0), out.stride(0), ntok, int(pair), cluster, split, stages, wgs, tile_rows, k_atoms, None,
                                     torch.cuda.current_stream(dev).cuda_stream), "muse_gemm_tc")
        torch.cuda.synchronize(dev)
        outs.append(out)
    assert int(status.item()) == 0 and int(cnt.abs().max()) == 0
    assert bool((outs[0][:, n:] == 3.0).all())
    err = float((outs[0][:, :n].double() - ref).norm() / ref.norm())
    assert err < 5e-3, err
    row_err = ((outs[0][:, :n].double() - ref).norm(dim=1) / ref.norm(dim=1).clamp(min=1e-6)).max()
    assert float(row_err) < 1e-2
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_gemm_rejections(dev):
    from llm_inference_engine_b200 import _capi
    from llm_inference_engine_b200._capi import TensorMap

    lib = _capi.load()
    w = torch.zeros((4096, 1024), device=dev, dtype=torch.bfloat16)
    x = torch.zeros((64, 1024), device=dev, dtype=torch.bfloat16)
    out = torch.zeros((64, 4096), device=dev, dtype=torch.bfloat16)
    ws = torch.zeros(1 << 22, device=dev)
    cnt = torch.zeros(64, device=dev, dtype=torch.int32)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    tm = TensorMap.for_matrix(w.data_ptr(), 4096, 1024, 2048, 128)
    call = lambda ntok=64, pair=0, cluster=1, split=1, stages=2, wgs=4, ws_=ws, rows=128, atoms=1: lib.muse_gemm_tc(
        tm.ptr, x.data_ptr(), out.data_ptr(), None if ws_ is None else ws_.data_ptr(), cnt.data_ptr(), status.data_ptr(), 64, 4096,
        1024, 1024, 4096, ntok, pair, cluster, split, stages, wgs, rows, atoms, None, None)
    assert call(ntok=40) == -7                      # tokens per tile: multiples of 16
    assert call(cluster=2, split=2) == -3           # slices meet in a cluster or in the workspace, not both
    assert call(cluster=17) == -3 and call(split=17) == -3   # more slices than 64-wide chunks of K
    assert call(split=4, ws_=None) == -4            # a workspace split needs the workspace
    assert call(split=8) == -10                     # 32 units x 8 slices cannot all be resident at once
    assert call(stages=13) == -5 and call(wgs=5) == -9
    assert call(atoms=0) == -12 and call(atoms=9) == -12 and call(cluster=5, atoms=4) == -3   # 16 atoms of K in steps of 4: four slices at most
    assert call(rows=100) == -11 and call(rows=136) == -11 and call(pair=1, rows=64) == -11   # multiples of 8 up to 128; pairs are whole tiles
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0 and float(out.abs().max()) == 0.0


FEWTOK_CASES = [  # (m, n, k, warps, unroll) + optional tok_split
    (2, 12288, 4096, 16, 4), (8, 12288, 4096, 32, 4), (16, 4096, 1024, 16, 2), (3, 1001, 4096, 32, 1), (9, 520, 2080, 16, 2),
    (1, 8, 32, 16, 1), (5, 3, 64, 32, 4), (13, 1024, 4096, 32, 4), (7, 300, 8192, 16, 4),
    (16, 12288, 4096, 16, 8), (9, 4093, 1024, 16, 2), (12, 1000, 2048, 32, 2), (5, 4096, 4096, 16, 8), (11, 777, 3072, 16, 8),
    (32, 12288, 4096, 16, 8, 2), (16, 12288, 4096, 32, 4, 2), (27, 1001, 4096, 32, 4, 4), (19, 4096, 1024, 16, 2, 2),
    (40, 300, 2048, 16, 4, 3), (3, 520, 1024, 32, 1, 2),
]


@pytest.mark.parametrize("case", FEWTOK_CASES, ids=lambda c: "m{}_n{}_k{}_w{}u{}".format(*c) + ("_t%d" % c[5] if len(c) > 5 else ""))
def test_fewtok_entry_point_matches_oracle_and_is_bit_stable(dev, case):
    """muse_fewtok_mma (register-level MMAs, 1..16 tokens) through the C ABI: FP64 product within the
    BF16 tolerance, ragged N (rows not a multiple of 8), strided x and out, columns beyond n untouched,
    identical bits on repeated calls (the warps' partial sums are added in a fixed order)."""
    from llm_inference_engine_b200 import _capi

    m, n, k, warps, unroll = case[:5]
    tok_split = case[5] if len(case) > 5 else 1
    lib = _capi.load()
    g = torch.Generator(device=dev).manual_seed(m * 11 + n)
    w = (torch.randn((n, k), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn((m, k + 24), generator=g, device=dev).to(torch.bfloat16)[:, :k]
    ref = x.double() @ w.double().T
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    outs = []
    for _ in range(3):
        out = torch.full((m, n + 5), 3.0, device=dev, dtype=torch.bfloat16)
        _capi.check(lib.muse_fewtok_mma(w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), out.stride(0), warps,
                                        unroll, tok_split, status.data_ptr(), None, torch.cuda.current_stream(dev).cuda_stream),
                    "muse_fewtok_mma")
        torch.cuda.synchronize(dev)
        outs.append(out)
    assert int(status.item()) == 0
    assert bool((outs[0][:, n:] == 3.0).all())
    err = float((outs[0][:, :n].double() - ref).norm() / ref.norm())
    assert err < 5e-3, err
    row_err = ((outs[0][:, :n].double() - ref).norm(dim=1) / ref.norm(dim=1).clamp(min=1e-6)).max()
    assert float(row_err) < 1e-2
    assert all(torch.equal(outs[0], o) for o in outs[1:])


def test_fewtok_rejections(dev):
    from llm_inference_engine_b200 import _capi

    lib = _capi.load()
    w = torch.zeros((64, 4096), device=dev, dtype=torch.bfloat16)
    x = torch.zeros((17, 4096), device=dev, dtype=torch.bfloat16)
    out = torch.zeros((17, 64), device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    call = lambda m, n, k, ldx, ldo, warps, unroll, split=1: lib.muse_fewtok_mma(
        w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n, k, ldx, ldo, warps, unroll, split, status.data_ptr(), None, None)
    assert call(17, 64, 4096, 4096, 64, 16, 4) == -9        # more than 16 tokens per copy of the walk
    assert call(17, 64, 4096, 4096, 64, 16, 4, split=2) == -9   # x in shared memory: one CTA holds all tokens
    assert call(4, 64, 4096, 4096, 64, 32, 4, split=5) == -9
    assert call(4, 64, 4080, 4096, 64, 16, 4) == -2         # K not a multiple of 32
    assert call(4, 64, 4096, 4096, 32, 16, 4) == -2         # out rows shorter than n
    assert call(4, 64, 4096, 4096, 64, 8, 4) != 0           # unsupported CTA size
    assert call(16, 64, 16384, 16384, 64, 32, 4) == -5      # 16 rows of x do not fit in shared memory
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0


def test_host_buffer_entry_point_matches_device_path(proj, dev, target_setup):
    """kernel_fn_host (x and the result in page-locked host memory) returns the bits of kernel_fn for the
    GEMV, register-MMA and TMEM plans, reuses its staging buffers, and rejects device tensors."""
    _, state = target_setup
    g = torch.Generator().manual_seed(99)
    for layer, m, n, k in (("qkv_gate", 1, 12288, 4096), ("qkv_gate", 8, 12288, 4096), ("qkv_gate", 32, 12288, 4096),
                           ("router", 8, 256, 4096), ("unpooler", 5, 2048, 1024)):
        cfg = {"m": m, "n": n, "k": k, "layer": layer}
        x = torch.randn((m, k), generator=g).to(torch.bfloat16).pin_memory()
        want = proj.kernel_fn({"x": x.to(dev), "config": cfg}, state).cpu()
        got = proj.kernel_fn_host({"x": x, "config": cfg}, state)
        assert not got.is_cuda and got.dtype == want.dtype and torch.equal(got, want)
        out = torch.empty_like(want).pin_memory()
        again = proj.kernel_fn_host({"x": x, "config": cfg}, state, out=out)      # records the round trip
        assert again is out and torch.equal(out, want)
        x.copy_(torch.randn((m, k), generator=g).to(torch.bfloat16))               # same buffers, new contents
        want2 = proj.kernel_fn({"x": x.to(dev), "config": cfg}, state).cpu()
        out.zero_()
        assert torch.equal(proj.kernel_fn_host({"x": x, "config": cfg}, state, out=out), want2)   # replays it
        assert torch.equal(proj.kernel_fn_host({"x": x, "config": cfg}, state, out=out, record=False), want2)
    assert len(state["_host_slots"]) == 5 and len(state["_host_graphs"]) == 5
    with pytest.raises(TypeError):
        proj.kernel_fn_host({"x": x.to(dev), "config": cfg}, state)
    proj.check_status(state)


def test_an_activation_buffer_that_is_rewritten_between_calls(proj, dev, target_setup):
    """A decode loop hands every call the same x buffer with new contents, written by a kernel just ahead in the
    stream. The projections may become resident under that kernel's tail (programmatic dependent launch), so they
    read x through L2-coherent loads after their grid-dependency wait: 24 rounds per plan behind a torch copy kernel
    and 24 behind the library's fetch kernel, each against the same call on a fresh copy of x, bit for bit. (The
    case that showed stale activations with non-coherent loads is the column-parallel host round trip at 32 tokens
    in tests/tp_worker.py; this is the one-GPU form of the same contract.)"""
    _, state = target_setup
    g = torch.Generator(device=dev).manual_seed(4242)
    for layer, m, n, k in (("qkv_gate", 8, 12288, 4096), ("o", 16, 4096, 4096), ("o", 1, 4096, 4096), ("router", 8, 256, 4096),
                           ("pooler", 32, 1024, 4096), ("unpooler", 4, 4096, 1024), ("o", 32, 4096, 4096), ("o", 100, 4096, 4096)):
        cfg = {"m": m, "n": n, "k": k, "layer": layer}
        x = torch.zeros((m, k), device=dev, dtype=torch.bfloat16)
        src = [torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16) for _ in range(4)]
        want = [proj.kernel_fn({"x": s.clone(), "config": cfg}, state).clone() for s in src]
        torch.cuda.synchronize(dev)
        for r in range(24):
            x.copy_(src[r % 4])                                     # a kernel rewrites the buffer ...
            got = proj.kernel_fn({"x": x, "config": cfg}, state)    # ... and the projection is launched right behind it
            assert torch.equal(got, want[r % 4]), (layer, m, r)
        # The same with the library's own fetch kernel as the writer: it lets its dependents start at once, so the
        # projection is resident, weights in flight, while x is still being written.
        from llm_inference_engine_b200 import _capi

        lib = _capi.load()
        pinned = [t.cpu().pin_memory() for t in src]
        stream = torch.cuda.current_stream(dev).cuda_stream
        for r in range(24):
            _capi.check(lib.muse_fetch_host(x.data_ptr(), pinned[r % 4].data_ptr(), m * k * 2, stream), "muse_fetch_host")
            got = proj.kernel_fn({"x": x, "config": cfg}, state)
            assert torch.equal(got, want[r % 4]), (layer, m, r, "behind the fetch kernel")
    proj.check_status(state)


def test_ordinary_launches_give_the_same_bits(proj, dev, target_setup):
    """muse_set_programmatic_launch(0): every launch an ordinary one. Launch ordering is all the switch changes, so
    every plan family returns the bits it returns as a programmatic dependent; the previous setting comes back."""
    from llm_inference_engine_b200 import _capi

    lib = _capi.load()
    _, state = target_setup
    g = torch.Generator(device=dev).manual_seed(77)
    cases = (("qkv_gate", 8, 12288, 4096), ("o", 1, 4096, 4096), ("o", 16, 4096, 4096), ("o", 32, 4096, 4096), ("o", 200, 4096, 4096),
             ("router", 1, 256, 4096), ("router", 8, 256, 4096), ("router", 100, 256, 4096), ("pooler", 256, 1024, 4096))
    datas = [{"x": torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16), "config": {"m": m, "n": n, "k": k, "layer": layer}}
             for layer, m, n, k in cases]
    with_pdl = [proj.kernel_fn(d, state).clone() for d in datas]
    assert lib.muse_set_programmatic_launch(0) == 1
    try:
        plain = [proj.kernel_fn(d, state).clone() for d in datas]
    finally:
        assert lib.muse_set_programmatic_launch(1) == 0
    torch.cuda.synchronize(dev)
    for d, a, b in zip(datas, with_pdl, plain):
        assert torch.equal(a, b), d["config"]
    proj.check_status(state)


FEWTOK_F32_CASES = [  # (m, n, k, unroll, tok_split)
    (8, 256, 4096, 8, 1), (32, 256, 4096, 8, 4), (1, 256, 4096, 8, 1), (5, 100, 1024, 2, 1), (20, 77, 2048, 4, 3), (13, 1003, 512, 2, 2),
]


@pytest.mark.parametrize("case", FEWTOK_F32_CASES, ids=lambda c: "m{}_n{}_k{}_u{}t{}".format(*c))
def test_fewtok_f32_entry_point_meets_the_router_tolerance(dev, case):
    """muse_fewtok_f32 (FP32 weights split to BF16 hi + lo in registers) through the C ABI: within the
    router's 1e-5 relative L2 of the FP64 product, identical bits on repeated calls, ragged N, strided
    x and out, columns beyond n untouched."""
    from llm_inference_engine_b200 import _capi

    m, n, k, unroll, tok_split = case
    lib = _capi.load()
    g = torch.Generator(device=dev).manual_seed(m * 13 + n)
    w = torch.randn((n, k), generator=g, device=dev) * 0.02
    x = torch.randn((m, k + 8), generator=g, device=dev).to(torch.bfloat16)[:, :k]
    ref = x.double() @ w.double().T
    outs = []
    for _ in range(3):
        out = torch.full((m, n + 3), 3.0, device=dev, dtype=torch.float32)
        _capi.check(lib.muse_fewtok_f32(w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n, k, x.stride(0), out.stride(0), unroll,
                                        tok_split, 0, torch.cuda.current_stream(dev).cuda_stream), "muse_fewtok_f32")
        torch.cuda.synchronize(dev)
        outs.append(out)
    assert bool((outs[0][:, n:] == 3.0).all())
    err = float((outs[0][:, :n].double() - ref).norm() / ref.norm())
    assert err < 1e-5, err
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    call = lambda m_, k_, unroll_, split_: lib.muse_fewtok_f32(w.data_ptr(), x.data_ptr(), outs[0].data_ptr(), m_, n, k_,
                                                               x.stride(0), outs[0].stride(0), unroll_, split_, 0, None)
    assert call(8 * tok_split + 1, k, unroll, tok_split) == -9     # more than 8 tokens per copy of the walk
    assert call(m, k, 1, tok_split) != 0                           # a row does not fit one batch of loads
    assert call(m, k, unroll, 5) == -9


@pytest.mark.parametrize("m", [1, 3, 8, 13, 32])
def test_router_takes_fp32_activations(oracle, proj, dev, target_setup, m):
    """The decode layer's FP32-input router mode through kernel_fn: x FP32, split to BF16 hi + lo in the
    kernel like the weight. Against the FP64 product of the unsplit inputs the error is at the 2^-16
    level the reference states (here: relative L2 <= 1e-5, the router's tolerance); against the FP64
    evaluation of the same three-term split it is FP32 summation error only; and it is far closer
    than the BF16-x call on the same numbers."""
    w_cpu, state = target_setup
    g = torch.Generator().manual_seed(300 + m)
    x = torch.randn((m, 4096), generator=g)
    cfg = {"m": m, "n": 256, "k": 4096, "layer": "router"}
    out = proj.kernel_fn({"x": x.to(dev), "config": cfg}, state)
    proj.check_status(state)
    assert out.dtype == torch.float32 and tuple(out.shape) == (m, 256)
    out = out.cpu().double()
    ref = oracle.router_f32_input_reference(x, w_cpu["router"])
    model = oracle.router_f32_input_model(x, w_cpu["router"]).double()
    rel = lambda a, b: float((a - b).norm() / b.norm())
    assert rel(out, ref) < 1e-5, rel(out, ref)
    assert rel(out, model) < 2e-6, rel(out, model)
    coarse = proj.kernel_fn({"x": x.to(torch.bfloat16).to(dev), "config": cfg}, state).cpu().double()
    assert rel(coarse, ref) > 20 * rel(out, ref)
    # strided FP32 x and a preallocated output
    xs = torch.zeros((m, 4096 + 8))
    xs[:, :4096] = x
    dst = torch.full((m, 300), 7.0, device=dev)
    proj.kernel_fn({"x": xs.to(dev)[:, :4096], "config": cfg}, state, out=dst)
    assert torch.equal(dst[:, :256].cpu().double(), out) and bool((dst[:, 256:] == 7.0).all())
    with pytest.raises(TypeError):
        proj.kernel_fn({"x": torch.zeros((33, 4096), device=dev), "config": dict(cfg, m=33)}, state)   # beyond 32 tokens
    with pytest.raises(TypeError):
        proj.kernel_fn({"x": torch.zeros((2, 4096), device=dev), "config": {"m": 2, "n": 1024, "k": 4096, "layer": "pooler"}}, state)


@pytest.mark.parametrize("m", [8, 32])
def test_router_on_a_side_stream_beside_the_pooler(oracle, proj, dev, target_setup, m):
    """The decode layer's use of the path (best_submissions/muse_decode_layer.py:226-233, :861-869): the router
    runs on a side stream while the pooler runs on the main one, each through a plan that reduces in the
    global workspace, so the two calls overlap on the GPU with a workspace each. Fork and join are captured in
    one CUDA graph; 200 cold replays; both outputs against the oracle every time, and both streams'
    workspaces and counters zero afterwards."""
    from llm_inference_engine_b200.graph_timer import ColdReplayTimer

    w_cpu, state = target_setup
    timer = ColdReplayTimer(dev, flush_bytes=256 << 20)
    main, side = timer.stream, torch.cuda.Stream(dev)
    pool = oracle.target_input(m, "pooler", 6100 + m, device="cpu")
    rout = oracle.target_input(m, "router", 6200 + m, device="cpu")
    xp, xr = pool["x"].to(dev), rout["x"].to(dev)
    want_p = (pool["x"].double() @ w_cpu["pooler"].double().T).to(dev)
    want_r = (rout["x"].double() @ w_cpu["router"].double().T).to(dev)
    state["_override"][("pooler", m)] = dict(cluster=2, groups=9, stages=3)
    state["_override"][("router", m)] = dict(cluster=1, groups=37, stages=2)
    hold = {}

    def both():
        side.wait_stream(torch.cuda.current_stream(dev))
        hold["p"] = proj.kernel_fn({"x": xp, "config": pool["config"]}, state)
        with torch.cuda.stream(side):
            hold["r"] = proj.kernel_fn({"x": xr, "config": rout["config"]}, state)
        torch.cuda.current_stream(dev).wait_stream(side)

    try:
        with torch.cuda.stream(main):
            both()                      # in the open first: each stream's workspace is made outside the capture
            main.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=main):
                both()
            bad = torch.zeros((), device=dev, dtype=torch.int32)
            for i in range(200):
                if i % 2 == 0:
                    timer.flush.fill_(i & 0xFF)
                graph.replay()
                ep = (hold["p"].double() - want_p).norm() / want_p.norm()
                er = (hold["r"].double() - want_r).norm() / want_r.norm()
                bad += ((ep > 5e-3) | (er > 2e-5)).int()
            main.synchronize()
        assert int(bad) == 0, f"{int(bad)}/200 replays with a wrong pooler or router output"
        assert hold["p"].dtype == torch.bfloat16 and hold["r"].dtype == torch.float32
        pools = state["_ws_by_stream"]
        assert main.cuda_stream in pools and side.cuda_stream in pools and pools[main.cuda_stream][0] is not pools[side.cuda_stream][0]
        for key in (main.cuda_stream, side.cuda_stream):
            ws, cnt = pools[key]
            assert float(ws.abs().max()) == 0.0 and int(cnt.abs().max()) == 0
    finally:
        state["_override"].pop(("pooler", m), None)
        state["_override"].pop(("router", m), None)
    proj.check_status(state)
