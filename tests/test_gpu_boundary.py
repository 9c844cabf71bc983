"""GPU parity of the post-attention boundary (the producer of the pooler's and the router's input in the
reference's decode layer) against the CPU oracle's restatement of decode_layer/reference.py:452-454, which
tests/test_oracle_golden.py pins to the reference: as a kernel of its own, and fused into the pooler and router
projections as their prologue. Tolerances: stream1 and the FP32 h within 2e-6 relative L2 of the FP32
reference (same arithmetic, other summation order); the BF16 h within one BF16 rounding; the pooler output
within the path's BF16 tolerance and the router logits within the FP32-input mode's 2e-5 of the FP64 product."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-30))


@pytest.fixture(scope="module")
def proj():
    from llm_inference_engine_b200 import muse_bf16_proj

    return muse_bf16_proj


def _state(oracle, proj, d, seed, layers):
    stream, attn_out, gate, norm_w = oracle.boundary_inputs(1, d, seed)
    w_cpu = oracle.target_weights(layers=layers)
    state = proj.prepare({k: v.to(DEV) for k, v in w_cpu.items()}, warmup=False)
    proj.prepare_boundary(state, gate.to(DEV), norm_w.to(DEV))
    return state, w_cpu, gate, norm_w


@pytest.mark.parametrize("m,d", [(1, 4096), (8, 4096), (5, 1024), (32, 8192), (3, 4104), (200, 2048)])
def test_standalone_boundary_matches_the_oracle(oracle, proj, m, d):
    stream, attn_out, gate, norm_w = oracle.boundary_inputs(m, d, 900 + m)
    state = {}
    proj.prepare_boundary(state, gate.to(DEV), norm_w.to(DEV))
    a_cpu, b_cpu = oracle.residual_coefficients(gate)
    assert rel(state["_boundary"][0].cpu(), a_cpu) < 1e-6 and rel(state["_boundary"][1].cpu(), b_cpu) < 1e-6
    s1, h, hf = proj.attn_boundary(stream.to(DEV), attn_out.to(DEV), state)
    torch.cuda.synchronize(DEV)
    want_s1, want_h = oracle.attn_boundary(stream, attn_out, gate, norm_w)
    assert s1.dtype == torch.float32 and h.dtype == torch.bfloat16 and (hf is None) == (m > 8)
    assert rel(s1.cpu(), want_s1) < 2e-6
    assert rel(h.cpu().float(), want_h) < 4e-3 and bool(((h.cpu().float() - want_h).abs() <= 2.0 ** -8 * want_h.abs() + 1e-6).all())
    if hf is not None:
        assert rel(hf.cpu(), want_h) < 2e-6


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("layer", ["pooler", "router"])
def test_fused_boundary_projection_matches_the_oracle(oracle, proj, layer, m):
    """h @ W.T through muse_fewtok_boundary equals the boundary followed by the projection: against the oracle's
    FP64 product of the oracle's h (BF16-rounded for the pooler, as the reference's kernel hands it over), and
    bit for bit against this library's own two-kernel route for the pooler."""
    layers = {layer: oracle.TARGET_LAYERS[layer]}
    n, k = layers[layer]
    state, w_cpu, gate, norm_w = _state(oracle, proj, k, 77, layers)
    stream, attn_out, _, _ = oracle.boundary_inputs(m, k, 77)          # the same gate and norm weight (same seed, same draws first)
    stream, attn_out = stream[:m].contiguous(), attn_out[:m].contiguous()
    want_s1, want_h = oracle.attn_boundary(stream, attn_out, gate, norm_w)
    s1 = torch.full((m, k), float("nan"), device=DEV)
    h = torch.full((m, k), float("nan"), device=DEV, dtype=torch.bfloat16)
    hf = torch.full((m, k), float("nan"), device=DEV)
    data = {"stream": stream.to(DEV), "attn_out": attn_out.to(DEV), "config": {"layer": layer, "m": m, "n": n, "k": k}}
    outs = [proj.kernel_fn_boundary(data, state, stream1=s1, h=h, h_f32=hf) for _ in range(3)]
    proj.check_status(state)
    assert all(torch.equal(outs[0], o) for o in outs[1:])                 # fixed summation order
    assert rel(s1.cpu(), want_s1) < 2e-6 and rel(hf.cpu(), want_h) < 2e-6 and rel(h.cpu().float(), want_h) < 4e-3
    if layer == "router":
        exact = want_h.double() @ w_cpu[layer].double().T
        assert outs[0].dtype == torch.float32 and rel(outs[0].cpu(), exact) < 2e-5
    else:
        exact = want_h.to(torch.bfloat16).double() @ w_cpu[layer].double().T
        assert outs[0].dtype == torch.bfloat16 and rel(outs[0].cpu(), exact) < 6e-3
        # the two-kernel route of this library: boundary kernel, then the projection on its BF16 h
        _, h2, _ = proj.attn_boundary(data["stream"], data["attn_out"], state)
        two = proj.kernel_fn({"x": h2, "config": data["config"]}, state)
        assert torch.equal(h2, h) and rel(two.cpu(), exact) < 6e-3
        assert rel(outs[0].cpu(), two.cpu()) < 2e-3                      # same inputs, other kernel (other summation order)
    # without the optional outputs
    again = proj.kernel_fn_boundary(data, state)
    assert torch.equal(again, outs[0])


@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_one_launch_boundary_pooler_router(oracle, proj, m):
    """muse_boundary_pooler_router: both outputs, stream1, h and the FP32 h against the oracle, and bit for bit
    against the per-layer fused entry (same walk, same summation order), over repeated calls."""
    layers = {name: oracle.TARGET_LAYERS[name] for name in ("pooler", "router")}
    k = layers["pooler"][1]
    state, w_cpu, gate, norm_w = _state(oracle, proj, k, 41, layers)
    stream, attn_out, _, _ = oracle.boundary_inputs(m, k, 41)
    stream, attn_out = stream[:m].contiguous(), attn_out[:m].contiguous()
    want_s1, want_h = oracle.attn_boundary(stream, attn_out, gate, norm_w)
    s1 = torch.full((m, k), float("nan"), device=DEV)
    h = torch.full((m, k), float("nan"), device=DEV, dtype=torch.bfloat16)
    hf = torch.full((m, k), float("nan"), device=DEV)
    data = {"stream": stream.to(DEV), "attn_out": attn_out.to(DEV)}
    outs = [proj.boundary_pooler_router(data, state, stream1=s1, h=h, h_f32=hf) for _ in range(3)]
    torch.cuda.synchronize(DEV)
    assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])
    pooled, logits = outs[0]
    assert pooled.dtype == torch.bfloat16 and tuple(pooled.shape) == (m, layers["pooler"][0])
    assert logits.dtype == torch.float32 and tuple(logits.shape) == (m, layers["router"][0])
    assert rel(s1.cpu(), want_s1) < 2e-6 and rel(hf.cpu(), want_h) < 2e-6 and rel(h.cpu().float(), want_h) < 4e-3
    assert rel(logits.cpu(), want_h.double() @ w_cpu["router"].double().T) < 2e-5
    assert rel(pooled.cpu(), want_h.to(torch.bfloat16).double() @ w_cpu["pooler"].double().T) < 6e-3
    for layer, got in (("pooler", pooled), ("router", logits)):
        cfg = {"layer": layer, "m": m, "n": layers[layer][0], "k": k}
        one = proj.kernel_fn_boundary(dict(data, config=cfg), state)
        assert rel(got.cpu(), one.cpu()) < (2e-3 if layer == "pooler" else 2e-6)
    again = proj.boundary_pooler_router(data, state)                     # without the optional outputs
    assert torch.equal(again[0], pooled) and torch.equal(again[1], logits)
    with pytest.raises(ValueError):
        big = {"stream": torch.zeros((9, k), device=DEV), "attn_out": torch.zeros((9, k), device=DEV, dtype=torch.bfloat16)}
        proj.boundary_pooler_router(big, state)


def test_one_launch_replays_leave_the_flags_clear(oracle, proj):
    """The kernel's CTAs hand h over through ready flags that the last CTA re-arms: 600 replays of one captured
    call, with the inputs changed between two batches, give the eager results bit for bit, the flag words end at
    zero and no wait ran out."""
    layers = {name: oracle.TARGET_LAYERS[name] for name in ("pooler", "router")}
    k = layers["pooler"][1]
    state, _, _, _ = _state(oracle, proj, k, 43, layers)
    m = 8
    stream, attn_out, _, _ = oracle.boundary_inputs(m, k, 43)
    data = {"stream": stream[:m].contiguous().to(DEV), "attn_out": attn_out[:m].contiguous().to(DEV)}
    want = [t.clone() for t in proj.boundary_pooler_router(data, state)]
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side):
        proj.boundary_pooler_router(data, state)                        # this stream's workspace exists before the capture
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            got = proj.boundary_pooler_router(data, state)
        for _ in range(300):
            graph.replay()
        side.synchronize()
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        data["stream"].mul_(1.5)
        data["attn_out"].mul_(0.5)
        for _ in range(300):
            graph.replay()
        side.synchronize()
        key = side.cuda_stream
    torch.cuda.current_stream(DEV).wait_stream(side)
    want2 = proj.boundary_pooler_router(data, state)
    torch.cuda.synchronize(DEV)
    assert torch.equal(got[0], want2[0]) and torch.equal(got[1], want2[1])
    assert not torch.equal(want2[0], want[0])
    for _, cnt in state["_ws_by_stream"].values():
        assert int(cnt[:16].abs().max()) == 0
    assert key in state["_ws_by_stream"]
    proj.check_status(state)


def test_fused_boundary_rejections(oracle, proj):
    layers = {"pooler": oracle.TARGET_LAYERS["pooler"]}
    state, _, _, _ = _state(oracle, proj, 4096, 5, layers)
    cfg = {"layer": "pooler", "m": 9, "n": 1024, "k": 4096}
    s = torch.zeros((9, 4096), device=DEV)
    a = torch.zeros((9, 4096), device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        proj.kernel_fn_boundary({"stream": s, "attn_out": a, "config": cfg}, state)          # more than 8 tokens
    with pytest.raises(TypeError):
        proj.kernel_fn_boundary({"stream": s[:4].half(), "attn_out": a[:4], "config": dict(cfg, m=4)}, state)
    with pytest.raises(RuntimeError):
        proj.kernel_fn_boundary({"stream": s[:4], "attn_out": a[:4], "config": dict(cfg, m=4)}, {"pooler": state["pooler"]})
