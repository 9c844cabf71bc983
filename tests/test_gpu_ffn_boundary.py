"""GPU parity of the post-FFN boundary (the consumer of the unpooler's output in the reference's decode layer)
against the CPU oracle's restatement of decode_layer/reference.py:466-476, which tests/test_oracle_golden.py pins
to the reference: as a kernel of its own, and as one launch together with the unpooler projection. Tolerances:
stream2 within 2e-6 relative L2 of the FP32 reference given the same f (same arithmetic, other summation order);
hidden within one BF16 rounding; with the projection inside, f carries the projection's own FP32 summation error
(relative 1e-5) instead of a BF16 rounding, so the one-launch form is held to the FP64 projection directly."""

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


def bf16_close(got: torch.Tensor, want: torch.Tensor) -> bool:
    return bool(((got.float() - want).abs() <= 2.0 ** -8 * want.abs() + 1e-6).all())


@pytest.mark.parametrize("m,d,nf", [(1, 4096, 1024), (8, 4096, 1024), (16, 4096, 4096), (5, 2048, 512), (3, 8192, 8192), (200, 1024, 256)])
def test_standalone_ffn_boundary_matches_the_oracle(oracle, proj, m, d, nf):
    stream1, f, gate, post_w, next_w = oracle.ffn_boundary_inputs(m, d, nf, 40 + m)
    state = {}
    proj.prepare_ffn_boundary(state, gate.to(DEV), post_w.to(DEV), next_w.to(DEV))
    s2, hidden = proj.ffn_boundary(stream1.to(DEV), f.to(DEV), state)
    torch.cuda.synchronize(DEV)
    want_s2, want_h = oracle.ffn_boundary(stream1, f, gate, post_w, next_w)
    assert s2.dtype == torch.float32 and hidden.dtype == torch.bfloat16
    assert rel(s2.cpu(), want_s2) < 2e-6
    assert rel(hidden.cpu().float(), want_h) < 4e-3 and bf16_close(hidden.cpu(), want_h)


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("nf", [1024, 4096])
def test_unpooler_and_boundary_in_one_launch(oracle, proj, m, nf):
    layers = {"unpooler": oracle.TARGET_LAYERS["unpooler"]}
    n, k = layers["unpooler"]
    d = n
    w_cpu = oracle.target_weights(layers=layers)
    state = proj.prepare({"unpooler": w_cpu["unpooler"].to(DEV)}, warmup=False)
    stream1, _, gate, post_w, next_w = oracle.ffn_boundary_inputs(m, d, nf, 60 + m)
    proj.prepare_ffn_boundary(state, gate.to(DEV), post_w.to(DEV), next_w.to(DEV))
    g = torch.Generator().manual_seed(70 + m)
    x = torch.randn((m, k), generator=g).bfloat16()
    f_exact = x.double() @ w_cpu["unpooler"][:nf].double().T
    want_s2, want_h = oracle.ffn_boundary(stream1, f_exact.float(), gate, post_w, next_w)
    data = {"x": x.to(DEV), "stream1": stream1.to(DEV), "config": {"layer": "unpooler", "m": m, "n": nf, "k": k}}
    outs = [proj.unpooler_ffn_boundary(data, state) for _ in range(3)]
    torch.cuda.synchronize(DEV)
    proj.check_status(state)
    assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs[1:])
    s2, hidden = outs[0]
    assert rel(s2.cpu(), want_s2) < 2e-5
    assert rel(hidden.cpu().float(), want_h) < 4e-3 and bool(((hidden.cpu().float() - want_h).abs() <= 2.0 ** -7 * want_h.abs() + 1e-5).all())
    # the two-kernel route of this library rounds f to BF16 in between: close, not equal
    f2 = proj.kernel_fn({"x": data["x"], "config": data["config"]}, state)
    s2b, hb = proj.ffn_boundary(data["stream1"], f2, state)
    assert rel(s2b.cpu(), want_s2) < 3e-3 and rel(hb.cpu().float(), hidden.cpu().float()) < 8e-3
    for _, cnt in state["_ws_by_stream"].values():
        assert int(cnt[:32].abs().max()) == 0


def test_one_launch_replays_and_rejections(oracle, proj):
    layers = {"unpooler": oracle.TARGET_LAYERS["unpooler"]}
    n, k = layers["unpooler"]
    w_cpu = oracle.target_weights(layers=layers)
    state = proj.prepare({"unpooler": w_cpu["unpooler"].to(DEV)}, warmup=False)
    stream1, _, gate, post_w, next_w = oracle.ffn_boundary_inputs(8, n, 1024, 91)
    cfg = {"layer": "unpooler", "m": 8, "n": 1024, "k": k}
    x = torch.randn((8, k), generator=torch.Generator().manual_seed(92)).bfloat16().to(DEV)
    with pytest.raises(RuntimeError):
        proj.unpooler_ffn_boundary({"x": x, "stream1": stream1.to(DEV), "config": cfg}, state)
    proj.prepare_ffn_boundary(state, gate.to(DEV), post_w.to(DEV), next_w.to(DEV))
    data = {"x": x, "stream1": stream1.to(DEV), "config": cfg}
    want = [t.clone() for t in proj.unpooler_ffn_boundary(data, state)]
    side = torch.cuda.Stream(DEV)
    side.wait_stream(torch.cuda.current_stream(DEV))
    with torch.cuda.stream(side):
        proj.unpooler_ffn_boundary(data, state)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            got = proj.unpooler_ffn_boundary(data, state)
        for _ in range(500):
            graph.replay()
        side.synchronize()
    torch.cuda.current_stream(DEV).wait_stream(side)
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    for _, cnt in state["_ws_by_stream"].values():
        assert int(cnt[:32].abs().max()) == 0
    proj.check_status(state)
    with pytest.raises(ValueError):
        proj.unpooler_ffn_boundary({"x": torch.zeros((9, k), device=DEV, dtype=torch.bfloat16), "stream1": torch.zeros((9, n), device=DEV),
                                    "config": dict(cfg, m=9)}, state)
    with pytest.raises(ValueError):
        proj.unpooler_ffn_boundary({"x": x, "stream1": stream1.to(DEV), "config": dict(cfg, n=1004)}, state)
    with pytest.raises(TypeError):
        proj.ffn_boundary(stream1.to(DEV), torch.zeros((8, 1024), device=DEV), state)


def test_a_count_that_never_completes_gives_up_and_recovers(oracle, proj):
    """Failure detection without a fault: the token CTAs wait for every CTA of the launch to count itself. With the
    counter started three short, the count never completes: the wait is bounded (0.5 s), the kernel comes back by
    itself, reports ST_X_TIMEOUT and re-arms the counters, and the next call is correct."""
    import time

    layers = {"unpooler": oracle.TARGET_LAYERS["unpooler"]}
    n, k = layers["unpooler"]
    w_cpu = oracle.target_weights(layers=layers)
    state = proj.prepare({"unpooler": w_cpu["unpooler"].to(DEV)}, warmup=False)
    stream1, _, gate, post_w, next_w = oracle.ffn_boundary_inputs(2, n, 1024, 95)
    proj.prepare_ffn_boundary(state, gate.to(DEV), post_w.to(DEV), next_w.to(DEV))
    x = torch.randn((2, k), generator=torch.Generator().manual_seed(96)).bfloat16().to(DEV)
    data = {"x": x, "stream1": stream1.to(DEV), "config": {"layer": "unpooler", "m": 2, "n": 1024, "k": k}}
    good = [t.clone() for t in proj.unpooler_ffn_boundary(data, state)]
    proj.check_status(state)
    _, cnt = proj._stream_workspace(state, DEV)
    cnt[16] = -3
    torch.cuda.synchronize(DEV)
    t0 = time.perf_counter()
    proj.unpooler_ffn_boundary(data, state)
    torch.cuda.synchronize(DEV)
    waited = time.perf_counter() - t0
    assert 0.3 < waited < 5.0, waited                      # the bounded wait, not a hang and not a skip
    with pytest.raises(Exception, match="timed-out wait"):
        proj.check_status(state)
    assert int(cnt[:32].abs().max()) == 0                  # the last token CTA re-armed the counters
    again = proj.unpooler_ffn_boundary(data, state)
    proj.check_status(state)
    assert torch.equal(again[0], good[0]) and torch.equal(again[1], good[1])
