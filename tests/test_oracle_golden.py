"""Pins the CPU oracle (oracle/muse_proj_oracle.py) to the reference: every vector that
tests/golden/make_golden.py recorded by importing bf16_proj/reference.py + checks.py is replayed
through the restatement and must come out identical (digests of generated tensors, probe rows,
verdicts and messages of the checks, speed-of-light floors)."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import pytest
import torch

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_vectors.json").read_text())
HEAD = 16


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def head(t: torch.Tensor) -> list[float]:
    return [float(v) for v in t.flatten()[:HEAD].double()]


@pytest.fixture(scope="module")
def ref_weights(oracle):
    return oracle.generate_weights(oracle.WEIGHTS_SEED, device="cpu")


def test_constants_match_reference(oracle):
    c = GOLDEN["constants"]
    assert oracle.UNPOOL_SLICE_ROWS == c["UNPOOL_SLICE"]
    assert oracle.SLICE_UP_TO_TOKENS == c["SLICED_MAX_TOKENS"]
    assert oracle.WEIGHTS_SEED == c["WEIGHTS_SEED"]
    assert oracle.BF16_REL_L2_TOL == c["REL_L2_TOL"]
    assert oracle.ROUTER_REL_L2_TOL == c["ROUTER_TOL"]
    assert oracle.PROBE_ONE_IN == c["PROBE_EVERY"]
    assert oracle.PROBE_REL_TOL == c["PROBE_TOL"]
    assert oracle.ROW_TOL_FACTOR == GOLDEN["row_factor"]
    assert oracle.ROW_NORM_FLOOR_FRACTION == GOLDEN["row_norm_floor"]
    assert {k: list(v) for k, v in oracle.REFERENCE_LAYERS.items()} == GOLDEN["layers"]


def test_weights_bit_identical(ref_weights):
    assert GOLDEN["torch"].split("+")[0] == torch.__version__.split("+")[0], "golden vectors are tied to the CPU RNG of this torch"
    for name, rec in GOLDEN["weights"].items():
        w = ref_weights[name]
        assert list(w.shape) == rec["shape"] and str(w.dtype) == rec["dtype"]
        assert head(w) == rec["head"]
        assert digest(w) == rec["sha256"], name


def _variants(oracle, data, want, seed, layer, m):
    g = torch.Generator().manual_seed(seed + 1000)
    noise = torch.randn(want.shape, generator=g)
    scale = want.float().abs().mean()
    out = {
        "exact": want.clone(),
        "noise_small": (want.float() + 1e-6 * scale * noise).to(want.dtype),
        "noise_large": (want.float() + 0.2 * scale * noise).to(want.dtype),
        "wrong_dtype": want.to(torch.float16),
    }
    tol = oracle.ROUTER_REL_L2_TOL if layer in oracle.FP32_LAYERS else oracle.BF16_REL_L2_TOL
    bad = want.float().clone()
    bad[m // 2] *= 1.0 + 5.5 * tol
    out["one_bad_row"] = bad.to(want.dtype)
    rows = oracle.probe_rows(data["x"])
    if len(rows):
        off = want.float().clone()
        off[rows[0]] *= 1.0 + 4e-3
        out["probe_row_off"] = off.to(want.dtype)
    return out


@pytest.mark.parametrize("rec", GOLDEN["cases"], ids=lambda r: f"{r['layer']}-m{r['m']}-{r['dist']}")
def test_inputs_reference_and_checks(oracle, ref_weights, rec):
    layer, m, seed = rec["layer"], rec["m"], rec["seed"]
    data = oracle.generate_input(m, layer, seed, rec["dist"], device="cpu")
    assert data["config"] == rec["config"]
    assert digest(data["x"]) == rec["x_sha256"]
    assert head(data["x"]) == rec["x_head"]
    assert [int(i) for i in oracle.probe_rows(data["x"])] == rec["probe_rows"]
    want = oracle.ref_kernel(data, ref_weights)
    assert str(want.dtype) == rec["ref_dtype"]
    assert head(want) == rec["ref_head"]
    assert head(want.float().norm(dim=-1)) == pytest.approx(rec["ref_row_norms"], rel=1e-6)
    variants = _variants(oracle, data, want, seed, layer, m)
    if layer == "router":
        w_bf = ref_weights["router"].to(torch.bfloat16).double()
        variants["bf16_weights"] = (data["x"].double() @ w_bf[: data["config"]["n"]].T).to(want.dtype)
    recorded = {c["variant"]: c for c in rec["checks"]}
    assert set(recorded) == set(variants)
    for name, cand in variants.items():
        ok, msg = oracle.check_implementation(data, cand, ref_weights)
        assert (ok, msg) == (recorded[name]["ok"], recorded[name]["msg"]), name


def test_speed_of_light_and_slice_rule(oracle):
    hw = {"hbm_bytes_per_s": 4.8e12, "bf16_dense_flops_per_s": 989e12}
    for rec in GOLDEN["speed_of_light"]:
        assert oracle.speed_of_light_ns(rec["m"], rec["layer"], hw) == rec["ns"]
    for rec in GOLDEN["out_features"]:
        assert oracle.out_features(rec["layer"], rec["m"]) == rec["n"]


def test_cpu_baseline_restatement_agrees_with_fp64(oracle, ref_weights):
    """The timed CPU baseline (baseline.py restated) passes the reference's own check."""
    state = oracle.cpu_prepare(ref_weights)
    for layer, m in (("o", 1), ("o", 16), ("router", 4), ("router", 32), ("unpooler", 8)):
        data = oracle.generate_input(m, layer, 7 + m, device="cpu")
        ok, msg = oracle.check_implementation(data, oracle.cpu_kernel_fn(data, state), ref_weights)
        assert ok, f"{layer} m={m}: {msg}"


def test_target_generators_and_rule(oracle):
    """The benchmark's own synthetic data: shapes, dtypes, distribution, and the acceptance rule."""
    w = oracle.target_weights(only={"pooler", "router"})
    assert w["pooler"].shape == (1024, 4096) and w["pooler"].dtype == torch.bfloat16
    assert w["router"].shape == (256, 4096) and w["router"].dtype == torch.float32
    assert abs(float(w["router"].std()) - 0.02) < 5e-4
    w2 = oracle.target_weights(only={"router"})
    assert torch.equal(w["router"], w2["router"])  # per-layer generators: independent of `only`
    d = oracle.target_input(32, "pooler", 1000)
    assert d["x"].shape == (32, 4096) and d["config"] == {"m": 32, "n": 1024, "k": 4096, "layer": "pooler"}
    good = oracle.fp32_reference(d, w).to(torch.bfloat16)
    assert oracle.target_check(d, good, w)[0]
    assert not oracle.target_check(d, (good.float() * 1.05 + 0.02).to(torch.bfloat16), w)[0]
    assert not oracle.target_check(d, good.float(), w)[0]  # dtype is part of the contract
    dr = oracle.target_input(8, "router", 1001)
    hi = w["router"].to(torch.bfloat16)
    lo = (w["router"] - hi.float()).to(torch.bfloat16)
    hilo = dr["x"].float() @ hi.float().T + dr["x"].float() @ lo.float().T
    assert oracle.target_check(dr, hilo, w)[0]          # the hi + lo pair meets 1e-5
    assert not oracle.target_check(dr, dr["x"].float() @ hi.float().T, w)[0]  # hi alone does not


BOUNDARY = json.loads((Path(__file__).parent / "golden" / "boundary_vectors.json").read_text())


def test_boundary_constants_match_reference(oracle):
    c = BOUNDARY["constants"]
    assert (oracle.RMS_EPS, oracle.POST_NORM_EPS, oracle.RESIDUAL_TEMPERATURE, oracle.RESIDUAL_GATE_EPS) == (
        c["RMS_EPS"], c["POST_NORM_EPS"], c["RESIDUAL_TEMPERATURE"], c["RESIDUAL_GATE_EPS"])
    assert oracle.ROUTER_FP32_INPUT_UP_TO_TOKENS == c["SLICED_MAX_TOKENS"] == 8


@pytest.mark.parametrize("rec", BOUNDARY["cases"], ids=lambda r: "m{}_d{}".format(r["m"], r["d"]))
def test_boundary_restatement_is_bit_identical(oracle, rec):
    """The post-attention boundary (decode_layer/reference.py:452-454 with :189-191 and :339-344) as restated
    in the oracle, on inputs regenerated from the recorded seeds."""
    stream, attn_out, gate, norm_w = oracle.boundary_inputs(rec["m"], rec["d"], rec["seed"])
    assert digest(torch.cat([stream.flatten(), attn_out.float().flatten(), gate, norm_w.float()])) == rec["inputs_sha256"]
    alpha, beta = oracle.residual_coefficients(gate)
    assert digest(alpha) == rec["alpha_sha256"] and digest(beta) == rec["beta_sha256"] and head(alpha) == rec["alpha_head"]
    stream1, h = oracle.attn_boundary(stream, attn_out, gate, norm_w)
    assert head(stream1) == rec["stream1_head"] and digest(stream1) == rec["stream1_sha256"]
    assert head(h) == rec["h_head"] and digest(h) == rec["h_sha256"]


@pytest.mark.parametrize("rec", BOUNDARY["ffn_cases"], ids=lambda r: "m{}_d{}_nf{}".format(r["m"], r["d"], r["nf"]))
def test_ffn_boundary_restatement_is_bit_identical(oracle, rec):
    """The post-FFN boundary (the tail of ref_back, decode_layer/reference.py:466-476) as restated in the oracle,
    on inputs regenerated from the recorded seeds."""
    stream1, f, gate, post_w, next_w = oracle.ffn_boundary_inputs(rec["m"], rec["d"], rec["nf"], rec["seed"])
    assert digest(torch.cat([stream1.flatten(), f.float().flatten(), gate, post_w.float(), next_w.float()])) == rec["inputs_sha256"]
    stream2, hidden = oracle.ffn_boundary(stream1, f, gate, post_w, next_w)
    assert head(stream2) == rec["stream2_head"] and digest(stream2) == rec["stream2_sha256"]
    assert head(hidden) == rec["hidden_head"] and digest(hidden) == rec["hidden_sha256"]
