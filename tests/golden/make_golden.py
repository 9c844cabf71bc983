"""Writes tests/golden/reference_vectors.json from the reference itself.

Run where a checkout of the reference is available, naming it in REFERENCE_ROOT:

    REFERENCE_ROOT=<checkout of Sagor0078/llm-inference-engine> python tests/golden/make_golden.py

It imports bf16_proj/reference.py + checks.py UNMODIFIED (CPU generators, FP64 product) and
records, for a fixed list of cases: digests and leading values of the generated weights and inputs,
probe-row indices, leading values of the reference outputs, the verdict + message of
check_implementation / compare on exact and on deliberately perturbed outputs, and the
speed-of-light floor. tests/test_oracle_golden.py replays the same cases through the oracle
restatement and demands equality. Nothing at test time reads the reference checkout.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
if "REFERENCE_ROOT" not in os.environ:
    sys.exit("set REFERENCE_ROOT to a checkout of the reference (see the module docstring)")
REF_ROOT = Path(os.environ["REFERENCE_ROOT"])

INPUT_CASES = [  # (layer, m, seed, dist)
    ("qkv_gate", 1, 11, "normal"), ("qkv_gate", 8, 12, "normal"), ("qkv_gate", 32, 13, "outliers"),
    ("o", 1, 21, "normal"), ("o", 16, 22, "outliers"), ("o", 32, 23, "normal"),
    ("pooler", 1, 31, "normal"), ("pooler", 8, 32, "outliers"), ("pooler", 128, 33, "normal"),
    ("unpooler", 1, 41, "normal"), ("unpooler", 8, 42, "normal"), ("unpooler", 16, 43, "normal"),
    ("unpooler", 256, 44, "outliers"),
    ("router", 1, 51, "normal"), ("router", 8, 52, "normal"), ("router", 32, 53, "outliers"),
    ("router", 256, 54, "normal"),
]
HEAD = 16  # leading values kept per tensor


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def head(t: torch.Tensor) -> list[float]:
    return [float(v) for v in t.flatten()[:HEAD].double()]


def main() -> None:
    sys.dont_write_bytecode = True  # the reference tree is read-only
    sys.path.insert(0, str(REF_ROOT / "bf16_proj"))
    import checks as ref_checks  # noqa: PLC0415
    import reference as ref  # noqa: PLC0415

    torch.manual_seed(0)
    out: dict = {"torch": torch.__version__, "source": "bf16_proj/reference.py + checks.py, imported unmodified",
                 "constants": {k: getattr(ref, k) for k in
                               ("UNPOOL_SLICE", "SLICED_MAX_TOKENS", "WEIGHTS_SEED", "REL_L2_TOL", "ROUTER_TOL",
                                "PROBE_EVERY", "PROBE_TOL")},
                 "layers": {k: list(v) for k, v in ref.LAYERS.items()},
                 "row_factor": ref_checks.ROW_FACTOR, "row_norm_floor": ref_checks.ROW_NORM_FLOOR}
    weights = ref.generate_weights(ref.WEIGHTS_SEED, device="cpu")
    out["weights"] = {name: {"shape": list(w.shape), "dtype": str(w.dtype), "sha256": digest(w), "head": head(w)}
                      for name, w in weights.items()}

    cases = []
    for layer, m, seed, dist in INPUT_CASES:
        data = ref.generate_input(m, layer, seed, dist, device="cpu")
        want = ref.ref_kernel(data, weights)
        rec = {"layer": layer, "m": m, "seed": seed, "dist": dist, "config": data["config"],
               "x_sha256": digest(data["x"]), "x_head": head(data["x"]),
               "probe_rows": [int(i) for i in ref.probe_rows(data["x"])],
               "ref_dtype": str(want.dtype), "ref_head": head(want), "ref_row_norms": head(want.float().norm(dim=-1)),
               "checks": []}
        # verdicts on: the exact answer, small noise (passes), large noise (fails whole-output),
        # one bad row (fails per-row), a wrong dtype, and a probe row computed from rounded weights.
        g = torch.Generator().manual_seed(seed + 1000)
        noise = torch.randn(want.shape, generator=g)
        scale = want.float().abs().mean()
        variants = {
            "exact": want.clone(),
            "noise_small": (want.float() + 1e-6 * scale * noise).to(want.dtype),
            "noise_large": (want.float() + 0.2 * scale * noise).to(want.dtype),
            "wrong_dtype": want.to(torch.float16),
        }
        tol = ref.ROUTER_TOL if layer in ref.FP32_LAYERS else ref.REL_L2_TOL
        bad_row = want.float().clone()
        bad_row[m // 2] *= 1.0 + 5.5 * tol  # above the per-row limit, below the whole-output one when m > 30
        variants["one_bad_row"] = bad_row.to(want.dtype)
        rows = ref.probe_rows(data["x"])
        if len(rows):
            off = want.float().clone()
            off[rows[0]] *= 1.0 + 4e-3  # passes compare(), fails the probe-row limit
            variants["probe_row_off"] = off.to(want.dtype)
        if layer == "router":
            # what a BF16-only router produces: must fail the probe rows / tolerance
            w_bf = weights["router"].to(torch.bfloat16).double()
            variants["bf16_weights"] = (data["x"].double() @ w_bf[: data["config"]["n"]].T).to(want.dtype)
        for name, candidate in variants.items():
            ok, msg = ref.check_implementation(data, candidate, weights)
            rec["checks"].append({"variant": name, "ok": bool(ok), "msg": msg})
        cases.append(rec)
    out["cases"] = cases

    hw = {"hbm_bytes_per_s": 4.8e12, "bf16_dense_flops_per_s": 989e12}
    out["speed_of_light"] = [{"layer": layer, "m": m, "ns": ref.speed_of_light_ns(m, layer, hw)}
                             for layer in ref.LAYERS for m in (1, 8, 16, 32, 128, 256)]
    out["out_features"] = [{"layer": layer, "m": m, "n": ref.out_features(layer, m)}
                           for layer in ref.LAYERS for m in (1, 8, 9, 256)]
    (HERE / "reference_vectors.json").write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {HERE / 'reference_vectors.json'} ({len(cases)} cases)")


if __name__ == "__main__":
    main()
