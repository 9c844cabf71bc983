"""Writes tests/golden/boundary_vectors.json from the reference itself.

    REFERENCE_ROOT=<checkout of Sagor0078/llm-inference-engine> python tests/golden/make_boundary_golden.py

Imports decode_layer/reference.py UNMODIFIED (it runs on the CPU) and applies its own `residual_coefficients`
and `_rms` exactly as its `ref_front` does after the `o` projection (:452-454) to seeded inputs, which the
test regenerates from the same seeds with the oracle's `boundary_inputs`. Recorded per case: digests and leading
values of alpha, beta, stream1 and h; and the same for the post-FFN boundary (the tail of its `ref_back`,
:466-476: stream2 and the next layer's normalised input) on `ffn_boundary_inputs`. tests/test_oracle_golden.py replays the cases through the oracle's
restatement (`residual_coefficients`, `rms`, `attn_boundary`) and demands bit equality.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
CASES = [(1, 4096, 701), (8, 4096, 702), (5, 1024, 703), (32, 8192, 704), (3, 4096, 705)]   # (tokens, hidden, seed)
FFN_CASES = [(1, 4096, 1024, 801), (8, 4096, 1024, 802), (16, 4096, 4096, 803), (5, 2048, 512, 804)]   # (tokens, hidden, f columns, seed)
HEAD = 16


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def head(t: torch.Tensor) -> list[float]:
    return [float(v) for v in t.flatten()[:HEAD].double()]


def main() -> None:
    if "REFERENCE_ROOT" not in os.environ:
        sys.exit("set REFERENCE_ROOT to a checkout of the reference (see the module docstring)")
    sys.dont_write_bytecode = True   # the reference tree is read-only
    sys.path.insert(0, str(Path(os.environ["REFERENCE_ROOT"]) / "decode_layer"))
    sys.path.insert(0, str(ROOT))
    import reference as ref  # noqa: PLC0415
    from oracle import muse_proj_oracle as oracle  # noqa: PLC0415  (only its seeded input generator is used here)

    out = {"torch": torch.__version__, "source": "decode_layer/reference.py, imported unmodified",
           "constants": {k: getattr(ref, k) for k in ("RMS_EPS", "POST_NORM_EPS", "RESIDUAL_TEMPERATURE", "RESIDUAL_GATE_EPS",
                                                      "SLICED_MAX_TOKENS")},
           "cases": []}
    for m, d, seed in CASES:
        stream, attn_out, gate, norm_w = oracle.boundary_inputs(m, d, seed)
        alpha, beta = ref.residual_coefficients(gate)
        stream1 = alpha * stream.float() + beta * ref._rms(attn_out, ref.POST_NORM_EPS)   # ref_front, :453
        h = ref._rms(stream1) * (1.0 + norm_w.float())                                    # :454
        out["cases"].append({"m": m, "d": d, "seed": seed,
                             "inputs_sha256": digest(torch.cat([stream.flatten(), attn_out.float().flatten(), gate, norm_w.float()])),
                             "alpha_sha256": digest(alpha), "beta_sha256": digest(beta), "alpha_head": head(alpha),
                             "stream1_sha256": digest(stream1), "stream1_head": head(stream1),
                             "h_sha256": digest(h), "h_head": head(h)})
    out["ffn_cases"] = []
    for m, d, nf, seed in FFN_CASES:
        stream1, f, gate, post_w, next_w = oracle.ffn_boundary_inputs(m, d, nf, seed)
        full = torch.zeros_like(stream1)                                                   # ref_back, :469-472
        full[:, :nf] = f.float()
        full = full * (1.0 + post_w.float())                                               # :473
        alpha, beta = ref.residual_coefficients(gate)                                      # :474
        stream2 = alpha * stream1 + beta * ref._rms(full, ref.POST_NORM_EPS)               # :475
        hidden = ref._rms(stream2) * (1.0 + next_w.float())                                # :476
        out["ffn_cases"].append({"m": m, "d": d, "nf": nf, "seed": seed,
                                 "inputs_sha256": digest(torch.cat([stream1.flatten(), f.float().flatten(), gate, post_w.float(),
                                                                    next_w.float()])),
                                 "stream2_sha256": digest(stream2), "stream2_head": head(stream2),
                                 "hidden_sha256": digest(hidden), "hidden_head": head(hidden)})
    (HERE / "boundary_vectors.json").write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {HERE / 'boundary_vectors.json'} ({len(out['cases'])} + {len(out['ffn_cases'])} cases)")


if __name__ == "__main__":
    main()
