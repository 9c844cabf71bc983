"""GPU parity of the 12-bit weight path (muse_fewtok_zip) against the FP64 product of the BF16 weights the form stands
for (the oracle's decoder returns them bit for bit: tests/test_zip12.py) and, bit for bit, against the plain
register-MMA walk on weights with nothing outside the window; with weights salted outside the window the two may
differ by an FP32 rounding of the sum, so those are held to the path's BF16 tolerance instead."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def rel(a, b) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp(min=1e-30))


@pytest.fixture(scope="module")
def proj():
    from llm_inference_engine_b200 import muse_bf16_proj

    return muse_bf16_proj


@pytest.mark.parametrize("layer,shape", [("o", (4096, 4096)), ("unpooler", (4096, 1024)), ("pooler", (1024, 4096)), ("odd", (1000, 2048))])
@pytest.mark.parametrize("m", [1, 5, 8])
def test_zip12_matches_the_plain_walk_and_the_product(proj, layer, shape, m):
    n, k = shape
    g = torch.Generator().manual_seed(100 + m + n)
    w = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
    salted = w.clone()
    salted[0, 0], salted[n - 1, k - 1], salted[n // 2, 7], salted[9 % n, 100] = 0.0, 2.5, -1e-20, float(2.0 ** -30)
    x = torch.randn((m, k), generator=g).bfloat16()
    for weights, exact in ((w, False), (salted, False)):
        state = proj.prepare({layer: weights.to(DEV)}, warmup=False)
        frac = proj.prepare_zip12(state)
        assert layer in frac and frac[layer] < 1e-3
        data = {"x": x.to(DEV), "config": {"layer": layer, "m": m, "n": n, "k": k}}
        outs = [proj.kernel_fn_zip12(data, state) for _ in range(3)]
        torch.cuda.synchronize(DEV)
        assert all(torch.equal(outs[0], o) for o in outs[1:])
        want = x.double() @ weights.double().T
        assert outs[0].dtype == torch.bfloat16 and rel(outs[0].cpu(), want) < 4e-3
        err = (outs[0].cpu().double() - want).abs()
        assert bool((err <= 1e-2 * want.abs() + 1e-2).all())                       # the reference's BF16 tolerance
        plain = proj.kernel_fn(data, state)
        assert rel(outs[0].cpu(), plain.cpu()) < 2e-3


def test_zip12_equals_the_plain_register_walk_bit_for_bit(proj):
    """Weights whose high bytes all sit inside the window (no table): the decode hands the MMAs the same BF16 pairs in
    the same order as the plain kernel of the same shape (32 warps x 4), so the outputs are identical."""
    from llm_inference_engine_b200 import _capi

    n, k, m = 2048, 4096, 8
    g = torch.Generator().manual_seed(7)
    w = (torch.rand((n, k), generator=g) * 0.04 + 0.01).bfloat16() * torch.where(torch.rand((n, k), generator=g) < 0.5, -1.0, 1.0).bfloat16()
    state = proj.prepare({"o": w.to(DEV)}, warmup=False)
    proj.prepare_zip12(state)
    z = state["_zip12"]["o"]
    assert z.exceptions == 0 and z.cap == 0
    x = torch.randn((m, k), generator=g).bfloat16().to(DEV)
    got = proj.kernel_fn_zip12({"x": x, "config": {"layer": "o", "m": m, "n": n, "k": k}}, state)
    plain = torch.empty_like(got)
    lib = _capi.load()
    rc = lib.muse_fewtok_mma(state["o"].data_ptr(), x.data_ptr(), plain.data_ptr(), m, n, k, k, n, 32, 4, 1, state["_status"].data_ptr(),
                             None, torch.cuda.current_stream(DEV).cuda_stream)
    torch.cuda.synchronize(DEV)
    assert rc == 0 and torch.equal(got, plain)


def test_zip12_rejections(proj):
    w = (torch.randn((256, 1024)) * 0.02).bfloat16().to(DEV)
    state = proj.prepare({"o": w}, warmup=False)
    cfg = {"layer": "o", "m": 4, "n": 256, "k": 1024}
    with pytest.raises(KeyError):
        proj.kernel_fn_zip12({"x": torch.zeros((4, 1024), device=DEV, dtype=torch.bfloat16), "config": cfg}, state)
    proj.prepare_zip12(state)
    with pytest.raises(ValueError):
        proj.kernel_fn_zip12({"x": torch.zeros((9, 1024), device=DEV, dtype=torch.bfloat16), "config": dict(cfg, m=9)}, state)
    with pytest.raises(ValueError):
        proj.kernel_fn_zip12({"x": torch.zeros((4, 1024), device=DEV, dtype=torch.bfloat16), "config": dict(cfg, n=128)}, state)
