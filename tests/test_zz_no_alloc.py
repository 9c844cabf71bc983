"""muse_skinny_tc_noalloc (split-K scratch inside the library, for hosts that may not allocate device
memory) against muse_skinny_tc with a caller-owned workspace, through the C ABI: equal results on two
calls in a row, refusal beyond the stated capacity. Sorts last so that a run that stops at the first
failure has run every other test; passes alone in a fresh process too."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(lib, dev, m, n, k, hilo, seed):
    from llm_inference_engine_b200._capi import TensorMap

    g = torch.Generator(device=dev).manual_seed(seed)
    wf = torch.randn((n, k), generator=g, device=dev) * 0.02
    x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
    if hilo:
        hi = wf.to(torch.bfloat16)
        lo = (wf - hi.float()).to(torch.bfloat16)
        keep = (hi, lo)
    else:
        keep = (wf.to(torch.bfloat16),)
    maps = tuple(TensorMap.for_matrix(t.data_ptr(), n, k, k * 2, 128) for t in keep)
    return x, keep, maps


# (m, n, k, ntok, cluster, groups, stages, hilo): groups > 1, so the scratch array is really used
CASES = [
    (8, 1024, 4096, 16, 2, 9, 3, False),
    (32, 4096, 1024, 32, 1, 4, 4, False),
    (32, 256, 4096, 32, 1, 37, 2, True),
    (100, 1024, 2048, 128, 4, 2, 3, False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "m{}_n{}_k{}_cl{}_gr{}".format(c[0], c[1], c[2], c[4], c[5]))
def test_noalloc_matches_ordinary_entry_point_twice_in_a_row(case):
    from llm_inference_engine_b200 import _capi

    m, n, k, ntok, cluster, groups, stages, hilo = case
    lib = _capi.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    x, keep, maps = _setup(lib, dev, m, n, k, hilo, seed=m + n)
    lo_ptr = maps[1].ptr if hilo else None
    odt = torch.float32 if hilo else torch.bfloat16
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    assert lib.muse_skinny_ws_floats(m, n, ntok) <= lib.muse_static_scratch_floats()
    assert lib.muse_skinny_tiles(m, n, ntok) <= lib.muse_static_scratch_tiles()

    # the ordinary entry point, with a workspace this test owns
    ws = torch.zeros(lib.muse_skinny_ws_floats(m, n, ntok), device=dev, dtype=torch.float32)
    cnt = torch.zeros(lib.muse_skinny_tiles(m, n, ntok), device=dev, dtype=torch.int32)
    want = torch.full((m, n), float("nan"), device=dev, dtype=odt)
    _capi.check(lib.muse_skinny_tc(maps[0].ptr, lo_ptr, x.data_ptr(), want.data_ptr(), ws.data_ptr(), cnt.data_ptr(),
                                   status.data_ptr(), m, n, k, k, n, ntok, cluster, groups, stages, int(hilo), None, stream),
                "muse_skinny_tc")
    torch.cuda.synchronize(dev)
    exact = x.double() @ (keep[0].double() + (keep[1].double() if hilo else 0)).T
    assert float((want.double() - exact).norm() / exact.norm()) < (2e-5 if hilo else 5e-3)

    for call in (1, 2):
        got = torch.full((m, n), float("nan"), device=dev, dtype=odt)
        _capi.check(lib.muse_skinny_tc_noalloc(maps[0].ptr, lo_ptr, x.data_ptr(), got.data_ptr(), status.data_ptr(), m, n,
                                               k, k, n, ntok, cluster, groups, stages, int(hilo), stream),
                    f"muse_skinny_tc_noalloc (call {call})")
        torch.cuda.synchronize(dev)
        assert int(status.item()) == 0
        # split-K sums meet through FP32 atomics whose order varies: the tolerance of the other GPU tests
        if hilo:
            assert float((got.double() - want.double()).norm() / want.double().norm()) < 1e-5, f"call {call}"
        else:
            assert torch.allclose(got.float(), want.float(), rtol=1e-2, atol=1e-3), f"call {call}"


def test_noalloc_refuses_shapes_beyond_its_scratch():
    from llm_inference_engine_b200 import _capi

    lib = _capi.load()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    m, n, k, ntok = 256, 12288, 4096, 256          # 96 tiles x 128 x 256 floats = 3 Mi > 1 Mi
    assert lib.muse_skinny_ws_floats(m, n, ntok) > lib.muse_static_scratch_floats()
    x, keep, maps = _setup(lib, dev, m, n, k, False, seed=1)
    out = torch.zeros((m, n), device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    rc = lib.muse_skinny_tc_noalloc(maps[0].ptr, None, x.data_ptr(), out.data_ptr(), status.data_ptr(), m, n, k, k, n,
                                    ntok, 1, 2, 3, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -20                                 # MUSE_ERR_STATIC_SCRATCH: nothing was launched
    torch.cuda.synchronize(dev)
    assert float(out.abs().max()) == 0.0
    # a rejected argument (13 stages) is refused before the clears of the shared array are enqueued
    rc = lib.muse_skinny_tc_noalloc(maps[0].ptr, None, x.data_ptr(), out.data_ptr(), status.data_ptr(), 8, 1024, k, k, n,
                                    16, 1, 2, 13, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == -5
    # with one cluster per tile the scratch is not used, so the same large shape runs
    rc = lib.muse_skinny_tc_noalloc(maps[0].ptr, None, x.data_ptr(), out.data_ptr(), status.data_ptr(), m, n, k, k, n,
                                    ntok, 1, 1, 3, 0, torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(dev)
    exact = x.double() @ keep[0].double().T
    assert float((out.double() - exact).norm() / exact.norm()) < 5e-3 and int(status.item()) == 0
