"""Failure detection on the column-parallel exchange, without any fault: a peer that never shows up.

One GPU plays rank 0 of a world of two; "rank 1" is a set of local buffers that nothing ever writes.
Every wait on a peer is bounded (0.5 s), so the kernels must come back on their own, report the
time-out through the status word, leave this rank's own slice correct and the context usable."""

from __future__ import annotations

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

ST_PEER_ENTER_TIMEOUT, ST_PEER_DONE_TIMEOUT = 32, 64


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _absent_peer(capi, dev, max_tokens: int, n_total: int, n_loc: int, dtype):
    """A descriptor for rank 0 of 2 whose peer is silent memory; returns it with the buffers it points at."""
    keep = {
        "out": [torch.zeros((max_tokens, n_total), device=dev, dtype=dtype) for _ in range(2)],
        "flags": [torch.zeros(32, device=dev, dtype=torch.int32) for _ in range(2)],
        "ll": [torch.zeros((2, 2, capi.LL_TOKENS, n_loc), device=dev, dtype=torch.int32) for _ in range(2)],
    }
    ps = capi.PeerSync()
    ps.world, ps.rank, ps.col0 = 2, 0, 0
    for p in range(2):
        ps.out[p], ps.flags[p], ps.ll[p] = keep["out"][p].data_ptr(), keep["flags"][p].data_ptr(), keep["ll"][p].data_ptr()
    return ps, keep


def test_line_exchange_gives_up_on_a_silent_peer(dev):
    from llm_inference_engine_b200 import _capi

    lib = _capi.load()
    m, n_loc, k = 2, 128, 1024
    g = torch.Generator(device=dev).manual_seed(3)
    w = (torch.randn((n_loc, k), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16)
    ps, keep = _absent_peer(_capi, dev, 32, 2 * n_loc, n_loc, torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    t0 = time.perf_counter()
    rc = lib.muse_fewtok_mma(w.data_ptr(), x.data_ptr(), None, m, n_loc, k, k, 2 * n_loc, 16, 2, 1, status.data_ptr(),
                             ctypes.addressof(ps), torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(dev)
    waited = time.perf_counter() - t0
    assert int(status.item()) == ST_PEER_DONE_TIMEOUT, hex(int(status.item()))
    assert 0.3 < waited < 5.0, waited                      # the bounded wait, not a hang and not a skip
    ref = (x.double() @ w.double().T)
    mine = keep["out"][0][:m, :n_loc].double()
    assert float((mine - ref).norm() / ref.norm()) < 5e-3  # this rank's slice is there
    assert int(keep["flags"][0][16]) == 1                   # the call number advanced: the next call is call 2
    # the context is usable: an ordinary call right after
    out = torch.empty((m, n_loc), device=dev, dtype=torch.bfloat16)
    status.zero_()
    assert lib.muse_fewtok_mma(w.data_ptr(), x.data_ptr(), out.data_ptr(), m, n_loc, k, k, n_loc, 16, 2, 1, status.data_ptr(), None,
                               torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0 and float((out.double() - ref).norm() / ref.norm()) < 5e-3


def test_flag_exchange_gives_up_on_a_silent_peer(dev):
    from llm_inference_engine_b200 import _capi

    lib = _capi.load()
    n_loc, k = 256, 1024
    g = torch.Generator(device=dev).manual_seed(4)
    w = (torch.randn((n_loc, k), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn((1, k), generator=g, device=dev).to(torch.bfloat16)
    ps, keep = _absent_peer(_capi, dev, 32, 2 * n_loc, n_loc, torch.bfloat16)
    status = torch.zeros(1, device=dev, dtype=torch.int32)
    t0 = time.perf_counter()
    rc = lib.muse_gemv1(w.data_ptr(), x.data_ptr(), None, n_loc, k, 0, 4, 4, 0, status.data_ptr(), ctypes.addressof(ps),
                        torch.cuda.current_stream(dev).cuda_stream)
    assert rc == 0
    torch.cuda.synchronize(dev)
    waited = time.perf_counter() - t0
    assert int(status.item()) == ST_PEER_ENTER_TIMEOUT | ST_PEER_DONE_TIMEOUT, hex(int(status.item()))
    assert 0.6 < waited < 5.0, waited                      # two bounded waits: the peer's entry, then its done flag
    ref = (x.double() @ w.double().T)
    assert float((keep["out"][0][:1, :n_loc].double() - ref).norm() / ref.norm()) < 5e-3
    out = torch.empty((1, n_loc), device=dev, dtype=torch.bfloat16)
    status.zero_()
    assert lib.muse_gemv1(w.data_ptr(), x.data_ptr(), out.data_ptr(), n_loc, k, 0, 4, 4, 0, status.data_ptr(), None,
                          torch.cuda.current_stream(dev).cuda_stream) == 0
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0 and float((out.double() - ref).norm() / ref.norm()) < 5e-3
