"""The lossless 12-bit weight form (the reference author's `_zip`, bf16_proj/probe18.py:332-362): the encoder of
llm_inference_engine_b200/zip12.py against the oracle's independent decoder, bit for bit, on Gaussian weights, on
weights salted with values outside any window (zeros, signed zeros, tiny, large, infinities), and on shapes where
the form does not apply."""

from __future__ import annotations

import pytest
import torch

from llm_inference_engine_b200 import zip12


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("n,k,seed", [(1024, 4096, 1), (250, 1024, 2), (64, 128, 3), (9, 256, 4), (4096, 1024, 5)])
def test_round_trip_is_exact(oracle, n, k, seed):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn((n, k), generator=g) * 0.02).bfloat16()
    w[0, 0], w[min(1, n - 1), 5], w[n - 1, k - 1], w[n // 2, 3] = 0.0, -0.0, 1e-30, 3.0
    w[n // 3, 17] = float("inf")
    z = zip12.encode(w)
    assert z is not None and z.low.shape == (n, k) and z.code.shape == (n, k // 2) and z.cap % 4 == 0
    assert z.table.shape == ((n + 7) // 8, z.cap, 2) and z.exceptions >= 5
    back = oracle.zip12_decode(z.low, z.code, z.table, z.base)
    assert torch.equal(_bits(back), _bits(w))
    assert z.nbytes < 0.78 * n * k * 2                                  # 12 bits a weight and a small table


def test_gaussian_weights_need_few_table_entries(oracle):
    """The window of 8 high-byte values holds all but ~1e-4 of Gaussian weights (the reference's figure,
    bf16_proj/LOG.md), at any scale."""
    g = torch.Generator().manual_seed(11)
    for scale in (0.02, 1.0, 3e-4):
        w = (torch.randn((512, 2048), generator=g) * scale).bfloat16()
        z = zip12.encode(w)
        assert z.exceptions / w.numel() < 3e-4 and z.cap <= 16
        assert torch.equal(_bits(oracle.zip12_decode(z.low, z.code, z.table, z.base)), _bits(w))


def test_table_entries_are_sorted_by_group_and_padded(oracle):
    w = torch.full((16, 128), 0.01).bfloat16()
    w[3, 7], w[3, 100], w[12, 0] = 0.0, 1e-20, -0.0
    z = zip12.encode(w)
    t = z.table
    assert z.cap == 4 and z.exceptions == 3
    assert (t[0, :2, 0] >= 0).all() and (t[0, 2:, 0] == -1).all() and (t[1, :1, 0] >= 0).all() and (t[1, 1:, 0] == -1).all()
    assert sorted(int(v) for v in t[0, :2, 0]) == [(3 << 16) | 7, (3 << 16) | 100] and int(t[1, 0, 0]) == (4 << 16)
    assert torch.equal(_bits(oracle.zip12_decode(z.low, z.code, z.table, z.base)), _bits(w))


def test_shapes_the_form_does_not_cover():
    assert zip12.encode(torch.zeros((8, 96)).bfloat16()) is None        # K not a multiple of 128
    flat = torch.zeros((8, 1024))
    flat[0, :200] = torch.logspace(-30, 30, 200)                        # one row group with 200 values spread over 200 binades
    assert zip12.encode(flat.bfloat16()) is None
    with pytest.raises(TypeError):
        zip12.encode(torch.zeros((8, 128)))
