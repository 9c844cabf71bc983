"""The lossless 12-bit weight form read by muse_fewtok_zip (the reference author's format, bf16_proj/probe18.py:332-362
`_zip`, laid out for the register-MMA walk): per BF16 weight the raw low byte and a 4-bit code (sign, index of the
high byte in an 8-value window starting at `base`); weights whose high byte is outside the window are coded as the
window's smallest magnitude and listed, with their true value, in a per-row-group table.

Layouts (K % 128 == 0), chosen so that lane q of a warp (q = lane & 3, the lane's 8 weights of a 32-weight piece
are k = 32 piece + 8 q .. + 7) still loads 16-byte vectors:
  low   uint8 [N, K]:     per 64-byte span = two pieces: q-major, then piece, then the 8 bytes
  code  uint8 [N, K / 2]: per 64-byte span = four pieces: q-major, then piece, then 4 bytes; byte i = code of the
                          lane's weight i | code of weight i + 4 << 4
  table int32 [groups, cap, 2]: {row in group << 16 | column, FP32 bits of the true weight}, unused {-1, 0} last
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

MAX_CAP = 64          # ZIP_MAX_CAP of csrc/fewtok_zip.cu
WINDOW = 8


@dataclass
class Zip12:
    low: torch.Tensor      # uint8 [N, K]
    code: torch.Tensor     # uint8 [N, K // 2]
    table: torch.Tensor    # int32 [groups, cap, 2] (cap may be 0: then an empty tensor)
    base: int
    cap: int
    n: int
    k: int
    exceptions: int

    @property
    def nbytes(self) -> int:
        return self.low.numel() + self.code.numel() + self.table.numel() * 4


def encode(w: torch.Tensor) -> Zip12 | None:
    """BF16 W [N, K] -> Zip12 on W's device, or None where the format does not apply (K not a multiple of 128, more
    than 65535 columns, or a row group with more than MAX_CAP weights outside the window)."""
    if w.dtype != torch.bfloat16 or w.dim() != 2:
        raise TypeError("encode() takes a BF16 matrix")
    n, k = w.shape
    if k % 128 or k > 65535:
        return None
    bits = w.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    low = bits & 0xFF
    sign, top = bits >> 15, (bits >> 8) & 0x7F
    counts = torch.bincount(top.flatten(), minlength=128)
    base = int(counts.unfold(0, WINDOW, 1).sum(-1).argmax())        # the window that holds the most weights
    idx = top - base
    ok = (idx >= 0) & (idx < WINDOW)
    code = torch.where(ok, (sign << 3) | idx, sign << 3)
    low = torch.where(ok, low, torch.zeros_like(low))
    # low plane: [N, K/64, piece 2, q 4, 8] -> q-major
    low_p = low.to(torch.uint8).view(n, k // 64, 2, 4, 8).permute(0, 1, 3, 2, 4).contiguous().view(n, k)
    # code plane: per lane-piece [half 2, i 4] -> 4 bytes; then [N, K/128, piece 4, q 4, 4] -> q-major
    c = code.view(n, k // 32, 4, 2, 4)
    nb = (c[:, :, :, 0, :] | (c[:, :, :, 1, :] << 4)).to(torch.uint8)           # [N, K/32, q, 4]
    code_p = nb.view(n, k // 128, 4, 4, 4).permute(0, 1, 3, 2, 4).contiguous().view(n, k // 2)
    # the table
    groups = (n + 7) // 8
    rows, cols = (~ok).nonzero(as_tuple=True)
    total = int(rows.numel())
    cap = 0
    table = torch.empty((groups, 0, 2), dtype=torch.int32, device=w.device)
    if total:
        grp = rows // 8
        per = torch.bincount(grp, minlength=groups)
        cap = int(per.max())
        cap = -(-cap // 4) * 4
        if cap > MAX_CAP:
            return None
        order = torch.argsort(grp, stable=True)
        rows, cols, grp = rows[order], cols[order], grp[order]
        start = torch.cumsum(per, 0) - per
        slot = torch.arange(total, device=w.device) - start[grp]
        table = torch.full((groups, cap, 2), -1, dtype=torch.int32, device=w.device)
        table[:, :, 1] = 0
        table[grp, slot, 0] = (((rows % 8) << 16) | cols).to(torch.int32)
        table[grp, slot, 1] = w[rows, cols].float().view(torch.int32)
    return Zip12(low_p, code_p, table.contiguous(), base, cap, n, k, total)
