"""Host-side helpers of the decode-step kernels (`csrc/decode.cu`).

The decode GEMM streams every weight exactly once, so its speed is the speed of the DRAM reads.
A `[rows, k]` row-major weight read through a 128-row x 64-column TMA box is 128 pieces of 128
bytes that lie one full weight row (4 KiB and more) apart; the same tile stored contiguously is
one 16 KiB burst.  `pack_weight` makes that tile-by-tile copy once, when a serving engine is built.

The reference keeps `nn.Linear` weights row-major and decodes through eager `F.linear`
(reference warpstate/model.py:222-274); it has no serving-side weight layout.
"""
from __future__ import annotations

import torch

TILE_ROWS = 128
TILE_COLS = 64


def pack_weight(w: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """``w [rows, k]`` -> BF16 ``[slabs, ceil(k/64), 128, 64]`` with every tile contiguous.

    Plain projections: slab ``s`` holds weight rows ``128 s .. 128 s + 127`` (zero padded past the
    last row).  ``swiglu=True``: ``w`` is ``[2 h, k]`` (``h`` up rows, then ``h`` gate rows, ``h`` a
    multiple of 64) and slab ``s`` holds up rows ``64 s .. 64 s + 63`` followed by the gate rows of
    the same hidden units, which is the pairing the SwiGLU epilogue of the kernel expects.
    Columns are zero padded to a multiple of 64.
    """
    if w.dim() != 2:
        raise ValueError("pack_weight expects a 2-D weight")
    w = w.detach().to(torch.bfloat16)
    rows, k = w.shape
    k_blocks = (k + TILE_COLS - 1) // TILE_COLS
    if k_blocks * TILE_COLS != k:
        w = torch.nn.functional.pad(w, (0, k_blocks * TILE_COLS - k))
    if swiglu:
        if rows % 2 != 0 or (rows // 2) % 64 != 0:
            raise ValueError("a SwiGLU weight needs 2*h rows with h a multiple of 64")
        h = rows // 2
        up = w[:h].view(h // 64, 64, k_blocks, TILE_COLS)
        gate = w[h:].view(h // 64, 64, k_blocks, TILE_COLS)
        tiles = torch.cat([up, gate], dim=1)
    else:
        slabs = (rows + TILE_ROWS - 1) // TILE_ROWS
        if slabs * TILE_ROWS != rows:
            w = torch.nn.functional.pad(w, (0, 0, 0, slabs * TILE_ROWS - rows))
        tiles = w.view(slabs, TILE_ROWS, k_blocks, TILE_COLS)
    return tiles.permute(0, 2, 1, 3).contiguous()


def unpack_weight(packed: torch.Tensor, rows: int, k: int, swiglu: bool = False) -> torch.Tensor:
    """Inverse of `pack_weight` (for tests and for reading a weight back out of an engine)."""
    slabs, k_blocks, tile_rows, tile_cols = packed.shape
    tiles = packed.permute(0, 2, 1, 3)
    if swiglu:
        h = rows // 2
        up = tiles[:, :64].reshape(h, k_blocks * tile_cols)
        gate = tiles[:, 64:].reshape(h, k_blocks * tile_cols)
        return torch.cat([up, gate], dim=0)[:, :k].contiguous()
    return tiles.reshape(slabs * tile_rows, k_blocks * tile_cols)[:rows, :k].contiguous()
