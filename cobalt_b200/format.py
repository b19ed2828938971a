"""Host-side packer for the tile image the sm_100a kernels stream.

The reference packs its bitmap-sparse matrices row by row
(src/cobaltkernel/pack_cobalt.py:201-250: per-row bitmap, optional per-group
offsets, nibble codes, separate scale/zero arrays).  This packer takes the same
RAW inputs (src/cobaltkernel/quantize_cobalt.py:326-329: occupancy mask, codes
with 0 at pruned positions, fp16 scale and zero per 128-wide group) and emits a
tile-major image instead, so that one warp can pull a 16-row x 512-column tile
with a single bulk copy:

  blob = [tile_off: u32 x (n_tiles + 1), padded to 256 B] [tile 0] [tile 1] ...

  tile (row block rb, column tile ct), w = min(4, G - 4*ct) groups wide:
    mask   16*w segments x 16 B   segment (r, gi) at index r*w + gi; 4 u32 words,
                                  bit b of word j = column 128*(4*ct+gi) + 32*j + b
    sz     16*w x 4 B             {fp16 scale, fp16 zero} of the segment
    codes  bit stream             `bits`-wide codes of the survivors, segment
                                  order, ascending column, little-endian bits
    padded to a multiple of 16 B

``tile_off`` counts 16-byte units from the first tile; 64 zero bytes follow the last tile.  Rows are padded to a
multiple of 16 with empty (all-pruned) rows.  Everything is torch, so packing
runs on whatever device the inputs live on.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

GROUP = 128
TILE_ROWS = 16
TILE_GROUPS = 4
HEADER_ALIGN = 256
TAIL_SLACK = 64          # bytes after the last tile: the decoders read whole words a little past the codes


@dataclass
class TileImage:
    """A packed matrix: one uint8 tensor plus the integers the kernels need."""
    blob: torch.Tensor          # uint8, 1-D, 256-B aligned sections
    K: int
    N: int
    bits: int
    nnz: int
    n_row_blocks: int
    n_col_tiles: int
    header_bytes: int
    max_tile_bytes: int
    max_tile_nnz: int = TILE_ROWS * TILE_GROUPS * GROUP

    @property
    def n_tiles(self) -> int:
        return self.n_row_blocks * self.n_col_tiles

    def meta(self) -> dict:
        return dict(K=self.K, N=self.N, bits=self.bits, nnz=self.nnz, n_row_blocks=self.n_row_blocks,
                    n_col_tiles=self.n_col_tiles, header_bytes=self.header_bytes,
                    max_tile_bytes=self.max_tile_bytes, max_tile_nnz=self.max_tile_nnz, group_size=GROUP)

    @staticmethod
    def from_meta(blob: torch.Tensor, meta: dict) -> "TileImage":
        return TileImage(blob=blob, K=int(meta["K"]), N=int(meta["N"]), bits=int(meta["bits"]),
                         nnz=int(meta["nnz"]), n_row_blocks=int(meta["n_row_blocks"]),
                         n_col_tiles=int(meta["n_col_tiles"]), header_bytes=int(meta["header_bytes"]),
                         max_tile_bytes=int(meta["max_tile_bytes"]),
                         max_tile_nnz=int(meta.get("max_tile_nnz", TILE_ROWS * TILE_GROUPS * GROUP)))

    def algorithmic_bytes(self) -> int:
        """Bitmask + codes + fp16 scale/zero, without padding or the offset table."""
        return self.K * self.N // 8 + (self.bits * self.nnz + 7) // 8 + self.K * (self.N // GROUP) * 4


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def pack_tiles(keep: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor,
               bits: int) -> TileImage:
    """Pack RAW tensors into the tile image.

    keep  bool/uint8/float [K, N]  non-zero = survivor
    q     integer/float    [K, N]  codes in [0, 2**bits) (value at pruned positions ignored)
    scale, zero  fp16      [K, G] or [K, G, 1]
    """
    if bits not in (2, 3, 4):
        raise ValueError(f"bits must be 2, 3 or 4, got {bits}")
    K, N = keep.shape
    if N % GROUP != 0:
        raise ValueError(f"in_features {N} is not a multiple of the group size {GROUP}")
    dev = keep.device
    G = N // GROUP
    RB = (K + TILE_ROWS - 1) // TILE_ROWS
    CT = (G + TILE_GROUPS - 1) // TILE_GROUPS
    Kp, Gp = RB * TILE_ROWS, CT * TILE_GROUPS

    keep_b = keep != 0
    qi = q.to(torch.int64)
    if bool(((qi < 0) | (qi >= (1 << bits)))[keep_b].any()):
        raise ValueError("code outside [0, 2**bits) at a surviving position")
    sc16 = scale.reshape(K, G).to(torch.float16)
    zr16 = zero.reshape(K, G).to(torch.float16)

    # ---- tile-major views: [RB, CT, 16, 4, 128]
    kp = torch.zeros(Kp, Gp * GROUP, dtype=torch.bool, device=dev)
    kp[:K, :N] = keep_b
    qp = torch.zeros(Kp, Gp * GROUP, dtype=torch.uint8, device=dev)
    qp[:K, :N] = qi.to(torch.uint8)
    kt = kp.view(RB, TILE_ROWS, CT, TILE_GROUPS, GROUP).permute(0, 2, 1, 3, 4).contiguous()
    qt = qp.view(RB, TILE_ROWS, CT, TILE_GROUPS, GROUP).permute(0, 2, 1, 3, 4).contiguous()
    del kp, qp

    # ---- tile geometry
    w = torch.full((CT,), TILE_GROUPS, dtype=torch.int64, device=dev)
    w[CT - 1] = G - TILE_GROUPS * (CT - 1)
    nnz_tile = kt.view(RB, CT, -1).sum(-1, dtype=torch.int64)                       # [RB, CT]
    code_bytes = (nnz_tile * bits + 7) // 8
    fixed_bytes = (TILE_ROWS * w * 20).view(1, CT).expand(RB, CT)
    tile_bytes = (fixed_bytes + code_bytes + 15) // 16 * 16
    tb_flat = tile_bytes.reshape(-1)
    tile_base = torch.cumsum(tb_flat, 0) - tb_flat                                  # bytes from first tile
    total_tiles_bytes = int(tb_flat.sum())
    n_tiles = RB * CT
    header_bytes = _round_up(4 * (n_tiles + 1), HEADER_ALIGN)
    nwords = (header_bytes + total_tiles_bytes) // 4 + TAIL_SLACK // 4     # readable slack after the last tile
    words = torch.zeros(nwords + 2, dtype=torch.int64, device=dev)

    # ---- header
    off16 = torch.cat([tile_base, tile_base.new_tensor([total_tiles_bytes])]) // 16
    words[: n_tiles + 1] = off16
    tile_word0 = (header_bytes + tile_base).view(RB, CT) // 4                        # word index of each tile

    # ---- mask words and scale/zero, valid segments only
    sh = torch.arange(32, dtype=torch.int64, device=dev)
    mw = (kt.view(RB, CT, TILE_ROWS, TILE_GROUPS, 4, 32).to(torch.int64) << sh).sum(-1)   # [RB,CT,16,4,4]
    r_idx = torch.arange(TILE_ROWS, device=dev).view(1, 1, TILE_ROWS, 1)
    g_idx = torch.arange(TILE_GROUPS, device=dev).view(1, 1, 1, TILE_GROUPS)
    w_b = w.view(1, CT, 1, 1)
    seg = r_idx * w_b + g_idx                                                       # [1,CT,16,4]
    valid = (g_idx < w_b).expand(RB, CT, TILE_ROWS, TILE_GROUPS)
    seg = seg.expand(RB, CT, TILE_ROWS, TILE_GROUPS)
    base = tile_word0.view(RB, CT, 1, 1)
    j_idx = torch.arange(4, device=dev).view(1, 1, 1, 1, 4)
    mdst = (base + seg * 4).unsqueeze(-1) + j_idx                                   # [RB,CT,16,4,4]
    vmask5 = valid.unsqueeze(-1).expand_as(mdst)
    words[mdst[vmask5]] = mw[vmask5]

    scp = torch.zeros(Kp, Gp, dtype=torch.float16, device=dev)
    zrp = torch.zeros(Kp, Gp, dtype=torch.float16, device=dev)
    scp[:K, :G] = sc16
    zrp[:K, :G] = zr16
    sbits = scp.view(torch.int16).to(torch.int64) & 0xFFFF
    zbits = zrp.view(torch.int16).to(torch.int64) & 0xFFFF
    sz = (sbits | (zbits << 16)).view(RB, TILE_ROWS, CT, TILE_GROUPS).permute(0, 2, 1, 3)   # [RB,CT,16,4]
    sdst = base + TILE_ROWS * w_b * 4 + seg
    words[sdst[valid]] = sz[valid]

    # ---- survivor codes: boolean selection walks (rb, ct, r, gi, column) in order
    codes = qt[kt].to(torch.int64)
    nnz = int(codes.numel())
    if nnz:
        first = torch.cumsum(nnz_tile.reshape(-1), 0) - nnz_tile.reshape(-1)       # first survivor of each tile
        tile_of = torch.repeat_interleave(torch.arange(n_tiles, device=dev), nnz_tile.reshape(-1))
        rank = torch.arange(nnz, device=dev) - first[tile_of]
        code_bit0 = (tile_word0.reshape(-1) * 4 + (TILE_ROWS * w.view(1, CT).expand(RB, CT).reshape(-1) * 20)) * 8
        bitpos = code_bit0[tile_of] + rank * bits
        wi = bitpos >> 5
        shv = bitpos & 31
        val = codes << shv
        words.index_add_(0, wi, val & 0xFFFFFFFF)
        words.index_add_(0, wi + 1, val >> 32)
    words = words[:nwords]
    blob = (words & 0xFFFFFFFF).to(torch.int64)
    # int64 -> little-endian uint32 bytes
    blob32 = torch.where(blob >= 2 ** 31, blob - 2 ** 32, blob).to(torch.int32)
    blob8 = blob32.view(torch.uint8).clone()
    return TileImage(blob=blob8, K=K, N=N, bits=bits, nnz=nnz, n_row_blocks=RB, n_col_tiles=CT,
                     header_bytes=header_bytes, max_tile_bytes=int(tb_flat.max()),
                     max_tile_nnz=int(nnz_tile.max()))


def bytes_to_keep(mask_u8: torch.Tensor, N: int) -> torch.Tensor:
    """RAW ``mask u8[K, N/8]`` (LSB = lowest column) -> bool ``[K, N]``."""
    K = mask_u8.shape[0]
    sh = torch.arange(8, dtype=torch.uint8, device=mask_u8.device)
    return ((mask_u8.view(K, N // 8, 1) >> sh) & 1).view(K, N).bool()


def slice_rows(keep, q, scale, zero, r0: int, r1: int):
    """Output-row shard ``[r0, r1)`` of RAW tensors (column-parallel projections)."""
    return keep[r0:r1], q[r0:r1], scale.reshape(keep.shape[0], -1)[r0:r1], zero.reshape(keep.shape[0], -1)[r0:r1]


def slice_cols(keep, q, scale, zero, c0: int, c1: int):
    """Input-column shard ``[c0, c1)`` of RAW tensors (row-parallel projections).
    The cut must fall on group boundaries so that no scale/zero group straddles ranks."""
    if c0 % GROUP or c1 % GROUP:
        raise ValueError(f"column shard [{c0}, {c1}) is not aligned to the group size {GROUP}")
    K = keep.shape[0]
    return (keep[:, c0:c1], q[:, c0:c1], scale.reshape(K, -1)[:, c0 // GROUP: c1 // GROUP],
            zero.reshape(K, -1)[:, c0 // GROUP: c1 // GROUP])
