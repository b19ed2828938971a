"""Offline compression of a dense weight: keep mask + low-bit survivors.

This is compress-time code (runs once per layer, on CPU or GPU tensors alike);
the hot path only ever sees its output.  It reproduces the reference recipe:

* keep mask  -- column-balanced Wanda, src/cobaltkernel/cobalt_math.py:15-32
  (same selection as src/nosink.py:264-299): score ``|W| * norm``, divide each
  row by its ``int(N*sp)``-th smallest score, rescale, divide each column by its
  ``int(K*sp)``-th smallest score to the power ``beta``, rescale, prune the
  ``int(K*N*sp)`` smallest scores with one global threshold (strict ``>``).
* codes      -- asymmetric min-max round-to-nearest per 128-wide group with the
  hull over survivors, src/cobaltkernel/cobalt_math.py:144-168; codes zeroed at
  pruned positions (src/nosink.py:1319); scale and zero stored as fp16
  (src/cobaltkernel/quantize_cobalt.py:441-442).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .format import GROUP


@dataclass
class SparseQuantConfig:
    """Knobs of the compression recipe (reference: ``meta`` dict of
    benchmarks/benchmark_suite.py:1178-1198 plus the mask parameters of
    src/cobaltkernel/cobalt_math.py:336-394)."""
    bits: int = 4
    sparsity: float = 0.5
    beta: float = 0.5
    group_size: int = GROUP

    def validate(self):
        if self.bits not in (2, 3, 4):
            raise ValueError("bits must be 2, 3 or 4")
        if not (0.0 <= self.sparsity < 1.0):
            raise ValueError("sparsity must be in [0, 1)")
        if self.group_size != GROUP:
            raise ValueError(f"group_size must be {GROUP}")


def _normalise_by_max(score: torch.Tensor) -> torch.Tensor:
    top = score.amax()
    if bool(torch.isfinite(top)) and bool(top > 0):
        return score / top
    return torch.nan_to_num(score, nan=0.0, posinf=0.0, neginf=0.0)


def _global_kth_smallest(flat: torch.Tensor, k: int) -> torch.Tensor:
    if flat.numel() <= 32_000_000:
        return torch.kthvalue(flat, k).values
    # Above 32 M elements the reference brackets the k-th smallest value by bisection on
    # the value range and then takes the largest element not above the bracket.
    lo, hi = flat.min().float(), flat.max().float()
    for _ in range(64):
        mid = (lo + hi) * 0.5
        if not bool(torch.isfinite(mid)) or bool(mid <= lo) or bool(mid >= hi):
            break
        if int((flat <= mid).sum()) < k:
            lo = mid
        else:
            hi = mid
    below = flat[flat <= hi]
    return below.max() if below.numel() else hi


def keep_mask(weight: torch.Tensor, act_norm: torch.Tensor, sparsity: float, beta: float) -> torch.Tensor:
    """bool ``[K, N]`` keep mask (True = survivor)."""
    K, N = weight.shape
    if sparsity <= 0.0:
        return torch.ones(K, N, dtype=torch.bool, device=weight.device)
    score = weight.float().abs() * act_norm.float().view(1, -1)
    n_row, n_col = int(N * sparsity), int(K * sparsity)
    if n_row > 0:
        row_q = torch.kthvalue(score, n_row, dim=1, keepdim=True).values
        score = _normalise_by_max(score / row_q.clamp(min=1e-30))
    if beta > 0 and n_col > 0:
        col_q = torch.kthvalue(score, n_col, dim=0, keepdim=True).values
        score = _normalise_by_max(score / col_q.clamp(min=1e-30).pow(beta))
    flat = score.reshape(-1)
    threshold = _global_kth_smallest(flat, int(K * N * sparsity))
    return (flat > threshold).view(K, N)


def quantize_survivors(weight: torch.Tensor, keep: torch.Tensor, bits: int, group_size: int = GROUP):
    """Group RTN over survivors.  Returns ``q uint8[K,N]`` (0 at pruned),
    ``scale f16[K,G]``, ``zero f16[K,G]``."""
    K, N = weight.shape
    if N % group_size:
        raise ValueError(f"in_features {N} is not a multiple of group_size {group_size}")
    G = N // group_size
    top_code = (1 << bits) - 1
    wg = weight.float().view(K, G, group_size)
    kg = keep.view(K, G, group_size)
    limit = torch.finfo(torch.float32).max
    lo = wg.masked_fill(~kg, limit).amin(-1, keepdim=True)
    hi = wg.masked_fill(~kg, -limit).amax(-1, keepdim=True)
    has_any = kg.any(-1, keepdim=True)
    lo = lo * has_any
    hi = hi * has_any
    scale = (hi - lo).clamp(min=1e-4) / torch.full_like(hi, float(top_code))     # tensor / tensor: see quantize_dense
    zero = -torch.round(lo / scale)
    q = torch.clamp(torch.round(wg / scale + zero), 0, top_code).view(K, N)
    q = (q * keep).to(torch.uint8)
    return q, scale.view(K, G).half(), zero.view(K, G).half()


def quantize_dense(weight: torch.Tensor, bits: int, group_size: int = GROUP):
    """Plain asymmetric min-max RTN per 128-wide group, no mask: the recipe the reference applies to the (tied)
    embedding / head matrix, which is read as a lookup (src/cobaltkernel/pack_cobalt.py:375-386).  The hull always
    contains 0, so the zero point is an integer code in ``[0, 2**bits)``.  Returns ``q uint8[K,N]``, ``scale f16[K,G]``,
    ``zero f16[K,G]`` (the reference stores the zero point as uint8; fp16 holds the same integers)."""
    K, N = weight.shape
    if N % group_size:
        raise ValueError(f"in_features {N} is not a multiple of group_size {group_size}")
    G = N // group_size
    top_code = (1 << bits) - 1
    wg = weight.float().view(K, G, group_size)
    lo = wg.amin(-1).clamp(max=0.0)
    hi = wg.amax(-1).clamp(min=0.0)
    # tensor / tensor is an IEEE division on every device; tensor / python-number is a multiplication by the rounded
    # reciprocal on CUDA, which moves the scale by an ulp and with it 0.7 % of the codes
    scale = ((hi - lo) / torch.full_like(hi, float(top_code))).clamp(min=1e-12)
    zero = torch.round(-lo / scale).clamp(0, top_code)
    q = torch.clamp(torch.round(wg / scale.unsqueeze(-1) + zero.unsqueeze(-1)), 0, top_code).view(K, N)
    return q.to(torch.uint8), scale.half(), zero.half()


def compress_weight(weight: torch.Tensor, act_norm: torch.Tensor, cfg: SparseQuantConfig):
    """``weight [K,N]`` -> RAW tensors ``(keep bool, q uint8, scale f16, zero f16)``."""
    cfg.validate()
    keep = keep_mask(weight, act_norm, cfg.sparsity, cfg.beta)
    q, scale, zero = quantize_survivors(weight, keep, cfg.bits, cfg.group_size)
    return keep, q, scale, zero
