"""CPU restatement of the reference's compress -> dequantise -> matmul path.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  Plain torch on the CPU:
the reference's own arithmetic is torch, so the same primitives (``kthvalue``,
round-half-even ``round``, fp32 products, bf16 RNE casts, ``matmul``) are used and
every result can be compared bit for bit.

Index convention (reference: sinq/sparse_quant.py:1463, docs/FORMAT.md:37):
``W[K, N]`` = ``[out_features, in_features]``; quantisation groups are 128 wide and
run along ``N``.
"""
from __future__ import annotations

import math

import numpy as np
import torch

GROUP = 128


# --------------------------------------------------------------------------- mask
def _rescale(imp: torch.Tensor) -> torch.Tensor:
    """Divide by the global maximum when it is finite and positive.

    Follows src/cobaltkernel/cobalt_math.py:66-76."""
    m = imp.amax()
    if torch.isfinite(m) and m > 0:
        return imp / m
    return torch.nan_to_num(imp, nan=0.0, posinf=0.0, neginf=0.0)


def _kth_global(flat: torch.Tensor, k: int) -> torch.Tensor:
    """k-th smallest (1-based) of a flat tensor; bisection above 32 M elements.

    Follows src/cobaltkernel/cobalt_math.py:79-101 (same branch point, same
    bracket refinement, same final "largest value <= hi" selection)."""
    n = flat.numel()
    if n <= 32_000_000:
        return torch.kthvalue(flat, k).values
    lo = flat.min().float()
    hi = flat.max().float()
    for _ in range(64):
        mid = (lo + hi) * 0.5
        if not torch.isfinite(mid) or mid <= lo or mid >= hi:
            break
        cnt = (flat <= mid).sum()
        if cnt.item() < k:
            lo = mid
        else:
            hi = mid
    sel = flat[flat <= hi]
    return sel.max() if sel.numel() else hi


def balanced_keepmask(imp: torch.Tensor, sparsity: float, col_exp: float) -> torch.Tensor:
    """Column-balanced Wanda keep mask: row quantile, column quantile**beta, one
    global threshold, strict ``>``.

    Follows src/cobaltkernel/cobalt_math.py:15-32.  ``imp`` is ``|W| * norm[j]``
    in fp32; the result is a float {0,1} tensor of the same shape."""
    K, N = imp.shape
    if sparsity <= 0.0:
        return torch.ones_like(imp)
    kr, kc = int(N * sparsity), int(K * sparsity)
    if kr > 0:
        imp = imp / torch.kthvalue(imp, kr, dim=1, keepdim=True).values.clamp(min=1e-30)
        imp = _rescale(imp)
    if col_exp > 0 and kc > 0:
        imp = imp / torch.kthvalue(imp, kc, dim=0, keepdim=True).values.clamp(min=1e-30).pow(col_exp)
        imp = _rescale(imp)
    n_prune = int(K * N * sparsity)
    flat = imp.reshape(-1)
    thr = _kth_global(flat, n_prune)
    return (flat > thr).view(K, N).float()


# --------------------------------------------------------------------------- RTN
def group_rtn_survivor(W: torch.Tensor, keep: torch.Tensor, nbits: int, gsize: int = GROUP):
    """Asymmetric unsigned min-max group RTN with the hull taken over survivors.

    Follows src/cobaltkernel/cobalt_math.py:144-168 with ``hull="survivor"``:
    empty group -> min = max = 0; ``scale = (max-min).clamp(1e-4)/n_levels``;
    ``zero = -round(min/scale)`` (not clamped); codes are computed for every
    position and clamped to ``[0, n_levels]``.  Returns fp32 ``q[K,N]``,
    ``scale[K,G]``, ``zero[K,G]``."""
    K, N = W.shape
    assert N % gsize == 0
    ng = N // gsize
    Wg = W.view(K, ng, gsize)
    n_levels = 2 ** nbits - 1
    Mg = keep.view(K, ng, gsize).bool()
    big = torch.finfo(torch.float32).max
    w_min = torch.where(Mg, Wg, torch.full_like(Wg, big)).amin(-1, keepdim=True)
    w_max = torch.where(Mg, Wg, torch.full_like(Wg, -big)).amax(-1, keepdim=True)
    empty = ~Mg.any(-1, keepdim=True)
    w_min = torch.where(empty, torch.zeros_like(w_min), w_min)
    w_max = torch.where(empty, torch.zeros_like(w_max), w_max)
    scale = (w_max - w_min).clamp(min=1e-4) / n_levels
    zero = -torch.round(w_min / scale)
    q = torch.clamp(torch.round(Wg / scale + zero), 0, n_levels)
    return q.view(K, N), scale.view(K, ng), zero.view(K, ng)


def rtn_dense(W: torch.Tensor, nbits: int, gsize: int = GROUP):
    """Restatement of ``rtn_dense`` (src/cobaltkernel/pack_cobalt.py:375-386): asymmetric group min-max RTN with a
    0-inclusive hull, no mask - the recipe of the tied embedding / head.  Returns fp32 codes, fp16 scale, uint8 zero."""
    K, N = W.shape
    G = N // gsize
    nl = (1 << nbits) - 1
    Wg = W.float().view(K, G, gsize)
    wmin = Wg.amin(-1).clamp(max=0.0)
    wmax = Wg.amax(-1).clamp(min=0.0)
    scale = ((wmax - wmin) / nl).clamp(min=1e-12)
    zero = torch.round(-wmin / scale).clamp(0, nl)
    q = torch.clamp(torch.round(Wg / scale.unsqueeze(-1) + zero.unsqueeze(-1)), 0, nl).view(K, N)
    return q, scale.half(), zero.to(torch.uint8)


def compress(W: torch.Tensor, act_norm: torch.Tensor, nbits: int, sparsity: float,
             beta: float = 0.5, gsize: int = GROUP):
    """The whole recipe of the benchmark configurations for one matrix.

    importance ``|W| * norm`` -> balanced keep mask -> survivor-hull RTN ->
    ``q *= keep`` (src/nosink.py:1319) -> scale/zero stored as fp16
    (src/cobaltkernel/quantize_cobalt.py:441-442).  Returns the RAW schema of
    src/cobaltkernel/quantize_cobalt.py:326-329 as torch tensors:
    ``keep bool[K,N]``, ``q uint8[K,N]`` (0 at pruned), ``scale f16[K,G]``,
    ``zero f16[K,G]``."""
    W = W.float()
    keep = balanced_keepmask(W.abs() * act_norm.float().view(1, -1), sparsity, beta)
    q, sc, zr = group_rtn_survivor(W, keep, nbits, gsize)
    q = q * keep
    return keep.bool(), q.to(torch.uint8), sc.half(), zr.half()


# --------------------------------------------------------------------------- dequant + linear
def dequantize(q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, keep: torch.Tensor,
               scale2: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``((Q - z) * s) * scale2 * mask`` in exactly that order.

    Follows sinq/sparse_quant.py:1657-1681 (group-wise branch).  ``scale`` and
    ``zero`` are the stored fp16 values ``[K,G]`` (or ``[K,G,1]``)."""
    K, N = q.shape
    Q = q.float()
    s1 = scale.float().reshape(K, -1, 1)
    z = zero.float().reshape(K, -1, 1)
    ng = s1.shape[1]
    W = ((Q.view(K, ng, N // ng) - z) * s1).view(K, N)
    s2 = torch.ones(N, device=q.device) if scale2 is None else scale2.float()
    W = W * s2
    W = W * keep.float()
    return W


def linear_forward(x: torch.Tensor, q, scale, zero, keep, scale2=None, bias=None) -> torch.Tensor:
    """``SparseQuantLinear.forward``: dequantise, cast to ``x.dtype``, ``x @ W.T``
    (+ bias).  Follows benchmarks/benchmark_suite.py:1200-1217."""
    W = dequantize(q, scale, zero, keep, scale2).to(x.dtype)
    out = torch.matmul(x, W.t())
    if bias is not None:
        out = out + bias
    return out


# --------------------------------------------------------------------------- seeded inputs
def seeded_matrix(K: int, N: int, seed: int):
    """Weights N(0, 0.02) stored as fp16 and activation norms |N(0,1)| + 0.1, the
    synthetic stand-ins the benchmark configurations prescribe."""
    g = torch.Generator().manual_seed(seed)
    W = (torch.randn(K, N, generator=g) * 0.02).half().float()
    norm = torch.randn(N, generator=g).abs() + 0.1
    return W, norm


def seeded_activation(M: int, N: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(M, N, generator=g).to(torch.bfloat16)


def synth_raw(K: int, N: int, sparsity: float, bits: int, seed: int, balanced: bool = True):
    """Random RAW-schema matrix in the shape of the reference's kernel-test
    generator: row/column-normalised uniform importances with one global
    threshold, uniform random codes, scale in [0.001, 0.011), integer zero in
    [0, n_levels], column scale in [0.5, 2).

    Follows src/cobaltkernel/pack_cobalt.py:338-371 (``block = 0`` branch),
    including the order in which the generator is consumed."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    imp = torch.rand(K, N, generator=g)
    if balanced:
        kr = max(1, int(N * sparsity))
        kc = max(1, int(K * sparsity))
        imp = imp / torch.kthvalue(imp, kr, dim=1, keepdim=True).values.clamp(min=1e-30)
        imp = imp / torch.kthvalue(imp, kc, dim=0, keepdim=True).values.clamp(min=1e-30).pow(0.5)
    thr = torch.kthvalue(imp.reshape(-1), max(1, int(K * N * sparsity))).values
    keep = imp > thr
    G = N // GROUP
    nl = (1 << bits) - 1
    q = torch.randint(0, nl + 1, (K, N), generator=g, dtype=torch.uint8)
    q = q * keep.to(torch.uint8)
    scale = (torch.rand(K, G, generator=g) * 0.01 + 0.001).half()
    zero = torch.randint(0, nl + 1, (K, G), generator=g).half()
    col_scale = (torch.rand(N, generator=g) * 1.5 + 0.5).half()
    return dict(keep=keep, q=q, scale=scale, zero=zero, col_scale=col_scale)


def mask_to_bytes(keep: torch.Tensor) -> torch.Tensor:
    """RAW ``mask u8[K, N/8]``, LSB = lowest column
    (src/cobaltkernel/quantize_cobalt.py:326, pack_cobalt.py:368-369)."""
    K, N = keep.shape
    sh = torch.arange(8, dtype=torch.uint8)
    return (keep.view(K, N // 8, 8).to(torch.uint8) << sh).sum(-1).to(torch.uint8)


# --------------------------------------------------------------------------- packed-tile reader
def unpack_tiles_numpy(blob: np.ndarray, K: int, N: int, bits: int):
    """Independent, loop-based reader of the packed tile image the CUDA kernels
    stream (layout described in ``include/cobalt_b200.h``).  Written from the
    layout description alone so that it can check the packer and the
    ``cobalt_unpack`` kernel; slow, use on small matrices.

    Returns ``codes u8[K,N]``, ``keep bool[K,N]``, ``scale f16[K,G]``, ``zero f16[K,G]``."""
    assert blob.dtype == np.uint8
    G = N // GROUP
    RB = (K + 15) // 16
    CT = (G + 3) // 4
    ntiles = RB * CT
    hdr = 256 * ((4 * (ntiles + 1) + 255) // 256)
    tile_off = blob[: 4 * (ntiles + 1)].view(np.uint32).astype(np.int64) * 16
    codes = np.zeros((RB * 16, N), np.uint8)
    keep = np.zeros((RB * 16, N), bool)
    scale = np.zeros((RB * 16, G), np.float16)
    zero = np.zeros((RB * 16, G), np.float16)
    for rb in range(RB):
        for ct in range(CT):
            w = min(4, G - 4 * ct)
            t = blob[hdr + tile_off[rb * CT + ct]: hdr + tile_off[rb * CT + ct + 1]]
            nseg = 16 * w
            mask_words = t[: nseg * 16].view(np.uint32).reshape(nseg, 4)
            sz = t[nseg * 16: nseg * 20].view(np.float16).reshape(nseg, 2)
            stream = t[nseg * 20:]
            bitpos = 0
            for s in range(nseg):
                r, gi = divmod(s, w)
                row = rb * 16 + r
                col0 = (ct * 4 + gi) * GROUP
                scale[row, ct * 4 + gi] = sz[s, 0]
                zero[row, ct * 4 + gi] = sz[s, 1]
                for j in range(4):
                    m = int(mask_words[s, j])
                    for b in range(32):
                        if (m >> b) & 1:
                            v = 0
                            for i in range(bits):
                                p = bitpos + i
                                v |= ((int(stream[p >> 3]) >> (p & 7)) & 1) << i
                            bitpos += bits
                            codes[row, col0 + 32 * j + b] = v
                            keep[row, col0 + 32 * j + b] = True
    return codes[:K], keep[:K], scale[:K], zero[:K]


def compressed_bytes(K: int, N: int, bits: int, nnz: int) -> int:
    """Algorithmic weight bytes of one matrix: occupancy bitmask, survivor codes,
    fp16 scale + fp16 zero per 128-wide group (no padding, no offset table)."""
    return K * N // 8 + math.ceil(bits * nnz / 8) + K * (N // GROUP) * 4
