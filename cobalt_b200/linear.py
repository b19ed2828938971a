"""``CobaltSparseLinear``: drop-in for the reference's sparse-quant linear module.

Same constructor as ``SparseQuantLinear(W_q, scales, zeros, mask, scale2, bias, meta)``
(benchmarks/benchmark_suite.py:1175-1198, built at src/nosink.py:1353-1356) and the
``from_linear`` / ``dequantize`` / ``state_dict`` / ``from_state_dict`` / ``extra_repr``
conventions of ``CPRLinear`` (sinq/cprlinear.py:129-171, 292-330, 357-398, 400-544).

The module keeps only the packed tile image on the device.  ``forward`` calls the CUDA
library through its C ABI: the decode GEMV for up to 16 tokens, the tcgen05 GEMM above.
There is no torch fallback: on a non-CUDA tensor ``forward`` raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn as nn

from . import _lib
from .compress import SparseQuantConfig, compress_weight
from .format import GROUP, TileImage, bytes_to_keep, pack_tiles

GEMV_MAX_TOKENS = 16
FUSED_MAX = 4


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


class CobaltSparseLinear(nn.Module):
    """y = x @ dequant(W).T (+ bias), weights held as bitmask + low-bit survivors."""

    def __init__(self, W_q, scales, zeros, mask, scale2=None, bias=None, meta=None):
        super().__init__()
        meta = dict(meta or {})
        K, N = W_q.shape
        bits = int(meta.get("nbits", meta.get("bits", 4)))
        if int(meta.get("group_size", GROUP)) != GROUP:
            raise ValueError(f"group_size must be {GROUP}")
        img = pack_tiles(mask, W_q, scales.reshape(K, -1), zeros.reshape(K, -1), bits)
        self._install(img, scale2, bias, meta)

    # ------------------------------------------------------------------ construction
    def _install(self, img: TileImage, scale2, bias, meta):
        self.in_features = img.N
        self.out_features = img.K
        self.bits = img.bits
        self.group_size = GROUP
        self.meta = dict(meta or {})
        self.meta.update(nbits=img.bits, group_size=GROUP, shape=(img.K, img.N))
        self._img_meta = img.meta()
        self.register_buffer("packed", img.blob)
        has_scale2 = scale2 is not None and not bool((scale2.float() == 1).all())
        self.register_buffer("scale2", scale2.reshape(-1).to(torch.float16).to(img.blob.device) if has_scale2 else None)
        self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False) if bias is not None else None
        self._scratch = None
        self._desc = None
        self._desc_key = None

    @classmethod
    def _blank(cls):
        obj = cls.__new__(cls)
        nn.Module.__init__(obj)
        return obj

    @classmethod
    def from_raw(cls, mask_u8, q_u8, scale_f16, zero_f16, col_scale=None, bits: int = 4, bias=None):
        """Build from the RAW schema of src/cobaltkernel/quantize_cobalt.py:326-329
        (``mask u8[K, N/8]`` LSB-first, ``q u8[K, N]``, ``scale/zero f16[K, G]``, ``col_scale f16[N]``)."""
        K, N = q_u8.shape
        keep = bytes_to_keep(mask_u8, N) if mask_u8.shape[1] * 8 == N and mask_u8.dtype == torch.uint8 and \
            mask_u8.shape != q_u8.shape else (mask_u8 != 0)
        obj = cls._blank()
        obj._install(pack_tiles(keep, q_u8, scale_f16, zero_f16, bits), col_scale, bias,
                     dict(nbits=bits, group_size=GROUP, shape=(K, N)))
        return obj

    @classmethod
    def from_linear(cls, linear: nn.Linear, act_norms: Optional[torch.Tensor] = None, bits: int = 4,
                    sparsity: float = 0.5, beta: float = 0.5, group_size: int = GROUP):
        """Compress an ``nn.Linear`` (mask + RTN run on the linear's device), then pack."""
        cfg = SparseQuantConfig(bits=bits, sparsity=sparsity, beta=beta, group_size=group_size)
        W = linear.weight.detach()
        if act_norms is None:
            act_norms = torch.ones(W.shape[1], device=W.device)
        keep, q, scale, zero = compress_weight(W, act_norms.to(W.device), cfg)
        obj = cls._blank()
        obj._install(pack_tiles(keep, q, scale, zero, bits), None,
                     None if linear.bias is None else linear.bias.detach().to(torch.bfloat16),
                     dict(nbits=bits, group_size=group_size, shape=tuple(W.shape), sparsity=sparsity, beta=beta))
        return obj

    @classmethod
    def from_dense_rtn(cls, weight: torch.Tensor, bits: int = 4, rows: Optional[slice] = None):
        """Plain group-128 RTN without a mask (``compress.quantize_dense``): the recipe of the reference's tied
        embedding / head (src/cobaltkernel/pack_cobalt.py:375-386, 538-558), packed with an all-ones bitmask so that the
        same kernels multiply by it.  ``rows`` keeps only that slice of output rows (vocab-parallel head).  The matrix is
        quantised in row chunks so that a 262144 x 5376 head does not need an fp32 copy of itself."""
        from .compress import quantize_dense
        K, N = weight.shape
        r0, r1 = (0, K) if rows is None else (rows.start or 0, K if rows.stop is None else rows.stop)
        qs, scs, zrs = [], [], []
        step = max(16, (1 << 25) // max(N, 1))
        for k0 in range(r0, r1, step):
            q, sc, zr = quantize_dense(weight[k0:min(k0 + step, r1)], bits)
            qs.append(q); scs.append(sc); zrs.append(zr)
        q, sc, zr = torch.cat(qs), torch.cat(scs), torch.cat(zrs)
        keep = torch.ones_like(q, dtype=torch.bool)
        obj = cls._blank()
        obj._install(pack_tiles(keep, q, sc, zr, bits), None, None,
                     dict(nbits=bits, group_size=GROUP, shape=(r1 - r0, N), sparsity=0.0, recipe="dense_rtn"))
        return obj

    # ------------------------------------------------------------------ descriptors
    def _descriptor(self) -> _lib.CobaltMat:
        key = (self.packed.data_ptr(), None if self.scale2 is None else self.scale2.data_ptr())
        if self._desc is None or self._desc_key != key:
            m = self._img_meta
            d = _lib.CobaltMat()
            base = self.packed.data_ptr()
            d.tile_off = base
            d.tiles = base + m["header_bytes"]
            d.col_scale = _ptr(self.scale2)
            d.K, d.N, d.bits, d.group = m["K"], m["N"], m["bits"], GROUP
            d.n_row_blocks, d.n_col_tiles = m["n_row_blocks"], m["n_col_tiles"]
            d.max_tile_bytes = m["max_tile_bytes"]
            d.max_tile_nnz = m.get("max_tile_nnz", 8192)
            d.nnz = m["nnz"]
            self._desc, self._desc_key = d, key
        return self._desc

    def _scratch_for(self, M: int) -> torch.Tensor:
        lib = _lib.load()
        d = self._descriptor()
        if M <= GEMV_MAX_TOKENS:
            # sized for the largest GEMV batch once, so that the buffer never moves: a captured CUDA graph keeps its address
            need = lib.cobalt_gemv_scratch_bytes(ctypes.byref(d), GEMV_MAX_TOKENS)
        else:
            need = lib.cobalt_gemm_scratch_bytes(ctypes.byref(d), M)
        if need == 0:
            raise _lib.CobaltError("cobalt_*_scratch_bytes", -1, "could not size the scratch buffer")
        # one buffer per kernel kind: the GEMV buffer has a fixed size (see above), the GEMM buffer grows with M
        kind = "gemv" if M <= GEMV_MAX_TOKENS else "gemm"
        cur = self._scratch.get(kind) if isinstance(self._scratch, dict) else None
        if cur is None or cur.numel() < need + 256 or cur.device != self.packed.device:
            if not isinstance(self._scratch, dict):
                self._scratch = {}
            cur = torch.zeros(need + 256, dtype=torch.uint8, device=self.packed.device)
            self._scratch[kind] = cur
        return cur

    @staticmethod
    def _aligned(t: torch.Tensor, a: int = 256) -> int:
        return (t.data_ptr() + a - 1) // a * a

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, out_fp32: bool = False, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``out_fp32`` returns the raw fp32 sums (no bias, no rounding) -- the partial output a row-parallel
        shard hands to its all-reduce.  ``out`` (contiguous ``[M, out_features]`` of the result dtype) receives the
        result instead of a fresh tensor, e.g. a slot of a buffer that peers read."""
        if not x.is_cuda:
            raise RuntimeError("CobaltSparseLinear.forward needs a CUDA tensor; there is no CPU path")
        if x.dtype != torch.bfloat16:
            raise TypeError(f"CobaltSparseLinear computes in bfloat16, got {x.dtype}")
        lib = _lib.load()
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features)
        if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        M = x2.shape[0]
        want = torch.float32 if out_fp32 else torch.bfloat16
        if out is not None:
            if out.dtype != want or out.numel() != M * self.out_features or not out.is_contiguous() or out.device != x.device:
                raise ValueError("`out` must be a contiguous [M, out_features] tensor of the result dtype on x's device")
            y = out.view(M, self.out_features)
        else:
            y = torch.empty(M, self.out_features, dtype=want, device=x.device)
        if M == 0:
            return y.reshape(*lead, self.out_features)
        d = self._descriptor()
        scratch = self._scratch_for(M)
        sp = self._aligned(scratch)
        sbytes = scratch.numel() - (sp - scratch.data_ptr())
        stream = torch.cuda.current_stream(x.device).cuda_stream
        bias = None if self.bias is None else self.bias.data.to(torch.bfloat16)
        if out_fp32:
            rc = lib.cobalt_linear_f32(ctypes.byref(d), x2.data_ptr(), x2.stride(0), y.data_ptr(), y.stride(0), M, sp, sbytes,
                                       stream)
            _lib.check("cobalt_linear_f32", rc)
        elif M <= GEMV_MAX_TOKENS:
            rc = lib.cobalt_gemv(ctypes.byref(d), x2.data_ptr(), x2.stride(0), y.data_ptr(), y.stride(0), _ptr(bias), M,
                                 sp, sbytes, stream)
            _lib.check("cobalt_gemv", rc)
        else:
            rc = lib.cobalt_gemm(ctypes.byref(d), x2.data_ptr(), x2.stride(0), y.data_ptr(), y.stride(0), _ptr(bias), M,
                                 sp, sbytes, stream)
            _lib.check("cobalt_gemm", rc)
        return y.reshape(*lead, self.out_features)

    # ------------------------------------------------------------------ inspection
    def dequantize(self) -> torch.Tensor:
        """Dense bf16 ``[K, N]`` weight, bit-identical to the reference's dequantisation cast to bf16."""
        lib = _lib.load()
        W = torch.empty(self.out_features, self.in_features, dtype=torch.bfloat16, device=self.packed.device)
        rc = lib.cobalt_dequant(ctypes.byref(self._descriptor()), W.data_ptr(),
                                torch.cuda.current_stream(W.device).cuda_stream)
        _lib.check("cobalt_dequant", rc)
        return W

    def unpack(self):
        """``(codes uint8[K, N], keep bool[K, N])`` recovered from the packed image."""
        lib = _lib.load()
        dev = self.packed.device
        codes = torch.empty(self.out_features, self.in_features, dtype=torch.uint8, device=dev)
        keep = torch.empty_like(codes)
        rc = lib.cobalt_unpack(ctypes.byref(self._descriptor()), codes.data_ptr(), keep.data_ptr(),
                               torch.cuda.current_stream(dev).cuda_stream)
        _lib.check("cobalt_unpack", rc)
        return codes, keep.bool()

    def device_status(self) -> int:
        """Status word of the last kernels that used this module's scratch buffer (0 = healthy)."""
        if not self._scratch:
            return 0
        worst = 0
        for buf in self._scratch.values():
            out = ctypes.c_uint32(0)
            _lib.load().cobalt_device_status(self._aligned(buf), torch.cuda.current_stream(self.packed.device).cuda_stream,
                                             ctypes.byref(out))
            worst = max(worst, int(out.value))
        return worst

    def compressed_bytes(self) -> int:
        return TileImage.from_meta(self.packed, self._img_meta).algorithmic_bytes()

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self, *args, **kwargs):
        """Plain dict of CPU tensors plus ``"meta"`` (layout of sinq/cprlinear.py:400-440)."""
        sd = {"packed": self.packed.detach().cpu(), "meta": dict(self.meta, image=dict(self._img_meta))}
        if self.scale2 is not None:
            sd["scale2"] = self.scale2.detach().cpu()
        if self.bias is not None:
            sd["bias"] = self.bias.detach().cpu()
        return sd

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        meta = dict(state_dict["meta"])
        img = TileImage.from_meta(state_dict["packed"].to(self.packed.device if hasattr(self, "packed") else "cpu"),
                                  meta.pop("image"))
        for name in ("packed", "scale2"):
            if name in self._buffers:
                del self._buffers[name]
        dev = img.blob.device
        self._install(img, state_dict.get("scale2"), state_dict.get("bias"), meta)
        if self.scale2 is not None:
            self.scale2 = self.scale2.to(dev)
        return self

    @classmethod
    def from_state_dict(cls, state_dict, device="cuda", compute_dtype=torch.bfloat16):
        if compute_dtype != torch.bfloat16:
            raise TypeError("CobaltSparseLinear computes in bfloat16")
        meta = dict(state_dict["meta"])
        img = TileImage.from_meta(state_dict["packed"].to(device), meta.pop("image"))
        obj = cls._blank()
        s2 = state_dict.get("scale2")
        b = state_dict.get("bias")
        obj._install(img, None if s2 is None else s2.to(device), None if b is None else b.to(device), meta)
        return obj

    def _apply(self, fn, *a, **k):
        out = super()._apply(fn, *a, **k)
        self._desc = None
        self._scratch = None
        return out

    def extra_repr(self) -> str:
        m = self._img_meta
        dens = m["nnz"] / float(m["K"] * m["N"])
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"group_size={GROUP}, density={dens:.3f}, bias={self.bias is not None}")


class FusedProjections:
    """Several ``CobaltSparseLinear`` that read the same activations (q|k|v, gate|up), evaluated with one
    GEMV launch for up to 16 tokens (``cobalt_gemv_fused``) and one call each above that.  The reference
    reaches the same goal by concatenating the matrices row-wise at pack time (docs/FORMAT.md:126-151)."""

    def __init__(self, mods):
        mods = list(mods)
        if not 1 <= len(mods) <= FUSED_MAX:
            raise ValueError(f"between 1 and {FUSED_MAX} projections can be fused")
        n0 = mods[0].in_features
        if any(m.in_features != n0 or m.bits != mods[0].bits or m.scale2 is not None or m.bias is not None for m in mods):
            raise ValueError("fused projections need equal in_features and bit width, no column scale and no bias")
        self.mods = mods
        self._scratch = None
        self._arrays = None

    def _prepare(self, M, device):
        lib = _lib.load()
        n = len(self.mods)
        descs = (ctypes.POINTER(_lib.CobaltMat) * n)(*[ctypes.pointer(m._descriptor()) for m in self.mods])
        need = lib.cobalt_gemv_fused_scratch_bytes(n, descs, GEMV_MAX_TOKENS)   # fixed size: the address survives graph capture
        if need == 0:
            raise _lib.CobaltError("cobalt_gemv_fused_scratch_bytes", -1, "could not size the scratch buffer")
        if self._scratch is None or self._scratch.numel() < need + 256 or self._scratch.device != device:
            self._scratch = torch.zeros(need + 256, dtype=torch.uint8, device=device)
        return descs

    def __call__(self, x: torch.Tensor):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.mods[0].in_features)
        M = x2.shape[0]
        if M > GEMV_MAX_TOKENS or M == 0:
            return [m(x) for m in self.mods]
        if not x2.is_cuda or x2.dtype != torch.bfloat16:
            raise TypeError("FusedProjections needs a bf16 CUDA tensor")
        if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        lib = _lib.load()
        n = len(self.mods)
        descs = self._prepare(M, x.device)
        ys = [torch.empty(M, m.out_features, dtype=torch.bfloat16, device=x.device) for m in self.mods]
        yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
        ld = (ctypes.c_int64 * n)(*[y.stride(0) for y in ys])
        sp = (self._scratch.data_ptr() + 255) // 256 * 256
        rc = lib.cobalt_gemv_fused(n, descs, x2.data_ptr(), x2.stride(0), yp, ld, None, M, sp,
                                   self._scratch.numel() - (sp - self._scratch.data_ptr()),
                                   torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check("cobalt_gemv_fused", rc)
        return [y.reshape(*lead, m.out_features) for y, m in zip(ys, self.mods)]

    def staged(self, kind: int, a: torch.Tensor, b: Optional[torch.Tensor], flavor: int, w: Optional[torch.Tensor] = None,
               w_branch: Optional[torch.Tensor] = None, h_out: Optional[torch.Tensor] = None, eps: float = 0.0,
               out_fp32: bool = False, outs=None, push=None, delta_slots=None):
        """One launch in which the kernel computes its activation rows while it stages them (``cobalt_gemv_fused_staged``):
        ``kind = _lib.IN_GLU``: rows ``act(a) * b``; ``kind = _lib.IN_ADDNORM``: rows ``RMSNorm(a + b) * w`` with
        ``a + b`` written to ``h_out``; ``kind = _lib.IN_PLAIN``: rows ``a``.  ``a``, ``b``, ``h_out``: ``[M, in_features]``
        bf16.  Tensor parallelism: ``push`` (a ``tp.PeerReducer``) sends the fp32 sums of this rank into every rank's
        slot instead of returning them (one matrix; returns ``[]``); ``delta_slots`` (a ``tp.PeerReducer``) takes
        ``b`` = the sum over ranks of the partials pushed before.  Returns the outputs, or ``None`` when this shape cannot
        take the fused path (nothing was launched: call the separate steps)."""
        M = a.shape[0]
        if M > GEMV_MAX_TOKENS or M == 0 or a.dim() != 2 or a.stride(-1) != 1:
            return None
        for t in (b, h_out):
            if t is not None and (t.shape != a.shape or t.stride() != a.stride()):
                raise ValueError("a, b and h_out must have the same shape and strides")
        lib = _lib.load()
        n = len(self.mods)
        descs = self._prepare(M, a.device)
        ptr = lambda t: None if t is None else t.data_ptr()
        inp = _lib.CobaltStagedInput(kind, flavor, a.data_ptr(), ptr(b), a.stride(0), ptr(w), ptr(w_branch), ptr(h_out), eps,
                                     None if delta_slots is None else ctypes.pointer(delta_slots.slots))
        sp = (self._scratch.data_ptr() + 255) // 256 * 256
        if push is not None:
            ys, yp, ld, out_fp32 = [], None, None, True
        else:
            ys = outs if outs is not None else [torch.empty(M, m.out_features, dtype=torch.float32 if out_fp32 else torch.bfloat16,
                                                             device=a.device) for m in self.mods]
            yp = (ctypes.c_void_p * n)(*[y.data_ptr() for y in ys])
            ld = (ctypes.c_int64 * n)(*[m.out_features if y.dim() == 1 else y.stride(0) for y, m in zip(ys, self.mods)])
        rc = lib.cobalt_gemv_fused_staged(n, descs, ctypes.byref(inp), yp, ld, None, M, 1 if out_fp32 else 0,
                                          None if push is None else ctypes.byref(push.slots), sp,
                                          self._scratch.numel() - (sp - self._scratch.data_ptr()),
                                          torch.cuda.current_stream(a.device).cuda_stream)
        if rc == _lib.EUNSUPPORTED:
            return None
        _lib.check("cobalt_gemv_fused_staged", rc)
        return ys
