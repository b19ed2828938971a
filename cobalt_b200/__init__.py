"""cobalt_b200: the sparse low-bit compressed linear layer of CoBALT, written for B200 (sm_100a).

Public surface
  CobaltSparseLinear   nn.Module, drop-in for the reference's SparseQuantLinear
  patch_model          swap nn.Linear layers of a model for CobaltSparseLinear
  SparseQuantConfig    bits / sparsity / beta / group_size
  compress_weight      dense weight -> RAW tensors (keep, codes, scale, zero)
  pack_tiles           RAW tensors -> tile image streamed by the kernels

The CUDA kernels live in ``libcobalt_b200.so`` (built by ``python -m cobalt_b200.build``) and
are reached through the C ABI in ``include/cobalt_b200.h``; there is no fallback path.
"""
from .compress import SparseQuantConfig, compress_weight, keep_mask, quantize_dense, quantize_survivors
from .format import TileImage, pack_tiles, slice_cols, slice_rows
from .linear import CobaltSparseLinear, FusedProjections
from .patch import patch_linearlayers, patch_model
from .artifact import import_raw_layer, load_artifact, save_artifact, verify_artifact

__all__ = ["import_raw_layer", "load_artifact", "save_artifact", "verify_artifact", "CobaltSparseLinear", "FusedProjections", "patch_model", "patch_linearlayers", "SparseQuantConfig", "compress_weight",
           "keep_mask", "quantize_dense", "quantize_survivors", "pack_tiles", "TileImage", "slice_rows", "slice_cols"]
__version__ = "0.1.0"
