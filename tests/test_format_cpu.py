"""Host-side packer, compressor and patcher (no GPU): the packed tile image is read back by an
independent loop-based reader and must return the RAW tensors bit for bit."""
import numpy as np
import pytest
import torch

from cobalt_b200 import compress as C
from cobalt_b200 import format as F
from cobalt_b200.patch import get_linear_tags_from_model, name_to_linear_tag
from oracle import cobalt_oracle as O


def _roundtrip(keep, q, sc, zr, bits):
    img = F.pack_tiles(keep, q, sc, zr, bits)
    K, N = keep.shape
    codes, k2, s2, z2 = O.unpack_tiles_numpy(img.blob.numpy(), K, N, bits)
    assert np.array_equal(k2, keep.numpy().astype(bool))
    assert np.array_equal(codes, (q.to(torch.uint8) * keep.to(torch.uint8)).numpy())
    assert np.array_equal(s2.view(np.uint16), sc.numpy().view(np.uint16))
    assert np.array_equal(z2.view(np.uint16), zr.numpy().view(np.uint16))
    return img


@pytest.mark.parametrize("name,bits", [("c3s70", 3), ("c4s50", 4), ("c2s50", 2), ("c3s60", 3), ("c4s90_b0", 4), ("c4s00", 4)])
def test_pack_roundtrip_golden(golden, name, bits):
    keep = torch.from_numpy(golden[f"{name}.keep"])
    q = torch.from_numpy(golden[f"{name}.q"])
    sc = torch.from_numpy(golden[f"{name}.scale"])
    zr = torch.from_numpy(golden[f"{name}.zero"])
    img = _roundtrip(keep, q, sc, zr, bits)
    assert img.nnz == int(keep.sum())
    assert img.algorithmic_bytes() == O.compressed_bytes(keep.shape[0], keep.shape[1], bits, img.nnz)


@pytest.mark.parametrize("K,N,bits,dens", [(16, 128, 4, 0.5), (17, 128, 3, 0.3), (1, 640, 2, 0.9), (40, 1152, 3, 0.0),
                                           (33, 256, 4, 1.0), (48, 2688, 3, 0.4)])
def test_pack_roundtrip_ragged(K, N, bits, dens):
    """Row counts that are not multiples of 16, column counts that are not multiples of 512,
    empty and full masks."""
    g = torch.Generator().manual_seed(K * 1000 + N + bits)
    keep = torch.rand(K, N, generator=g) < dens
    q = torch.randint(0, 1 << bits, (K, N), generator=g, dtype=torch.uint8)
    sc = (torch.rand(K, N // 128, generator=g) * 0.01 + 0.001).half()
    zr = torch.randint(0, 1 << bits, (K, N // 128), generator=g).half()
    img = _roundtrip(keep, q, sc, zr, bits)
    assert img.n_row_blocks == (K + 15) // 16 and img.n_col_tiles == (N // 128 + 3) // 4
    assert img.blob.numel() % 16 == 0 and img.header_bytes % 256 == 0


def test_pack_rejects_bad_input():
    keep = torch.ones(16, 128, dtype=torch.bool)
    q = torch.full((16, 128), 9, dtype=torch.uint8)
    sc = torch.ones(16, 1).half()
    with pytest.raises(ValueError):
        F.pack_tiles(keep, q, sc, sc, 3)            # code 9 does not fit 3 bits
    with pytest.raises(ValueError):
        F.pack_tiles(keep[:, :100], q[:, :100], sc, sc, 4)   # N not a multiple of 128
    with pytest.raises(ValueError):
        F.pack_tiles(keep, q, sc, sc, 5)


@pytest.mark.parametrize("name", ["c3s70", "c4s50", "c2s50", "c4s90_b0", "c4s00"])
def test_product_compressor_equals_reference(golden, digests, name):
    """cobalt_b200.compress (product code) against the reference's outputs."""
    c = next(x for x in digests["cases"] if x["name"] == name)
    W = torch.from_numpy(golden[f"{name}.W"])
    norm = torch.from_numpy(golden[f"{name}.norm"])
    keep, q, sc, zr = C.compress_weight(W, norm, C.SparseQuantConfig(c["bits"], c["sparsity"], c["beta"]))
    assert np.array_equal(keep.numpy(), golden[f"{name}.keep"])
    assert np.array_equal(q.numpy(), golden[f"{name}.q"])
    assert np.array_equal(sc.numpy(), golden[f"{name}.scale"])
    assert np.array_equal(zr.numpy(), golden[f"{name}.zero"])


def test_shard_algebra_cpu():
    """Column-parallel shards concatenate, row-parallel shards sum, to the unsharded result."""
    raw = O.synth_raw(64, 1024, 0.5, 4, seed=5)
    keep, q, sc, zr = raw["keep"], raw["q"], raw["scale"], raw["zero"]
    x = O.seeded_activation(4, 1024, 6)
    Wfull = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)
    y = (x.float() @ Wfull.float().t())
    for T in (2, 4, 8):
        rows = [F.slice_rows(keep, q, sc, zr, r * 64 // T, (r + 1) * 64 // T) for r in range(T)]
        ycat = torch.cat([x.float() @ O.dequantize(b, c, d, a).to(torch.bfloat16).float().t() for a, b, c, d in rows], 1)
        assert torch.equal(ycat, y)
        cols = [F.slice_cols(keep, q, sc, zr, r * 1024 // T, (r + 1) * 1024 // T) for r in range(T)]
        ysum = sum(x[:, r * 1024 // T:(r + 1) * 1024 // T].float() @
                   O.dequantize(b, c, d, a).to(torch.bfloat16).float().t() for r, (a, b, c, d) in enumerate(cols))
        assert torch.allclose(ysum, y, rtol=0, atol=1e-4)
    with pytest.raises(ValueError):
        F.slice_cols(keep, q, sc, zr, 0, 100)


def test_linear_tags():
    assert name_to_linear_tag("model.layers.31.self_attn.k_proj") == "self_attn.k_proj"
    m = torch.nn.Sequential()
    m.add_module("model", torch.nn.Sequential())
    m.model.add_module("layers", torch.nn.ModuleList([torch.nn.ModuleDict({"q_proj": torch.nn.Linear(128, 16)})]))
    m.add_module("lm_head", torch.nn.Linear(128, 8))
    assert get_linear_tags_from_model(m) == ["q_proj"]
