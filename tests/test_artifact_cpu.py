"""Artifact I/O on the CPU: the blob image and manifest round-trip, the structural verifier accepts what the
packer wrote and names what is wrong with a damaged copy (counterpart of src/prod/verify.py:64-152), and a RAW
safetensors layer (schema of src/cobaltkernel/quantize_cobalt.py:326-329, 436-443) imports to the same tile image."""
import json
import os

import numpy as np
import pytest
import torch

from cobalt_b200 import CobaltSparseLinear
from cobalt_b200 import artifact as A
from cobalt_b200.format import pack_tiles
from oracle import cobalt_oracle as O


def make_modules():
    mods, raws = {}, {}
    specs = {"model.layers.0.self_attn.q_proj": (48, 384, 4, 0.5), "model.layers.0.mlp.down_proj": (40, 640, 3, 0.6),
             "model.layers.1.self_attn.k_proj": (16, 256, 2, 0.5), "lm_head": (32, 128, 4, 0.0)}
    for i, (name, (K, N, bits, sp)) in enumerate(specs.items()):
        W, norm = O.seeded_matrix(K, N, 50 + i)
        keep, q, sc, zr = O.compress(W, norm, bits, sp, 0.5)
        m = CobaltSparseLinear._blank()
        m._install(pack_tiles(keep, q, sc, zr, bits), None, None, {"nbits": bits})
        mods[name] = m
        raws[name] = (keep, q, sc, zr, bits)
    return mods, raws


def test_save_verify_load_roundtrip(tmp_path):
    mods, _ = make_modules()
    man = A.save_artifact(str(tmp_path), mods, config={"note": "test"})
    assert man["format"] == "CBT1" and sorted(l["file"] for l in man["layers"]) == ["layer_00.bin", "layer_01.bin", "misc.bin"]
    rep = A.verify_artifact(str(tmp_path))
    assert rep["ok"] and abs(rep["bpw_recomputed"] - man["bpw"]["bpw_packed"]) < 1e-6
    for lay in man["layers"]:                      # disk bytes are the device bytes, every array 256-byte aligned
        assert os.path.getsize(tmp_path / lay["file"]) == lay["bytes"]
        for e in lay["matrices"].values():
            assert all(a["off"] % 256 == 0 for a in e["arrays"].values())
    back = A.load_artifact(str(tmp_path), device="cpu")
    assert set(back) == set(mods)
    for name, m in mods.items():
        assert torch.equal(back[name].packed, m.packed) and back[name]._img_meta == m._img_meta
        im = m._img_meta
        keep = O.unpack_tiles_numpy(back[name].packed.numpy(), im["K"], im["N"], im["bits"])[1]
        assert int(np.asarray(keep).sum()) == im["nnz"]


def test_verifier_names_damage(tmp_path):
    mods, _ = make_modules()
    A.save_artifact(str(tmp_path), mods)
    man = json.load(open(tmp_path / "manifest.json"))
    lay = next(l for l in man["layers"] if l["file"] == "layer_00.bin")
    e = lay["matrices"]["model.layers.0.self_attn.q_proj"]
    blob = np.fromfile(tmp_path / "layer_00.bin", dtype=np.uint8)
    # flip one bitmask bit of the first tile: the tile's stored size no longer matches its mask (or the count changes)
    bad = blob.copy()
    bad[e["arrays"]["tiles"]["off"] + e["image"]["header_bytes"]] ^= 0x01
    bad.tofile(tmp_path / "layer_00.bin")
    with pytest.raises(A.ArtifactError, match="q_proj"):
        A.verify_artifact(str(tmp_path))
    assert not A.verify_artifact(str(tmp_path), strict=False)["ok"]
    # truncated blob
    blob[: blob.size // 2].tofile(tmp_path / "layer_00.bin")
    with pytest.raises(A.ArtifactError, match="runs past the blob"):
        A.verify_artifact(str(tmp_path))
    # wrong survivor count in the manifest
    blob.tofile(tmp_path / "layer_00.bin")
    e["n_survivors"] += 1
    json.dump(man, open(tmp_path / "manifest.json", "w"))
    with pytest.raises(A.ArtifactError, match="survivors"):
        A.verify_artifact(str(tmp_path))


def test_raw_safetensors_import(tmp_path):
    from safetensors.torch import save_file
    _, raws = make_modules()
    tensors, bits = {}, {}
    for name in ("model.layers.0.self_attn.q_proj", "model.layers.0.mlp.down_proj"):
        keep, q, sc, zr, b = raws[name]
        short = name.split("layers.0.")[1]
        mb = O.mask_to_bytes(keep)
        tensors[f"{short}.mask"] = mb if isinstance(mb, torch.Tensor) else torch.from_numpy(mb)
        tensors[f"{short}.q"] = (q * keep).to(torch.uint8)
        tensors[f"{short}.scale"] = sc.half()
        tensors[f"{short}.zero"] = zr.half()
        tensors[f"{short}.col_scale"] = torch.ones(q.shape[1], dtype=torch.float16)
        bits[short] = b
    path = str(tmp_path / "layer_00.safetensors")
    save_file(tensors, path)
    got = A.import_raw_layer(path, bits=bits, device="cpu")
    assert set(got) == {"self_attn.q_proj", "mlp.down_proj"}
    for short, m in got.items():
        keep, q, sc, zr, b = raws["model.layers.0." + short]
        want = pack_tiles(keep, q, sc, zr, b)
        assert torch.equal(m.packed, want.blob) and m.scale2 is None     # a column scale of ones is dropped
