"""On-disk artifacts of compressed layers: RAW import, a blob image whose bytes are the bytes the
GPU holds, a manifest, and a structural verifier.

The reference ships two things this mirrors:

* RAW safetensors, one file per decoder layer, tensors ``<proj>.mask`` (u8 ``[K, N/8]`` bitmap,
  LSB-first), ``<proj>.q`` (u8 ``[K, N]``, 0 at pruned positions), ``<proj>.scale`` / ``<proj>.zero``
  (fp16 ``[K, N/128]``) and ``<proj>.col_scale`` (fp16 ``[N]``): src/cobaltkernel/quantize_cobalt.py:326-329,
  436-443, 467.  ``import_raw_layer`` reads one and packs it.
* a packed container - ``manifest.json`` plus blobs that are concatenations of 256-byte-aligned
  arrays, so that disk bytes equal device bytes (docs/FORMAT.md:13-37; writer
  src/cobaltkernel/pack_cobalt.py:561-714) - and a verifier that re-derives the bits per weight from
  the manifest, checks that every array lies inside its blob and that pruned positions decode to
  exactly zero (src/prod/verify.py:64-152).  ``save_artifact`` / ``load_artifact`` /
  ``verify_artifact`` are the counterparts for the tile image of this library.

Layout written here: ``manifest.json`` and one ``layer_XX.bin`` per layer index (``misc.bin`` for
modules without a layer index).  Every matrix contributes its tile-image blob (header of tile
offsets + tiles + 64 bytes of slack, exactly ``CobaltSparseLinear.packed``) and, when present, its
fp16 column scale and bf16 bias; every array starts on a 256-byte boundary.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict, Optional

import numpy as np
import torch

from .format import GROUP, TILE_GROUPS, TILE_ROWS, TileImage
from .linear import CobaltSparseLinear

FORMAT = "CBT1"
ALIGN = 256
RAW_SUFFIXES = ("mask", "q", "scale", "zero", "col_scale")


class ArtifactError(RuntimeError):
    pass


# ----------------------------------------------------------------------------- RAW import
def import_raw_layer(path: str, bits: int = 4, device="cuda") -> Dict[str, CobaltSparseLinear]:
    """Read one RAW ``layer_XX.safetensors`` and pack every matrix in it.  ``bits`` may also be a dict
    ``{module name: bits}`` (the RAW schema stores codes as bytes and does not record their width)."""
    from safetensors import safe_open
    out: Dict[str, CobaltSparseLinear] = {}
    with safe_open(path, framework="pt", device="cpu") as f:
        names = sorted({k.rsplit(".", 1)[0] for k in f.keys() if k.rsplit(".", 1)[-1] in RAW_SUFFIXES})
        for name in names:
            have = {s: f"{name}.{s}" in f.keys() for s in RAW_SUFFIXES}
            if not all(have[s] for s in ("mask", "q", "scale", "zero")):
                raise ArtifactError(f"{path}: {name} lacks one of mask/q/scale/zero")
            b = bits[name] if isinstance(bits, dict) else bits
            cs = f.get_tensor(f"{name}.col_scale").to(device) if have["col_scale"] else None
            out[name] = CobaltSparseLinear.from_raw(f.get_tensor(f"{name}.mask").to(device), f.get_tensor(f"{name}.q").to(device),
                                                    f.get_tensor(f"{name}.scale").to(device), f.get_tensor(f"{name}.zero").to(device),
                                                    cs, bits=int(b))
    return out


# ----------------------------------------------------------------------------- blob image
def _layer_file(name: str) -> str:
    m = re.search(r"(?:^|\.)layers\.(\d+)\.", name)
    return f"layer_{int(m.group(1)):02d}.bin" if m else "misc.bin"


def _pad(n: int) -> int:
    return (n + ALIGN - 1) // ALIGN * ALIGN


def save_artifact(out_dir: str, modules: Dict[str, CobaltSparseLinear], config: Optional[dict] = None) -> dict:
    """Write ``manifest.json`` + blobs for ``{module name: CobaltSparseLinear}``.  Returns the manifest."""
    os.makedirs(out_dir, exist_ok=True)
    files: Dict[str, list] = {}
    for name in sorted(modules):
        files.setdefault(_layer_file(name), []).append(name)
    layers = []
    params = stream = 0
    for fname in sorted(files):
        off = 0
        entries = {}
        with open(os.path.join(out_dir, fname), "wb") as fh:
            def put(arr: np.ndarray) -> dict:
                nonlocal off
                raw = np.ascontiguousarray(arr).tobytes()
                fh.write(raw)
                fh.write(b"\0" * (_pad(len(raw)) - len(raw)))
                rec = {"off": off, "bytes": len(raw)}
                off += _pad(len(raw))
                return rec
            for name in files[fname]:
                mod = modules[name]
                img = mod._img_meta
                arrays = {"tiles": put(mod.packed.detach().cpu().numpy())}
                if mod.scale2 is not None:
                    arrays["col_scale"] = put(mod.scale2.detach().cpu().view(torch.int16).numpy())
                if mod.bias is not None:
                    arrays["bias"] = put(mod.bias.detach().to(torch.bfloat16).cpu().view(torch.int16).numpy())
                sb = mod.compressed_bytes()
                entries[name] = {"K": img["K"], "N": img["N"], "G": img["N"] // GROUP, "bits": img["bits"],
                                 "n_survivors": img["nnz"], "stream_bytes": sb, "bpw": round(8.0 * sb / (img["K"] * img["N"]), 6),
                                 "image": dict(img), "arrays": arrays}
                params += img["K"] * img["N"]
                stream += sb
        layers.append({"file": fname, "bytes": off, "matrices": entries})
    man = {"format": FORMAT, "version": 1, "tile": {"rows": TILE_ROWS, "groups": TILE_GROUPS, "group": GROUP},
           "config": config or {}, "bpw": {"bpw_packed": round(8.0 * stream / max(params, 1), 6), "params": params, "stream_bytes": stream},
           "layers": layers}
    with open(os.path.join(out_dir, "manifest.json"), "w") as fh:
        json.dump(man, fh, indent=1)
    return man


def load_artifact(art_dir: str, device="cuda") -> Dict[str, CobaltSparseLinear]:
    """Map the blobs back into modules; the tile bytes go to the device unchanged."""
    with open(os.path.join(art_dir, "manifest.json")) as fh:
        man = json.load(fh)
    if man.get("format") != FORMAT:
        raise ArtifactError(f"format is {man.get('format')!r}, want {FORMAT!r}")
    out: Dict[str, CobaltSparseLinear] = {}
    for lay in man["layers"]:
        blob = np.fromfile(os.path.join(art_dir, lay["file"]), dtype=np.uint8)
        for name, e in lay["matrices"].items():
            def get(key, dtype):
                a = e["arrays"].get(key)
                if a is None:
                    return None
                if a["off"] + a["bytes"] > blob.size:
                    raise ArtifactError(f"{lay['file']}:{name}.{key} runs past the blob")
                return torch.from_numpy(blob[a["off"]:a["off"] + a["bytes"]].copy()).view(dtype)
            tiles = get("tiles", torch.uint8)
            cs, bias = get("col_scale", torch.float16), get("bias", torch.bfloat16)
            mod = CobaltSparseLinear._blank()
            mod._install(TileImage.from_meta(tiles.to(device), e["image"]), None if cs is None else cs.to(device),
                         None if bias is None else bias.to(device), dict(nbits=e["bits"], group_size=GROUP, shape=(e["K"], e["N"])))
            out[name] = mod
    return out


# ----------------------------------------------------------------------------- verifier
def _walk_tiles(blob: np.ndarray, img: dict):
    """Structure of a tile image, from its bytes alone: yields (tile index, width in groups, survivors per
    segment [16, w], byte size) and raises on any inconsistency."""
    RB, CT, bits = img["n_row_blocks"], img["n_col_tiles"], img["bits"]
    G = img["N"] // GROUP
    n_tiles = RB * CT
    hdr = img["header_bytes"]
    if hdr != _pad(4 * (n_tiles + 1)) or hdr > blob.size:
        raise ArtifactError("header size does not match the tile count")
    off = blob[:4 * (n_tiles + 1)].view("<u4").astype(np.int64) * 16
    if off[0] != 0 or np.any(np.diff(off) <= 0):
        raise ArtifactError("tile offsets are not strictly increasing from 0")
    if hdr + off[-1] + 64 > blob.size:
        raise ArtifactError("tiles (plus 64 bytes of slack) run past the blob")
    pop = np.array([bin(i).count("1") for i in range(256)], dtype=np.int64)
    for t in range(n_tiles):
        ct = t % CT
        w = min(TILE_GROUPS, G - TILE_GROUPS * ct)
        base = hdr + off[t]
        masks = blob[base:base + TILE_ROWS * w * 16].reshape(TILE_ROWS, w, 16)
        nnz = pop[masks].sum(-1)
        need = TILE_ROWS * w * 20 + (int(nnz.sum()) * bits + 7) // 8
        need = (need + 15) // 16 * 16
        size = int(off[t + 1] - off[t])
        if size != need:
            raise ArtifactError(f"tile {t}: {size} bytes stored, {need} implied by its bitmask")
        if size > img["max_tile_bytes"] or int(nnz.sum()) > img["max_tile_nnz"]:
            raise ArtifactError(f"tile {t} exceeds the recorded maxima")
        yield t, w, nnz, size


def verify_artifact(art_dir: str, device: Optional[str] = None, strict: bool = True) -> dict:
    """Structural check from the bytes on disk: arrays inside their blobs and 256-byte aligned, tile offsets
    consistent with the bitmasks, survivor counts and bits per weight re-derived, rows beyond K empty.  With a
    CUDA ``device`` every matrix is also dequantised there and pruned positions must be exactly zero."""
    problems = []
    with open(os.path.join(art_dir, "manifest.json")) as fh:
        man = json.load(fh)
    rep = {"artifact": art_dir, "format": man.get("format"), "matrices": {}, "problems": problems}
    if man.get("format") != FORMAT:
        problems.append(f"format is {man.get('format')!r}, want {FORMAT!r}")
    params = stream = 0
    for lay in man.get("layers", []):
        path = os.path.join(art_dir, lay["file"])
        if not os.path.exists(path):
            problems.append(f"missing blob {lay['file']}")
            continue
        blob = np.fromfile(path, dtype=np.uint8)
        for name, e in lay["matrices"].items():
            tag = f"{lay['file']}:{name}"
            bad = False
            for an, a in e["arrays"].items():
                if a["off"] % ALIGN:
                    problems.append(f"{tag}.{an} is not {ALIGN}-byte aligned")
                if a["off"] + a["bytes"] > blob.size:
                    problems.append(f"{tag}.{an} runs past the blob ({a['off']}+{a['bytes']} > {blob.size})")
                    bad = True
            if bad:
                continue
            img, a = e["image"], e["arrays"]["tiles"]
            tiles = blob[a["off"]:a["off"] + a["bytes"]]
            try:
                nnz = 0
                last_rb_rows = img["K"] - TILE_ROWS * (img["n_row_blocks"] - 1)
                for t, w, cnt, _ in _walk_tiles(tiles, img):
                    nnz += int(cnt.sum())
                    if t // img["n_col_tiles"] == img["n_row_blocks"] - 1 and int(cnt[last_rb_rows:].sum()):
                        raise ArtifactError(f"tile {t}: survivors in rows beyond K")
                if nnz != e["n_survivors"] or nnz != img["nnz"]:
                    raise ArtifactError(f"{nnz} survivors in the bitmasks, manifest says {e['n_survivors']}")
                sb = img["K"] * img["N"] // 8 + (nnz * img["bits"] + 7) // 8 + img["K"] * (img["N"] // GROUP) * 4
                if sb != e["stream_bytes"]:
                    raise ArtifactError(f"stream bytes {e['stream_bytes']} in the manifest, {sb} recomputed")
            except ArtifactError as err:
                problems.append(f"{tag}: {err}")
                continue
            params += img["K"] * img["N"]
            stream += e["stream_bytes"]
            info = {"shape": [img["K"], img["N"]], "bits": img["bits"], "n_survivors": nnz,
                    "bpw": round(8.0 * e["stream_bytes"] / (img["K"] * img["N"]), 6)}
            if device is not None:
                mod = CobaltSparseLinear._blank()
                mod._install(TileImage.from_meta(torch.from_numpy(tiles.copy()).to(device), img), None, None,
                             dict(nbits=img["bits"]))
                W = mod.dequantize().float()
                _, keep = mod.unpack()
                info["finite"] = bool(torch.isfinite(W).all())
                info["pruned_nonzero"] = int((W[~keep] != 0).sum())
                if not info["finite"]:
                    problems.append(f"{tag} has non-finite weights")
                if info["pruned_nonzero"]:
                    problems.append(f"{tag} has {info['pruned_nonzero']} pruned positions that do not decode to zero")
            rep["matrices"][tag] = info
    if params:
        bpw = 8.0 * stream / params
        rep["bpw_recomputed"] = round(bpw, 6)
        if abs(bpw - man["bpw"]["bpw_packed"]) > 1e-6:
            problems.append(f"bpw recompute {bpw:.6f} != manifest {man['bpw']['bpw_packed']:.6f}")
    rep["ok"] = not problems
    if problems and strict:
        raise ArtifactError("\n  ".join(["artifact check FAILED:"] + problems))
    return rep
