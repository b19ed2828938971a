"""The CPU oracle must reproduce, bit for bit, what the reference itself produced
(fixtures written by tests/golden/make_golden.py, which runs the reference's own modules)."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import cobalt_oracle as O

CASES = ["c3s70", "c4s50", "c2s50", "c3s60", "c4s90_b0", "c4s00"]


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


def _sha(t):
    if isinstance(t, torch.Tensor):
        t = t.contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def _spec(digests, name):
    return next(c for c in digests["cases"] if c["name"] == name)


@pytest.mark.parametrize("name", CASES)
def test_mask_and_rtn_match_reference(golden, digests, name):
    c = _spec(digests, name)
    W = torch.from_numpy(golden[f"{name}.W"])
    norm = torch.from_numpy(golden[f"{name}.norm"])
    keep = O.balanced_keepmask(W.abs() * norm.view(1, -1), c["sparsity"], c["beta"])
    assert np.array_equal(keep.bool().numpy(), golden[f"{name}.keep"])
    q, sc, zr = O.group_rtn_survivor(W, keep, c["bits"])
    assert np.array_equal(sc.numpy(), golden[f"{name}.scale_f32"])
    assert np.array_equal(zr.numpy(), golden[f"{name}.zero_f32"])
    assert np.array_equal((q * keep).to(torch.uint8).numpy(), golden[f"{name}.q"])
    k2, q2, s2, z2 = O.compress(W, norm, c["bits"], c["sparsity"], c["beta"])
    assert np.array_equal(k2.numpy(), golden[f"{name}.keep"])
    assert np.array_equal(q2.numpy(), golden[f"{name}.q"])
    assert np.array_equal(s2.numpy(), golden[f"{name}.scale"])
    assert np.array_equal(z2.numpy(), golden[f"{name}.zero"])


@pytest.mark.parametrize("name", CASES)
def test_dequant_and_forward_match_reference(golden, name):
    q = torch.from_numpy(golden[f"{name}.q"])
    keep = torch.from_numpy(golden[f"{name}.keep"])
    sc = torch.from_numpy(golden[f"{name}.scale"])
    zr = torch.from_numpy(golden[f"{name}.zero"])
    Wd = O.dequantize(q, sc, zr, keep)
    assert np.array_equal(Wd.numpy(), golden[f"{name}.Wdeq"])
    assert torch.equal(Wd.to(torch.bfloat16).view(torch.int16), torch.from_numpy(golden[f"{name}.Wdeq_bf16"]))
    for M in (1, 4, 16):
        x = _bf16(golden[f"{name}.x{M}"])
        y = O.linear_forward(x, q, sc, zr, keep)
        assert torch.equal(y.view(torch.int16), torch.from_numpy(golden[f"{name}.y{M}"]))


def test_offgrid_zero_points_present(golden):
    """The very sparse fixture must exercise zero points outside [0, n_levels]."""
    z = golden["c4s90_b0.zero"].astype(np.float32)
    assert (z < 0).any() and (z > 15).any()


def test_column_scale_and_bias_match_reference(golden):
    q = torch.from_numpy(golden["colscale.q"])
    keep = torch.from_numpy(golden["colscale.keep"])
    sc = torch.from_numpy(golden["colscale.scale"])
    zr = torch.from_numpy(golden["colscale.zero"])
    cs = torch.from_numpy(golden["colscale.col_scale"])
    bias = _bf16(golden["colscale.bias"])
    x = _bf16(golden["colscale.x4"])
    Wb = O.dequantize(q, sc, zr, keep, cs).to(torch.bfloat16)
    assert torch.equal(Wb.view(torch.int16), torch.from_numpy(golden["colscale.Wdeq_bf16"]))
    y = O.linear_forward(x, q, sc, zr, keep, cs, bias)
    assert torch.equal(y.view(torch.int16), torch.from_numpy(golden["colscale.y4"]))


def test_synth_raw_matches_reference_generator(digests):
    """Same seeds and shapes as the reference's GEMV unit test (src/cobaltkernel/test_gemv.py:145)."""
    for d in digests["synth_raw"]:
        raw = O.synth_raw(d["K"], d["N"], d["sparsity"], d["bits"], d["seed"])
        assert _sha(O.mask_to_bytes(raw["keep"])) == d["mask"]
        assert _sha(raw["q"]) == d["q"]
        assert _sha(raw["scale"]) == d["scale"]
        assert _sha(raw["zero"]) == d["zero"]
        assert _sha(raw["col_scale"]) == d["col_scale"]


def test_config1_recipe_matches_reference(digests):
    """4096 x 4096, 3 bit, 70 % sparse, beta 0.5: the first benchmark configuration."""
    d = digests["config1"]
    W, norm = O.seeded_matrix(d["K"], d["N"], d["seed"])
    keep, q, sc, zr = O.compress(W, norm, d["bits"], d["sparsity"], d["beta"])
    assert int(keep.sum()) == d["nnz"]
    assert _sha(keep) == d["keep"]
    assert _sha(q) == d["q"]
    assert _sha(sc) == d["scale"]
    assert _sha(zr) == d["zero"]


def test_head_rtn_matches_reference(golden_head):
    """Plain group-128 RTN of the embedding / head (reference: rtn_dense, src/cobaltkernel/pack_cobalt.py:375-386): the
    oracle's restatement and the product's quantiser both reproduce the reference's codes, scales and zero points."""
    from cobalt_b200 import quantize_dense
    W = torch.from_numpy(golden_head["W"].copy()).view(torch.bfloat16)
    q, sc, zr = O.rtn_dense(W, 4)
    assert np.array_equal(q.to(torch.uint8).numpy(), golden_head["q"])
    assert np.array_equal(sc.numpy(), golden_head["scale"])
    assert np.array_equal(zr.numpy(), golden_head["zero"])
    q2, sc2, zr2 = quantize_dense(W, 4)
    assert np.array_equal(q2.numpy(), golden_head["q"])
    assert np.array_equal(sc2.numpy(), golden_head["scale"])
    assert np.array_equal(zr2.to(torch.uint8).numpy(), golden_head["zero"])


@pytest.mark.parametrize("idx", [0, 1])
def test_large_matrix_mask_takes_the_bisection_branch(digests, idx):
    """Above 32 M elements the global threshold of the keep mask comes from the reference's bisection
    (src/cobaltkernel/cobalt_math.py:79-101): 14336 x 4096 (4 bit, 50 %) and 21504 x 5376 (3 bit, 60 %), seeded as
    tests/golden/make_golden.py seeds them.  The oracle and the product compressor both reproduce the digests of the
    reference's mask, codes, scales and zero points."""
    from cobalt_b200 import SparseQuantConfig, compress_weight
    d = digests["large"][idx]
    g = torch.Generator().manual_seed(d["seed"])
    W = (torch.randn(d["K"], d["N"], generator=g) * 0.02).half().float()
    norm = torch.randn(d["N"], generator=g).abs() + 0.1
    assert W.numel() > 32_000_000
    keep, q, sc, zr = O.compress(W, norm, d["bits"], d["sparsity"], d["beta"])
    assert int(keep.sum()) == d["nnz"]
    assert (_sha(keep.bool()), _sha(q.to(torch.uint8)), _sha(sc.half()), _sha(zr.half())) == (d["keep"], d["q"], d["scale"], d["zero"])
    del keep, q, sc, zr
    k2, q2, s2, z2 = compress_weight(W, norm, SparseQuantConfig(d["bits"], d["sparsity"], d["beta"]))
    assert (_sha(k2.bool()), _sha(q2), _sha(s2), _sha(z2)) == (d["keep"], d["q"], d["scale"], d["zero"])
