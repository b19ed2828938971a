"""Parity of the CUDA path (through the C ABI) against the CPU oracle.  Needs a B200.

Bars
  * unpacked codes, keep mask and dequantised bf16 weights: bit-exact;
  * layer outputs in bf16: rel-L2 <= 1e-3 and max-abs <= 1e-2 against the oracle's CPU result.
    bf16 values at |y| >= 2 are 2^-6 = 0.0156 apart, so two correct fp32 accumulations that
    straddle a rounding boundary differ by more than 1e-2 there.  An element may exceed 1e-2
    only if it is such a case: the oracle's value and ours must both lie within 0.52 bf16
    spacings of the exact fp64 dot product of the same bf16 weights and activations (half a
    spacing for the final rounding plus 2 % of a spacing, about 8e-5 relative, for the fp32
    accumulation: the tensor cores truncate when they align addends, which over 14336 columns
    was measured at up to 5e-5 relative).
"""
import numpy as np
import pytest
import torch

from cobalt_b200 import CobaltSparseLinear, SparseQuantConfig, compress_weight
from oracle import cobalt_oracle as O

pytestmark = pytest.mark.gpu

MAX_ABS = 1e-2
REL_L2 = 1e-3
MAX_EXEMPT = 0.01          # largest share of elements that may differ by more than MAX_ABS as rounding-boundary cases
EXEMPT = []                # (exempted, total) of every comparison that used the exemption, for the summary test


def bf16_spacing(v: torch.Tensor) -> torch.Tensor:
    """Distance between neighbouring bf16 values around |v| (normal range)."""
    e = torch.floor(torch.log2(v.abs().double().clamp(min=1e-30)))
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), e - 7)


def check_output(y: torch.Tensor, y_ref: torch.Tensor, y_exact: torch.Tensor):
    y, y_ref = y.detach().cpu(), y_ref.detach().cpu()
    assert y.dtype == torch.bfloat16 and y.shape == y_ref.shape
    assert torch.isfinite(y.float()).all()
    d = (y.double() - y_ref.double()).abs()
    rel = float(d.norm() / y_ref.double().norm().clamp(min=1e-30))
    assert rel <= REL_L2, f"rel-L2 {rel:.3e}"
    bad = d > MAX_ABS
    if bad.any():
        ex = y_exact.double()[bad]
        for name, val in (("ours", y.double()[bad]), ("oracle", y_ref.double()[bad])):
            err = (val - ex).abs()
            lim = 0.52 * bf16_spacing(val)
            assert bool((err <= lim).all()), f"{name}: {int(bad.sum())} elements off by more than {MAX_ABS} and not a rounding-boundary case"
        # the exemption is for isolated rounding-boundary flips, not for a result that is systematically one
        # spacing off: at most MAX_EXEMPT of the elements may take it (a handful of elements for tiny outputs)
        frac = float(bad.sum()) / bad.numel()
        EXEMPT.append((int(bad.sum()), bad.numel()))
        print(f"rounding-boundary exemptions: {int(bad.sum())} of {bad.numel()} ({100 * frac:.3f} %)")
        assert int(bad.sum()) <= max(4, int(MAX_EXEMPT * bad.numel())), f"{int(bad.sum())} of {bad.numel()} elements exempted"
    return rel, float(d.max())


def exact_fp64(x, Wb):
    return x.double() @ Wb.double().t()


def to_module(keep, q, sc, zr, bits, scale2=None, bias=None):
    K, N = q.shape
    G = N // 128
    dev = "cuda"
    meta = {"nbits": bits, "group_size": 128, "shape": (K, N)}
    return CobaltSparseLinear(q.to(dev), sc.view(K, G, 1).to(dev), zr.view(K, G, 1).to(dev), keep.to(dev),
                              None if scale2 is None else scale2.to(dev), None if bias is None else bias.to(dev), meta)


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


GOLD = [("c3s70", 3), ("c4s50", 4), ("c2s50", 2), ("c3s60", 3), ("c4s90_b0", 4), ("c4s00", 4)]


def _gold(golden, name):
    return (torch.from_numpy(golden[f"{name}.keep"]), torch.from_numpy(golden[f"{name}.q"]),
            torch.from_numpy(golden[f"{name}.scale"]), torch.from_numpy(golden[f"{name}.zero"]))


# ----------------------------------------------------------------------------- bit-exact parts
@pytest.mark.parametrize("name,bits", GOLD)
def test_unpack_and_dequant_bitexact(golden, name, bits):
    keep, q, sc, zr = _gold(golden, name)
    mod = to_module(keep, q, sc, zr, bits)
    codes, k2 = mod.unpack()
    assert torch.equal(codes.cpu(), q)
    assert torch.equal(k2.cpu(), keep)
    W = mod.dequantize().cpu()
    want = torch.from_numpy(golden[f"{name}.Wdeq_bf16"]).view(torch.bfloat16)
    assert torch.equal(W.view(torch.int16), want.view(torch.int16))
    assert bool((W[~keep] == 0).all())


def test_dequant_with_column_scale_bitexact(golden):
    keep, q, sc, zr = _gold(golden, "colscale")
    cs = torch.from_numpy(golden["colscale.col_scale"])
    mod = to_module(keep, q, sc, zr, 4, scale2=cs)
    W = mod.dequantize().cpu()
    assert torch.equal(W.view(torch.int16), torch.from_numpy(golden["colscale.Wdeq_bf16"]))


# ----------------------------------------------------------------------------- GEMV
@pytest.mark.parametrize("name,bits", GOLD)
@pytest.mark.parametrize("M", [1, 4, 16])
def test_gemv_golden(golden, name, bits, M):
    keep, q, sc, zr = _gold(golden, name)
    mod = to_module(keep, q, sc, zr, bits)
    x = _bf16(golden[f"{name}.x{M}"])
    y_ref = _bf16(golden[f"{name}.y{M}"])
    Wb = torch.from_numpy(golden[f"{name}.Wdeq_bf16"]).view(torch.bfloat16)
    y = mod(x.cuda())
    check_output(y, y_ref, exact_fp64(x, Wb))
    assert mod.device_status() == 0


@pytest.mark.parametrize("name,bits", GOLD)
def test_gemv_rowwalk_golden(golden, name, bits):
    import ctypes
    from cobalt_b200 import _lib
    keep, q, sc, zr = _gold(golden, name)
    mod = to_module(keep, q, sc, zr, bits)
    lib = _lib.load()
    for M in (1, 4, 16):
        x = _bf16(golden[f"{name}.x{M}"]).cuda()
        y = torch.empty(M, q.shape[0], dtype=torch.bfloat16, device="cuda")
        rc = lib.cobalt_gemv_rowwalk(ctypes.byref(mod._descriptor()), x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0),
                                     None, M, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        Wb = torch.from_numpy(golden[f"{name}.Wdeq_bf16"]).view(torch.bfloat16)
        check_output(y, _bf16(golden[f"{name}.y{M}"]), exact_fp64(x.cpu(), Wb))


def test_gemv_column_scale_and_bias(golden):
    keep, q, sc, zr = _gold(golden, "colscale")
    cs = torch.from_numpy(golden["colscale.col_scale"])
    bias = _bf16(golden["colscale.bias"])
    x = _bf16(golden["colscale.x4"])
    mod = to_module(keep, q, sc, zr, 4, scale2=cs, bias=bias)
    y = mod(x.cuda())
    Wb = torch.from_numpy(golden["colscale.Wdeq_bf16"]).view(torch.bfloat16)
    yb = (exact_fp64(x, Wb)).to(torch.bfloat16).double() + bias.double()
    check_output(y, _bf16(golden["colscale.y4"]), yb)


def test_gemv_batch_equals_single_and_is_deterministic():
    """Token m of a batched call equals the single-token call bit for bit (the reference's
    M=4 == 4 x M=1 gate, src/cobaltkernel/verify_kernel.py:415-461); two runs are identical."""
    raw = O.synth_raw(192, 4096, 0.5, 4, seed=192 + 4096)
    mod = to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)
    x = O.seeded_activation(16, 4096, 77).cuda()
    y16 = mod(x)
    assert torch.equal(y16, mod(x))
    y4 = mod(x[:4])
    for m in range(4):
        y1 = mod(x[m:m + 1])
        assert torch.equal(y1[0], y4[m])
        assert torch.equal(y1[0], y16[m])


def test_pruned_positions_contribute_exactly_zero():
    """Huge activations at pruned columns leave the output bit-identical
    (src/cobaltkernel/test_gemv.py:403-455), also with an off-grid zero point."""
    K, N, bits = 256, 5376, 4
    g = torch.Generator().manual_seed(7)
    pat = torch.rand(N, generator=g) < 0.5
    keep = pat.view(1, N).expand(K, N).contiguous()
    q = torch.randint(0, 16, (K, N), generator=g, dtype=torch.uint8) * keep.to(torch.uint8)
    sc = (torch.rand(K, N // 128, generator=g) * 0.01 + 1e-3).half()
    for zero in (torch.randint(0, 16, (K, N // 128), generator=g).half(), torch.full((K, N // 128), 52.0).half()):
        mod = to_module(keep, q, sc, zero, bits)
        x0 = O.seeded_activation(1, N, 8)
        xh = x0.clone()
        xh[0, ~pat] = 1.0e4
        assert torch.equal(mod(x0.cuda()), mod(xh.cuda()))
        assert bool((mod.dequantize()[:, (~pat).cuda()] == 0).all())


@pytest.mark.parametrize("K,N", [(256, 5376), (128, 21504), (192, 4096), (64, 1024)])
def test_gemv_reference_test_shapes(K, N):
    """The shapes and seeds of the reference's GEMV unit test (src/cobaltkernel/test_gemv.py:142-181),
    4 bit, 50 % sparse, generator pinned by tests/test_oracle_golden.py."""
    raw = O.synth_raw(K, N, 0.5, 4, seed=K + N)
    mod = to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)
    Wb = O.dequantize(raw["q"], raw["scale"], raw["zero"], raw["keep"]).to(torch.bfloat16)
    assert torch.equal(mod.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
    for M in (1, 2, 4, 8):
        x = O.seeded_activation(M, N, K + M)
        check_output(mod(x.cuda()), torch.matmul(x, Wb.t()), exact_fp64(x, Wb))


@pytest.mark.parametrize("K,N,bits", [(512, 14336, 4), (1024, 28672, 3)])
def test_gemv_balanced_partition_long_rows(K, N, bits):
    """Few, long row blocks: the launch balances 32-column words over all SMs and the row blocks that straddle
    CTAs are exchanged through global scratch (about 1.5 and 6 words per warp here)."""
    raw = O.synth_raw(K, N, 0.5, bits, seed=K + N + bits)
    mod = to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], bits)
    Wb = O.dequantize(raw["q"], raw["scale"], raw["zero"], raw["keep"]).to(torch.bfloat16)
    for M in (1, 3, 8, 16):
        x = O.seeded_activation(M, N, K + M)
        y = mod(x.cuda())
        check_output(y, torch.matmul(x, Wb.t()), exact_fp64(x, Wb))
        assert torch.equal(y, mod(x.cuda()))              # the exchange order is fixed: same bits every run
    assert mod.device_status() == 0


def test_gemv_scratch_survives_graph_replay_after_a_larger_batch():
    """A graph captured at M = 1 keeps the scratch address: a later 12-token call must not move or dirty the buffer."""
    raw = O.synth_raw(640, 2048, 0.5, 4, seed=5150)
    mod = to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)
    x1 = O.seeded_activation(1, 2048, 1).cuda()
    x12 = O.seeded_activation(12, 2048, 2).cuda()
    want = mod(x1).clone()
    addr = mod._scratch["gemv"].data_ptr()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        y_static = mod(x1)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            y_static = mod(x1)
    torch.cuda.current_stream().wait_stream(s)
    y12 = mod(x12)                                            # larger batch between capture and replay
    assert mod._scratch["gemv"].data_ptr() == addr
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y_static, want)
    assert torch.equal(y12[:1], mod(x12[:1]))


# ----------------------------------------------------------------------------- benchmark configurations
def _compress_on_gpu(K, N, bits, sparsity, seed):
    """Seeded weights and norms from the oracle's generator; mask + RTN by the product
    compressor on the GPU; the same RAW tensors are then given to both sides."""
    W, norm = O.seeded_matrix(K, N, seed)
    keep, q, sc, zr = compress_weight(W.cuda(), norm.cuda(), SparseQuantConfig(bits, sparsity, 0.5))
    return keep, q, sc, zr


def test_config1_single_linear():
    """4096 x 4096, 3 bit, 70 % sparse, x = 1 x 4096: mask and codes from the oracle on the CPU."""
    W, norm = O.seeded_matrix(4096, 4096, 1)
    keep, q, sc, zr = O.compress(W, norm, 3, 0.7, 0.5)
    mod = to_module(keep, q, sc, zr, 3)
    Wb = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)
    assert torch.equal(mod.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
    codes, k2 = mod.unpack()
    assert torch.equal(codes.cpu(), q) and torch.equal(k2.cpu(), keep)
    x = O.seeded_activation(1, 4096, 3001)
    check_output(mod(x.cuda()), O.linear_forward(x, q, sc, zr, keep), exact_fp64(x, Wb))


@pytest.mark.parametrize("name,K,N", [("q", 4096, 4096), ("kv", 1024, 4096), ("gate_up", 14336, 4096), ("down", 4096, 14336)])
def test_config2_block_shapes(name, K, N):
    """Mistral-7B projection shapes, 4 bit, 50 % sparse, M in {1, 4, 16}."""
    keep, q, sc, zr = _compress_on_gpu(K, N, 4, 0.5, 1000 + K % 97 + N % 89)
    mod = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": 4})
    kc, qc, scc, zrc = keep.cpu(), q.cpu(), sc.cpu(), zr.cpu()
    Wb = O.dequantize(qc, scc, zrc, kc).to(torch.bfloat16)
    assert torch.equal(mod.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
    for M in (1, 4, 16):
        x = O.seeded_activation(M, N, 3000 + M)
        check_output(mod(x.cuda()), torch.matmul(x, Wb.t()), exact_fp64(x, Wb))
    assert mod.device_status() == 0


# ----------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("name,bits", GOLD)
@pytest.mark.parametrize("M", [17, 100, 128, 300])
def test_gemm_golden_matrices(golden, name, bits, M):
    keep, q, sc, zr = _gold(golden, name)
    mod = to_module(keep, q, sc, zr, bits)
    Wb = torch.from_numpy(golden[f"{name}.Wdeq_bf16"]).view(torch.bfloat16)
    x = O.seeded_activation(M, q.shape[1], 500 + M)
    y = mod(x.cuda())
    check_output(y, torch.matmul(x, Wb.t()), exact_fp64(x, Wb))
    assert mod.device_status() == 0


def test_gemm_column_scale_and_bias(golden):
    keep, q, sc, zr = _gold(golden, "colscale")
    cs = torch.from_numpy(golden["colscale.col_scale"])
    bias = _bf16(golden["colscale.bias"])
    mod = to_module(keep, q, sc, zr, 4, scale2=cs, bias=bias)
    x = O.seeded_activation(64, q.shape[1], 11)
    y_ref = O.linear_forward(x, q, sc, zr, keep, cs, bias)
    Wb = torch.from_numpy(golden["colscale.Wdeq_bf16"]).view(torch.bfloat16)
    check_output(mod(x.cuda()), y_ref, exact_fp64(x, Wb).to(torch.bfloat16).double() + bias.double())


@pytest.mark.parametrize("bits,sparsity", [(3, 0.7), (2, 0.5)])
@pytest.mark.parametrize("K,N,M", [(4096, 4096, 128), (4096, 4096, 512), (1024, 4096, 2048), (14336, 4096, 128),
                                    (4096, 14336, 512)])
def test_config4_prefill_shapes(bits, sparsity, K, N, M):
    """Prefill sweep shapes on the 7B projections; the oracle matmul runs on the CPU."""
    keep, q, sc, zr = _compress_on_gpu(K, N, bits, sparsity, 4000 + bits)
    mod = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": bits})
    Wb = O.dequantize(q.cpu(), sc.cpu(), zr.cpu(), keep.cpu()).to(torch.bfloat16)
    x = O.seeded_activation(M, N, 4100 + M)
    y = mod(x.cuda())
    check_output(y, torch.matmul(x, Wb.t()), exact_fp64(x, Wb))
    # the first 16 tokens through the GEMV agree with the GEMM (both accumulate the same products in fp32)
    y16 = mod(x[:16].cuda())
    d = (y16.float() - y[:16].float()).abs()
    assert float(d.norm() / y16.float().norm()) <= REL_L2
    assert mod.device_status() == 0


def test_state_dict_roundtrip(golden):
    keep, q, sc, zr = _gold(golden, "c4s50")
    mod = to_module(keep, q, sc, zr, 4)
    sd = mod.state_dict()
    assert all(not v.is_cuda for v in sd.values() if isinstance(v, torch.Tensor))
    mod2 = CobaltSparseLinear.from_state_dict(sd, device="cuda")
    x = _bf16(golden["c4s50.x4"]).cuda()
    assert torch.equal(mod(x), mod2(x))


def test_patch_model_swaps_linears():
    import torch.nn as nn
    from cobalt_b200 import patch_model

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(256, 64, bias=False)
            self.up_proj = nn.Linear(256, 128, bias=False)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Block(), Block()])
            self.lm_head = nn.Linear(256, 32, bias=False)

    torch.manual_seed(0)
    net = Net()
    ref = {n: m.weight.detach().clone() for n, m in net.named_modules() if isinstance(m, nn.Linear)}
    patch_model(net, SparseQuantConfig(bits=4, sparsity=0.5))       # compress + pack on the CPU ...
    net = net.cuda()                                                # ... then move the packed images
    assert isinstance(net.lm_head, nn.Linear)
    assert net.cobalt_quantized and sorted(net.linear_tags) == ["q_proj", "up_proj"]
    for i in range(2):
        for nme in ("q_proj", "up_proj"):
            mod = getattr(net.layers[i], nme)
            assert isinstance(mod, CobaltSparseLinear)
            W = ref[f"layers.{i}.{nme}"].cpu()
            keep, q, sc, zr = O.compress(W, torch.ones(W.shape[1]), 4, 0.5, 0.5)
            Wb = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)
            assert torch.equal(mod.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
            x = O.seeded_activation(2, 256, 5)
            check_output(mod(x.cuda()), torch.matmul(x, Wb.t()), exact_fp64(x, Wb))


def test_fused_projections_equal_separate_calls():
    """q|k|v-style fused launch: bit-identical to one cobalt_gemv call per matrix."""
    from cobalt_b200 import FusedProjections
    mods = []
    for i, K in enumerate((512, 128, 128)):
        raw = O.synth_raw(K, 1536, 0.5, 4, seed=70 + i)
        mods.append(to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4))
    fused = FusedProjections(mods)
    for M in (1, 5, 16):
        x = O.seeded_activation(M, 1536, 80 + M).cuda()
        outs = fused(x)
        for m, y in zip(mods, outs):
            assert torch.equal(y, m(x))
    outs = fused(O.seeded_activation(40, 1536, 99).cuda())          # above 16 tokens: one GEMM each
    assert [o.shape[-1] for o in outs] == [512, 128, 128]
    with pytest.raises(ValueError):
        raw = O.synth_raw(64, 1024, 0.5, 4, seed=1)
        FusedProjections([mods[0], to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)])


GEMMA27B = {"q": (4096, 5376, "column"), "kv": (2048, 5376, "column"), "o": (5376, 4096, "row"),
            "gate_up": (21504, 5376, "column"), "down": (5376, 21504, "row")}


@pytest.mark.parametrize("T", [1, 2, 4, 8])
@pytest.mark.parametrize("name", list(GEMMA27B))
def test_config5_gemma27b_shard_shapes(name, T):
    """Gemma-3-27B projection shapes (hidden 5376, intermediate 21504, 32 q / 16 kv heads of 128) as one rank of a
    T-way tensor-parallel split sees them, T = 1 (whole matrix), 2, 4, 8: 3 bit, 60 % sparse.  in_features of 5376,
    10752, 2688 and 512 exercise partial column tiles.  Decode batch 1 and 8, prefill (2048 tokens at T = 8, 128 for the
    larger shards, whose CPU oracle would otherwise run for minutes)."""
    K, N, kind = GEMMA27B[name]
    K, N = (K // T, N) if kind == "column" else (K, N // T)
    prefill = 2048 if T == 8 else 128
    keep, q, sc, zr = _compress_on_gpu(K, N, 3, 0.6, 5000 + K % 101 + N % 103)
    mod = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": 3})
    Wb = O.dequantize(q.cpu(), sc.cpu(), zr.cpu(), keep.cpu()).to(torch.bfloat16)
    assert torch.equal(mod.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
    for M in (1, 8, prefill):
        x = O.seeded_activation(M, N, 5100 + M)
        check_output(mod(x.cuda()), torch.matmul(x, Wb.t()), exact_fp64(x, Wb))
    # fp32 partial sums of a row-parallel shard: within fp32 accumulation noise of the exact product
    x = O.seeded_activation(8, N, 5200)
    part = mod(x.cuda(), out_fp32=True).cpu().double()
    ex = exact_fp64(x, Wb)
    assert float((part - ex).norm() / ex.norm()) <= 1e-5
    assert mod.device_status() == 0


@pytest.mark.gpu
def test_artifact_roundtrip_on_device(tmp_path):
    """Blob image written from device modules, checked by the verifier with the device pass (pruned positions decode
    to exactly zero, src/prod/verify.py:137-145), loaded back: same bytes on the device, same outputs bit for bit."""
    from cobalt_b200 import load_artifact, save_artifact, verify_artifact
    dev = torch.device("cuda")
    mods = {}
    for i, (name, K, N, bits, sp) in enumerate([("model.layers.0.self_attn.q_proj", 256, 512, 4, 0.5),
                                               ("model.layers.0.mlp.down_proj", 200, 1024, 3, 0.6),
                                               ("model.layers.1.mlp.up_proj", 512, 256, 2, 0.5)]):
        W, norm = O.seeded_matrix(K, N, 70 + i)
        keep, q, sc, zr = O.compress(W, norm, bits, sp, 0.5)
        mods[name] = CobaltSparseLinear(q.to(dev), sc.to(dev), zr.to(dev), keep.to(dev), None, None, {"nbits": bits})
    save_artifact(str(tmp_path), mods)
    rep = verify_artifact(str(tmp_path), device="cuda")
    assert rep["ok"] and all(m["pruned_nonzero"] == 0 and m["finite"] for m in rep["matrices"].values())
    back = load_artifact(str(tmp_path), device="cuda")
    for name, m in mods.items():
        assert torch.equal(back[name].packed, m.packed)
        x = O.seeded_activation(3, m.in_features, 90).to(dev)
        assert torch.equal(back[name](x), m(x))


@pytest.mark.gpu
@pytest.mark.parametrize("M", [1, 5, 200])
def test_host_buffer_entry_points(M):
    """cobalt_linear_host and its non-synchronising variant: pinned host activations in, host results out, equal bit for bit
    to the module's forward on device tensors."""
    import ctypes
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    W, norm = O.seeded_matrix(384, 1024, 21)
    keep, q, sc, zr = O.compress(W, norm, 4, 0.5, 0.5)
    mod = CobaltSparseLinear(q.to(dev), sc.to(dev), zr.to(dev), keep.to(dev), None, None, {"nbits": 4})
    x = O.seeded_activation(M, 1024, 22)
    want = mod(x.to(dev)).cpu()
    hx, hy, hy2 = x.pin_memory(), torch.empty(M, 384, dtype=torch.bfloat16).pin_memory(), torch.empty(M, 384, dtype=torch.bfloat16).pin_memory()
    dx, dy = torch.empty(M, 1024, dtype=torch.bfloat16, device=dev), torch.empty(M, 384, dtype=torch.bfloat16, device=dev)
    d = mod._descriptor()
    need = max(lib.cobalt_gemv_scratch_bytes(ctypes.byref(d), min(M, 16)), lib.cobalt_gemm_scratch_bytes(ctypes.byref(d), M), 65536)
    scr = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
    sp = (scr.data_ptr() + 255) // 256 * 256
    st = torch.cuda.current_stream().cuda_stream
    assert lib.cobalt_linear_host(ctypes.byref(d), hx.data_ptr(), hy.data_ptr(), None, M, dx.data_ptr(), dy.data_ptr(), sp, need, st) == 0
    assert torch.equal(hy, want)
    assert lib.cobalt_linear_host_async(ctypes.byref(d), hx.data_ptr(), hy2.data_ptr(), None, M, dx.data_ptr(), dy.data_ptr(), sp, need, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(hy2, want)


@pytest.mark.parametrize("M", [1, 7])
def test_fused_host_buffer_entry_point(M):
    """cobalt_gemv_fused_host_async: one copy of the activations in, one launch for three matrices, three copies out,
    equal bit for bit to the modules' forwards on device tensors."""
    import ctypes
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    mods = []
    for j, K in enumerate((384, 128, 64)):
        W, norm = O.seeded_matrix(K, 1024, 31 + j)
        keep, q, sc, zr = O.compress(W, norm, 4, 0.5, 0.5)
        mods.append(CobaltSparseLinear(q.to(dev), sc.to(dev), zr.to(dev), keep.to(dev), None, None, {"nbits": 4}))
    x = O.seeded_activation(M, 1024, 35)
    want = [m(x.to(dev)).cpu() for m in mods]
    hx = x.pin_memory()
    hy = [torch.empty(M, m.out_features, dtype=torch.bfloat16).pin_memory() for m in mods]
    dx = torch.empty(M, 1024, dtype=torch.bfloat16, device=dev)
    dy = [torch.empty(M, m.out_features, dtype=torch.bfloat16, device=dev) for m in mods]
    n = len(mods)
    descs = (ctypes.POINTER(_lib.CobaltMat) * n)(*[ctypes.pointer(m._descriptor()) for m in mods])
    need = lib.cobalt_gemv_fused_scratch_bytes(n, descs, M)
    scr = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
    sp = (scr.data_ptr() + 255) // 256 * 256
    yh = (ctypes.c_void_p * n)(*[t.data_ptr() for t in hy])
    yd = (ctypes.c_void_p * n)(*[t.data_ptr() for t in dy])
    rc = lib.cobalt_gemv_fused_host_async(n, descs, hx.data_ptr(), yh, M, dx.data_ptr(), yd, sp, need,
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    for got, w in zip(hy, want):
        assert torch.equal(got, w)
    assert lib.cobalt_gemv_fused_host_async(n, descs, hx.data_ptr(), yh, 17, dx.data_ptr(), yd, sp, need,
                                            torch.cuda.current_stream().cuda_stream) == -1      # more than 16 tokens: GEMV only


@pytest.mark.gpu
def test_one_scratch_serves_gemv_and_gemm_in_any_order():
    """A scratch buffer zeroed once is reused by GEMM-sized (split-K) and GEMV-sized host calls in turn: every kernel
    returns its arrival counters to zero and neither finds the other's partial sums where it expects counters."""
    import ctypes
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    W, norm = O.seeded_matrix(384, 2048, 23)
    keep, q, sc, zr = O.compress(W, norm, 3, 0.6, 0.5)
    mod = CobaltSparseLinear(q.to(dev), sc.to(dev), zr.to(dev), keep.to(dev), None, None, {"nbits": 3})
    d = mod._descriptor()
    Ms = (200, 1, 64, 5, 16, 130, 2)
    need = max(max(lib.cobalt_gemv_scratch_bytes(ctypes.byref(d), min(M, 16)), lib.cobalt_gemm_scratch_bytes(ctypes.byref(d), M)) for M in Ms)
    scr = torch.zeros(need + 256, dtype=torch.uint8, device=dev)
    sp = (scr.data_ptr() + 255) // 256 * 256
    st = torch.cuda.current_stream().cuda_stream
    for rnd in range(2):
        for M in Ms:
            x = O.seeded_activation(M, 2048, 24 + M)
            want = mod(x.to(dev)).cpu()
            hx, hy = x.pin_memory(), torch.empty(M, 384, dtype=torch.bfloat16).pin_memory()
            dx, dy = torch.empty(M, 2048, dtype=torch.bfloat16, device=dev), torch.empty(M, 384, dtype=torch.bfloat16, device=dev)
            assert lib.cobalt_linear_host(ctypes.byref(d), hx.data_ptr(), hy.data_ptr(), None, M, dx.data_ptr(), dy.data_ptr(), sp, need, st) == 0
            assert torch.equal(hy, want), (rnd, M)


@pytest.mark.gpu
def test_peer_allreduce_single_rank_and_layout_check():
    """world = 1: the kernel pushes the partial into its own slot, sees its own flag and writes the sum; three calls
    in a row alternate the slots.  A flag block that overlaps the slots is refused on the host."""
    import ctypes
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    n, stride = 2048, 8192
    flags_off = 3 * stride
    buf = torch.zeros((flags_off + 256) // 4, dtype=torch.float32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_uint64 * 1)(buf.data_ptr())
    st = torch.cuda.current_stream().cuda_stream
    for call in range(3):
        part = torch.randn(n, device=dev)
        buf[:n] = part
        out = torch.empty(n, dtype=torch.bfloat16, device=dev)
        assert lib.cobalt_allreduce_peer(ptrs, 0, 1, n, stride, flags_off, out.data_ptr(), 0, status.data_ptr(), st) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, part.to(torch.bfloat16)) and int(status[0]) == 0
    two = (ctypes.c_uint64 * 2)(buf.data_ptr(), buf.data_ptr())
    assert lib.cobalt_allreduce_peer(two, 0, 2, n, stride, flags_off, out.data_ptr(), 0, status.data_ptr(), st) == -1


@pytest.mark.gpu
def test_peer_allreduce_wait_expires_cleanly():
    """Failure detection without a fault: a peer that never publishes its flag (here: a second buffer in the same
    process that nothing writes to) makes the bounded wait of the all-reduce kernel run out; the kernel records the
    status code, writes no output, returns, and the context keeps working."""
    import ctypes
    import time
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    n, stride = 1024, 4096
    flags_off = (1 + 2 * 2) * stride                      # staging + two slots of two rows
    mine = torch.zeros((flags_off + 256) // 4, dtype=torch.float32, device=dev)
    silent = torch.zeros_like(mine)                       # stands for a rank that never arrives
    mine[:n] = 1.0
    out = torch.full((n,), -7.0, dtype=torch.float32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    ptrs = (ctypes.c_uint64 * 2)(mine.data_ptr(), silent.data_ptr())
    t0 = time.time()
    rc = lib.cobalt_allreduce_peer(ptrs, 0, 2, n, stride, flags_off, out.data_ptr(), 1, status.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 20.0
    assert int(status[0]) == 6                             # DEV_TIMEOUT_PEER
    assert bool((out == -7.0).all())                       # nothing was written
    # the context is intact: an ordinary call still works
    W, norm = O.seeded_matrix(64, 256, 3)
    keep, q, sc, zr = O.compress(W, norm, 4, 0.5, 0.5)
    mod = CobaltSparseLinear(q.to(dev), sc.to(dev), zr.to(dev), keep.to(dev), None, None, {"nbits": 4})
    x = O.seeded_activation(1, 256, 4)
    Wb = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)
    check_output(mod(x.to(dev)), torch.matmul(x, Wb.t()), exact_fp64(x, Wb))


@pytest.mark.gpu
@pytest.mark.parametrize("nh,nkv,D,ctx,pos,window", [(32, 8, 128, 2304, 2047, 0), (32, 8, 128, 300, 0, 0), (16, 16, 64, 512, 511, 0),
                                                     (32, 16, 128, 1024, 700, 256), (8, 1, 256, 200, 130, 0), (4, 2, 64, 130, 129, 70)])
def test_attn_decode_matches_torch(nh, nkv, D, ctx, pos, window):
    """Single-token attention over the KV cache against the same arithmetic in torch (rounding points of
    src/cobaltkernel/ref_llama.py:117-137).  The two differ only in fp32 summation order, so outputs may differ
    by a bf16 rounding step on a few elements: rel-L2 <= 2e-3, max-abs <= 2 % of the largest output."""
    import torch.nn.functional as F
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(1234 + nh + ctx)
    q = torch.randn(1, nh * D, generator=g).to(torch.bfloat16).to(dev)
    kc = torch.randn(nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    positions = torch.tensor([pos], dtype=torch.long, device=dev)
    need = lib.cobalt_attn_decode_scratch_bytes(nh, D, ctx)
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    out = torch.empty_like(q)
    scale = float(D) ** -0.5
    rc = lib.cobalt_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), positions.data_ptr(), scratch.data_ptr(), need, out.data_ptr(),
                                nh, nkv, D, ctx, window, scale, 1, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    rep = nh // nkv
    qg = q.view(1, nkv, rep, D).permute(1, 0, 2, 3).reshape(nkv, rep, D)
    att = torch.bmm(qg, kc.transpose(1, 2)) * scale
    kv_pos = torch.arange(ctx, device=dev)
    allowed = kv_pos <= pos
    if window:
        allowed &= kv_pos > pos - window
    att = att.masked_fill(~allowed[None, None, :], float("-inf"))
    att = F.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
    ref = torch.bmm(att, vc).reshape(1, nh * D)
    torch.cuda.synchronize()
    d = (out.float() - ref.float())
    rel = float(d.norm() / ref.float().norm())
    assert rel <= 2e-3, rel
    assert float(d.abs().max()) <= 0.02 * float(ref.float().abs().max()), float(d.abs().max())


@pytest.mark.parametrize("nh,nkv,D,ctx,positions,window", [(32, 8, 128, 2304, [2047], 0), (32, 8, 128, 300, [0], 0), (16, 16, 64, 512, [511], 0),
                                                           (32, 16, 128, 1024, [700], 256), (8, 2, 128, 640, [5, 639, 130], 0),
                                                           (8, 4, 64, 1024, [1000, 77], 200)])
def test_attn_decode_one_kernel_equals_three(nh, nkv, D, ctx, positions, window):
    """cobalt_attn_decode_fused (one cooperative kernel whose CTAs wait for each other's softmax statistics) gives the
    bits of the three-kernel cobalt_attn_decode, for single sequences, batches and sliding windows; it leaves its
    counters at zero (three calls in a row on one scratch) and its status word clean."""
    import ctypes
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    B = len(positions)
    g = torch.Generator(device="cpu").manual_seed(77 + nh + ctx)
    q = torch.randn(B, nh * D, generator=g).to(torch.bfloat16).to(dev)
    kc = torch.randn(B, nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(B, nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    pos = torch.tensor(positions, dtype=torch.long, device=dev)
    stride = nkv * ctx * D if B > 1 else 0
    scale = float(D) ** -0.5
    st = torch.cuda.current_stream().cuda_stream
    need = lib.cobalt_attn_decode_scratch_bytes(nh, D, ctx) * B
    scratch = torch.empty(need, dtype=torch.uint8, device=dev)
    want = torch.empty_like(q)
    assert lib.cobalt_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), scratch.data_ptr(), need, want.data_ptr(),
                                  nh, nkv, D, ctx, window, scale, B, stride, st) == 0
    nf = lib.cobalt_attn_decode_fused_scratch_bytes(nh, nkv, D, ctx, B)
    fs = torch.zeros(nf, dtype=torch.uint8, device=dev)
    for rnd in range(3):
        got = torch.zeros_like(q)
        rc = lib.cobalt_attn_decode_fused(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), fs.data_ptr(), nf, got.data_ptr(),
                                          nh, nkv, D, ctx, window, scale, B, stride, st)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want), rnd
    status = ctypes.c_uint32(0)
    assert lib.cobalt_device_status(fs.data_ptr(), st, ctypes.byref(status)) == 0 and status.value == 0
    assert int(fs[256:256 + B * nkv * 8].view(torch.int32).abs().sum()) == 0       # counters back at zero


def test_attn_decode_one_kernel_refuses_grids_that_do_not_fit():
    """The CTAs of the one-kernel attention wait for each other, so all of them must be resident: a grid beyond that is
    refused (nothing launched) and the caller uses the three-kernel entry point."""
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    nh, nkv, D, ctx, B = 32, 16, 128, 8192, 4                     # 64 chunks x 16 KV heads x 4 sequences = 4096 CTAs
    nf = lib.cobalt_attn_decode_fused_scratch_bytes(nh, nkv, D, ctx, B)
    fs = torch.zeros(nf, dtype=torch.uint8, device=dev)
    q = torch.zeros(B, nh * D, dtype=torch.bfloat16, device=dev)
    kc = torch.zeros(B, nkv, ctx, D, dtype=torch.bfloat16, device=dev)
    pos = torch.zeros(B, dtype=torch.long, device=dev)
    rc = lib.cobalt_attn_decode_fused(q.data_ptr(), kc.data_ptr(), kc.data_ptr(), pos.data_ptr(), fs.data_ptr(), nf, q.data_ptr(),
                                      nh, nkv, D, ctx, 0, 1.0, B, nkv * ctx * D, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.EUNSUPPORTED


@pytest.mark.gpu
def test_attn_decode_batch_equals_single_sequences():
    """n_seq sequences in one call (own caches, own positions) give the bits of n_seq single-sequence calls."""
    from cobalt_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    B, nh, nkv, D, ctx, window = 3, 16, 4, 128, 700, 300
    g = torch.Generator(device="cpu").manual_seed(77)
    q = torch.randn(B, nh * D, generator=g).to(torch.bfloat16).to(dev)
    kc = torch.randn(B, nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(B, nkv, ctx, D, generator=g).to(torch.bfloat16).to(dev)
    positions = torch.tensor([699, 5, 412], dtype=torch.long, device=dev)
    need = lib.cobalt_attn_decode_scratch_bytes(nh, D, ctx)
    scratch = torch.empty(need * B, dtype=torch.uint8, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    out = torch.empty_like(q)
    assert lib.cobalt_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), positions.data_ptr(), scratch.data_ptr(), need * B,
                                  out.data_ptr(), nh, nkv, D, ctx, window, 0.1, B, nkv * ctx * D, st) == 0
    assert lib.cobalt_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), positions.data_ptr(), scratch.data_ptr(), need,
                                  out.data_ptr(), nh, nkv, D, ctx, window, 0.1, B, nkv * ctx * D, st) == -2     # scratch too small
    for b in range(B):
        one = torch.empty(1, nh * D, dtype=torch.bfloat16, device=dev)
        assert lib.cobalt_attn_decode(q[b].data_ptr(), kc[b].data_ptr(), vc[b].data_ptr(), positions[b:b + 1].data_ptr(),
                                      scratch.data_ptr(), need, one.data_ptr(), nh, nkv, D, ctx, window, 0.1, 1, 0, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(one[0], out[b]), b


@pytest.mark.gpu
def test_compressed_head_matches_oracle(golden_head):
    """Group-128 RTN head (no mask): codes from the product quantiser equal the reference's, the packed all-ones-mask
    image dequantises bit-exactly, logits and arg-max agree with the oracle's dequantise + matmul."""
    from cobalt_b200 import quantize_dense
    W = torch.from_numpy(golden_head["W"].copy()).view(torch.bfloat16)
    # codes as the reference produced them (on the CPU: a GPU may round a tie in the division differently, which is
    # why both sides of a parity check always share one set of RAW tensors)
    q, sc, zr = quantize_dense(W, 4)
    assert torch.equal(q, torch.from_numpy(golden_head["q"]))
    assert torch.equal(sc, torch.from_numpy(golden_head["scale"]))
    assert torch.equal(zr.to(torch.uint8), torch.from_numpy(golden_head["zero"]))
    head = CobaltSparseLinear.from_dense_rtn(W, 4).cuda()
    keep = torch.ones(W.shape, dtype=torch.bool)
    Wb = O.dequantize(q, sc, zr, keep).to(torch.bfloat16)
    assert torch.equal(head.dequantize().cpu().view(torch.int16), Wb.view(torch.int16))
    qg, scg, zrg = quantize_dense(W.cuda(), 4)                 # quantised on the GPU: at most a few ties differ
    assert float((qg.cpu() != q).float().mean()) < 1e-3
    for M in (1, 8, 40):                                       # GEMV and tcgen05 GEMM
        x = O.seeded_activation(M, W.shape[1], 600 + M)
        y = head(x.cuda())
        y_ref = torch.matmul(x, Wb.t())
        check_output(y, y_ref, exact_fp64(x, Wb))
    part = CobaltSparseLinear.from_dense_rtn(W, 4, rows=slice(32, 64)).cuda()     # a vocabulary slice of a parallel head
    x = O.seeded_activation(2, W.shape[1], 9)
    assert torch.equal(part(x.cuda()), head(x.cuda())[:, 32:64])


def _separate_addnorm(h, delta, w, w_branch, flavor, eps):
    """cobalt_add_rmsnorm through the C ABI: (h + delta', normalised rows)."""
    from cobalt_b200 import _lib
    lib = _lib.load()
    y = torch.empty_like(h)
    h_out = torch.empty_like(h) if delta is not None else None
    ptr = lambda t: None if t is None else t.data_ptr()
    rc = lib.cobalt_add_rmsnorm(h.data_ptr(), ptr(delta), w.data_ptr(), ptr(h_out), y.data_ptr(), h.shape[0], h.shape[1], eps,
                                flavor, ptr(w_branch), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return (h if delta is None else h_out), y


@pytest.mark.parametrize("N,M", [(4096, 1), (4096, 2), (1024, 8), (5376, 1), (2048, 3), (512, 2)])
@pytest.mark.parametrize("mode", ["llama", "llama_first", "gemma", "gemma_branch"])
def test_norm_folded_into_staging_equals_separate_kernels(N, M, mode):
    """Residual add + RMSNorm computed by the GEMV while it stages its activations (cobalt_gemv_fused_staged) against
    cobalt_add_rmsnorm followed by cobalt_gemv_fused: identical h + delta and identical projections, bit for bit."""
    from cobalt_b200 import _lib
    from cobalt_b200.linear import FusedProjections
    mods = []
    for j, K in enumerate((256, 64)):
        raw = O.synth_raw(K, N, 0.5, 4, seed=700 + j)
        mods.append(to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4))
    fused = FusedProjections(mods)
    g = torch.Generator().manual_seed(N + M)
    h = torch.randn(M, N, generator=g).bfloat16().cuda()
    delta = None if mode == "llama_first" else (torch.randn(M, N, generator=g) * 0.5).bfloat16().cuda()
    w = (torch.randn(N, generator=g) * 0.1 + (1.0 if mode.startswith("llama") else 0.0)).bfloat16().cuda()
    wb = (torch.randn(N, generator=g) * 0.1).bfloat16().cuda() if mode == "gemma_branch" else None
    flavor, eps = (0, 1e-5) if mode.startswith("llama") else (1, 1e-6)
    h_ref, x_ref = _separate_addnorm(h, delta, w, wb, flavor, eps)
    want = fused(x_ref)
    h_out = torch.empty_like(h) if delta is not None else None
    got = fused.staged(_lib.IN_ADDNORM, h, delta, flavor, w=w, w_branch=wb, h_out=h_out, eps=eps)
    assert got is not None
    torch.cuda.synchronize()
    if delta is not None:
        assert torch.equal(h_out, h_ref)
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    # the normalised rows themselves against torch in fp32 (the kernels' own arithmetic is pinned by the model tests)
    hf = h_ref.float()
    r = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    xt = (w.float() * (hf * r).bfloat16().float()) if flavor == 0 else (hf * r * (1.0 + w.float()))
    assert float((x_ref.float() - xt).abs().max()) <= 2.0 ** -6 * float(xt.abs().max())


@pytest.mark.parametrize("N,M,act", [(14336, 1, 0), (14336, 2, 0), (21504, 1, 1), (4096, 8, 1), (1024, 5, 0)])
def test_gated_activation_folded_into_staging_equals_separate_kernels(N, M, act):
    """act(gate) * up computed by the GEMV while it stages (cobalt_gemv_fused_staged, COBALT_IN_GLU) against cobalt_swiglu
    followed by cobalt_gemv: identical outputs, bf16 and raw fp32 sums."""
    from cobalt_b200 import _lib
    from cobalt_b200.linear import FusedProjections
    raw = O.synth_raw(192, N, 0.5, 4, seed=800 + M)
    mod = to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)
    fused = FusedProjections([mod])
    g = torch.Generator().manual_seed(N + M)
    gate = torch.randn(M, N, generator=g).bfloat16().cuda()
    up = torch.randn(M, N, generator=g).bfloat16().cuda()
    x = torch.empty_like(gate)
    rc = _lib.load().cobalt_swiglu(gate.data_ptr(), up.data_ptr(), x.data_ptr(), gate.numel(), act, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    got = fused.staged(_lib.IN_GLU, gate, up, act)
    assert got is not None and torch.equal(got[0], mod(x))
    got32 = fused.staged(_lib.IN_GLU, gate, up, act, out_fp32=True)
    assert torch.equal(got32[0], mod(x, out_fp32=True))
    xf = gate.float()
    a = torch.nn.functional.silu(xf) if act == 0 else torch.nn.functional.gelu(xf, approximate="tanh")
    assert float((x.float() - a.bfloat16().float() * up.float()).abs().max()) <= 2.0 ** -6 * float(x.float().abs().max())


def test_staging_refuses_shapes_it_cannot_hold():
    """Eight tokens of 14336 values do not fit beside the weight ring: the fused entry point launches nothing and says so."""
    from cobalt_b200 import _lib
    from cobalt_b200.linear import FusedProjections
    raw = O.synth_raw(64, 14336, 0.5, 4, seed=3)
    fused = FusedProjections([to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)])
    gate = torch.zeros(8, 14336, dtype=torch.bfloat16, device="cuda")
    assert fused.staged(_lib.IN_GLU, gate, gate, 0) is None
    raw = O.synth_raw(64, 1152, 0.5, 4, seed=4)                   # 1152 = 4.5 * 256: rows the norm's sum order does not cover
    fused = FusedProjections([to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)])
    h = torch.zeros(1, 1152, dtype=torch.bfloat16, device="cuda")
    assert fused.staged(_lib.IN_ADDNORM, h, None, 0, w=h[0], eps=1e-5) is None
    raw = O.synth_raw(64, 4096, 0.5, 4, seed=5)                   # eight tokens: every CTA repeating the norm costs more than its kernel
    fused = FusedProjections([to_module(raw["keep"], raw["q"], raw["scale"], raw["zero"], 4)])
    h = torch.zeros(8, 4096, dtype=torch.bfloat16, device="cuda")
    assert fused.staged(_lib.IN_ADDNORM, h, None, 0, w=h[0], eps=1e-5) is None


class _LoopbackRanks:
    """`world` peer buffers on ONE GPU laid out like tp.PeerReducer's symmetric buffers, so that the pushing epilogue, the
    flags and the summing staging can be exercised rank after rank in one stream (no kernel ever waits for a kernel
    that has not been launched: every push precedes the sums)."""

    def __init__(self, world, max_floats):
        import ctypes
        from cobalt_b200 import _lib
        self.world = world
        self.stride = (max_floats * 4 + 255) // 256 * 256
        self.flags_off = (1 + 2 * world) * self.stride
        self.bufs = [torch.zeros((self.flags_off + 256) // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
        self._ptrs = (ctypes.c_uint64 * world)(*[b.data_ptr() for b in self.bufs])
        self.ranks = []
        for r in range(world):
            ns = type("Rank", (), {})()
            ns.slots = _lib.CobaltPeerSlots(ctypes.cast(self._ptrs, ctypes.c_void_p), r, world, self.stride, self.flags_off)
            self.ranks.append(ns)
        self.status = torch.zeros(64, dtype=torch.int32, device="cuda")

    def sum(self, rank, n, dtype=torch.bfloat16):
        import ctypes
        from cobalt_b200 import _lib
        out = torch.empty(n, dtype=dtype, device="cuda")
        rc = _lib.load().cobalt_peer_sum(ctypes.byref(self.ranks[rank].slots), n, out.data_ptr(), 1 if dtype == torch.float32 else 0,
                                         self.status.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert rc == 0
        return out


@pytest.mark.parametrize("world,M", [(1, 1), (2, 1), (2, 4), (4, 8)])
def test_pushed_partials_and_summing_staging(world, M):
    """Row-parallel projection split over `world` column shards, every shard's GEMV pushing its fp32 partial into every
    rank's slot; then (a) cobalt_peer_sum and (b) the next projection's staging that adds the partials, joins the
    residual and normalises.  Against: fp32 partials added in rank order and rounded once, then the separate kernels.
    Three rounds, so both slots and several epochs are used."""
    from cobalt_b200 import _lib, tp
    from cobalt_b200.linear import FusedProjections
    K, N = 512, 1024 * world
    raw = O.synth_raw(K, N, 0.5, 4, seed=900 + world)
    keep, q, sc, zr = raw["keep"], raw["q"], raw["scale"], raw["zero"]
    shards = []
    for r in range(world):
        k, qq, s_, z = tp.shard_raw("row", keep, q, sc, zr, r, world)
        shards.append(to_module(k, qq, s_, z, 4))
    pushers = [FusedProjections([m]) for m in shards]
    nxt_raw = O.synth_raw(128, K, 0.5, 4, seed=77)
    nxt = FusedProjections([to_module(nxt_raw["keep"], nxt_raw["q"], nxt_raw["scale"], nxt_raw["zero"], 4)])
    ranks = _LoopbackRanks(world, M * K)
    g = torch.Generator().manual_seed(world * 10 + M)
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).bfloat16().cuda()
    for rnd in range(3):
        x = torch.randn(M, N, generator=g).bfloat16().cuda()
        h = torch.randn(M, K, generator=g).bfloat16().cuda()
        parts = []
        for r in range(world):
            c0, c1 = tp.shard_bounds(N, r, world, 128)
            xr = x[:, c0:c1].contiguous()
            parts.append(shards[r](xr, out_fp32=True))
            assert pushers[r].staged(_lib.IN_PLAIN, xr, None, 0, push=ranks.ranks[r]) == []
        want32 = torch.zeros_like(parts[0])
        for p_ in parts:
            want32 = want32 + p_                                       # rank order, fp32
        want = want32.bfloat16()
        for r in range(world):
            assert torch.equal(ranks.sum(r, M * K).view(M, K), want), (rnd, r)
            assert torch.equal(ranks.sum(r, M * K, torch.float32).view(M, K), want32), (rnd, r)
        h_ref, x_ref = _separate_addnorm(h, want, w, None, 0, 1e-5)
        y_ref = nxt(x_ref)
        for r in range(world):
            h_out = torch.empty_like(h)
            got = nxt.staged(_lib.IN_ADDNORM, h, None, 0, w=w, h_out=h_out, eps=1e-5, delta_slots=ranks.ranks[r])
            assert got is not None
            assert torch.equal(h_out, h_ref) and torch.equal(got[0], y_ref[0]), (rnd, r)
    torch.cuda.synchronize()
    assert int(ranks.status[0]) == 0
    for m in shards:
        assert m.device_status() == 0


def test_zz_exemption_summary():
    """Collected after the other tests of this file: how often the rounding-boundary exemption was used."""
    total = sum(t for _, t in EXEMPT)
    used = sum(e for e, _ in EXEMPT)
    print(f"rounding-boundary exemption used in {len(EXEMPT)} comparisons: {used} of {total} elements")
    assert used <= max(16, int(MAX_EXEMPT * max(total, 1)))
