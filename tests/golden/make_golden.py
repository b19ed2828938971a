"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/CoBALT

It imports the reference's own Python modules (nothing from this repository's
``oracle`` or ``cobalt_b200`` packages), evaluates them on seeded inputs and
writes ``golden_small.npz`` (full tensors for small matrices) and
``golden_digests.json`` (SHA-256 digests for the reference's own kernel-test
shapes, which are too large to store).  The tests never need the reference
checkout: they read only the files written here.
"""
import argparse
import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def sha(t):
    if isinstance(t, torch.Tensor):
        t = t.contiguous().cpu()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        t = t.numpy()
    return hashlib.sha256(np.ascontiguousarray(t).tobytes()).hexdigest()


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy().copy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    args = ap.parse_args()
    ref = args.reference
    sys.path.insert(0, os.path.join(ref, "src", "cobaltkernel"))
    sys.path.insert(0, os.path.join(ref, "src"))
    sys.path.insert(0, ref)
    import cobalt_math as cm                       # reference: mask + RTN
    import pack_cobalt as pc                       # reference: synthetic RAW generator
    from sinq.sparse_quant import dequantize_sparse_sinq
    os.environ.pop("PRISM_LOWMEM", None)
    from benchmarks.benchmark_suite import SparseQuantLinear

    out = {}
    cases = []
    # (name, K, N, bits, sparsity, beta, seed)
    specs = [
        ("c3s70", 64, 512, 3, 0.7, 0.5, 11),
        ("c4s50", 48, 384, 4, 0.5, 0.5, 12),
        ("c2s50", 32, 256, 2, 0.5, 0.5, 13),
        ("c3s60", 80, 640, 3, 0.6, 0.5, 14),
        ("c4s90_b0", 32, 256, 4, 0.9, 0.0, 15),     # very sparse rows: off-grid zero points, empty groups
        ("c4s00", 16, 128, 4, 0.0, 0.5, 16),        # sparsity 0: mask of ones
    ]
    for name, K, N, bits, sp, beta, seed in specs:
        g = torch.Generator().manual_seed(seed)
        W = (torch.randn(K, N, generator=g) * 0.02).half().float()
        norm = torch.randn(N, generator=g).abs() + 0.1
        if name == "c4s90_b0":
            W[3, 128:256] = W[3, 128:256].abs() + 0.01      # survivors all positive -> zero < 0
            W[5, 0:128] = -(W[5, 0:128].abs() + 0.01)       # survivors all negative -> zero > n_levels
        keep = cm.balanced_keepmask(W.abs() * norm.view(1, -1), sp, beta)
        q, sc, zr = cm.group_rtn(W, keep, bits, 128, "survivor")
        q = q * keep
        sc16, zr16 = sc.half(), zr.half()
        G = N // 128
        meta = {"nbits": bits, "group_size": 128, "shape": (K, N), "sparsity": sp}
        Wd = dequantize_sparse_sinq(q.half(), sc16.view(K, G, 1), zr16.view(K, G, 1), keep.half(),
                                    torch.ones(N).half(), meta)
        mod = SparseQuantLinear(q.half(), sc16.view(K, G, 1), zr16.view(K, G, 1), keep.half(),
                                torch.ones(N).half(), None, meta)
        ys = {}
        for M in (1, 4, 16):
            x = torch.randn(M, N, generator=g).to(torch.bfloat16)
            with torch.no_grad():
                y = mod(x)
            out[f"{name}.x{M}"] = bf16_bits(x)
            out[f"{name}.y{M}"] = bf16_bits(y)
        out[f"{name}.W"] = W.numpy()
        out[f"{name}.norm"] = norm.numpy()
        out[f"{name}.keep"] = keep.bool().numpy()
        out[f"{name}.q"] = q.to(torch.uint8).numpy()
        out[f"{name}.scale_f32"] = sc.numpy()
        out[f"{name}.zero_f32"] = zr.numpy()
        out[f"{name}.scale"] = sc16.numpy()
        out[f"{name}.zero"] = zr16.numpy()
        out[f"{name}.Wdeq"] = Wd.numpy()
        out[f"{name}.Wdeq_bf16"] = bf16_bits(Wd.to(torch.bfloat16))
        cases.append(dict(name=name, K=K, N=N, bits=bits, sparsity=sp, beta=beta, seed=seed))

    # a case with a column scale (scale2 != 1) and a bias
    K, N, bits = 32, 256, 4
    raw = pc.synth_raw_matrix(K, N, 0.5, bits, seed=99)
    keep = ((raw["mask"].view(K, N // 8, 1) >> torch.arange(8, dtype=torch.uint8)) & 1).view(K, N).bool()
    G = N // 128
    meta = {"nbits": bits, "group_size": 128, "shape": (K, N), "sparsity": 0.5}
    g = torch.Generator().manual_seed(100)
    bias = torch.randn(K, generator=g).to(torch.bfloat16)
    mod = SparseQuantLinear(raw["q"].half(), raw["scale"].view(K, G, 1), raw["zero"].view(K, G, 1),
                            keep.half(), raw["col_scale"], bias, meta)
    x = torch.randn(4, N, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        y = mod(x)
    out["colscale.keep"] = keep.numpy()
    out["colscale.q"] = raw["q"].numpy()
    out["colscale.scale"] = raw["scale"].numpy()
    out["colscale.zero"] = raw["zero"].numpy()
    out["colscale.col_scale"] = raw["col_scale"].numpy()
    out["colscale.bias"] = bf16_bits(bias)
    out["colscale.x4"] = bf16_bits(x)
    out["colscale.y4"] = bf16_bits(y)
    out["colscale.Wdeq_bf16"] = bf16_bits(mod._W_cached)

    np.savez_compressed(os.path.join(HERE, "golden_small.npz"), **out)

    # digests for the reference's own GEMV test shapes and seeds
    # (src/cobaltkernel/test_gemv.py:145: seed = K + N + layout, sparsity 0.5, 4 bits; layout 0 = SPARSE4)
    dig = {"cases": cases, "synth_raw": []}
    for (K, N) in [(256, 5376), (128, 21504), (192, 4096), (64, 1024)]:
        raw = pc.synth_raw_matrix(K, N, 0.5, 4, seed=K + N + 0)
        dig["synth_raw"].append(dict(K=K, N=N, bits=4, sparsity=0.5, seed=K + N,
                                     mask=sha(raw["mask"]), q=sha(raw["q"]), scale=sha(raw["scale"]),
                                     zero=sha(raw["zero"]), col_scale=sha(raw["col_scale"])))
    # config-1-shaped mask/RTN digest (4096 x 4096, 3 bit, 70 %), seed 1
    g = torch.Generator().manual_seed(1)
    K = N = 4096
    W = (torch.randn(K, N, generator=g) * 0.02).half().float()
    norm = torch.randn(N, generator=g).abs() + 0.1
    keep = cm.balanced_keepmask(W.abs() * norm.view(1, -1), 0.7, 0.5)
    q, sc, zr = cm.group_rtn(W, keep, 3, 128, "survivor")
    q = q * keep
    dig["config1"] = dict(K=K, N=N, bits=3, sparsity=0.7, beta=0.5, seed=1, nnz=int(keep.sum()),
                          keep=sha(keep.bool()), q=sha(q.to(torch.uint8)), scale=sha(sc.half()),
                          zero=sha(zr.half()))
    # tiny random Mistral-shaped model through the reference's executable spec
    # (src/cobaltkernel/ref_llama.py): logits of a prefill and greedy continuation
    import ref_llama as RL
    mcfg = dict(model_type="mistral", hidden_size=256, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=320,
                rms_norm_eps=1e-5, rope_theta=1e6)
    g = torch.Generator().manual_seed(2024)
    Wm = {}

    def rnd(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)
    Wm["model.embed_tokens.weight"] = rnd(320, 256, std=1.0)
    Wm["lm_head.weight"] = rnd(320, 256)
    Wm["model.norm.weight"] = (1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16)
    for i in range(2):
        pfx = f"model.layers.{i}."
        Wm[pfx + "input_layernorm.weight"] = (1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16)
        Wm[pfx + "post_attention_layernorm.weight"] = (1.0 + 0.1 * torch.randn(256, generator=g)).to(torch.bfloat16)
        Wm[pfx + "self_attn.q_proj.weight"] = rnd(256, 256)
        Wm[pfx + "self_attn.k_proj.weight"] = rnd(128, 256)
        Wm[pfx + "self_attn.v_proj.weight"] = rnd(128, 256)
        Wm[pfx + "self_attn.o_proj.weight"] = rnd(256, 256)
        Wm[pfx + "mlp.gate_proj.weight"] = rnd(512, 256)
        Wm[pfx + "mlp.up_proj.weight"] = rnd(512, 256)
        Wm[pfx + "mlp.down_proj.weight"] = rnd(256, 512)
    rcfg = RL.LlamaRefConfig(mcfg)
    state = {"cfg": rcfg, "W": Wm, "device": "cpu", "dtype": torch.bfloat16,
             "rope": {lt: RL._inv_freq(rcfg.rope_theta, rcfg.head_dim, "cpu") for lt in set(rcfg.layer_types)}}
    ids = torch.randint(0, 320, (12,), generator=g)
    logits, kvs = RL.prefill(state, ids)
    toks, step_logits = [], []
    last = logits[0, -1]
    pos = 12
    for _ in range(6):
        t = int(last.float().argmax())
        toks.append(t)
        last = RL.forward_step(state, t, pos, kvs)
        step_logits.append(bf16_bits(last))
        pos += 1
    mout = {k: (bf16_bits(v)) for k, v in Wm.items()}
    mout["__ids"] = ids.numpy()
    mout["__prefill_logits"] = bf16_bits(logits[0])
    mout["__tokens"] = np.array(toks)
    mout["__step_logits"] = np.stack(step_logits)
    np.savez_compressed(os.path.join(HERE, "golden_model.npz"), **mout)
    dig["model_cfg"] = mcfg

    # tiny random Gemma-3-shaped model through src/cobaltkernel/ref_gemma3.py: sliding and full layers, linear RoPE
    # scaling on the global base, a window short enough to cut the context
    import ref_gemma3 as RG
    gcfg = dict(model_type="gemma3_text", hidden_size=256, num_hidden_layers=3, num_attention_heads=4,
                num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=320, rms_norm_eps=1e-6,
                sliding_window=8, sliding_window_pattern=2, query_pre_attn_scalar=96, rope_theta=1e6,
                rope_local_base_freq=1e4, rope_scaling={"rope_type": "linear", "factor": 8.0}, tie_word_embeddings=True)
    g = torch.Generator().manual_seed(2025)
    Wg = {"model.embed_tokens.weight": rnd(320, 256, std=0.05), "model.norm.weight": rnd(256, std=0.1)}
    for i in range(3):
        pfx = f"model.layers.{i}."
        for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
            Wg[pfx + nm + ".weight"] = rnd(256, std=0.1)
        Wg[pfx + "self_attn.q_norm.weight"] = rnd(64, std=0.1)
        Wg[pfx + "self_attn.k_norm.weight"] = rnd(64, std=0.1)
        Wg[pfx + "self_attn.q_proj.weight"] = rnd(256, 256)
        Wg[pfx + "self_attn.k_proj.weight"] = rnd(128, 256)
        Wg[pfx + "self_attn.v_proj.weight"] = rnd(128, 256)
        Wg[pfx + "self_attn.o_proj.weight"] = rnd(256, 256)
        Wg[pfx + "mlp.gate_proj.weight"] = rnd(512, 256)
        Wg[pfx + "mlp.up_proj.weight"] = rnd(512, 256)
        Wg[pfx + "mlp.down_proj.weight"] = rnd(256, 512)
    gc = RG.Gemma3RefConfig(gcfg)
    Wfull = dict(Wg)
    Wfull["lm_head.weight"] = Wfull["model.embed_tokens.weight"]
    gstate = {"cfg": gc, "W": Wfull, "device": "cpu", "dtype": torch.bfloat16,
              "rope": {lt: RG._inv_freq(gc.rope_parameters[lt], gc.head_dim, "cpu") for lt in set(gc.layer_types)}}
    gids = torch.randint(0, 320, (12,), generator=g)
    glogits, gkv = RG.prefill(gstate, gids)
    gtoks, gsteps = [], []
    last = glogits[0, -1]
    pos = 12
    for _ in range(6):
        t = int(last.float().argmax())
        gtoks.append(t)
        last = RG.forward_step(gstate, t, pos, gkv)
        gsteps.append(bf16_bits(last))
        pos += 1
    gout = {k: bf16_bits(v) for k, v in Wg.items()}
    gout["__ids"] = gids.numpy()
    gout["__prefill_logits"] = bf16_bits(glogits[0])
    gout["__tokens"] = np.array(gtoks)
    gout["__step_logits"] = np.stack(gsteps)
    np.savez_compressed(os.path.join(HERE, "golden_model_gemma3.npz"), **gout)
    dig["gemma3_cfg"] = gcfg

    # plain group-128 RTN of the tied embedding / head matrix (src/cobaltkernel/pack_cobalt.py:375-386): small case in full
    g = torch.Generator().manual_seed(606)
    Wh = (torch.randn(96, 384, generator=g) * 0.02).to(torch.bfloat16)
    Wh[7, 128:256] = Wh[7, 128:256].abs() + 0.004             # a group without negative values: the hull still contains 0
    hq, hsc, hzr = pc.rtn_dense(Wh, 4)
    np.savez_compressed(os.path.join(HERE, "golden_head.npz"), W=bf16_bits(Wh), q=hq.to(torch.uint8).numpy(),
                        scale=hsc.numpy(), zero=hzr.numpy())

    # matrices above 32 M elements: the global threshold of the mask comes from the reference's bisection branch
    # (src/cobaltkernel/cobalt_math.py:79-101).  Digests only (the tensors are hundreds of megabytes).
    dig["large"] = []
    for (K, N, bits, sp, seed) in [(14336, 4096, 4, 0.5, 1004), (21504, 5376, 3, 0.6, 1005)]:
        g = torch.Generator().manual_seed(seed)
        W = (torch.randn(K, N, generator=g) * 0.02).half().float()
        norm = torch.randn(N, generator=g).abs() + 0.1
        keep = cm.balanced_keepmask(W.abs() * norm.view(1, -1), sp, 0.5)
        q, sc, zr = cm.group_rtn(W, keep, bits, 128, "survivor")
        q = q * keep
        dig["large"].append(dict(K=K, N=N, bits=bits, sparsity=sp, beta=0.5, seed=seed, nnz=int(keep.bool().sum()),   # bool: an fp32 sum of 0/1 rounds above 2**24
                                 keep=sha(keep.bool()), q=sha(q.to(torch.uint8)), scale=sha(sc.half()), zero=sha(zr.half())))
        del W, keep, q, sc, zr

    with open(os.path.join(HERE, "golden_digests.json"), "w") as f:
        json.dump(dig, f, indent=1)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
