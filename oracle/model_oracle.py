"""Executable specification of the decoders that call the compressed linears
(Mistral / Llama family and Gemma-3 text), restated from the reference.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows src/cobaltkernel/ref_llama.py:82-195 and the dtype policy stated at its top
(:10-16): RMSNorm normalises in fp32, casts to bf16 and then multiplies by ``w``;
RoPE tables are computed in fp32 and cast to bf16; attention scores and the context
product are bf16 matmuls with an fp32 softmax cast back to bf16; SwiGLU and the
residual adds are bf16; no embedding scale; untied ``lm_head``.

Gemma-3 follows src/cobaltkernel/ref_gemma3.py:138-294: RMSNorm multiplies by ``(1 + w)`` in fp32 and
casts once; q and k get a per-head RMSNorm before RoPE; every branch is normalised again before it
is added to the residual (four norms per layer); the MLP is GeGLU with the tanh GELU; embeddings are
scaled by ``bf16(sqrt(hidden))``; sliding-window and full-attention layers alternate and use
different RoPE bases; the attention scale is ``query_pre_attn_scalar ** -0.5``; the head is tied.

Weights are a plain dict ``{hf_parameter_name: tensor}``; every linear weight is the
dense dequantised ``[out, in]`` matrix in bf16, which is what the reference's module
multiplies with (benchmarks/benchmark_suite.py:1211-1214).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

# Control switch (src/cobaltkernel/verify_kernel.py:160-169, 262-285 runs the same oracle code under a
# second, equally legitimate arithmetic to measure what accumulation order alone does to the logits):
# when set, every linear accumulates in fp32 from upcast operands and rounds once to bf16.
EXACT_LINEAR = False


def _linear(x, w):
    if EXACT_LINEAR:
        return torch.matmul(x.float(), w.float().t()).to(x.dtype)
    return F.linear(x, w)


def llama_config(hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128, inter=14336, vocab=32000,
                 eps=1e-5, theta=1e6, sliding_window=None):
    """Config fields read by src/cobaltkernel/ref_llama.py:26-54."""
    return dict(model_type="mistral", hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, vocab_size=vocab,
                rms_norm_eps=eps, rope_theta=theta, sliding_window=sliding_window)


def gemma3_config(hidden=5376, layers=62, heads=32, kv_heads=16, head_dim=128, inter=21504, vocab=262144, eps=1e-6,
                  sliding_window=1024, pattern=6, query_pre_attn_scalar=168, rope_theta=1e6, rope_local_base_freq=1e4,
                  rope_scaling=None):
    """Config fields read by src/cobaltkernel/ref_gemma3.py:40-87 (old dialect).  Defaults: Gemma-3-27B text."""
    return dict(model_type="gemma3_text", hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, vocab_size=vocab,
                rms_norm_eps=eps, sliding_window=sliding_window, sliding_window_pattern=pattern,
                query_pre_attn_scalar=query_pre_attn_scalar, rope_theta=rope_theta,
                rope_local_base_freq=rope_local_base_freq, rope_scaling=rope_scaling, tie_word_embeddings=True)


def gemma3_layer_types(cfg):
    """src/cobaltkernel/ref_gemma3.py:57-67: every `pattern`-th layer attends globally."""
    if cfg.get("layer_types"):
        return list(cfg["layer_types"])
    pat = cfg.get("sliding_window_pattern", 6)
    return ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(cfg["num_hidden_layers"])]


def gemma3_inv_freq(cfg, layer_type, device):
    """src/cobaltkernel/ref_gemma3.py:70-101: local base for sliding layers; global base, optionally with linear scaling."""
    D = cfg["head_dim"]
    if layer_type == "sliding_attention":
        return inv_freq(float(cfg.get("rope_local_base_freq", 1e4)), D, device)
    inv = inv_freq(float(cfg.get("rope_theta", 1e6)), D, device)
    sc = cfg.get("rope_scaling")
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        if kind == "linear":
            inv = inv / float(sc["factor"])
        elif kind != "default":
            raise NotImplementedError(kind)
    return inv


def gemma_rms_norm(x, w, eps):
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return (h * (1.0 + w.float())).to(x.dtype)


def inv_freq(theta, head_dim, device):
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))


def rms_norm(x, w, eps):
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return w * h.to(x.dtype)


def rotate_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def rope_tables(inv, positions, dtype):
    freqs = positions.float()[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x, cos, sin):
    return (x * cos[None, None]) + (rotate_half(x) * sin[None, None])


def _repeat_kv(x, n):
    if n == 1:
        return x
    b, h, t, d = x.shape
    return x[:, :, None].expand(b, h, n, t, d).reshape(b, h * n, t, d)


def _attention(cfg, W, p, h, cos, sin, kv, positions):
    T, D = h.shape[1], cfg["head_dim"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    q = _linear(h, W[p + "self_attn.q_proj.weight"]).view(1, T, nh, D).transpose(1, 2)
    k = _linear(h, W[p + "self_attn.k_proj.weight"]).view(1, T, nkv, D).transpose(1, 2)
    v = _linear(h, W[p + "self_attn.v_proj.weight"]).view(1, T, nkv, D).transpose(1, 2)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    kv["k"] = k if kv["k"] is None else torch.cat([kv["k"], k], dim=2)
    kv["v"] = v if kv["v"] is None else torch.cat([kv["v"], v], dim=2)
    Kc, Vc = kv["k"], kv["v"]
    S = Kc.shape[2]
    att = torch.matmul(q, _repeat_kv(Kc, nh // nkv).transpose(2, 3)) * (float(D) ** -0.5)
    kv_pos = torch.arange(S, device=q.device)
    allowed = kv_pos[None, :] <= positions[:, None]
    if cfg.get("sliding_window"):
        allowed &= kv_pos[None, :] > positions[:, None] - cfg["sliding_window"]
    att = att.masked_fill(~allowed[None, None], float("-inf"))
    att = F.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(att, _repeat_kv(Vc, nh // nkv)).transpose(1, 2).reshape(1, T, -1)
    return _linear(out, W[p + "self_attn.o_proj.weight"])


def _mlp(W, p, h):
    g = _linear(h, W[p + "mlp.gate_proj.weight"])
    u = _linear(h, W[p + "mlp.up_proj.weight"])
    return _linear(F.silu(g) * u, W[p + "mlp.down_proj.weight"])


def new_kv(cfg):
    return [{"k": None, "v": None} for _ in range(cfg["num_hidden_layers"])]


def _gemma3_attention(cfg, W, p, h, cos, sin, kv, positions, sliding):
    T, D = h.shape[1], cfg["head_dim"]
    nh, nkv, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["rms_norm_eps"]
    q = _linear(h, W[p + "self_attn.q_proj.weight"]).view(1, T, nh, D).transpose(1, 2)
    k = _linear(h, W[p + "self_attn.k_proj.weight"]).view(1, T, nkv, D).transpose(1, 2)
    v = _linear(h, W[p + "self_attn.v_proj.weight"]).view(1, T, nkv, D).transpose(1, 2)
    q = gemma_rms_norm(q, W[p + "self_attn.q_norm.weight"], eps)
    k = gemma_rms_norm(k, W[p + "self_attn.k_norm.weight"], eps)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    kv["k"] = k if kv["k"] is None else torch.cat([kv["k"], k], dim=2)
    kv["v"] = v if kv["v"] is None else torch.cat([kv["v"], v], dim=2)
    Kc, Vc = kv["k"], kv["v"]
    S = Kc.shape[2]
    att = torch.matmul(q, _repeat_kv(Kc, nh // nkv).transpose(2, 3)) * (float(cfg["query_pre_attn_scalar"]) ** -0.5)
    kv_pos = torch.arange(S, device=q.device)
    allowed = kv_pos[None, :] <= positions[:, None]
    if sliding:
        allowed &= kv_pos[None, :] > positions[:, None] - cfg["sliding_window"]
    att = att.masked_fill(~allowed[None, None], float("-inf"))
    att = F.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
    out = torch.matmul(att, _repeat_kv(Vc, nh // nkv)).transpose(1, 2).reshape(1, T, -1)
    return _linear(out, W[p + "self_attn.o_proj.weight"])


def _run_gemma3(cfg, W, ids, positions, kv):
    eps = cfg["rms_norm_eps"]
    e = W["model.embed_tokens.weight"][ids]
    scale = torch.tensor(float(cfg["hidden_size"]) ** 0.5, dtype=e.dtype, device=e.device)      # rounded to bf16 first
    h = (e * scale).unsqueeze(0)
    types = gemma3_layer_types(cfg)
    tables = {lt: rope_tables(gemma3_inv_freq(cfg, lt, h.device), positions, h.dtype) for lt in set(types)}
    for i, lt in enumerate(types):
        p = f"model.layers.{i}."
        cos, sin = tables[lt]
        x = gemma_rms_norm(h, W[p + "input_layernorm.weight"], eps)
        x = _gemma3_attention(cfg, W, p, x, cos, sin, kv[i], positions, lt == "sliding_attention")
        h = h + gemma_rms_norm(x, W[p + "post_attention_layernorm.weight"], eps)
        x = gemma_rms_norm(h, W[p + "pre_feedforward_layernorm.weight"], eps)
        g = _linear(x, W[p + "mlp.gate_proj.weight"])
        u = _linear(x, W[p + "mlp.up_proj.weight"])
        x = _linear(F.gelu(g, approximate="tanh") * u, W[p + "mlp.down_proj.weight"])
        h = h + gemma_rms_norm(x, W[p + "post_feedforward_layernorm.weight"], eps)
    h = gemma_rms_norm(h, W["model.norm.weight"], eps)
    return F.linear(h, W["model.embed_tokens.weight"])                                          # tied head


@torch.no_grad()
def run(cfg, W, ids, positions, kv):
    """Logits ``[1, T, vocab]`` for tokens ``ids`` at ``positions``; ``kv`` is extended in place."""
    if cfg.get("model_type") == "gemma3_text":
        return _run_gemma3(cfg, W, ids, positions, kv)
    h = W["model.embed_tokens.weight"][ids].unsqueeze(0)
    inv = inv_freq(float(cfg["rope_theta"]), cfg["head_dim"], h.device)
    cos, sin = rope_tables(inv, positions, h.dtype)
    eps = cfg["rms_norm_eps"]
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        x = rms_norm(h, W[p + "input_layernorm.weight"], eps)
        h = h + _attention(cfg, W, p, x, cos, sin, kv[i], positions)
        x = rms_norm(h, W[p + "post_attention_layernorm.weight"], eps)
        h = h + _mlp(W, p, x)
    h = rms_norm(h, W["model.norm.weight"], eps)
    return F.linear(h, W["lm_head.weight"])


def prefill(cfg, W, ids):
    kv = new_kv(cfg)
    pos = torch.arange(ids.shape[0], device=ids.device)
    return run(cfg, W, ids, pos, kv), kv


def forward_step(cfg, W, token_id, pos, kv):
    dev = W["model.embed_tokens.weight"].device
    ids = torch.tensor([token_id], device=dev, dtype=torch.long)
    return run(cfg, W, ids, torch.tensor([pos], device=dev), kv)[0, 0]


def teacher_forced(cfg, W, prompt_ids, tokens):
    """Logits [len(tokens), V] when the continuation `tokens` is fed back regardless of the argmax:
    row i is the distribution from which token i is drawn."""
    logits, kv = prefill(cfg, W, prompt_ids)
    rows = [logits[0, -1]]
    pos = prompt_ids.shape[0]
    for t in tokens[:-1]:
        rows.append(forward_step(cfg, W, int(t), pos, kv))
        pos += 1
    return torch.stack(rows)


def greedy(cfg, W, prompt_ids, n_new):
    """Prefill the prompt, then ``n_new`` greedy tokens.  Returns the token list and, per step,
    the margin between the two largest logits (a zero margin is an exact tie:
    src/cobaltkernel/verify_kernel.py:341-358 allows a fork only there)."""
    logits, kv = prefill(cfg, W, prompt_ids)
    last = logits[0, -1].float()
    toks, margins = [], []
    pos = prompt_ids.shape[0]
    for _ in range(n_new):
        top2 = torch.topk(last, 2)
        toks.append(int(top2.indices[0]))
        margins.append(float(top2.values[0] - top2.values[1]))
        last = forward_step(cfg, W, toks[-1], pos, kv).float()
        pos += 1
    return toks, margins
