"""Executable specification of the decoder that calls the compressed linears
(Mistral / Llama family), restated from the reference.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows src/cobaltkernel/ref_llama.py:82-195 and the dtype policy stated at its top
(:10-16): RMSNorm normalises in fp32, casts to bf16 and then multiplies by ``w``;
RoPE tables are computed in fp32 and cast to bf16; attention scores and the context
product are bf16 matmuls with an fp32 softmax cast back to bf16; SwiGLU and the
residual adds are bf16; no embedding scale; untied ``lm_head``.

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


@torch.no_grad()
def run(cfg, W, ids, positions, kv):
    """Logits ``[1, T, vocab]`` for tokens ``ids`` at ``positions``; ``kv`` is extended in place."""
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
    dev = W["lm_head.weight"].device
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
