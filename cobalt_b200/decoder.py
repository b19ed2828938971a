"""Minimal decoder (Mistral/Llama family and Gemma-3 text) that calls the compressed linears.

This is the caller side of the hot path (the seven projections of every block): residual add +
RMSNorm, RoPE + KV-cache append and SwiGLU are small fused CUDA kernels of the library;
grouped-query attention over the preallocated KV cache and the dense ``lm_head`` (the reference
leaves ``lm_head`` uncompressed: sinq/patch_model.py:49) are PyTorch matmuls.  The dtype policy follows the reference's executable spec
src/cobaltkernel/ref_llama.py:10-16, 82-143: fp32 normalise -> bf16 -> times w; bf16 RoPE
tables; bf16 score/context matmuls with an fp32 softmax cast back to bf16; bf16 residuals.
With ``model_type == "gemma3_text"`` the block follows src/cobaltkernel/ref_gemma3.py:138-294 instead:
``bf16(x * rr * (1 + w))`` norms, a per-head norm of q and k before RoPE, a second norm on every
branch before it joins the residual, GeGLU (tanh), embeddings times ``bf16(sqrt(hidden))``,
sliding-window and full-attention layers with their own RoPE bases, the attention scale
``query_pre_attn_scalar ** -0.5`` and a head tied to the embedding.

Tensor parallel (``tp_world > 1``, one process per GPU): every rank holds its heads' rows of q/k/v, its
columns of o, its rows of gate/up and its columns of down (``tp.shard_raw``); attention runs on the local
heads; the fp32 partial outputs of o and down are summed over ranks (peer-memory kernel for decode-sized
outputs, NCCL otherwise) and rounded once.  Norms, residuals, embedding and head are replicated.

One decode step has static shapes (attention runs over the whole cache with a position mask;
token id and position live in device tensors), so ``generate`` captures it once in a CUDA
graph and replays it per token with no host round trip.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .compress import SparseQuantConfig, compress_weight
from . import _lib
from .linear import CobaltSparseLinear, FusedProjections

PROJ = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
        "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")


def proj_shapes(cfg: dict) -> Dict[str, tuple]:
    H, D = cfg["hidden_size"], cfg["head_dim"]
    nh, nkv, I = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["intermediate_size"]
    return {"self_attn.q_proj": (nh * D, H), "self_attn.k_proj": (nkv * D, H), "self_attn.v_proj": (nkv * D, H),
            "self_attn.o_proj": (H, nh * D), "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}


def random_raw_layer(cfg: dict, layer: int, qcfg: SparseQuantConfig, device, seed0: int = 1000):
    """Seeded random weights of one block, compressed: {proj: (keep, q, scale, zero)} on `device`.
    Weights N(0, 0.02) stored as fp16, activation norms |N(0,1)| + 0.1 (seed ``seed0 + 7*layer + idx``)."""
    out = {}
    for idx, (name, (K, N)) in enumerate(proj_shapes(cfg).items()):
        g = torch.Generator().manual_seed(seed0 + layer * 7 + idx)
        W = (torch.randn(K, N, generator=g) * 0.02).half().float().to(device)
        norm = (torch.randn(N, generator=g).abs() + 0.1).to(device)
        out[name] = compress_weight(W, norm, qcfg)
    return out


def is_gemma(cfg: dict) -> bool:
    return cfg.get("model_type") == "gemma3_text"


def layer_types(cfg: dict):
    """Per-layer attention kind: Gemma-3 alternates (src/cobaltkernel/ref_gemma3.py:57-67); Llama is uniform."""
    L = cfg["num_hidden_layers"]
    if not is_gemma(cfg):
        return ["sliding_attention" if cfg.get("sliding_window") else "full_attention"] * L
    if cfg.get("layer_types"):
        return list(cfg["layer_types"])
    pat = cfg.get("sliding_window_pattern", 6)
    return ["sliding_attention" if (i + 1) % pat else "full_attention" for i in range(L)]


def rope_inv_freq(cfg: dict, layer_type: str, device):
    """fp32 inverse frequencies of one layer kind (src/cobaltkernel/ref_gemma3.py:70-101, src/cobaltkernel/ref_llama.py:56-60)."""
    D = cfg["head_dim"]
    base = float(cfg.get("rope_theta", 1e6))
    if is_gemma(cfg) and layer_type == "sliding_attention":
        base = float(cfg.get("rope_local_base_freq", 1e4))
    inv = 1.0 / (base ** (torch.arange(0, D, 2, dtype=torch.float32, device=device) / D))
    sc = cfg.get("rope_scaling") if is_gemma(cfg) and layer_type == "full_attention" else None
    if sc:
        kind = sc.get("rope_type", sc.get("type", "default"))
        if kind == "linear":
            inv = inv / float(sc["factor"])
        elif kind != "default":
            raise NotImplementedError(kind)
    return inv


def random_dense_params(cfg: dict, device, seed: int = 7):
    """Embedding, final norm, lm_head and per-layer norm weights (bf16), seeded.  Norm weights are the identity of
    their family: ones for Llama (``w * x``), small random values around zero for Gemma (``(1 + w) * x``)."""
    g = torch.Generator().manual_seed(seed)
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    if is_gemma(cfg):
        def nw(n):
            return (torch.randn(n, generator=g) * 0.05).to(torch.bfloat16).to(device)
        P = {"model.embed_tokens.weight": (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16).to(device),
             "model.norm.weight": nw(H)}
        for i in range(cfg["num_hidden_layers"]):
            pfx = f"model.layers.{i}."
            for nm in ("input_layernorm", "post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"):
                P[pfx + nm + ".weight"] = nw(H)
            P[pfx + "self_attn.q_norm.weight"] = nw(cfg["head_dim"])
            P[pfx + "self_attn.k_norm.weight"] = nw(cfg["head_dim"])
        return P
    P = {"model.embed_tokens.weight": (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16).to(device),
         "lm_head.weight": (torch.randn(V, H, generator=g) * 0.02).to(torch.bfloat16).to(device),
         "model.norm.weight": torch.ones(H, dtype=torch.bfloat16, device=device)}
    for i in range(cfg["num_hidden_layers"]):
        P[f"model.layers.{i}.input_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16, device=device)
        P[f"model.layers.{i}.post_attention_layernorm.weight"] = torch.ones(H, dtype=torch.bfloat16, device=device)
    return P


class _PendingSum:
    """Output [T, K] of a row-parallel projection whose fp32 partial sums sit in every rank's peer slot, not added yet."""
    __slots__ = ("T", "K")

    def __init__(self, T: int, K: int):
        self.T, self.K = T, K


class CobaltDecoder:
    """Decoder over compressed projections for ``batch`` independent sequences (each with its own KV cache; up to 16,
    the token limit of the decode GEMV).  ``linears[(layer, proj)]`` are ``CobaltSparseLinear`` modules; ``dense`` holds
    embedding / norms / lm_head.  ``head`` (optional) is the head as a compressed module - group-128 RTN without a mask,
    the reference's recipe for the tied embedding / head (src/cobaltkernel/pack_cobalt.py:375-386, 538-558); with tensor
    parallelism it holds this rank's slice of the vocabulary and the logits are gathered over the ranks."""

    def __init__(self, cfg: dict, linears: Dict[tuple, CobaltSparseLinear], dense: Dict[str, torch.Tensor],
                 max_ctx: int, device, tp_world: int = 1, reducer=None, group=None, batch: int = 1,
                 head: Optional[CobaltSparseLinear] = None, fuse_steps: bool = True):
        self.cfg, self.lin, self.P, self.max_ctx, self.dev = cfg, linears, dense, max_ctx, device
        self.world, self.reducer, self.group = tp_world, reducer, group
        self.head, self.B = head, int(batch)
        if not 1 <= self.B <= 16:
            raise ValueError("batch must be between 1 and 16 sequences")
        self.fused_prompt_attention = False
        if cfg["num_attention_heads"] % tp_world or cfg["num_key_value_heads"] % tp_world:
            raise ValueError("heads must split evenly over the tensor-parallel ranks")
        self.nh, self.nkv = cfg["num_attention_heads"] // tp_world, cfg["num_key_value_heads"] // tp_world   # local heads
        L, nkv, D = cfg["num_hidden_layers"], self.nkv, cfg["head_dim"]
        self.k_cache = torch.zeros(L, self.B, nkv, max_ctx, D, dtype=torch.bfloat16, device=device)     # [layer][sequence][kv head][slot][D]
        self.v_cache = torch.zeros(L, self.B, nkv, max_ctx, D, dtype=torch.bfloat16, device=device)
        self.seq_stride = nkv * max_ctx * D                                    # elements of one sequence's cache in a layer
        self.gemma = is_gemma(cfg)
        self.types = layer_types(cfg)
        self.inv_freq = {lt: rope_inv_freq(cfg, lt, device) for lt in set(self.types)}
        self.scale = float(cfg["query_pre_attn_scalar"]) ** -0.5 if self.gemma else float(D) ** -0.5
        if self.gemma:
            self.embed_scale = torch.tensor(float(cfg["hidden_size"]) ** 0.5, dtype=torch.bfloat16, device=device)
        self.kv_pos = torch.arange(max_ctx, device=device)
        need = _lib.load().cobalt_attn_decode_scratch_bytes(self.nh, D, max_ctx) * self.B
        self.att_scratch = torch.empty(need, dtype=torch.uint8, device=device) if self.nh // self.nkv <= 8 and D % 64 == 0 and D <= 256 \
            and max_ctx <= 65536 else None
        # One-kernel attention (cooperative launch; its scratch starts zeroed; only while its whole grid fits on the GPU).
        # Off by default: bit-identical to the three kernels but slower inside the decode graph (4-layer 7B-shaped step
        # 0.574 ms against 0.524 ms) - a cooperative launch does not overlap its neighbours.  Set the flag before the
        # first decode step to use it.
        self.att_fused = None
        self.one_kernel_attention = False
        self.tok = torch.zeros(self.B, dtype=torch.long, device=device)   # next token of every sequence
        self.pos = torch.zeros(self.B, dtype=torch.long, device=device)   # its position
        self.qkv = [FusedProjections([linears[(i, "self_attn.q_proj")], linears[(i, "self_attn.k_proj")],
                                      linears[(i, "self_attn.v_proj")]]) for i in range(L)]
        self.gate_up = [FusedProjections([linears[(i, "mlp.gate_proj")], linears[(i, "mlp.up_proj")]]) for i in range(L)]
        # Element-wise steps folded into the next projection's activation staging for up to 8 tokens (residual add +
        # RMSNorm in front of q|k|v, gate|up and a compressed head; the gated activation in front of down): same results
        # bit for bit as the separate kernels, three launches fewer per layer.
        self.fuse_steps = bool(fuse_steps)
        # Tensor parallel: let the o / down GEMVs push their partial sums into every rank's slot and the next projection's
        # staging add them up (no all-reduce kernel at all).  Off by default: at two ranks the step measured 10.0 ms with it
        # against 9.1 ms with the copy-based peer kernel (one system-scope fence per CTA costs more than the launch it saves).
        self.push_partials = False
        self.down = [FusedProjections([linears[(i, "mlp.down_proj")]]) for i in range(L)]
        self.o_f = [FusedProjections([linears[(i, "self_attn.o_proj")]]) for i in range(L)]
        self.head_f = FusedProjections([head]) if head is not None else None
        self._lib = _lib.load()
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._logits = None

    # ------------------------------------------------------------------ fused element-wise steps (C ABI)
    def _add_rmsnorm(self, h, delta, w, w_branch=None):
        """(h + delta, rmsnorm(h + delta) * w); ``delta`` may be None.  Gemma: ``w_branch`` normalises ``delta`` first."""
        T, H = h.shape
        y = torch.empty_like(h)
        h_out = torch.empty_like(h) if delta is not None else h
        rc = self._lib.cobalt_add_rmsnorm(h.data_ptr(), None if delta is None else delta.data_ptr(), w.data_ptr(),
                                          h_out.data_ptr() if delta is not None else None, y.data_ptr(), T, H,
                                          float(self.cfg["rms_norm_eps"]), 1 if self.gemma else 0,
                                          None if (w_branch is None or delta is None) else w_branch.data_ptr(),
                                          torch.cuda.current_stream(self.dev).cuda_stream)
        _lib.check("cobalt_add_rmsnorm", rc)
        return h_out, y

    def _rope_kv(self, q, k, v, positions, layer, seq: Optional[int]):
        """``seq`` = the sequence the T tokens belong to, or None: token t belongs to sequence t (batched decode)."""
        cfg = self.cfg
        kc = self.k_cache[layer] if seq is None else self.k_cache[layer][seq]
        vc = self.v_cache[layer] if seq is None else self.v_cache[layer][seq]
        qn = kn = None
        if self.gemma:                                                                 # per-head norm of q and k, fused in
            qn = self.P[f"model.layers.{layer}.self_attn.q_norm.weight"].data_ptr()
            kn = self.P[f"model.layers.{layer}.self_attn.k_norm.weight"].data_ptr()
        rc = self._lib.cobalt_rope_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), positions.data_ptr(),
                                      self.inv_freq[self.types[layer]].data_ptr(),
                                      kc.data_ptr(), vc.data_ptr(), q.shape[0],
                                      self.nh, self.nkv, cfg["head_dim"], self.max_ctx, qn, kn, float(cfg["rms_norm_eps"]),
                                      self.seq_stride if seq is None else 0, torch.cuda.current_stream(self.dev).cuda_stream)
        _lib.check("cobalt_rope_kv", rc)

    def _attn_one(self, q, positions, layer, seq: Optional[int]):
        """Attention of one new token per sequence over cache slots 0..positions[b] (three small launches, lengths read on
        the device).  ``seq`` = a single sequence (q [1, nh*D]) or None = all ``batch`` sequences (q [B, nh*D])."""
        cfg = self.cfg
        ctx = torch.empty_like(q)
        window = int(cfg.get("sliding_window") or 0) if self.types[layer] == "sliding_attention" else 0
        kc = self.k_cache[layer] if seq is None else self.k_cache[layer][seq]
        vc = self.v_cache[layer] if seq is None else self.v_cache[layer][seq]
        if self.one_kernel_attention and self.att_scratch is not None:
            if self.att_fused is None:
                nf = self._lib.cobalt_attn_decode_fused_scratch_bytes(self.nh, self.nkv, cfg["head_dim"], self.max_ctx, self.B)
                self.att_fused = torch.zeros(nf, dtype=torch.uint8, device=self.dev)
            rc = self._lib.cobalt_attn_decode_fused(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), positions.data_ptr(),
                                                    self.att_fused.data_ptr(), self.att_fused.numel(), ctx.data_ptr(),
                                                    self.nh, self.nkv, cfg["head_dim"], self.max_ctx, window, self.scale,
                                                    q.shape[0], self.seq_stride if seq is None else 0,
                                                    torch.cuda.current_stream(self.dev).cuda_stream)
            if rc == 0:
                return ctx
            if rc != _lib.EUNSUPPORTED:
                _lib.check("cobalt_attn_decode_fused", rc)
            self.one_kernel_attention = False                 # the grid does not fit on this GPU at once: three kernels from now on
        rc = self._lib.cobalt_attn_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                          positions.data_ptr(), self.att_scratch.data_ptr(), self.att_scratch.numel(), ctx.data_ptr(),
                                          self.nh, self.nkv, cfg["head_dim"], self.max_ctx, window, self.scale,
                                          q.shape[0], self.seq_stride if seq is None else 0,
                                          torch.cuda.current_stream(self.dev).cuda_stream)
        _lib.check("cobalt_attn_decode", rc)
        return ctx

    def _row_parallel(self, lin, x):
        """o / down: the whole layer on one GPU; with tensor parallelism the sum over ranks of the local fp32 partials."""
        if self.world == 1:
            return lin(x)
        T, K = x.shape[0], lin.out_features
        if self.reducer is not None and T * K * 4 <= self.reducer.stride:
            lin(x, out_fp32=True, out=self.reducer.slot_view(T * K))
            return self.reducer.reduce(T * K, torch.empty(T * K, dtype=x.dtype, device=x.device)).view(T, K)
        import torch.distributed as dist
        acc = lin(x, out_fp32=True)
        dist.all_reduce(acc, group=self.group)
        return acc.to(x.dtype)

    def _swiglu(self, g, u):
        out = torch.empty_like(g)
        rc = self._lib.cobalt_swiglu(g.data_ptr(), u.data_ptr(), out.data_ptr(), g.numel(), 1 if self.gemma else 0,
                                     torch.cuda.current_stream(self.dev).cuda_stream)
        _lib.check("cobalt_swiglu", rc)
        return out

    def _can_push(self, T: int, K: int) -> bool:
        """Tensor parallel, few tokens: the projection's partial sums can go straight into every rank's peer slot."""
        return (self.world > 1 and self.reducer is not None and self.fuse_steps and self.push_partials and T <= 8
                and T * K * 4 <= self.reducer.stride)

    def _settled(self, delta):
        """A branch output as a tensor: partial sums that are still spread over the ranks' slots are added now."""
        if isinstance(delta, _PendingSum):
            n = delta.T * delta.K
            return self.reducer.sum_pushed(n, torch.empty(n, dtype=torch.bfloat16, device=self.dev)).view(delta.T, delta.K)
        return delta

    def _norm_then(self, fused: FusedProjections, h, delta, w, w_branch=None):
        """``(h + delta', outputs of the projections applied to RMSNorm(h + delta') * w)``: one launch when the kernel can
        normalise while it stages its activations, else the norm kernel followed by the projections.  ``delta`` may be a
        row-parallel output whose partial sums still sit in the ranks' slots: the staging then adds them up as well."""
        if delta is None:
            w_branch = None
        if self.fuse_steps and h.shape[0] <= 8:
            h_out = torch.empty_like(h) if delta is not None else None
            pending = isinstance(delta, _PendingSum)
            ys = fused.staged(_lib.IN_ADDNORM, h, None if pending else delta, 1 if self.gemma else 0, w=w, w_branch=w_branch,
                              h_out=h_out, eps=float(self.cfg["rms_norm_eps"]), delta_slots=self.reducer if pending else None)
            if ys is not None:
                return (h if delta is None else h_out), ys
        h, x = self._add_rmsnorm(h, self._settled(delta), w, w_branch)
        return h, fused(x)

    def _o_proj(self, layer: int, ctx):
        lin = self.lin[(layer, "self_attn.o_proj")]
        if self._can_push(ctx.shape[0], lin.out_features):
            if self.o_f[layer].staged(_lib.IN_PLAIN, ctx, None, 0, push=self.reducer) is not None:
                return _PendingSum(ctx.shape[0], lin.out_features)
        return self._row_parallel(lin, ctx)

    def _glu_down(self, layer: int, g, u):
        """down(act(g) * u), summed over the ranks with tensor parallelism; the activation is applied while the kernel
        stages its input when the shape allows, else by its own kernel."""
        lin = self.lin[(layer, "mlp.down_proj")]
        T, K = g.shape[0], lin.out_features
        if self.fuse_steps and T <= 8:
            act = 1 if self.gemma else 0
            if self.world == 1:
                ys = self.down[layer].staged(_lib.IN_GLU, g, u, act)
                if ys is not None:
                    return ys[0]
            elif self._can_push(T, K):
                if self.down[layer].staged(_lib.IN_GLU, g, u, act, push=self.reducer) is not None:
                    return _PendingSum(T, K)
        return self._row_parallel(lin, self._swiglu(g, u))

    # ------------------------------------------------------------------ one forward over T tokens
    def _head_logits(self, x: torch.Tensor) -> torch.Tensor:
        """Head: dense bf16 matmul, or the compressed head (GEMV up to 16 rows, tcgen05 GEMM above); with a vocabulary
        split over the ranks the local logits are gathered in rank order."""
        if self.head is None:
            w = self.P["model.embed_tokens.weight"] if self.gemma else self.P["lm_head.weight"]   # Gemma ties the head
            return F.linear(x, w)
        lg = self.head(x)
        if self.world > 1:
            import torch.distributed as dist
            parts = [torch.empty_like(lg) for _ in range(self.world)]
            dist.all_gather(parts, lg.contiguous(), group=self.group)
            lg = torch.cat(parts, dim=-1)
        return lg

    def _forward(self, ids: torch.Tensor, positions: torch.Tensor, attend_len: int, seq: Optional[int] = 0) -> torch.Tensor:
        """ids, positions: [T] device tensors.  Keys/values are written at ``positions``; attention
        looks at cache slots [0, attend_len) under the causal mask ``slot <= position``.  ``seq`` names the sequence
        whose cache is used; ``seq=None`` is the batched decode step: token t is the next token of sequence t."""
        cfg, P = self.cfg, self.P
        nh, nkv, D = self.nh, self.nkv, cfg["head_dim"]                                # heads of this rank
        T, rep, S = ids.shape[0], nh // nkv, attend_len
        h = P["model.embed_tokens.weight"].index_select(0, ids)                        # [T, H]
        if self.gemma:
            h = h * self.embed_scale                                                   # scale rounded to bf16 first
        causal = self.kv_pos[None, :S] <= positions[:, None]                           # [T, S]
        blocked, allowed_of = {}, {}
        for lt in set(self.types):
            allowed = causal
            if lt == "sliding_attention" and cfg.get("sliding_window"):
                allowed = allowed & (self.kv_pos[None, :S] > positions[:, None] - cfg["sliding_window"])
            blocked[lt] = ~allowed[None, :, None, :]                                   # [1, T, 1, S]
            allowed_of[lt] = allowed[None, None]                                       # [1, 1, T, S]
        scale = self.scale
        delta, delta_w = None, None                                                    # pending branch and (Gemma) its norm weight
        for i in range(cfg["num_hidden_layers"]):
            p = f"model.layers.{i}."
            h, (q, k, v) = self._norm_then(self.qkv[i], h, delta, P[p + "input_layernorm.weight"], delta_w)   # one launch for up to 8 tokens
            self._rope_kv(q, k, v, positions, i, seq)                                  # q in place, k/v into the caches
            if seq is not None:
                Kc, Vc = self.k_cache[i][seq][:, :S], self.v_cache[i][seq][:, :S]      # [nkv, S, D]
            if seq is None:                                                            # one new token per sequence
                if self.att_scratch is None:
                    raise NotImplementedError("batched decode needs the library's decode attention (head_dim % 64 == 0, <= 8 q heads per kv head)")
                ctx = self._attn_one(q, positions, i, None)
            elif T == 1 and self.att_scratch is not None:
                ctx = self._attn_one(q, positions, i, seq)
            elif self.fused_prompt_attention and T > 16:
                # opt-in for prompts: the library's fused attention (fp32 scores and softmax inside; no [T, S] score
                # tensor in memory).  It skips the spec's bf16 rounding of scores and probabilities; on a small model the
                # prefill logits then sit 7e-3 (rel-L2) from the spec against 2e-3 for a change of accumulation order,
                # which is why it is off by default.
                ctx = F.scaled_dot_product_attention(q.view(1, T, nh, D).transpose(1, 2), Kc.unsqueeze(0), Vc.unsqueeze(0),
                                                     attn_mask=allowed_of[self.types[i]], scale=scale, enable_gqa=True)
                ctx = ctx.transpose(1, 2).reshape(T, nh * D)
            elif T > 64:
                # prompts: one KV head at a time, so that its [T * rep, S] scores (bf16), probabilities (fp32, then bf16)
                # stay in the L2 cache between the element-wise passes; same arithmetic as below
                ctx = torch.empty(T, nkv, rep, D, dtype=q.dtype, device=q.device)
                q4 = q.view(T, nkv, rep, D)
                blk = blocked[self.types[i]][0]                                        # [T, 1, S]
                for hk in range(nkv):
                    att = torch.mm(q4[:, hk].reshape(T * rep, D), Kc[hk].t())
                    att.mul_(scale)
                    att.view(T, rep, S).masked_fill_(blk, float("-inf"))
                    pr = F.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype)
                    ctx[:, hk] = torch.mm(pr, Vc[hk]).view(T, rep, D)
                ctx = ctx.view(T, nh * D)
            else:
                # grouped-query attention as one batched matmul per KV head (no expanded copies of K/V)
                qg = q.view(T, nkv, rep, D).permute(1, 0, 2, 3).reshape(nkv, T * rep, D)
                att = torch.bmm(qg, Kc.transpose(1, 2)) * scale                        # bf16 scores, scaled in bf16
                att = att.view(nkv, T, rep, S).masked_fill(blocked[self.types[i]], float("-inf"))
                att = F.softmax(att, dim=-1, dtype=torch.float32).to(q.dtype).view(nkv, T * rep, S)
                ctx = torch.bmm(att, Vc).view(nkv, T, rep, D).permute(1, 0, 2, 3).reshape(T, nh * D)
            o = self._o_proj(i, ctx)
            if self.gemma:                                                             # the branch is normalised before it joins
                h, (g, u) = self._norm_then(self.gate_up[i], h, o, P[p + "pre_feedforward_layernorm.weight"],
                                            P[p + "post_attention_layernorm.weight"])
            else:
                h, (g, u) = self._norm_then(self.gate_up[i], h, o, P[p + "post_attention_layernorm.weight"])
            delta = self._glu_down(i, g, u)
            if self.gemma:
                delta_w = P[p + "post_feedforward_layernorm.weight"]
        if self.head_f is not None and self.world == 1:                                # final norm folded into the compressed head
            h, (lg,) = self._norm_then(self.head_f, h, delta, P["model.norm.weight"], delta_w)
            return lg.unsqueeze(0)
        h, x = self._add_rmsnorm(h, self._settled(delta), P["model.norm.weight"], delta_w)
        return self._head_logits(x).unsqueeze(0)                                            # [1, T, V]

    @torch.no_grad()
    def time_head_ms(self, reps: int = 20) -> float:
        """Device time of what a decode step spends outside the blocks: embedding lookup, final norm, head, argmax."""
        def once():
            h = self.P["model.embed_tokens.weight"].index_select(0, self.tok)
            _, y = self._add_rmsnorm(h, None, self.P["model.norm.weight"])
            return torch.argmax(self._head_logits(y).float(), dim=-1)

        for _ in range(3):
            once()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            once()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def _check_room(self, n_tokens: int, start: int = 0):
        if start < 0 or start + n_tokens > self.max_ctx:
            raise ValueError(f"{n_tokens} tokens from position {start} do not fit the KV cache of {self.max_ctx} slots")

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt(s), fill the cache(s), return the logits: ``ids [T]`` -> ``[T, V]`` (sequence 0), or
        ``ids [B, T]`` (one prompt per sequence, equal lengths) -> ``[B, T, V]``."""
        ids = ids.to(self.dev)
        single = ids.dim() == 1
        ids2 = ids.view(1, -1) if single else ids
        if ids2.shape[0] > self.B:
            raise ValueError(f"{ids2.shape[0]} prompts for a decoder built for {self.B} sequences")
        T = ids2.shape[1]
        self._check_room(T)
        pos = torch.arange(T, device=self.dev)
        logits = torch.stack([self._forward(ids2[b], pos, T, seq=b)[0] for b in range(ids2.shape[0])])
        self.pos.fill_(T)
        return logits[0] if single else logits

    @torch.no_grad()
    def step(self) -> torch.Tensor:
        """One decode step for the tokens in ``self.tok`` at ``self.pos`` (one per sequence); returns the logits
        (``[V]`` for a single sequence, else ``[B, V]``) and advances ``tok`` (greedy) and ``pos`` on the device."""
        if self.B == 1:
            logits = self._forward(self.tok, self.pos, self.max_ctx, seq=0)[0, 0]
            self.tok.copy_(torch.argmax(logits.float(), dim=-1, keepdim=True))
        else:
            logits = self._forward(self.tok, self.pos, self.max_ctx, seq=None)[0]
            self.tok.copy_(torch.argmax(logits.float(), dim=-1))
        self.pos.add_(1)
        return logits

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, n_new: int, use_graph: bool = True, teacher: Optional[torch.Tensor] = None):
        """Greedy continuation.  ``prompt [T]``: returns (tokens [n_new] on the CPU, logits of every step [n_new, V]);
        ``prompt [B, T]``: (tokens [n_new, B], logits [n_new, B, V]).  With ``teacher`` (token ids, ``[n_new]`` or
        ``[n_new, B]``), the fed-back token of step i is ``teacher[i]`` instead of the argmax (teacher-forced run,
        src/cobaltkernel/verify_kernel.py:288-339)."""
        single = prompt.dim() == 1
        if not single and prompt.shape[0] != self.B:
            raise ValueError(f"{prompt.shape[0]} prompts for a decoder built for {self.B} sequences")
        if single and self.B != 1:
            raise ValueError("a batched decoder needs one prompt per sequence: prompt [B, T]")
        self._check_room(int(prompt.shape[-1]) + n_new)      # the captured step advances the position on the device
        logits = self.prefill(prompt)
        last = logits[-1] if single else logits[:, -1]       # [V] or [B, V]
        first = torch.argmax(last.float(), dim=-1, keepdim=single)
        self.tok.copy_(first if teacher is None else teacher[0].reshape(-1).to(self.dev))
        toks = [first.clone()]
        all_logits = [last.clone()]
        if use_graph and self._graph is None:
            s = torch.cuda.Stream(self.dev)
            s.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(s):                       # warm-up outside capture (lazy inits, scratch)
                tok0, pos0 = self.tok.clone(), self.pos.clone()
                self.step()
                self.tok.copy_(tok0)
                self.pos.copy_(pos0)
            torch.cuda.current_stream(self.dev).wait_stream(s)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._logits = self.step()
        for i in range(1, n_new):
            if use_graph:
                self._graph.replay()
                lg = self._logits
            else:
                lg = self.step()
            toks.append(torch.argmax(lg.float(), dim=-1, keepdim=single).clone())
            all_logits.append(lg.clone())
            if teacher is not None:
                self.tok.copy_(teacher[i].reshape(-1).to(self.dev))
        toks = torch.cat(toks).cpu() if single else torch.stack(toks).cpu()
        return toks, torch.stack(all_logits)


def compress_head(dense: Dict[str, torch.Tensor], cfg: dict, bits: int, tp_rank: int = 0, tp_world: int = 1):
    """Replace the head (and, for a tied head, the embedding table) by its group-128 RTN version: returns the compressed
    module holding this rank's slice of the vocabulary.  The bf16 tensor in ``dense`` becomes the dequantised matrix, so
    that embedding lookups and any oracle see exactly the weights the compressed head multiplies by."""
    from .compress import quantize_dense
    key = "model.embed_tokens.weight" if is_gemma(cfg) else "lm_head.weight"
    W = dense[key]
    V = W.shape[0]
    if V % (16 * tp_world):
        raise ValueError("the vocabulary must split into multiples of 16 rows per rank")
    lo, hi = tp_rank * (V // tp_world), (tp_rank + 1) * (V // tp_world)
    head = CobaltSparseLinear.from_dense_rtn(W, bits, rows=slice(lo, hi))
    step = max(16, (1 << 25) // W.shape[1])
    for k0 in range(0, V, step):                              # dequantised copy, chunked: (q - z) * s in fp32, one rounding
        q, sc, zr = quantize_dense(W[k0:k0 + step], bits)
        G = sc.shape[1]
        wd = (q.float().view(q.shape[0], G, -1) - zr.float().unsqueeze(-1)) * sc.float().unsqueeze(-1)
        W[k0:k0 + step] = wd.view(q.shape[0], -1).to(torch.bfloat16)
    return head


def build_random_decoder(cfg: dict, qcfg: SparseQuantConfig, max_ctx: int, device, keep_raw: bool = False,
                         tp_rank: int = 0, tp_world: int = 1, reducer=None, group=None, clone_first_layer: bool = False,
                         batch: int = 1, head_bits: int = 0, fuse_steps: bool = True):
    """Random-init model of the given shape with every projection compressed.  Returns the decoder
    and, when ``keep_raw``, the RAW tensors per (layer, proj) for an oracle to dequantise.  With
    ``tp_world > 1`` every matrix is compressed whole (same seeds on every rank) and this rank keeps its shard.
    ``clone_first_layer`` compresses only layer 0 and gives every other layer its own copy of those packed bytes
    (for timing very large shapes: the bytes streamed per token are the same, the compression time is not).
    ``batch`` sequences decode together; ``head_bits`` (2..4) compresses the head with group-128 RTN and, with
    tensor parallelism, splits its vocabulary over the ranks."""
    from .format import TileImage
    from .tp import kind_of, shard_raw
    lin, raws = {}, {}
    for i in range(cfg["num_hidden_layers"]):
        if clone_first_layer and i > 0:
            for name in PROJ:
                src = lin[(0, name)]
                m = CobaltSparseLinear._blank()
                m._install(TileImage.from_meta(src.packed.clone(), src._img_meta), None, None, {"nbits": src.bits})
                lin[(i, name)] = m
            continue
        layer = random_raw_layer(cfg, i, qcfg, device)
        for name, (keep, q, sc, zr) in layer.items():
            if keep_raw:
                raws[(i, name)] = (keep, q, sc, zr)
            if tp_world > 1:
                keep, q, sc, zr = shard_raw(kind_of(name), keep, q, sc, zr, tp_rank, tp_world)
            lin[(i, name)] = CobaltSparseLinear(q, sc, zr, keep, None, None, {"nbits": qcfg.bits})
    dense = random_dense_params(cfg, device)
    head = compress_head(dense, cfg, head_bits, tp_rank, tp_world) if head_bits else None
    dec = CobaltDecoder(cfg, lin, dense, max_ctx, device, tp_world=tp_world, reducer=reducer, group=group, batch=batch, head=head,
                        fuse_steps=fuse_steps)
    return (dec, raws) if keep_raw else dec
