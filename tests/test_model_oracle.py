"""The decoder oracle must reproduce the reference's executable spec (ref_llama) on a tiny
random model: prefill logits, greedy tokens and per-step logits, bit for bit."""
import os

import numpy as np
import torch

from oracle import model_oracle as MO

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_model_fixture(name="golden_model.npz"):
    z = np.load(os.path.join(ROOT, "tests", "golden", name))
    W = {k: torch.from_numpy(z[k].copy()).view(torch.bfloat16) for k in z.files if not k.startswith("__")}
    return z, W


def test_llama_oracle_matches_reference(digests):
    z, W = load_model_fixture()
    cfg = digests["model_cfg"]
    ids = torch.from_numpy(z["__ids"])
    logits, kv = MO.prefill(cfg, W, ids)
    assert torch.equal(logits[0].view(torch.int16), torch.from_numpy(z["__prefill_logits"]))
    last = logits[0, -1]
    pos = ids.shape[0]
    for i, tok in enumerate(z["__tokens"].tolist()):
        assert int(last.float().argmax()) == tok
        last = MO.forward_step(cfg, W, tok, pos, kv)
        assert torch.equal(last.view(torch.int16), torch.from_numpy(z["__step_logits"][i]))
        pos += 1
    toks, margins = MO.greedy(cfg, W, ids, 6)
    assert toks == z["__tokens"].tolist() and min(margins) >= 0


def test_gemma3_oracle_matches_reference(digests):
    """Same pin for the Gemma-3 spec (src/cobaltkernel/ref_gemma3.py): sliding + full layers, q/k norms, four norms per
    layer, GeGLU, scaled embeddings, tied head, linear RoPE scaling, a window that cuts the context."""
    z, W = load_model_fixture("golden_model_gemma3.npz")
    cfg = digests["gemma3_cfg"]
    ids = torch.from_numpy(z["__ids"])
    logits, kv = MO.prefill(cfg, W, ids)
    assert torch.equal(logits[0].view(torch.int16), torch.from_numpy(z["__prefill_logits"]))
    last = logits[0, -1]
    pos = ids.shape[0]
    for i, tok in enumerate(z["__tokens"].tolist()):
        assert int(last.float().argmax()) == tok
        last = MO.forward_step(cfg, W, tok, pos, kv)
        assert torch.equal(last.view(torch.int16), torch.from_numpy(z["__step_logits"][i]))
        pos += 1
