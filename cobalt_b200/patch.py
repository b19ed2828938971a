"""Swap ``nn.Linear`` layers of a model for ``CobaltSparseLinear``.

Follows the traversal of the reference's HQQ-style patcher (sinq/patch_model.py:47-87,
239-265): visit ``named_modules()``, take leaf modules whose type is a linear type, derive
the tag by dropping ``model`` / ``layers`` / numeric path components
(``model.layers.31.self_attn.k_proj`` -> ``self_attn.k_proj``), look the tag up in the
per-tag parameters (``None`` leaves the layer dense) and ``setattr`` the replacement on the
parent.  ``lm_head`` is ignored by default (sinq/patch_model.py:49, sinq/cpr_model.py:612-706)
and the model is marked so that patching twice is a no-op.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional, Union

import torch
import torch.nn as nn

from .compress import SparseQuantConfig
from .linear import CobaltSparseLinear

LINEAR_TYPES = (nn.Linear,)
IGNORE_LINEAR = ("lm_head",)


def find_parent(model: nn.Module, name: str) -> nn.Module:
    parent = model
    for part in name.split(".")[:-1]:
        parent = parent._modules[part]
    return parent


def is_leaf_module(module: nn.Module) -> bool:
    return len(module._modules) == 0


def name_to_linear_tag(name: str) -> str:
    return ".".join(p for p in name.split(".") if p not in ("model", "layers") and not p.isnumeric())


def get_linear_tags_from_model(model: nn.Module, ignore: Iterable[str] = IGNORE_LINEAR):
    tags = []
    for name, module in model.named_modules():
        if type(module) in LINEAR_TYPES and name.split(".")[-1] not in ignore:
            tag = name_to_linear_tag(name)
            if tag not in tags:
                tags.append(tag)
    return tags


def patch_linearlayers(model: nn.Module, patch_fct: Callable, patch_params: Optional[dict],
                       ignore: Iterable[str] = IGNORE_LINEAR) -> int:
    """Replace every eligible linear by ``patch_fct(module, params_for_its_tag, name)``.
    Returns the number of layers replaced."""
    targets = {}
    for name, module in model.named_modules():
        if name and type(module) in LINEAR_TYPES and is_leaf_module(module) and name.split(".")[-1] not in ignore:
            targets[name] = module
    n = 0
    for name, module in targets.items():
        tag = name_to_linear_tag(name)
        params = None
        if patch_params is not None:
            params = patch_params.get(tag, patch_params.get(name))
            if params is None:
                continue                       # reference: a tag without parameters stays dense
        setattr(find_parent(model, name), name.split(".")[-1], patch_fct(module, params, name))
        n += 1
    return n


def patch_model(model: nn.Module, cfg: Union[SparseQuantConfig, Dict[str, SparseQuantConfig]],
                act_norms: Optional[Dict[str, torch.Tensor]] = None,
                ignore: Iterable[str] = IGNORE_LINEAR) -> nn.Module:
    """Compress and replace the linear layers of ``model`` in place.

    ``cfg``        one configuration for every layer, or a dict tag -> configuration
                   (tags without an entry are left dense).
    ``act_norms``  module name -> per-input-channel activation norm ``[in_features]``
                   (the Wanda statistic); missing entries mean all ones.
    """
    if getattr(model, "cobalt_quantized", False):
        return model
    model.eval()
    for p in model.parameters():
        p.requires_grad = False
    for name, module in model.named_modules():
        module.name = name
    act_norms = act_norms or {}

    def fct(linear, params, name):
        return CobaltSparseLinear.from_linear(linear, act_norms.get(name), bits=params.bits, sparsity=params.sparsity,
                                              beta=params.beta, group_size=params.group_size)

    if isinstance(cfg, SparseQuantConfig):
        tags = get_linear_tags_from_model(model, ignore)
        params = {t: cfg for t in tags}
    else:
        params = dict(cfg)
    model.linear_tags = list(params.keys())
    patch_linearlayers(model, fct, params, ignore)
    model.cobalt_quantized = True
    return model
