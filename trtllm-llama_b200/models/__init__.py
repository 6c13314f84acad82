"""Model registry: which class serves a model folder is decided by its ``config.json``.

``architecture_of`` reads the architecture's name (key ``architecture``, or the first of ``architectures``; a folder
written by ``builder.save_config`` has a ``builder_config`` section and is a LLaMA plugin engine).  ``load_model``
returns what the runtime needs to serve it:

  ragged-batch models (``LayerStackModel``)  -> served by ``inflight.InflightSession`` (paged pools, state slots,
                                                chunked prefill beside decode, the scheduler's ``generate``)
  ``llama`` engines                          -> ``(ModelConfig, engine tensors)`` for ``runtime.GenerationSession``
"""
from __future__ import annotations

import json
import os

_REGISTRY = {}


def register_model(*names):
    def deco(fn):
        for n in names:
            _REGISTRY[n.lower()] = fn
        return fn
    return deco


def registered_models():
    return sorted(_REGISTRY)


def architecture_of(config: dict) -> str:
    if "architecture" in config:
        return str(config["architecture"])
    if config.get("architectures"):
        return str(config["architectures"][0])
    if "builder_config" in config:
        return "llama"
    raise ValueError("config.json names no architecture")


def load_model(model_dir: str, dtype="bfloat16", device="cuda", **kw):
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    arch = architecture_of(config)
    try:
        loader = _REGISTRY[arch.lower()]
    except KeyError:
        raise ValueError(f"no model class is registered for architecture {arch!r} (known: {registered_models()})") from None
    return loader(model_dir, config, dtype=dtype, device=device, **kw)


@register_model("llama", "LlamaForCausalLM")
def _load_llama_engine(model_dir, config, dtype="float16", device="cuda", rank=0, **_):
    """An engine folder written by examples/llama_quant/build.py: (ModelConfig, tensors) for GenerationSession."""
    from .. import builder as B
    mc = B.model_config_from_json(os.path.join(model_dir, "config.json"), rank)
    tensors = B.deserialize_engine(os.path.join(model_dir, B.get_engine_name("llama", "float16", mc.tp_size, rank)), device)
    return mc, tensors


from . import duzizen, mimolix, nililix, zobasun  # noqa: E402,F401  (they register themselves)
