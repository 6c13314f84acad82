"""Mimolix: a decoder-only stack of PARALLEL layers — one layer norm (weight and bias), then a sequence mixer and a
mixture-of-experts feed-forward side by side on its output, x <- x + m (mixer(h) + ff(h)) — whose mixers are either
differential attention (two softmax maps per head over shared values, RMS-normalised queries and keys, a query
temperature that grows with the logarithm of the position, no rotation) or a gated delta rule (short convolutions, unit
queries and keys, a matrix state per head).  The feed-forward routes by a softmax over all experts, renormalises the chosen
scores, runs squared-ReLU experts and adds a shared expert.  A block of layers runs several times with the same weights and
a cache / state of its own per pass; before each pass the stream is re-projected together with the embedding output.

``config.json``:
  architecture, vocab, width, embedding.scale, norm.eps, residual_mult, loop: {start, stop, times},
  layers[i] = {type: "attention" | "delta", mixer: {...}, mlp: null | {kind: "moe", expert: {ff}, router: {experts, top, scale},
               shared: null | {ff}}}
    attention mixer: heads, kv_heads, dim, vdim, scale, diff, q_temp: {coef, every}
    delta mixer:     heads, kv_heads, dim, vdim, conv (taps)
Tensors (``model.safetensors``, linear weights [out, in]): embed, head, final.norm, final.norm.b, loop.in [width, 2 width], and
per layer ``l<i>.``: norm1, norm1.b, mix.{q, k, v, q.norm, k.norm, lq1, lk1, lq2, lk2, o} or
mix.{q, k, v, q.conv, k.conv, v.conv, b, a, A_log, dt_bias, norm, g, o}, mlp.{router, e<j>.up, e<j>.down, shared.up, shared.down}.
This file only maps those names and keys onto the mechanisms of ``layers``; it holds no arithmetic."""
from __future__ import annotations

import os

import torch

from .. import ops
from ..checkpoint import read_safetensors
from ..layers import DifferentialAttention, GatedDeltaRule, LayerStackModel, RoutedExpertsMLP, SquaredReluMLP
from . import register_model

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def build_mimolix(config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda") -> LayerStackModel:
    """``tensors``: name -> CPU tensor as stored.  Everything is moved to ``device`` in ``dtype`` once, here."""
    dtype = _DTYPES[dtype]

    def t(name, optional=False):
        if name not in tensors:
            if optional:
                return None
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    eps = float(config["norm"]["eps"])
    layers = []
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        heads, kv_heads = int(m["heads"]), int(m.get("kv_heads", m["heads"]))
        dim, vdim = int(m["dim"]), int(m.get("vdim", m["dim"]))
        if lc["type"] == "attention":
            qt = m.get("q_temp") or {}
            mixer = DifferentialAttention(
                i, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=m["scale"], diff=m.get("diff", 0.0), eps=eps,
                temp_coef=qt.get("coef", 0.0), temp_every=qt.get("every", 0), w_q=t(p + "mix.q"), w_k=t(p + "mix.k"),
                w_v=t(p + "mix.v"), q_norm=t(p + "mix.q.norm"), k_norm=t(p + "mix.k.norm"), lq1=t(p + "mix.lq1"),
                lk1=t(p + "mix.lk1"), lq2=t(p + "mix.lq2"), lk2=t(p + "mix.lk2"), w_o=t(p + "mix.o"))
        elif lc["type"] == "delta":
            mixer = GatedDeltaRule(
                i, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, taps=int(m.get("conv", 1)), eps=eps, w_q=t(p + "mix.q"),
                w_k=t(p + "mix.k"), w_v=t(p + "mix.v"), conv_q=t(p + "mix.q.conv"), conv_k=t(p + "mix.k.conv"),
                conv_v=t(p + "mix.v.conv"), w_b=t(p + "mix.b"), w_a=t(p + "mix.a"), a_log=t(p + "mix.A_log"),
                dt_bias=t(p + "mix.dt_bias"), norm=t(p + "mix.norm"), w_g=t(p + "mix.g"), w_o=t(p + "mix.o"))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {lc['type']!r}")
        mlp, f = None, lc.get("mlp")
        if f is not None:
            if f.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f['kind']!r}")
            r = f["router"]
            ex = range(int(r["experts"]))
            shared = None
            if f.get("shared"):
                shared = SquaredReluMLP(w_up=t(p + "mlp.shared.up"), w_down=t(p + "mlp.shared.down"))
            mlp = RoutedExpertsMLP(
                w_router=t(p + "mlp.router"), w_up=torch.stack([t(f"{p}mlp.e{j}.up") for j in ex]),
                w_down=torch.stack([t(f"{p}mlp.e{j}.down") for j in ex]), top=r["top"], router="softmax", renorm=True,
                route_scale=r.get("scale", 1.0), act=ops.ACT_RELU_SQUARED, shared=shared)
        layers.append({"mixer": mixer, "mlp": mlp, "pre1": t(p + "norm1"), "pre1_b": t(p + "norm1.b")})
    lp = config.get("loop")
    looped = bool(lp) and lp["stop"] > lp["start"]
    return LayerStackModel(vocab=int(config["vocab"]), width=int(config["width"]), dtype=dtype, embed=t("embed"),
                           embed_scale=(config.get("embedding") or {}).get("scale", 1.0), layers=layers, final_norm=t("final.norm"),
                           final_norm_b=t("final.norm.b"), head=t("head"), eps=eps, residual_mult=config.get("residual_mult", 1.0),
                           norm="layer", parallel=True, loop=(lp["start"], lp["stop"], lp.get("times", 1)) if looped else None,
                           loop_in=t("loop.in", optional=True) if looped else None)


@register_model("Mimolix")
def _load(model_dir, config, dtype="bfloat16", device="cuda", **_):
    return build_mimolix(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype, device)
