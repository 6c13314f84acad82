"""Duzizen: a decoder-only stack whose layers wrap every sublayer in two layer norms (weight and bias),
x <- x + LN_b(f(LN_a(x))), and whose sequence mixer is either an mLSTM matrix memory or a PAIR of mixers side by side — a
sliding-window grouped-query attention that keeps a sequence's first tokens visible (short convolutions on q and k, an RMS
norm over the whole q and the whole k projection, partial interleaved rotation with scaled frequencies, a softmax sink at
score 0, values that are the convolved keys) and a retention (fixed decay per head, rotate-half rotation) — whose normalised
outputs are averaged.  The feed-forward is a gated GELU or a mixture of clamped gated experts whose sigmoid router score weighs
the expert's input.  After its sublayers every layer adds a projection of its slice of a side embedding of the token, and the
token embedding itself is joined by a hashed embedding of the (previous, current) token pair.

``config.json``:
  architecture, vocab, width, norm.eps, embedding.bigram: {buckets, mul_prev, mul_cur}, token_side: {dim},
  layers[i] = {type: "mlstm" | "parallel", mixer: {...}, mlp: null | {kind: "dense", ff} | {kind: "moe", expert: {ff, limit},
               router: {experts, top}}}
    mlstm mixer:    heads, dim, vdim, gate_cap
    parallel mixer: left:  heads, kv_heads, dim, vdim, conv (taps), scale, mask: {size, keep_first}, rot: {base, dims, scaling: {factor,
                           low, high, original}}
                    right: heads, dim, vdim, decay [heads], rot: {base, dims}
Tensors (``model.safetensors``, linear weights [out, in]): embed, bigram [buckets + 1, width], side.embed [vocab, layers * dim], head,
final.norm, final.norm.b, and per layer ``l<i>.``: norm1, norm1b, norm2, norm2b (each with ``.b``), side.{gate, proj, norm},
mix.{q, k, v, g, o, norm, i, i.b, f, f.b} or mix.left.{q, k, q.conv, k.conv, q.norm, k.norm, o}, mix.right.{q, k, v, g, o},
mix.left.out, mix.right.out, and mlp.{gate, up, down} or mlp.{router, e<j>.gate, e<j>.up, e<j>.down}.
This file only maps those names and keys onto the mechanisms of ``layers``; it holds no arithmetic."""
from __future__ import annotations

import os

import torch

from ..checkpoint import read_safetensors
from ..layers import (ClampedGatedMLP, LayerStackModel, MatrixMemory, Retention, RoutedExpertsMLP, SideBySideMixers, TokenSideInput,
                      WindowedAttention)
from . import register_model

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}

# constants the design fixes
_EXPERT_ALPHA = 1.702          # experts: g * sigmoid(alpha g) * (u + shift)
_EXPERT_UP_SHIFT = 1.0
_MEMORY_DEN_EPS = 1e-6         # matrix memory: o / (max(|n . q|, exp(-m)) + this)
_SIDE_BY_SIDE_MULT = 0.5


def build_duzizen(config: dict, tensors: dict, dtype=torch.bfloat16, device="cuda") -> LayerStackModel:
    """``tensors``: name -> CPU tensor as stored.  Everything is moved to ``device`` in ``dtype`` once, here."""
    dtype = _DTYPES[dtype]

    def t(name, optional=False):
        if name not in tensors:
            if optional:
                return None
            raise KeyError(f"checkpoint has no tensor {name!r}")
        return tensors[name].to(device=device, dtype=dtype).contiguous()

    eps = float(config["norm"]["eps"])

    def rotation(m):
        rot = m.get("rot") or {}
        sc = rot.get("scaling")
        return dict(rot_dims=int(rot.get("dims", 0)), rot_base=rot.get("base", 10000.0),
                    rot_scaling=(sc["factor"], sc["low"], sc["high"], sc["original"]) if sc else None)

    def attention(i, p, m):
        heads, dim = int(m["heads"]), int(m["dim"])
        taps = int(m.get("conv", 1)) if (p + "q.conv") in tensors else 1
        mask = m.get("mask") or {}
        return WindowedAttention(
            i, heads=heads, kv_heads=int(m.get("kv_heads", heads)), dim=dim, vdim=int(m.get("vdim", dim)), taps=taps, scale=m["scale"],
            window=int(mask.get("size", 0)), keep_first=int(mask.get("keep_first", 0)), eps=eps, w_q=t(p + "q"), w_k=t(p + "k"),
            conv_q=t(p + "q.conv", optional=True), conv_k=t(p + "k.conv", optional=True), q_norm=t(p + "q.norm"), k_norm=t(p + "k.norm"),
            w_o=t(p + "o"), sink=torch.zeros(heads, dtype=torch.float32, device=device), **rotation(m))

    def retention(i, p, m):
        heads, dim = int(m["heads"]), int(m["dim"])
        return Retention(i, heads=heads, dim=dim, vdim=int(m.get("vdim", dim)), decay=m["decay"], eps=eps, k_scale=dim ** -0.5,
                         w_q=t(p + "q"), w_k=t(p + "k"), w_v=t(p + "v"), w_g=t(p + "g"), w_o=t(p + "o"), rot_layout="half", **rotation(m))

    side_cfg = config.get("token_side")
    side_embed = t("side.embed") if side_cfg else None
    layers = []
    for i, lc in enumerate(config["layers"]):
        p, m = f"l{i}.", lc["mixer"]
        if lc["type"] == "mlstm":
            heads, dim = int(m["heads"]), int(m["dim"])
            mixer = MatrixMemory(i, heads=heads, dim=dim, vdim=int(m.get("vdim", dim)), eps=eps, gate_cap=m.get("gate_cap", 0.0),
                                 den_eps=_MEMORY_DEN_EPS, w_q=t(p + "mix.q"), w_k=t(p + "mix.k"), w_v=t(p + "mix.v"), w_g=t(p + "mix.g"),
                                 w_i=t(p + "mix.i"), b_i=t(p + "mix.i.b"), w_f=t(p + "mix.f"), b_f=t(p + "mix.f.b"), norm=t(p + "mix.norm"),
                                 w_o=t(p + "mix.o"))
        elif lc["type"] == "parallel":
            mixer = SideBySideMixers(i, attention(i, p + "mix.left.", m["left"]), retention(i, p + "mix.right.", m["right"]),
                                     w_left=t(p + "mix.left.out"), w_right=t(p + "mix.right.out"), eps=eps, mult=_SIDE_BY_SIDE_MULT)
        else:
            raise ValueError(f"layer {i}: unknown mixer type {lc['type']!r}")
        mlp, f = None, lc.get("mlp")
        if f is not None:
            kind = f.get("kind", "dense")
            if kind == "dense":
                mlp = ClampedGatedMLP(w_gate=t(p + "mlp.gate"), w_up=t(p + "mlp.up"), w_down=t(p + "mlp.down"), gate="gelu_tanh")
            elif kind == "moe":
                r, ex = f["router"], range(int(f["router"]["experts"]))
                mlp = RoutedExpertsMLP(
                    w_router=t(p + "mlp.router"), w_gate=torch.stack([t(f"{p}mlp.e{j}.gate") for j in ex]),
                    w_up=torch.stack([t(f"{p}mlp.e{j}.up") for j in ex]), w_down=torch.stack([t(f"{p}mlp.e{j}.down") for j in ex]),
                    top=r["top"], router="sigmoid_groups", groups=1, keep=1, gate_alpha=_EXPERT_ALPHA,
                    gate_limit=(f.get("expert") or {}).get("limit", 0.0), gate_up_shift=_EXPERT_UP_SHIFT, weight_on="input")
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
        side = None
        if side_cfg:
            sd = int(side_cfg["dim"])
            side = TokenSideInput(side_embed=side_embed, offset=i * sd, w_gate=t(p + "side.gate"), w_proj=t(p + "side.proj"),
                                  norm=t(p + "side.norm"), eps=eps)
        layers.append({"mixer": mixer, "mlp": mlp, "side": side,
                       "pre1": t(p + "norm1"), "pre1_b": t(p + "norm1.b"), "post1": t(p + "norm1b"), "post1_b": t(p + "norm1b.b"),
                       "pre2": t(p + "norm2") if mlp else None, "pre2_b": t(p + "norm2.b") if mlp else None,
                       "post2": t(p + "norm2b") if mlp else None, "post2_b": t(p + "norm2b.b") if mlp else None})
    bg = (config.get("embedding") or {}).get("bigram")
    pair = None
    if bg:
        table = t("bigram")
        if table.shape[0] != int(bg["buckets"]) + 1:
            raise ValueError(f"pair embedding has {table.shape[0]} rows for {bg['buckets']} buckets and the row of first tokens")
        pair = (table, int(bg["mul_prev"]), int(bg["mul_cur"]))
    return LayerStackModel(vocab=int(config["vocab"]), width=int(config["width"]), dtype=dtype, embed=t("embed"), layers=layers,
                           final_norm=t("final.norm"), final_norm_b=t("final.norm.b"), head=t("head"), eps=eps, norm="layer",
                           embed_pair=pair)


@register_model("Duzizen")
def _load(model_dir, config, dtype="bfloat16", device="cuda", **_):
    return build_duzizen(config, read_safetensors(os.path.join(model_dir, "model.safetensors")), dtype, device)
