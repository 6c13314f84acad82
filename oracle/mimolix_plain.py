"""Plain float64 restatement of the Mimolix design (differential attention with normalised, temperature-scaled queries;
gated delta-rule layers with short convolutions; a softmax-routed mixture of squared-ReLU experts with a shared expert;
parallel layers under one layer norm; a looped block of layers that re-reads the embedding), written from the
equations and sharing no code with the product path.  Slow on purpose: whole sequences at once, explicit loops over
positions and heads, no cache, nothing carried between calls.  Test infrastructure only.

Notation: h [T, W] is one sequence, positions 0..T-1; ``P`` maps tensor names ('l3.mix.q', ...) to float64 tensors;
linear weights are [out, in] and applied as W x; ``cfg`` is the parsed configuration."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def short_conv(u, w):
    """u [T, C], w [C, taps]: the last tap weighs the current input, tap j the one ``taps - 1 - j`` positions back; inputs
    before position 0 are zero."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            back = taps - 1 - j
            if t - back >= 0:
                y[t] += w[:, j] * u[t - back]
    return y


def silu(x):
    return x * torch.sigmoid(x)


def query_temperature(p, coef, every):
    """The factor on the query at position p: it grows with the logarithm of the number of whole ``every``-blocks."""
    return 1.0 + coef * math.log((p + 1) // every + 1)


def causal_softmax_attention(q, k, v, scale):
    """q [T, d], k [T, d], v [T, dv] of one head and one map -> [T, dv]."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        s = (k[:i + 1] @ q[i]) * scale
        e = torch.exp(s - s.max())
        out[i] = (e / e.sum()) @ v[:i + 1]
    return out


def differential_lambda(P, pre, diff):
    return math.exp(float((P[pre + "lq1"] * P[pre + "lk1"]).sum())) - math.exp(float((P[pre + "lq2"] * P[pre + "lk2"]).sum())) + diff


def differential_attention_mixer(h, P, pre, mc, eps):
    T = h.shape[0]
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    diff = float(mc.get("diff", 0.0))
    q = (h @ P[pre + "q"].T).view(T, H, 2, d)
    k = (h @ P[pre + "k"].T).view(T, G, 2, d)
    v = (h @ P[pre + "v"].T).view(T, G, dv)
    q = rms(q, eps) * P[pre + "q.norm"]
    k = rms(k, eps) * P[pre + "k.norm"]
    qt = mc.get("q_temp")
    if qt:
        for p in range(T):
            q[p] = q[p] * query_temperature(p, qt["coef"], qt["every"])
    lam = differential_lambda(P, pre, diff)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        a1 = causal_softmax_attention(q[:, hd, 0], k[:, g, 0], v[:, g], mc["scale"])
        a2 = causal_softmax_attention(q[:, hd, 1], k[:, g, 1], v[:, g], mc["scale"])
        o[:, hd] = rms(a1 - lam * a2, eps) * (1.0 - diff)
    return o.reshape(T, H * dv) @ P[pre + "o"].T


def unit(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def delta_rule(q, k, v, beta, g):
    """One head: q, k [T, d], v [T, dv], beta, g [T].  S decays, is corrected towards v along k, and is read with q after
    the write."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out[t] = S.T @ q[t]
    return out


def delta_mixer(h, P, pre, mc, eps):
    T = h.shape[0]
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = silu(short_conv(h @ P[pre + "q"].T, P[pre + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ P[pre + "k"].T, P[pre + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ P[pre + "v"].T, P[pre + "v.conv"])).view(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    beta = torch.sigmoid(h @ P[pre + "b"].T)
    g = torch.exp(-torch.exp(P[pre + "A_log"]) * torch.nn.functional.softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    gate = silu(h @ P[pre + "g"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        j = hd // (H // G)
        o[:, hd] = rms(delta_rule(q[:, j], k[:, j], v[:, hd], beta[:, hd], g[:, hd]), eps) * P[pre + "norm"] * gate[:, hd]
    return o.reshape(T, H * dv) @ P[pre + "o"].T


def relu2_expert(h, up, down):
    return down @ (torch.relu(up @ h) ** 2)


def route(h, P, pre, rc):
    """-> per token (expert ids, weights): softmax over all experts, the ``top`` largest, renormalised, times scale."""
    s = torch.softmax(h @ P[pre + "router"].T, dim=-1)
    picks = []
    for t in range(h.shape[0]):
        ids = sorted(range(rc["experts"]), key=lambda e: (-float(s[t, e]), e))[:rc["top"]]
        tot = sum(float(s[t, e]) for e in ids) + 1e-20
        picks.append((ids, [float(s[t, e]) / tot * rc.get("scale", 1.0) for e in ids]))
    return picks


def moe_mlp(h, P, pre, fc):
    out = torch.zeros_like(h)
    for t, (ids, ws) in enumerate(route(h, P, pre, fc["router"])):
        for e, w in zip(ids, ws):
            out[t] += w * relu2_expert(h[t], P[f"{pre}e{e}.up"], P[f"{pre}e{e}.down"])
        if fc.get("shared"):
            out[t] += relu2_expert(h[t], P[pre + "shared.up"], P[pre + "shared.down"])
    return out


def layer(x, P, i, lc, cfg):
    m, eps, pre = cfg.get("residual_mult", 1.0), cfg["norm"]["eps"], f"l{i}."
    h = layer_norm(x, P[pre + "norm1"], P[pre + "norm1.b"], eps)
    if lc["type"] == "attention":
        y = differential_attention_mixer(h, P, pre + "mix.", lc["mixer"], eps)
    elif lc["type"] == "delta":
        y = delta_mixer(h, P, pre + "mix.", lc["mixer"], eps)
    else:
        raise ValueError(lc["type"])
    if lc.get("mlp"):
        y = y + moe_mlp(h, P, pre + "mlp.", lc["mlp"])
    return x + m * y


def layer_runs(cfg):
    """[(layer index, pass number, first of its pass)] in execution order."""
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp or lp["stop"] <= lp["start"]:
        return [(i, 0, False) for i in range(n)]
    runs = [(i, 0, False) for i in range(lp["start"])]
    for t in range(lp["times"]):
        runs += [(i, t, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, 0, False) for i in range(lp["stop"], n)]


def forward(tokens, P, cfg, trace=None):
    """-> logits [T, vocab]; ``trace`` (a list) receives the residual stream after every layer run."""
    x0 = P["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    x = x0
    for i, t, first in layer_runs(cfg):
        if first:
            x = torch.cat([x, x0], dim=-1) @ P["loop.in"].T
        x = layer(x, P, i, cfg["layers"][i], cfg)
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, P["final.norm"], P["final.norm.b"], cfg["norm"]["eps"]) @ P["head"].T


def random_mimolix(layers, *, width=48, vocab=61, eps=1e-5, residual_mult=0.8, embed_scale=0.7, loop=None, seed=0,
                   dtype=torch.bfloat16, spaced_router=False):
    """A small random model.  ``layers``: list of dicts, either
      {type: "attention", heads, kv_heads, dim, vdim, [scale], [diff], [q_temp: (coef, every)], mlp}
      {type: "delta", heads, kv_heads, dim, vdim, conv, mlp}
    with mlp: None | (ff, experts, top, scale, shared ff or None).  ``loop`` = (start, stop, times).  Returns (config,
    tensors) in the checkpoint's naming; values are rounded to ``dtype`` so that product and oracle start from the same
    numbers.

    ``spaced_router``: the router's rows are multiples (steps of 0.3) of ONE unit direction and the layer norm's bias has a
    component of 6 along it, while the normalised stream's own component along a unit direction is of order 1: every token
    ranks the experts alike with logits about 1.8 apart, so a run in reduced precision can be compared position by position
    without a close call deciding which experts ran, and the chosen experts still share the weight."""
    g = torch.Generator().manual_seed(seed)

    def n(*shape, std=None, mean=0.0):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    cfg_layers, t = [], {"embed": n(vocab, width, std=1.0), "head": n(vocab, width, std=3.0 * width ** -0.5),
                         "final.norm": n(width, std=0.2, mean=1.0), "final.norm.b": n(width, std=0.2)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        H, G, d, dv = l["heads"], l["kv_heads"], l["dim"], l["vdim"]
        t[p + "norm1"], t[p + "norm1.b"] = n(width, std=0.2, mean=1.0), n(width, std=0.2)
        if l["type"] == "attention":
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": l.get("scale", d ** -0.5), "diff": l.get("diff", 0.4)}
            if l.get("q_temp"):
                m["q_temp"] = {"coef": l["q_temp"][0], "every": l["q_temp"][1]}
            t.update({p + "mix.q": n(H * 2 * d, width, std=2.0 * width ** -0.5), p + "mix.k": n(G * 2 * d, width, std=2.0 * width ** -0.5),
                      p + "mix.v": n(G * dv, width), p + "mix.q.norm": n(d, std=0.3, mean=1.5), p + "mix.k.norm": n(d, std=0.3, mean=1.5),
                      p + "mix.o": n(width, H * dv)})
            for k in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + k] = n(d, std=0.5 * d ** -0.5, mean=0.0)
        else:
            taps = l["conv"]
            m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
            t.update({p + "mix.q": n(G * d, width, std=2.0 * width ** -0.5), p + "mix.k": n(G * d, width, std=2.0 * width ** -0.5),
                      p + "mix.v": n(H * dv, width, std=2.0 * width ** -0.5), p + "mix.q.conv": n(G * d, taps, std=0.6),
                      p + "mix.k.conv": n(G * d, taps, std=0.6), p + "mix.v.conv": n(H * dv, taps, std=0.6),
                      p + "mix.b": n(H, width, std=2.0 * width ** -0.5), p + "mix.a": n(H, width, std=2.0 * width ** -0.5),
                      p + "mix.A_log": n(H, std=0.7, mean=-1.0), p + "mix.dt_bias": n(H, std=0.7, mean=-1.0),
                      p + "mix.norm": n(dv, std=0.2, mean=1.0), p + "mix.g": n(H * dv, width, std=2.0 * width ** -0.5),
                      p + "mix.o": n(width, H * dv)})
        mlp = None
        if l.get("mlp"):
            ff, E, top, scale, shared = l["mlp"]
            mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top, "scale": scale},
                   "shared": {"ff": shared} if shared else None}
            t[p + "mlp.router"] = n(E, width, std=3.0 * width ** -0.5)
            if spaced_router:
                direction = torch.randn(width, generator=g)
                direction = direction / direction.norm()
                factors = torch.randperm(E, generator=g).double() - (E - 1) / 2
                t[p + "mlp.router"] = (factors[:, None] * direction[None, :] * 0.3).to(dtype)
                t[p + "norm1.b"] = (t[p + "norm1.b"].double() + 6.0 * direction).to(dtype)
            for e in range(E):
                t.update({f"{p}mlp.e{e}.up": n(ff, width, std=2.0 * width ** -0.5), f"{p}mlp.e{e}.down": n(width, ff)})
            if shared:
                t.update({p + "mlp.shared.up": n(shared, width, std=2.0 * width ** -0.5), p + "mlp.shared.down": n(width, shared)})
        cfg_layers.append({"type": l["type"], "mixer": m, "mlp": mlp})
    config = {"architecture": "Mimolix", "vocab": vocab, "width": width, "embedding": {"scale": embed_scale}, "norm": {"eps": eps},
              "residual_mult": residual_mult, "layers": cfg_layers}
    if loop:
        config["loop"] = dict(zip(("start", "stop", "times"), loop))
        t["loop.in"] = n(width, 2 * width, std=(1.5 * width) ** -0.5)
    return config, t


def mimolix_forward(config, tensors, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with ``return_layers`` also the residual stream after every
    layer run."""
    P = {k: v.to(F64) for k, v in tensors.items()}
    trace = []
    with torch.no_grad():
        z = forward(tokens, P, config, trace)
    return (z, trace) if return_layers else z
