"""Plain float64 restatement of the Duzizen design (token + hashed-bigram embedding; layers with a layer norm before and
after each sublayer; an mLSTM matrix memory; a sliding-window attention with kept first tokens beside a retention; gated
GELU and clamped routed-expert feed-forwards; a per-layer token input), written from the equations and sharing no code
with the product path.  Slow on purpose: whole sequences at once, explicit loops over positions and heads, no cache,
nothing carried between calls.  Test infrastructure only.

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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(x):
    return x * torch.sigmoid(x)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table per position: a hash of (previous, current) token; the first position reads the extra last row."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(tokens, P, cfg):
    x = P["embed"][list(tokens)].clone()
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + P["bigram"][bigram_rows(tokens, int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"]))]
    return x


def short_conv(u, w):
    """u [T, C], w [C, taps]: the last tap weighs the current input, tap j the one ``taps - 1 - j`` positions back; inputs
    before position 0 are zero."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def rotary_frequencies(dims, base, scaling=None):
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f:
            lam = 2.0 * math.pi / fi
            if lam < orig / high:
                out.append(fi)
            elif lam > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / lam - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate(x, dims, freqs, layout):
    """x [T, heads, dim]: the first ``dims`` elements of every head are rotated by position * freqs; ``layout`` pairs element
    2i with 2i + 1 ("interleaved") or i with i + dims / 2 ("half")."""
    if not dims:
        return x
    T = x.shape[0]
    ang = torch.arange(T, dtype=F64)[:, None] * freqs[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    y = x.clone()
    if layout == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2] = a * c - b * s
        y[..., 1:dims:2] = b * c + a * s
    else:
        half = dims // 2
        a, b = x[..., :half], x[..., half:dims]
        y[..., :half] = a * c - b * s
        y[..., half:dims] = b * c + a * s
    return y


def window_attention_with_sink(q, k, v, scale, window, keep_first):
    """One head: q, k [T, d], v [T, dv].  Position i sees j <= i with i - j < window or j < keep_first; the softmax denominator
    holds one extra term exp(0) that carries no value."""
    T = q.shape[0]
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for i in range(T):
        js = [j for j in range(i + 1) if (window <= 0 or i - j < window) or j < keep_first]
        s = (k[js] @ q[i]) * scale
        m = max(float(s.max()), 0.0)
        e = torch.exp(s - m)
        out[i] = (e / (e.sum() + math.exp(-m))) @ v[js]
    return out


def tied_window_mixer(h, P, pre, mc, eps):
    """The attention half: values are the convolved keys before norm and rotation."""
    T = h.shape[0]
    H, G, d = int(mc["heads"]), int(mc.get("kv_heads", mc["heads"])), int(mc["dim"])
    q, k = h @ P[pre + "q"].T, h @ P[pre + "k"].T
    if pre + "q.conv" in P:
        q, k = short_conv(q, P[pre + "q.conv"]), short_conv(k, P[pre + "k.conv"])
    v = k.clone().view(T, G, d)
    q = (rms(q, eps) * P[pre + "q.norm"]).view(T, H, d)
    k = (rms(k, eps) * P[pre + "k.norm"]).view(T, G, d)
    rot = mc.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        fr = rotary_frequencies(dims, rot.get("base", 10000.0), rot.get("scaling"))
        q, k = rotate(q, dims, fr, "interleaved"), rotate(k, dims, fr, "interleaved")
    mask = mc.get("mask") or {}
    out = torch.zeros(T, H, d, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = window_attention_with_sink(q[:, hd], k[:, g], v[:, g], float(mc["scale"]), int(mask.get("size", 0)),
                                                int(mask.get("keep_first", 0)))
    return out.reshape(T, H * d) @ P[pre + "o"].T


def retention(q, k, v, decay):
    """One head: S <- decay S + k v^T, o = S^T q."""
    T = q.shape[0]
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out


def retention_mixer(h, P, pre, mc, eps):
    T = h.shape[0]
    H, d, dv = int(mc["heads"]), int(mc["dim"]), int(mc.get("vdim", mc["dim"]))
    q, k = (h @ P[pre + "q"].T).view(T, H, d), (h @ P[pre + "k"].T).view(T, H, d)
    v, g = (h @ P[pre + "v"].T).view(T, H, dv), h @ P[pre + "g"].T
    rot = mc.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        fr = rotary_frequencies(dims, rot.get("base", 10000.0), rot.get("scaling"))
        q, k = rotate(q, dims, fr, "half"), rotate(k, dims, fr, "half")
    k = k * d ** -0.5
    o = torch.stack([rms(retention(q[:, i], k[:, i], v[:, i], float(mc["decay"][i])), eps) for i in range(H)], dim=1)
    return (o.reshape(T, H * dv) * silu(g)) @ P[pre + "o"].T


def parallel_mixer(h, P, pre, mc, eps):
    a = tied_window_mixer(h, P, pre + "left.", mc["left"], eps)
    b = retention_mixer(h, P, pre + "right.", mc["right"], eps)
    return 0.5 * (rms(a, eps) * P[pre + "left.out"] + rms(b, eps) * P[pre + "right.out"])


def mlstm(q, k, v, ig, fg):
    """One head of the matrix memory with a running maximum that starts at 0: q, k [T, d], v [T, dv], ig / fg [T] the log input
    gate and the log forget gate."""
    T = q.shape[0]
    S = torch.zeros(q.shape[1], v.shape[1], dtype=F64)
    n = torch.zeros(q.shape[1], dtype=F64)
    m = 0.0
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        m_new = max(float(fg[t]) + m, float(ig[t]))
        a, b = math.exp(float(fg[t]) + m - m_new), math.exp(float(ig[t]) - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = (S.T @ q[t]) / (max(abs(float(n @ q[t])), math.exp(-m)) + 1e-6)
    return out


def mlstm_mixer(h, P, pre, mc, eps):
    T = h.shape[0]
    H, d, dv, cap = int(mc["heads"]), int(mc["dim"]), int(mc.get("vdim", mc["dim"])), float(mc["gate_cap"])
    q = (h @ P[pre + "q"].T).view(T, H, d) * d ** -0.5
    k, v = (h @ P[pre + "k"].T).view(T, H, d), (h @ P[pre + "v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ P[pre + "i"].T + P[pre + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ P[pre + "f"].T + P[pre + "f.b"]) / cap))
    o = torch.stack([rms(mlstm(q[:, i], k[:, i], v[:, i], ig[:, i], fg[:, i]), eps) for i in range(H)], dim=1)
    y = o.reshape(T, H * dv) * P[pre + "norm"] * torch.sigmoid(h @ P[pre + "g"].T)
    return y @ P[pre + "o"].T


def gated_gelu_mlp(h, P, pre):
    return (gelu_tanh(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def clamped_expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, P, pre, rc):
    """-> per token the chosen experts and their sigmoid scores (largest first; ties: lower index)."""
    s = torch.sigmoid(h @ P[pre + "router"].T)
    ids = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :int(rc["top"])]
    return ids, torch.gather(s, 1, ids)


def moe_mlp(h, P, pre, fc):
    """The score scales the expert's INPUT."""
    ids, w = route(h, P, pre, fc["router"])
    out = torch.zeros(h.shape[0], P[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j, e in enumerate(ids[t].tolist()):
            out[t] += clamped_expert(w[t, j] * h[t], P[f"{pre}e{e}.gate"], P[f"{pre}e{e}.up"], P[f"{pre}e{e}.down"],
                                     float(fc["expert"]["limit"]))
    return out


def token_side(x, tokens, P, i, cfg):
    sd = int(cfg["token_side"]["dim"])
    e = P["side.embed"][list(tokens)][:, i * sd:(i + 1) * sd]
    y = (gelu_tanh(x @ P[f"l{i}.side.gate"].T) * e) @ P[f"l{i}.side.proj"].T
    return rms(y, float(cfg["norm"]["eps"])) * P[f"l{i}.side.norm"]


def layer(x, tokens, P, i, lc, cfg):
    eps, p = float(cfg["norm"]["eps"]), f"l{i}."
    h = layer_norm(x, P[p + "norm1"], P[p + "norm1.b"], eps)
    if lc["type"] == "mlstm":
        y = mlstm_mixer(h, P, p + "mix.", lc["mixer"], eps)
    elif lc["type"] == "parallel":
        y = parallel_mixer(h, P, p + "mix.", lc["mixer"], eps)
    else:
        raise ValueError(lc["type"])
    x = x + layer_norm(y, P[p + "norm1b"], P[p + "norm1b.b"], eps)
    f = lc.get("mlp")
    if f is not None:
        h = layer_norm(x, P[p + "norm2"], P[p + "norm2.b"], eps)
        y = gated_gelu_mlp(h, P, p + "mlp.") if f["kind"] == "dense" else moe_mlp(h, P, p + "mlp.", f)
        x = x + layer_norm(y, P[p + "norm2b"], P[p + "norm2b.b"], eps)
    if cfg.get("token_side"):
        x = x + token_side(x, tokens, P, i, cfg)
    return x


def forward(tokens, P, cfg, trace=None):
    """-> logits [T, vocab]; ``trace`` (a list) receives the stream after every layer."""
    x = embed(tokens, P, cfg)
    for i, lc in enumerate(cfg["layers"]):
        x = layer(x, tokens, P, i, lc, cfg)
        if trace is not None:
            trace.append(x.clone())
    return layer_norm(x, P["final.norm"], P["final.norm.b"], float(cfg["norm"]["eps"])) @ P["head"].T


def duzizen_forward(config, tensors, tokens, return_layers=False):
    P = {k: v.to(F64) for k, v in tensors.items()}
    trace = []
    z = forward(list(tokens), P, config, trace)
    return (z, torch.stack(trace)) if return_layers else z


def random_duzizen(layers, *, width=48, vocab=61, eps=1e-5, side_dim=4, bigram=(13, 5, 3), seed=0, dtype=torch.bfloat16,
                   spaced_router=False, steady_memory=False):
    """A small random model.  ``layers``: list of dicts, either
      {type: "mlstm", heads, dim, vdim, [gate_cap], mlp}
      {type: "parallel", left: {heads, kv_heads, dim, [conv], [scale], [window], [keep_first], [rot_dims], [rot_base], [scaling]},
                         right: {heads, dim, vdim, decay, [rot_dims], [rot_base]}, mlp}
    with mlp: None | ("dense", ff) | ("moe", ff, experts, top, limit).  ``side_dim`` 0: no per-layer token input; ``bigram`` =
    (buckets, mul_prev, mul_cur) or None.  Returns (config, tensors) in the checkpoint's naming; values are rounded to ``dtype``
    so that product and oracle start from the same numbers.

    ``spaced_router``: the router's rows are multiples (steps of 0.3) of ONE unit direction and the bias of the norm in front of
    the feed-forward has a component of 6 along it, so every token ranks the experts alike with logits about 1.8 apart and a
    run in reduced precision can be compared position by position without a close call deciding which experts ran.

    ``steady_memory``: queries and keys of a matrix memory share a component (every row of W_q and W_k gets 0.5 times ONE unit
    direction, along which the bias of the norm in front of the mixer has a component of 4), so that n . q stays well away
    from 0.  With random weights some token's query is nearly orthogonal to n, the read-out divides by a difference of large
    terms, and a run whose projections see bf16 inputs differs there by far more than rounding — which is no kernel's error."""
    g = torch.Generator().manual_seed(seed)

    def n(*shape, std=None, mean=0.0):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    def lin(out, inp, gain=1.0):
        return n(out, inp, std=gain * inp ** -0.5)

    t = {"embed": n(vocab, width, std=1.0), "head": n(vocab, width, std=3.0 * width ** -0.5),
         "final.norm": n(width, std=0.2, mean=1.0), "final.norm.b": n(width, std=0.2)}
    config = {"architecture": "Duzizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": []}
    if bigram:
        config["embedding"] = {"bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))}
        t["bigram"] = n(bigram[0] + 1, width, std=0.7)
    if side_dim:
        config["token_side"] = {"dim": side_dim}
        t["side.embed"] = n(vocab, side_dim * len(layers), std=1.0)
    for i, l in enumerate(layers):
        p = f"l{i}."
        for k in ("norm1", "norm1b", "norm2", "norm2b"):
            t[p + k], t[p + k + ".b"] = n(width, std=0.2, mean=1.0), n(width, std=0.2)
        if l["type"] == "mlstm":
            H, d, dv = l["heads"], l["dim"], l["vdim"]
            m = {"heads": H, "dim": d, "vdim": dv, "gate_cap": l.get("gate_cap", 10.0)}
            t.update({p + "mix.q": lin(H * d, width, 2.0), p + "mix.k": lin(H * d, width, 2.0), p + "mix.v": lin(H * dv, width, 2.0),
                      p + "mix.g": lin(H * dv, width, 2.0), p + "mix.o": lin(width, H * dv), p + "mix.norm": n(H * dv, std=0.2, mean=1.0),
                      p + "mix.i": lin(H, width, 3.0), p + "mix.i.b": n(H, std=1.0), p + "mix.f": lin(H, width, 3.0),
                      p + "mix.f.b": n(H, std=1.0, mean=2.0)})
            if steady_memory:
                direction = torch.randn(width, generator=g)
                direction = direction / direction.norm()
                for k in ("mix.q", "mix.k"):
                    t[p + k] = (t[p + k].double() + 0.5 * direction[None, :]).to(dtype)
                t[p + "norm1.b"] = (t[p + "norm1.b"].double() + 4.0 * direction).to(dtype)
        else:
            a, r = l["left"], l["right"]
            H, G, d = a["heads"], a["kv_heads"], a["dim"]
            left = {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": a.get("scale", d ** -0.5)}
            if a.get("conv", 0):
                left["conv"] = a["conv"]
                t[p + "mix.left.q.conv"], t[p + "mix.left.k.conv"] = n(H * d, a["conv"], std=0.6), n(G * d, a["conv"], std=0.6)
            if a.get("window", 0):
                left["mask"] = {"size": a["window"], "keep_first": a.get("keep_first", 0)}
            if a.get("rot_dims", 0):
                left["rot"] = {"base": a.get("rot_base", 10000.0), "dims": a["rot_dims"]}
                if a.get("scaling"):
                    left["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), a["scaling"]))
            t.update({p + "mix.left.q": lin(H * d, width, 2.0), p + "mix.left.k": lin(G * d, width, 2.0),
                      p + "mix.left.q.norm": n(H * d, std=0.3, mean=1.5), p + "mix.left.k.norm": n(G * d, std=0.3, mean=1.5),
                      p + "mix.left.o": lin(width, H * d), p + "mix.left.out": n(width, std=0.2, mean=1.0)})
            Hr, dr, dvr = r["heads"], r["dim"], r["vdim"]
            right = {"heads": Hr, "dim": dr, "vdim": dvr, "decay": [float(x) for x in r["decay"]]}
            if r.get("rot_dims", 0):
                right["rot"] = {"base": r.get("rot_base", 10000.0), "dims": r["rot_dims"]}
            t.update({p + "mix.right.q": lin(Hr * dr, width, 2.0), p + "mix.right.k": lin(Hr * dr, width, 2.0),
                      p + "mix.right.v": lin(Hr * dvr, width, 2.0), p + "mix.right.g": lin(Hr * dvr, width, 2.0),
                      p + "mix.right.o": lin(width, Hr * dvr), p + "mix.right.out": n(width, std=0.2, mean=1.0)})
            m = {"left": left, "right": right}
        mlp = None
        if l.get("mlp"):
            if l["mlp"][0] == "dense":
                ff = l["mlp"][1]
                mlp = {"kind": "dense", "ff": ff}
                t.update({p + "mlp.gate": lin(ff, width, 2.0), p + "mlp.up": lin(ff, width, 2.0), p + "mlp.down": lin(width, ff)})
            else:
                _, ff, E, top, limit = l["mlp"]
                mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top}}
                t[p + "mlp.router"] = lin(E, width, 3.0)
                if spaced_router:
                    direction = torch.randn(width, generator=g)
                    direction = direction / direction.norm()
                    factors = torch.randperm(E, generator=g).double() - (E - 1) / 2
                    t[p + "mlp.router"] = (factors[:, None] * direction[None, :] * 0.3).to(dtype)
                    t[p + "norm2.b"] = (t[p + "norm2.b"].double() + 6.0 * direction).to(dtype)
                for e in range(E):
                    t.update({f"{p}mlp.e{e}.gate": lin(ff, width, 3.0), f"{p}mlp.e{e}.up": lin(ff, width, 3.0), f"{p}mlp.e{e}.down": lin(width, ff)})
        else:
            for k in ("norm2", "norm2b"):
                del t[p + k], t[p + k + ".b"]
        if side_dim:
            t.update({p + "side.gate": lin(side_dim, width, 2.0), p + "side.proj": lin(width, side_dim), p + "side.norm": n(width, std=0.2, mean=0.7)})
        config["layers"].append({"type": l["type"], "mixer": m, "mlp": mlp})
    return config, t
