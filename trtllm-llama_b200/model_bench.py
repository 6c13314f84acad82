"""``bench.py --model zobasun | nililix | mimolix``: prefill and decode throughput of an in-flight served design at layer
sizes that resemble real models (random bf16 weights), beside a LLaMA engine of equal width / depth / feed-forward size
served by ``GenerationSession`` (fp16) — for Mimolix beside Nililix, the closest in-flight design, at equal size — and every
operator's distance from its roofline.

Timing: CUDA events on the launching stream, >= 3 warm-up runs; every timed run works on tensors far larger than L2 or is
preceded by an L2 flush (a 256 MB fill).  Whole steps are timed from an idle device (synchronise, then the start event);
single operators with the flush still running when the start event is enqueued (``_time_kernel``).  Roofline denominators: MEASURED_PEAKS.json (copy bandwidth, cuBLAS bf16 burst)."""
from __future__ import annotations

import json
import os

SIZES = {
    # name: width, heads, dim, rot_dim, vdim, kv_rank, q_rank, ff, recurrent width, blocks, vocab
    "w2048": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768, ff=5632, rnn=2048, blocks=16, vocab=32000),
    "w4096": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1536, ff=11008, rnn=4096, blocks=32, vocab=32000),
}


def random_zobasun(torch, s, seed=0):
    """config + bf16 tensors of a 4-layer stack: latent attention, latent attention on the first layer's cache, two
    gated linear recurrences; every layer with a feed-forward."""
    g = torch.Generator().manual_seed(seed)
    W = s["width"]

    def n(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    att = dict(heads=s["heads"], dim=s["dim"], rot_dim=s["rot_dim"], vdim=s["vdim"], kv_rank=s["kv_rank"], q_rank=s["q_rank"],
               scale=(s["dim"] + s["rot_dim"]) ** -0.5, rot=dict(base=10000.0, dims=s["rot_dim"]))
    rec = dict(width=s["rnn"], blocks=s["blocks"], conv=4)
    mlp = dict(kind="dense", ff=s["ff"], limit=7.0)
    layers = [dict(type="latent_attention", mixer=dict(att), mlp=mlp),
              dict(type="latent_attention", mixer=dict(att, kv_from=0), mlp=mlp),
              dict(type="rglru", mixer=rec, mlp=mlp), dict(type="rglru", mixer=rec, mlp=mlp)]
    cfg = dict(architecture="Zobasun", vocab=s["vocab"], width=W, embedding=dict(scale=1.0), norm=dict(eps=1e-6), layers=layers)
    t = {"embed": n(s["vocab"], W, std=1.0), "head": n(s["vocab"], W), "final.norm": n(W, std=0.1)}
    H, dn, dr, dv, R, Q, C, nb = s["heads"], s["dim"], s["rot_dim"], s["vdim"], s["kv_rank"], s["q_rank"], s["rnn"], s["blocks"]
    for i, l in enumerate(layers):
        p = f"l{i}."
        t[p + "norm1"], t[p + "norm2"] = n(W, std=0.1), n(W, std=0.1)
        if l["type"] == "latent_attention":
            t.update({p + "mix.dq": n(Q, W), p + "mix.dq.norm": n(Q, std=0.1) + 1, p + "mix.uq": n(H * (dn + dr), Q),
                      p + "mix.uk": n(H * dn, R), p + "mix.uv": n(H * dv, R), p + "mix.o": n(W, H * dv)})
            if "kv_from" not in l["mixer"]:
                t.update({p + "mix.dkv": n(R + dr, W), p + "mix.dkv.norm": n(R, std=0.1) + 1})
        else:
            bw = C // nb
            t.update({p + "mix.y": n(C, W), p + "mix.y.b": n(C, std=0.1), p + "mix.x": n(C, W), p + "mix.x.b": n(C, std=0.1),
                      p + "mix.conv": n(C, 4, std=0.5), p + "mix.conv.b": n(C, std=0.1), p + "mix.ra": n(nb, bw, bw),
                      p + "mix.ra.b": n(nb, bw, std=0.1), p + "mix.ri": n(nb, bw, bw), p + "mix.ri.b": n(nb, bw, std=0.1),
                      p + "mix.lam": n(C, std=1.0), p + "mix.o": n(W, C)})
        t.update({p + "mlp.gate": n(s["ff"], W), p + "mlp.up": n(s["ff"], W), p + "mlp.down": n(W, s["ff"])})
    return cfg, t


NILILIX_SIZES = {
    # attention: heads x dim over kv_heads, window; feed-forward: dense ff, or `experts` experts of eff with `top` active
    # (top * eff = ff, so a routed layer does the dense layer's work per token)
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, window=512, rot_dims=64, ff=5632, experts=16, top=4,
                  eff=1408, groups=4, keep=2, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, rot_dims=64, ff=11008, experts=16, top=4,
                  eff=2752, groups=4, keep=2, vocab=32000),
}


def random_nililix(torch, s, seed=0):
    """config + bf16 tensors of a 4-layer stack [dense, routed, dense, routed] whose middle two layers run twice."""
    g = torch.Generator().manual_seed(seed)
    W, H, G, d, dv = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"]

    def n(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    mixer = dict(heads=H, kv_heads=G, dim=d, vdim=dv, conv=4, scale=d ** -0.5, mask=dict(size=s["window"]),
                 rot=dict(base=500000.0, dims=s["rot_dims"], scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    dense = dict(kind="dense", ff=s["ff"])
    moe = dict(kind="moe", expert=dict(ff=s["eff"]),
               router=dict(experts=s["experts"], top=s["top"], groups=dict(count=s["groups"], keep=s["keep"])))
    layers = [dict(type="attention", mixer=mixer, mlp=m) for m in (dense, moe, dense, moe)]
    cfg = dict(architecture="Nililix", vocab=s["vocab"], width=W, norm=dict(eps=1e-6), residual_mult=0.7, logit_softcap=30.0,
               loop=dict(start=1, stop=3, times=2), layers=layers)
    t = {"embed": n(s["vocab"], W, std=1.0), "head": n(s["vocab"], W), "final.norm": n(W, std=0.1) + 1, "loop.step": n(2, W, std=0.1)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        for k in ("norm1", "norm1b", "norm2", "norm2b"):
            t[p + k] = n(W, std=0.1) + 1
        t.update({p + "mix.q": n(H * d, W), p + "mix.k": n(G * d, W), p + "mix.v": n(G * dv, W), p + "mix.q.conv": n(H * d, 4, std=0.5),
                  p + "mix.k.conv": n(G * d, 4, std=0.5), p + "mix.v.conv": n(G * dv, 4, std=0.5), p + "mix.sink": n(H, std=1.0),
                  p + "mix.g": n(H, W), p + "mix.o": n(W, H * dv)})
        if l["mlp"]["kind"] == "dense":
            t.update({p + "mlp.up": n(s["ff"], W), p + "mlp.down": n(W, s["ff"])})
        else:
            t.update({p + "mlp.router": n(s["experts"], W), p + "mlp.correction": n(s["experts"], std=0.1)})
            for e in range(s["experts"]):
                t.update({f"{p}mlp.e{e}.gate": n(s["eff"], W), f"{p}mlp.e{e}.up": n(s["eff"], W), f"{p}mlp.e{e}.down": n(W, s["eff"])})
    return cfg, t


MIMOLIX_SIZES = {
    # differential attention: heads x (2 maps of dim) over kv_heads, values of vdim; delta rule: heads x vdim over kv_heads x dim;
    # feed-forward: `experts` experts of eff with `top` active plus a shared expert of eff
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, d_heads=16, d_kv_heads=4, d_dim=128, d_vdim=128, experts=16,
                  top=4, eff=1408, ff=5632, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=64, vdim=128, d_heads=32, d_kv_heads=8, d_dim=128, d_vdim=128, experts=16,
                  top=4, eff=2752, ff=11008, vocab=32000),
}


def random_mimolix(torch, s, seed=0):
    """config + bf16 tensors of a 4-layer stack [delta, attention, delta, attention] whose middle two layers run twice; every
    layer with routed experts and a shared expert."""
    g = torch.Generator().manual_seed(seed)
    W, H, G, d, dv = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"]
    DH, DG, dd, ddv = s["d_heads"], s["d_kv_heads"], s["d_dim"], s["d_vdim"]

    def n(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    att = dict(heads=H, kv_heads=G, dim=d, vdim=dv, scale=d ** -0.5, diff=0.4, q_temp=dict(coef=0.3, every=1024))
    dlt = dict(heads=DH, kv_heads=DG, dim=dd, vdim=ddv, conv=4)
    moe = dict(kind="moe", expert=dict(ff=s["eff"]), router=dict(experts=s["experts"], top=s["top"], scale=1.5), shared=dict(ff=s["eff"]))
    layers = [dict(type=ty, mixer=dict(att if ty == "attention" else dlt), mlp=moe) for ty in ("delta", "attention", "delta", "attention")]
    cfg = dict(architecture="Mimolix", vocab=s["vocab"], width=W, embedding=dict(scale=1.0), norm=dict(eps=1e-6), residual_mult=0.8,
               loop=dict(start=1, stop=3, times=2), layers=layers)
    t = {"embed": n(s["vocab"], W, std=1.0), "head": n(s["vocab"], W), "final.norm": n(W, std=0.1) + 1, "final.norm.b": n(W, std=0.1),
         "loop.in": n(W, 2 * W)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        t[p + "norm1"], t[p + "norm1.b"] = n(W, std=0.1) + 1, n(W, std=0.1)
        if l["type"] == "attention":
            t.update({p + "mix.q": n(H * 2 * d, W), p + "mix.k": n(G * 2 * d, W), p + "mix.v": n(G * dv, W), p + "mix.q.norm": n(d, std=0.1) + 1,
                      p + "mix.k.norm": n(d, std=0.1) + 1, p + "mix.o": n(W, H * dv)})
            for k in ("lq1", "lk1", "lq2", "lk2"):
                t[p + "mix." + k] = n(d, std=0.1)
        else:
            t.update({p + "mix.q": n(DG * dd, W), p + "mix.k": n(DG * dd, W), p + "mix.v": n(DH * ddv, W), p + "mix.q.conv": n(DG * dd, 4, std=0.5),
                      p + "mix.k.conv": n(DG * dd, 4, std=0.5), p + "mix.v.conv": n(DH * ddv, 4, std=0.5), p + "mix.b": n(DH, W),
                      p + "mix.a": n(DH, W), p + "mix.A_log": n(DH, std=0.5) - 2, p + "mix.dt_bias": n(DH, std=0.5), p + "mix.norm": n(ddv, std=0.1) + 1,
                      p + "mix.g": n(DH * ddv, W), p + "mix.o": n(W, DH * ddv)})
        t.update({p + "mlp.router": n(s["experts"], W), p + "mlp.shared.up": n(s["eff"], W), p + "mlp.shared.down": n(W, s["eff"])})
        for e in range(s["experts"]):
            t.update({f"{p}mlp.e{e}.up": n(s["eff"], W), f"{p}mlp.e{e}.down": n(W, s["eff"])})
    return cfg, t


DUZIZEN_SIZES = {
    # window attention: heads x dim over kv_heads (values = keys); retention: r_heads x (r_dim, r_vdim); matrix memory: m_heads x
    # (m_dim, m_vdim); feed-forward: one gated GELU layer of ff, then `experts` clamped experts of eff with `top` active
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, keep_first=4, r_heads=8, r_dim=128, r_vdim=256, m_heads=16,
                  m_dim=128, m_vdim=128, experts=16, top=4, eff=1408, ff=5632, side=128, buckets=50021, vocab=32000),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=1024, keep_first=4, r_heads=16, r_dim=128, r_vdim=256, m_heads=32,
                  m_dim=128, m_vdim=128, experts=16, top=4, eff=2752, ff=11008, side=256, buckets=50021, vocab=32000),
}


def random_duzizen(torch, s, seed=0):
    """config + bf16 tensors of a 6-layer stack [pair, memory, pair, memory, pair, memory] (pair = window attention beside a
    retention); the first layer with a gated GELU feed-forward, the others with routed experts."""
    g = torch.Generator().manual_seed(seed)
    W, H, G, d = s["width"], s["heads"], s["kv_heads"], s["dim"]
    RH, rd, rdv, MH, md, mdv = s["r_heads"], s["r_dim"], s["r_vdim"], s["m_heads"], s["m_dim"], s["m_vdim"]

    def n(*shape, std=None):
        std = std if std is not None else shape[-1] ** -0.5
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    left = dict(heads=H, kv_heads=G, dim=d, vdim=d, conv=4, scale=d ** -0.5, mask=dict(size=s["window"], keep_first=s["keep_first"]),
                rot=dict(base=10000.0, dims=d // 2, scaling=dict(factor=8.0, low=1.0, high=4.0, original=8192)))
    right = dict(heads=RH, dim=rd, vdim=rdv, decay=[1.0 - 2.0 ** (-5 - 5 * i / max(RH - 1, 1)) for i in range(RH)],
                 rot=dict(base=10000.0, dims=rd))
    mem = dict(heads=MH, dim=md, vdim=mdv, gate_cap=20.0)
    moe = dict(kind="moe", expert=dict(ff=s["eff"], limit=7.0), router=dict(experts=s["experts"], top=s["top"]))
    kinds = ["parallel", "mlstm"] * 3
    layers = [dict(type=ty, mixer=dict(left=left, right=right) if ty == "parallel" else dict(mem),
                   mlp=dict(kind="dense", ff=s["ff"]) if i == 0 else moe) for i, ty in enumerate(kinds)]
    cfg = dict(architecture="Duzizen", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), token_side=dict(dim=s["side"]),
               embedding=dict(bigram=dict(buckets=s["buckets"], mul_prev=31, mul_cur=17)), layers=layers)
    t = {"embed": n(s["vocab"], W, std=1.0), "bigram": n(s["buckets"] + 1, W, std=0.5), "side.embed": n(s["vocab"], s["side"] * len(layers), std=1.0),
         "head": n(s["vocab"], W), "final.norm": n(W, std=0.1) + 1, "final.norm.b": n(W, std=0.1)}
    for i, l in enumerate(layers):
        p = f"l{i}."
        for k in ("norm1", "norm1b", "norm2", "norm2b"):
            t[p + k], t[p + k + ".b"] = n(W, std=0.1) + 1, n(W, std=0.1)
        if l["type"] == "parallel":
            t.update({p + "mix.left.q": n(H * d, W), p + "mix.left.k": n(G * d, W), p + "mix.left.q.conv": n(H * d, 4, std=0.5),
                      p + "mix.left.k.conv": n(G * d, 4, std=0.5), p + "mix.left.q.norm": n(H * d, std=0.1) + 1,
                      p + "mix.left.k.norm": n(G * d, std=0.1) + 1, p + "mix.left.o": n(W, H * d), p + "mix.left.out": n(W, std=0.1) + 1,
                      p + "mix.right.q": n(RH * rd, W), p + "mix.right.k": n(RH * rd, W), p + "mix.right.v": n(RH * rdv, W),
                      p + "mix.right.g": n(RH * rdv, W), p + "mix.right.o": n(W, RH * rdv), p + "mix.right.out": n(W, std=0.1) + 1})
        else:
            t.update({p + "mix.q": n(MH * md, W), p + "mix.k": n(MH * md, W), p + "mix.v": n(MH * mdv, W), p + "mix.g": n(MH * mdv, W),
                      p + "mix.o": n(W, MH * mdv), p + "mix.norm": n(MH * mdv, std=0.1) + 1, p + "mix.i": n(MH, W), p + "mix.i.b": n(MH, std=0.5),
                      p + "mix.f": n(MH, W), p + "mix.f.b": n(MH, std=0.5) + 3})
        if l["mlp"]["kind"] == "dense":
            t.update({p + "mlp.gate": n(s["ff"], W), p + "mlp.up": n(s["ff"], W), p + "mlp.down": n(W, s["ff"])})
        else:
            t[p + "mlp.router"] = n(s["experts"], W)
            for e in range(s["experts"]):
                t.update({f"{p}mlp.e{e}.gate": n(s["eff"], W), f"{p}mlp.e{e}.up": n(s["eff"], W), f"{p}mlp.e{e}.down": n(W, s["eff"])})
        t.update({p + "side.gate": n(s["side"], W), p + "side.proj": n(W, s["side"]), p + "side.norm": n(W, std=0.1) + 1})
    return cfg, t


class OpTimer:
    """Wraps the ragged operators of ``ops`` with CUDA-event timers and the bytes / flops each call moves."""

    NAMES = ("linear", "linear_gated", "embed_scaled", "rmsnorm_rows", "gated_act", "rope_table", "rope_query_tail", "latent_kv_append",
             "latent_attention", "causal_conv1d", "rglru_scan", "qkv_conv_rope_append", "window_attention", "moe_route",
             "moe_plan", "moe_linear", "moe_linear_tc", "moe_gemv", "moe_gather_rows", "moe_combine", "add_row_vector", "tanh_cap",
             "residual_norm_rows", "layernorm_rows", "residual_layernorm_rows", "concat_rows", "qk_norm_append", "diff_combine",
             "delta_prepare", "delta_rule_scan", "gated_rmsnorm_heads", "moe_route_softmax", "embed_bigram", "qk_conv_norm_rope_append",
             "rope_heads", "mlstm_gates", "decay_attention_scan", "head_norm_gate", "residual_sandwich_layernorm_rows",
             "token_side_input", "rmsnorm_pair_sum")

    def __init__(self, torch, ops):
        self.torch, self.ops, self.rec, self.saved = torch, ops, [], {}

    @staticmethod
    def _nbytes(*ts):
        return sum(t.numel() * t.element_size() for t in ts if t is not None)

    def _cost(self, name, args, kw, out):
        nb = self._nbytes
        if name == "linear":
            a, w = args[0], args[1]
            o = kw.get("out", out)
            B = w.shape[0] if w.dim() == 3 else 1
            N, K = w.shape[-2], w.shape[-1]
            kind = "fp32-fma" if kw.get("compute", 0) else ("batched" if B > 1 else "dense")
            return f"linear {kind} {a.shape[0]}x{N}x{K}" + (f"x{B}" if B > 1 else ""), 2.0 * a.shape[0] * N * K * B, \
                nb(w) + a.shape[0] * B * K * a.element_size() + nb(o)
        if name == "linear_gated":
            if out is None:
                return "linear_gated (not taken)", 0.0, 0
            a, w = args[0], args[1]
            return f"linear gated {a.shape[0]}x{w.shape[0]}x{w.shape[1]}", 2.0 * a.shape[0] * w.shape[0] * w.shape[1], nb(w, a, out)
        if name == "latent_attention":
            qa, pool, batch = args[0], args[1], args[2]
            heads, lat, rot = args[4], args[5], args[6]
            pos = batch._host[batch.num_rows * 2:batch.num_rows * 3].double()
            keys = float((pos + 1).sum())
            # minimal traffic: every sequence's cache entries once, queries and outputs once
            seqlen = {}
            for s, p in zip(batch._host[batch.num_rows:batch.num_rows * 2].tolist(), pos.tolist()):
                seqlen[s] = max(seqlen.get(s, 0), p + 1)
            return name, 2.0 * keys * heads * (2 * lat + rot), sum(seqlen.values()) * (lat + rot) * pool.element_size() + nb(qa, out)
        if name == "window_attention":
            q, pool, batch, page, G, dv, window = args[0], args[1], args[2], args[3], args[4], args[5], args[7]
            H, d = q.shape[1], q.shape[2]
            vsh = kw.get("v_share", 1)
            pos = batch._host[batch.num_rows * 2:batch.num_rows * 3].double()
            keys = float(((pos + 1).clamp(max=window + kw.get("keep_first", 0)) if window else (pos + 1)).sum())
            seq = batch._host[batch.num_rows:batch.num_rows * 2].tolist()
            first, last = {}, {}
            for sq, p in zip(seq, pos.tolist()):
                first[sq] = min(first.get(sq, p), p)
                last[sq] = max(last.get(sq, p), p)
            # minimal traffic: the cached positions any row of the sequence sees, once; queries and outputs once
            seen = sum(last[sq] + 1 - (max(0, first[sq] - window + 1) if window else 0) for sq in first)
            return name, 2.0 * keys * H * (d + dv), seen * (G * d + G // vsh * dv) * pool.element_size() + nb(q, out)
        if name == "qkv_conv_rope_append":
            proj, H, G, d, dv = args[0], args[8], args[9], args[10], args[11]
            C = H * d + G * (d + dv)
            return name, 0.0, proj.shape[0] * C * (4 + args[5].element_size())
        if name == "moe_route":
            self._pairs = args[0].shape[0] * args[2]            # rows * top: the pairs the expert products below work on
            return name, 0.0, nb(args[0], *out)
        if name == "moe_route_softmax":
            self._pairs = args[0].shape[0] * args[1]
            return name, 0.0, nb(args[0], *out)
        if name == "delta_rule_scan":
            u, bg, state, batch, H, G, d, dv = args
            # the state of every sequence in the step is read and written once; rows in and out once
            return name, 6.0 * u.shape[0] * H * d * dv, nb(u, bg, out) + 2 * batch.num_seqs * H * d * dv * 4
        if name == "decay_attention_scan":
            q, k, v, state, batch, H, d, dv = args[:8]
            vc = dv + (1 if kw.get("ones_col") else 0)
            # rows in and out once; the state of every sequence in the step read and written once
            return name, 4.0 * q.shape[0] * H * d * vc, q.shape[0] * H * (2 * d + dv + vc) * 4 + 2 * batch.num_seqs * H * d * vc * 4
        if name == "qk_conv_norm_rope_append":
            proj, pool, H, G, d, dv = args[0], args[8], args[11], args[12], args[13], args[14]
            return name, 0.0, proj.shape[0] * ((H + G) * d * 4 + (H * d + G * (d + dv)) * pool.element_size())
        if name == "rope_heads":
            return name, 0.0, args[0].shape[0] * args[2] * args[3] * 8
        if name == "mlstm_gates":
            return name, 0.0, args[0].shape[0] * args[8] * (2 + 3) * 4
        if name == "head_norm_gate":
            o, dv = args[0], args[1]
            return name, 0.0, nb(o, out) + (o.shape[0] * o.shape[1] * dv * 4 if kw.get("gate") is not None else 0)
        if name == "token_side_input":
            x, wg, wp = args[0], args[4], args[5]
            return name, 0.0, 2 * nb(x) + nb(wg, wp, out) + x.shape[0] * wg.shape[0] * wg.element_size()
        if name == "residual_sandwich_layernorm_rows":
            return name, 0.0, 2 * nb(args[0]) + nb(args[1], out)
        if name == "delta_prepare":
            return name, 0.0, args[0].shape[0] * (2 * kw.get("C", args[8] * args[11] + 2 * args[9] * args[10]) * 4) + nb(*out[1:])
        if name == "qk_norm_append":
            proj, pool, qv, kv, d, vc = args[0], args[4], args[7], args[8], args[9], args[10]
            return name, 0.0, proj.shape[0] * ((qv + kv) * d + vc) * (4 + pool.element_size())
        if name in ("moe_linear", "moe_linear_tc", "moe_gemv"):
            a, w = args[0], args[1]
            if out is None:
                return name + " (not taken)", 0.0, 0
            E, N, K = w.shape
            used = min(E, self._pairs)
            return f"{name} {self._pairs}x{N}x{K} of {E}", 2.0 * self._pairs * N * K, \
                used * N * K * w.element_size() + self._pairs * (K * a.element_size() + out.shape[1] * out.element_size())
        if name == "latent_kv_append":
            pool, kv, lat, rot = args[0], args[1], args[8], args[9]
            return name, 0.0, kv.shape[0] * (lat + rot) * (4 + pool.element_size())
        if name == "causal_conv1d":
            return name, 0.0, 2 * nb(args[0])
        if name == "rglru_scan":
            return name, 0.0, nb(args[0], args[1], args[3], out)
        ts = [a for a in args if isinstance(a, self.torch.Tensor)] + [v for v in kw.values() if isinstance(v, self.torch.Tensor)]
        if isinstance(out, self.torch.Tensor) and all(out is not x for x in ts):
            ts.append(out)
        return name, 0.0, nb(*ts)

    def __enter__(self):
        torch = self.torch
        for nm in self.NAMES:
            fn = getattr(self.ops, nm)
            self.saved[nm] = fn

            def wrapped(*a, _fn=fn, _nm=nm, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = _fn(*a, **kw)
                e1.record()
                self.rec.append((self._cost(_nm, a, kw, out), e0, e1))
                return out
            setattr(self.ops, nm, wrapped)
        return self

    def __exit__(self, *exc):
        for nm, fn in self.saved.items():
            setattr(self.ops, nm, fn)

    def summary(self, peaks):
        self.torch.cuda.synchronize()
        agg = {}
        for (name, flops, nbytes), e0, e1 in self.rec:
            a = agg.setdefault(name, [0.0, 0.0, 0.0, 0])
            a[0] += e0.elapsed_time(e1) * 1e-3
            a[1] += flops
            a[2] += nbytes
            a[3] += 1
        out = {}
        for name, (t, fl, by, calls) in agg.items():
            ideal = max(fl / (peaks["bf16_tflops"] * 1e12), by / (peaks["hbm_gbs"] * 1e9))
            out[name] = {"calls": calls, "us": round(t * 1e6, 1), "tflops": round(fl / t / 1e12, 1), "gbs": round(by / t / 1e9, 1),
                         "of_roofline": round(ideal / t, 3)}
        return out


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def _time(torch, fn, steps, warmup, flush):
    for _ in range(max(3, warmup)):
        fn()
    ts = []
    for _ in range(steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return sorted(ts)[len(ts) // 2]


def _time_kernel(torch, fn, steps, warmup, flush):
    """One operator alone: as ``_time``, but the L2 flush is enqueued right before the start event WITHOUT a host synchronise
    in between, so the host's launch latency (tens of microseconds of Python and ctypes per call, which a single launch
    after a synchronise would carry) is hidden behind the flush and the events bracket the kernel's own time."""
    for _ in range(max(3, warmup)):
        fn()
    ts = []
    for _ in range(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        flush.fill_(1)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e-3)
    return sorted(ts)[len(ts) // 2]


def _llama_side(torch, ops, rt, s, n_layers, res, prompt, S, B, steps, warmup, flush, peaks):
    """LLaMA (MHA, SwiGLU; fp16) of equal width / depth / feed-forward / vocabulary through ``GenerationSession``, and its
    like kernels alone.  Fills ``res``; returns (L, engine tensors' gate weight shape) for the caller's own like kernels."""
    # the closest existing model at equal size: LLaMA (MHA, SwiGLU), fp16, same width / depth / feed-forward / vocabulary
    import bench as HB
    L = {"hidden": s["width"], "inter": s["ff"], "vocab": s["vocab"], "layers": n_layers, "heads": s["width"] // 128}
    mc = rt.ModelConfig(vocab_size=L["vocab"], num_layers=L["layers"], num_heads=L["heads"], hidden_size=L["hidden"],
                        inter_size=L["inter"], max_batch_size=B, max_input_len=S, max_output_len=64)
    lt = rt.build_engine_tensors(HB.make_weights(torch, L, 0, 1), mc)
    ls = rt.GenerationSession(mc, lt)
    ls.setup(B, S, 64)
    ids1 = torch.tensor([prompt], dtype=torch.int32)
    t = _time(torch, lambda: ls.context(ids1, torch.tensor([S], dtype=torch.int32)), steps, warmup, flush)
    res["llama_prefill_tokens_per_s"] = round(S / t, 1)
    idsB = ids1.repeat(B, 1)
    ls.context(idsB, torch.tensor([S] * B, dtype=torch.int32))
    ts = []
    for i in range(max(3, warmup) + steps):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ls.step()
        e1.record()
        torch.cuda.synchronize()
        if i >= max(3, warmup):
            ts.append(e0.elapsed_time(e1) * 1e-3)
    t = sorted(ts)[len(ts) // 2]
    res["llama_decode_tokens_per_s"] = round(B / t, 1)
    res["llama_decode_ms_per_step"] = round(t * 1e3, 3)
    # like kernels, timed alone on the same shapes: prefill / decode projection, prefill / decode attention
    like = {}
    x = torch.randn(S, L["hidden"], device="cuda").half()
    w = lt["layers.0.mlp.fc_gate.weight"]
    fl = 2.0 * S * w.shape[0] * w.shape[1]
    t = _time_kernel(torch, lambda: ops.matmul_f16(x, w), steps, warmup, flush)
    like["linear_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(fl / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    xd = x[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.matmul_f16(xd, w), steps, warmup, flush)
    like["linear_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(w.numel() * 2 / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    H = L["heads"]
    qkv = torch.randn(1, S, 3 * H * 128, device="cuda").half()
    kvc = torch.zeros(B, 2, H, S + 64, 128, device="cuda", dtype=torch.float16)
    lens1 = torch.tensor([S], dtype=torch.int32, device="cuda")
    t = _time_kernel(torch, lambda: ops.context_attention(qkv, kvc, lens1, num_heads=H, head_size=128), steps, warmup, flush)
    like["attention_prefill"] = {"us": round(t * 1e6, 1),
                                 "of_roofline": round(4.0 * S * S / 2 * 128 * H / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    qd = torch.randn(B, 3 * H * 128, device="cuda").half()
    t = _time_kernel(torch, lambda: ops.mmha_decode(qd, kvc, S, num_heads=H, head_size=128, max_input_len=S), steps, warmup, flush)
    like["attention_decode"] = {"us": round(t * 1e6, 1),
                                "of_roofline": round(B * 2 * H * S * 128 * 2 / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    res["llama_like_kernels"] = like
    del x, xd, qkv, kvc, qd, ls
    torch.cuda.empty_cache()
    return L, tuple(w.shape), fl


def bench_size(torch, name, steps, warmup, S=2048, B=4):
    from . import ops
    from . import runtime as rt
    from .inflight import InflightSession
    from .models.zobasun import build_zobasun
    s, peaks = SIZES[name], _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    cfg, tensors = random_zobasun(torch, s)
    model = build_zobasun(cfg, tensors, torch.bfloat16, "cuda")
    del tensors
    sess = InflightSession(model, max_tokens=(B + 1) * (S + 64), max_seqs=B + 1)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, s["vocab"], (S,), generator=g).tolist()
    res = {"size": dict(s), "layers": [l["type"] + ("+kv_from" if "kv_from" in l["mixer"] else "") for l in cfg["layers"]],
           "prefill_tokens": S, "decode_batch": B, "decode_context": S}

    def prefill():
        sess.step([("p", prompt, [S - 1])])
        sess.end("p")
    t = _time(torch, prefill, steps, warmup, flush)
    res["prefill_tokens_per_s"] = round(S / t, 1)
    with OpTimer(torch, ops) as ot:
        prefill()
    res["prefill_ops"] = ot.summary(peaks)
    for b in range(B):
        sess.step([(("d", b), prompt, [])])
    dec = [(("d", b), [7 + b], [0]) for b in range(B)]
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_tokens_per_s"] = round(B / t, 1)
    res["decode_ms_per_step"] = round(t * 1e3, 3)
    sess.use_cuda_graph = False          # the operators are timed one by one on eager launches
    with OpTimer(torch, ops) as ot:
        sess.step(dec)
    res["decode_ops"] = ot.summary(peaks)
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_ms_per_step_eager"] = round(t * 1e3, 3)
    del sess, model
    torch.cuda.empty_cache()

    L, w_shape, fl = _llama_side(torch, ops, rt, s, len(cfg["layers"]), res, prompt, S, B, steps, warmup, flush, peaks)
    H = L["heads"]
    # this design's kernels alone on the same problem sizes (bf16)
    own = {}
    xb = torch.randn(S, L["hidden"], device="cuda").bfloat16()
    wb = (torch.randn(w_shape[0], w_shape[1], device="cuda") * 0.02).bfloat16()
    t = _time_kernel(torch, lambda: ops.linear(xb, wb, out_dtype=torch.bfloat16), steps, warmup, flush)
    own["linear_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(fl / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    xf = torch.randn(B, L["hidden"], device="cuda")
    t = _time_kernel(torch, lambda: ops.linear(xf, wb, out_dtype=torch.float32), steps, warmup, flush)
    own["linear_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(wb.numel() * 2 / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    from .inflight import RaggedBatch
    lat, rot, Hh, page = s["kv_rank"], s["rot_dim"], s["heads"], 64
    nblk = -(-S // page)
    pool = torch.randn((B * nblk * page, lat + rot), device="cuda").bfloat16()
    pb = RaggedBatch([([0] * S, 0, 0, list(range(nblk)))], [], "cuda")
    qa = torch.randn(S, Hh, lat + rot, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.latent_attention(qa, pool, pb, page, Hh, lat, rot, 0.07), steps, warmup, flush)
    fl_a = 2.0 * (S * (S + 1) / 2) * Hh * (2 * lat + rot)
    own["attention_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(fl_a / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    db = RaggedBatch([([0], S - 1, b, list(range(b * nblk, (b + 1) * nblk))) for b in range(B)], [], "cuda")
    qd2 = qa[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.latent_attention(qd2, pool, db, page, Hh, lat, rot, 0.07), steps, warmup, flush)
    own["attention_decode"] = {"us": round(t * 1e6, 1),
                               "of_roofline": round(B * S * (lat + rot) * 2 / (peaks["hbm_gbs"] * 1e9) / t, 3),
                               "cache_bytes": B * S * (lat + rot) * 2, "llama_cache_bytes": B * 2 * H * S * 128 * 2}
    res["zobasun_like_kernels"] = own
    res["peaks"] = peaks
    torch.cuda.empty_cache()
    return res


def bench_nililix_size(torch, name, steps, warmup, S=2048, B=4):
    from . import ops
    from . import runtime as rt
    from .inflight import InflightSession, RaggedBatch
    from .models.nililix import build_nililix
    s, peaks = NILILIX_SIZES[name], _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    cfg, tensors = random_nililix(torch, s)
    model = build_nililix(cfg, tensors, torch.bfloat16, "cuda")
    del tensors
    sess = InflightSession(model, max_tokens=(B + 1) * (S + 64), max_seqs=B + 1)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, s["vocab"], (S,), generator=g).tolist()
    res = {"size": dict(s), "layers": [l["mlp"]["kind"] for l in cfg["layers"]], "layer_runs": len(model.runs),
           "prefill_tokens": S, "decode_batch": B, "decode_context": S}

    def prefill():
        sess.step([("p", prompt, [S - 1])])
        sess.end("p")
    t = _time(torch, prefill, steps, warmup, flush)
    res["prefill_tokens_per_s"] = round(S / t, 1)
    with OpTimer(torch, ops) as ot:
        prefill()
    res["prefill_ops"] = ot.summary(peaks)
    for b in range(B):
        sess.step([(("d", b), prompt, [])])
    dec = [(("d", b), [7 + b], [0]) for b in range(B)]
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_tokens_per_s"] = round(B / t, 1)
    res["decode_ms_per_step"] = round(t * 1e3, 3)
    sess.use_cuda_graph = False          # the operators are timed one by one on eager launches
    with OpTimer(torch, ops) as ot:
        sess.step(dec)
    res["decode_ops"] = ot.summary(peaks)
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_ms_per_step_eager"] = round(t * 1e3, 3)
    del sess, model
    torch.cuda.empty_cache()
    # LLaMA with as many layers as this stack RUNS layers (a looped layer counts each time)
    L, w_shape, fl = _llama_side(torch, ops, rt, s, res["layer_runs"], res, prompt, S, B, steps, warmup, flush, peaks)
    own = {}
    xb = torch.randn(S, L["hidden"], device="cuda").bfloat16()
    wb = (torch.randn(w_shape[0], w_shape[1], device="cuda") * 0.02).bfloat16()
    t = _time_kernel(torch, lambda: ops.linear(xb, wb, out_dtype=torch.bfloat16), steps, warmup, flush)
    own["linear_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(fl / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    xf = torch.randn(B, L["hidden"], device="cuda")
    t = _time_kernel(torch, lambda: ops.linear(xf, wb, out_dtype=torch.float32), steps, warmup, flush)
    own["linear_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(wb.numel() * 2 / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    H, G, d, dv, win, page = s["heads"], s["kv_heads"], s["dim"], s["vdim"], s["window"], 64
    nblk = -(-S // page)
    pool = torch.randn((B * nblk * page, G * (d + dv)), device="cuda").bfloat16()
    sink = torch.zeros(H, device="cuda").bfloat16()
    pb = RaggedBatch([([0] * S, 0, 0, list(range(nblk)))], [], "cuda")
    q = torch.randn(S, H, d, device="cuda").bfloat16()
    gate = torch.randn(S, H, device="cuda")
    t = _time_kernel(torch, lambda: ops.window_attention(q, pool, pb, page, G, dv, 0.09, win, sink=sink, gate=gate), steps, warmup, flush)
    keys = sum(min(p + 1, win) for p in range(S))
    own["attention_prefill"] = {"us": round(t * 1e6, 1), "keys_per_row": round(keys / S, 1),
                                "of_roofline": round(2.0 * keys * H * (d + dv) / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    db = RaggedBatch([([0], S - 1, b, list(range(b * nblk, (b + 1) * nblk))) for b in range(B)], [], "cuda")
    qd = q[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.window_attention(qd, pool, db, page, G, dv, 0.09, win, sink=sink, gate=gate[:B]), steps, warmup, flush)
    cache_bytes = B * min(S, win) * G * (d + dv) * 2
    own["attention_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(cache_bytes / (peaks["hbm_gbs"] * 1e9) / t, 3),
                               "cache_bytes": cache_bytes, "llama_cache_bytes": B * 2 * L["heads"] * S * 128 * 2}
    res["nililix_like_kernels"] = own
    res["peaks"] = peaks
    torch.cuda.empty_cache()
    return res


def _serve(torch, ops, model, vocab, S, B, steps, warmup, flush, peaks):
    """Prefill of one S-token prompt in one step and generation steps of B sequences at context S through ``InflightSession``,
    with every operator timed once on eager launches."""
    from .inflight import InflightSession
    sess = InflightSession(model, max_tokens=(B + 1) * (S + 64), max_seqs=B + 1)
    prompt = torch.randint(0, vocab, (S,), generator=torch.Generator().manual_seed(1)).tolist()
    res = {}

    def prefill():
        sess.step([("p", prompt, [S - 1])])
        sess.end("p")
    t = _time(torch, prefill, steps, warmup, flush)
    res["prefill_tokens_per_s"] = round(S / t, 1)
    res["prefill_ms"] = round(t * 1e3, 3)
    with OpTimer(torch, ops) as ot:
        prefill()
    res["prefill_ops"] = ot.summary(peaks)
    for b in range(B):
        sess.step([(("d", b), prompt, [])])
    dec = [(("d", b), [7 + b], [0]) for b in range(B)]
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_tokens_per_s"] = round(B / t, 1)
    res["decode_ms_per_step"] = round(t * 1e3, 3)
    sess.use_cuda_graph = False          # the operators are timed one by one on eager launches
    with OpTimer(torch, ops) as ot:
        sess.step(dec)
    res["decode_ops"] = ot.summary(peaks)
    t = _time(torch, lambda: sess.step(dec), steps, warmup, flush)
    res["decode_ms_per_step_eager"] = round(t * 1e3, 3)
    return res


def bench_mimolix_size(torch, name, steps, warmup, S=2048, B=4):
    """Mimolix beside Nililix (the closest design served in-flight: grouped-query attention, routed experts, a looped block) at
    equal width, heads, expert sizes, vocabulary and number of layer runs; then the like kernels alone on the same shapes:
    differential against windowed attention, the delta rule against the gated linear recurrence, the fused residual steps."""
    from . import ops
    from .inflight import RaggedBatch
    from .models.mimolix import build_mimolix
    from .models.nililix import build_nililix
    s, peaks = MIMOLIX_SIZES[name], _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    cfg, tensors = random_mimolix(torch, s)
    model = build_mimolix(cfg, tensors, torch.bfloat16, "cuda")
    del tensors
    res = {"size": dict(s), "layers": [l["type"] for l in cfg["layers"]], "layer_runs": len(model.runs), "prefill_tokens": S,
           "decode_batch": B, "decode_context": S}
    res["mimolix"] = _serve(torch, ops, model, s["vocab"], S, B, steps, warmup, flush, peaks)
    del model
    torch.cuda.empty_cache()
    ns = dict(NILILIX_SIZES[name], window=0)          # all keys visible, as here
    ncfg, ntensors = random_nililix(torch, ns)
    nmodel = build_nililix(ncfg, ntensors, torch.bfloat16, "cuda")
    del ntensors
    res["nililix"] = _serve(torch, ops, nmodel, ns["vocab"], S, B, steps, warmup, flush, peaks)
    res["nililix"]["layers"] = [l["mlp"]["kind"] for l in ncfg["layers"]]
    del nmodel
    torch.cuda.empty_cache()

    like = {}
    H, G, d, dv, page = s["heads"], s["kv_heads"], s["dim"], s["vdim"], 64
    nblk = -(-S // page)
    pb = RaggedBatch([([0] * S, 0, 0, list(range(nblk)))], [], "cuda")
    db = RaggedBatch([([0], S - 1, b, list(range(b * nblk, (b + 1) * nblk))) for b in range(B)], [], "cuda")
    keys = S * (S + 1) / 2
    # differential attention: 2 H (head, map) queries of d against 2 G key heads, G value heads
    pool = torch.randn((B * nblk * page, G * (2 * d + dv)), device="cuda").bfloat16()
    q = torch.randn(S, 2 * H, d, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.window_attention(q, pool, pb, page, 2 * G, dv, 0.1, 0, v_share=2, out_f32=True), steps, warmup, flush)
    like["differential_attention_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(2.0 * keys * 2 * H * (d + dv) / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    qd = q[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.window_attention(qd, pool, db, page, 2 * G, dv, 0.1, 0, v_share=2, out_f32=True), steps, warmup, flush)
    cb = B * S * G * (2 * d + dv) * 2
    like["differential_attention_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(cb / (peaks["hbm_gbs"] * 1e9) / t, 3), "cache_bytes": cb}
    # Nililix' attention on its own shapes, all keys visible
    NH, NG, nd, ndv = ns["heads"], ns["kv_heads"], ns["dim"], ns["vdim"]
    npool = torch.randn((B * nblk * page, NG * (nd + ndv)), device="cuda").bfloat16()
    nq = torch.randn(S, NH, nd, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.window_attention(nq, npool, pb, page, NG, ndv, 0.1, 0), steps, warmup, flush)
    like["nililix_attention_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(2.0 * keys * NH * (nd + ndv) / (peaks["bf16_tflops"] * 1e12) / t, 3)}
    nqd = nq[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.window_attention(nqd, npool, db, page, NG, ndv, 0.1, 0), steps, warmup, flush)
    cb = B * S * NG * (nd + ndv) * 2
    like["nililix_attention_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(cb / (peaks["hbm_gbs"] * 1e9) / t, 3), "cache_bytes": cb}
    del pool, npool, q, nq
    # the recurrences: delta rule (matrix state per head) against the gated linear recurrence (vector state) of equal width
    DH, DG, dd, ddv = s["d_heads"], s["d_kv_heads"], s["d_dim"], s["d_vdim"]
    C = 2 * DG * dd + DH * ddv
    u, bg = torch.randn(S, C, device="cuda") * 0.05, torch.rand(S, 2 * DH, device="cuda")
    state = torch.zeros(B + 1, DH * ddv * dd, device="cuda")
    t = _time_kernel(torch, lambda: ops.delta_rule_scan(u, bg, state, pb, DH, DG, dd, ddv), steps, warmup, flush)
    by = (u.numel() + bg.numel() + S * DH * ddv) * 4 + 2 * DH * dd * ddv * 4
    like["delta_rule_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / (peaks["hbm_gbs"] * 1e9) / t, 3),
                                  "fp32_tflops": round(6.0 * S * DH * dd * ddv / t / 1e12, 2)}
    ud, bgd = u[:B].contiguous(), bg[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.delta_rule_scan(ud, bgd, state, db, DH, DG, dd, ddv), steps, warmup, flush)
    by = 2 * B * DH * dd * ddv * 4
    like["delta_rule_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / (peaks["hbm_gbs"] * 1e9) / t, 3), "state_bytes": by}
    Cr, blocks = s["width"], s["width"] // 128
    ur, gates = torch.randn(S, Cr, device="cuda"), torch.randn(S, blocks, 2 * (Cr // blocks), device="cuda")
    lam, y = torch.randn(Cr, device="cuda").bfloat16(), torch.randn(S, Cr, device="cuda").bfloat16()
    rstate = torch.zeros(B + 1, Cr, device="cuda")
    t = _time_kernel(torch, lambda: ops.rglru_scan(ur, gates, lam, y, rstate, pb, blocks, 8.0), steps, warmup, flush)
    by = ur.numel() * 4 + gates.numel() * 4 + 2 * y.numel() * 2
    like["gated_linear_recurrence_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    # residual step + next norm: parallel layers' layer norm against the sandwich RMS norms
    W = s["width"]
    x, y1, y2 = (torch.randn(S, W, device="cuda") for _ in range(3))
    w, b = torch.ones(W, device="cuda").bfloat16(), torch.zeros(W, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.residual_layernorm_rows(x, y1, y2, 0.7, w, b, 1e-6, torch.bfloat16), steps, warmup, flush)
    like["residual_layernorm"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * W * (4 * 4 + 2) / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    t = _time_kernel(torch, lambda: ops.residual_norm_rows(x, y1, w, w, 1e-6, 0.0, 0.7, torch.bfloat16), steps, warmup, flush)
    like["nililix_residual_norm"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * W * (3 * 4 + 2) / (peaks["hbm_gbs"] * 1e9) / t, 3)}
    res["like_kernels"] = like
    res["peaks"] = peaks
    torch.cuda.empty_cache()
    return res


def bench_duzizen_size(torch, name, steps, warmup, S=2048, B=4):
    """Duzizen beside Mimolix (the closest design served in-flight: layer norms with biases, a recurrence with a matrix state per
    head beside softmax attention, routed experts) at equal width, expert sizes, vocabulary and number of layer runs; then the
    like kernels alone on the same shapes: the decayed linear attention (matrix memory, retention) against the delta rule, the
    window attention with kept first tokens against the plain window, the two front kernels of the attention, the residual steps."""
    from . import ops
    from .inflight import RaggedBatch
    from .models.duzizen import build_duzizen
    from .models.mimolix import build_mimolix
    s, peaks = DUZIZEN_SIZES[name], _peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    cfg, tensors = random_duzizen(torch, s)
    model = build_duzizen(cfg, tensors, torch.bfloat16, "cuda")
    del tensors
    res = {"size": dict(s), "layers": [l["type"] for l in cfg["layers"]], "layer_runs": len(model.runs), "prefill_tokens": S,
           "decode_batch": B, "decode_context": S}
    res["duzizen"] = _serve(torch, ops, model, s["vocab"], S, B, steps, warmup, flush, peaks)
    del model
    torch.cuda.empty_cache()
    ms = MIMOLIX_SIZES[name]
    mcfg, mtensors = random_mimolix(torch, ms)
    mmodel = build_mimolix(mcfg, mtensors, torch.bfloat16, "cuda")
    del mtensors
    res["mimolix"] = _serve(torch, ops, mmodel, ms["vocab"], S, B, steps, warmup, flush, peaks)
    res["mimolix"]["layer_runs"] = len(mmodel.runs)
    del mmodel
    torch.cuda.empty_cache()

    like = {}
    page = 64
    nblk = -(-S // page)
    pb = RaggedBatch([([0] * S, 0, 0, list(range(nblk)))], [], "cuda")
    db = RaggedBatch([([0], S - 1, b, list(range(b * nblk, (b + 1) * nblk))) for b in range(B)], [], "cuda")
    hbm, tfl = peaks["hbm_gbs"] * 1e9, peaks["bf16_tflops"] * 1e12

    def scan(tag, H, d, dv, ones, gated):
        """prompt and generation step of the decayed linear attention: bytes of rows and state against the copy roofline, and
        the fp32 multiply-adds it runs (4 per state element and token) against nothing — CUDA cores, no tensor-core peak applies"""
        vc = dv + (1 if ones else 0)
        q, k, v = (torch.randn(S, H * n_, device="cuda") * 0.05 for n_ in (d, d, dv))
        lab = -torch.rand(S, H, 2, device="cuda") * 0.1 if gated else None
        dec = None if gated else torch.full((H,), 0.98, device="cuda")
        state = torch.zeros(B + 1, H * vc * d, device="cuda")
        t = _time_kernel(torch, lambda: ops.decay_attention_scan(q, k, v, state, pb, H, d, dv, log_ab=lab, head_decay=dec, ones_col=ones), steps, warmup, flush)
        by = S * H * (2 * d + dv + vc) * 4 + 2 * H * d * vc * 4
        like[tag + "_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3), "fp32_tflops": round(4.0 * S * H * d * vc / t / 1e12, 2)}
        qd, kd, vd = q[:B].contiguous(), k[:B].contiguous(), v[:B].contiguous()
        labd = lab[:B].contiguous() if gated else None
        t = _time_kernel(torch, lambda: ops.decay_attention_scan(qd, kd, vd, state, db, H, d, dv, log_ab=labd, head_decay=dec, ones_col=ones), steps, warmup, flush)
        by = 2 * B * H * d * vc * 4
        like[tag + "_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3), "state_bytes": by}

    scan("matrix_memory", s["m_heads"], s["m_dim"], s["m_vdim"], True, True)
    scan("retention", s["r_heads"], s["r_dim"], s["r_vdim"], False, False)
    # the delta rule on Mimolix' shapes (the recurrence of the closest model)
    DH, DG, dd, ddv = ms["d_heads"], ms["d_kv_heads"], ms["d_dim"], ms["d_vdim"]
    C = 2 * DG * dd + DH * ddv
    u, bg = torch.randn(S, C, device="cuda") * 0.05, torch.rand(S, 2 * DH, device="cuda")
    state = torch.zeros(B + 1, DH * ddv * dd, device="cuda")
    t = _time_kernel(torch, lambda: ops.delta_rule_scan(u, bg, state, pb, DH, DG, dd, ddv), steps, warmup, flush)
    by = (u.numel() + bg.numel() + S * DH * ddv) * 4 + 2 * DH * dd * ddv * 4
    like["delta_rule_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3), "fp32_tflops": round(6.0 * S * DH * dd * ddv / t / 1e12, 2)}
    ud, bgd = u[:B].contiguous(), bg[:B].contiguous()
    t = _time_kernel(torch, lambda: ops.delta_rule_scan(ud, bgd, state, db, DH, DG, dd, ddv), steps, warmup, flush)
    by = 2 * B * DH * dd * ddv * 4
    like["delta_rule_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3), "state_bytes": by}
    del u, bg, state
    # window attention: with kept first tokens (values = keys) against the same kernel without them
    H, G, d, win, keep = s["heads"], s["kv_heads"], s["dim"], s["window"], s["keep_first"]
    pool = torch.randn((B * nblk * page, 2 * G * d), device="cuda").bfloat16()
    q = torch.randn(S, H, d, device="cuda").bfloat16()
    zeros = torch.zeros(H, device="cuda")
    pos = torch.arange(S, dtype=torch.float64)
    for tag, kf in (("window_attention_kept_first", keep), ("window_attention_plain", 0)):
        keys = float((pos + 1).clamp(max=win + kf).sum())
        t = _time_kernel(torch, lambda: ops.window_attention(q, pool, pb, page, G, d, 0.1, win, sink=zeros, keep_first=kf), steps, warmup, flush)
        like[tag + "_prefill"] = {"us": round(t * 1e6, 1), "of_roofline": round(2.0 * keys * H * 2 * d / tfl / t, 3)}
        qd = q[:B].contiguous()
        t = _time_kernel(torch, lambda: ops.window_attention(qd, pool, db, page, G, d, 0.1, win, sink=zeros, keep_first=kf), steps, warmup, flush)
        cb = B * min(S, win + kf) * 2 * G * d * 2
        like[tag + "_decode"] = {"us": round(t * 1e6, 1), "of_roofline": round(cb / hbm / t, 3), "cache_bytes": cb}
    # the attention's front kernel: convolution + whole-projection norm + rotation + paged store, against convolution + rotation + store
    Cq = (H + G) * d
    proj = torch.randn(S, Cq + G * d, device="cuda")
    conv = torch.randn(Cq, 4, device="cuda").bfloat16()
    conv3 = torch.randn(Cq + G * d, 4, device="cuda").bfloat16()
    nq, nk = torch.ones(H * d, device="cuda").bfloat16(), torch.ones(G * d, device="cuda").bfloat16()
    st, st3 = torch.zeros(B + 1, 3, Cq, device="cuda"), torch.zeros(B + 1, 3, Cq + G * d, device="cuda")
    table = ops.rope_table(pb.tok_pos, d // 2, 10000.0)
    t = _time_kernel(torch, lambda: ops.qk_conv_norm_rope_append(proj, conv, nq, nk, 1e-5, st, table, d // 2, pool, pb, page, H, G, d, d, True), steps, warmup, flush)
    by = S * (Cq * 4 + (H * d + 2 * G * d) * 2)
    like["conv_norm_rope_append"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3)}
    t = _time_kernel(torch, lambda: ops.qkv_conv_rope_append(proj, conv3, st3, table, d // 2, pool, pb, page, H, G, d, d), steps, warmup, flush)
    by = S * (Cq + G * d) * (4 + 2)
    like["nililix_conv_rope_append"] = {"us": round(t * 1e6, 1), "of_roofline": round(by / hbm / t, 3)}
    del pool, q, proj
    # residual steps and the norms behind the recurrences
    W = s["width"]
    x, y1, y2 = (torch.randn(S, W, device="cuda") for _ in range(3))
    w, b = torch.ones(W, device="cuda").bfloat16(), torch.zeros(W, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.residual_sandwich_layernorm_rows(x, y1, w, b, 1.0, 1e-5, w, b, torch.bfloat16), steps, warmup, flush)
    like["residual_sandwich_layernorm"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * W * (3 * 4 + 2) / hbm / t, 3)}
    t = _time_kernel(torch, lambda: ops.residual_layernorm_rows(x, y1, y2, 0.7, w, b, 1e-6, torch.bfloat16), steps, warmup, flush)
    like["mimolix_residual_layernorm"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * W * (4 * 4 + 2) / hbm / t, 3)}
    t = _time_kernel(torch, lambda: ops.rmsnorm_pair_sum(y1, y2, w, w, 1e-5, 0.5), steps, warmup, flush)
    like["pair_norm_mean"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * W * 3 * 4 / hbm / t, 3)}
    sd = s["side"]
    se, wg, wp = torch.randn(s["vocab"], 6 * sd, device="cuda").bfloat16(), torch.randn(sd, W, device="cuda").bfloat16() * W ** -0.5, torch.randn(W, sd, device="cuda").bfloat16()
    ids = torch.randint(0, s["vocab"], (S,), device="cuda", dtype=torch.int32)
    t = _time_kernel(torch, lambda: ops.token_side_input(x, se, sd, ids, wg, wp, w, 1e-5, w_pre=w, b_pre=b, out_dtype=torch.bfloat16), steps, warmup, flush)
    like["token_side_input"] = {"us": round(t * 1e6, 1), "of_roofline": round((S * W * (2 * 4 + 2) + 2 * sd * W * 2) / hbm / t, 3)}
    MH, mdv = s["m_heads"], s["m_vdim"]
    o, gate, mm = torch.randn(S, MH, mdv + 1, device="cuda"), torch.randn(S, MH * mdv, device="cuda"), torch.randn(S, MH, device="cuda")
    wn = torch.ones(MH * mdv, device="cuda").bfloat16()
    t = _time_kernel(torch, lambda: ops.head_norm_gate(o, mdv, 1e-5, torch.bfloat16, w=wn, w_per_head=True, gate=gate, gate_act="sigmoid", m=mm), steps, warmup, flush)
    like["head_norm_gate"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * MH * mdv * (4 + 4 + 2) / hbm / t, 3)}
    o2, wv = torch.randn(S, DH, ddv, device="cuda"), torch.ones(ddv, device="cuda").bfloat16()
    g2 = torch.randn(S, DH * ddv, device="cuda")
    t = _time_kernel(torch, lambda: ops.gated_rmsnorm_heads(o2, wv, 1e-6, torch.bfloat16, gate=g2), steps, warmup, flush)
    like["mimolix_gated_rmsnorm_heads"] = {"us": round(t * 1e6, 1), "of_roofline": round(S * DH * ddv * (4 + 4 + 2) / hbm / t, 3)}
    res["like_kernels"] = like
    res["peaks"] = peaks
    torch.cuda.empty_cache()
    return res


def run(args):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --model needs a B200 (sm_100a): there is no CPU path")
    sizes, fn = {"nililix": (NILILIX_SIZES, bench_nililix_size), "mimolix": (MIMOLIX_SIZES, bench_mimolix_size),
                 "zobasun": (SIZES, bench_size), "duzizen": (DUZIZEN_SIZES, bench_duzizen_size)}[args.model]
    names = args.model_sizes.split(",") if args.model_sizes else list(sizes)
    out = {"bench": "model_compare", "model": args.model, "dtype": "bf16" if args.model in ("mimolix", "duzizen") else "bf16 (llama: fp16)", "data": "synthetic",
           "steps": args.steps, "warmup": max(3, args.warmup), "sizes": {}}
    for nm in names:
        out["sizes"][nm] = fn(torch, nm, args.steps, args.warmup)
    print(json.dumps(out))
