"""Sequence-mixing and feed-forward mechanisms for models served as a ragged in-flight batch.

Each class holds one layer's device tensors in the layout its kernels want and has ``forward(x, ctx)``: ``x`` is the
fp32 residual stream [rows, width] of this step's token rows, ``ctx`` (``inflight.StepContext``) carries the batch
description, the paged pools and the state slots.  Every size and constant is a constructor argument, so a model
definition (``models/``) only maps its configuration and tensor names onto them.  The arithmetic is in the CUDA
operators of ``ops`` (include/trtllm_b200_ragged.h); nothing here computes on the host.

Precision: the residual stream, normalisations, softmax, the recurrent state and all that feeds the recurrence are fp32;
projections run in the storage type ``dtype`` (bf16 on tensor cores with fp32 accumulation, or fp32 throughout).
"""
from __future__ import annotations

import torch

from . import ops


class LatentAttention:
    """Attention whose keys and values are up-projections of one cached low-rank latent per position.

    h -> query latent (RMS-normed) -> per-head queries [dim unrotated | rot_dim rotated];
    h -> [lat latent (RMS-normed) | rot_dim rotated key part shared by the heads] = the cache entry.
    score_h(i, j) = scale * (q_h^nope(i) . (W_uk,h c_j) + q_h^rot(i) . k^rot_j), causal softmax, out = W_o concat_h(W_uv,h sum_j p c_j).

    The key up-projection is applied to the QUERY (q_h^nope W_uk,h, a [lat] vector) and the value up-projection to the
    attention-weighted latent, so prefill and decode both run one multi-query kernel over the cache entries and nothing
    per head is ever stored per position.  ``kv_source`` names the layer whose pool is read: the layer itself, or an
    earlier layer with the same latent geometry when this layer has no down-projection of its own."""

    def __init__(self, index, *, heads, dim, rot_dim, vdim, lat, rot_dims, rot_base, scale, eps, w_dq, w_dq_norm, w_uq,
                 w_uk, w_uv, w_o, w_dkv=None, w_dkv_norm=None, kv_source=None):
        self.index, self.heads, self.dim, self.rot_dim, self.vdim, self.lat = index, heads, dim, rot_dim, vdim, lat
        self.rot_dims, self.rot_base, self.scale, self.eps = rot_dims, float(rot_base), float(scale), float(eps)
        self.dtype = w_dq.dtype
        self.w_dq, self.w_dq_norm, self.w_uq, self.w_o = w_dq, w_dq_norm, w_uq, w_o
        # per head: [lat, dim] so that the "output" of the batched product is the absorbed query
        self.w_uk_t = w_uk.view(heads, dim, lat).transpose(1, 2).contiguous()
        self.w_uv = w_uv.view(heads, vdim, lat).contiguous()
        self.w_dkv, self.w_dkv_norm = w_dkv, w_dkv_norm
        self.owns_cache = w_dkv is not None
        self.kv_source = index if self.owns_cache else kv_source
        if not self.owns_cache and (kv_source is None or kv_source >= index):
            raise ValueError(f"layer {index}: a layer without its own latent projection reads an EARLIER layer's cache")
        if rot_dims > rot_dim or rot_dims % 2:
            raise ValueError(f"layer {index}: rotary dims {rot_dims} must be even and at most rot_dim {rot_dim}")

    @property
    def cache_entry(self):
        return self.lat + self.rot_dim

    def cache_entries(self):
        return {"own": self.cache_entry} if self.owns_cache else {}

    def conv_state(self):
        return None

    def forward(self, x, ctx, rep=0):
        n, H, dn, dr, R = x.shape[0], self.heads, self.dim, self.rot_dim, self.lat
        f32 = torch.float32
        cq = ops.rmsnorm_rows(ops.linear(x, self.w_dq, out_dtype=f32), self.w_dq_norm, self.eps, out_dtype=self.dtype)
        q = ops.linear(cq, self.w_uq, out_dtype=f32)
        table = ctx.rope_table(self.rot_dims, self.rot_base)
        if self.owns_cache:
            kv = ops.linear(x, self.w_dkv, out_dtype=f32)
            ops.latent_kv_append(ctx.pools[(self.index, rep)], kv, self.w_dkv_norm, self.eps, table, self.rot_dims, ctx.batch,
                                 ctx.page, R, dr)
        qa = torch.empty((n, H, R + dr), dtype=self.dtype, device=x.device)
        ops.linear(q.view(n, H, dn + dr)[:, :, :dn], self.w_uk_t, out=qa[:, :, :R])
        ops.rope_query_tail(qa, q, table, H, dn, dr, self.rot_dims, R)
        lat_out = ops.latent_attention(qa, ctx.pools[(self.kv_source, rep)], ctx.batch, ctx.page, H, R, dr, self.scale)
        heads_out = torch.empty((n, H, self.vdim), dtype=self.dtype, device=x.device)
        ops.linear(lat_out, self.w_uv, out=heads_out)
        return ops.linear(heads_out.view(n, H * self.vdim), self.w_o, out_dtype=f32)


class GatedLinearRecurrence:
    """Recurrent block with a real-gated linear recurrent unit (De et al., "Griffin: Mixing Gated Linear Recurrences
    with Local Attention for Efficient Language Models", 2024).

    Two branches of ``channels``: y = gelu_tanh(W_y h + b_y); u = causal per-channel conv over ``taps`` inputs of
    (W_x h + b_x).  With u cut into ``blocks`` parts, r = sigmoid(A_b u_b + a_b), i = sigmoid(B_b u_b + b_b),
    a = exp(-decay_scale * r * softplus(lam)), S <- a S + sqrt(1 - a^2) i u, output W_o (S * y).
    Per sequence the layer carries S (fp32 [channels]) and the last taps - 1 convolution inputs in a state slot."""

    def __init__(self, index, *, channels, blocks, taps, w_y, b_y, w_x, b_x, conv_w, conv_b, w_ra, b_ra, w_ri, b_ri, lam,
                 w_o, decay_scale=8.0):
        if channels % blocks:
            raise ValueError(f"layer {index}: {channels} channels do not split into {blocks} blocks")
        self.index, self.channels, self.blocks, self.taps, self.decay_scale = index, channels, blocks, taps, decay_scale
        self.dtype = w_y.dtype
        self.w_y, self.b_y, self.w_x, self.b_x, self.conv_w, self.conv_b = w_y, b_y, w_x, b_x, conv_w.contiguous(), conv_b
        # per block: the recurrence-gate rows, then the input-gate rows -> one batched product gives both logits
        self.w_gates = torch.cat([w_ra, w_ri], dim=1).contiguous()       # [blocks, 2 bw, bw]
        self.b_gates = torch.cat([b_ra, b_ri], dim=1).contiguous()       # [blocks, 2 bw]
        self.lam, self.w_o = lam, w_o

    def cache_entries(self):
        return {}

    def conv_state(self):
        return (self.taps, self.channels, self.channels)

    def forward(self, x, ctx, rep=0):
        n, f32 = x.shape[0], torch.float32
        bw = self.channels // self.blocks
        y = ops.linear(x, self.w_y, bias=self.b_y, out_dtype=self.dtype, act=ops.ACT_GELU_TANH)
        xb = ops.linear(x, self.w_x, bias=self.b_x, out_dtype=f32)
        conv_state, rec_state = ctx.states[(self.index, rep)]
        u = ops.causal_conv1d(xb, self.conv_w, self.conv_b, conv_state, ctx.batch)
        gates = torch.empty((n, self.blocks, 2 * bw), dtype=f32, device=x.device)
        ops.linear(u.view(n, self.blocks, bw), self.w_gates, bias=self.b_gates, out=gates, compute=ops.COMPUTE_FMA32)
        s = ops.rglru_scan(u, gates, self.lam, y, rec_state, ctx.batch, self.blocks, self.decay_scale)
        return ops.linear(s, self.w_o, out_dtype=f32)


class WindowedAttention:
    """Grouped-query attention over a sliding window with short convolutions, a softmax sink and per-head output gates.

    q = W_q h, k = W_k h, v = W_v h (``heads`` query heads and ``kv_heads`` key/value heads of size ``dim``; values of
    size ``vdim``; query head i reads key/value head i // (heads / kv_heads)).  Every channel of q, k and v then runs a
    causal convolution over time with ``taps`` taps (tap j weighs the input taps - 1 - j positions back; tap taps - 1 the
    current one), and the first
    ``rot_dims`` elements of each query and key head are rotated as interleaved pairs (2i, 2i + 1) by position times
    base^(-2i / rot_dims), optionally with the long wavelengths slowed (``rot_scaling`` = (factor, low, high, original)).
    score(i, j) = scale * q_i . k_j for 0 <= i - j < window (window 0: all j <= i); the softmax denominator holds one
    more term exp(sink_head) without a value; head outputs are multiplied by sigmoid(W_g h)_head and projected by W_o.

    Variants, all optional: ``keep_first`` > 0 — with a window, the first positions of a sequence stay visible to every later
    row (at their true positions); ``q_norm`` / ``k_norm`` — between convolution and rotation the whole q projection and the
    whole k projection (all heads at once) are RMS-normalised with a weight per channel (``eps``); ``w_v`` None — the values
    are the keys as they leave the convolution, before norm and rotation (vdim == dim); ``conv_q`` None — no convolution.

    The input projections are ONE product against the stacked [q | k | v | g] rows.  Per sequence the layer carries
    the last taps - 1 projected q | k | v rows (fp32) in a state slot and its rotated keys and values in pages of a pool
    (entry = [kv_heads * dim keys | kv_heads * vdim values])."""

    def __init__(self, index, *, heads, kv_heads, dim, vdim, taps, scale, window=0, rot_dims=0, rot_base=10000.0,
                 rot_scaling=None, w_q, w_k, w_v=None, conv_q=None, conv_k=None, conv_v=None, w_o, sink=None, w_g=None,
                 keep_first=0, q_norm=None, k_norm=None, eps=1e-6):
        if heads % kv_heads:
            raise ValueError(f"layer {index}: {heads} query heads do not split over {kv_heads} key/value heads")
        if rot_dims % 2 or rot_dims > dim or (rot_dims and dim % 2):
            raise ValueError(f"layer {index}: rotary dims {rot_dims} must be even and at most the (even) head size {dim}")
        self.index, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = index, heads, kv_heads, dim, vdim, int(taps)
        self.scale, self.window, self.rot_dims, self.rot_base = float(scale), int(window or 0), int(rot_dims), float(rot_base)
        self.rot_scaling = tuple(float(v) for v in rot_scaling) if rot_scaling else None
        self.dtype = w_q.dtype
        self.tied = w_v is None
        if self.tied and vdim != dim:
            raise ValueError(f"layer {index}: values that are the keys have the keys' size ({vdim} != {dim})")
        if (q_norm is None) != (k_norm is None):
            raise ValueError(f"layer {index}: query and key norm come together")
        self.keep_first, self.q_norm, self.k_norm, self.eps = int(keep_first or 0), q_norm, k_norm, float(eps)
        self.channels = heads * dim + kv_heads * dim + (0 if self.tied else kv_heads * vdim)
        self.w_in = torch.cat([w_q, w_k] + ([] if self.tied else [w_v]) + ([w_g] if w_g is not None else []), dim=0).contiguous()
        if conv_q is None:
            self.conv_w, self.taps = None, 1
        else:
            self.conv_w = torch.cat([conv_q, conv_k] + ([] if self.tied else [conv_v]), dim=0).contiguous()
            if self.conv_w.shape != (self.channels, self.taps):
                raise ValueError(f"layer {index}: convolution weights {tuple(self.conv_w.shape)} != {(self.channels, self.taps)}")
        # the plain form (projected values, no norm) keeps its own kernel, whose rows may be spread over several CTAs
        self.whole_norm = self.tied or q_norm is not None or self.conv_w is None
        self.gated, self.sink, self.w_o = w_g is not None, sink, w_o

    def cache_entries(self):
        return {"own": self.kv_heads * (self.dim + self.vdim)}

    def conv_state(self):
        return None if self.whole_norm and self.taps == 1 else (self.taps, self.channels, 0)

    def forward(self, x, ctx, rep=0, proj=None):
        """``proj``: the rows' input projection (fp32 [N, >= w_in rows], any row stride) when a caller has already run it as part
        of a wider stacked product; ``x`` is then not read."""
        n, key = x.shape[0], (self.index, rep)
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        table = ctx.rope_table(self.rot_dims, self.rot_base, self.rot_scaling) if self.rot_dims else None
        if self.whole_norm:
            q = ops.qk_conv_norm_rope_append(proj, self.conv_w, self.q_norm, self.k_norm, self.eps,
                                             ctx.states[key][0] if self.taps > 1 else None, table, self.rot_dims, ctx.pools[key],
                                             ctx.batch, ctx.page, self.heads, self.kv_heads, self.dim, self.vdim, self.tied)
        else:
            q = ops.qkv_conv_rope_append(proj, self.conv_w, ctx.states[key][0], table, self.rot_dims, ctx.pools[key], ctx.batch,
                                         ctx.page, self.heads, self.kv_heads, self.dim, self.vdim)
        o = ops.window_attention(q, ctx.pools[key], ctx.batch, ctx.page, self.kv_heads, self.vdim, self.scale, self.window,
                                 sink=self.sink, gate=proj[:, self.channels:] if self.gated else None, keep_first=self.keep_first)
        return ops.linear(o.view(n, self.heads * self.vdim), self.w_o, out_dtype=torch.float32)


class DifferentialAttention:
    """Grouped-query attention in which every query head holds TWO attention maps over one set of values; the head's output
    is the first map's minus lambda times the second's, normalised.

    q = W_q h has ``heads`` x 2 vectors of ``dim`` ([head][map]), k = W_k h has ``kv_heads`` x 2, v = W_v h has ``kv_heads``
    vectors of ``vdim``; query head i reads key/value head i // (heads / kv_heads).  Every query and key vector is
    RMS-normalised over dim with one weight for all queries and one for all keys; a query at position p is also multiplied by
    the temperature 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every 0: none).  Nothing is rotated.
    a_m(i) = softmax_j(scale * q_m(i) . k_m(j)) v(j) over j <= i (and i - j < window, if one is given), m = 1, 2;
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff;  o = a_1 - lambda a_2;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff);
    out = W_o concat_heads(o).

    The three input projections are ONE product against the stacked rows, with the query rows reordered at load to
    [kv head][map][head of the group]: the 2 * heads (head, map) queries are then plain grouped queries over 2 * kv_heads key
    heads ([kv head][map], the stored order) whose neighbouring pairs share a value head, and the attention kernels of the
    other models run them (``ops.window_attention`` with ``v_share`` = 2), returning both maps in fp32.  Per sequence the layer
    keeps its normalised keys and its values in pages of a pool (entry = [2 kv_heads * dim keys | kv_heads * vdim values])."""

    def __init__(self, index, *, heads, kv_heads, dim, vdim, scale, diff, eps, w_q, w_k, w_v, q_norm, k_norm, lq1, lk1, lq2, lk2,
                 w_o, temp_coef=0.0, temp_every=0, window=0):
        if heads % kv_heads:
            raise ValueError(f"layer {index}: {heads} query heads do not split over {kv_heads} key/value heads")
        per, width = heads // kv_heads, w_q.shape[1]
        if w_q.shape[0] != heads * 2 * dim or w_k.shape[0] != kv_heads * 2 * dim or w_v.shape[0] != kv_heads * vdim:
            raise ValueError(f"layer {index}: projections {tuple(w_q.shape)}, {tuple(w_k.shape)}, {tuple(w_v.shape)} do not hold two "
                             f"maps of {heads} / {kv_heads} heads of {dim} and values of {vdim}")
        self.index, self.heads, self.kv_heads, self.dim, self.vdim = index, heads, kv_heads, dim, vdim
        self.scale, self.diff, self.eps, self.window = float(scale), float(diff), float(eps), int(window or 0)
        self.temp_coef, self.temp_every = float(temp_coef), int(temp_every or 0)
        self.dtype = w_q.dtype
        w_q = w_q.view(kv_heads, per, 2, dim, width).permute(0, 2, 1, 3, 4).reshape(heads * 2 * dim, width)
        self.w_in = torch.cat([w_q, w_k, w_v], dim=0).contiguous()
        self.q_norm, self.k_norm, self.lam = q_norm, k_norm, (lq1, lk1, lq2, lk2)
        self.w_o = w_o

    def cache_entries(self):
        return {"own": self.kv_heads * (2 * self.dim + self.vdim)}

    def conv_state(self):
        return None

    def forward(self, x, ctx, rep=0):
        n, pool = x.shape[0], ctx.pools[(self.index, rep)]
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        q = ops.qk_norm_append(proj, self.q_norm, self.k_norm, self.eps, pool, ctx.batch, ctx.page, 2 * self.heads, 2 * self.kv_heads,
                               self.dim, self.kv_heads * self.vdim, self.temp_coef, self.temp_every)
        maps = ops.window_attention(q, pool, ctx.batch, ctx.page, 2 * self.kv_heads, self.vdim, self.scale, self.window, v_share=2,
                                    out_f32=True)
        o = ops.diff_combine(maps, *self.lam, self.diff, self.eps, 1.0 - self.diff, self.kv_heads, self.dtype)
        return ops.linear(o.view(n, self.heads * self.vdim), self.w_o, out_dtype=torch.float32)


class GatedDeltaRule:
    """Recurrent layer with a matrix state per head that is updated by the delta rule under a learned decay (Yang, Kautz,
    Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule", 2024).

    q = W_q h, k = W_k h (``kv_heads`` vectors of ``dim``), v = W_v h (``heads`` vectors of ``vdim``; head i reads query / key
    head i // (heads / kv_heads)); every channel of q, k, v runs a causal convolution over ``taps`` inputs (the last tap weighs
    the current one) and SiLU; q and k become unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q also times dim^-1/2.
    beta = sigmoid(W_b h), g = exp(-exp(A_log) * softplus(W_a h + dt_bias)) per head.  Per head and token, in this order:
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    then o / sqrt(mean(o^2) + eps) * norm * silu(W_g h) per head, and W_o on the concatenated heads.

    The six input projections are ONE product against the stacked [q | k | v | g | b | a] rows (fp32 out: beta, the decay
    and everything else that enters the recurrence is fp32).  Per sequence the layer carries S (fp32, [heads, vdim, dim]) and
    the last taps - 1 projected q | k | v rows in a state slot."""

    def __init__(self, index, *, heads, kv_heads, dim, vdim, taps, eps, w_q, w_k, w_v, conv_q, conv_k, conv_v, w_b, w_a, a_log,
                 dt_bias, norm, w_g, w_o, unit_eps=1e-6):
        if heads % kv_heads:
            raise ValueError(f"layer {index}: {heads} heads do not split over {kv_heads} query/key heads")
        self.index, self.heads, self.kv_heads, self.dim, self.vdim, self.taps = index, heads, kv_heads, dim, vdim, int(taps)
        self.eps, self.unit_eps, self.dtype = float(eps), float(unit_eps), w_q.dtype
        self.channels = 2 * kv_heads * dim + heads * vdim
        if w_q.shape[0] != kv_heads * dim or w_k.shape[0] != kv_heads * dim or w_v.shape[0] != heads * vdim \
                or w_g.shape[0] != heads * vdim or w_b.shape[0] != heads or w_a.shape[0] != heads:
            raise ValueError(f"layer {index}: projection shapes do not match {heads} heads of {vdim} over {kv_heads} x {dim}")
        self.w_in = torch.cat([w_q, w_k, w_v, w_g, w_b, w_a], dim=0).contiguous()
        self.col_g = self.channels
        self.col_b = self.col_g + heads * vdim
        self.col_a = self.col_b + heads
        self.conv_w = torch.cat([conv_q, conv_k, conv_v], dim=0).contiguous()
        if self.conv_w.shape != (self.channels, self.taps):
            raise ValueError(f"layer {index}: convolution weights {tuple(self.conv_w.shape)} != {(self.channels, self.taps)}")
        self.a_log, self.dt_bias, self.norm, self.w_o = a_log, dt_bias, norm, w_o

    def cache_entries(self):
        return {}

    def conv_state(self):
        return (self.taps, self.channels, self.heads * self.vdim * self.dim)

    def forward(self, x, ctx, rep=0):
        n = x.shape[0]
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        conv_state, rec_state = ctx.states[(self.index, rep)]
        u, bg = ops.delta_prepare(proj, self.conv_w, self.a_log, self.dt_bias, self.col_b, self.col_a, conv_state, ctx.batch,
                                  self.heads, self.kv_heads, self.dim, self.vdim, self.unit_eps)
        o = ops.delta_rule_scan(u, bg, rec_state, ctx.batch, self.heads, self.kv_heads, self.dim, self.vdim)
        y = ops.gated_rmsnorm_heads(o, self.norm, self.eps, self.dtype, gate=proj[:, self.col_g:self.col_b])
        return ops.linear(y.view(n, self.heads * self.vdim), self.w_o, out_dtype=torch.float32)


class Retention:
    """Linear attention with a fixed decay per head and no softmax or denominator (Sun et al., "Retentive Network: A Successor to
    Transformer for Large Language Models", 2023, in its recurrent form).

    q = W_q h, k = W_k h (``heads`` vectors of ``dim``), v = W_v h (``heads`` vectors of ``vdim``); the first ``rot_dims``
    elements of every q and k head are rotated by position (``rot_layout``: element i pairs with i + rot_dims / 2 ("half") or 2i
    with 2i + 1 ("interleaved")), then k is multiplied by ``k_scale``.  Per head S <- decay_h S + k v^T, o = S^T q; o is divided
    by its root mean square over vdim (no weight), the heads are concatenated, multiplied by silu(W_g h) and projected by W_o.

    The four input projections are ONE product against the stacked [q | k | v | g] rows (fp32 out: what enters the recurrence
    is fp32).  Per sequence the layer carries S (fp32 [heads, vdim, dim]) in a state slot."""

    def __init__(self, index, *, heads, dim, vdim, decay, eps, w_q, w_k, w_v, w_g, w_o, k_scale=1.0, rot_dims=0, rot_base=10000.0,
                 rot_scaling=None, rot_layout="half"):
        if len(decay) != heads:
            raise ValueError(f"layer {index}: {len(decay)} decays for {heads} heads")
        if w_q.shape[0] != heads * dim or w_k.shape[0] != heads * dim or w_v.shape[0] != heads * vdim or w_g.shape[0] != heads * vdim:
            raise ValueError(f"layer {index}: projection shapes do not match {heads} heads of {dim} / {vdim}")
        if rot_dims % 2 or rot_dims > dim:
            raise ValueError(f"layer {index}: rotary dims {rot_dims} must be even and at most the head size {dim}")
        self.index, self.heads, self.dim, self.vdim, self.eps, self.k_scale = index, heads, dim, vdim, float(eps), float(k_scale)
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.rot_scaling = tuple(float(v) for v in rot_scaling) if rot_scaling else None
        self.rot_layout = {"half": ops.ROPE_HALF, "interleaved": ops.ROPE_INTERLEAVED}[rot_layout]
        self.dtype = w_q.dtype
        self.decay = torch.tensor([float(d) for d in decay], dtype=torch.float32, device=w_q.device)
        self.w_in = torch.cat([w_q, w_k, w_v, w_g], dim=0).contiguous()
        self.col_v = 2 * heads * dim
        self.col_g = self.col_v + heads * vdim
        self.w_o = w_o

    def cache_entries(self):
        return {}

    def conv_state(self):
        return (1, 0, self.heads * self.vdim * self.dim)

    def forward(self, x, ctx, rep=0, proj=None):
        """``proj``: the rows' input projection (fp32 [N, >= w_in rows], any row stride) when a caller has already run it as part
        of a wider stacked product; ``x`` is then not read."""
        n, H = x.shape[0], self.heads
        if proj is None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        table = ctx.rope_table(self.rot_dims, self.rot_base, self.rot_scaling) if self.rot_dims else None
        qk = ops.rope_heads(proj, table, 2 * H, self.dim, self.rot_dims, self.rot_layout, split=H, scale_lo=1.0, scale_hi=self.k_scale)
        o = ops.decay_attention_scan(qk, qk[:, H * self.dim:], proj[:, self.col_v:self.col_g], ctx.states[(self.index, rep)][1],
                                     ctx.batch, H, self.dim, self.vdim, head_decay=self.decay)
        y = ops.head_norm_gate(o, self.vdim, self.eps, self.dtype, gate=proj[:, self.col_g:], gate_act="silu")
        return ops.linear(y.view(n, H * self.vdim), self.w_o, out_dtype=torch.float32)


class MatrixMemory:
    """The matrix memory of an mLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory", 2024) with exponential gates that a
    running maximum keeps in range.

    q = W_q h * dim^-1/2, k = W_k h (``heads`` vectors of ``dim``), v = W_v h (``heads`` vectors of ``vdim``).  Per head a log
    input gate i = cap * tanh((W_i h + b_i) / cap) and a log forget gate f = logsigmoid(cap * tanh((W_f h + b_f) / cap)) (``gate_cap``
    0: no cap).  With m_0 = 0, S_0 = 0, n_0 = 0:  m_t = max(f_t + m_(t-1), i_t);  S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) +
    exp(i_t - m_t) k_t v_t^T;  n_t likewise with k_t alone;  o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps).
    Each head's o is divided by its root mean square over vdim, the heads are concatenated, multiplied by ``norm``
    ([heads * vdim]) and by sigmoid(W_g h), and projected by W_o.

    The six input projections are ONE product against the stacked [q | k | v | g | i | f] rows (fp32 out).  n is the state of one
    more value column whose value is 1 at every token, so the recurrence is the decayed linear attention the retention runs
    (``ops.decay_attention_scan`` with ``ones_col``).  Per sequence the layer carries [S | n] (fp32 [heads, vdim + 1, dim]) and m
    ([heads]) in a state slot."""

    def __init__(self, index, *, heads, dim, vdim, eps, w_q, w_k, w_v, w_g, w_i, b_i, w_f, b_f, norm, w_o, gate_cap=0.0, den_eps=1e-6):
        if w_q.shape[0] != heads * dim or w_k.shape[0] != heads * dim or w_v.shape[0] != heads * vdim or w_g.shape[0] != heads * vdim \
                or w_i.shape[0] != heads or w_f.shape[0] != heads or norm.shape[0] != heads * vdim:
            raise ValueError(f"layer {index}: projection shapes do not match {heads} heads of {dim} / {vdim}")
        self.index, self.heads, self.dim, self.vdim, self.eps = index, heads, dim, vdim, float(eps)
        self.gate_cap, self.den_eps, self.dtype = float(gate_cap or 0.0), float(den_eps), w_q.dtype
        self.w_in = torch.cat([w_q, w_k, w_v, w_g, w_i, w_f], dim=0).contiguous()
        self.col_k = heads * dim
        self.col_v = 2 * heads * dim
        self.col_g = self.col_v + heads * vdim
        self.col_i = self.col_g + heads * vdim
        self.col_f = self.col_i + heads
        self.b_i, self.b_f, self.norm, self.w_o = b_i, b_f, norm, w_o
        self.state_cols = heads * (vdim + 1) * dim           # [S | n]; the maxima follow

    def cache_entries(self):
        return {}

    def conv_state(self):
        return (1, 0, self.state_cols + self.heads)

    def forward(self, x, ctx, rep=0):
        n, H = x.shape[0], self.heads
        proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        rec = ctx.states[(self.index, rep)][1]
        log_ab, m = ops.mlstm_gates(proj, self.col_i, self.col_f, self.b_i, self.b_f, self.gate_cap, rec[:, self.state_cols:], ctx.batch, H)
        o = ops.decay_attention_scan(proj, proj[:, self.col_k:self.col_v], proj[:, self.col_v:self.col_g], rec, ctx.batch, H, self.dim,
                                     self.vdim, log_ab=log_ab, ones_col=True, q_scale=self.dim ** -0.5)
        y = ops.head_norm_gate(o, self.vdim, self.eps, self.dtype, w=self.norm, w_per_head=True, gate=proj[:, self.col_g:self.col_i],
                               gate_act="sigmoid", m=m, den_eps=self.den_eps)
        return ops.linear(y.view(n, H * self.vdim), self.w_o, out_dtype=torch.float32)


class SideBySideMixers:
    """Two sequence mixers that read the same input; the result is ``mult`` * (rms_norm(left(h)) * w_left + rms_norm(right(h)) *
    w_right), each output normalised over the model width with its own weight.  Caches and states are the union of the two
    (at most one of them may page a cache, at most one may carry convolution inputs, at most one a recurrent state).
    Mixers that open with one stacked input projection (``w_in``, and ``forward(..., proj=)``) share ONE product against
    [left rows | right rows]: the input is read once and a generation step launches one streaming product instead of two."""

    def __init__(self, index, left, right, *, w_left, w_right, eps, mult=0.5):
        self.index, self.left, self.right, self.w_left, self.w_right = index, left, right, w_left, w_right
        self.eps, self.mult, self.dtype = float(eps), float(mult), left.dtype
        cl, cr = left.conv_state() or (1, 0, 0), right.conv_state() or (1, 0, 0)
        if (left.cache_entries() and right.cache_entries()) or (cl[0] > 1 and cr[0] > 1) or (cl[2] and cr[2]):
            raise NotImplementedError(f"layer {index}: both side-by-side mixers want the same kind of cache or state")
        conv = cl if cl[0] > 1 else cr
        self._state = (conv[0], conv[1], cl[2] or cr[2]) if (conv[0] > 1 or cl[2] or cr[2]) else None
        self.w_in = None
        if getattr(left, "w_in", None) is not None and getattr(right, "w_in", None) is not None and left.w_in.dtype == right.w_in.dtype:
            self.split = left.w_in.shape[0]
            self.w_in = torch.cat([left.w_in, right.w_in], dim=0).contiguous()
            left.w_in = right.w_in = None                    # held once, stacked

    def cache_entries(self):
        return self.left.cache_entries() or self.right.cache_entries()

    def conv_state(self):
        return self._state

    def forward(self, x, ctx, rep=0):
        if self.w_in is not None:
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
            a = self.left.forward(x, ctx, rep, proj=proj[:, :self.split])
            b = self.right.forward(x, ctx, rep, proj=proj[:, self.split:])
        else:
            a = self.left.forward(x, ctx, rep)
            b = self.right.forward(x, ctx, rep)
        return ops.rmsnorm_pair_sum(a, b, self.w_left, self.w_right, self.eps, self.mult)


class TokenSideInput:
    """A per-layer input from the token itself, added to the residual stream after the layer's sublayers: e = the layer's
    ``dim`` columns (from ``offset``) of a side embedding of the token; g = gelu_tanh(W_gate x) * e; y = W_proj g;
    x <- x + y / rms(y) * norm.  One kernel, which also emits the next sublayer's normalised input when asked to."""

    def __init__(self, *, side_embed, offset, w_gate, w_proj, norm, eps):
        if tuple(w_proj.shape) != (w_gate.shape[1], w_gate.shape[0]) or side_embed.shape[1] < offset + w_gate.shape[0]:
            raise ValueError(f"token side input: gate {tuple(w_gate.shape)}, proj {tuple(w_proj.shape)}, columns {offset}.. of "
                             f"{tuple(side_embed.shape)}")
        self.side_embed, self.offset, self.w_gate, self.w_proj, self.norm, self.eps = side_embed, int(offset), w_gate, w_proj, norm, float(eps)

    def forward(self, x, ctx, next_norm=None, out_dtype=torch.float32):
        """In place on x.  next_norm = (weight, bias or None, is_rms): -> that norm of the new x in ``out_dtype``; else None."""
        w, b, rms = next_norm if next_norm is not None else (None, None, False)
        return ops.token_side_input(x, self.side_embed, self.offset, ctx.batch.tok_ids, self.w_gate, self.w_proj, self.norm, self.eps,
                                    w_pre=w, b_pre=b, pre_rms=rms, out_dtype=out_dtype)


class SquaredReluMLP:
    """out = W_down max(W_up h, 0)^2; the activation is the up projection's epilogue."""

    def __init__(self, *, w_up, w_down):
        self.w_up, self.w_down, self.dtype = w_up, w_down, w_down.dtype

    def forward(self, x, ctx):
        return ops.linear(ops.linear(x, self.w_up, out_dtype=self.dtype, act=ops.ACT_RELU_SQUARED), self.w_down,
                          out_dtype=torch.float32)


class RoutedExpertsMLP:
    """Mixture of experts: each token runs ``top`` of ``experts`` small feed-forwards, gated ones
    W_down (silu(W_gate h) * W_up h) or, without ``w_gate``, plain ones W_down act(W_up h) (``act``: squared ReLU, ...).

    Router (fp32 logits W_router h), one of
      ``"sigmoid_groups"``: s = sigmoid(logit); choice = s + correction; the experts form ``groups`` equal groups of
        neighbours, a group scores the sum of its two largest choices and only the ``keep`` best groups stay eligible; the
        ``top`` largest eligible choices are taken and weighted by their plain s (not renormalised);
      ``"softmax"``: s = softmax over all experts; the ``top`` largest are taken and weighted by s / (sum of the chosen s +
        1e-20) * ``route_scale`` (``renorm``) or s * ``route_scale``.
    ``shared``: a feed-forward every token runs besides (anything with ``forward(x, ctx)``); its output joins the weighted sum.
    Gated experts may clamp: ``gate_alpha``, ``gate_limit``, ``gate_up_shift`` as in ``ClampedGatedMLP`` (1, 0, 0 is silu(gate) * up).
    ``weight_on`` = "input": the chosen score multiplies the expert's INPUT, out = sum expert(s h) (gated experts only).  Gate and
    up projections are linear, so the score is applied to their fp32 results, in front of the activation, and the experts'
    outputs are summed unweighted.
    The (token, choice) pairs are sorted by expert on the device into whole tiles and both expert products walk that plan
    (tcgen05 tiles of 128 rows for bf16, warp-MMA / FMA tiles of 64 otherwise), so a step costs ``top`` experts per token
    whatever the batch; a generation step's few pairs run one streaming product each instead."""

    def __init__(self, *, w_router, w_up, w_down, top, w_gate=None, correction=None, groups=1, keep=1, router="sigmoid_groups",
                 renorm=True, route_scale=1.0, act=ops.ACT_RELU_SQUARED, shared=None, gate_alpha=1.0, gate_limit=0.0,
                 gate_up_shift=0.0, weight_on="output"):
        """w_gate, w_up: [experts, ff, width]; w_down: [experts, width, ff]."""
        self.experts, self.top, self.groups, self.keep = w_up.shape[0], int(top), int(groups), int(keep)
        if self.experts % self.groups or not 1 <= self.keep <= self.groups or not 1 <= self.top <= self.experts:
            raise ValueError(f"router: {self.experts} experts, {groups} groups (keep {keep}), top {top}")
        if router not in ("sigmoid_groups", "softmax"):
            raise ValueError(f"unknown router kind {router!r}")
        self.router, self.renorm, self.route_scale, self.shared = router, bool(renorm), float(route_scale), shared
        self.w_router, self.correction = w_router, correction
        self.gated, self.act = w_gate is not None, int(act)
        if weight_on not in ("output", "input") or (weight_on == "input" and not self.gated):
            raise ValueError(f"router weights on the {weight_on!r} of {'gated' if self.gated else 'plain'} experts")
        self.on_input = weight_on == "input"
        self.g_alpha, self.g_limit, self.g_shift = float(gate_alpha), float(gate_limit), float(gate_up_shift)
        if self.gated:
            self.w_gate_up = torch.cat([w_gate, w_up], dim=1).contiguous()      # [experts, 2 ff, width]: gate rows, then up rows
        else:
            self.w_up = w_up.contiguous()
        self.w_down, self.dtype = w_down.contiguous(), w_down.dtype

    def forward(self, x, ctx):
        n, top, K = x.shape[0], self.top, x.shape[1]
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32, compute=ops.COMPUTE_FMA32)
        if self.router == "softmax":
            ids, weights = ops.moe_route_softmax(logits, top, self.renorm, self.route_scale)
        else:
            ids, weights = ops.moe_route(logits, self.correction, top, self.groups, self.keep)
        add = self.shared.forward(x, ctx) if self.shared is not None else None
        bf16 = self.dtype == torch.bfloat16
        if not self.gated:
            # plain experts: the activation is the up projection's epilogue in every kernel
            if bf16 and n * top <= ops.MOE_GEMV_MAX_PAIRS and not ops.FORCE_TILE_LINEAR:
                h = ops.moe_gemv(x, self.w_up, ids, a_div=top, out_dtype=self.dtype, act=self.act)
                y = ops.moe_gemv(h, self.w_down, ids, a_div=0, out_dtype=torch.float32) if h is not None else None
                if y is not None:
                    return ops.moe_combine(y, weights, add=add)
            if bf16 and n * top >= ops.TC_MIN_ROWS and K % 8 == 0 and self.w_down.shape[2] % 8 == 0 and not ops.FORCE_TILE_LINEAR:
                slot_pair, tile_expert, pair_slot = ops.moe_plan(ids, self.experts, ops.MOE_TILE_TC)
                h = ops.moe_linear_tc(ops.moe_gather_rows(x, slot_pair, top), self.w_up, tile_expert, self.dtype, act=self.act)
                y = ops.moe_linear_tc(h, self.w_down, tile_expert, torch.float32)
                return ops.moe_combine(y, weights, pair_slot, add=add)
            slot_pair, tile_expert, pair_slot = ops.moe_plan(ids, self.experts, ops.MOE_TILE)
            h = ops.moe_linear(x, self.w_up, slot_pair, tile_expert, a_div=top, out_dtype=self.dtype, act=self.act)
            y = ops.moe_linear(h, self.w_down, slot_pair, tile_expert, a_div=0, out_dtype=torch.float32)
            return ops.moe_combine(y, weights, pair_slot, add=add)
        ga = (self.g_alpha, self.g_limit, self.g_shift)
        scale = weights.view(-1) if self.on_input else None          # per pair, in front of the activation
        out_w = (n, top) if self.on_input else weights               # ... and then the outputs are summed as they are
        if bf16 and n * top <= ops.MOE_GEMV_MAX_PAIRS and not ops.FORCE_TILE_LINEAR:
            # generation steps: one streaming product per pair, gate / up and the activation in one kernel, no plan
            act = ops.moe_gemv(x, self.w_gate_up, ids, a_div=top, out_dtype=self.dtype, gated=True, alpha=ga[0], limit=ga[1],
                               up_shift=ga[2], pair_scale=scale)
            y = ops.moe_gemv(act, self.w_down, ids, a_div=0, out_dtype=torch.float32) if act is not None else None
            if y is not None:
                return ops.moe_combine(y, out_w, add=add)
        if bf16 and n * top >= ops.TC_MIN_ROWS and K % 8 == 0 and self.w_down.shape[2] % 8 == 0 and not ops.FORCE_TILE_LINEAR:
            # prompt-sized steps: the tcgen05 kernel over a plan of 128-row tiles
            slot_pair, tile_expert, pair_slot = ops.moe_plan(ids, self.experts, ops.MOE_TILE_TC)
            gu = ops.moe_linear_tc(ops.moe_gather_rows(x, slot_pair, top), self.w_gate_up, tile_expert, torch.float32)
            act = ops.gated_act(gu, self.dtype, *ga, row_scale=scale, row_index=slot_pair if self.on_input else None)
            y = ops.moe_linear_tc(act, self.w_down, tile_expert, torch.float32)
            return ops.moe_combine(y, out_w, pair_slot, add=add)
        slot_pair, tile_expert, pair_slot = ops.moe_plan(ids, self.experts, ops.MOE_TILE)
        gu = ops.moe_linear(x, self.w_gate_up, slot_pair, tile_expert, a_div=top, out_dtype=torch.float32)
        act = ops.gated_act(gu, self.dtype, *ga, row_scale=scale, row_index=slot_pair if self.on_input else None)
        y = ops.moe_linear(act, self.w_down, slot_pair, tile_expert, a_div=0, out_dtype=torch.float32)
        return ops.moe_combine(y, out_w, pair_slot, add=add)


class ClampedGatedMLP:
    """g = min(W_gate h, limit), u = clamp(W_up h, +-limit), y = g * sigmoid(alpha g) * (u + up_shift), out = W_down y; or, with
    ``gate`` = "gelu_tanh", y = gelu_tanh(W_gate h) * (W_up h).
    Gate and up rows are stored as one [2 ff, width] matrix (gate rows first), as the other models' fc_gate is."""

    def __init__(self, *, w_gate, w_up, w_down, limit=0.0, alpha=1.702, up_shift=1.0, gate="sigmoid"):
        self.w_gate_up = torch.cat([w_gate, w_up], dim=0).contiguous()
        self.w_down, self.limit, self.alpha, self.up_shift = w_down, float(limit), float(alpha), float(up_shift)
        self.gate = {"sigmoid": ops.GATE_SIGMOID, "gelu_tanh": ops.GATE_GELU_TANH}[gate]
        self.dtype = w_down.dtype

    def forward(self, x, ctx):
        act = ops.linear_gated(x, self.w_gate_up, self.dtype, self.alpha, self.limit, self.up_shift, gate=self.gate)    # generation steps
        if act is None:
            gu = ops.linear(x, self.w_gate_up, out_dtype=torch.float32)
            act = ops.gated_act(gu, self.dtype, self.alpha, self.limit, self.up_shift, gate=self.gate)
        return ops.linear(act, self.w_down, out_dtype=torch.float32)


class LayerStackModel:
    """Embedding, a stack of (mixer, optional feed-forward) layers, output norm and head.

    A layer is a dict: ``mixer``, ``mlp`` (or None) and per sublayer a norm weight applied to its INPUT (``pre1`` /
    ``pre2``, None: the sublayer reads the residual stream itself) and one applied to its OUTPUT (``post1`` / ``post2``):
    x <- x + residual_mult * norm_post(f(norm_pre(x))).  Norm weights are stored around ``norm_offset`` below 1 (the
    multiplier is w + norm_offset).

    ``parallel``: the layer's sublayers run side by side on ONE normalised input instead, x <- x + residual_mult *
    (mixer(h) + mlp(h)) with h = norm(x; ``pre1``).  ``norm`` = "layer" (every norm of the stack and the output norm): layer norm
    (x - mean) / sqrt(var + eps) * w + b with the biases in ``pre1_b`` / ``post1_b`` / ``pre2_b`` / ``post2_b`` /
    ``final_norm_b``; "rms": the RMS norm above.

    A layer's ``side`` (``TokenSideInput`` or None) is added to the stream after the layer's sublayers.  ``embed_pair`` =
    (table [buckets + 1, width], mul_prev, mul_cur): a hashed embedding of the (previous, current) token pair is added to the
    token embedding (``ops.embed_bigram``); the previous token of a sequence's first new row comes with the batch.

    ``loop`` = (start, stop, times): layers start .. stop - 1 run ``times`` times in a row with the same weights; every
    pass has caches and states of its own.  Right before pass t's first layer row t of ``loop_step`` is added to the residual
    stream, and / or the stream is re-projected together with the embedding output x0, x <- ``loop_in`` [x ; x0] (``loop_in``
    [width, 2 width], the stream's columns first).  ``logit_cap`` > 0: logits <- cap * tanh(logits / cap)."""

    def __init__(self, *, vocab, width, dtype, embed, layers, final_norm, head, eps, embed_scale=1.0, norm_offset=0.0,
                 residual_mult=1.0, loop=None, loop_step=None, logit_cap=0.0, norm="rms", parallel=False, final_norm_b=None,
                 loop_in=None, embed_pair=None):
        self.vocab, self.width, self.dtype, self.eps, self.norm_offset = vocab, width, dtype, float(eps), float(norm_offset)
        self.embed, self.embed_scale, self.layers, self.final_norm, self.head = embed, float(embed_scale), layers, final_norm, head
        self.residual_mult, self.logit_cap, self.loop_step = float(residual_mult), float(logit_cap or 0.0), loop_step
        if norm not in ("rms", "layer"):
            raise ValueError(f"unknown norm kind {norm!r}")
        if norm == "rms" and parallel:
            raise NotImplementedError("side-by-side sublayers go with layer norm")
        if norm == "layer" and norm_offset:
            raise NotImplementedError("layer norm weights are stored as they are applied")
        self.norm, self.parallel, self.final_norm_b, self.loop_in = norm, bool(parallel), final_norm_b, loop_in
        self.embed_pair = embed_pair
        if embed_pair is not None and tuple(embed_pair[0].shape[1:]) != (width,):
            raise ValueError(f"pair embedding {tuple(embed_pair[0].shape)} is not [buckets + 1, {width}]")
        if loop_in is not None and tuple(loop_in.shape) != (width, 2 * width):
            raise ValueError(f"loop input projection {tuple(loop_in.shape)} != {(width, 2 * width)}")
        for l in layers:
            for k in ("pre1", "post1", "pre2", "post2", "pre1_b", "post1_b", "pre2_b", "post2_b", "side"):
                l.setdefault(k, None)
            if parallel and l["side"] is not None:
                raise NotImplementedError("a per-layer token input with side-by-side sublayers")
        n = len(layers)
        if loop is None or loop[1] <= loop[0]:
            self.runs = [(i, 0, False) for i in range(n)]
        else:
            start, stop, times = (int(v) for v in loop)
            if not (0 <= start < stop <= n) or times < 1:
                raise ValueError(f"loop {loop} does not fit {n} layers")
            if loop_step is not None and tuple(loop_step.shape) != (times, width):
                raise ValueError(f"loop step vectors {tuple(loop_step.shape)} != {(times, width)}")
            self.runs = [(i, 0, False) for i in range(start)]
            for t in range(times):
                self.runs += [(i, t, i == start) for i in range(start, stop)]
            self.runs += [(i, 0, False) for i in range(stop, n)]

    # what the session has to provide: one pool / state per (layer, pass)
    def cache_layers(self):
        return {(i, t): self.layers[i]["mixer"].cache_entries()["own"] for i, t, _ in self.runs
                if self.layers[i]["mixer"].cache_entries()}

    def state_layers(self):
        return {(i, t): self.layers[i]["mixer"].conv_state() for i, t, _ in self.runs
                if self.layers[i]["mixer"].conv_state() is not None}

    def forward(self, ctx, on_layer=None):
        """-> the fp32 residual stream after the last layer; ``on_layer(run, x)`` sees it after every layer run.

        Each sublayer is x <- x + residual_mult * norm_post(f(norm_pre(x))).  Where the next sublayer has a norm on its
        input and nothing is added to x in between, its input comes out of the same kernel as this sublayer's residual
        update (``ops.residual_norm_rows``)."""
        if self.parallel:
            return self._forward_parallel(ctx, on_layer)
        if self.loop_in is not None:
            raise NotImplementedError("loop input projection with sublayers in a row")
        x = self._embed(ctx)
        layer_norm = self.norm == "layer"
        subs = []                # (function of h, pre (weight, bias), post (weight, bias), step vector, run if it ends one, side input)
        for run, (i, t, first) in enumerate(self.runs):
            l = self.layers[i]
            step = self.loop_step[t] if first and self.loop_step is not None else None
            subs.append((lambda h, l=l, t=t: l["mixer"].forward(h, ctx, t), (l["pre1"], l["pre1_b"]), (l["post1"], l["post1_b"]), step,
                         None if l["mlp"] else run, None if l["mlp"] else l["side"]))
            if l["mlp"] is not None:
                subs.append((lambda h, l=l: l["mlp"].forward(h, ctx), (l["pre2"], l["pre2_b"]), (l["post2"], l["post2_b"]), None, run,
                             l["side"]))
        h = None
        for k, (f, pre, post, step, ends_run, side) in enumerate(subs):
            if step is not None:
                ops.add_row_vector(x, step)
            if h is None:
                if pre[0] is None:
                    h = x
                elif layer_norm:
                    h = ops.layernorm_rows(x, pre[0], pre[1], self.eps, out_dtype=self.dtype)
                else:
                    h = ops.rmsnorm_rows(x, pre[0], self.eps, self.norm_offset, out_dtype=self.dtype)
            y = f(h)
            if post[0] is None:
                raise NotImplementedError("a sublayer whose output is added without a norm")
            nxt = subs[k + 1] if k + 1 < len(subs) else None
            fuse = nxt is not None and nxt[1][0] is not None and nxt[3] is None and nxt[1][0].dtype == post[0].dtype
            npre = nxt[1] if fuse else (None, None)
            # the residual step; the next sublayer's input leaves the same kernel — or the token input's, when one follows
            if layer_norm:
                h = ops.residual_sandwich_layernorm_rows(x, y, post[0], post[1], self.residual_mult, self.eps,
                                                         None if side else npre[0], None if side else npre[1], self.dtype)
            elif fuse and side is None:
                h = ops.residual_norm_rows(x, y, post[0], npre[0], self.eps, self.norm_offset, self.residual_mult, self.dtype)
            else:
                ops.rmsnorm_rows(y, post[0], self.eps, self.norm_offset, out=x, accumulate=True, out_scale=self.residual_mult)
                h = None
            if side is not None:
                fuse_side = fuse and (layer_norm or not self.norm_offset)
                h = side.forward(x, ctx, (npre[0], npre[1], not layer_norm) if fuse_side else None, self.dtype)
            if ends_run is not None and on_layer is not None:
                on_layer(ends_run, x)
        return x

    def _embed(self, ctx):
        if self.embed_pair is None:
            return ops.embed_scaled(self.embed, ctx.batch.tok_ids, self.embed_scale)
        table, mul_prev, mul_cur = self.embed_pair
        return ops.embed_bigram(self.embed, table, ctx.batch.tok_ids, ctx.batch.tok_prev, self.embed_scale, mul_prev, mul_cur)

    def _forward_parallel(self, ctx, on_layer=None):
        """Layers whose mixer and feed-forward read one layer-normalised input.  The residual step of a layer and the next
        layer's norm are ONE kernel (``ops.residual_layernorm_rows``) unless the stream is re-projected in between."""
        x = self._embed(ctx)
        reproject = self.loop_in is not None
        x0 = x.clone() if reproject and not self.runs[0][2] else x      # layers ahead of the looped block update x in place
        h = None
        for run, (i, t, first) in enumerate(self.runs):
            l = self.layers[i]
            if first and self.loop_step is not None:
                ops.add_row_vector(x, self.loop_step[t])
                h = None
            if first and reproject:
                x, h = ops.linear(ops.concat_rows(x, x0, self.dtype), self.loop_in, out_dtype=torch.float32), None
            if h is None:
                h = ops.layernorm_rows(x, l["pre1"], l.get("pre1_b"), self.eps, out_dtype=self.dtype)
            y1 = l["mixer"].forward(h, ctx, t)
            y2 = l["mlp"].forward(h, ctx) if l["mlp"] is not None else None
            nxt = self.runs[run + 1] if run + 1 < len(self.runs) else None
            if nxt is not None and not (nxt[2] and (reproject or self.loop_step is not None)):
                nl = self.layers[nxt[0]]
                h = ops.residual_layernorm_rows(x, y1, y2, self.residual_mult, nl["pre1"], nl.get("pre1_b"), self.eps, self.dtype)
            else:
                ops.residual_layernorm_rows(x, y1, y2, self.residual_mult)
                h = None
            if on_layer is not None:
                on_layer(run, x)
        return x

    def logits(self, x, rows_idx):
        if self.norm == "layer":
            h = ops.layernorm_rows(x, self.final_norm, self.final_norm_b, self.eps, out_dtype=self.dtype, rows_idx=rows_idx)
            z = ops.linear(h, self.head, out_dtype=torch.float32)
            return ops.tanh_cap(z, self.logit_cap) if self.logit_cap > 0 else z
        h = ops.rmsnorm_rows(x, self.final_norm, self.eps, self.norm_offset, out_dtype=self.dtype, rows_idx=rows_idx)
        z = ops.linear(h, self.head, out_dtype=torch.float32)
        return ops.tanh_cap(z, self.logit_cap) if self.logit_cap > 0 else z
