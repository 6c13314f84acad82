"""The Mimolix design (differential attention with normalised, temperature-scaled queries; gated delta-rule layers; softmax
routed squared-ReLU experts with a shared expert; parallel layers under a layer norm; a looped block that re-reads the
embedding) on the GPU against the plain float64 oracle (oracle/mimolix_plain.py): every mechanism alone, prefill against
token-by-token decoding, portions down to two tokens, unequal batches against each request alone, pages and slots used
again, keys far away and at page borders, the temperature's steps, the first tokens of a sequence, long decoding, other
sizes, and greedy generation through the scheduler."""
import json
import math
import os

import pytest
import torch

from oracle import mimolix_plain as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}      # relative to the largest magnitude of the compared tensor


def _close(got, want, dtype, what, scale=1.0):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    err = (got - want).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= TOL[dtype] * scale * ref, f"{what}: max error {err:.3e} against magnitude {ref:.3e}"


AT_ODD = dict(type="attention", heads=6, kv_heads=2, dim=10, vdim=6, diff=0.3, q_temp=(0.7, 5), scale=0.5)
AT_MQ = dict(type="attention", heads=5, kv_heads=1, dim=8, vdim=40, diff=0.0, scale=0.6)                     # group of 5 > 4 warps, no temperature
AT_MH = dict(type="attention", heads=3, kv_heads=3, dim=16, vdim=16, diff=0.6, q_temp=(0.25, 1), scale=0.3)  # a group of one
AT_TC = dict(type="attention", heads=8, kv_heads=2, dim=32, vdim=32, diff=0.45, q_temp=(0.6, 16), scale=0.25)  # tensor-core sizes
DL_ODD = dict(type="delta", heads=6, kv_heads=2, dim=10, vdim=7, conv=3)
DL_ONE = dict(type="delta", heads=3, kv_heads=3, dim=48, vdim=9, conv=1)          # no convolution, one query head per head
DL_BIG = dict(type="delta", heads=4, kv_heads=1, dim=64, vdim=32, conv=4)
DL_WIDE = dict(type="delta", heads=2, kv_heads=2, dim=130, vdim=20, conv=2)       # dim neither a power of two nor a multiple of 32
STACKS = {
    "odd": dict(layers=[dict(DL_ODD, mlp=(20, 6, 2, 1.7, 14)), dict(AT_ODD, mlp=(12, 5, 3, 1.0, None)), dict(DL_ONE, mlp=None),
                        dict(AT_MQ, mlp=(16, 4, 1, 2.5, 8))], width=40, vocab=61, loop=(1, 3, 3)),
    "tc": dict(layers=[dict(AT_TC, mlp=(32, 8, 3, 2.0, 48)), dict(DL_BIG, mlp=(24, 8, 2, 1.0, 32)),
                       dict(AT_TC, dim=64, kv_heads=8, mlp=(16, 5, 5, 0.5, None)), dict(DL_BIG, kv_heads=2, conv=2, mlp=None)],
               width=64, vocab=130, loop=(0, 2, 2), residual_mult=1.3, embed_scale=1.5),
    "plain": dict(layers=[dict(AT_MH, mlp=(30, 3, 2, 1.0, 10)), dict(DL_WIDE, mlp=None), dict(AT_MQ, q_temp=(1.0, 3), mlp=None)],
                  width=32, vocab=40, loop=None, residual_mult=1.0, embed_scale=1.0, eps=1e-6),
    "one-pass": dict(layers=[dict(DL_ODD, conv=2, mlp=(8, 2, 2, 3.0, 8)), dict(AT_ODD, mlp=None)], width=24, vocab=33, loop=(1, 2, 1)),
}

_ORACLE = {}


def _weights(name, dtype, seed):
    """Whole stacks run in bf16 get routers whose ranking cannot hang on rounding (``spaced_router``): with random routers
    some token's two best scores lie within bf16 rounding of each other, another expert runs for it, and everything that
    reads that token differs — which is no kernel's error.  The fp32 runs keep random routers."""
    return O.random_mimolix(seed=seed, spaced_router=dtype == torch.bfloat16, **STACKS[name])


def _oracle(name, dtype, seed, toks, layers=False):
    key = (name, dtype == torch.bfloat16, seed, tuple(toks))
    if key not in _ORACLE:
        cfg, t = _weights(name, dtype, seed)
        _ORACLE[key] = O.mimolix_forward(cfg, t, toks, return_layers=True)
    return _ORACLE[key] if layers else _ORACLE[key][0]


def _model(name, dtype, seed=0):
    from trtllm_llama_b200.models.mimolix import build_mimolix
    cfg, t = _weights(name, dtype, seed)
    return cfg, t, build_mimolix(cfg, t, dtype, "cuda")


def _session(model, max_tokens=512, max_seqs=4, page=64):
    from trtllm_llama_b200.inflight import InflightSession
    return InflightSession(model, max_tokens, max_seqs, page)


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ---------------------------------------------------------------------------------------------------------------
# operators alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("cols", [24, 72, 300, 1030])
def test_layer_norm_and_the_fused_residual_step(cols):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(cols)
    x = torch.randn(11, cols, generator=g) * 3 + 5.0            # a mean far from zero: the variance must be of the deviations
    w, b = (torch.randn(cols, generator=g) * 0.2 + 1).to(torch.bfloat16), (torch.randn(cols, generator=g) * 0.3).to(torch.bfloat16)
    want = O.layer_norm(x.double(), w.double(), b.double(), 1e-5)
    _close(ops.layernorm_rows(x.cuda(), w.cuda(), b.cuda(), 1e-5), want, torch.float32, "layer norm")
    idx = torch.tensor([7, 0, 7, 3], dtype=torch.int32)
    _close(ops.layernorm_rows(x.cuda(), w.cuda(), b.cuda(), 1e-5, rows_idx=idx.cuda()), want[idx.long()], torch.float32, "layer norm of chosen rows")
    y1, y2 = torch.randn(11, cols, generator=g), torch.randn(11, cols, generator=g)
    for second in (y2, None):
        xs = x.clone().cuda()
        h = ops.residual_layernorm_rows(xs, y1.cuda(), second.cuda() if second is not None else None, 0.7, w.cuda(), b.cuda(), 1e-5)
        new = x.double() + 0.7 * (y1.double() + (second.double() if second is not None else 0.0))
        _close(xs, new, torch.float32, "residual step")
        _close(h, O.layer_norm(new, w.double(), b.double(), 1e-5), torch.float32, "next layer's norm from the same kernel")
        xs = x.clone().cuda()
        assert ops.residual_layernorm_rows(xs, y1.cuda(), second.cuda() if second is not None else None, 1.3) is None
        _close(xs, x.double() + 1.3 * (y1.double() + (second.double() if second is not None else 0.0)), torch.float32, "residual step alone")
    for dt in DTYPES:
        cat = ops.concat_rows(x.cuda(), y1.cuda()[:, :cols - 3], dt)
        _close(cat, torch.cat([x, y1[:, :cols - 3]], dim=1), dt, "two streams side by side", scale=0.25)


@pytest.mark.parametrize("E,top,renorm,scale", [(8, 3, True, 2.0), (6, 1, True, 1.0), (5, 5, True, 0.5), (64, 6, False, 1.5), (2, 2, True, 3.0),
                                                (40, 2, True, 1.0)])
def test_softmax_router(E, top, renorm, scale):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    n, W = 57, 24
    h = torch.randn(n, W, generator=g)
    P = {"router": torch.randn(E, W, generator=g) * 0.6}
    logits = ops.linear(h.cuda(), P["router"].cuda(), out_dtype=torch.float32, compute=ops.COMPUTE_FMA32)
    ids, wts = ops.moe_route_softmax(logits, top, renorm, scale)
    ids, wts = ids.cpu().tolist(), wts.cpu()
    want = O.route(h.double(), {k: v.double() for k, v in P.items()}, "", {"experts": E, "top": top, "scale": scale})
    s = torch.softmax(h.double() @ P["router"].double().T, -1)
    for t, (wi, ww) in enumerate(want):
        assert sorted(ids[t]) == sorted(wi), f"token {t}: experts {ids[t]} against {wi}"
        for k, e in enumerate(ids[t]):
            ref = ww[wi.index(e)] if renorm else float(s[t, e]) * scale
            assert abs(float(wts[t, k]) - ref) < 1e-5 * max(1.0, scale), f"token {t}: weight of expert {e}"
    if renorm:
        assert torch.allclose(wts.sum(1), torch.full((n,), scale), atol=1e-5 * scale)


@pytest.mark.parametrize("dtype,tiles", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)],
                         ids=["fp32-fma-tiles", "bf16-streaming-or-tcgen05", "bf16-warp-mma-tiles"])
@pytest.mark.parametrize("shared", [True, False], ids=["shared", "no-shared"])
@pytest.mark.parametrize("n", [1, 5, 40, 150, 700])
def test_routed_experts_alone(dtype, n, tiles, shared, monkeypatch):
    """Every form of the expert products with the squared ReLU as the up projection's epilogue: fp32 FMA tiles, bf16
    warp-MMA tiles, one streaming product per pair (few tokens), tcgen05 tiles over a plan of 128-row tiles (many)."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.layers import RoutedExpertsMLP, SquaredReluMLP
    monkeypatch.setattr(ops, "FORCE_TILE_LINEAR", tiles)
    g = torch.Generator().manual_seed(n)
    W, ff, E, top = 40, 24, 6, 3
    r = lambda *s, std: (torch.randn(*s, generator=g) * std).to(dtype)
    P = {"router": r(E, W, std=0.5), "shared.up": r(32, W, std=0.3), "shared.down": r(W, 32, std=0.2)}
    for e in range(E):
        P.update({f"e{e}.up": r(ff, W, std=0.3), f"e{e}.down": r(W, ff, std=0.2)})
    mlp = RoutedExpertsMLP(w_router=P["router"].cuda(), w_up=torch.stack([P[f"e{e}.up"] for e in range(E)]).cuda(),
                           w_down=torch.stack([P[f"e{e}.down"] for e in range(E)]).cuda(), top=top, router="softmax", route_scale=1.7,
                           shared=SquaredReluMLP(w_up=P["shared.up"].cuda(), w_down=P["shared.down"].cuda()) if shared else None)
    h = torch.randn(n, W, generator=g).to(dtype)
    got = mlp.forward(h.cuda(), None)
    fc = {"router": {"experts": E, "top": top, "scale": 1.7}, "shared": {"ff": 32} if shared else None}
    _close(got, O.moe_mlp(h.double(), {k: v.double() for k, v in P.items()}, "", fc), dtype, f"routed experts, {n} tokens")


# ---------------------------------------------------------------------------------------------------------------
# the mixers alone, driven through the session's batch description
# ---------------------------------------------------------------------------------------------------------------
def _mixer_ctx(model, lens, page=16, max_seqs=4):
    """A step context for whole sequences of the given lengths: pages dealt in shuffled order, state slots poisoned."""
    from trtllm_llama_b200.inflight import RaggedBatch, StepContext
    sess = _session(model, max_tokens=page * sum(-(-n // page) for n in lens), max_seqs=max_seqs, page=page)
    for conv_state, rec_state in sess.states.values():
        conv_state.fill_(1e3)                   # whatever a slot held before must not matter at a sequence's start
        if rec_state is not None:
            rec_state.fill_(-7.0)
    for pool in sess.pools.values():
        pool.fill_(float("nan"))
    perm = torch.randperm(sess.kv_cache_manager.blocks, generator=torch.Generator().manual_seed(5)).tolist()
    rows, used = [], 0
    for i, n in enumerate(lens):
        nb = -(-n // page)
        rows.append(([0] * n, 0, max_seqs - 1 - i, perm[used:used + nb]))
        used += nb
    return sess, StepContext(RaggedBatch(rows, [], "cuda"), sess.pools, sess.states, page)


def _mixer_alone(dtype, spec, lens, what, fn):
    from trtllm_llama_b200.models.mimolix import build_mimolix
    cfg, t = O.random_mimolix([dict(spec, mlp=None)], width=40, seed=3)
    model = build_mimolix(cfg, t, dtype, "cuda")
    sess, ctx = _mixer_ctx(model, lens)
    h = torch.randn(sum(lens), 40, generator=torch.Generator().manual_seed(4))
    got = model.layers[0]["mixer"].forward(h.to(dtype).cuda(), ctx)
    P, at = {k: v.double() for k, v in t.items()}, 0
    for n in lens:
        want = fn(h[at:at + n].to(dtype).double(), P, "l0.mix.", cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
        _close(got[at:at + n], want, dtype, f"{what}, sequence of {n}")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [AT_ODD, AT_MQ, AT_MH, AT_TC, dict(AT_TC, dim=64, vdim=64, kv_heads=4), dict(AT_TC, dim=64, vdim=32, heads=2, kv_heads=1),
                                  dict(AT_MQ, vdim=70, q_temp=(2.0, 2)), dict(AT_TC, dim=128, vdim=128, heads=2, kv_heads=2)],
                         ids=["odd", "one-kv-head", "group-of-one", "tc", "tc-64", "tc-64-32", "vdim70", "tc-128"])
def test_differential_attention_alone(dtype, spec):
    _mixer_alone(dtype, spec, [75, 5, 1], "differential attention", O.differential_attention_mixer)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [DL_ODD, DL_ONE, DL_BIG, DL_WIDE, dict(DL_ODD, conv=6, vdim=33), dict(DL_BIG, dim=128, vdim=16, heads=2, kv_heads=2)],
                         ids=["odd", "no-conv", "big", "dim130", "six-taps", "dim128"])
def test_delta_rule_mixer_alone(dtype, spec):
    _mixer_alone(dtype, spec, [45, 5, 1, 19], "gated delta rule", O.delta_mixer)


def _diff_attention_ops(q, k, v, lam4, scale, diff, eps, coef, every, cuts, dtype, page, blocks, wq=None, wk=None):
    """q [P, H, 2, d], k [P, G, 2, d], v [P, G, dv] as projected -> the three operators of the layer over the cache, the prompt
    cut as ``cuts``."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    P, H, _, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    per = H // G
    qp = q.view(P, G, per, 2, d).permute(0, 1, 3, 2, 4)               # [g][map][head of the group]
    proj = torch.cat([qp.reshape(P, -1), k.reshape(P, -1), v.reshape(P, -1)], dim=1).float().cuda()
    pool = torch.full((len(blocks) * page, G * (2 * d + dv)), float("nan"), dtype=dtype, device="cuda")
    at, outs = 0, []
    for n in cuts:
        b = RaggedBatch([([0] * n, at, 0, blocks)], [], "cuda")
        qq = ops.qk_norm_append(proj[at:at + n], wq, wk, eps, pool, b, page, 2 * H, 2 * G, d, G * dv, coef, every)
        maps = ops.window_attention(qq, pool, b, page, 2 * G, dv, scale, 0, v_share=2, out_f32=True)
        outs.append(ops.diff_combine(maps, *[x.to(dtype).cuda() for x in lam4], diff, eps, 1.0 - diff, G, dtype))
        at += n
    return torch.cat(outs)


def _diff_attention_plain(q, k, v, lam4, scale, diff, eps, coef, every):
    P, H, _, d = q.shape
    G = k.shape[1]
    qn, kn = O.rms(q.double(), eps), O.rms(k.double(), eps)
    if every:
        for p in range(P):
            qn[p] = qn[p] * O.query_temperature(p, coef, every)
    lam = O.differential_lambda(dict(zip(("lq1", "lk1", "lq2", "lk2"), [x.double() for x in lam4])), "", diff)
    out = torch.zeros(P, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        g = h // (H // G)
        a1 = O.causal_softmax_attention(qn[:, h, 0], kn[:, g, 0], v[:, g].double(), scale)
        a2 = O.causal_softmax_attention(qn[:, h, 1], kn[:, g, 1], v[:, g].double(), scale)
        out[:, h] = O.rms(a1 - lam * a2, eps) * (1.0 - diff)
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("dist", [0, 1, 15, 16, 17, 31, 32, 33, 64, 150, 290])
def test_one_key_stands_out_in_one_map(dtype, where, dist):
    """ONE key decides the first map and nothing the second: the query and that key are large along one direction in map 1
    only, the key's value is far from the others.  The key sits on the query's own position, at page borders (pages of 16),
    or far back among hundreds of keys, in a prompt or with the last tokens decoded one by one."""
    page, P, H, G, d, dv = 16, 300, 4, 2, 8, 8
    g = torch.Generator().manual_seed(dist)
    q, k = torch.randn(P, H, 2, d, generator=g) * 0.3, torch.randn(P, G, 2, d, generator=g) * 0.3
    v = torch.randn(P, G, dv, generator=g)
    qi = P - 1 if where == "decoded" else P - 4
    kj = qi - dist
    k[:, :, 0, 0] *= 0.03                      # no other key of map 1 points along the query's direction
    q[qi, :, 0, :] = 0.01
    q[qi, :, 0, 0] = 5.0
    k[kj, :, 0, :] = 0.01
    k[kj, :, 0, 0] = 5.0
    v[kj] = torch.tensor([40.0, -40.0] * (dv // 2))
    lam4 = [torch.full((d,), 0.2), torch.full((d,), 0.3), torch.full((d,), -0.1), torch.full((d,), 0.4)]
    want = _diff_attention_plain(q, k, v, lam4, 2.0, 0.25, 1e-6, 0.0, 0)
    diffuse = _diff_attention_plain(q, k, torch.where(torch.arange(P)[:, None, None] == kj, torch.zeros(()), v), lam4, 2.0, 0.25, 1e-6, 0.0, 0)
    assert (want[qi] - diffuse[qi]).abs().max() > 0.3, "the case does not show the key"
    blocks = torch.randperm(-(-P // page), generator=g).tolist()
    cuts = [P] if where == "prompt" else [P - 5, 1, 1, 1, 1, 1]
    got = _diff_attention_ops(q, k, v, lam4, 2.0, 0.25, 1e-6, 0.0, 0, cuts, dtype, page, blocks)
    _close(got[qi], want[qi], dtype, f"key {dist} back ({where})")
    if dtype == torch.float32:        # elsewhere the two maps nearly cancel, and the normalisation enlarges what bf16 keys and values lose
        _close(got, want, dtype, f"all rows, key {dist} back ({where})", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("every,coef", [(1, 0.5), (4, 1.5), (16, 0.5), (64, 2.0)])
def test_query_temperature_steps(dtype, every, coef):
    """The temperature steps where floor((p + 1) / every) does: positions every - 2, every - 1 (the first with one whole block)
    and the multiples after it, as a prompt and decoded one by one behind a prompt that ends right before a step."""
    page, H, G, d, dv = 16, 2, 1, 16, 8
    sc = 0.9 if dtype == torch.float32 else 0.15        # bf16 queries and keys: scores small enough that their rounding stays small
    P = max(3 * every + 2, 8)
    g = torch.Generator().manual_seed(every)
    q, k, v = torch.randn(P, H, 2, d, generator=g), torch.randn(P, G, 2, d, generator=g), torch.randn(P, G, dv, generator=g)
    wq, wk = torch.randn(d, generator=g) * 0.3 + 1.5, torch.randn(d, generator=g) * 0.3 + 1.5
    lam4 = [torch.randn(d, generator=g) * 0.2 for _ in range(4)]
    # the plain form applies the weight after the norm: norm(x) * w
    def plain(coef_, every_):
        qn, kn = O.rms(q.double(), 1e-5) * wq.to(dtype).double(), O.rms(k.double(), 1e-5) * wk.to(dtype).double()
        for p in range(P):
            qn[p] = qn[p] * O.query_temperature(p, coef_, every_)
        lam = O.differential_lambda(dict(zip(("lq1", "lk1", "lq2", "lk2"), [x.to(dtype).double() for x in lam4])), "", 0.4)
        out = torch.zeros(P, H, dv, dtype=torch.float64)
        for h in range(H):
            a1 = O.causal_softmax_attention(qn[:, h, 0], kn[:, 0, 0], v[:, 0].double(), sc)
            a2 = O.causal_softmax_attention(qn[:, h, 1], kn[:, 0, 1], v[:, 0].double(), sc)
            out[:, h] = O.rms(a1 - lam * a2, 1e-5) * 0.6
        return out
    want = plain(coef, every)
    if every > 1:
        assert (want[every - 1] - plain(0.0, 1)[every - 1]).abs().max() > 1e-3, "the temperature does not show at its first step"
    blocks = torch.randperm(-(-P // page), generator=g).tolist()
    for cuts in ([P], [max(every - 1, 1)] + [1] * (P - max(every - 1, 1))):
        got = _diff_attention_ops(q, k, v, lam4, sc, 0.4, 1e-5, coef, every, cuts, dtype, page, blocks, wq.to(dtype).cuda(), wk.to(dtype).cuda())
        _close(got, want, dtype, f"temperature every {every}, cuts {cuts[:3]}", scale=2.0)


@pytest.mark.parametrize("d,dv,H,G", [(32, 32, 4, 2), (64, 32, 6, 1), (64, 64, 8, 2), (96, 96, 2, 1), (128, 64, 4, 2), (128, 128, 8, 2), (48, 24, 4, 2),
                                      (32, 16, 3, 3)])
def test_differential_attention_head_sizes(d, dv, H, G):
    """Every head size the tensor-core attention kernel is built for (and one it is not), with value heads shared by the two
    maps and fp32 results: a prompt of 300 positions over shuffled pages, then three tokens decoded one by one — few rows over a
    long context, so their key tiles are dealt to several CTAs and merged — against the plain formula and the SIMT kernel."""
    from trtllm_llama_b200 import ops
    page, P, dt = 16, 303, torch.bfloat16
    g = torch.Generator().manual_seed(d * 7 + dv)
    q, k, v = torch.randn(P, H, 2, d, generator=g).to(dt), torch.randn(P, G, 2, d, generator=g).to(dt), torch.randn(P, G, dv, generator=g).to(dt)
    lam4 = [torch.randn(d, generator=g) * 0.1 for _ in range(4)]
    want = _diff_attention_plain(q, k, v, [x.to(dt) for x in lam4], d ** -0.5 * 2, 0.3, 1e-6, 0.4, 100)
    blocks = torch.randperm(-(-P // page), generator=g).tolist()
    outs = {}
    for simt in (False, True):
        ops.FORCE_SIMT_ATTENTION = simt
        try:
            outs[simt] = _diff_attention_ops(q.float(), k.float(), v.float(), lam4, d ** -0.5 * 2, 0.3, 1e-6, 0.4, 100, [P - 3, 1, 1, 1], dt, page, blocks)
        finally:
            ops.FORCE_SIMT_ATTENTION = False
    _close(outs[True], want, dt, f"SIMT attention {d}/{dv}")
    _close(outs[False], want, dt, f"attention {d}/{dv}")


@pytest.mark.parametrize("cuts", [[600], [1] * 40 + [560], [17, 16, 15, 2, 250, 300], [599, 1]])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 12), (2, 1, 64, 8), (3, 3, 40, 33), (16, 4, 128, 80), (40, 8, 24, 32), (30, 6, 10, 50), (10, 2, 130, 128)])
def test_delta_rule_remembers_far_tokens(H, G, d, dv, cuts):
    """The recurrence over 600 tokens with decays close to 1, so that what was written hundreds of tokens ago still decides the
    read-out: cut into portions (state carried in a slot that held another sequence's state) against the plain loop."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    g = torch.Generator().manual_seed(d)
    P = sum(cuts)
    q, k = O.unit(torch.randn(P, G, d, generator=g).double()) * d ** -0.5, O.unit(torch.randn(P, G, d, generator=g).double())
    v = torch.randn(P, H, dv, generator=g).double()
    beta, dec = 0.1 * torch.rand(P, H, generator=g).double(), 1.0 - 0.004 * torch.rand(P, H, generator=g).double()
    want = torch.stack([O.delta_rule(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], dec[:, h]) for h in range(H)], dim=1)
    recent = torch.stack([O.delta_rule(q[300:, h // (H // G)], k[300:, h // (H // G)], v[300:, h], beta[300:, h], dec[300:, h]) for h in range(H)], dim=1)
    assert (want[-1] - recent[-1]).abs().max() > 1e-2 * want[-1].abs().max(), "the first 300 tokens do not show at the end"
    u = torch.cat([q.reshape(P, -1), k.reshape(P, -1), v.reshape(P, -1)], dim=1).float().cuda()
    bg = torch.cat([beta, dec], dim=1).float().cuda()
    for serial in (False, True):              # eight rows at a time (portions of three rows and more), and row by row
        ops.FORCE_SERIAL_SCAN = serial
        try:
            state = torch.full((3, H * dv * d), 9.0, device="cuda")
            at, outs = 0, []
            for n in cuts:
                b = RaggedBatch([([0] * n, at, 1, [0])], [], "cuda")
                outs.append(ops.delta_rule_scan(u[at:at + n], bg[at:at + n], state, b, H, G, d, dv))
                at += n
        finally:
            ops.FORCE_SERIAL_SCAN = False
        _close(torch.cat(outs), want, torch.float32, f"delta rule over {P} tokens, cuts {cuts[:4]}, row by row: {serial}")
        assert bool((state[0] == 9.0).all()) and bool((state[2] == 9.0).all()), "another slot's state was touched"


# ---------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(STACKS))
def test_prefill_matches_oracle_and_decode(dtype, name):
    cfg, t, model = _model(name, dtype)
    toks = _tokens(83, cfg["vocab"], 9)
    want, want_layers = _oracle(name, dtype, 0, toks, layers=True)
    sess = _session(model, max_tokens=256, page=16)
    layers = []
    got = sess.step([("a", toks, list(range(len(toks))))], on_layer=lambda i, x: layers.append(x.clone()))
    assert len(layers) == len(want_layers)
    for i, (g_, w_) in enumerate(zip(layers, want_layers)):
        _close(g_, w_, dtype, f"{name}: residual stream after layer run {i}", scale=2.0)
    _close(got, want, dtype, f"{name}: whole prompt", scale=2.0)
    rows = [sess.step([("b", [tok], [0])])[0] for tok in toks]          # token by token from position 0
    _close(torch.stack(rows), want, dtype, f"{name}: token-by-token", scale=2.0)
    _close(torch.stack(rows), got, dtype, f"{name}: prefill against decoding", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "tc"])
@pytest.mark.parametrize("cuts", [[2, 2, 2, 77], [1, 15, 1, 16, 17, 33], [31, 2, 50], [64, 19], [3] * 27 + [2]])
def test_portions(dtype, cuts, name):
    cfg, t, model = _model(name, dtype)
    toks = _tokens(sum(cuts), cfg["vocab"], 10)
    want = _oracle(name, dtype, 0, toks)
    sess = _session(model, max_tokens=128, page=16)
    at, rows = 0, []
    for n in cuts:
        rows.append(sess.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    _close(torch.cat(rows), want, dtype, f"{name}: portions {cuts[:6]}", scale=2.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "tc", "plain"])
def test_mixed_batches_and_reuse(dtype, name):
    """Five requests of unequal length through FOUR slots and a pool that cannot hold them all at once: portions beside
    single tokens, requests that sit a step out, pages and slots handed on — every logit equals the request run alone."""
    cfg, t, model = _model(name, dtype)
    lens = {"a": 70, "b": 33, "c": 5, "d": 90, "e": 41}
    toks = {k: _tokens(n, cfg["vocab"], 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: _oracle(name, dtype, 0, v) for k, v in toks.items()}
    sess = _session(model, max_tokens=16 * 16, max_seqs=4, page=16)      # 16 pages; the five need 5 + 3 + 1 + 6 + 3 = 18
    plan = [  # (request, tokens it brings) per step
        [("a", 3), ("b", 2)], [("a", 30), ("b", 1), ("c", 2)], [("a", 1), ("c", 3), ("d", 17)], [("b", 29), ("d", 2)],
        [("a", 36), ("b", 1), ("d", 40)], [("d", 1), ("e", 16)], [("d", 30), ("e", 1)], [("e", 24)],
    ]
    at, got = {k: 0 for k in lens}, {k: [] for k in lens}
    for step in plan:
        entries = [(k, toks[k][at[k]:at[k] + n], list(range(n))) for k, n in step]
        out, row = sess.step(entries), 0
        for k, n in step:
            got[k].append(out[row:row + n])
            row, at[k] = row + n, at[k] + n
            if at[k] == lens[k]:
                sess.end(k)
    assert at == lens and not sess.live
    assert len(sess.kv_cache_manager.free_blocks) == 16 and sorted(sess.slot_manager.free) == [0, 1, 2, 3]
    for k in lens:
        _close(torch.cat(got[k]), want[k], dtype, f"{name}: request {k} in mixed batches", scale=2.0)


@pytest.mark.parametrize("graph", [True, False], ids=["replayed-graph", "eager"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tc", "odd"])
def test_long_decoding_across_pages(dtype, graph, name):
    """180 generated tokens: the temperature steps several times, the block table outgrows its captured width and the
    recurrent state is carried 180 times; replayed graphs and eager launches of the same step give the same answer."""
    cfg, t, model = _model(name, dtype, seed=2)
    toks = _tokens(20 + 180, cfg["vocab"], 30)
    want = _oracle(name, dtype, 2, toks)
    sess = _session(model, max_tokens=208, page=16)
    sess.use_cuda_graph = graph
    rows = [sess.step([("a", toks[:20], [19])])[0]]
    rows += [sess.step([("a", [tok], [0])])[0] for tok in toks[20:]]
    _close(torch.stack(rows), want[19:], dtype, f"{name}: 180 decoded tokens", scale=2.0)
    assert bool(sess._graphs) == graph


@pytest.mark.parametrize("dtype,name", [(torch.float32, "odd"), (torch.float32, "tc"), (torch.bfloat16, "tc"), (torch.bfloat16, "plain")])
def test_greedy_generation_through_the_scheduler(dtype, name):
    """Six prompts through four slots with a small per-step budget (chunked prefill beside decodes); every generated
    id is the oracle's arg-max on the same history unless the oracle's two best logits are closer than the tolerance."""
    from trtllm_llama_b200.runtime import SamplingConfig
    cfg, t, model = _model(name, dtype, seed=4)
    prompts = [_tokens(n, cfg["vocab"], 40 + n) for n in (1, 9, 40, 17, 3, 26)]
    sess = _session(model, max_tokens=16 * 12, max_seqs=4, page=16)
    new = 12
    outs = sess.generate(prompts, new, SamplingConfig(end_id=None), max_step_tokens=24)
    assert not sess.live and len(sess.kv_cache_manager.free_blocks) == 12
    cfg, t = _weights(name, dtype, 4)
    for p, o in zip(prompts, outs):
        assert len(o) == new
        lg = O.mimolix_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[dtype] * float(lg.abs().max()), f"step {i}: id {tok} is not the arg-max"


def test_registry_and_trace_tool_end_to_end(tmp_path):
    """A checkpoint folder is recognised by its config.json, and bin/trace_run replays steps on it as a user runs it."""
    import subprocess
    import sys
    import numpy as np
    from trtllm_llama_b200 import models
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_mimolix(**STACKS["odd"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    assert "mimolix" in models.registered_models()
    toks = {"a": _tokens(40, cfg["vocab"], 1), "b": _tokens(9, cfg["vocab"], 2)}
    want = {k: O.mimolix_forward(cfg, t, v) for k, v in toks.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][30:31], "want": [0]}, {"id": "b", "tokens": toks["b"], "want": [8]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": toks["a"][31:], "want": []}], "end": []},
        {"step": 3, "entries": [], "end": ["a"]},
    ]
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path / "m"), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "128"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == ["done 0", "done 1", "done 2", "done 3"]
    got0 = torch.from_numpy(np.fromfile(tmp_path / "o" / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(tmp_path / "o" / "1.f32", dtype="<f4").reshape(2, -1))
    _close(got0, want["a"][[0, 29]], torch.float32, "trace step 0", scale=2.0)
    _close(got1, torch.stack([want["a"][30], want["b"][8]]), torch.float32, "trace step 1", scale=2.0)
    assert not os.path.exists(tmp_path / "o" / "2.f32")


def test_generation_example_from_the_command_line(tmp_path):
    """examples/inflight/run.py on a Mimolix folder: the registry picks the class, the scheduler runs the prompts, and the
    ids are the oracle's greedy continuation."""
    import csv
    import subprocess
    import sys
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_mimolix(**STACKS["plain"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    prompts = [_tokens(n, cfg["vocab"], 70 + n) for n in (5, 31)]
    with open(tmp_path / "in.csv", "w") as f:
        csv.writer(f).writerows(prompts)
    r = subprocess.run([sys.executable, os.path.join(root, "examples", "inflight", "run.py"), "--model_dir", str(tmp_path / "m"),
                        "--input_tokens", str(tmp_path / "in.csv"), "--max_output_len", "6", "--dtype", "float32",
                        "--output_csv", str(tmp_path / "out.csv"), "--max_step_tokens", "16"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    with open(tmp_path / "out.csv") as f:
        outs = [[int(x) for x in row] for row in csv.reader(f) if row]
    assert len(outs) == 2
    for p, o in zip(prompts, outs):
        o = o[-6:]
        lg = O.mimolix_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[torch.float32] * float(lg.abs().max()), f"step {i}: id {tok}"
