"""Host-side parts of the Mimolix design: the configuration reader and what it asks of the session (one cache pool or one
state — carried convolution inputs and a matrix per head — per layer RUN of a looped block), configuration errors, and
properties of the plain oracle that the GPU tests lean on (the temperature's steps, the two maps cancelling, the delta
rule's closed forms, the router's weights, the order of a looped block)."""
import math

import pytest
import torch

from oracle import mimolix_plain as O

ATT = dict(type="attention", heads=4, kv_heads=2, dim=8, vdim=6, diff=0.3, q_temp=(0.5, 4))
DLT = dict(type="delta", heads=4, kv_heads=2, dim=8, vdim=6, conv=3)
F64 = torch.float64


def _build(layers, **kw):
    from trtllm_llama_b200.models.mimolix import build_mimolix
    cfg, t = O.random_mimolix(layers, width=24, vocab=30, **kw)
    return cfg, t, build_mimolix(cfg, t, "float32", "cpu")


def test_layer_runs_pools_and_states_of_a_looped_block():
    layers = [dict(DLT, mlp=(16, 6, 2, 2.0, 12)), dict(ATT, kv_heads=4, mlp=None), dict(DLT, conv=1, mlp=(8, 4, 1, 1.0, None))]
    cfg, t, model = _build(layers, loop=(1, 3, 2))
    assert model.runs == [(0, 0, False), (1, 0, True), (2, 0, False), (1, 1, True), (2, 1, False)]
    assert model.runs == O.layer_runs(cfg)
    pools, states = model.cache_layers(), model.state_layers()
    assert set(pools) == {(1, 0), (1, 1)} and pools[(1, 0)] == 4 * (2 * 8 + 6)          # two key maps, one set of values
    assert set(states) == {(0, 0), (2, 0), (2, 1)}
    assert states[(0, 0)] == (3, 2 * 2 * 8 + 4 * 6, 4 * 6 * 8) and states[(2, 1)][0] == 1
    assert model.parallel and model.norm == "layer" and model.residual_mult == cfg["residual_mult"]
    assert tuple(model.loop_in.shape) == (24, 48) and model.embed_scale == cfg["embedding"]["scale"]
    mlp = model.layers[0]["mlp"]
    assert (mlp.experts, mlp.top, mlp.router, mlp.route_scale, mlp.gated) == (6, 2, "softmax", 2.0, False)
    assert tuple(mlp.w_up.shape) == (6, 16, 24) and mlp.shared is not None and model.layers[2]["mlp"].shared is None


def test_query_rows_are_grouped_by_key_head_and_map():
    """The stacked projection holds the query rows as [key/value head][map][head of the group]."""
    cfg, t, model = _build([dict(ATT, mlp=None)])
    mixer, w = model.layers[0]["mixer"], t["l0.mix.q"].float()
    per, d = 2, 8
    for g in range(2):
        for m in range(2):
            for hl in range(per):
                src = ((g * per + hl) * 2 + m) * d
                dst = ((g * 2 + m) * per + hl) * d
                assert torch.equal(mixer.w_in[dst:dst + d], w[src:src + d])
    assert torch.equal(mixer.w_in[4 * 2 * 8:4 * 2 * 8 + 2 * 2 * 8], t["l0.mix.k"].float())


def test_no_loop_no_feed_forward_no_temperature():
    cfg, t, model = _build([dict(ATT, q_temp=None, mlp=None)], loop=None)
    assert model.runs == [(0, 0, False)] and model.loop_in is None
    assert model.layers[0]["mixer"].temp_every == 0 and model.layers[0]["mlp"] is None


def test_configuration_errors():
    from trtllm_llama_b200.models.mimolix import build_mimolix
    cfg, t = O.random_mimolix([dict(ATT, mlp=None), dict(DLT, mlp=None)], width=24, vocab=30)
    bad = dict(cfg, layers=[dict(cfg["layers"][0], type="recurrent"), cfg["layers"][1]])
    with pytest.raises(ValueError):
        build_mimolix(bad, t, "float32", "cpu")
    for i in (0, 1):
        layers = list(cfg["layers"])
        layers[i] = dict(layers[i], mixer=dict(layers[i]["mixer"], kv_heads=3))
        with pytest.raises(ValueError):
            build_mimolix(dict(cfg, layers=layers), t, "float32", "cpu")
    with pytest.raises(KeyError):
        build_mimolix(cfg, {k: v for k, v in t.items() if k != "l1.mix.A_log"}, "float32", "cpu")
    with pytest.raises(ValueError):
        build_mimolix(dict(cfg, loop={"start": 0, "stop": 3, "times": 2}), t, "float32", "cpu")


def test_oracle_temperature_steps():
    assert O.query_temperature(0, 0.5, 4) == 1.0 and O.query_temperature(2, 0.5, 4) == 1.0
    assert abs(O.query_temperature(3, 0.5, 4) - (1 + 0.5 * math.log(2))) < 1e-15          # the first position with a whole block
    assert abs(O.query_temperature(6, 0.5, 4) - (1 + 0.5 * math.log(2))) < 1e-15
    assert abs(O.query_temperature(7, 0.5, 4) - (1 + 0.5 * math.log(3))) < 1e-15
    assert abs(O.query_temperature(0, 2.0, 1) - (1 + 2.0 * math.log(2))) < 1e-15


def test_oracle_equal_maps_cancel_up_to_lambda():
    """With both maps alike, o = (1 - lambda) a before the normalisation, so the normalised output is that of one plain
    attention; with lambda = 1 the difference is zero and the output vanishes."""
    g = torch.Generator().manual_seed(0)
    T, d, dv = 7, 4, 6
    h = torch.randn(T, 10, generator=g, dtype=F64)
    wq, wk = torch.randn(d, 10, generator=g, dtype=F64), torch.randn(d, 10, generator=g, dtype=F64)
    P = {"q": torch.cat([wq, wq]), "k": torch.cat([wk, wk]), "v": torch.randn(dv, 10, generator=g, dtype=F64),
         "q.norm": torch.ones(d, dtype=F64), "k.norm": torch.ones(d, dtype=F64), "o": torch.eye(dv, dtype=F64),
         "lq1": torch.zeros(d, dtype=F64), "lk1": torch.zeros(d, dtype=F64), "lq2": torch.zeros(d, dtype=F64), "lk2": torch.zeros(d, dtype=F64)}
    mc = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "scale": 0.5, "diff": 0.25}
    assert abs(O.differential_lambda(P, "", 0.25) - 0.25) < 1e-15
    out = O.differential_attention_mixer(h, P, "", mc, 1e-12)
    a = O.causal_softmax_attention(O.rms(h @ wq.T, 1e-12), O.rms(h @ wk.T, 1e-12), h @ P["v"].T, 0.5)
    assert (out - O.rms(a, 1e-12) * 0.75).abs().max() < 1e-9
    out = O.differential_attention_mixer(h, P, "", dict(mc, diff=1.0), 1e-12)
    assert out.abs().max() < 1e-9


def test_oracle_delta_rule_closed_forms():
    """beta = 1, no decay, orthonormal keys: the state stores every value exactly and a query along key j reads value j; a
    second write along the same key replaces the first; the read-out sees the current token's write."""
    d, dv = 4, 3
    k = torch.eye(d, dtype=F64)
    v = torch.arange(12, dtype=F64).view(4, 3) + 1
    ones = torch.ones(4, dtype=F64)
    out = O.delta_rule(k, k, v, ones, ones)
    assert (out - v).abs().max() < 1e-12                              # position t reads its own write
    q = k[[0, 0, 0, 0]]
    out = O.delta_rule(q, k, v, ones, ones)
    assert (out - v[[0, 0, 0, 0]]).abs().max() < 1e-12                # value 0 stays retrievable
    k2 = k[[0, 1, 0, 2]]
    out = O.delta_rule(q, k2, v, ones, ones)
    assert (out[3] - v[2]).abs().max() < 1e-12                        # rewritten at position 2
    out = O.delta_rule(q, k, v, ones, torch.full((4,), 0.5, dtype=F64))
    assert (out[3] - v[0] * 0.125).abs().max() < 1e-12                # decayed three times after its write
    out = O.delta_rule(q, k2, v, torch.full((4,), 0.5, dtype=F64), ones)
    assert (out[2] - (0.5 * v[0] + 0.5 * (v[2] - 0.5 * v[0]))).abs().max() < 1e-12


def test_oracle_router_weights():
    P = {"router": torch.eye(5, dtype=F64)}
    h = torch.tensor([[2.0, 0.0, 3.0, -1.0, 2.5]], dtype=F64)
    (ids, ws), = O.route(h, P, "", {"experts": 5, "top": 2, "scale": 3.0})
    assert ids == [2, 4]
    e = [math.exp(3.0), math.exp(2.5)]
    assert abs(ws[0] - 3.0 * e[0] / sum(e)) < 1e-12 and abs(sum(ws) - 3.0) < 1e-12
    (ids, ws), = O.route(h, P, "", {"experts": 5, "top": 1, "scale": 0.5})
    assert ids == [2] and abs(ws[0] - 0.5) < 1e-12


def test_oracle_loop_rereads_the_embedding():
    """A token change at position j reaches only positions >= j, and the re-projection before each pass matters."""
    layers = [dict(DLT, mlp=None), dict(ATT, mlp=(8, 4, 2, 1.0, 8))]
    cfg, t = O.random_mimolix(layers, width=24, vocab=30, loop=(0, 2, 2), seed=1)
    toks = list(range(12))
    base, runs = O.mimolix_forward(cfg, t, toks, return_layers=True)
    assert len(runs) == 4
    other = list(toks)
    other[5] = 29
    z = O.mimolix_forward(cfg, t, other)
    changed = [(z[i] - base[i]).abs().max().item() > 1e-9 for i in range(12)]
    assert changed == [i >= 5 for i in range(12)]
    t2 = dict(t)
    t2["loop.in"] = torch.cat([t["loop.in"][:, :24], torch.zeros(24, 24, dtype=t["loop.in"].dtype)], dim=1)
    assert (O.mimolix_forward(cfg, t2, toks) - base).abs().max() > 1e-3
