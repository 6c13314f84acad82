"""Host-side parts of the Duzizen design: the configuration reader and what it asks of the session (one cache pool, carried
convolution inputs and a retention state for a pair of mixers side by side; a matrix memory's state with its normaliser
column and running maxima), the previous token carried with a sequence, configuration errors, and properties of the plain
oracle that the GPU tests lean on (the mask's edges, the sink, the running maximum, closed forms of the retention, the
router's score on the expert's input, the pair embedding's rows)."""
import math

import pytest
import torch

from oracle import duzizen_plain as O

ATT = dict(heads=4, kv_heads=2, dim=8, conv=3, scale=0.4, window=5, keep_first=2, rot_dims=4, scaling=(4.0, 1.0, 4.0, 16))
RET = dict(heads=2, dim=6, vdim=4, decay=[0.9, 0.99], rot_dims=6)
MEM = dict(type="mlstm", heads=2, dim=6, vdim=5, gate_cap=7.0)
F64 = torch.float64


def _build(layers, **kw):
    from trtllm_llama_b200.models.duzizen import build_duzizen
    args = dict(width=24, vocab=30)
    args.update(kw)
    cfg, t = O.random_duzizen(layers, **args)
    return cfg, t, build_duzizen(cfg, t, "float32", "cpu")


def test_pools_states_and_mechanisms_of_a_stack():
    layers = [dict(type="parallel", left=ATT, right=RET, mlp=("dense", 20)), dict(MEM, mlp=("moe", 8, 6, 2, 1.25)),
              dict(type="parallel", left=dict(ATT, conv=0, window=0), right=dict(RET, rot_dims=0), mlp=None)]
    cfg, t, model = _build(layers, side_dim=3, bigram=(11, 5, 3))
    assert model.runs == [(0, 0, False), (1, 0, False), (2, 0, False)] and not model.parallel and model.norm == "layer"
    pools, states = model.cache_layers(), model.state_layers()
    assert pools == {(0, 0): 2 * (8 + 8), (2, 0): 2 * (8 + 8)}                       # keys and the values that are the keys
    assert states[(0, 0)] == (3, (4 + 2) * 8, 2 * 4 * 6)                             # carried q | k inputs; the retention's S
    assert states[(1, 0)] == (1, 0, 2 * (5 + 1) * 6 + 2)                             # [S | n] per head, then the running maxima
    assert states[(2, 0)] == (1, 0, 2 * 4 * 6)                                       # no convolution: only the retention's S
    left, right = model.layers[0]["mixer"].left, model.layers[0]["mixer"].right
    assert (left.window, left.keep_first, left.tied, left.taps, left.rot_dims) == (5, 2, True, 3, 4)
    assert left.rot_scaling == (4.0, 1.0, 4.0, 16.0) and left.sink is not None and float(left.sink.abs().max()) == 0.0
    assert abs(right.k_scale - 6 ** -0.5) < 1e-12 and right.decay.tolist() == pytest.approx([0.9, 0.99])
    assert model.layers[2]["mixer"].left.conv_w is None and model.layers[2]["mixer"].left.window == 0
    mem = model.layers[1]["mixer"]
    assert (mem.gate_cap, mem.den_eps, mem.state_cols) == (7.0, 1e-6, 2 * 6 * 6)
    mlp = model.layers[1]["mlp"]
    assert (mlp.experts, mlp.top, mlp.on_input, mlp.g_alpha, mlp.g_limit, mlp.g_shift) == (6, 2, True, 1.702, 1.25, 1.0)
    assert model.layers[2]["mlp"] is None and model.layers[2]["pre2"] is None
    assert [l["side"].offset for l in model.layers] == [0, 3, 6]
    assert model.embed_pair[1:] == (5, 3) and model.embed_pair[0].shape[0] == 12


def test_optional_pieces_may_be_absent():
    cfg, t, model = _build([dict(MEM, mlp=None)], side_dim=0, bigram=None)
    assert model.embed_pair is None and model.layers[0]["side"] is None and "token_side" not in cfg


def test_configuration_errors():
    from trtllm_llama_b200.models.duzizen import build_duzizen
    cfg, t = O.random_duzizen([dict(type="parallel", left=ATT, right=RET, mlp=None), dict(MEM, mlp=("dense", 8))], width=24, vocab=30)
    with pytest.raises(ValueError):
        build_duzizen(dict(cfg, layers=[dict(cfg["layers"][0], type="recurrent"), cfg["layers"][1]]), t, "float32", "cpu")
    bad = dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], left=dict(cfg["layers"][0]["mixer"]["left"], kv_heads=3)))
    with pytest.raises(ValueError):
        build_duzizen(dict(cfg, layers=[bad, cfg["layers"][1]]), t, "float32", "cpu")
    bad = dict(cfg["layers"][0], mixer=dict(cfg["layers"][0]["mixer"], right=dict(cfg["layers"][0]["mixer"]["right"], decay=[0.5])))
    with pytest.raises(ValueError):
        build_duzizen(dict(cfg, layers=[bad, cfg["layers"][1]]), t, "float32", "cpu")
    with pytest.raises(KeyError):
        build_duzizen(cfg, {k: v for k, v in t.items() if k != "l1.mix.i.b"}, "float32", "cpu")
    with pytest.raises(ValueError):
        build_duzizen(dict(cfg, layers=[cfg["layers"][0], dict(cfg["layers"][1], mlp={"kind": "sparse"})]), t, "float32", "cpu")
    with pytest.raises(ValueError):
        build_duzizen(dict(cfg, embedding={"bigram": {"buckets": 5, "mul_prev": 1, "mul_cur": 1}}), t, "float32", "cpu")


def test_the_batch_carries_the_token_before_every_row():
    from trtllm_llama_b200.inflight import RaggedBatch
    b = RaggedBatch([([7, 8, 9], 0, 0, [0], 55), ([4], 6, 1, [1], 3), ([5, 6], 2, 2, [2])], [], "cpu")
    assert b.tok_prev.tolist() == [-1, 7, 8, 3, -1, 5]          # position 0 has none; a batch built without one says so
    assert b.tok_ids.tolist() == [7, 8, 9, 4, 5, 6] and b.tok_pos.tolist() == [0, 1, 2, 6, 2, 3]


def test_oracle_pair_rows():
    assert O.bigram_rows([3, 4, 3], 7, 5, 2) == [7, (3 * 5 + 4 * 2) % 7, (4 * 5 + 3 * 2) % 7]


def test_oracle_mask_edges_and_sink():
    """A query sees its window and the kept first tokens, nothing between; one score of 0 always shares the denominator."""
    T, d = 12, 4
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(T, d, generator=g, dtype=F64), torch.randn(T, d, generator=g, dtype=F64)
    v = torch.eye(T, dtype=F64)                                  # the output row lists the weights themselves
    w = O.window_attention_with_sink(q, k, v, 0.7, 4, 2)
    for i in range(T):
        seen = [j for j in range(T) if w[i, j] > 0]
        assert seen == [j for j in range(i + 1) if i - j < 4 or j < 2]
        s = torch.tensor([float(k[j] @ q[i]) * 0.7 for j in seen], dtype=F64)
        assert torch.allclose(w[i, seen], torch.exp(s) / (1.0 + torch.exp(s).sum()))
        assert float(w[i].sum()) < 1.0
    full = O.window_attention_with_sink(q, k, v, 0.7, 0, 0)
    assert all(int((full[i] > 0).sum()) == i + 1 for i in range(T))


def test_oracle_retention_closed_form():
    T, d, dv = 9, 3, 2
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, n, generator=g, dtype=F64) for n in (d, d, dv))
    o = O.retention(q, k, v, 0.8)
    for t in range(T):
        want = sum(0.8 ** (t - s) * float(q[t] @ k[s]) * v[s] for s in range(t + 1))
        assert torch.allclose(o[t], want)


def test_oracle_matrix_memory_maximum_starts_at_zero():
    """With strongly negative gates the maximum stays at its start, 0, and the read-out is divided by at least exp(0) = 1."""
    T, d, dv = 5, 3, 2
    g = torch.Generator().manual_seed(2)
    q, k, v = (torch.randn(T, n, generator=g, dtype=F64) for n in (d, d, dv))
    ig, fg = torch.full((T,), -9.0, dtype=F64), torch.full((T,), -0.1, dtype=F64)
    o = O.mlstm(q, k, v, ig, fg)
    S = torch.zeros(d, dv, dtype=F64)
    for t in range(T):
        S = math.exp(-0.1) * S + math.exp(-9.0) * torch.outer(k[t], v[t])       # m stays 0: the weights are the gates themselves
        assert torch.allclose(o[t], (S.T @ q[t]) / (1.0 + 1e-6))
    # a large input gate lifts the maximum: the newest token's weight becomes exp(0)
    ig[3] = 6.0
    o = O.mlstm(q, k, v, ig, fg)
    n3 = k[3] + math.exp(-6.0) * sum(math.exp(-0.1 * (3 - s) - 9.0) * k[s] for s in range(3))
    S3 = torch.outer(k[3], v[3]) + math.exp(-6.0) * sum(math.exp(-0.1 * (3 - s) - 9.0) * torch.outer(k[s], v[s]) for s in range(3))
    assert torch.allclose(o[3], (S3.T @ q[3]) / (max(abs(float(n3 @ q[3])), math.exp(-6.0)) + 1e-6))


def test_oracle_router_score_weighs_the_input():
    g = torch.Generator().manual_seed(3)
    W, ff, E = 8, 5, 4
    P = {"router": torch.randn(E, W, generator=g, dtype=F64)}
    for e in range(E):
        P.update({f"e{e}.gate": torch.randn(ff, W, generator=g, dtype=F64), f"e{e}.up": torch.randn(ff, W, generator=g, dtype=F64),
                  f"e{e}.down": torch.randn(W, ff, generator=g, dtype=F64)})
    h = torch.randn(6, W, generator=g, dtype=F64)
    fc = {"expert": {"ff": ff, "limit": 0.7}, "router": {"experts": E, "top": 2}}
    ids, w = O.route(h, P, "", fc["router"])
    s = torch.sigmoid(h @ P["router"].T)
    for t in range(6):
        assert ids[t].tolist() == s[t].argsort(descending=True)[:2].tolist() and torch.equal(w[t], s[t, ids[t]])
        want = sum(O.clamped_expert(s[t, e] * h[t], P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], 0.7) for e in ids[t].tolist())
        assert torch.allclose(O.moe_mlp(h, P, "", fc)[t], want)
    y = O.clamped_expert(h, P["e0.gate"], P["e0.up"], P["e0.down"], 0.7)
    gte, up = torch.clamp(h @ P["e0.gate"].T, max=0.7), torch.clamp(h @ P["e0.up"].T, -0.7, 0.7)
    assert torch.allclose(y, (gte * torch.sigmoid(1.702 * gte) * (up + 1)) @ P["e0.down"].T)


def test_oracle_is_causal_and_reads_the_previous_token():
    layers = [dict(type="parallel", left=ATT, right=RET, mlp=("dense", 12)), dict(MEM, mlp=("moe", 8, 4, 1, 2.0))]
    cfg, t = O.random_duzizen(layers, width=24, vocab=30, dtype=torch.float32)
    toks = [3, 9, 1, 22, 7, 7, 15, 4, 28, 11]
    z = O.duzizen_forward(cfg, t, toks)
    changed = list(toks)
    changed[6] = 2
    z2 = O.duzizen_forward(cfg, t, changed)
    assert torch.equal(z[:6], z2[:6]) and not torch.allclose(z[6], z2[6])
    # the pair embedding alone tells position 1's token from the same token behind another one
    P = {k: v.double() for k, v in t.items()}
    a, b = O.embed([3, 9], P, cfg)[1], O.embed([4, 9], P, cfg)[1]
    assert not torch.allclose(a, b)
