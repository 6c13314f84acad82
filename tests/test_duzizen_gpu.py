"""The Duzizen design (token + hashed pair embedding; layer norms around every sublayer; an mLSTM matrix memory; a sliding-window
attention that keeps the first tokens, beside a retention; gated GELU and clamped experts whose score weighs their input; a
per-layer token input) on the GPU against the plain float64 oracle (oracle/duzizen_plain.py): every mechanism alone, prefill
against token-by-token decoding, portions down to two tokens, unequal batches against each request alone, pages and slots
used again, keys far away, at page borders and just inside / outside the window and the kept first tokens, the first tokens
of a sequence, long decoding, other sizes, and greedy generation through the scheduler."""
import json
import math
import os

import pytest
import torch

from oracle import duzizen_plain as O

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 2e-4, torch.bfloat16: 4e-2}      # relative to the largest magnitude of the compared tensor


def _close(got, want, dtype, what, scale=1.0):
    got, want = got.double().cpu(), want.double().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} against {tuple(want.shape)}"
    err = (got - want).abs().max().item()
    ref = max(want.abs().max().item(), 1e-6)
    assert err <= TOL[dtype] * scale * ref, f"{what}: max error {err:.3e} against magnitude {ref:.3e}"


ML_ODD = dict(type="mlstm", heads=3, dim=10, vdim=7, gate_cap=6.0)
ML_BIG = dict(type="mlstm", heads=2, dim=64, vdim=40, gate_cap=12.0)
ML_WIDE = dict(type="mlstm", heads=1, dim=130, vdim=33, gate_cap=8.0)          # dim neither a power of two nor a multiple of 8
AT_ODD = dict(heads=6, kv_heads=2, dim=10, conv=3, scale=0.4, window=7, keep_first=3, rot_dims=6, rot_base=100.0, scaling=(4.0, 1.0, 4.0, 24))
AT_MQ = dict(heads=5, kv_heads=1, dim=8, conv=2, scale=0.5, window=20, keep_first=1, rot_dims=8)               # group of 5 > 4 warps
AT_TC = dict(heads=8, kv_heads=2, dim=32, conv=4, scale=0.25, window=40, keep_first=5, rot_dims=16, rot_base=5000.0, scaling=(8.0, 1.0, 4.0, 64))
AT_ALL = dict(heads=2, kv_heads=2, dim=16, scale=0.3)                                                        # no window, no convolution, no rotation
RT_ODD = dict(heads=3, dim=10, vdim=7, decay=[0.9, 0.99, 0.5], rot_dims=6, rot_base=50.0)
RT_BIG = dict(heads=4, dim=32, vdim=64, decay=[0.9375, 0.984375, 0.998046875, 0.75], rot_dims=32, rot_base=2e5)
RT_ONE = dict(heads=1, dim=48, vdim=24, decay=[0.995])                                                       # no rotation
STACKS = {
    "odd": dict(layers=[dict(type="parallel", left=AT_ODD, right=RT_ODD, mlp=("dense", 20)), dict(ML_ODD, mlp=("moe", 12, 5, 2, 1.2)),
                        dict(type="parallel", left=AT_MQ, right=RT_ONE, mlp=None), dict(ML_WIDE, mlp=("moe", 9, 3, 3, 2.5))],
                width=40, vocab=61, side_dim=3, bigram=(13, 5, 3)),
    "tc": dict(layers=[dict(ML_BIG, mlp=("moe", 32, 8, 1, 1.25)), dict(type="parallel", left=AT_TC, right=RT_BIG, mlp=("moe", 16, 6, 2, 2.0)),
                       dict(type="parallel", left=dict(AT_TC, dim=64, kv_heads=8, window=33, keep_first=0), right=RT_BIG, mlp=("dense", 96))],
               width=64, vocab=130, side_dim=8, bigram=(31, 113, 11)),
    "plain": dict(layers=[dict(type="parallel", left=AT_ALL, right=RT_ONE, mlp=("dense", 24)), dict(ML_ODD, heads=1, mlp=None)],
                  width=32, vocab=40, side_dim=0, bigram=None, eps=1e-6),
}

_ORACLE = {}


def _weights(name, dtype, seed):
    """Whole stacks run in bf16 get routers whose ranking cannot hang on rounding (``spaced_router``): with random routers
    some token's two best scores lie within bf16 rounding of each other, another expert runs for it, and everything that
    reads that token differs — which is no kernel's error.  Likewise their matrix memories get queries that never stand
    orthogonal to the normaliser (``steady_memory``), and their token inputs are at least 12 wide: the input's RMS norm follows a
    projection from that few numbers, and with three of them some token's are all near zero, where the normalised direction
    turns on rounding.  The fp32 runs keep random weights and the narrow token input."""
    bf16 = dtype == torch.bfloat16
    spec = dict(STACKS[name])
    if bf16 and spec["side_dim"]:
        spec["side_dim"] = max(spec["side_dim"], 12)
    return O.random_duzizen(seed=seed, spaced_router=bf16, steady_memory=bf16, **spec)


def _oracle(name, dtype, seed, toks, layers=False):
    key = (name, dtype == torch.bfloat16, seed, tuple(toks))
    if key not in _ORACLE:
        cfg, t = _weights(name, dtype, seed)
        _ORACLE[key] = O.duzizen_forward(cfg, t, toks, return_layers=True)
    return _ORACLE[key] if layers else _ORACLE[key][0]


def _model(name, dtype, seed=0):
    from trtllm_llama_b200.models.duzizen import build_duzizen
    cfg, t = _weights(name, dtype, seed)
    return cfg, t, build_duzizen(cfg, t, dtype, "cuda")


def _session(model, max_tokens=512, max_seqs=4, page=64):
    from trtllm_llama_b200.inflight import InflightSession
    return InflightSession(model, max_tokens, max_seqs, page)


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _batch(lens, pasts=None, slots=None, prev=None):
    from trtllm_llama_b200.inflight import RaggedBatch
    pasts = pasts or [0] * len(lens)
    return RaggedBatch([([0] * n, pasts[i], slots[i] if slots else i, [0], prev[i] if prev else -1) for i, n in enumerate(lens)], [], "cuda")


# ---------------------------------------------------------------------------------------------------------------
# operators alone
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_embedding_reads_the_previous_token(dtype):
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    g = torch.Generator().manual_seed(1)
    vocab, width, buckets, mp, mc = 50, 24, 11, 89, 5
    emb, pair = torch.randn(vocab, width, generator=g).to(dtype), torch.randn(buckets + 1, width, generator=g).to(dtype)
    toks = _tokens(9, vocab, 2)
    P = {"embed": emb.double(), "bigram": pair.double()}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    want = O.embed(toks, P, cfg)
    # the sequence cut in three: the first row of a later portion reads the token the batch carries for it
    b = RaggedBatch([(toks[:4], 0, 0, [0], -1), (toks[4:5], 4, 1, [0], toks[3]), (toks[5:], 5, 2, [0], toks[4])], [], "cuda")
    got = ops.embed_bigram(emb.cuda(), pair.cuda(), b.tok_ids, b.tok_prev, 1.0, mp, mc)
    _close(got, want, torch.float32, "token + pair embedding")
    assert torch.equal(got[0].cpu(), (emb[toks[0]].float() + pair[buckets].float())), "a first token reads the table's last row"
    # a portion that starts at position 0 ignores whatever token is handed in for it
    b0 = RaggedBatch([(toks[:2], 0, 0, [0], 17)], [], "cuda")
    _close(ops.embed_bigram(emb.cuda(), pair.cuda(), b0.tok_ids, b0.tok_prev, 1.0, mp, mc), want[:2], torch.float32, "position 0")


@pytest.mark.parametrize("cols", [24, 72, 300, 1030])
def test_residual_step_between_two_layer_norms(cols):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(cols)
    x, y = torch.randn(11, cols, generator=g) * 3 + 5.0, torch.randn(11, cols, generator=g) * 2 - 4.0   # means far from zero
    w = [(torch.randn(cols, generator=g) * 0.2 + 1).to(torch.bfloat16) for _ in range(2)]
    b = [(torch.randn(cols, generator=g) * 0.3).to(torch.bfloat16) for _ in range(2)]
    new = x.double() + 0.7 * O.layer_norm(y.double(), w[0].double(), b[0].double(), 1e-5)
    xs = x.clone().cuda()
    h = ops.residual_sandwich_layernorm_rows(xs, y.cuda(), w[0].cuda(), b[0].cuda(), 0.7, 1e-5, w[1].cuda(), b[1].cuda())
    _close(xs, new, torch.float32, "residual step")
    _close(h, O.layer_norm(new, w[1].double(), b[1].double(), 1e-5), torch.float32, "next sublayer's norm from the same kernel")
    xs = x.clone().cuda()
    assert ops.residual_sandwich_layernorm_rows(xs, y.cuda(), w[0].cuda(), None, 1.0, 1e-5) is None
    _close(xs, x.double() + O.layer_norm(y.double(), w[0].double(), 0.0, 1e-5), torch.float32, "residual step alone, no bias")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [5, 45], ids=["one-kernel", "products-as-projections"])
@pytest.mark.parametrize("width,sd,layer,nl", [(40, 3, 1, 4), (64, 16, 0, 1), (300, 1, 2, 3), (1030, 7, 5, 6), (256, 72, 1, 2), (512, 16, 0, 2)])
def test_token_side_input(dtype, width, sd, layer, nl, n):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(width + sd)
    vocab = 37
    toks = _tokens(n, vocab, 3)
    t = {"side.embed": torch.randn(vocab, nl * sd, generator=g), f"l{layer}.side.gate": torch.randn(sd, width, generator=g) * width ** -0.5,
         f"l{layer}.side.proj": torch.randn(width, sd, generator=g), f"l{layer}.side.norm": torch.randn(width, generator=g) * 0.2 + 0.7}
    t = {k: v.to(dtype) for k, v in t.items()}
    P = {k: v.double() for k, v in t.items()}
    x = (torch.randn(n, width, generator=g) * 2).to(dtype).float()          # exactly representable: the gate product rounds its operand
    cfg = {"token_side": {"dim": sd}, "norm": {"eps": 1e-5}}
    new = x.double() + O.token_side(x.double(), toks, P, layer, cfg)
    w, b = (torch.randn(width, generator=g) * 0.2 + 1).to(dtype), (torch.randn(width, generator=g) * 0.3).to(dtype)
    ids = torch.tensor(toks, dtype=torch.int32).cuda()
    args = [t["side.embed"].cuda(), layer * sd, ids, t[f"l{layer}.side.gate"].cuda(), t[f"l{layer}.side.proj"].cuda(), t[f"l{layer}.side.norm"].cuda(), 1e-5]
    xs = x.clone().cuda()
    assert ops.token_side_input(xs, *args) is None
    _close(xs - x.cuda(), new - x.double(), dtype, "token input", scale=0.5)
    xs = x.clone().cuda()
    h = ops.token_side_input(xs, *args, w_pre=w.cuda(), b_pre=b.cuda())
    _close(h, O.layer_norm(new, w.double(), b.double(), 1e-5), dtype, "next layer's layer norm from the same kernel", scale=0.5)
    xs = x.clone().cuda()
    h = ops.token_side_input(xs, *args, w_pre=w.cuda(), pre_rms=True)
    _close(h, O.rms(new, 1e-5) * w.double(), dtype, "next layer's RMS norm from the same kernel", scale=0.5)


@pytest.mark.parametrize("dims,dim,layout", [(6, 10, "half"), (32, 32, "half"), (4, 4, "interleaved"), (16, 64, "interleaved"), (0, 12, "half")])
def test_rotation_layouts(dims, dim, layout):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(dims + dim)
    n, H = 9, 3
    x = torch.randn(n, 2 * H * dim + 5, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 700, 701, 5, 64, 4095], dtype=torch.int32)
    fr = O.rotary_frequencies(dims, 1000.0) if dims else None
    xq = x[:, :2 * H * dim].double().view(n, 2 * H, dim)
    want = xq.clone()
    for r in range(n):          # the oracle rotates by the row index: feed it one row at a time at its position
        if dims:
            ang = float(pos[r]) * fr
            c, s = torch.cos(ang), torch.sin(ang)
            a, b = (xq[r, :, 0:dims:2], xq[r, :, 1:dims:2]) if layout == "interleaved" else (xq[r, :, :dims // 2], xq[r, :, dims // 2:dims])
            ra, rb = a * c - b * s, b * c + a * s
            if layout == "interleaved":
                want[r, :, 0:dims:2], want[r, :, 1:dims:2] = ra, rb
            else:
                want[r, :, :dims // 2], want[r, :, dims // 2:dims] = ra, rb
    want[:, H:] *= 0.25
    table = ops.rope_table(pos.cuda(), dims, 1000.0) if dims else None
    got = ops.rope_heads(x.cuda(), table, 2 * H, dim, dims, ops.ROPE_HALF if layout == "half" else ops.ROPE_INTERLEAVED, split=H, scale_hi=0.25)
    _close(got.view(n, 2 * H, dim), want, torch.float32, f"rotation {layout} {dims}/{dim}")
    if dims and layout == "half":       # the oracle's own rotation agrees with the loop above at consecutive positions
        seq = O.rotate(xq[:4], dims, fr, "half")
        _close(got.view(n, 2 * H, dim)[:4, :H], seq[:, :H], torch.float32, "rotation against the oracle's")


def _gates_plain(zi, zf, bi, bf, cap):
    """-> (ln a, ln b, m) [T, H] by the recurrence of the running maximum, row by row."""
    i = cap * torch.tanh((zi + bi) / cap) if cap > 0 else zi + bi
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((zf + bf) / cap) if cap > 0 else zf + bf)
    T, H = zi.shape
    la, lb, ms = torch.zeros(T, H, dtype=torch.float64), torch.zeros(T, H, dtype=torch.float64), torch.zeros(T, H, dtype=torch.float64)
    m = torch.zeros(H, dtype=torch.float64)
    for t in range(T):
        mn = torch.maximum(f[t] + m, i[t])
        la[t], lb[t], ms[t] = f[t] + m - mn, i[t] - mn, mn
        m = mn
    return la, lb, ms


@pytest.mark.parametrize("cap", [15.0, 2.0, 0.0])
@pytest.mark.parametrize("cuts", [[200], [1] * 5 + [31, 32, 33, 98], [2, 198], [255, 257, 1, 600]])
def test_matrix_memory_gates_and_running_maximum(cap, cuts):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(int(cap) + len(cuts))
    T, H = sum(cuts), 3
    proj = torch.randn(T, 2 * H + 4, generator=g) * 4.0
    proj[50:60, 2:2 + H] += 30.0            # a burst of large input gates: the maximum jumps, then decays with the forget gates
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g) + 2.0
    la, lb, ms = _gates_plain(proj[:, 2:2 + H].double(), proj[:, 2 + H:2 + 2 * H].double(), bi.double(), bf.double(), cap)
    state = torch.full((4, 7 + H), 123.0, device="cuda")         # the maxima sit behind 7 other state columns; slot 2 is used
    at, got = 0, []
    for n in cuts:
        b = _batch([n], [at], [2])
        got.append(ops.mlstm_gates(proj[at:at + n].cuda(), 2, 2 + H, bi.cuda(), bf.cuda(), cap, state[:, 7:], b, H))
        at += n
    log_ab, m = torch.cat([x[0] for x in got]), torch.cat([x[1] for x in got])
    _close(m, ms, torch.float32, "running maximum")
    _close(log_ab[..., 0], la, torch.float32, "log decay", scale=5.0)
    _close(log_ab[..., 1], lb, torch.float32, "log input weight")
    assert (log_ab <= 0).all(), "decay and input weight never exceed 1"
    _close(state[2, 7:], ms[-1], torch.float32, "carried maximum")
    assert (state[[0, 1, 3]] == 123.0).all() and (state[2, :7] == 123.0).all(), "other slots and columns are untouched"


def _scan_plain(q, k, v, la, lb):
    """q, k [T, H, d], v [T, H, dv], la / lb [T, H] -> o [T, H, dv] of S <- e^la S + e^lb k v^T, o = S^T q, and the last S."""
    T, H, d = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=torch.float64)
    S = torch.zeros(H, d, v.shape[2], dtype=torch.float64)
    for t in range(T):
        for h in range(H):
            S[h] = math.exp(la[t, h]) * S[h] + math.exp(lb[t, h]) * torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out, S


@pytest.mark.parametrize("rows_only", [False, True], ids=["chunks", "row-by-row"])
@pytest.mark.parametrize("cuts", [[300], [1] * 6 + [3, 4, 31, 32, 33, 191], [2, 298], [299, 1]])
@pytest.mark.parametrize("H,d,dv,ones", [(2, 10, 7, True), (1, 64, 40, True), (3, 48, 48, False), (2, 130, 33, True), (1, 32, 64, False),
                                         (2, 128, 20, False), (1, 256, 9, True), (1, 300, 5, False)])
def test_decayed_linear_attention_remembers_far_tokens(H, d, dv, ones, cuts, rows_only, monkeypatch):
    """Decays near 1 with a few strong early tokens: the first rows still decide the read-out 300 rows later.  Cut anywhere — also
    inside a block of 32 rows and down to single rows — the result is the row-by-row recurrence's; the state of the neighbouring
    slots is not touched."""
    from trtllm_llama_b200 import ops
    monkeypatch.setattr(ops, "FORCE_ROW_SCAN", rows_only)
    g = torch.Generator().manual_seed(H * 1000 + d + dv)
    T = sum(cuts)
    q, k = torch.randn(T, H, d, generator=g) * d ** -0.5, torch.randn(T, H, d, generator=g)
    v = torch.randn(T, H, dv, generator=g)
    v[3:6] *= 30.0
    la = -torch.rand(T, H, generator=g) * 0.01
    lb = -torch.rand(T, H, generator=g) * 2.0
    vv = torch.cat([v, torch.ones(T, H, 1)], dim=2) if ones else v
    want, S = _scan_plain(q.double(), k.double(), vv.double(), la.double(), lb.double())
    vc = dv + (1 if ones else 0)
    state = torch.full((3, H * vc * d + 2), -7.0, device="cuda")
    log_ab = torch.stack([la, lb], dim=-1).cuda()
    at, outs = 0, []
    for n in cuts:
        b = _batch([n], [at], [1])
        outs.append(ops.decay_attention_scan(q[at:at + n].reshape(n, -1).cuda(), k[at:at + n].reshape(n, -1).cuda(), v[at:at + n].reshape(n, -1).cuda(),
                                             state, b, H, d, dv, log_ab=log_ab[at:at + n].contiguous(), ones_col=ones))
        at += n
    _close(torch.cat(outs), want, torch.float32, "read-out", scale=2.0)
    _close(state[1, :H * vc * d].view(H, vc, d), S.transpose(1, 2), torch.float32, "carried state", scale=2.0)
    assert (state[[0, 2]] == -7.0).all() and (state[1, H * vc * d:] == -7.0).all(), "neighbouring slots and columns are untouched"
    far = _scan_plain(q.double()[6:], k.double()[6:], vv.double()[6:], la.double()[6:], lb.double()[6:])[0]
    assert (want[-1] - far[-1]).abs().max() > 0.1 * want[-1].abs().max(), "the test's early rows must matter at the end"


@pytest.mark.parametrize("H,d,dv,ones", [(2, 16, 12, True), (1, 64, 70, False), (3, 48, 48, True)])
@pytest.mark.parametrize("lens,pasts", [([900], [0]), ([700, 130, 1, 64], [0, 40, 7, 0]), ([128, 129], [5, 0])])
def test_long_portions_run_as_segments_side_by_side(H, d, dv, ones, lens, pasts):
    """Portions long enough to be cut into segments (each segment's own end state, the carry in order, then every segment from its
    carried state) beside short ones in one batch, sequences that start from a state in their slot and sequences that start from
    zero: the read-out and the state left behind are the row-by-row recurrence's."""
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(sum(lens) + d)
    vc = dv + (1 if ones else 0)
    assert ops._rl.tb_decay_scan_segments(len(lens), H, vc, max(lens)) > 1
    N = sum(lens)
    q, k, v = torch.randn(N, H, d, generator=g) * d ** -0.5, torch.randn(N, H, d, generator=g), torch.randn(N, H, dv, generator=g)
    la, lb = -torch.rand(N, H, generator=g) * 0.02, -torch.rand(N, H, generator=g)
    state0 = torch.randn(len(lens) + 1, H * vc * d + 3, generator=g)
    state = state0.clone().cuda()
    b = _batch(lens, pasts, list(range(1, len(lens) + 1)))
    out = ops.decay_attention_scan(q.reshape(N, -1).cuda(), k.reshape(N, -1).cuda(), v.reshape(N, -1).cuda(), state, b, H, d, dv,
                                   log_ab=torch.stack([la, lb], dim=-1).cuda(), ones_col=ones)
    at = 0
    for i, n in enumerate(lens):
        S = state0[i + 1, :H * vc * d].double().view(H, vc, d).transpose(1, 2).clone() if pasts[i] else torch.zeros(H, d, vc, dtype=torch.float64)
        vv = torch.cat([v[at:at + n], torch.ones(n, H, 1)], dim=2) if ones else v[at:at + n]
        want = torch.zeros(n, H, vc, dtype=torch.float64)
        for t in range(n):
            for h in range(H):
                S[h] = math.exp(la[at + t, h]) * S[h] + math.exp(lb[at + t, h]) * torch.outer(k[at + t, h].double(), vv[t, h].double())
                want[t, h] = S[h].T @ q[at + t, h].double()
        _close(out[at:at + n], want, torch.float32, f"read-out of sequence {i}", scale=2.0)
        _close(state[i + 1, :H * vc * d].view(H, vc, d), S.transpose(1, 2), torch.float32, f"state of sequence {i}", scale=2.0)
        at += n
    assert torch.equal(state[0].cpu(), state0[0]) and torch.equal(state[1:, H * vc * d:].cpu(), state0[1:, H * vc * d:])


@pytest.mark.parametrize("cuts", [[150], [70, 1, 1, 78]])
def test_fixed_decay_per_head_is_the_retention(cuts):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(7)
    T, H, d, dv = sum(cuts), 3, 16, 12
    q, k, v = torch.randn(T, H, d, generator=g) * 0.3, torch.randn(T, H, d, generator=g), torch.randn(T, H, dv, generator=g)
    decay = [0.5, 0.9375, 0.998046875]
    want = torch.stack([O.retention(q[:, h].double(), k[:, h].double(), v[:, h].double(), decay[h]) for h in range(H)], dim=1)
    state = torch.zeros((2, H * dv * d), device="cuda") + 5.0
    at, outs = 0, []
    for n in cuts:
        b = _batch([n], [at], [0])
        outs.append(ops.decay_attention_scan(q[at:at + n].reshape(n, -1).cuda(), k[at:at + n].reshape(n, -1).cuda(), v[at:at + n].reshape(n, -1).cuda(),
                                             state, b, H, d, dv, head_decay=torch.tensor(decay).cuda()))
        at += n
    _close(torch.cat(outs), want, torch.float32, "retention")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dv,per_head,act,den", [(3, 7, True, "sigmoid", True), (2, 64, False, "silu", False), (1, 40, True, "silu", True),
                                                   (4, 33, False, "sigmoid", False)])
def test_head_norm_and_gate(dtype, H, dv, per_head, act, den):
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(H + dv)
    n = 19
    vc = dv + (1 if den else 0)
    o = torch.randn(n, H, vc, generator=g) * 3
    if den:
        o[::2, :, dv] *= 1e-3                     # |n . q| below exp(-m): the other branch of the maximum
    m = torch.randn(n, H, generator=g)
    gate = torch.randn(n, H * dv + 3, generator=g)
    w = (torch.randn(H * dv if per_head else dv, generator=g) * 0.2 + 1).to(dtype)
    x = o[..., :dv].double()
    if den:
        x = x / (torch.maximum(o[..., dv].double().abs(), torch.exp(-m.double())) + 1e-6)[..., None]
    x = O.rms(x, 1e-5) * (w.double().view(H, dv) if per_head else w.double())
    gl = gate[:, :H * dv].double().view(n, H, dv)
    want = x * (torch.sigmoid(gl) if act == "sigmoid" else O.silu(gl))
    got = ops.head_norm_gate(o.cuda(), dv, 1e-5, dtype, w=w.cuda(), w_per_head=per_head, gate=gate.cuda(), gate_act=act,
                             m=m.cuda() if den else None)
    _close(got, want, dtype, "head norm and gate", scale=0.5)
    got = ops.head_norm_gate(o.cuda(), dv, 1e-5, torch.float32, m=m.cuda() if den else None)
    _close(got, O.rms(x / (w.double().view(H, dv) if per_head else w.double()), 1e-5), torch.float32, "no weight, no gate")


@pytest.mark.parametrize("dtype,tiles", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)],
                         ids=["fp32-fma-tiles", "bf16-streaming-or-tcgen05", "bf16-warp-mma-tiles"])
@pytest.mark.parametrize("top", [1, 3])
@pytest.mark.parametrize("n", [1, 5, 40, 150, 700])
def test_experts_whose_score_weighs_their_input(dtype, n, top, tiles, monkeypatch):
    """Every form of the expert products (fp32 FMA tiles, bf16 warp-MMA tiles, one streaming product per pair, tcgen05 tiles over a
    plan) with the clamps and the score in front of the activation.  Scores near 0.5 and a small limit: weighing the OUTPUT
    instead would be far off."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.layers import RoutedExpertsMLP
    monkeypatch.setattr(ops, "FORCE_TILE_LINEAR", tiles)
    g = torch.Generator().manual_seed(n + top)
    W, ff, E, limit = 64, 24, 6, 0.8
    fc = {"expert": {"ff": ff, "limit": limit}, "router": {"experts": E, "top": top}}
    t = {"router": torch.randn(E, W, generator=g) * 0.2}
    for e in range(E):
        t.update({f"e{e}.gate": torch.randn(ff, W, generator=g) * 3 * W ** -0.5, f"e{e}.up": torch.randn(ff, W, generator=g) * 3 * W ** -0.5,
                  f"e{e}.down": torch.randn(W, ff, generator=g) * ff ** -0.5})
    t = {k: v.to(dtype) for k, v in t.items()}
    h = torch.randn(n, W, generator=g).to(dtype)
    P = {k: v.double() for k, v in t.items()}
    want = O.moe_mlp(h.double(), P, "", fc)
    ex = range(E)
    mlp = RoutedExpertsMLP(w_router=t["router"].cuda(), w_gate=torch.stack([t[f"e{j}.gate"] for j in ex]).cuda(),
                           w_up=torch.stack([t[f"e{j}.up"] for j in ex]).cuda(), w_down=torch.stack([t[f"e{j}.down"] for j in ex]).cuda(),
                           top=top, router="sigmoid_groups", groups=1, keep=1, gate_alpha=1.702, gate_limit=limit, gate_up_shift=1.0,
                           weight_on="input")
    got = mlp.forward(h.cuda(), None)
    ids, w = O.route(h.double(), P, "", fc["router"])
    if dtype == torch.bfloat16:       # a close call of the router in reduced precision is no product kernel's error: compare the others
        s = torch.sigmoid(h.double() @ P["router"].T).sort(dim=-1, descending=True).values
        sure = (s[:, top - 1] - s[:, top]) > 2e-2 if top < E else torch.ones(n, dtype=torch.bool)
        got, want = got[sure.cuda()], want[sure]
        if not sure.any():
            return
    _close(got, want, dtype, f"{n} tokens, top {top}", scale=1.5)
    on_output = torch.zeros_like(want)                    # what weighing the expert's OUTPUT would give: the test must tell the two apart
    for r in range(min(n, 8)):
        for j, e in enumerate(ids[r].tolist()):
            on_output[r] += w[r, j] * O.clamped_expert(h[r].double(), P[f"e{e}.gate"], P[f"e{e}.up"], P[f"e{e}.down"], limit)
    assert (want[:8] - on_output[:8]).abs().max() > 0.05 * want[:8].abs().max() or dtype == torch.bfloat16


@pytest.mark.parametrize("top", [1, 2, 4])
def test_router_choice_where_the_sigmoid_saturates(top):
    """Logits of 17 and more all have the score 1 in fp32; the largest LOGITS are still the ones chosen (in their order), their weights
    are the rounded scores, and small or negative logits are ranked as before."""
    from trtllm_llama_b200 import ops
    g = torch.Generator().manual_seed(top)
    n, E = 37, 9
    z = torch.stack([torch.randperm(E, generator=g).float() * 1.5 + 16.0 for _ in range(n)])
    z[1::3] -= 24.0                                          # rows in the ordinary range, rows far below it
    z[2::3] -= 60.0
    ids, w = ops.moe_route(z.cuda(), None, top, 1, 1)
    want = z.double().topk(top, dim=-1)
    assert torch.equal(ids.cpu().long(), want.indices)
    assert torch.allclose(w.cpu().double(), torch.sigmoid(want.values), rtol=3e-6, atol=1e-30)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [3, 50])
def test_gated_gelu_feed_forward(dtype, n):
    from trtllm_llama_b200.layers import ClampedGatedMLP
    g = torch.Generator().manual_seed(n)
    W, ff = 48, 40
    t = {"gate": torch.randn(ff, W, generator=g) * 2 * W ** -0.5, "up": torch.randn(ff, W, generator=g) * 2 * W ** -0.5,
         "down": torch.randn(W, ff, generator=g) * ff ** -0.5}
    t = {k: v.to(dtype) for k, v in t.items()}
    h = torch.randn(n, W, generator=g).to(dtype)
    mlp = ClampedGatedMLP(w_gate=t["gate"].cuda(), w_up=t["up"].cuda(), w_down=t["down"].cuda(), gate="gelu_tanh")
    _close(mlp.forward(h.cuda(), None), O.gated_gelu_mlp(h.double(), {k: v.double() for k, v in t.items()}, ""), dtype, "gated GELU")


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


def _mixer_alone(dtype, layer, lens, what, fn, pre, sub=None):
    from trtllm_llama_b200.models.duzizen import build_duzizen
    cfg, t = O.random_duzizen([dict(layer, mlp=None)], width=40, seed=3, side_dim=0, bigram=None)
    model = build_duzizen(cfg, t, dtype, "cuda")
    sess, ctx = _mixer_ctx(model, lens)
    h = torch.randn(sum(lens), 40, generator=torch.Generator().manual_seed(4))
    from trtllm_llama_b200 import ops
    mixer = model.layers[0]["mixer"]
    if sub:           # one of two mixers side by side: its rows of the pair's stacked input projection
        proj = ops.linear(h.to(dtype).cuda(), mixer.w_in, out_dtype=torch.float32)
        got = getattr(mixer, sub).forward(h.to(dtype).cuda(), ctx, proj=proj[:, :mixer.split] if sub == "left" else proj[:, mixer.split:])
    else:
        got = mixer.forward(h.to(dtype).cuda(), ctx)
    P, at = {k: v.double() for k, v in t.items()}, 0
    mc = cfg["layers"][0]["mixer"]
    for n in lens:
        want = fn(h[at:at + n].to(dtype).double(), P, pre, mc[sub] if sub else mc, cfg["norm"]["eps"])
        _close(got[at:at + n], want, dtype, f"{what}, sequence of {n}")
        at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [ML_ODD, ML_BIG, ML_WIDE, dict(ML_BIG, dim=128, vdim=16, heads=1), dict(ML_ODD, dim=48, vdim=40, heads=2)],
                         ids=["odd", "big", "dim130", "dim128", "dim48"])
def test_matrix_memory_alone(dtype, spec):
    _mixer_alone(dtype, spec, [45, 5, 1, 70], "matrix memory", O.mlstm_mixer, "l0.mix.")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [RT_ODD, RT_BIG, RT_ONE], ids=["odd", "big", "one-head-no-rotation"])
def test_retention_alone(dtype, spec):
    _mixer_alone(dtype, dict(type="parallel", left=AT_ALL, right=spec), [45, 5, 1, 70], "retention", O.retention_mixer, "l0.mix.right.", sub="right")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("spec", [AT_ODD, AT_MQ, AT_TC, AT_ALL, dict(AT_TC, dim=64, kv_heads=4, window=16, keep_first=16),
                                  dict(AT_TC, dim=128, heads=2, kv_heads=2, window=70, keep_first=2, conv=0)],
                         ids=["odd", "one-kv-head", "tc", "no-window", "tc-64", "tc-128-no-conv"])
def test_window_attention_with_tied_values_alone(dtype, spec):
    _mixer_alone(dtype, dict(type="parallel", left=spec, right=RT_ONE), [75, 5, 1, 90], "window attention", O.tied_window_mixer, "l0.mix.left.",
                 sub="left")


@pytest.mark.parametrize("dtype", DTYPES)
def test_side_by_side_mixers(dtype):
    _mixer_alone(dtype, dict(type="parallel", left=AT_ODD, right=RT_ODD), [60, 3, 1], "two mixers side by side", O.parallel_mixer, "l0.mix.")


def _window_ops(q, k, scale, window, keep, cuts, dtype, page, blocks, sink=True):
    """q [P, H, d], k [P, G, d] as they reach the cache (values = keys) -> the attention kernel over the pages, the prompt cut as ``cuts``."""
    from trtllm_llama_b200 import ops
    from trtllm_llama_b200.inflight import RaggedBatch
    P, H, d = q.shape
    G = k.shape[1]
    proj = torch.cat([q.reshape(P, -1), k.reshape(P, -1)], dim=1).float().cuda()
    pool = torch.full((len(blocks) * page, 2 * G * d), float("nan"), dtype=dtype, device="cuda")
    zeros = torch.zeros(H, device="cuda")
    at, outs = 0, []
    for n in cuts:
        b = RaggedBatch([([0] * n, at, 0, blocks)], [], "cuda")
        qq = ops.qk_conv_norm_rope_append(proj[at:at + n], None, None, None, 1e-5, None, None, 0, pool, b, page, H, G, d, d, True)
        outs.append(ops.window_attention(qq, pool, b, page, G, d, scale, window, sink=zeros if sink else None, keep_first=keep))
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [8, 64], ids=["simt", "tensor-cores"])
@pytest.mark.parametrize("where", ["prompt", "decoded"])
@pytest.mark.parametrize("key", ["w-1", "w", "w+1", "first-last-kept", "first-not-kept", "0", "self", 15, 16, 17, 33, 64])
def test_one_key_stands_out_at_the_windows_edges(dtype, d, where, key):
    """ONE key decides the softmax: query and key are large along one direction, the key's value (the key itself) is far from
    the others.  The key sits just inside the window, just outside it, among the kept first tokens, right behind them, or at
    page borders (pages of 16) — in a prompt, and with the last tokens decoded one by one.  Outside the mask the row must
    look as if that key were not there."""
    page, P, H, G, window, keep = 16, 300, 4, 2, 80, 3
    g = torch.Generator().manual_seed(sum(map(ord, str(key))))
    q, k = torch.randn(P, H, d, generator=g) * 0.3, torch.randn(P, G, d, generator=g) * 0.3
    qi = P - 1 if where == "decoded" else P - 4
    kj = {"w-1": qi - (window - 1), "w": qi - window, "w+1": qi - window - 1, "first-last-kept": keep - 1, "first-not-kept": keep, "0": 0,
          "self": qi}.get(key)
    kj = qi - key if kj is None else kj
    seen = qi - kj < window or kj < keep
    k[:, :, 0] *= 0.03                       # no other key points along the query's direction
    q[qi] = 0.01
    q[qi, :, 0] = 6.0
    k[kj] = 0.01
    k[kj, :, 0] = 6.0
    k[kj, :, 1] = 9.0                        # the value is the key: its second element tells whether it was read
    cuts = [P] if where == "prompt" else [P - 8] + [1] * 8
    blocks = torch.randperm(-(-P // page), generator=g).tolist()          # every page id lies inside the pool
    got = _window_ops(q.to(dtype), k.to(dtype), 1.0, window, keep, cuts, dtype, page, blocks)[qi]
    qd, kd = q.to(dtype).double(), k.to(dtype).double()
    want = torch.stack([O.window_attention_with_sink(qd[:, h], kd[:, h // (H // G)], kd[:, h // (H // G)], 1.0, window, keep)[qi] for h in range(H)])
    _close(got, want, dtype, f"key {kj} for query {qi}")
    if seen:
        assert (got[:, 1].float() > 8.0).all(), "the one key carries the row"
    else:
        assert (got[:, 1].float().abs() < 1.0).all(), "a key outside the mask must not be read"


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_sink_takes_its_share(dtype):
    """Scores far below 0: the sink's term of the denominator (score 0, no value) takes nearly everything, also for the very first
    token of a sequence, whose only key is itself."""
    g = torch.Generator().manual_seed(3)
    P, H, G, d = 40, 2, 1, 8
    q, k = torch.randn(P, H, d, generator=g) * 0.3, torch.randn(P, G, d, generator=g) * 0.3
    q[:, :, 0], k[:, :, 0] = 4.0, -2.0                      # q . k = -8 + a little
    qd, kd = q.to(dtype).double(), k.to(dtype).double()
    got = _window_ops(q.to(dtype), k.to(dtype), 1.0, 8, 2, [1, 2, 37], dtype, 16, [2, 0, 1])
    want = torch.stack([O.window_attention_with_sink(qd[:, h], kd[:, 0], kd[:, 0], 1.0, 8, 2) for h in range(H)], dim=1)
    _close(got, want, dtype, "attention under a dominant sink", scale=0.5)
    assert got.float().abs().max() < 0.2 * kd.abs().max(), "without the sink the rows would be averages of the keys"


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
        _close(g_, w_, dtype, f"{name}: residual stream after layer {i}", scale=2.0)
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
    """180 generated tokens: the window passes over decoded tokens and leaves the kept ones behind, the block table outgrows its
    captured width and the recurrent states are carried 180 times; replayed graphs and eager launches give the same answer."""
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
        lg = O.duzizen_forward(cfg, t, p + o[:-1])[len(p) - 1:]
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
    cfg, t = O.random_duzizen(**STACKS["odd"])
    os.makedirs(tmp_path / "m")
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), t)
    assert "duzizen" in models.registered_models()
    toks = {"a": _tokens(40, cfg["vocab"], 1), "b": _tokens(9, cfg["vocab"], 2)}
    want = {k: O.duzizen_forward(cfg, t, v) for k, v in toks.items()}
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
    """examples/inflight/run.py on a Duzizen folder: the registry picks the class, the scheduler runs the prompts, and the
    ids are the oracle's greedy continuation."""
    import csv
    import subprocess
    import sys
    from trtllm_llama_b200.checkpoint import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg, t = O.random_duzizen(**STACKS["plain"])
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
        lg = O.duzizen_forward(cfg, t, p + o[:-1])[len(p) - 1:]
        for i, tok in enumerate(o):
            best = lg[i].topk(2)
            if int(best.indices[0]) != tok:
                assert float(best.values[0] - lg[i][tok]) <= 2 * TOL[torch.float32] * float(lg.abs().max()), f"step {i}: id {tok}"
