"""Torch-tensor front end of the C ABI (include/trtllm_b200.h).

PyTorch is used for device memory and streams only; every function below launches the hand-written
sm_100a kernels in ``libtrtllm_llama_b200.so`` through ctypes and raises if the call is rejected.
Names follow the reference's functional layer (T/tensorrt_llm/quantization/functional.py:12-212,
T/tensorrt_llm/functional.py:2695-2928) so call sites read like the reference's.
"""
from __future__ import annotations

import torch

from ._lib import check, lib

KIND_F16, KIND_W8, KIND_W4, KIND_A8W8 = 0, 1, 2, 3
_OUT_TYPES = {torch.float16: 0, torch.float32: 1, torch.int32: 2}


def _p(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _chk_cuda(*ts):
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("expected contiguous CUDA tensors")


_ws_cache = {}
_cnt_cache = {}


def _counters(device) -> torch.Tensor:
    """zeroed once; split-K / split-L arrival counters reset themselves after every launch."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    cur = _cnt_cache.get(key)
    if cur is None:
        cur = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        _cnt_cache[key] = cur
    return cur


def _workspace(nbytes: int, device) -> torch.Tensor:
    """scratch for split-K / split-L partials (contents need not be initialised)."""
    key = (device.index if device.index is not None else torch.cuda.current_device())
    cur = _ws_cache.get(key)
    if cur is None or cur.numel() < nbytes:
        cur = torch.empty(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
        _ws_cache[key] = cur
    return cur


# ------------------------------------------------------------------------------------------------
def rms_norm(x, weight, eps=1e-6, residual=None, return_sum=False):
    """T/tensorrt_llm/functional.py:3195-3219 rms_norm (+ fused residual add)."""
    _chk_cuda(x, weight, residual)
    rows, hidden = x.numel() // x.shape[-1], x.shape[-1]
    out = torch.empty_like(x)
    s = torch.empty_like(x) if (residual is not None and return_sum) else None
    check(lib.tb_rmsnorm(_p(out), _p(x), _p(residual), _p(s), _p(weight), eps, rows, hidden, _stream()), "tb_rmsnorm")
    return (out, s) if return_sum else out


def smooth_quant_rms_norm(x, weight, scale=None, eps=1e-6, dynamic_act_scaling=True, residual=None,
                          return_sum=False, bias=None, layernorm=False):
    """RmsnormQuantization plugin op (modelled on smooth_quant_layer_norm,
    T/tensorrt_llm/quantization/functional.py:77-129): returns int8 (and per-token scales if dynamic)."""
    _chk_cuda(x, weight, residual, scale, bias)
    rows, hidden = x.numel() // x.shape[-1], x.shape[-1]
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    ds = torch.empty(x.shape[:-1] + (1,), dtype=torch.float32, device=x.device) if dynamic_act_scaling else None
    s = torch.empty_like(x) if (residual is not None and return_sum) else None
    check(lib.tb_rmsnorm_quant(_p(q), _p(ds), _p(x), _p(residual), _p(s), _p(weight), _p(bias), _p(scale), eps, rows,
                               hidden, int(dynamic_act_scaling), int(layernorm), _stream()), "tb_rmsnorm_quant")
    res = (q, ds) if dynamic_act_scaling else (q,)
    return res + ((s,) if return_sum else ())


def quantize_per_token(x):
    """T/tensorrt_llm/quantization/functional.py:160-186."""
    _chk_cuda(x)
    rows, cols = x.numel() // x.shape[-1], x.shape[-1]
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(x.shape[:-1] + (1,), dtype=torch.float32, device=x.device)
    check(lib.tb_quantize_per_token(_p(q), _p(s), _p(x), rows, cols, int(x.dtype == torch.float32), _stream()),
          "tb_quantize_per_token")
    return q, s


def quantize_tensor(x, scale):
    """T/tensorrt_llm/quantization/functional.py:188-212."""
    _chk_cuda(x, scale)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    check(lib.tb_quantize_tensor(_p(q), _p(x), x.numel(), _p(scale), int(x.dtype == torch.float32), _stream()),
          "tb_quantize_tensor")
    return q


# ------------------------------------------------------------------------------------------------
PRO_NONE, PRO_RMS, PRO_RMS_QUANT, PRO_QUANT = 0, 1, 2, 3


def gemv(kind, x, w, *, w_scale=None, sc=None, sr=None, residual=None, swiglu=False, out_fp32=False, prologue=0,
         gamma=None, eps=1e-6):
    _chk_cuda(x, w, w_scale, sc, sr, residual, gamma)
    M, K = x.numel() // x.shape[-1], x.shape[-1]
    N = w.shape[0]
    n_out = N // 2 if swiglu else N
    if out_fp32:
        y32 = torch.empty(x.shape[:-1] + (n_out,), dtype=torch.float32, device=x.device)
        y = None
    else:
        y = torch.empty(x.shape[:-1] + (n_out,), dtype=torch.float16, device=x.device)
        y32 = None
    check(lib.tb_gemv_fused(kind, _p(y), _p(y32), _p(x), _p(w), _p(w_scale), _p(sc), _p(sr),
                            int(sc is not None and sc.numel() > 1), int(sr is not None and sr.numel() > 1), _p(residual),
                            M, N, K, int(swiglu), int(prologue), _p(gamma), float(eps), _stream()), "tb_gemv_fused")
    return y32 if out_fp32 else y


def gemm_tc(kind, x, w, *, w_scale=None, sc=None, sr=None, residual=None, out_dtype=torch.float16, force_splits=0,
            force_nt=0):
    _chk_cuda(x, w, w_scale, sc, sr, residual)
    M, K = x.numel() // x.shape[-1], x.shape[-1]
    N = w.shape[0]
    c = torch.empty(x.shape[:-1] + (N,), dtype=out_dtype, device=x.device)
    need = lib.tb_gemm_tc_workspace_bytes(M, N, K) * (4 if force_splits else 1) + (1 << 20)
    if force_splits:
        need = max(need, 4096 + ((N + 127) // 128) * ((M + 15) // 16) * force_splits * 256 * 128 * 4)
    ws = _workspace(need, x.device)
    check(lib.tb_gemm_tc(kind, _p(c), _OUT_TYPES[out_dtype], _p(x), _p(w), _p(w_scale), _p(sc), _p(sr),
                         int(sc is not None and sc.numel() > 1), int(sr is not None and sr.numel() > 1), _p(residual),
                         M, N, K, _p(ws), ws.numel(), _p(_counters(x.device)), force_splits, force_nt, _stream()),
          "tb_gemm_tc")
    return c


def smooth_quant_gemm(x_i8, w_i8, scale_tokens, scale_channels, per_token_scaling, per_channel_scaling,
                      out_dtype=torch.float16, use_gemv=None):
    """SmoothQuantGemm plugin op — T/tensorrt_llm/quantization/functional.py:12-53.
    x int8 [..., K], w int8 [N, K]; scales fp32 ([M,1]|[1,1], [1,N]|[1,1])."""
    M = x_i8.numel() // x_i8.shape[-1]
    if use_gemv is None:
        use_gemv = M <= lib.tb_gemv_max_rows(KIND_A8W8, x_i8.shape[-1]) and out_dtype == torch.float16
    if use_gemv:
        return gemv(KIND_A8W8, x_i8, w_i8, sc=scale_channels, sr=scale_tokens)
    return gemm_tc(KIND_A8W8, x_i8, w_i8, sc=scale_channels, sr=scale_tokens, out_dtype=out_dtype)


def weight_only_quant_matmul(x, w_processed, scales, weight_type_id, use_gemv=None):
    """WeightOnlyQuantMatmul plugin op — T/tensorrt_llm/quantization/functional.py:56-74.
    weight_type_id 1 = int8 ([N,K] processed), 2 = int4 ([N,K/2] processed)."""
    kind = KIND_W8 if weight_type_id == 1 else KIND_W4
    M = x.numel() // x.shape[-1]
    if use_gemv is None:
        use_gemv = M <= lib.tb_gemv_max_rows(kind, x.shape[-1])
    if use_gemv:
        return gemv(kind, x, w_processed, w_scale=scales)
    return gemm_tc(kind, x, w_processed, w_scale=scales)


def matmul_f16(x, w, residual=None, out_fp32=False, use_gemv=None):
    """Gemm plugin / TRT-native MatMul(x, W^T), W [N,K] (T/tensorrt_llm/layers/linear.py:13-35)."""
    M = x.numel() // x.shape[-1]
    if use_gemv is None:
        use_gemv = M <= lib.tb_gemv_max_rows(KIND_F16, x.shape[-1])
    if use_gemv:
        return gemv(KIND_F16, x, w, residual=residual, out_fp32=out_fp32)
    return gemm_tc(KIND_F16, x, w, residual=residual, out_dtype=torch.float32 if out_fp32 else torch.float16)


# ------------------------------------------------------------------------------------------------
def mmha_decode(qkv, kv_cache, past_len, *, num_heads, head_size, max_input_len, seq_lens=None, input_lengths=None,
                masked_tokens=None, kv_scale_orig_quant=None, kv_scale_quant_orig=None, q_scaling=1.0,
                rotary_dim=None, nsplit=0, len_cap=None, max_splits=32, max_input_len_dev=None):
    """GPTAttention plugin, generation phase (T/tensorrt_llm/functional.py:2695-2928 with
    past_key_value_length = [past_len, 0]).  kv_cache [B,2,H,S_max,Dh] is updated in place."""
    _chk_cuda(qkv, kv_cache, seq_lens, input_lengths, masked_tokens, kv_scale_orig_quant, kv_scale_quant_orig)
    B = qkv.shape[0]
    S_max = kv_cache.shape[3]
    int8_kv = kv_cache.dtype == torch.int8
    rot = head_size if rotary_dim is None else rotary_dim
    cap = past_len if len_cap is None else len_cap
    if nsplit <= 0:
        nsplit = lib.tb_mmha_num_splits(B, num_heads, cap, max_splits)
    ws = _workspace(lib.tb_mmha_workspace_bytes(B, num_heads, max(nsplit, max_splits)), qkv.device)
    out = torch.empty((B, num_heads * head_size), dtype=torch.float16, device=qkv.device)
    # max_input_len_dev: one device int that overrides max_input_len (what the engine's replayed step graph passes)
    check(lib.tb_mmha_decode_dev(_p(out), _p(qkv), _p(kv_cache), _p(seq_lens), _p(input_lengths), _p(masked_tokens),
                                 _p(max_input_len_dev), _p(kv_scale_orig_quant), _p(kv_scale_quant_orig), _p(ws), None, B,
                                 num_heads, head_size, S_max, int(past_len), int(max_input_len), int(cap), rot,
                                 float(q_scaling), int(int8_kv), nsplit, _stream()), "tb_mmha_decode")
    return out


def context_attention(qkv, kv_cache, input_lengths, *, num_heads, head_size, kv_scale_orig_quant=None, q_scaling=1.0,
                      rotary_dim=None, use_tc=True):
    """GPTAttention plugin, context phase (past_key_value_length = [0, 1]).  qkv [B,S,3*H*Dh] is
    rotated in place; kv_cache written for positions [0, S)."""
    _chk_cuda(qkv, kv_cache, input_lengths, kv_scale_orig_quant)
    B, S = qkv.shape[0], qkv.shape[1]
    rot = head_size if rotary_dim is None else rotary_dim
    out = torch.empty((B, S, num_heads * head_size), dtype=torch.float16, device=qkv.device)
    ws = _workspace(lib.tb_context_attention_workspace_bytes(B, S, num_heads), qkv.device) if use_tc else None
    check(lib.tb_context_attention(_p(out), _p(qkv), _p(kv_cache), _p(input_lengths), _p(kv_scale_orig_quant), _p(ws), B, S,
                                   num_heads, head_size, kv_cache.shape[3], rot, float(q_scaling),
                                   int(kv_cache.dtype == torch.int8), _stream()), "tb_context_attention")
    return out


def sample(logits, top_k=0, top_p=1.0, temperature=1.0, seed=0, step=0, finished=None, end_id=2, return_uniform=False):
    """DynamicDecodeOp's sampling for one step (T/cpp/tensorrt_llm/thop/dynamicDecodeOp.cpp:359-363): logits fp32 [B, V]
    -> ids int32 [B].  ``step`` may be a device int32 tensor (graph-replayable counter)."""
    _chk_cuda(logits, finished)
    B, V = logits.shape
    out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    u = torch.empty((B,), dtype=torch.float32, device=logits.device) if return_uniform else None
    step_dev = step if isinstance(step, torch.Tensor) else None
    check(lib.tb_sample(_p(out), _p(logits), B, V, logits.stride(0), int(top_k), float(top_p), float(temperature), int(seed),
                        _p(step_dev), 0 if step_dev is not None else int(step), _p(finished), int(end_id), _p(u), _stream()),
          "tb_sample")
    return (out, u) if return_uniform else out


# ------------------------------------------------------------------------------------------------
def embedding(ids, table):
    _chk_cuda(ids, table)
    out = torch.empty(ids.shape + (table.shape[1],), dtype=torch.float16, device=table.device)
    check(lib.tb_embedding(_p(out), _p(table), _p(ids), ids.numel(), table.shape[1], table.shape[0], _stream()),
          "tb_embedding")
    return out


def swiglu(gate_up):
    """gate_up [..., 2*inter] (gate | up) -> silu(gate) * up."""
    _chk_cuda(gate_up)
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // gate_up.shape[-1]
    out = torch.empty(gate_up.shape[:-1] + (inter,), dtype=torch.float16, device=gate_up.device)
    g = gate_up.view(rows, 2 * inter)
    check(lib.tb_swiglu(_p(out), g.data_ptr(), g.data_ptr() + inter * 2, rows, inter, 2 * inter, _stream()), "tb_swiglu")
    return out


def swiglu_quant(gate_up):
    """SwiGLU + per-token int8 quantisation in one pass: gate_up [..., 2*inter] -> (int8 [..., inter], fp32 scales [..., 1])."""
    _chk_cuda(gate_up)
    inter = gate_up.shape[-1] // 2
    rows = gate_up.numel() // gate_up.shape[-1]
    q = torch.empty(gate_up.shape[:-1] + (inter,), dtype=torch.int8, device=gate_up.device)
    sc = torch.empty(gate_up.shape[:-1] + (1,), dtype=torch.float32, device=gate_up.device)
    g = gate_up.view(rows, 2 * inter)
    check(lib.tb_swiglu_quant(_p(q), _p(sc), g.data_ptr(), g.data_ptr() + inter * 2, rows, inter, 2 * inter, _stream()),
          "tb_swiglu_quant")
    return q, sc


def add(a, b):
    _chk_cuda(a, b)
    out = torch.empty_like(a)
    check(lib.tb_add(_p(out), _p(a), _p(b), a.numel(), _stream()), "tb_add")
    return out


def argmax(logits):
    _chk_cuda(logits)
    rows, vocab = logits.numel() // logits.shape[-1], logits.shape[-1]
    out = torch.empty(logits.shape[:-1], dtype=torch.int32, device=logits.device)
    check(lib.tb_argmax(_p(out), _p(logits), rows, vocab, vocab, _stream()), "tb_argmax")
    return out


def mmha_decode_beams(qkv, kv_cache, cache_indirection, past_len, *, num_heads, head_size, max_input_len, input_lengths=None,
                      kv_scale_orig_quant=None, kv_scale_quant_orig=None, q_scaling=1.0, nsplit=0):
    """GPTAttention plugin, generation phase with beam search: cache_indirection [batch, beam, S_max] int32 names, per cached
    position, the beam whose cache row is read (T/tensorrt_llm/functional.py:2695-2928, input 7)."""
    _chk_cuda(qkv, kv_cache, cache_indirection, input_lengths, kv_scale_orig_quant, kv_scale_quant_orig)
    rows, S_max = qkv.shape[0], kv_cache.shape[3]
    beam = cache_indirection.shape[1]
    if nsplit <= 0:
        nsplit = lib.tb_mmha_num_splits(rows, num_heads, past_len, 32)
    out = torch.empty((rows, num_heads * head_size), dtype=torch.float16, device=qkv.device)
    check(lib.tb_mmha_decode_beams(_p(out), _p(qkv), _p(kv_cache), _p(cache_indirection), beam, None, _p(input_lengths), None,
                                   None, _p(kv_scale_orig_quant), _p(kv_scale_quant_orig), rows, num_heads, head_size, S_max,
                                   int(past_len), int(max_input_len), int(past_len), head_size, float(q_scaling),
                                   int(kv_cache.dtype == torch.int8), nsplit, _stream()), "tb_mmha_decode_beams")
    return out


class BeamSearchState:
    """Device-resident decoder state of tb_beam_search_step (the beam half of DynamicDecodeOp)."""

    def __init__(self, batch, beam_width, max_new, max_seq_len, max_input_len, device="cuda"):
        rows = batch * beam_width
        i32 = dict(dtype=torch.int32, device=device)
        self.rows, self.W, self.S_max = rows, beam_width, max_seq_len
        self.cum = torch.empty(rows, dtype=torch.float32, device=device)
        self.finished, self.lens, self.next_ids = (torch.empty(rows, **i32) for _ in range(3))
        self.ids_t, self.parent_t = (torch.zeros((max_new, rows), **i32) for _ in range(2))
        self.indir = [torch.empty((batch, beam_width, max_seq_len), **i32) for _ in range(2)]
        self.step = torch.zeros(1, **i32)
        self.max_in = torch.full((1,), max_input_len, **i32)
        self.ws = _workspace(lib.tb_beam_workspace_bytes(rows, beam_width), device)
        check(lib.tb_beam_init(_p(self.cum), _p(self.finished), _p(self.lens), _p(self.indir[0]), _p(self.indir[1]),
                               _p(self.max_in), rows, beam_width, max_seq_len, _stream()), "tb_beam_init")

    def advance(self, logits, end_id, length_penalty=1.0, broadcast=False):
        """logits fp32 [rows, V] ([batch, V] with broadcast) -> writes column ``step`` and the target indirection."""
        check(lib.tb_beam_search_step(_p(logits), logits.shape[1], logits.stride(0), int(broadcast), self.rows, self.W,
                                      float(length_penalty), int(end_id), _p(self.step), _p(self.max_in), _p(self.cum),
                                      _p(self.finished), _p(self.lens), _p(self.ids_t), _p(self.parent_t), _p(self.next_ids),
                                      _p(self.indir[0]), _p(self.indir[1]), self.S_max, _p(self.ws), _stream()),
              "tb_beam_search_step")
        self.indir[0].copy_(self.indir[1])
        self.step += 1

    def gather_tree(self, n, end_id):
        out = torch.empty((self.rows, n), dtype=torch.int32, device=self.cum.device)
        check(lib.tb_gather_tree(_p(out), _p(self.ids_t), _p(self.parent_t), self.rows, self.W, n, int(end_id), _stream()),
              "tb_gather_tree")
        return out


def gemm_tc_swiglu(kind, x, w_gate_up, *, sc=None, sr=None):
    """The gate / up projection with SwiGLU in the tcgen05 epilogue: w_gate_up [2*inter, K] (gate rows, then up rows) ->
    fp16 [..., inter] = silu(x.gate^T) * (x.up^T).  kind KIND_F16 or KIND_A8W8.  Bit-identical to gemm_tc + swiglu."""
    _chk_cuda(x, w_gate_up, sc, sr)
    M, K = x.numel() // x.shape[-1], x.shape[-1]
    N = w_gate_up.shape[0]
    c = torch.empty(x.shape[:-1] + (N // 2,), dtype=torch.float16, device=x.device)
    check(lib.tb_gemm_tc_swiglu(kind, _p(c), _p(x), _p(w_gate_up), _p(sc), _p(sr), int(sc is not None and sc.numel() > 1),
                                int(sr is not None and sr.numel() > 1), M, N, K, _stream()), "tb_gemm_tc_swiglu")
    return c


# ------------------------------------------------------------------------------------------------
# operators over a ragged in-flight batch (include/trtllm_b200_ragged.h).  They are served by whichever
# library holds them (the full one, or the ragged subset), so a model that needs only these does not need the rest.
# ------------------------------------------------------------------------------------------------
from ._lib import ragged_lib as _rl  # noqa: E402

DT_F32, DT_BF16 = 1, 2
ACT_NONE, ACT_GELU_TANH, ACT_RELU_SQUARED = 0, 1, 3
GATE_SIGMOID, GATE_GELU_TANH = 0, 1        # gated activations of a (gate, up) pair (TB_GATE_*)
ROPE_INTERLEAVED, ROPE_HALF = 0, 1         # which elements a rotation pairs (TB_ROPE_*)
COMPUTE_AUTO, COMPUTE_FMA32 = 0, 1
# rows from which a bf16 projection goes to the tcgen05 kernel; below, the streaming GEMV (<= 8 rows) or the warp-MMA tiles
TC_MIN_ROWS = 17
# A/B switches (tests and measurements): keep bf16 attention on the warp-per-head kernel / bf16 projections of few rows on
# the tile kernel instead of the streaming GEMV
FORCE_SIMT_ATTENTION = False
FORCE_TILE_LINEAR = False
FORCE_SERIAL_SCAN = False      # A/B: the delta rule row by row also for prompt portions
COMPUTE_TILES = 2


def _dt(t):
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"ragged operators take float32 or bfloat16 tensors, not {t.dtype}")


def _chk_dev(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("expected CUDA tensors (there is no CPU path)")


def linear(a, w, bias=None, out=None, out_dtype=None, act=ACT_NONE, compute=COMPUTE_AUTO):
    """out[b][m, n] = act(sum_k a[b][m, k] w[b][n, k] + bias[b][n]).

    ``w`` is [N, K] or, for a batch of independent products, [B, N, K]; ``a`` is then a [M, B, K] view (any row
    stride, unit stride on k) and ``out`` a [M, B, N] view of the caller's buffer.  Unbatched: a [M, K], out [M, N]."""
    _chk_dev(a, w, bias, out)
    batched = w.dim() == 3
    if not w.is_contiguous() or (bias is not None and not bias.is_contiguous()):
        raise ValueError("weights and biases must be contiguous")
    if batched:
        B, N, K = w.shape
        M = a.shape[0]
        if out is None:
            out = torch.empty((M, B, N), dtype=out_dtype or a.dtype, device=a.device)
        if a.shape != (M, B, K) or out.shape != (M, B, N) or a.stride(2) != 1 or out.stride(2) != 1:
            raise ValueError("batched linear: a [M, B, K], out [M, B, N] with unit inner stride")
        lda, a_bs, ldc, c_bs = a.stride(0), a.stride(1), out.stride(0), out.stride(1)
        w_bs, b_bs = N * K, N
    else:
        (N, K), B = w.shape, 1
        M = a.shape[0]
        if out is None:
            out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
        if a.shape != (M, K) or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1:
            raise ValueError("linear: a [M, K], out [M, N] with unit inner stride")
        lda, a_bs, ldc, c_bs, w_bs, b_bs = a.stride(0), 0, out.stride(0), 0, 0, 0
    if bias is not None and bias.dtype != w.dtype:
        raise TypeError("bias must have the weight's type")
    if (not batched and M >= TC_MIN_ROWS and compute == COMPUTE_AUTO and w.dtype == torch.bfloat16 and K % 8 == 0
            and out.stride(0) == N and out.dtype in (torch.float32, torch.bfloat16)):
        # prompt-sized bf16 products: the tcgen05 kernel.  fp32 rows (the residual stream) are rounded to bf16 once.
        if a.dtype != torch.bfloat16 or a.stride(0) != K:
            a = cast_rows_bf16(a)
        ws = _workspace(1 << 22, a.device)
        check(_rl.tb_gemm_tc_bf16(_p(out), 1 if out.dtype == torch.float32 else 3, _p(a), _p(w), _p(bias), act, M, N, K,
                                  _p(ws), ws.numel(), _p(_counters(a.device)), _stream()), "tb_gemm_tc_bf16")
        return out
    if FORCE_TILE_LINEAR and compute == COMPUTE_AUTO:
        compute = COMPUTE_TILES
    check(_rl.tb_linear(_p(out), _dt(out), ldc, c_bs, _p(a), _dt(a), lda, a_bs, _p(w), _dt(w), w_bs, _p(bias), b_bs,
                        M, N, K, B, act, compute, _stream()), "tb_linear")
    return out


def cast_rows_bf16(x):
    """fp32 [rows, cols] (any row stride) -> contiguous bf16."""
    _chk_dev(x)
    if x.dtype == torch.bfloat16:
        return x.contiguous()
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    check(_rl.tb_cast_rows_bf16(_p(out), _p(x), x.stride(0), x.shape[0], x.shape[1], _stream()), "tb_cast_rows_bf16")
    return out


def embed_bigram(table, pair, ids, prev_ids, scale, mul_prev, mul_cur):
    """table[ids] * scale + pair[(prev * mul_prev + id * mul_cur) mod buckets]; a token without a predecessor (prev < 0) reads
    the last row of ``pair`` ([buckets + 1, width])."""
    _chk_dev(table, pair, ids, prev_ids)
    if pair.dtype != table.dtype or pair.shape[1] != table.shape[1] or not pair.is_contiguous():
        raise ValueError("embed_bigram: the pair table has the embedding's type and width")
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    check(_rl.tb_embed_bigram(_p(out), _p(table), _p(pair), _dt(table), _p(ids), _p(prev_ids), float(scale), ids.numel(),
                              table.shape[1], table.shape[0], pair.shape[0] - 1, int(mul_prev), int(mul_cur), _stream()),
          "tb_embed_bigram")
    return out


def embed_scaled(table, ids, scale):
    _chk_dev(table, ids)
    out = torch.empty((ids.numel(), table.shape[1]), dtype=torch.float32, device=table.device)
    check(_rl.tb_embed_scaled(_p(out), _p(table), _dt(table), _p(ids), float(scale), ids.numel(), table.shape[1],
                              table.shape[0], _stream()), "tb_embed_scaled")
    return out


def rmsnorm_rows(x, w, eps, w_offset=0.0, out=None, out_dtype=None, accumulate=False, rows_idx=None, cols=None,
                 out_scale=1.0):
    """RMS norm of fp32 rows (``cols`` leading columns of each), times ``out_scale``; accumulate=True adds the result into
    fp32 ``out``."""
    _chk_dev(x, w, out, rows_idx)
    cols = x.shape[1] if cols is None else cols
    rows = x.shape[0] if rows_idx is None else rows_idx.numel()
    if x.dtype != torch.float32 or x.stride(1) != 1:
        raise ValueError("rmsnorm_rows normalises fp32 rows")
    if out is None:
        out = torch.empty((rows, cols), dtype=out_dtype or torch.float32, device=x.device)
    check(_rl.tb_rmsnorm_rows(_p(out), _dt(out), out.stride(0), _p(x), x.stride(0), _p(w), _dt(w) if w is not None else 0,
                              float(w_offset), float(eps), _p(rows_idx), rows, cols, int(accumulate), float(out_scale),
                              _stream()), "tb_rmsnorm_rows")
    return out


def linear_gated(a, w_gate_up, out_dtype, alpha, limit, up_shift, gate=GATE_SIGMOID):
    """gate‖up projection and the gated activation in one kernel when the step has few rows (streaming GEMV);
    returns None when the shape is not eligible — the caller then uses ``linear`` + ``gated_act``."""
    _chk_dev(a, w_gate_up)
    M, K, ff = a.shape[0], a.shape[1], w_gate_up.shape[0] // 2
    if FORCE_TILE_LINEAR or M > 8 or w_gate_up.dtype != torch.bfloat16 or a.stride(1) != 1:
        return None
    out = torch.empty((M, ff), dtype=out_dtype, device=a.device)
    rc = _rl.tb_linear_gated(_p(out), _dt(out), out.stride(0), _p(a), _dt(a), a.stride(0), _p(w_gate_up), _dt(w_gate_up),
                             M, ff, K, int(gate), float(alpha), float(limit), float(up_shift), _stream())
    if rc == -3:
        return None
    check(rc, "tb_linear_gated")
    return out


def gated_act(gu, out_dtype, alpha, limit, up_shift, gate=GATE_SIGMOID, row_scale=None, row_index=None):
    """Gated activation of fp32 [rows, 2 ff] (gate columns, then up columns).  ``row_scale`` (fp32): gate and up of row r are
    first multiplied by row_scale[row_index[r]] (row_index int32, negative: 0) or row_scale[r]."""
    _chk_cuda(gu, row_scale, row_index)
    rows, ff = gu.shape[0], gu.shape[1] // 2
    out = torch.empty((rows, ff), dtype=out_dtype, device=gu.device)
    check(_rl.tb_gated_act(_p(out), _dt(out), _p(gu), rows, ff, int(gate), float(alpha), float(limit), float(up_shift),
                           _p(row_scale), _p(row_index), _stream()), "tb_gated_act")
    return out


def rope_table(tok_pos, dims, base, scaling=None):
    """cos / sin per row and rotary pair; ``scaling`` = (factor, low, high, original) slows the long wavelengths."""
    _chk_dev(tok_pos)
    out = torch.empty((tok_pos.numel(), dims // 2, 2), dtype=torch.float32, device=tok_pos.device)
    factor, low, high, original = scaling or (0.0, 0.0, 0.0, 0.0)
    check(_rl.tb_rope_table_scaled(_p(out), _p(tok_pos), tok_pos.numel(), dims, float(base), float(factor), float(low),
                                   float(high), float(original), _stream()), "tb_rope_table_scaled")
    return out


def rope_query_tail(qa, q, table, heads, dim, rot_dim, dims, lat):
    _chk_cuda(qa, q, table)
    check(_rl.tb_rope_query_tail(_p(qa), _dt(qa), _p(q), _p(table), q.shape[0], heads, dim, rot_dim, dims, lat, _stream()),
          "tb_rope_query_tail")


def latent_kv_append(pool, kv, w, eps, table, dims, batch, page, lat, rot_dim):
    _chk_cuda(pool, kv, w, table)
    check(_rl.tb_latent_kv_append(_p(pool), _dt(pool), _p(kv), kv.stride(0), _p(w), _dt(w), float(eps), _p(table), dims,
                                  _p(batch.tok_seq), _p(batch.tok_pos), _p(batch.block_table), batch.max_blocks, page,
                                  kv.shape[0], lat, rot_dim, _stream()), "tb_latent_kv_append")


def latent_attention(qa, pool, batch, page, heads, lat, rot_dim, scale):
    """Causal multi-query attention of every row over its sequence's cache entries.  Steps with few rows and long
    contexts (decoding) deal each row's keys to several CTAs so that the whole chip reads the cache."""
    _chk_cuda(qa, pool)
    rows = qa.shape[0]
    out = torch.empty((rows, heads, lat), dtype=qa.dtype, device=qa.device)
    nsplit, ws = 1, None
    if FORCE_SIMT_ATTENTION:
        nsplit = -1
    elif _rl.tb_latent_attention_tensor_cores(_dt(pool), lat, rot_dim):
        ctas = rows * -(-heads // 16)
        nsplit = max(1, min(64, 296 // ctas, (batch.max_pos + 1) // 64))     # at least two key blocks per CTA
        if nsplit > 1:
            ws = torch.empty((rows * heads * nsplit * (lat + 2),), dtype=torch.float32, device=qa.device)
    check(_rl.tb_latent_attention(_p(out), _p(qa), _p(pool), _dt(pool), _p(batch.tok_seq), _p(batch.tok_pos),
                                  _p(batch.block_table), batch.max_blocks, page, rows, heads, lat, rot_dim,
                                  float(scale), nsplit, _p(ws), _stream()), "tb_latent_attention")
    return out


def causal_conv1d(x, w, bias, state, batch):
    """Ragged per-channel causal convolution; then the carried inputs in ``state`` move on by this step's rows."""
    _chk_cuda(x, w, bias, state)
    rows, ch = x.shape
    taps = w.shape[1]
    out = torch.empty_like(x)
    check(_rl.tb_causal_conv1d(_p(out), _p(x), _p(w), _p(bias), _dt(w), _p(state), _p(batch.tok_seq), _p(batch.tok_pos),
                               _p(batch.seq_start), _p(batch.seq_past), _p(batch.seq_slot), rows, ch, taps, _stream()),
          "tb_causal_conv1d")
    check(_rl.tb_causal_conv1d_update(_p(state), _p(x), x.stride(0), _p(batch.seq_start), _p(batch.seq_len), _p(batch.seq_past),
                                      _p(batch.seq_slot), batch.num_seqs, ch, taps, 0, _stream()), "tb_causal_conv1d_update")
    return out


def rglru_scan(u, gates, lam, y, state, batch, blocks, c):
    _chk_cuda(u, gates, lam, y, state)
    out = torch.empty_like(y)
    ws = None
    if batch.max_len > 32:          # long portions: parallel chunks of 32 rows, summaries carried in order
        ws = torch.empty((3 * batch.num_seqs * -(-batch.max_len // 32) * u.shape[1],), dtype=torch.float32, device=u.device)
    check(_rl.tb_rglru_scan(_p(out), _dt(out), _p(u), _p(gates), _p(lam), _dt(lam), _p(y), _p(state), _p(batch.seq_start),
                            _p(batch.seq_len), _p(batch.seq_past), _p(batch.seq_slot), batch.num_seqs, u.shape[1], blocks,
                            float(c), batch.max_len, _p(ws), _stream()), "tb_rglru_scan")
    return out


def residual_norm_rows(x, y, w_post, w_pre, eps, w_offset=0.0, out_scale=1.0, out_dtype=torch.float32):
    """x += out_scale * rmsnorm(y) * (w_post + w_offset) in place, and returns rmsnorm(x) * (w_pre + w_offset) — the
    post-norm residual update of one sublayer and the pre-norm input of the next in one kernel."""
    _chk_dev(x, y, w_post, w_pre)
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.stride(1) != 1 or y.stride(1) != 1 or w_post.dtype != w_pre.dtype:
        raise ValueError("residual_norm_rows: fp32 rows, norm weights of one type")
    h = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    check(_rl.tb_residual_norm_rows(_p(x), x.stride(0), _p(y), y.stride(0), _p(w_post), _p(w_pre), _dt(w_post), float(w_offset),
                                    float(eps), float(out_scale), _p(h), _dt(h), h.stride(0), x.shape[0], x.shape[1], _stream()),
          "tb_residual_norm_rows")
    return h


def add_row_vector(x, vec):
    """x[r, :] += vec, in place on the fp32 residual stream."""
    _chk_cuda(x, vec)
    check(_rl.tb_add_row_vector(_p(x), x.stride(0), _p(vec), _dt(vec), x.shape[0], x.shape[1], _stream()), "tb_add_row_vector")
    return x


def tanh_cap(x, cap):
    """x <- cap * tanh(x / cap) in place (contiguous fp32)."""
    _chk_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("tanh_cap works in place on contiguous fp32")
    check(_rl.tb_tanh_cap(_p(x), x.numel(), float(cap), _stream()), "tb_tanh_cap")
    return x


def qkv_conv_rope_append(proj, conv_w, state, table, dims, pool, batch, page, heads, kv_heads, dim, vdim):
    """Projected rows (fp32 [N, >= C], q | k | v) -> short causal convolution -> rotation of q and k -> queries
    [N, heads, dim] in the pool's type, keys and values into the pages; then the carried inputs move on."""
    _chk_dev(proj, conv_w, state, table, pool)
    rows, taps = proj.shape[0], conv_w.shape[1]
    C = heads * dim + kv_heads * (dim + vdim)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < C or conv_w.shape[0] != C or not conv_w.is_contiguous():
        raise ValueError("qkv_conv_rope_append: proj fp32 [N, >= C], conv_w [C, taps] contiguous")
    q = torch.empty((rows, heads, dim), dtype=pool.dtype, device=proj.device)
    check(_rl.tb_qkv_conv_rope_append(_p(q), _p(pool), _dt(pool), _p(proj), proj.stride(0), _p(conv_w), _dt(conv_w),
                                      _p(state), _p(table), dims, _p(batch.tok_seq), _p(batch.tok_pos), _p(batch.seq_start),
                                      _p(batch.seq_past), _p(batch.seq_slot), _p(batch.block_table), batch.max_blocks, page,
                                      rows, heads, kv_heads, dim, vdim, taps, _p(state) if taps > 1 else None,
                                      _p(batch.seq_len) if taps > 1 else None, _stream()), "tb_qkv_conv_rope_append")
    # sequences that bring one row were moved on by the kernel above; a generation step needs nothing more
    if taps > 1 and batch.max_len > 1:
        check(_rl.tb_causal_conv1d_update(_p(state), _p(proj), proj.stride(0), _p(batch.seq_start), _p(batch.seq_len),
                                          _p(batch.seq_past), _p(batch.seq_slot), batch.num_seqs, C, taps, 1, _stream()),
              "tb_causal_conv1d_update")
    return q


def window_attention(q, pool, batch, page, kv_heads, vdim, scale, window, sink=None, gate=None, v_share=1, out_f32=False,
                     keep_first=0):
    """Grouped-query attention of every row over the last ``window`` cached positions of its sequence (0: all), with an
    optional softmax sink per head and an optional per-head sigmoid gate (fp32 logits [N, >= heads], any row stride).
    ``v_share`` > 1: neighbouring key heads share a value head (key head g reads value head g // v_share; the pool entry
    holds kv_heads key heads and kv_heads // v_share value heads).  ``out_f32``: the result is fp32 in every storage mode.
    ``keep_first``: with a window, the first positions of a sequence that every later row still sees."""
    _chk_cuda(q, pool, sink)
    _chk_dev(gate)
    rows, heads, dim = q.shape
    out = torch.empty((rows, heads, vdim), dtype=torch.float32 if out_f32 else q.dtype, device=q.device)
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise ValueError("gate logits are fp32 with unit inner stride")
    nsplit, ws = 1, None
    if not FORCE_SIMT_ATTENTION and _rl.tb_window_attention_tensor_cores(_dt(pool), heads, kv_heads, dim, vdim):
        # few row blocks (generation steps): deal each block's key tiles to several CTAs so that the chip reads the cache
        ctas = -(-batch.max_len * (heads // kv_heads) // 64) * batch.num_seqs * kv_heads
        span = min(window + keep_first, batch.max_pos + 1) if window else batch.max_pos + 1
        nsplit = max(1, min(32, 296 // ctas, span // 64 + 1))
        if nsplit > 1:
            ws = torch.empty((rows * heads * nsplit * (vdim + 2),), dtype=torch.float32, device=q.device)
    check(_rl.tb_window_attention_shared_values(
        _p(out), int(out_f32), _p(q), _p(pool), _dt(pool), _p(gate), gate.stride(0) if gate is not None else 0, _p(sink),
        _dt(sink) if sink is not None else 0, _p(batch.tok_seq), _p(batch.tok_pos), _p(batch.block_table), _p(batch.seq_start),
        _p(batch.seq_len), _p(batch.seq_past), batch.num_seqs, batch.max_len, batch.max_blocks, page, rows, heads, kv_heads,
        int(v_share), dim, vdim, float(scale), int(window), int(keep_first) if window else 0, 1 if FORCE_SIMT_ATTENTION else 0,
        nsplit, _p(ws), _stream()),
        "tb_window_attention_shared_values")
    return out


def qk_conv_norm_rope_append(proj, conv_w, norm_q, norm_k, eps, state, table, dims, pool, batch, page, heads, kv_heads, dim, vdim,
                             tied_values):
    """Projected rows (fp32 [N, >= C], q | k [| v]) -> short causal convolution (``conv_w`` None: none) -> RMS norm of the whole
    q part and of the whole k part with a weight per channel (both None: none) -> rotation of q and k -> queries [N, heads, dim]
    in the pool's type, keys and values into the pages (``tied_values``: the values are the convolved keys before norm and
    rotation); then the carried inputs move on."""
    _chk_dev(proj, conv_w, norm_q, norm_k, state, table, pool)
    rows = proj.shape[0]
    taps = conv_w.shape[1] if conv_w is not None else 1
    C = (heads + kv_heads) * dim + (0 if tied_values else kv_heads * vdim)
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < C:
        raise ValueError("qk_conv_norm_rope_append: proj fp32 [N, >= C]")
    if conv_w is not None and (tuple(conv_w.shape) != (C, taps) or not conv_w.is_contiguous()):
        raise ValueError("qk_conv_norm_rope_append: conv_w [C, taps] contiguous")
    if pool.shape[1] != kv_heads * (dim + vdim):
        raise ValueError("qk_conv_norm_rope_append: pool entry != kv_heads * (dim + vdim)")
    wt = conv_w if conv_w is not None else norm_q
    q = torch.empty((rows, heads, dim), dtype=pool.dtype, device=proj.device)
    st = _p(state) if taps > 1 else None
    check(_rl.tb_qk_conv_norm_rope_append(
        _p(q), _p(pool), _dt(pool), _p(proj), proj.stride(0), _p(conv_w), _p(norm_q), _p(norm_k), _dt(wt) if wt is not None else DT_F32,
        float(eps), st, _p(table), int(dims), _p(batch.tok_seq), _p(batch.tok_pos), _p(batch.seq_start), _p(batch.seq_past),
        _p(batch.seq_slot), _p(batch.block_table), batch.max_blocks, page, rows, heads, kv_heads, dim, vdim, taps, int(bool(tied_values)),
        st, _p(batch.seq_len) if taps > 1 else None, _stream()), "tb_qk_conv_norm_rope_append")
    if taps > 1 and batch.max_len > 1:       # sequences that bring one row were moved on by the kernel above
        check(_rl.tb_causal_conv1d_update(_p(state), _p(proj), proj.stride(0), _p(batch.seq_start), _p(batch.seq_len),
                                          _p(batch.seq_past), _p(batch.seq_slot), batch.num_seqs, C, taps, 1, _stream()),
              "tb_causal_conv1d_update")
    return q


def qk_norm_append(proj, w_q, w_k, eps, pool, batch, page, q_vectors, k_vectors, dim, v_channels, temp_coef=0.0, temp_every=0):
    """Projected rows (fp32 [N, >= (q_vectors + k_vectors) * dim + v_channels]) -> RMS norm of every query and key vector
    over ``dim`` (weights [dim] or None), the queries' position temperature 1 + coef * ln(floor((pos + 1) / every) + 1)
    (every 0: none) -> queries [N, q_vectors, dim] in the pool's type, keys and values into the pages."""
    _chk_dev(proj, w_q, w_k, pool)
    rows = proj.shape[0]
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or proj.shape[1] < (q_vectors + k_vectors) * dim + v_channels:
        raise ValueError("qk_norm_append: proj fp32 [N, >= (q_vectors + k_vectors) * dim + v_channels]")
    if pool.shape[1] != k_vectors * dim + v_channels:
        raise ValueError("qk_norm_append: pool entry != k_vectors * dim + v_channels")
    w = w_q if w_q is not None else w_k
    q = torch.empty((rows, q_vectors, dim), dtype=pool.dtype, device=proj.device)
    check(_rl.tb_qk_norm_append(_p(q), _p(pool), _dt(pool), _p(proj), proj.stride(0), _p(w_q), _p(w_k), _dt(w) if w is not None else 0,
                                float(eps), float(temp_coef), int(temp_every), _p(batch.tok_seq), _p(batch.tok_pos),
                                _p(batch.block_table), batch.max_blocks, page, rows, q_vectors, k_vectors, dim, v_channels, _stream()),
          "tb_qk_norm_append")
    return q


def diff_combine(maps, lq1, lk1, lq2, lk2, diff, eps, mult, kv_heads, out_dtype):
    """maps fp32 [N, kv_heads * 2 * per, vdim] (per key/value head: map 1 of its ``per`` heads, then map 2) -> [N, kv_heads *
    per, vdim] = rms_normalised(map1 - lambda map2) * mult, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff."""
    _chk_cuda(maps, lq1, lk1, lq2, lk2)
    rows, h2, vdim = maps.shape
    per = h2 // (2 * kv_heads)
    if maps.dtype != torch.float32 or per * 2 * kv_heads != h2:
        raise ValueError("diff_combine: maps fp32 [N, kv_heads * 2 * per, vdim]")
    out = torch.empty((rows, kv_heads * per, vdim), dtype=out_dtype, device=maps.device)
    check(_rl.tb_diff_combine(_p(out), _dt(out), _p(maps), _p(lq1), _p(lk1), _p(lq2), _p(lk2), _dt(lq1), lq1.numel(), float(diff),
                              float(eps), float(mult), rows, kv_heads, per, vdim, _stream()), "tb_diff_combine")
    return out


def delta_prepare(proj, conv_w, a_log, dt_bias, col_b, col_a, conv_state, batch, heads, kv_heads, dim, vdim, eps_unit=1e-6):
    """Stacked projection rows (fp32; q | k | v first) -> (u fp32 [N, C]: unit q / sqrt(dim) | unit k | v after convolution
    and SiLU, bg fp32 [N, 2 heads]: beta | decay); then the carried convolution inputs move on."""
    _chk_dev(proj, conv_w, a_log, dt_bias, conv_state)
    rows, taps = proj.shape[0], conv_w.shape[1]
    C = 2 * kv_heads * dim + heads * vdim
    if proj.dtype != torch.float32 or proj.stride(1) != 1 or conv_w.shape[0] != C or not conv_w.is_contiguous():
        raise ValueError("delta_prepare: proj fp32 rows, conv_w [C, taps] contiguous")
    u = torch.empty((rows, C), dtype=torch.float32, device=proj.device)
    bg = torch.empty((rows, 2 * heads), dtype=torch.float32, device=proj.device)
    st = _p(conv_state) if taps > 1 else None
    check(_rl.tb_delta_prepare(_p(u), _p(bg), _p(proj), proj.stride(0), _p(conv_w), _p(a_log), _p(dt_bias), _dt(conv_w), int(col_b),
                               int(col_a), st, st, _p(batch.tok_seq), _p(batch.tok_pos), _p(batch.seq_start), _p(batch.seq_len),
                               _p(batch.seq_past), _p(batch.seq_slot), rows, heads, kv_heads, dim, vdim, taps, float(eps_unit),
                               _stream()), "tb_delta_prepare")
    if taps > 1 and batch.max_len > 1:       # sequences that bring one row were moved on by the kernel above
        check(_rl.tb_causal_conv1d_update(_p(conv_state), _p(proj), proj.stride(0), _p(batch.seq_start), _p(batch.seq_len),
                                          _p(batch.seq_past), _p(batch.seq_slot), batch.num_seqs, C, taps, 1, _stream()),
              "tb_causal_conv1d_update")
    return u, bg


def delta_rule_scan(u, bg, state, batch, heads, kv_heads, dim, vdim):
    """The gated delta rule over every sequence's rows, from and into ``state`` (fp32 [slots, heads * vdim * dim])."""
    _chk_cuda(u, bg, state)
    out = torch.empty((u.shape[0], heads, vdim), dtype=torch.float32, device=u.device)
    ws = None
    if batch.max_len >= 3 and not FORCE_SERIAL_SCAN:      # prompt portions: eight rows at a time over the blocks' own k.k and k.q products
        ws = torch.empty((u.shape[0] * (16 * kv_heads + 20 * heads),), dtype=torch.float32, device=u.device)
    check(_rl.tb_delta_rule_scan(_p(out), _p(u), _p(bg), _p(state), _p(batch.seq_start), _p(batch.seq_len), _p(batch.seq_past),
                                 _p(batch.seq_slot), u.shape[0], batch.num_seqs, heads, kv_heads, dim, vdim, batch.max_len, _p(ws),
                                 _stream()),
          "tb_delta_rule_scan")
    return out


def gated_rmsnorm_heads(o, w, eps, out_dtype, gate=None):
    """o fp32 [N, heads, vdim] -> o / rms(o) * w * silu(gate) per head (gate: fp32 logits [N, >= heads * vdim], any row stride)."""
    _chk_dev(o, w, gate)
    rows, heads, vdim = o.shape
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise ValueError("gate logits are fp32 with unit inner stride")
    out = torch.empty((rows, heads, vdim), dtype=out_dtype, device=o.device)
    check(_rl.tb_gated_rmsnorm_heads(_p(out), _dt(out), _p(o), _p(gate), gate.stride(0) if gate is not None else 0, _p(w),
                                     _dt(w) if w is not None else 0, float(eps), rows, heads, vdim, _stream()), "tb_gated_rmsnorm_heads")
    return out


def rope_heads(x, table, heads, dim, dims, layout, split=0, scale_lo=1.0, scale_hi=1.0, out=None):
    """x fp32 [N, >= heads * dim] (any row stride) -> fp32 [N, heads * dim] with the first ``dims`` elements of every head rotated
    (pairs by ``layout``: ROPE_INTERLEAVED / ROPE_HALF); heads below ``split`` are multiplied by scale_lo, the others by scale_hi."""
    _chk_dev(x, table, out)
    if x.dtype != torch.float32 or x.stride(1) != 1 or x.shape[1] < heads * dim:
        raise ValueError("rope_heads: fp32 rows of at least heads * dim columns")
    if out is None:
        out = torch.empty((x.shape[0], heads * dim), dtype=torch.float32, device=x.device)
    check(_rl.tb_rope_heads(_p(out), out.stride(0), _p(x), x.stride(0), _p(table), x.shape[0], heads, dim, int(dims), int(layout),
                            int(split), float(scale_lo), float(scale_hi), _stream()), "tb_rope_heads")
    return out


def mlstm_gates(proj, col_i, col_f, bias_i, bias_f, cap, m_state, batch, heads):
    """Exponential gates of a matrix memory from the projected logits (columns col_i.. / col_f.. of fp32 ``proj``): -> (log_ab fp32
    [N, heads, 2] = ln decay, ln input weight; m fp32 [N, heads] the running maximum).  ``m_state``: fp32 view [slots, >= heads] of
    the sequences' maxima (row stride = the slot stride), read and written."""
    _chk_dev(proj, bias_i, bias_f, m_state)
    rows = proj.shape[0]
    log_ab = torch.empty((rows, heads, 2), dtype=torch.float32, device=proj.device)
    m = torch.empty((rows, heads), dtype=torch.float32, device=proj.device)
    b = bias_i if bias_i is not None else bias_f
    check(_rl.tb_mlstm_gates(_p(log_ab), _p(m), _p(proj), proj.stride(0), int(col_i), int(col_f), _p(bias_i), _p(bias_f),
                             _dt(b) if b is not None else 0, float(cap or 0.0), _p(m_state), m_state.stride(0), _p(batch.seq_start),
                             _p(batch.seq_len), _p(batch.seq_past), _p(batch.seq_slot), batch.num_seqs, heads, _stream()),
          "tb_mlstm_gates")
    return log_ab, m


FORCE_ROW_SCAN = False      # A/B: the decayed linear attention row by row also for prompt portions
FORCE_ONE_SEGMENT = False   # A/B: ... and long portions as one segment


def decay_attention_scan(q, k, v, state, batch, heads, dim, vdim, log_ab=None, head_decay=None, ones_col=False, q_scale=1.0):
    """S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t per (sequence, head) over every sequence's rows, from and into ``state``
    (fp32 view [slots, >= heads * vcols * dim], row stride = the slot stride).  q, k fp32 [N, >= heads * dim], v fp32 [N, >= heads *
    vdim] (any row strides).  ``log_ab`` fp32 [N, heads, 2] (ln a, ln b) or ``head_decay`` fp32 [heads] (a fixed, b = 1).
    ``ones_col``: a further value column of ones (vcols = vdim + 1).  ``q_scale``: a factor on every query.  -> fp32 [N, heads, vcols]."""
    _chk_dev(q, k, v, state, log_ab, head_decay)
    for t in (q, k, v):
        if t.dtype != torch.float32 or t.stride(1) != 1:
            raise ValueError("decay_attention_scan: fp32 rows with unit inner stride")
    vcols = vdim + (1 if ones_col else 0)
    out = torch.empty((q.shape[0], heads, vcols), dtype=torch.float32, device=q.device)
    # long portions of few sequences: segments side by side, their states carried in order (a state per segment in the workspace)
    segs = 1 if FORCE_ROW_SCAN or FORCE_ONE_SEGMENT else _rl.tb_decay_scan_segments(batch.num_seqs, heads, vcols, batch.max_len)
    ws = None
    if segs > 1:
        ws = torch.empty((batch.num_seqs * segs * (heads * vcols * dim + heads),), dtype=torch.float32, device=q.device)
    check(_rl.tb_decay_attention_scan(_p(out), _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(log_ab), _p(head_decay),
                                      _p(state), state.stride(0), _p(batch.seq_start), _p(batch.seq_len), _p(batch.seq_past),
                                      _p(batch.seq_slot), q.shape[0], batch.num_seqs, heads, dim, vdim, int(bool(ones_col)), float(q_scale),
                                      1 if FORCE_ROW_SCAN else batch.max_len, _p(ws), segs, _stream()), "tb_decay_attention_scan")
    return out


def head_norm_gate(o, vdim, eps, out_dtype, w=None, w_per_head=False, gate=None, gate_act="silu", m=None, den_eps=1e-6):
    """o fp32 [N, heads, vcols] -> [N, heads, vdim]: with ``m`` (fp32 [N, heads]) first o / (max(|o[..., vdim]|, exp(-m)) + den_eps);
    then per head o / rms(o) * w * act(gate) (``w`` [vdim] or, ``w_per_head``, [heads * vdim]; gate fp32 logits [N, >= heads *
    vdim], ``gate_act`` "silu" | "sigmoid")."""
    _chk_dev(o, w, gate, m)
    rows, heads, vcols = o.shape
    if o.dtype != torch.float32 or not o.is_contiguous():
        raise ValueError("head_norm_gate: o fp32 contiguous")
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1):
        raise ValueError("gate logits are fp32 with unit inner stride")
    act = 0 if gate is None else {"silu": 1, "sigmoid": 2}[gate_act]
    out = torch.empty((rows, heads, vdim), dtype=out_dtype, device=o.device)
    check(_rl.tb_head_norm_gate(_p(out), _dt(out), _p(o), vcols, _p(m), float(den_eps), _p(gate), gate.stride(0) if gate is not None else 0,
                                act, _p(w), _dt(w) if w is not None else 0, int(bool(w_per_head)), float(eps), rows, heads, vdim,
                                _stream()), "tb_head_norm_gate")
    return out


def residual_sandwich_layernorm_rows(x, y, w_post, b_post, out_scale, eps, w_pre=None, b_pre=None, out_dtype=torch.float32):
    """x += out_scale * layer_norm(y; w_post, b_post) in place; with ``w_pre`` also returns layer_norm(x; w_pre, b_pre) — the
    residual step of a sublayer between two layer norms and the next sublayer's input in one kernel."""
    _chk_dev(x, y, w_post, b_post, w_pre, b_pre)
    if x.dtype != torch.float32 or y.dtype != torch.float32 or x.stride(1) != 1 or y.stride(1) != 1:
        raise ValueError("residual_sandwich_layernorm_rows: fp32 rows")
    h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if w_pre is not None else None
    check(_rl.tb_residual_sandwich_layernorm_rows(_p(x), x.stride(0), _p(y), y.stride(0), _p(w_post), _p(b_post), _p(w_pre), _p(b_pre),
                                                  _dt(w_post), float(eps), float(out_scale), _p(h), _dt(h) if h is not None else 0,
                                                  h.stride(0) if h is not None else 0, x.shape[0], x.shape[1], _stream()),
          "tb_residual_sandwich_layernorm_rows")
    return h


# The per-layer token input is ONE kernel (a CTA per row does both products) while the step has few rows and the two weight
# matrices are small — launch-bound steps of small models; otherwise its products run as projections (tensor cores / streaming
# kernels that spread the weights over the chip) and the kernel only finishes (norm, residual step, next norm).
SIDE_FUSED_MAX_ROWS = 8
SIDE_FUSED_MAX_WEIGHTS = 16384


def token_side_input(x, side_embed, e_off, ids, w_gate, w_proj, norm_w, eps, w_pre=None, b_pre=None, pre_rms=False,
                     out_dtype=torch.float32):
    """x += rms_norm(w_proj (gelu_tanh(w_gate x) * side_embed[ids, e_off : e_off + sd])) * norm_w in place (sd = w_gate.shape[0]);
    with ``w_pre`` also returns the next layer's input: layer_norm(x; w_pre, b_pre), or the RMS norm when ``pre_rms``."""
    _chk_dev(x, side_embed, ids, w_gate, w_proj, norm_w, w_pre, b_pre)
    sd, width = w_gate.shape
    if x.dtype != torch.float32 or x.stride(1) != 1 or x.shape[1] != width or tuple(w_proj.shape) != (width, sd) \
            or side_embed.shape[1] < e_off + sd or side_embed.stride(1) != 1:
        raise ValueError("token_side_input: x fp32 [N, width], w_gate [sd, width], w_proj [width, sd], side_embed [vocab, >= e_off + sd]")
    for t in (side_embed, w_proj, norm_w, w_pre, b_pre):
        if t is not None and t.dtype != w_gate.dtype:
            raise TypeError("token_side_input: tensors of one storage type")
    h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if w_pre is not None else None
    y = None
    if x.shape[0] > SIDE_FUSED_MAX_ROWS or sd * width > SIDE_FUSED_MAX_WEIGHTS:
        # the two products as projections, the kernel below finishes
        z = linear(x, w_gate, out_dtype=torch.float32)
        g = torch.empty((x.shape[0], sd), dtype=w_gate.dtype, device=x.device)
        check(_rl.tb_side_gate_mul(_p(g), _dt(g), _p(z), z.stride(0), _p(side_embed), _dt(side_embed), side_embed.stride(0), int(e_off),
                                   _p(ids), side_embed.shape[0], x.shape[0], sd, _stream()), "tb_side_gate_mul")
        y = linear(g, w_proj, out_dtype=torch.float32)
    check(_rl.tb_token_side_input(_p(x), x.stride(0), _p(y), y.stride(0) if y is not None else 0, _p(side_embed), side_embed.stride(0),
                                  int(e_off), _p(ids), side_embed.shape[0], _p(w_gate), _p(w_proj), _p(norm_w), _dt(w_gate), float(eps),
                                  x.shape[0], width, sd, _p(w_pre), _p(b_pre), int(bool(pre_rms)), _p(h), _dt(h) if h is not None else 0,
                                  h.stride(0) if h is not None else 0, _stream()), "tb_token_side_input")
    return h


def rmsnorm_pair_sum(a, b, wa, wb, eps, out_scale):
    """out_scale * (a / rms(a) * wa + b / rms(b) * wb) over fp32 rows."""
    _chk_dev(a, b, wa, wb)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.stride(1) != 1 or b.stride(1) != 1 or a.shape != b.shape \
            or wa.dtype != wb.dtype:
        raise ValueError("rmsnorm_pair_sum: two fp32 row sets of one shape, weights of one type")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    check(_rl.tb_rmsnorm_pair_sum(_p(out), out.stride(0), _p(a), a.stride(0), _p(b), b.stride(0), _p(wa), _p(wb), _dt(wa), float(eps),
                                  float(out_scale), a.shape[0], a.shape[1], _stream()), "tb_rmsnorm_pair_sum")
    return out


def layernorm_rows(x, w, b, eps, out_dtype=torch.float32, rows_idx=None):
    """Layer norm with weight and bias of fp32 rows (row r of the result from row rows_idx[r] when given)."""
    _chk_dev(x, w, b, rows_idx)
    if x.dtype != torch.float32 or x.stride(1) != 1:
        raise ValueError("layernorm_rows normalises fp32 rows")
    rows = x.shape[0] if rows_idx is None else rows_idx.numel()
    out = torch.empty((rows, x.shape[1]), dtype=out_dtype, device=x.device)
    check(_rl.tb_layernorm_rows(_p(out), _dt(out), out.stride(0), _p(x), x.stride(0), _p(w), _p(b), _dt(w), float(eps), _p(rows_idx),
                                rows, x.shape[1], _stream()), "tb_layernorm_rows")
    return out


def residual_layernorm_rows(x, y1, y2, out_scale, w=None, b=None, eps=0.0, out_dtype=torch.float32):
    """x += out_scale * (y1 + y2) in place (y2 may be None); with ``w`` also returns layer_norm(x; w, b) — the residual step of
    a layer with side-by-side sublayers and the next layer's input in one kernel."""
    _chk_dev(x, y1, y2, w, b)
    for t in (x, y1, y2):
        if t is not None and (t.dtype != torch.float32 or t.stride(1) != 1):
            raise ValueError("residual_layernorm_rows: fp32 rows")
    h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if w is not None else None
    check(_rl.tb_residual_layernorm_rows(_p(x), x.stride(0), _p(y1), y1.stride(0), _p(y2), y2.stride(0) if y2 is not None else 0,
                                         float(out_scale), _p(w), _p(b), _dt(w) if w is not None else 0, float(eps), _p(h),
                                         _dt(h) if h is not None else 0, h.stride(0) if h is not None else 0, x.shape[0], x.shape[1],
                                         _stream()), "tb_residual_layernorm_rows")
    return h


def concat_rows(a, b, out_dtype):
    """[a | b] row by row (fp32 inputs) as one contiguous operand of type ``out_dtype``."""
    _chk_dev(a, b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.stride(1) != 1 or b.stride(1) != 1 or a.shape[0] != b.shape[0]:
        raise ValueError("concat_rows: two fp32 row sets of equal height")
    out = torch.empty((a.shape[0], a.shape[1] + b.shape[1]), dtype=out_dtype, device=a.device)
    check(_rl.tb_concat_rows(_p(out), _dt(out), _p(a), a.stride(0), a.shape[1], _p(b), b.stride(0), b.shape[1], a.shape[0], _stream()),
          "tb_concat_rows")
    return out


MOE_TILE = 64            # tile height of the warp-MMA / FMA expert products
MOE_TILE_TC = 128        # ... of the tcgen05 expert products
MOE_GEMV_MAX_PAIRS = 64  # up to this many (token, choice) pairs a step runs the streaming kernel per pair, without a plan


def moe_route(logits, correction, top, groups, keep):
    """-> (ids int32 [N, top], weights fp32 [N, top]) from fp32 router logits [N, experts]."""
    _chk_cuda(logits, correction)
    rows, experts = logits.shape
    ids = torch.empty((rows, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((rows, top), dtype=torch.float32, device=logits.device)
    check(_rl.tb_moe_route(_p(ids), _p(weights), _p(logits.contiguous()), _p(correction),
                           _dt(correction) if correction is not None else 0, rows, experts, top, groups, keep, _stream()),
          "tb_moe_route")
    return ids, weights


def moe_route_softmax(logits, top, renorm=True, scale=1.0):
    """-> (ids int32 [N, top], weights fp32 [N, top]): softmax over all experts, the ``top`` largest, weights = score / (sum of
    the chosen + 1e-20) * scale (renorm) or score * scale."""
    _chk_cuda(logits)
    rows, experts = logits.shape
    ids = torch.empty((rows, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((rows, top), dtype=torch.float32, device=logits.device)
    check(_rl.tb_moe_route_softmax(_p(ids), _p(weights), _p(logits.contiguous()), rows, experts, top, int(bool(renorm)), float(scale),
                                   _stream()), "tb_moe_route_softmax")
    return ids, weights


def moe_plan(ids, experts, tile=MOE_TILE):
    """-> (slot_pair int32 [tiles * tile], tile_expert int32 [tiles], pair_slot int32 [pairs]): the pairs sorted by expert
    in whole tiles, and where each pair went."""
    _chk_cuda(ids)
    pairs = ids.numel()
    tiles = _rl.tb_moe_plan_tiles(pairs, experts, tile)
    slot_pair = torch.empty((tiles * tile,), dtype=torch.int32, device=ids.device)
    tile_expert = torch.empty((tiles,), dtype=torch.int32, device=ids.device)
    pair_slot = torch.empty((pairs,), dtype=torch.int32, device=ids.device)
    check(_rl.tb_moe_plan(_p(slot_pair), _p(tile_expert), _p(pair_slot), _p(ids), pairs, experts, tile, tiles, _stream()),
          "tb_moe_plan")
    return slot_pair, tile_expert, pair_slot


def moe_linear(a, w, slot_pair, tile_expert, *, a_div, out_dtype, act=ACT_NONE, compute=COMPUTE_AUTO):
    """Expert products over a plan with tiles of MOE_TILE rows (warp-MMA tiles for bf16 weights, fp32 FMA tiles otherwise).
    w [experts, N, K].  a_div > 0: ``a`` holds token rows and slot s reads row slot_pair[s] // a_div; a_div == 0: ``a``
    holds one row per slot.  The result has one row per slot."""
    _chk_dev(a, w, slot_pair, tile_expert)
    _, N, K = w.shape
    if not w.is_contiguous() or a.stride(1) != 1 or a.shape[1] != K:
        raise ValueError("moe_linear: w [experts, N, K] contiguous, a [*, K]")
    out = torch.empty((slot_pair.numel(), N), dtype=out_dtype, device=a.device)
    check(_rl.tb_moe_linear(_p(out), _dt(out), out.stride(0), _p(a), _dt(a), a.stride(0), _p(w), _dt(w), _p(slot_pair),
                            _p(tile_expert), tile_expert.numel(), int(a_div), 0, N, K, act, compute, _stream()),
          "tb_moe_linear")
    return out


def moe_gather_rows(x, slot_pair, top):
    """bf16 [slots, K]: the pairs' token rows in plan order (zeros in the padding)."""
    _chk_dev(x, slot_pair)
    out = torch.empty((slot_pair.numel(), x.shape[1]), dtype=torch.bfloat16, device=x.device)
    check(_rl.tb_moe_gather_rows(_p(out), _p(x), _dt(x), x.stride(0), _p(slot_pair), slot_pair.numel(), top, x.shape[1],
                                 _stream()), "tb_moe_gather_rows")
    return out


def moe_linear_tc(xs, w, tile_expert, out_dtype, act=ACT_NONE):
    """Expert products on the tcgen05 kernel over a plan with tiles of MOE_TILE_TC rows: xs bf16 [slots, K] contiguous in
    plan order, w bf16 [experts, N, K]; one result row per slot."""
    _chk_cuda(xs, w, tile_expert)
    E, N, K = w.shape
    out = torch.empty((xs.shape[0], N), dtype=out_dtype, device=xs.device)
    check(_rl.tb_gemm_tc_bf16_grouped(_p(out), 1 if out_dtype == torch.float32 else 3, _p(xs), _p(w), _p(tile_expert),
                                      tile_expert.numel(), E, act, N, K, _stream()), "tb_gemm_tc_bf16_grouped")
    return out


def moe_gemv(a, w, ids, *, a_div, out_dtype, gated=False, act=ACT_NONE, gate=GATE_SIGMOID, alpha=1.0, limit=0.0, up_shift=0.0,
             pair_scale=None):
    """Expert products for few pairs without a plan: pair b against expert ids[b].  gated: w [experts, 2 N, K] and the
    result is the gated activation (``gate``, alpha, limit, up_shift; the defaults are silu(gate) * up) of the two products, both
    first multiplied by ``pair_scale[b]`` (fp32) when given; else ``act`` is applied.  Returns None when the streaming kernel
    does not take the shape."""
    _chk_dev(a, w, ids)
    E, rows_w, K = w.shape
    N = rows_w // 2 if gated else rows_w
    pairs = ids.numel()
    out = torch.empty((pairs, N), dtype=out_dtype, device=a.device)
    rc = _rl.tb_moe_gemv(_p(out), _dt(out), out.stride(0), _p(a), _dt(a), a.stride(0), _p(w), _dt(w), _p(ids), pairs, int(a_div),
                         N, K, 2 if gated else act, int(gate), float(alpha), float(limit), float(up_shift), _p(pair_scale), _stream())
    if rc == -3:
        return None
    check(rc, "tb_moe_gemv")
    return out


def moe_combine(y, weights, pair_slot=None, add=None):
    """out[n] = add[n] + sum_k weights[n, k] * y[row of pair n * top + k]  (fp32); the pair's row is pair_slot[pair], or the
    pair's index when ``y`` is in pair order.  ``add``: fp32 [N, width] every token has besides (a shared expert), or None.
    ``weights`` may be ``(rows, top)`` instead of a tensor: a plain sum."""
    _chk_cuda(y, pair_slot, add)
    if isinstance(weights, tuple):
        (rows, top), weights = weights, None
    else:
        _chk_cuda(weights)
        rows, top = weights.shape
    out = torch.empty((rows, y.shape[1]), dtype=torch.float32, device=y.device)
    if add is not None and (add.dtype != torch.float32 or add.shape != out.shape):
        raise ValueError("moe_combine: add is fp32 [N, width]")
    check(_rl.tb_moe_combine_add(_p(out), _p(y), _p(weights), _p(pair_slot), _p(add), rows, y.shape[1], top, _stream()),
          "tb_moe_combine_add")
    return out


def argmax_rows(logits):
    _chk_cuda(logits)
    out = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
    check(_rl.tb_argmax(_p(out), _p(logits), logits.shape[0], logits.shape[1], logits.stride(0), _stream()), "tb_argmax")
    return out
