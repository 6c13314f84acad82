// Gated delta rule over a ragged in-flight batch: a recurrent layer whose state per head is a matrix S [dim, vdim] that
// decays, is corrected towards the value along the key, and is read with the query:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// Everything here is fp32: the state, the unit-normalised queries and keys, beta, the decay and the read-out.
//
//   delta_prepare_kernel   one CTA per row over the stacked projection q | k | v | (further columns): short causal convolution over
//                          the row's portion and the sequence's carried inputs, SiLU, then per head x / sqrt(sum x^2 + eps_unit)
//                          for queries (times dim^-1/2) and keys; beta = sigmoid(b) and g = exp(-exp(A_log) softplus(a + dt_bias))
//                          per head.  A sequence that brings ONE row has its carried inputs moved on here.
//   delta_scan_kernel      the columns of S are independent recurrences: one warp per (sequence, head, value column), the lanes
//                          hold the column's `dim` state elements (dim / 32 each).  Per token two dot products are reduced over
//                          the lanes at once, a = S^T k and b = S^T q of the OLD state, and with k . q (computed when the
//                          token chunk is staged) the step is u = beta (v - g a), o = g b + u (k . q), S <- g S + k u: one
//                          reduction round per token instead of two dependent ones.  Tokens are staged through shared memory
//                          in chunks of 16.  State layout per slot: [heads][vdim][dim] (a column's elements are contiguous).
//   gated_rmsnorm_heads    one warp per (row, head): o / sqrt(mean(o^2) + eps) * w * silu(gate), stored in the storage type.
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

constexpr int kMaxTaps = 16;

struct PrepArgs {
  const float* proj; int64_t ldp;          // [rows, >= C + ...]: q (G dim) | k (G dim) | v (H vdim) are the C convolved channels
  const void* conv_w; int w_dtype;         // [C, taps]
  const float* state; float* state_rw;     // carried inputs [slots, taps - 1, C]; state_rw == state: single rows move them on
  const void *a_log, *dt_bias;             // [H]
  int col_b, col_a;                        // columns of proj that hold the beta and the decay logits (H each)
  const int *tok_seq, *tok_pos, *seq_start, *seq_len, *seq_past, *seq_slot;
  int H, G, dim, vdim, taps;
  float eps_unit;
};

__device__ __forceinline__ float conv_silu_at(const PrepArgs& a, const float* st, int C, int ch, int pos, int past, int start) {
  float acc = 0.f;
  for (int k = 0; k < a.taps; ++k) {
    const int p = pos - (a.taps - 1 - k);
    float v = 0.f;
    if (p >= past) v = a.proj[(int64_t) (start + (p - past)) * a.ldp + ch];
    else if (p >= 0) v = st[(int64_t) (a.taps - 1 - (past - p)) * C + ch];     // state row j holds position past - (taps - 1) + j
    acc = fmaf(ld_w(a.conv_w, a.w_dtype, (int64_t) ch * a.taps + k), v, acc);
  }
  return silu_f(acc);
}

// u [rows, C] fp32 = unit q * dim^-1/2 | unit k | v ;  bg [rows, 2 H] = beta | g
__global__ void __launch_bounds__(256) delta_prepare_kernel(float* u, float* bg, PrepArgs a) {
  const int Cqk = 2 * a.G * a.dim, C = Cqk + a.H * a.vdim;
  const int row = blockIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int e = a.tok_seq[row], pos = a.tok_pos[row], past = a.seq_past[e], start = a.seq_start[e];
  const float* st = a.state + (int64_t) a.seq_slot[e] * (a.taps - 1) * C;
  const bool carry = a.state_rw && a.taps > 1 && a.seq_len[e] == 1;
  float* st_rw = carry ? a.state_rw + (int64_t) a.seq_slot[e] * (a.taps - 1) * C : nullptr;
  float* ur = u + (int64_t) row * C;
  auto move_on = [&](int c) {
    // row j of the new state holds position pos - n + 1 + j: the old row j + 1 (zero before the sequence's start), then this row's input
    const int n = a.taps - 1;
    for (int j = 0; j + 1 < n; ++j) st_rw[(int64_t) j * C + c] = pos - n + 1 + j >= 0 ? st_rw[(int64_t) (j + 1) * C + c] : 0.f;
    st_rw[(int64_t) (n - 1) * C + c] = a.proj[(int64_t) row * a.ldp + c];
  };
  // queries and keys: a warp per head vector
  for (int v = warp; v < 2 * a.G; v += 8) {
    const int c0 = v * a.dim;
    float ss = 0.f;
    for (int d = lane; d < a.dim; d += 32) {
      const float y = conv_silu_at(a, st, C, c0 + d, pos, past, start);
      ur[c0 + d] = y;
      ss = fmaf(y, y, ss);
      if (carry) move_on(c0 + d);
    }
    float f = 1.f / sqrtf(warp_sum(ss) + a.eps_unit);
    if (v < a.G) f *= 1.f / sqrtf((float) a.dim);
    for (int d = lane; d < a.dim; d += 32) ur[c0 + d] *= f;       // a lane re-reads what it wrote itself
  }
  for (int c = Cqk + threadIdx.x; c < C; c += 256) {
    ur[c] = conv_silu_at(a, st, C, c, pos, past, start);
    if (carry) move_on(c);
  }
  for (int h = threadIdx.x; h < a.H; h += 256) {
    const float* pr = a.proj + (int64_t) row * a.ldp;
    bg[(int64_t) row * 2 * a.H + h] = 1.f / (1.f + expf(-pr[a.col_b + h]));
    const float rate = expf(ld_w(a.a_log, a.w_dtype, h)) * softplus_f(pr[a.col_a + h] + ld_w(a.dt_bias, a.w_dtype, h));
    bg[(int64_t) row * 2 * a.H + a.H + h] = expf(-rate);
  }
}

constexpr int kScanCols = 8;     // value columns (= warps) per CTA
constexpr int kScanChunk = 16;   // tokens staged at a time

struct ScanArgs {
  const float* u; const float* bg;         // prepared rows (see above)
  float* state;                            // [slots, H, vdim, dim]
  const int *seq_start, *seq_len, *seq_past, *seq_slot;
  int H, G, dim, vdim;
};

// shared memory: k [chunk][dim] | q [chunk][dim] | v [chunk][8] | beta, g, k.q [chunk] each
template <int DPL>
__global__ void __launch_bounds__(kScanCols * 32) delta_scan_kernel(float* out, ScanArgs a) {
  extern __shared__ float smem[];
  float* ks = smem;
  float* qs = ks + kScanChunk * a.dim;
  float* vs = qs + kScanChunk * a.dim;
  float* bs = vs + kScanChunk * kScanCols;
  float* gs = bs + kScanChunk;
  float* kqs = gs + kScanChunk;
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * kScanCols;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int col = c0 + warp;
  const bool live = col < a.vdim;
  const int len = a.seq_len[e], past = a.seq_past[e], row0 = a.seq_start[e];
  const int j = h / (a.H / a.G);                                             // the head's query / key head
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  float* sp = a.state + (((int64_t) a.seq_slot[e] * a.H + h) * a.vdim + (live ? col : 0)) * a.dim;
  float S[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    S[i] = (live && past > 0 && d < a.dim) ? sp[d] : 0.f;                    // a sequence at position 0 starts from zeros
  }
  for (int t0 = 0; t0 < len; t0 += kScanChunk) {
    const int nt = min(kScanChunk, len - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * a.dim; i += kScanCols * 32) {
      const int t = i / a.dim, d = i % a.dim;
      const float* ur = a.u + (int64_t) (row0 + t0 + t) * C;
      qs[i] = ur[j * a.dim + d];
      ks[i] = ur[(a.G + j) * a.dim + d];
    }
    for (int i = threadIdx.x; i < nt * kScanCols; i += kScanCols * 32) {
      const int t = i / kScanCols, c = c0 + i % kScanCols;
      vs[i] = c < a.vdim ? a.u[(int64_t) (row0 + t0 + t) * C + 2 * a.G * a.dim + h * a.vdim + c] : 0.f;
    }
    if (threadIdx.x < nt) {
      bs[threadIdx.x] = a.bg[(int64_t) (row0 + t0 + threadIdx.x) * 2 * a.H + h];
      gs[threadIdx.x] = a.bg[(int64_t) (row0 + t0 + threadIdx.x) * 2 * a.H + a.H + h];
    }
    __syncthreads();
    for (int t = warp; t < nt; t += kScanCols) {
      float s = 0.f;
      for (int d = lane; d < a.dim; d += 32) s = fmaf(ks[t * a.dim + d], qs[t * a.dim + d], s);
      s = warp_sum(s);
      if (lane == 0) kqs[t] = s;
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      float kr[DPL], pa = 0.f, pb = 0.f;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int d = lane + 32 * i;
        const bool in = d < a.dim;
        kr[i] = in ? ks[t * a.dim + d] : 0.f;
        const float qv = in ? qs[t * a.dim + d] : 0.f;
        pa = fmaf(S[i], kr[i], pa);
        pb = fmaf(S[i], qv, pb);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        pa += __shfl_xor_sync(0xffffffffu, pa, o);
        pb += __shfl_xor_sync(0xffffffffu, pb, o);
      }
      const float g = gs[t];
      const float uu = bs[t] * (vs[t * kScanCols + warp] - g * pa);
#pragma unroll
      for (int i = 0; i < DPL; ++i) S[i] = fmaf(g, S[i], kr[i] * uu);
      if (live && lane == 0) out[((int64_t) (row0 + t0 + t) * a.H + h) * a.vdim + col] = fmaf(g, pb, uu * kqs[t]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < a.dim) sp[d] = S[i];
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) gated_rmsnorm_heads_kernel(T* out, const float* o, const float* gate, int64_t ldg, const void* w,
                                                                  int w_dtype, float eps, int64_t items, int H, int vdim) {
  const int lane = threadIdx.x % 32;
  const int64_t item = (int64_t) blockIdx.x * 4 + threadIdx.x / 32;          // (row, head)
  if (item >= items) return;
  const float* src = o + item * vdim;
  float ss = 0.f;
  for (int c = lane; c < vdim; c += 32) ss = fmaf(src[c], src[c], ss);
  const float inv = 1.f / sqrtf(warp_sum(ss) / (float) vdim + eps);
  const float* gr = gate ? gate + (item / H) * ldg + (item % H) * vdim : nullptr;
  for (int c = lane; c < vdim; c += 32) {
    float y = src[c] * inv;
    if (w) y *= ld_w(w, w_dtype, c);
    if (gr) y *= silu_f(gr[c]);
    out[item * vdim + c] = from_f<T>(y);
  }
}

template <int DPL>
int launch_scan(float* out, const ScanArgs& a, int seqs, cudaStream_t s) {
  const size_t smem = ((size_t) 2 * kScanChunk * a.dim + kScanChunk * kScanCols + 3 * kScanChunk) * sizeof(float);
  static size_t raised = 48 * 1024;
  if (smem > raised) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(delta_scan_kernel<DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = smem;
  }
  dim3 grid((a.vdim + kScanCols - 1) / kScanCols, a.H, seqs);
  delta_scan_kernel<DPL><<<grid, kScanCols * 32, smem, s>>>(out, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace
}  // namespace tb

using namespace tb;
static inline bool dt_ok(int d) { return d == TB_DT_F32 || d == TB_DT_BF16; }

extern "C" int tb_delta_prepare(float* u, float* bg, const float* proj, int64_t ldp, const void* conv_w, const void* a_log,
                                const void* dt_bias, int w_dtype, int col_b, int col_a, const float* state, float* state_rw,
                                const int* tok_seq, const int* tok_pos, const int* seq_start, const int* seq_len, const int* seq_past,
                                const int* seq_slot, int rows, int heads, int kv_heads, int dim, int vdim, int taps, float eps_unit,
                                tb_stream_t stream) {
  if (!u || !bg || !proj || !conv_w || !a_log || !dt_bias || !dt_ok(w_dtype) || !tok_seq || !tok_pos || !seq_start || !seq_len ||
      !seq_past || !seq_slot)
    return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || taps < 1 || taps > kMaxTaps || rows < 0 ||
      col_b < 0 || col_a < 0 || (taps > 1 && !state) || (state_rw && state_rw != state))
    return -1;
  if (rows == 0) return 0;
  PrepArgs a{proj, ldp, conv_w, w_dtype, state, state_rw, a_log, dt_bias, col_b, col_a, tok_seq, tok_pos, seq_start, seq_len,
             seq_past, seq_slot, heads, kv_heads, dim, vdim, taps, eps_unit};
  delta_prepare_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(u, bg, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_delta_rule_scan(float* out, const float* u, const float* bg, float* state, const int* seq_start, const int* seq_len,
                                  const int* seq_past, const int* seq_slot, int seqs, int heads, int kv_heads, int dim, int vdim,
                                  tb_stream_t stream) {
  if (!out || !u || !bg || !state || !seq_start || !seq_len || !seq_past || !seq_slot) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 512 || vdim <= 0 || seqs < 0 || seqs > 65535 || heads > 65535)
    return -1;
  if (seqs == 0) return 0;
  ScanArgs a{u, bg, state, seq_start, seq_len, seq_past, seq_slot, heads, kv_heads, dim, vdim};
  cudaStream_t s = (cudaStream_t) stream;
  const int dpl = (dim + 31) / 32;
  if (dpl <= 1) return launch_scan<1>(out, a, seqs, s);
  if (dpl <= 2) return launch_scan<2>(out, a, seqs, s);
  if (dpl <= 4) return launch_scan<4>(out, a, seqs, s);
  if (dpl <= 8) return launch_scan<8>(out, a, seqs, s);
  return launch_scan<16>(out, a, seqs, s);
}

extern "C" int tb_gated_rmsnorm_heads(void* out, int dtype, const float* o, const float* gate, int64_t ldg, const void* w, int w_dtype,
                                      float eps, int rows, int heads, int vdim, tb_stream_t stream) {
  if (!out || !o || !dt_ok(dtype) || (w && !dt_ok(w_dtype)) || heads <= 0 || vdim <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  const int64_t items = (int64_t) rows * heads;
  const unsigned grid = (unsigned) ((items + 3) / 4);
  if (dtype == TB_DT_F32)
    gated_rmsnorm_heads_kernel<float><<<grid, 128, 0, (cudaStream_t) stream>>>((float*) out, o, gate, ldg, w, w_dtype, eps, items, heads, vdim);
  else
    gated_rmsnorm_heads_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) out, o, gate, ldg, w, w_dtype, eps,
                                                                                       items, heads, vdim);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
