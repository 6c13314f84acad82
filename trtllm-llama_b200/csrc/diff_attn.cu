// Differential attention over a paged key/value pool for a ragged in-flight batch: every query head carries TWO attention
// maps (two queries against two keys) over ONE set of values, and the head's output is map 1 minus lambda times map 2,
// normalised.  The attention itself is the grouped-query kernel of window_attn.cu with shared value heads
// (tb_window_attention_shared_values): the 2 H (head, map) queries are laid out key head by key head, [g][map][head of the group], so
// that query head h' reads key head h' / (H / G) = (g, map) and value head g.  This file holds the steps around it:
//
//   qk_norm_append_kernel   one CTA per row, one warp per (head, map) vector: RMS norm over `dim` with a weight shared by all
//                           heads, for queries also the position's temperature 1 + coef * ln(floor((pos + 1) / every) + 1);
//                           queries to their buffer, normalised keys and the values to the row's place in its pages.
//   diff_combine_kernel     one warp per (row, head): o = a1 - lambda * a2 in fp32, o / sqrt(mean(o^2) + eps) * mult, stored in
//                           the storage type.  lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff is recomputed by every warp
//                           from the four vectors (dim multiply-adds), so nothing is computed on the host.
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

struct QkNormArgs {
  const float* proj; int64_t ldp;          // [rows, >= C]: q (QH dim) | k (KH dim) | v (VC)
  const void *wq, *wk; int w_dtype;        // norm weights [dim] (NULL: none)
  const int *tok_seq, *tok_pos, *block_table;
  int max_blocks, page, QH, KH, dim, VC;
  float eps, temp_coef; int temp_every;    // temp_every <= 0: no temperature
};

template <typename T>
__global__ void __launch_bounds__(256) qk_norm_append_kernel(T* q_out, T* pool, QkNormArgs a) {
  const int row = blockIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int e = a.tok_seq[row], pos = a.tok_pos[row];
  const int64_t slot = (int64_t) a.block_table[(int64_t) e * a.max_blocks + pos / a.page] * a.page + pos % a.page;
  const float* pr = a.proj + (int64_t) row * a.ldp;
  T* kv_row = pool + slot * ((int64_t) a.KH * a.dim + a.VC);
  const float temp = a.temp_every > 0 ? 1.f + a.temp_coef * logf((float) ((pos + 1) / a.temp_every + 1)) : 1.f;
  for (int v = warp; v < a.QH + a.KH; v += 8) {
    const bool is_q = v < a.QH;
    const float* src = pr + (int64_t) v * a.dim;
    float ss = 0.f;
    for (int d = lane; d < a.dim; d += 32) { const float x = src[d]; ss = fmaf(x, x, ss); }
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float) a.dim + a.eps);
    const void* w = is_q ? a.wq : a.wk;
    T* dst = is_q ? q_out + ((int64_t) row * a.QH + v) * a.dim : kv_row + (int64_t) (v - a.QH) * a.dim;
    for (int d = lane; d < a.dim; d += 32) {
      float y = src[d] * inv;
      if (w) y *= ld_w(w, a.w_dtype, d);
      if (is_q) y *= temp;
      dst[d] = from_f<T>(y);
    }
  }
  const float* vsrc = pr + (int64_t) (a.QH + a.KH) * a.dim;
  T* vdst = kv_row + (int64_t) a.KH * a.dim;
  for (int c = threadIdx.x; c < a.VC; c += 256) vdst[c] = from_f<T>(vsrc[c]);
}

struct CombineArgs {
  const float* maps;                       // [rows, G, 2, per, vdim] fp32
  const void *lq1, *lk1, *lq2, *lk2; int w_dtype; int ldim;
  float diff, eps, mult;
  int rows, G, per, vdim;
};

template <typename T>
__global__ void __launch_bounds__(128) diff_combine_kernel(T* out, CombineArgs a) {
  const int lane = threadIdx.x % 32;
  const int64_t item = (int64_t) blockIdx.x * 4 + threadIdx.x / 32;          // (row, head)
  const int H = a.G * a.per;
  if (item >= (int64_t) a.rows * H) return;
  float d1 = 0.f, d2 = 0.f;
  for (int d = lane; d < a.ldim; d += 32) {
    d1 = fmaf(ld_w(a.lq1, a.w_dtype, d), ld_w(a.lk1, a.w_dtype, d), d1);
    d2 = fmaf(ld_w(a.lq2, a.w_dtype, d), ld_w(a.lk2, a.w_dtype, d), d2);
  }
  const float lam = expf(warp_sum(d1)) - expf(warp_sum(d2)) + a.diff;
  const int64_t row = item / H;
  const int head = (int) (item % H), g = head / a.per, hl = head % a.per;
  const float* a1 = a.maps + ((row * a.G + g) * 2 * a.per + hl) * a.vdim;
  const float* a2 = a1 + (int64_t) a.per * a.vdim;
  float ss = 0.f;
  for (int c = lane; c < a.vdim; c += 32) { const float o = fmaf(-lam, a2[c], a1[c]); ss = fmaf(o, o, ss); }
  const float f = a.mult / sqrtf(warp_sum(ss) / (float) a.vdim + a.eps);
  T* dst = out + item * a.vdim;
  for (int c = lane; c < a.vdim; c += 32) dst[c] = from_f<T>(fmaf(-lam, a2[c], a1[c]) * f);
}

}  // namespace
}  // namespace tb

using namespace tb;
static inline bool dt_ok(int d) { return d == TB_DT_F32 || d == TB_DT_BF16; }

extern "C" int tb_qk_norm_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* wq, const void* wk,
                                 int w_dtype, float eps, float temp_coef, int temp_every, const int* tok_seq,
                                 const int* tok_pos, const int* block_table, int max_blocks, int page, int rows, int q_vectors,
                                 int k_vectors, int dim, int v_channels, tb_stream_t stream) {
  if (!q_out || !pool || !proj || !tok_seq || !tok_pos || !block_table || !dt_ok(dtype)) return -1;
  if ((wq || wk) && !dt_ok(w_dtype)) return -1;
  if (q_vectors <= 0 || k_vectors <= 0 || dim <= 0 || v_channels < 0 || page <= 0 || rows < 0 || max_blocks <= 0) return -1;
  if (rows == 0) return 0;
  QkNormArgs a{proj, ldp, wq, wk, w_dtype, tok_seq, tok_pos, block_table, max_blocks, page, q_vectors, k_vectors, dim,
               v_channels, eps, temp_coef, temp_every};
  if (dtype == TB_DT_F32) qk_norm_append_kernel<float><<<rows, 256, 0, (cudaStream_t) stream>>>((float*) q_out, (float*) pool, a);
  else qk_norm_append_kernel<__nv_bfloat16><<<rows, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) q_out, (__nv_bfloat16*) pool, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_diff_combine(void* out, int dtype, const float* maps, const void* lq1, const void* lk1, const void* lq2,
                               const void* lk2, int w_dtype, int ldim, float diff, float eps, float mult, int rows, int kv_heads,
                               int per, int vdim, tb_stream_t stream) {
  if (!out || !maps || !lq1 || !lk1 || !lq2 || !lk2 || !dt_ok(dtype) || !dt_ok(w_dtype)) return -1;
  if (ldim <= 0 || kv_heads <= 0 || per <= 0 || vdim <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  CombineArgs a{maps, lq1, lk1, lq2, lk2, w_dtype, ldim, diff, eps, mult, rows, kv_heads, per, vdim};
  const int64_t items = (int64_t) rows * kv_heads * per;
  const unsigned grid = (unsigned) ((items + 3) / 4);
  if (dtype == TB_DT_F32) diff_combine_kernel<float><<<grid, 128, 0, (cudaStream_t) stream>>>((float*) out, a);
  else diff_combine_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) out, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
