// Row-wise kernels of the ragged-batch models whose residual stream is fp32: scaled embedding, RMS normalisation of a
// sublayer's output accumulated into the residual, layer normalisation (alone and with the residual step of a layer whose
// sublayers run side by side), the clamped gated activation of the feed-forward, and the rotary table.  All are bandwidth-bound passes over [rows, width]; statistics and sums are fp32.
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

__device__ __forceinline__ float ld_f(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_f(void* p, int dtype, int64_t i, float v) {
  if (dtype == TB_DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__global__ void embed_scaled_kernel(float* out, const void* table, int t_dtype, const int* ids, float scale, int width,
                                    int vocab) {
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(int64_t) row * width + c] = ld_f(table, t_dtype, (int64_t) id * width + c) * scale;
}

// one CTA per row; the sum of squares is reduced in a fixed tree (warp shuffles, then warp 0 over the warp sums)
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi,
                                                           const void* w, int w_dtype, float w_offset, float eps,
                                                           const int* rows_idx, int cols, int accumulate, float out_scale) {
  __shared__ float red[8];
  __shared__ float inv_s;
  const int row = blockIdx.x;
  const float* xr = x + (int64_t) (rows_idx ? rows_idx[row] : row) * ldi;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float v = xr[c]; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) inv_s = 1.f / sqrtf(v / (float) cols + eps);
  }
  __syncthreads();
  const float inv = inv_s;
  for (int c = threadIdx.x; c < cols; c += 256) {
    float y = xr[c] * inv;
    if (w) y *= ld_f(w, w_dtype, c) + w_offset;
    y *= out_scale;
    const int64_t o = (int64_t) row * ldo + c;
    if (accumulate) reinterpret_cast<float*>(out)[o] += y;
    else st_f(out, out_dtype, o, y);
  }
}

// Sandwich-normalised residual step and the next sublayer's input in one pass over the row:
//   x <- x + out_scale * y / rms(y) * (w_post + off);   h = x / rms(x) * (w_pre + off)   (h in its own type)
// A thread re-reads only what it wrote itself, so the row needs no fence between the passes.
__global__ void __launch_bounds__(256) residual_norm_rows_kernel(float* x, int64_t ldx, const float* y, int64_t ldy, const void* w_post,
                                                                 const void* w_pre, int w_dtype, float w_offset, float eps,
                                                                 float out_scale, void* h, int h_dtype, int64_t ldh, int cols) {
  __shared__ float red[8];
  __shared__ float inv_s;
  const int row = blockIdx.x;
  const float* yr = y + (int64_t) row * ldy;
  float* xr = x + (int64_t) row * ldx;
  auto block_inv = [&](float ss) {
    ss = warp_sum(ss);
    __syncthreads();                               // red / inv_s of the previous reduction have been read
    if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float v = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
      v = warp_sum(v);
      if (threadIdx.x == 0) inv_s = 1.f / sqrtf(v / (float) cols + eps);
    }
    __syncthreads();
    return inv_s;
  };
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float v = yr[c]; ss = fmaf(v, v, ss); }
  const float inv_y = block_inv(ss);
  ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) {
    float v = yr[c] * inv_y;
    v *= ld_f(w_post, w_dtype, c) + w_offset;
    v = xr[c] + v * out_scale;
    xr[c] = v;
    ss = fmaf(v, v, ss);
  }
  const float inv_x = block_inv(ss);
  for (int c = threadIdx.x; c < cols; c += 256)
    st_f(h, h_dtype, (int64_t) row * ldh + c, xr[c] * inv_x * (ld_f(w_pre, w_dtype, c) + w_offset));
}

// Layer normalisation of fp32 rows with weight and bias: (x - mean) / sqrt(var + eps) * w + b, var = mean of the squared
// deviations (second pass over the row, not E[x^2] - mean^2).  Block sums run in a fixed tree.
__device__ __forceinline__ float block_sum_256(float v, float* red, float* bcast) {
  v = warp_sum(v);
  __syncthreads();                                 // red / bcast of the previous reduction have been read
  if (threadIdx.x % 32 == 0) red[threadIdx.x / 32] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) *bcast = t;
  }
  __syncthreads();
  return *bcast;
}

__global__ void __launch_bounds__(256) layernorm_rows_kernel(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi,
                                                             const void* w, const void* b, int w_dtype, float eps,
                                                             const int* rows_idx, int cols) {
  __shared__ float red[8];
  __shared__ float bc;
  const int row = blockIdx.x;
  const float* xr = x + (int64_t) (rows_idx ? rows_idx[row] : row) * ldi;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) s += xr[c];
  const float mean = block_sum_256(s, red, &bc) / (float) cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float d = xr[c] - mean; ss = fmaf(d, d, ss); }
  const float inv = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) cols + eps);
  for (int c = threadIdx.x; c < cols; c += 256) {
    float y = (xr[c] - mean) * inv * ld_f(w, w_dtype, c);
    if (b) y += ld_f(b, w_dtype, c);
    st_f(out, out_dtype, (int64_t) row * ldo + c, y);
  }
}

// Residual step of a layer whose sublayers all read ONE normalised input and are added together, with the next layer's
// input in the same pass: x <- x + out_scale * (y1 + y2);  h = layer_norm(x) (skipped when w is NULL).
// A thread re-reads only what it wrote itself, so the row needs no fence between the passes.
__global__ void __launch_bounds__(256) residual_layernorm_rows_kernel(float* x, int64_t ldx, const float* y1, int64_t ldy1,
                                                                      const float* y2, int64_t ldy2, float out_scale, const void* w,
                                                                      const void* b, int w_dtype, float eps, void* h, int h_dtype,
                                                                      int64_t ldh, int cols) {
  __shared__ float red[8];
  __shared__ float bc;
  const int row = blockIdx.x;
  float* xr = x + (int64_t) row * ldx;
  const float* ar = y1 + (int64_t) row * ldy1;
  const float* br = y2 ? y2 + (int64_t) row * ldy2 : nullptr;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) {
    float y = ar[c];
    if (br) y += br[c];
    const float v = fmaf(out_scale, y, xr[c]);
    xr[c] = v;
    s += v;
  }
  if (!w) return;
  const float mean = block_sum_256(s, red, &bc) / (float) cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float d = xr[c] - mean; ss = fmaf(d, d, ss); }
  const float inv = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) cols + eps);
  for (int c = threadIdx.x; c < cols; c += 256) {
    float y = (xr[c] - mean) * inv * ld_f(w, w_dtype, c);
    if (b) y += ld_f(b, w_dtype, c);
    st_f(h, h_dtype, (int64_t) row * ldh + c, y);
  }
}

// out[r] = [a[r, :cols_a] | b[r, :cols_b]] in out's type: the operand of a projection that reads two fp32 streams side by side
__global__ void concat_rows_kernel(void* out, int out_dtype, const float* a, int64_t lda, int cols_a, const float* b, int64_t ldb,
                                   int cols_b, int64_t n) {
  const int cols = cols_a + cols_b;
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
    const int64_t r = i / cols;
    const int c = (int) (i % cols);
    st_f(out, out_dtype, i, c < cols_a ? a[r * lda + c] : b[r * ldb + c - cols_a]);
  }
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// row_scale != NULL: gate and up values of row r are multiplied by row_scale[row_index ? row_index[r] : r] first (0 where the
// index is negative) — a routed expert whose score weighs its INPUT: the projections are linear, so the score moves behind them
__global__ void gated_act_kernel(void* out, int out_dtype, const float* gu, int64_t n, int ff, int gate, float alpha, float limit,
                                 float up_shift, const float* row_scale, const int* row_index) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
    const int64_t row = i / ff;
    const int j = (int) (i % ff);
    float g = gu[row * 2 * ff + j], u = gu[row * 2 * ff + ff + j];
    if (row_scale) {
      const int64_t r = row_index ? row_index[row] : row;
      const float sc = r >= 0 ? row_scale[r] : 0.f;
      g *= sc;
      u *= sc;
    }
    if (gate == TB_GATE_GELU_TANH) { st_f(out, out_dtype, i, gelu_tanh_f(g) * u); continue; }
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    const float sg = 1.f / (1.f + expf(-alpha * g));
    st_f(out, out_dtype, i, g * sg * (u + up_shift));
  }
}

// out[n, :] = table[ids[n], :] * scale + pair[row(n), :], row = (prev * mul_prev + id * mul_cur) mod buckets, or row `buckets`
// (the table's last) for a token without a predecessor (prev < 0): a hashed embedding of the (previous, current) pair
__global__ void embed_bigram_kernel(float* out, const void* table, const void* pair, int t_dtype, const int* ids, const int* prev,
                                    float scale, int width, int vocab, int buckets, int64_t mul_prev, int64_t mul_cur) {
  const int row = blockIdx.x;
  int id = ids[row];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const int pv = prev[row];
  const int64_t pr = pv < 0 ? buckets : (int64_t) (((int64_t) pv * mul_prev + (int64_t) id * mul_cur) % buckets);
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    out[(int64_t) row * width + c] = fmaf(ld_f(table, t_dtype, (int64_t) id * width + c), scale, ld_f(pair, t_dtype, pr * width + c));
}

// Residual step of a sublayer between two layer norms and the next sublayer's input in one pass over the row:
//   x <- x + out_scale * LN(y; w_post, b_post);   h = LN(x; w_pre, b_pre)   (skipped when w_pre is NULL)
// A thread re-reads only what it wrote itself, so the row needs no fence between the passes.
__global__ void __launch_bounds__(256) residual_sandwich_layernorm_kernel(float* x, int64_t ldx, const float* y, int64_t ldy,
                                                                          const void* w_post, const void* b_post, const void* w_pre,
                                                                          const void* b_pre, int w_dtype, float eps, float out_scale,
                                                                          void* h, int h_dtype, int64_t ldh, int cols) {
  __shared__ float red[8];
  __shared__ float bc;
  const int row = blockIdx.x;
  float* xr = x + (int64_t) row * ldx;
  const float* yr = y + (int64_t) row * ldy;
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) s += yr[c];
  const float mean_y = block_sum_256(s, red, &bc) / (float) cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float d = yr[c] - mean_y; ss = fmaf(d, d, ss); }
  const float inv_y = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) cols + eps);
  s = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) {
    float v = (yr[c] - mean_y) * inv_y * ld_f(w_post, w_dtype, c);
    if (b_post) v += ld_f(b_post, w_dtype, c);
    v = fmaf(out_scale, v, xr[c]);
    xr[c] = v;
    s += v;
  }
  if (!w_pre) return;
  const float mean = block_sum_256(s, red, &bc) / (float) cols;
  ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { const float d = xr[c] - mean; ss = fmaf(d, d, ss); }
  const float inv = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) cols + eps);
  for (int c = threadIdx.x; c < cols; c += 256) {
    float v = (xr[c] - mean) * inv * ld_f(w_pre, w_dtype, c);
    if (b_pre) v += ld_f(b_pre, w_dtype, c);
    st_f(h, h_dtype, (int64_t) row * ldh + c, v);
  }
}

// Per-layer token input (one CTA per row): e = the `sd` columns from e_off of side_embed[token]; g = gelu_tanh(W_gate x) * e;
// y = W_proj g; x <- x + y / rms(y) * norm_w; then, when w_pre is given, h = LN(x; w_pre, b_pre) or the RMS norm (b_pre NULL and
// pre_rms) of the NEXT layer.  Operands of the two products are rounded to the storage type (w_dtype) as a projection kernel
// would; sums, the norm and the residual are fp32.  Shared memory: x row [width] | g [sd] | y [width].
// y_in != NULL: the two products have been run as projections (prompt-sized steps) and y is read from there.
struct SideArgs {
  const float* y_in; int64_t ldy;
  float* x; int64_t ldx;
  const void* side_embed; int64_t lde; int e_off;
  const int* ids; int vocab;
  const void *w_gate, *w_proj, *norm_w;
  int w_dtype; float eps; int width, sd;
  const void *w_pre, *b_pre; int pre_rms; void* h; int h_dtype; int64_t ldh;
};
__device__ __forceinline__ float round_like(float v, int dtype) {
  return dtype == TB_DT_BF16 ? __bfloat162float(__float2bfloat16_rn(v)) : v;
}
__global__ void __launch_bounds__(256) token_side_input_kernel(SideArgs a) {
  extern __shared__ float sm[];
  __shared__ float red[8];
  __shared__ float bc;
  float* xs = sm;
  float* gs = xs + a.width;
  float* ys = gs + a.sd;
  const int row = blockIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float* xr = a.x + (int64_t) row * a.ldx;
  float ss = 0.f;
  if (a.y_in) {
    const float* yr = a.y_in + (int64_t) row * a.ldy;
    for (int c = threadIdx.x; c < a.width; c += 256) { const float v = yr[c]; ys[c] = v; ss = fmaf(v, v, ss); }
  } else {
    for (int c = threadIdx.x; c < a.width; c += 256) xs[c] = round_like(xr[c], a.w_dtype);
    __syncthreads();
    int id = a.ids[row];
    id = id < 0 ? 0 : (id >= a.vocab ? a.vocab - 1 : id);
    for (int j = warp; j < a.sd; j += 8) {
      float acc = 0.f;
      for (int c = lane; c < a.width; c += 32) acc = fmaf(ld_f(a.w_gate, a.w_dtype, (int64_t) j * a.width + c), xs[c], acc);
      acc = warp_sum(acc);
      if (lane == 0) gs[j] = round_like(gelu_tanh_f(acc) * ld_f(a.side_embed, a.w_dtype, (int64_t) id * a.lde + a.e_off + j), a.w_dtype);
    }
    __syncthreads();
    // a warp per output column, the column's sd weights (contiguous) over its lanes; every thread of the warp keeps the sum of
    // squares of the warp's columns, so the block sum below counts each column 32 times: divided out
    for (int c = warp; c < a.width; c += 8) {
      float acc = 0.f;
      for (int j = lane; j < a.sd; j += 32) acc = fmaf(ld_f(a.w_proj, a.w_dtype, (int64_t) c * a.sd + j), gs[j], acc);
      acc = warp_sum(acc);
      if (lane == 0) ys[c] = acc;
      ss = fmaf(acc, acc, ss);
    }
    ss *= 1.f / 32.f;
    __syncthreads();
  }
  const float inv_y = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) a.width + a.eps);
  float s = 0.f, s2 = 0.f;
  for (int c = threadIdx.x; c < a.width; c += 256) {
    const float v = fmaf(ys[c] * inv_y, ld_f(a.norm_w, a.w_dtype, c), xr[c]);
    xr[c] = v;
    ys[c] = v;
    s += v;
    s2 = fmaf(v, v, s2);
  }
  if (!a.w_pre) return;
  if (a.pre_rms) {
    const float inv = 1.f / sqrtf(block_sum_256(s2, red, &bc) / (float) a.width + a.eps);
    for (int c = threadIdx.x; c < a.width; c += 256) st_f(a.h, a.h_dtype, (int64_t) row * a.ldh + c, ys[c] * inv * ld_f(a.w_pre, a.w_dtype, c));
    return;
  }
  const float mean = block_sum_256(s, red, &bc) / (float) a.width;
  ss = 0.f;
  for (int c = threadIdx.x; c < a.width; c += 256) { const float d = ys[c] - mean; ss = fmaf(d, d, ss); }
  const float inv = 1.f / sqrtf(block_sum_256(ss, red, &bc) / (float) a.width + a.eps);
  for (int c = threadIdx.x; c < a.width; c += 256) {
    float v = (ys[c] - mean) * inv * ld_f(a.w_pre, a.w_dtype, c);
    if (a.b_pre) v += ld_f(a.b_pre, a.w_dtype, c);
    st_f(a.h, a.h_dtype, (int64_t) row * a.ldh + c, v);
  }
}

// g[n, j] = gelu_tanh(z[n, j]) * side_embed[ids[n], e_off + j] in g's type: between the two projections of the per-layer token
// input when they run as prompt-sized products
__global__ void side_gate_mul_kernel(void* g, int g_dtype, const float* z, int64_t ldz, const void* side_embed, int e_dtype, int64_t lde,
                                     int e_off, const int* ids, int vocab, int sd, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
    const int64_t row = i / sd;
    const int j = (int) (i % sd);
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    st_f(g, g_dtype, i, gelu_tanh_f(z[row * ldz + j]) * ld_f(side_embed, e_dtype, (int64_t) id * lde + e_off + j));
  }
}

// out = out_scale * (a / rms(a) * wa + b / rms(b) * wb): two streams side by side, each RMS-normalised with its own weight
__global__ void __launch_bounds__(256) rmsnorm_pair_sum_kernel(float* out, int64_t ldo, const float* a, int64_t lda, const float* b,
                                                               int64_t ldb, const void* wa, const void* wb, int w_dtype, float eps,
                                                               float out_scale, int cols) {
  __shared__ float red[8];
  __shared__ float bc;
  const int row = blockIdx.x;
  const float* ar = a + (int64_t) row * lda;
  const float* br = b + (int64_t) row * ldb;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < cols; c += 256) { sa = fmaf(ar[c], ar[c], sa); sb = fmaf(br[c], br[c], sb); }
  const float ia = 1.f / sqrtf(block_sum_256(sa, red, &bc) / (float) cols + eps);
  const float ib = 1.f / sqrtf(block_sum_256(sb, red, &bc) / (float) cols + eps);
  for (int c = threadIdx.x; c < cols; c += 256)
    out[(int64_t) row * ldo + c] = out_scale * (ar[c] * ia * ld_f(wa, w_dtype, c) + br[c] * ib * ld_f(wb, w_dtype, c));
}

// fp32 rows (row stride ld) -> contiguous bf16: the residual stream as the operand of a tcgen05 projection
__global__ void cast_rows_bf16_kernel(__nv_bfloat16* out, const float* x, int64_t ld, int cols, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(x[(i / cols) * ld + i % cols]);
}

// factor > 0: wavelengths above original / low turn `factor` times slower, those below original / high are kept, and the
// band between is blended linearly in original / wavelength
__global__ void rope_table_kernel(float* table, const int* tok_pos, int rows, int half, int dims, double base, double factor,
                                  double low, double high, double original) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * half) return;
  const int row = i / half, f = i % half;
  double freq = pow(base, -2.0 * (double) f / (double) dims);
  if (factor > 0.0) {
    const double wavelength = 6.283185307179586476925 / freq;
    if (wavelength > original / low) {
      freq /= factor;
    } else if (!(wavelength < original / high)) {
      const double keep = (original / wavelength - low) / (high - low);     // 0 at the slow end of the band, 1 at the fast end
      freq *= keep + (1.0 - keep) / factor;
    }
  }
  double s, c;
  sincos((double) tok_pos[row] * freq, &s, &c);
  table[2 * (int64_t) i] = (float) c;
  table[2 * (int64_t) i + 1] = (float) s;
}

// x[r, :] += vec — the vector a pass of a looped block adds to the residual stream before its first layer
__global__ void add_row_vector_kernel(float* x, int64_t ld, const void* vec, int v_dtype, int cols, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
    x[(i / cols) * ld + i % cols] += ld_f(vec, v_dtype, i % cols);
}

// x <- cap * tanh(x / cap): soft cap of the logits
__global__ void tanh_cap_kernel(float* x, int64_t n, float cap) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

__global__ void rope_query_tail_kernel(void* qa, int dtype, const float* q, const float* table, int rows, int heads, int dim,
                                       int rot_dim, int dims, int lat) {
  // one thread per (row, head, pair-or-passthrough element)
  const int per = rot_dim - dims / 2;            // dims/2 pairs + (rot_dim - dims) unrotated elements
  const int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
  if (i >= (int64_t) rows * heads * per) return;
  const int e = (int) (i % per);
  const int64_t rh = i / per;
  const int row = (int) (rh / heads);
  const float* src = q + rh * (dim + rot_dim) + dim;
  const int64_t dst = rh * (lat + rot_dim) + lat;
  if (e < dims / 2) {
    const float c = table[((int64_t) row * (dims / 2) + e) * 2], s = table[((int64_t) row * (dims / 2) + e) * 2 + 1];
    const float u = src[2 * e], v = src[2 * e + 1];
    st_f(qa, dtype, dst + 2 * e, u * c - v * s);
    st_f(qa, dtype, dst + 2 * e + 1, v * c + u * s);
  } else {
    const int j = dims + (e - dims / 2);
    st_f(qa, dtype, dst + j, src[j]);
  }
}

}  // namespace
}  // namespace tb

using namespace tb;
static inline bool dt_ok(int d) { return d == TB_DT_F32 || d == TB_DT_BF16; }

extern "C" int tb_embed_scaled(float* out, const void* table, int t_dtype, const int* ids, float scale, int rows, int width,
                               int vocab, tb_stream_t stream) {
  if (!out || !table || !ids || !dt_ok(t_dtype) || width <= 0 || vocab <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  embed_scaled_kernel<<<rows, 128, 0, (cudaStream_t) stream>>>(out, table, t_dtype, ids, scale, width, vocab);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rmsnorm_rows(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi, const void* w, int w_dtype,
                               float w_offset, float eps, const int* rows_idx, int rows, int cols, int accumulate,
                               float out_scale, tb_stream_t stream) {
  if (!out || !x || !dt_ok(out_dtype) || (w && !dt_ok(w_dtype)) || cols <= 0 || rows < 0) return -1;
  if (accumulate && out_dtype != TB_DT_F32) return -2;
  if (rows == 0) return 0;
  rmsnorm_rows_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(out, out_dtype, ldo, x, ldi, w, w_dtype, w_offset, eps,
                                                               rows_idx, cols, accumulate, out_scale);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_residual_norm_rows(float* x, int64_t ldx, const float* y, int64_t ldy, const void* w_post, const void* w_pre,
                                     int w_dtype, float w_offset, float eps, float out_scale, void* h, int h_dtype, int64_t ldh,
                                     int rows, int cols, tb_stream_t stream) {
  if (!x || !y || !w_post || !w_pre || !h || !dt_ok(w_dtype) || !dt_ok(h_dtype) || cols <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  residual_norm_rows_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(x, ldx, y, ldy, w_post, w_pre, w_dtype, w_offset, eps,
                                                                     out_scale, h, h_dtype, ldh, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_layernorm_rows(void* out, int out_dtype, int64_t ldo, const float* x, int64_t ldi, const void* w, const void* b,
                                 int w_dtype, float eps, const int* rows_idx, int rows, int cols, tb_stream_t stream) {
  if (!out || !x || !w || !dt_ok(out_dtype) || !dt_ok(w_dtype) || cols <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  layernorm_rows_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(out, out_dtype, ldo, x, ldi, w, b, w_dtype, eps, rows_idx, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_residual_layernorm_rows(float* x, int64_t ldx, const float* y1, int64_t ldy1, const float* y2, int64_t ldy2,
                                          float out_scale, const void* w, const void* b, int w_dtype, float eps, void* h, int h_dtype,
                                          int64_t ldh, int rows, int cols, tb_stream_t stream) {
  if (!x || !y1 || cols <= 0 || rows < 0) return -1;
  if (w && (!h || !dt_ok(w_dtype) || !dt_ok(h_dtype))) return -1;
  if (rows == 0) return 0;
  residual_layernorm_rows_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(x, ldx, y1, ldy1, y2, ldy2, out_scale, w, b, w_dtype, eps,
                                                                          h, h_dtype, ldh, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_concat_rows(void* out, int out_dtype, const float* a, int64_t lda, int cols_a, const float* b, int64_t ldb,
                              int cols_b, int rows, tb_stream_t stream) {
  if (!out || !a || !b || !dt_ok(out_dtype) || cols_a <= 0 || cols_b <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * (cols_a + cols_b);
  const int grid = (int) ((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  concat_rows_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(out, out_dtype, a, lda, cols_a, b, ldb, cols_b, n);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_gated_act(void* out, int out_dtype, const float* gu, int rows, int ff, int gate, float alpha, float limit,
                            float up_shift, const float* row_scale, const int* row_index, tb_stream_t stream) {
  if (!out || !gu || !dt_ok(out_dtype) || ff <= 0 || rows < 0 || (gate != TB_GATE_SIGMOID && gate != TB_GATE_GELU_TANH)) return -1;
  if (row_index && !row_scale) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * ff;
  const int grid = (int) ((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  gated_act_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(out, out_dtype, gu, n, ff, gate, alpha, limit, up_shift, row_scale, row_index);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_embed_bigram(float* out, const void* table, const void* pair, int t_dtype, const int* ids, const int* prev_ids,
                               float scale, int rows, int width, int vocab, int buckets, int mul_prev, int mul_cur,
                               tb_stream_t stream) {
  if (!out || !table || !pair || !ids || !prev_ids || !dt_ok(t_dtype) || width <= 0 || vocab <= 0 || buckets <= 0 || rows < 0 ||
      mul_prev < 0 || mul_cur < 0)
    return -1;
  if (rows == 0) return 0;
  embed_bigram_kernel<<<rows, 128, 0, (cudaStream_t) stream>>>(out, table, pair, t_dtype, ids, prev_ids, scale, width, vocab, buckets,
                                                               mul_prev, mul_cur);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_residual_sandwich_layernorm_rows(float* x, int64_t ldx, const float* y, int64_t ldy, const void* w_post,
                                                   const void* b_post, const void* w_pre, const void* b_pre, int w_dtype, float eps,
                                                   float out_scale, void* h, int h_dtype, int64_t ldh, int rows, int cols,
                                                   tb_stream_t stream) {
  if (!x || !y || !w_post || !dt_ok(w_dtype) || cols <= 0 || rows < 0) return -1;
  if (w_pre && (!h || !dt_ok(h_dtype))) return -1;
  if (rows == 0) return 0;
  residual_sandwich_layernorm_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(x, ldx, y, ldy, w_post, b_post, w_pre, b_pre, w_dtype,
                                                                              eps, out_scale, h, h_dtype, ldh, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_token_side_input(float* x, int64_t ldx, const float* y_in, int64_t ldy, const void* side_embed, int64_t lde, int e_off,
                                   const int* ids, int vocab, const void* w_gate, const void* w_proj, const void* norm_w, int w_dtype,
                                   float eps, int rows, int width, int sd, const void* w_pre, const void* b_pre, int pre_rms, void* h,
                                   int h_dtype, int64_t ldh, tb_stream_t stream) {
  if (!x || !norm_w || !dt_ok(w_dtype) || width <= 0 || sd <= 0 || rows < 0 || vocab <= 0 || e_off < 0) return -1;
  if (!y_in && (!side_embed || !ids || !w_gate || !w_proj)) return -1;
  if (w_pre && (!h || !dt_ok(h_dtype))) return -1;
  const size_t smem = ((size_t) 2 * width + sd) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (rows == 0) return 0;
  static size_t raised = 48 * 1024;
  if (smem > raised) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(token_side_input_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = smem;
  }
  SideArgs a{y_in, ldy, x, ldx, side_embed, lde, e_off, ids, vocab, w_gate, w_proj, norm_w, w_dtype, eps, width, sd, w_pre, b_pre,
             pre_rms, h, h_dtype, ldh};
  token_side_input_kernel<<<rows, 256, smem, (cudaStream_t) stream>>>(a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_side_gate_mul(void* g, int g_dtype, const float* z, int64_t ldz, const void* side_embed, int e_dtype, int64_t lde,
                                int e_off, const int* ids, int vocab, int rows, int sd, tb_stream_t stream) {
  if (!g || !z || !side_embed || !ids || !dt_ok(g_dtype) || !dt_ok(e_dtype) || rows < 0 || sd <= 0 || vocab <= 0 || e_off < 0) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * sd;
  const int grid = (int) ((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  side_gate_mul_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(g, g_dtype, z, ldz, side_embed, e_dtype, lde, e_off, ids, vocab, sd, n);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rmsnorm_pair_sum(float* out, int64_t ldo, const float* a, int64_t lda, const float* b, int64_t ldb, const void* wa,
                                   const void* wb, int w_dtype, float eps, float out_scale, int rows, int cols, tb_stream_t stream) {
  if (!out || !a || !b || !wa || !wb || !dt_ok(w_dtype) || cols <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  rmsnorm_pair_sum_kernel<<<rows, 256, 0, (cudaStream_t) stream>>>(out, ldo, a, lda, b, ldb, wa, wb, w_dtype, eps, out_scale, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_cast_rows_bf16(void* out, const float* x, int64_t ld, int rows, int cols, tb_stream_t stream) {
  if (!out || !x || cols <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * cols;
  const int grid = (int) ((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  cast_rows_bf16_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) out, x, ld, cols, n);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rope_table_scaled(float* table, const int* tok_pos, int rows, int dims, double base, double factor,
                                    double low, double high, double original, tb_stream_t stream) {
  if (!table || !tok_pos || dims <= 0 || dims % 2 || rows < 0 || !(base > 0.0)) return -1;
  if (factor > 0.0 && (!(low > 0.0) || !(high > low) || !(original > 0.0))) return -1;
  if (rows == 0) return 0;
  const int n = rows * (dims / 2);
  rope_table_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t) stream>>>(table, tok_pos, rows, dims / 2, dims, base, factor,
                                                                        low, high, original);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rope_table(float* table, const int* tok_pos, int rows, int dims, double base, tb_stream_t stream) {
  return tb_rope_table_scaled(table, tok_pos, rows, dims, base, 0.0, 0.0, 0.0, 0.0, stream);
}

extern "C" int tb_add_row_vector(float* x, int64_t ld, const void* vec, int v_dtype, int rows, int cols, tb_stream_t stream) {
  if (!x || !vec || !dt_ok(v_dtype) || cols <= 0 || rows < 0) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * cols;
  const int grid = (int) ((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  add_row_vector_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(x, ld, vec, v_dtype, cols, n);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_tanh_cap(float* x, int64_t n, float cap, tb_stream_t stream) {
  if (!x || n < 0 || !(cap > 0.f)) return -1;
  if (n == 0) return 0;
  const int grid = (int) ((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  tanh_cap_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(x, n, cap);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_rope_query_tail(void* qa, int dtype, const float* q, const float* table, int rows, int heads, int dim,
                                  int rot_dim, int dims, int lat, tb_stream_t stream) {
  if (!qa || !q || !table || !dt_ok(dtype) || heads <= 0 || dim < 0 || rot_dim <= 0 || dims <= 0 || dims % 2 ||
      dims > rot_dim || lat < 0 || rows < 0)
    return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * heads * (rot_dim - dims / 2);
  rope_query_tail_kernel<<<(unsigned) ((n + 255) / 256), 256, 0, (cudaStream_t) stream>>>(qa, dtype, q, table, rows, heads,
                                                                                           dim, rot_dim, dims, lat);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
