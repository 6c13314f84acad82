// Routed-expert feed-forward over a ragged batch: the router's choice, the plan that sorts (token, choice) pairs by
// expert, and the weighted sum of the chosen experts' outputs.  The expert products themselves are elsewhere: the tcgen05
// kernel in grouped mode (gemm_tc.cu, tb_gemm_tc_bf16_grouped) for prompt-sized bf16 steps, the tile kernels of tb_linear
// walking the plan (linear.cu, tb_moe_linear) for fp32, and one streaming product per pair (tb_moe_gemv) for generation steps.
//
//   moe_route_kernel    one warp per token: s = sigmoid(logit); choice = s + correction; experts form `groups` equal
//                       groups of neighbours, a group scores the sum of its two largest choices, only the `keep` best
//                       groups stay eligible; the `top` largest eligible choices are taken (ties: the lower index), and
//                       their weights are the plain s, not renormalised.  All fp32.  With neither correction nor
//                       groups the choice ranks the logits themselves (the same order, no saturation).
//   moe_route_softmax_kernel  one warp per token: s = softmax over all experts, the `top` largest, weights s / sum(chosen) * scale.
//   moe_plan_kernel     one CTA: pairs counted per expert, every expert's range padded to whole tiles of `tile` rows
//                       (so a tile never mixes experts), tile -> expert table, and sorted slot -> pair index (-1 in the
//                       padding).  Everything stays on the device: a replayed step graph re-plans with the same launch.
//   moe_gather_rows     the pairs' token rows in plan order as contiguous bf16 (the tcgen05 kernel's TMA operand).
//   moe_combine_kernel  out[n] = sum_k weight[n, k] * y[row of pair n * top + k], k in index order.
#include <cuda_bf16.h>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// arg-max over the warp's (value, index) candidates; ties go to the lower index; index -1 = no candidate
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi < i))) { v = ov; i = oi; }
  }
}

constexpr int kRouteWarps = 4;

// shared memory per warp: choice [E] | sigmoid [E] | state [E] (0 eligible, 1 masked, 2 taken) | group score [groups]
__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_kernel(int* ids, float* weights, const float* logits,
                                                                     const void* corr, int c_dtype, int rows, int E, int top,
                                                                     int groups, int keep) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int row = blockIdx.x * kRouteWarps + warp;
  if (row >= rows) return;
  float* choice = smem + (size_t) warp * (3 * E + groups);
  float* sig = choice + E;
  int* state = reinterpret_cast<int*>(sig + E);
  float* gscore = reinterpret_cast<float*>(state + E);
  // without a correction or groups the order of the scores is the order of the logits: ranking by the logit keeps apart
  // what the sigmoid rounds to one value in fp32 (above ~17 every score is 1)
  const bool by_logit = !corr && !(groups > 1 && keep < groups);
  for (int e = lane; e < E; e += 32) {
    const float z = logits[(int64_t) row * E + e];
    const float s = 1.f / (1.f + expf(-z));
    sig[e] = s;
    choice[e] = by_logit ? z : s + (corr ? ld_w(corr, c_dtype, e) : 0.f);
    state[e] = 0;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;              // the two largest of the group
      for (int e = g * per; e < (g + 1) * per; ++e) {
        const float c = choice[e];
        if (c > a) { b = a; a = c; } else if (c > b) b = c;
      }
      gscore[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    // mark everything masked, then free the `keep` best groups
    for (int e = lane; e < E; e += 32) state[e] = 1;
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY; int bi = -1;
      for (int g = lane; g < groups; g += 32) {
        const float v = gscore[g];
        if (v == v && state[g * per] == 1 && (bi < 0 || v > bv)) { bv = v; bi = g; }
      }
      warp_argmax(bv, bi);
      if (bi < 0) break;
      for (int e = bi * per + lane; e < (bi + 1) * per; e += 32) state[e] = 0;
      __syncwarp();
    }
  }
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY; int bi = -1;
    for (int e = lane; e < E; e += 32)
      if (state[e] == 0 && (bi < 0 || choice[e] > bv)) { bv = choice[e]; bi = e; }
    warp_argmax(bv, bi);
    if (bi < 0) {                                        // fewer eligible experts than `top`: fall back to masked ones
      for (int e = lane; e < E; e += 32)
        if (state[e] == 1 && (bi < 0 || choice[e] > bv)) { bv = choice[e]; bi = e; }
      warp_argmax(bv, bi);
    }
    if (lane == 0) {
      ids[(int64_t) row * top + k] = bi < 0 ? 0 : bi;
      weights[(int64_t) row * top + k] = bi < 0 ? 0.f : sig[bi];
      if (bi >= 0) state[bi] = 2;
    }
    __syncwarp();
  }
}

// Softmax router: s = softmax(logits) over ALL experts, the `top` largest are taken (ties: the lower index) and weighted by
// s / (sum of the chosen s + 1e-20) * scale (renorm) or s * scale.  One warp per token; shared memory per warp: s [E] | taken [E].
__global__ void __launch_bounds__(kRouteWarps * 32) moe_route_softmax_kernel(int* ids, float* weights, const float* logits, int rows,
                                                                             int E, int top, int renorm, float scale) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int row = blockIdx.x * kRouteWarps + warp;
  if (row >= rows) return;
  float* sc = smem + (size_t) warp * 2 * E;
  int* taken = reinterpret_cast<int*>(sc + E);
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, logits[(int64_t) row * E + e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(logits[(int64_t) row * E + e] - mx);
    sc[e] = p;
    taken[e] = 0;
    sum += p;
  }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) sc[e] = sc[e] / sum;
  __syncwarp();
  float chosen = 0.f;                                   // sum of the chosen scores, in choice order (the same on every lane)
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY; int bi = -1;
    for (int e = lane; e < E; e += 32)
      if (!taken[e] && (bi < 0 || sc[e] > bv)) { bv = sc[e]; bi = e; }
    warp_argmax(bv, bi);
    if (lane == 0) {
      ids[(int64_t) row * top + k] = bi < 0 ? 0 : bi;
      if (bi >= 0) taken[bi] = 1;
    }
    chosen += bi < 0 ? 0.f : bv;
    __syncwarp();
  }
  __syncwarp();
  for (int k = lane; k < top; k += 32) {
    const float v = sc[ids[(int64_t) row * top + k]];
    weights[(int64_t) row * top + k] = renorm ? v / (chosen + 1e-20f) * scale : v * scale;
  }
}

// one CTA of 1024 threads; shared: count [E] | cursor [E]
__global__ void __launch_bounds__(1024) moe_plan_kernel(int* slot_pair, int* tile_expert, int* pair_slot, const int* ids, int pairs,
                                                        int E, int tile, int max_tiles) {
  extern __shared__ int sm_i[];
  int* count = sm_i;
  int* cursor = sm_i + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) tile_expert[t] = -1;
  for (int s = threadIdx.x; s < max_tiles * tile; s += blockDim.x) slot_pair[s] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int e = 0; e < E; ++e) {
      const int nt = (count[e] + tile - 1) / tile;
      cursor[e] = t * tile;
      for (int k = 0; k < nt && t + k < max_tiles; ++k) tile_expert[t + k] = e;
      t += nt;
    }
  }
  __syncthreads();
  // a pair's slot inside its expert's range is whatever the atomic hands out: every output row is computed from its own
  // input row alone, in a k order of its own, so the slot does not reach the result
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) {
      const int s = atomicAdd(&cursor[e], 1);
      if (s < max_tiles * tile) slot_pair[s] = p;
      if (pair_slot) pair_slot[p] = s < max_tiles * tile ? s : -1;
    } else if (pair_slot) {
      pair_slot[p] = -1;
    }
  }
}

__global__ void moe_combine_kernel(float* out, const float* y, const float* weights, const int* pair_slot, const float* add,
                                   int64_t n, int width, int top) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
    const int64_t row = i / width;
    const int c = (int) (i % width);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int64_t r = pair_slot ? pair_slot[row * top + k] : row * top + k;
      if (r >= 0) acc = weights ? fmaf(weights[row * top + k], y[r * width + c], acc) : acc + y[r * width + c];
    }
    out[i] = add ? acc + add[i] : acc;
  }
}

// xs[s, :] = bf16(x[slot_pair[s] / top, :]) (zeros in the padding): the pairs' token rows in plan order, as the contiguous
// operand the tcgen05 kernel loads by TMA
template <typename T>
__global__ void moe_gather_rows_kernel(__nv_bfloat16* xs, const T* x, int64_t ldx, const int* slot_pair, int top, int cols) {
  const int s = blockIdx.x;
  const int pair = slot_pair[s];
  __nv_bfloat16* dst = xs + (int64_t) s * cols;
  if (pair < 0) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) dst[c] = __float2bfloat16_rn(0.f);
    return;
  }
  const T* src = x + (int64_t) (pair / top) * ldx;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    if constexpr (sizeof(T) == 4) dst[c] = __float2bfloat16_rn(src[c]);
    else dst[c] = src[c];
  }
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_moe_route(int* ids, float* weights, const float* logits, const void* correction, int c_dtype, int rows,
                            int experts, int top, int groups, int keep, tb_stream_t stream) {
  if (!ids || !weights || !logits || rows < 0 || experts <= 0 || top <= 0 || top > experts || groups <= 0 ||
      experts % groups || keep <= 0 || keep > groups)
    return -1;
  if (correction && c_dtype != TB_DT_F32 && c_dtype != TB_DT_BF16) return -1;
  const size_t smem = (size_t) kRouteWarps * (3 * experts + groups) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  if (rows == 0) return 0;
  moe_route_kernel<<<(rows + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, (cudaStream_t) stream>>>(
      ids, weights, logits, correction, c_dtype, rows, experts, top, groups, keep);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_moe_route_softmax(int* ids, float* weights, const float* logits, int rows, int experts, int top, int renorm,
                                    float scale, tb_stream_t stream) {
  if (!ids || !weights || !logits || rows < 0 || experts <= 0 || top <= 0 || top > experts) return -1;
  const size_t smem = (size_t) kRouteWarps * 2 * experts * sizeof(float);
  if (smem > 48 * 1024) return -2;
  if (rows == 0) return 0;
  moe_route_softmax_kernel<<<(rows + kRouteWarps - 1) / kRouteWarps, kRouteWarps * 32, smem, (cudaStream_t) stream>>>(
      ids, weights, logits, rows, experts, top, renorm, scale);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_moe_plan_tiles(int pairs, int experts, int tile) {
  if (pairs < 0 || experts <= 0 || tile <= 0) return -1;
  const int full = (pairs + tile - 1) / tile;
  return full + (experts < pairs ? experts : pairs);      // every expert in use may end in one partly filled tile
}

extern "C" int tb_moe_plan(int* slot_pair, int* tile_expert, int* pair_slot, const int* ids, int pairs, int experts, int tile,
                           int max_tiles, tb_stream_t stream) {
  if (!slot_pair || !tile_expert || !ids || pairs < 0 || experts <= 0 || tile <= 0 || max_tiles < tb_moe_plan_tiles(pairs, experts, tile))
    return -1;
  if ((size_t) experts * 2 * sizeof(int) > 48 * 1024) return -2;
  if (pairs == 0) return 0;
  moe_plan_kernel<<<1, 1024, (size_t) experts * 2 * sizeof(int), (cudaStream_t) stream>>>(slot_pair, tile_expert, pair_slot, ids,
                                                                                         pairs, experts, tile, max_tiles);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_moe_gather_rows(void* xs, const void* x, int x_dtype, int64_t ldx, const int* slot_pair, int slots, int top,
                                  int cols, tb_stream_t stream) {
  if (!xs || !x || !slot_pair || slots < 0 || top <= 0 || cols <= 0 || (x_dtype != TB_DT_F32 && x_dtype != TB_DT_BF16)) return -1;
  if (slots == 0) return 0;
  if (x_dtype == TB_DT_F32)
    moe_gather_rows_kernel<float><<<slots, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) xs, (const float*) x, ldx, slot_pair, top, cols);
  else
    moe_gather_rows_kernel<__nv_bfloat16><<<slots, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) xs, (const __nv_bfloat16*) x, ldx,
                                                                                    slot_pair, top, cols);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_moe_combine(float* out, const float* y, const float* weights, const int* pair_slot, int rows, int width, int top,
                              tb_stream_t stream) {
  return tb_moe_combine_add(out, y, weights, pair_slot, nullptr, rows, width, top, stream);
}

extern "C" int tb_moe_combine_add(float* out, const float* y, const float* weights, const int* pair_slot, const float* add, int rows,
                                  int width, int top, tb_stream_t stream) {
  if (!out || !y || rows < 0 || width <= 0 || top <= 0) return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * width;
  const int grid = (int) ((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  moe_combine_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(out, y, weights, pair_slot, add, n, width, top);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
