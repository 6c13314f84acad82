// Dense projections of the ragged-batch models: C = act(A W^T + bias) with bf16 or fp32 storage and fp32 accumulation.
//
//   linear_mma_kernel   bf16 weights on tensor cores (mma.sync m16n8k16 bf16, fp32 accumulators); A may arrive as fp32
//                       (the residual stream) and is rounded to bf16 while it is staged in shared memory, so no separate
//                       cast pass runs in front of a projection.  64 x 64 x 32 tiles, 4 warps of 32 x 32.
//   linear_fma_kernel   fp32 multiply-add with every product taken in fp32 (no TF32, no split-K): the all-32-bit mode and
//                       the small block-diagonal products that feed a recurrence.  64 x 64 x 16 tiles, 4 x 4 per thread.
//
//   linear_gemv_kernel  bf16 weights, at most 8 rows (generation steps): the step is bound by reading W once, so one warp
//                       owns an output column, streams its weight row with 16-byte loads (4 in flight per lane) against
//                       the rows staged once per CTA in shared memory as bf16, and reduces with shuffles.  Rows are
//                       dealt to the warps of the whole grid round-robin, so the chip reads one contiguous window of W.
//
//   linear_dot_kernel   few output columns in fp32 (a router's logits): one CTA per row, 16 columns at a time in registers.
//
// All walk k in one fixed order per output element, so a token's result is the same wherever it stands in a batch.
// blockIdx.z walks a batch of independent problems (per-head absorbed projections, block-diagonal gates).
// Routed experts use the same kernels: the tile kernels walk a plan that maps tile rows to (token, choice) pairs and tiles
// to experts (tb_moe_linear), the streaming kernel runs one pair per batch element against its expert (tb_moe_gemv).
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float gelu_tanh(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == TB_ACT_GELU_TANH) return gelu_tanh(v);
  if (act == TB_ACT_RELU_SQUARED) { v = fmaxf(v, 0.f); return v * v; }
  return v;
}

struct LinArgs {
  void* c; const void* a; const void* w; const void* bias;
  int64_t ldc, c_bs, lda, a_bs, w_bs, bias_bs;
  int M, N, K, act;
  float alpha, limit, up_shift;      // TB_ACT_GATED (GEMV only): W holds N gate rows, then N up rows
  // routed experts (tb_moe_linear): tile blockIdx.y belongs to expert tile_expert[blockIdx.y] (< 0: nothing to do) whose
  // weights are batch element `expert` of W; tile row gm is slot gm of the plan, slot_pair[gm] its (token, choice) pair
  // (< 0: padding).  A row = pair / a_div when a_div > 0 (the token's row), else the slot; C row = the pair when
  // c_by_pair, else the slot.
  const int* tile_expert; const int* slot_pair; int a_div, c_by_pair;
  // TB_ACT_GATED: which gated activation (TB_GATE_*), and an optional factor per batch element on gate and up before it (a
  // routed expert whose score weighs its input: the pair's score, applied behind the linear projections)
  int gate; const float* row_scale;
};

// row of A and of C behind tile row gm (-1: none)
__device__ __forceinline__ void lin_rows(const LinArgs& p, int gm, int& ar, int& cr) {
  if (gm >= p.M) { ar = cr = -1; return; }
  if (!p.slot_pair) { ar = cr = gm; return; }
  const int pair = p.slot_pair[gm];
  if (pair < 0) { ar = cr = -1; return; }
  ar = p.a_div > 0 ? pair / p.a_div : gm;
  cr = p.c_by_pair ? pair : gm;
}

// ---------------------------------------------------------------------------------------------------------------
template <typename AT, typename WT, typename CT>
__global__ void __launch_bounds__(256) linear_fma_kernel(LinArgs p) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int a_rows[BM], c_rows[BM];
  int b = blockIdx.z;
  if (p.tile_expert) { b = p.tile_expert[blockIdx.y]; if (b < 0) return; }
  const AT* A = reinterpret_cast<const AT*>(p.a) + (int64_t) b * p.a_bs;
  const WT* W = reinterpret_cast<const WT*>(p.w) + (int64_t) b * p.w_bs;
  CT* C = reinterpret_cast<CT*>(p.c) + (int64_t) b * p.c_bs;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;      // thread -> 4 rows (ty) x 4 cols (tx)
  if (threadIdx.x < BM) lin_rows(p, m0 + threadIdx.x, a_rows[threadIdx.x], c_rows[threadIdx.x]);
  __syncthreads();
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += BK) {
    // 64 x 16 elements per operand, 256 threads: 4 each; k fastest so global reads run along the rows
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int r = e / BK, k = e % BK;
      const int gm = a_rows[r], gn = n0 + r, gk = k0 + k;
      As[k][r] = (gm >= 0 && gk < p.K) ? to_f<AT>(A[(int64_t) gm * p.lda + gk]) : 0.f;
      Ws[k][r] = (gn < p.N && gk < p.K) ? to_f<WT>(W[(int64_t) gn * p.K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const WT* bias = p.bias ? reinterpret_cast<const WT*>(p.bias) + (int64_t) b * p.bias_bs : nullptr;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = c_rows[ty * 4 + i];
    if (gm < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      float v = acc[i][j];
      if (bias) v += to_f<WT>(bias[gn]);
      v = apply_act(v, p.act);
      C[(int64_t) gm * p.ldc + gn] = from_f<CT>(v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Few output columns (a router's logits): one CTA per ROW, 16 columns at a time in registers; the 256 threads stride over
// k in fp32 multiply-adds, then the partial sums are added in a fixed tree (lanes, then the eight warps in order).  The row is
// read once per 16 columns and W stays in L1 / L2 — the tile kernel above would leave all but a handful of SMs idle here.
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

template <typename AT, typename WT, typename CT>
__global__ void __launch_bounds__(256) linear_dot_kernel(LinArgs p, int vec) {
  __shared__ float part[8][16];
  const int m = blockIdx.x, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const AT* A = reinterpret_cast<const AT*>(p.a) + (int64_t) m * p.lda;
  const WT* W = reinterpret_cast<const WT*>(p.w);
  for (int n0 = 0; n0 < p.N; n0 += 16) {
    float acc[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] = 0.f;
    if (vec) {               // 8 | K, 16-byte aligned rows: a thread takes 8 consecutive k per trip
      for (int k = threadIdx.x * 8; k < p.K; k += 256 * 8) {
        float av[8];
        load8(A + k, av);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (n0 + j >= p.N) break;
          float wv[8];
          load8(W + (int64_t) (n0 + j) * p.K + k, wv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(av[i], wv[i], acc[j]);
        }
      }
    } else {
      for (int k = threadIdx.x; k < p.K; k += 256) {
        const float av = to_f<AT>(A[k]);
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (n0 + j < p.N) acc[j] = fmaf(av, to_f<WT>(W[(int64_t) (n0 + j) * p.K + k]), acc[j]);
      }
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float v = warp_sum(acc[j]);
      if (lane == 0) part[warp][j] = v;
    }
    __syncthreads();
    if (threadIdx.x < 16 && n0 + threadIdx.x < p.N) {
      float r = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) r += part[w][threadIdx.x];
      if (p.bias) r += to_f<WT>(reinterpret_cast<const WT*>(p.bias)[n0 + threadIdx.x]);
      reinterpret_cast<CT*>(p.c)[(int64_t) m * p.ldc + n0 + threadIdx.x] = from_f<CT>(apply_act(r, p.act));
    }
    __syncthreads();
  }
}

template <typename AT, typename WT>
int launch_dot(const LinArgs& p, int c_dtype, cudaStream_t s) {
  const int vec = p.K % 8 == 0 && (uintptr_t) p.a % 16 == 0 && (uintptr_t) p.w % 16 == 0 && (p.lda * sizeof(AT)) % 16 == 0;
  if (c_dtype == TB_DT_F32) linear_dot_kernel<AT, WT, float><<<p.M, 256, 0, s>>>(p, vec);
  else linear_dot_kernel<AT, WT, __nv_bfloat16><<<p.M, 256, 0, s>>>(p, vec);
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename AT, typename CT>
__global__ void __launch_bounds__(128) linear_mma_kernel(LinArgs p, int vec_a, int vec_w) {
  constexpr int BM = 64, BN = 64, BK = 32, LD = BK + 8;       // 80-byte rows: fragment reads hit 32 distinct banks
  __shared__ __align__(16) __nv_bfloat16 As[BM][LD];
  __shared__ __align__(16) __nv_bfloat16 Ws[BN][LD];
  __shared__ int a_rows[BM], c_rows[BM];
  int b = blockIdx.z;
  if (p.tile_expert) { b = p.tile_expert[blockIdx.y]; if (b < 0) return; }
  const AT* A = reinterpret_cast<const AT*>(p.a) + (int64_t) b * p.a_bs;
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.w) + (int64_t) b * p.w_bs;
  CT* C = reinterpret_cast<CT*>(p.c) + (int64_t) b * p.c_bs;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int wm = (warp / 2) * 32, wn = (warp % 2) * 32;
  const int g = lane / 4, t = lane % 4;
  if (threadIdx.x < BM) lin_rows(p, m0 + threadIdx.x, a_rows[threadIdx.x], c_rows[threadIdx.x]);
  __syncthreads();
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
    // stage A: 64 rows x 32 k = 256 groups of 8 elements, 2 per thread
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int e = threadIdx.x + it * 128;
      const int r = e / 4, kc = (e % 4) * 8;
      const int gm = a_rows[r], gk = k0 + kc;
      __align__(16) __nv_bfloat16 v[8];
      if (gm >= 0 && vec_a && gk + 8 <= p.K) {
        const AT* src = A + (int64_t) gm * p.lda + gk;
        if constexpr (sizeof(AT) == 4) {
          const float4 f0 = reinterpret_cast<const float4*>(src)[0], f1 = reinterpret_cast<const float4*>(src)[1];
          v[0] = __float2bfloat16_rn(f0.x); v[1] = __float2bfloat16_rn(f0.y); v[2] = __float2bfloat16_rn(f0.z);
          v[3] = __float2bfloat16_rn(f0.w); v[4] = __float2bfloat16_rn(f1.x); v[5] = __float2bfloat16_rn(f1.y);
          v[6] = __float2bfloat16_rn(f1.z); v[7] = __float2bfloat16_rn(f1.w);
        } else {
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (gm >= 0 && gk + j < p.K) ? __float2bfloat16_rn(to_f<AT>(A[(int64_t) gm * p.lda + gk + j]))
                                            : __float2bfloat16_rn(0.f);
      }
      *reinterpret_cast<uint4*>(&As[r][kc]) = *reinterpret_cast<const uint4*>(v);
    }
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int e = threadIdx.x + it * 128;
      const int r = e / 4, kc = (e % 4) * 8;
      const int gn = n0 + r, gk = k0 + kc;
      __align__(16) __nv_bfloat16 v[8];
      if (gn < p.N && vec_w && gk + 8 <= p.K) {
        *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(W + (int64_t) gn * p.K + gk);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          v[j] = (gn < p.N && gk + j < p.K) ? W[(int64_t) gn * p.K + gk + j] : __float2bfloat16_rn(0.f);
      }
      *reinterpret_cast<uint4*>(&Ws[r][kc]) = *reinterpret_cast<const uint4*>(v);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[2][4], bf[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + g;
        af[i][0] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * t]);
        af[i][1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * t]);
        af[i][2] = *reinterpret_cast<const uint32_t*>(&As[r][kk + 2 * t + 8]);
        af[i][3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = wn + j * 8 + g;
        bf[j][0] = *reinterpret_cast<const uint32_t*>(&Ws[c][kk + 2 * t]);
        bf[j][1] = *reinterpret_cast<const uint32_t*>(&Ws[c][kk + 2 * t + 8]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j]);
    }
    __syncthreads();
  }
  const __nv_bfloat16* bias = p.bias ? reinterpret_cast<const __nv_bfloat16*>(p.bias) + (int64_t) b * p.bias_bs : nullptr;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int gm = c_rows[wm + i * 16 + g + (k >= 2 ? 8 : 0)];
        const int gn = n0 + wn + j * 8 + 2 * t + (k & 1);
        if (gm < 0 || gn >= p.N) continue;
        float v = acc[i][j][k];
        if (bias) v += __bfloat162float(bias[gn]);
        v = apply_act(v, p.act);
        C[(int64_t) gm * p.ldc + gn] = from_f<CT>(v);
      }
}


// ---------------------------------------------------------------------------------------------------------------
template <typename AT, typename CT, int MR>
__global__ void __launch_bounds__(256) linear_gemv_kernel(LinArgs p, int vec_a) {
  extern __shared__ __align__(16) __nv_bfloat16 a_s[];          // [MR][K]
  const int b = blockIdx.y;
  // routed experts, few pairs (tb_moe_gemv): batch element b is pair b — its token's row (b / a_div) against the weights
  // of expert tile_expert[b]
  const int ab = p.tile_expert && p.a_div > 0 ? b / p.a_div : b;
  const int wb = p.tile_expert ? p.tile_expert[b] : b;
  const AT* A = reinterpret_cast<const AT*>(p.a) + (int64_t) ab * p.a_bs;
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(p.w) + (int64_t) wb * p.w_bs;
  CT* C = reinterpret_cast<CT*>(p.c) + (int64_t) b * p.c_bs;
  const int K = p.K;
  if (vec_a) {
    // 8 elements per thread and trip, no divisions: the staging must stay small beside the weight rows a CTA streams
    for (int m = 0; m < MR; ++m) {
      for (int k = threadIdx.x * 8; k < K; k += 256 * 8) {
        __align__(16) __nv_bfloat16 v[8];
        if (m < p.M) {
          const AT* src = A + (int64_t) m * p.lda + k;
          if constexpr (sizeof(AT) == 4) {
            const float4 f0 = reinterpret_cast<const float4*>(src)[0], f1 = reinterpret_cast<const float4*>(src)[1];
            v[0] = __float2bfloat16_rn(f0.x); v[1] = __float2bfloat16_rn(f0.y); v[2] = __float2bfloat16_rn(f0.z);
            v[3] = __float2bfloat16_rn(f0.w); v[4] = __float2bfloat16_rn(f1.x); v[5] = __float2bfloat16_rn(f1.y);
            v[6] = __float2bfloat16_rn(f1.z); v[7] = __float2bfloat16_rn(f1.w);
          } else {
            *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(src);
          }
        } else {
          *reinterpret_cast<uint4*>(v) = make_uint4(0, 0, 0, 0);
        }
        *reinterpret_cast<uint4*>(a_s + m * K + k) = *reinterpret_cast<const uint4*>(v);
      }
    }
  } else {
    for (int e = threadIdx.x; e < MR * K; e += 256) {
      const int m = e / K, k = e - m * K;
      a_s[e] = m < p.M ? __float2bfloat16_rn(to_f<AT>(A[(int64_t) m * p.lda + k])) : __float2bfloat16_rn(0.f);
    }
  }
  __syncthreads();
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const __nv_bfloat16* bias = p.bias ? reinterpret_cast<const __nv_bfloat16*>(p.bias) + (int64_t) b * p.bias_bs : nullptr;
  for (int n = blockIdx.x * 8 + warp; n < p.N; n += gridDim.x * 8) {
    const __nv_bfloat16* wr = W + (int64_t) n * K;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    if (p.act == TB_ACT_GATED) {
      // gated feed-forward: the warp streams gate row n and up row n + N together and applies the activation itself,
      // so the [M, 2 N] intermediate never exists
      const __nv_bfloat16* ur = wr + (int64_t) p.N * K;
      float up[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) up[m] = 0.f;
#pragma unroll 2
      for (int k = lane * 8; k < K; k += 256) {
        const uint4 gv = __ldg(reinterpret_cast<const uint4*>(wr + k)), uv = __ldg(reinterpret_cast<const uint4*>(ur + k));
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 av = *reinterpret_cast<const uint4*>(a_s + m * K + k);
          const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(a2[j]), gw = __bfloat1622float2(g2[j]), uw = __bfloat1622float2(u2[j]);
            acc[m] = fmaf(gw.x, f.x, acc[m]);
            acc[m] = fmaf(gw.y, f.y, acc[m]);
            up[m] = fmaf(uw.x, f.x, up[m]);
            up[m] = fmaf(uw.y, f.y, up[m]);
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MR; ++m) { acc[m] = warp_sum(acc[m]); up[m] = warp_sum(up[m]); }
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          if (m >= p.M) break;
          float gq = acc[m], uq = up[m];
          if (p.row_scale) { const float sc = p.row_scale[b]; gq *= sc; uq *= sc; }
          if (p.gate == TB_GATE_GELU_TANH) { C[(int64_t) m * p.ldc + n] = from_f<CT>(gelu_tanh(gq) * uq); continue; }
          if (p.limit > 0.f) { gq = fminf(gq, p.limit); uq = fminf(fmaxf(uq, -p.limit), p.limit); }
          C[(int64_t) m * p.ldc + n] = from_f<CT>(gq * (1.f / (1.f + expf(-p.alpha * gq))) * (uq + p.up_shift));
        }
      }
      continue;
    }
#pragma unroll 4
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wr + k));
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float wf[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(w2[j]); wf[2 * j] = f.x; wf[2 * j + 1] = f.y; }
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const uint4 av = *reinterpret_cast<const uint4*>(a_s + m * K + k);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(a2[j]);
          acc[m] = fmaf(wf[2 * j], f.x, acc[m]);
          acc[m] = fmaf(wf[2 * j + 1], f.y, acc[m]);
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
      const float bv = bias ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        if (m >= p.M) break;
        float v = apply_act(acc[m] + bv, p.act);
        C[(int64_t) m * p.ldc + n] = from_f<CT>(v);
      }
    }
  }
}

template <typename AT, typename CT>
int launch_gemv(const LinArgs& p, int batch, cudaStream_t s) {
  const int mr = p.M <= 1 ? 1 : (p.M <= 2 ? 2 : (p.M <= 4 ? 4 : 8));
  const size_t smem = (size_t) mr * p.K * sizeof(__nv_bfloat16);
  // as many CTAs as stay resident (shared memory and threads), but no more warps than output columns: every CTA pays
  // for staging the rows once, so it should stream as many weight rows as the grid allows
  int ctas = (p.N + 7) / 8;
  const int resident = (int) std::min<size_t>(8, (220 * 1024) / std::max<size_t>(smem, 1024));
  const int cap = std::max(1, 148 * std::max(1, resident) / batch);
  if (ctas > cap) ctas = cap;
  dim3 grid(ctas, batch);
  const int asz = (int) sizeof(AT);
  const int vec_a = ((uintptr_t) p.a % 16 == 0) && (p.lda * asz % 16 == 0) && (p.a_bs * asz % 16 == 0);
#define TB_GEMV_CASE(MR)                                                                                             \
  case MR: {                                                                                                         \
    static size_t raised = 48 * 1024; /* the opt-in only ever grows, and only outside a replayed region */           \
    if (smem > raised) {                                                                                             \
      TB_CHECK_CUDA(cudaFuncSetAttribute(linear_gemv_kernel<AT, CT, MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int) smem));                                                               \
      raised = smem;                                                                                                 \
    }                                                                                                                \
    linear_gemv_kernel<AT, CT, MR><<<grid, 256, smem, s>>>(p, vec_a);                                                     \
    break;                                                                                                           \
  }
  switch (mr) { TB_GEMV_CASE(1) TB_GEMV_CASE(2) TB_GEMV_CASE(4) TB_GEMV_CASE(8) }
#undef TB_GEMV_CASE
  return 0;
}

template <typename AT, typename WT>
int launch_fma(const LinArgs& p, int c_dtype, dim3 grid, cudaStream_t s) {
  if (c_dtype == TB_DT_F32) linear_fma_kernel<AT, WT, float><<<grid, 256, 0, s>>>(p);
  else linear_fma_kernel<AT, WT, __nv_bfloat16><<<grid, 256, 0, s>>>(p);
  return 0;
}

}  // namespace
}  // namespace tb

extern "C" int tb_linear(void* c, int c_dtype, int64_t ldc, int64_t c_bs, const void* a, int a_dtype, int64_t lda,
                         int64_t a_bs, const void* w, int w_dtype, int64_t w_bs, const void* bias, int64_t bias_bs, int M,
                         int N, int K, int batch, int act, int compute, tb_stream_t stream) {
  using namespace tb;
  auto ok = [](int d) { return d == TB_DT_F32 || d == TB_DT_BF16; };
  if (!c || !a || !w || !ok(c_dtype) || !ok(a_dtype) || !ok(w_dtype) || N <= 0 || K <= 0 || batch <= 0 || M < 0) return -1;
  if (M == 0) return 0;
  if (batch > 65535 || (M + 63) / 64 > 65535) return -2;
  if (act == TB_ACT_GATED) return -1;      // tb_linear_gated
  LinArgs p{c, a, w, bias, ldc, c_bs, lda, a_bs, w_bs, bias_bs, M, N, K, act, 0.f, 0.f, 0.f, nullptr, nullptr, 0, 0};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
  if (compute == TB_COMPUTE_TILES && w_dtype != TB_DT_BF16) compute = TB_COMPUTE_AUTO;
  const bool gemv_ok = w_dtype == TB_DT_BF16 && compute == TB_COMPUTE_AUTO && M <= 8 && K % 8 == 0 && (uintptr_t) w % 16 == 0 &&
                       w_bs % 8 == 0 && (size_t) (M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8))) * K * 2 <= 200 * 1024 && batch <= 65535;
  if (gemv_ok) {
    int rc;
    if (a_dtype == TB_DT_F32) rc = c_dtype == TB_DT_F32 ? launch_gemv<float, float>(p, batch, s) : launch_gemv<float, __nv_bfloat16>(p, batch, s);
    else rc = c_dtype == TB_DT_F32 ? launch_gemv<__nv_bfloat16, float>(p, batch, s) : launch_gemv<__nv_bfloat16, __nv_bfloat16>(p, batch, s);
    if (rc) return rc;
  } else if (w_dtype == TB_DT_BF16 && (compute == TB_COMPUTE_AUTO || compute == TB_COMPUTE_TILES)) {
    const int asz = a_dtype == TB_DT_F32 ? 4 : 2;
    const int vec_a = ((uintptr_t) a % 16 == 0) && (lda * asz % 16 == 0) && (a_bs * asz % 16 == 0);
    const int vec_w = ((uintptr_t) w % 16 == 0) && (K % 8 == 0) && (w_bs % 8 == 0);
    if (a_dtype == TB_DT_F32) {
      if (c_dtype == TB_DT_F32) linear_mma_kernel<float, float><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
      else linear_mma_kernel<float, __nv_bfloat16><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
    } else {
      if (c_dtype == TB_DT_F32) linear_mma_kernel<__nv_bfloat16, float><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
      else linear_mma_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
    }
  } else if (batch == 1 && N <= 64) {
    if (w_dtype == TB_DT_BF16) {
      if (a_dtype == TB_DT_F32) launch_dot<float, __nv_bfloat16>(p, c_dtype, s);
      else launch_dot<__nv_bfloat16, __nv_bfloat16>(p, c_dtype, s);
    } else {
      if (a_dtype == TB_DT_F32) launch_dot<float, float>(p, c_dtype, s);
      else launch_dot<__nv_bfloat16, float>(p, c_dtype, s);
    }
  } else if (w_dtype == TB_DT_BF16) {
    if (a_dtype == TB_DT_F32) launch_fma<float, __nv_bfloat16>(p, c_dtype, grid, s);
    else launch_fma<__nv_bfloat16, __nv_bfloat16>(p, c_dtype, grid, s);
  } else {
    if (a_dtype == TB_DT_F32) launch_fma<float, float>(p, c_dtype, grid, s);
    else launch_fma<__nv_bfloat16, float>(p, c_dtype, grid, s);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_linear_gated(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w,
                               int w_dtype, int M, int ff, int K, int gate, float alpha, float limit, float up_shift,
                               tb_stream_t stream) {
  using namespace tb;
  if (!c || !a || !w || ff <= 0 || K <= 0 || M < 0 || (gate != TB_GATE_SIGMOID && gate != TB_GATE_GELU_TANH)) return -1;
  if ((c_dtype != TB_DT_F32 && c_dtype != TB_DT_BF16) || (a_dtype != TB_DT_F32 && a_dtype != TB_DT_BF16)) return -1;
  if (M == 0) return 0;
  // the fused form exists for the streaming kernel only: the caller runs projection + activation otherwise
  const int mr = M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8));
  if (w_dtype != TB_DT_BF16 || M > 8 || K % 8 || (uintptr_t) w % 16 || (size_t) mr * K * 2 > 200 * 1024) return -3;
  LinArgs p{c, a, w, nullptr, ldc, 0, lda, 0, 0, 0, M, ff, K, TB_ACT_GATED, alpha, limit, up_shift, nullptr, nullptr, 0, 0, gate, nullptr};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  if (a_dtype == TB_DT_F32) rc = c_dtype == TB_DT_F32 ? launch_gemv<float, float>(p, 1, s) : launch_gemv<float, __nv_bfloat16>(p, 1, s);
  else rc = c_dtype == TB_DT_F32 ? launch_gemv<__nv_bfloat16, float>(p, 1, s) : launch_gemv<__nv_bfloat16, __nv_bfloat16>(p, 1, s);
  if (rc) return rc;
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Expert products over a plan (tb_moe_plan): the tile kernels above, tile row -> plan slot.  w [experts, N, K];
// a_div > 0: A [tokens, K] and slot s reads row slot_pair[s] / a_div (the token of the pair); a_div == 0: A [slots, K].
// c_by_pair: C row = the pair's index ([pairs, N]); else C row = the slot ([max_tiles * 64, N]).  Padding slots are neither
// read nor written.  The tile height is 64 (TB_MOE_TILE).
extern "C" int tb_moe_linear(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w,
                             int w_dtype, const int* slot_pair, const int* tile_expert, int max_tiles, int a_div,
                             int c_by_pair, int N, int K, int act, int compute, tb_stream_t stream) {
  using namespace tb;
  auto ok = [](int d) { return d == TB_DT_F32 || d == TB_DT_BF16; };
  if (!c || !a || !w || !slot_pair || !tile_expert || !ok(c_dtype) || !ok(a_dtype) || !ok(w_dtype) || N <= 0 || K <= 0 ||
      max_tiles < 0 || a_div < 0 || act == TB_ACT_GATED)
    return -1;
  if (max_tiles == 0) return 0;
  if (max_tiles > 65535) return -2;
  LinArgs p{c, a, w, nullptr, ldc, 0, lda, 0, (int64_t) N * K, 0, max_tiles * 64, N, K, act, 0.f, 0.f, 0.f,
            tile_expert, slot_pair, a_div, c_by_pair};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((N + 63) / 64, max_tiles, 1);
  if (w_dtype == TB_DT_BF16 && compute != TB_COMPUTE_FMA32) {
    const int asz = a_dtype == TB_DT_F32 ? 4 : 2;
    const int vec_a = ((uintptr_t) a % 16 == 0) && (lda * asz % 16 == 0);
    const int vec_w = ((uintptr_t) w % 16 == 0) && (K % 8 == 0);
    if (a_dtype == TB_DT_F32) {
      if (c_dtype == TB_DT_F32) linear_mma_kernel<float, float><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
      else linear_mma_kernel<float, __nv_bfloat16><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
    } else {
      if (c_dtype == TB_DT_F32) linear_mma_kernel<__nv_bfloat16, float><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
      else linear_mma_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 128, 0, s>>>(p, vec_a, vec_w);
    }
  } else if (w_dtype == TB_DT_BF16) {
    if (a_dtype == TB_DT_F32) launch_fma<float, __nv_bfloat16>(p, c_dtype, grid, s);
    else launch_fma<__nv_bfloat16, __nv_bfloat16>(p, c_dtype, grid, s);
  } else {
    if (a_dtype == TB_DT_F32) launch_fma<float, float>(p, c_dtype, grid, s);
    else launch_fma<__nv_bfloat16, float>(p, c_dtype, grid, s);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// Expert products for a handful of (token, choice) pairs (generation steps): pair b is one single-row product of the
// streaming kernel against expert ids[b]'s weights, so only the chosen experts' weights are read and no plan is needed.
// a_div > 0: a [tokens, K], pair b reads row b / a_div; a_div == 0: a [pairs, K].  c [pairs, N] in pair order.
// act TB_ACT_GATED: w holds per expert N gate rows, then N up rows; c = the gated activation `gate` (TB_GATE_*) of them, both
// first multiplied by pair_scale[b] when that is given.
// Returns -3 when the shape is not one the streaming kernel takes.
extern "C" int tb_moe_gemv(void* c, int c_dtype, int64_t ldc, const void* a, int a_dtype, int64_t lda, const void* w, int w_dtype,
                           const int* ids, int pairs, int a_div, int N, int K, int act, int gate, float alpha, float limit,
                           float up_shift, const float* pair_scale, tb_stream_t stream) {
  using namespace tb;
  auto ok = [](int d) { return d == TB_DT_F32 || d == TB_DT_BF16; };
  if (!c || !a || !w || !ids || !ok(c_dtype) || !ok(a_dtype) || N <= 0 || K <= 0 || pairs < 0 || a_div < 0) return -1;
  if (pairs == 0) return 0;
  const int asz = a_dtype == TB_DT_F32 ? 4 : 2;
  if (w_dtype != TB_DT_BF16 || pairs > 65535 || K % 8 || (uintptr_t) w % 16 || (size_t) K * 2 > 200 * 1024 || (lda * asz) % 16 ||
      (uintptr_t) a % 16)
    return -3;
  const int64_t w_bs = (int64_t) (act == TB_ACT_GATED ? 2 : 1) * N * K;
  if (act == TB_ACT_GATED && gate != TB_GATE_SIGMOID && gate != TB_GATE_GELU_TANH) return -1;
  LinArgs p{c, a, w, nullptr, ldc, ldc, lda, lda, w_bs, 0, 1, N, K, act, alpha, limit, up_shift, ids, nullptr, a_div, 0, gate,
            act == TB_ACT_GATED ? pair_scale : nullptr};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int rc;
  if (a_dtype == TB_DT_F32) rc = c_dtype == TB_DT_F32 ? launch_gemv<float, float>(p, pairs, s) : launch_gemv<float, __nv_bfloat16>(p, pairs, s);
  else rc = c_dtype == TB_DT_F32 ? launch_gemv<__nv_bfloat16, float>(p, pairs, s) : launch_gemv<__nv_bfloat16, __nv_bfloat16>(p, pairs, s);
  if (rc) return rc;
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
