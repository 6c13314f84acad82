// Gated delta rule over a ragged in-flight batch: a recurrent layer whose state per head is a matrix S [dim, vdim] that
// decays, is corrected towards the value along the key, and is read with the query:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q.
// Everything here is fp32: the state, the unit-normalised queries and keys, beta, the decay and the read-out.
//
//   delta_prepare_kernel   one CTA per row over the stacked projection q | k | v | (further columns): short causal convolution over
//                          the row's portion and the sequence's carried inputs, SiLU, then per head x / sqrt(sum x^2 + eps_unit)
//                          for queries (times dim^-1/2) and keys; beta = sigmoid(b) and g = exp(-exp(A_log) softplus(a + dt_bias))
//                          per head.  A sequence that brings ONE row has its carried inputs moved on here.  Steps of few rows
//                          spread a row's channels over several CTAs.
//   delta_scan_kernel      the columns of S are independent recurrences: one warp per (sequence, head, value column), the lanes
//                          hold the column's `dim` state elements (dim / 32 each).  Per token two dot products are reduced over
//                          the lanes at once, a = S^T k and b = S^T q of the OLD state, and with k . q (computed when the
//                          token chunk is staged) the step is u = beta (v - g a), o = g b + u (k . q), S <- g S + k u: one
//                          reduction round per token instead of two dependent ones.  Tokens are staged through shared memory
//                          in chunks of 16.  State layout per slot: [heads][vdim][dim] (a column's elements are contiguous).
//                          For steps whose sequences bring a token or two (generation).
//   delta_scan_blocked_kernel   prompt portions: the same recurrence resolved EIGHT tokens at a time.  With S the state ahead of the
//                          block, D_j the product of the block's decays up to token j, and the block's own products
//                          KK_ij = k_i . k_j, KQ_ij = k_i . q_j (i <= j; delta_gram_kernel computes them once per query / key head):
//                              a_j = D_j (S^T k_j) + sum_{i<j} (D_j / D_i) KK_ij u_i,    u_j = beta_j (v_j - a_j),
//                              o_j = D_j (S^T q_j) + sum_{i<j} (D_j / D_i) KQ_ij u_i + KQ_jj u_j,
//                              S  <- D_7 S + sum_j (D_7 / D_j) k_j u_j^T.
//                          The u_j of a block solve a triangular system whose matrix is the same for every value column,
//                          (I + diag(beta) L) u = diag(beta) r with L_ji = (D_j / D_i) KK_ij (i < j) and r_j = v_j - D_j (S^T k_j),
//                          so delta_block_matrices_kernel inverts it once per (block, head): M = (I + diag(beta) L)^-1 diag(beta),
//                          W_ji = (D_j / D_i) KQ_ij.  Per column then u = M r and o = D (S^T q) + W u are short products without
//                          a dependent chain, the sixteen dot products against S are reduced over the lanes in ONE round per
//                          block, and the eight rank-one updates are one pass over the registers.  One warp per value column,
//                          chunks of 16 tokens through a two-stage cp.async ring.  Differs from the token-serial form only by
//                          fp32 rounding.
//   delta_scan_tiled_kernel    the same with FOUR columns per warp (steps with columns enough to fill the chip): see its comment.
//   delta_block_matrices_kernel   M, W, D_j and D_last / D_j per (block, head), one thread each.
//   delta_gram_kernel      KK and KQ of every block of eight rows of a portion (blocks count from the portion's first row).
//   gated_rmsnorm_heads    one warp per (row, head): o / sqrt(mean(o^2) + eps) * w * silu(gate), stored in the storage type.
#include <cuda_bf16.h>

#include <algorithm>

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
  for (int v = blockIdx.y * 8 + warp; v < 2 * a.G; v += 8 * gridDim.y) {
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
  for (int c = Cqk + blockIdx.y * 256 + threadIdx.x; c < C; c += 256 * gridDim.y) {
    ur[c] = conv_silu_at(a, st, C, c, pos, past, start);
    if (carry) move_on(c);
  }
  for (int h = threadIdx.x; h < a.H && blockIdx.y == 0; h += 256) {
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

__device__ __forceinline__ void cp_async_f(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(dst);
  const int n = valid ? 4 : 0;                        // 0 source bytes: the destination is zero-filled
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_f4(float* dst, const float* src, bool valid) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit_wait_all(bool commit) {
  if (commit) asm volatile("cp.async.commit_group;");
  else asm volatile("cp.async.wait_group 0;");
}

constexpr int kBlk = 8;          // tokens resolved at a time
constexpr int kBlkChunk = 16;    // tokens per staged chunk (two blocks)

// gram [rows][G][8][2]: for row j of its block and i <= j, k_i . k_j and k_i . q_j.  One CTA per (block, query / key head, sequence);
// a dot product per group of 8 lanes.
__global__ void __launch_bounds__(256) delta_gram_kernel(float* gram, ScanArgs a) {
  const int e = blockIdx.z, g = blockIdx.y, t0 = blockIdx.x * kBlk;
  const int len = a.seq_len[e], row0 = a.seq_start[e];
  if (t0 >= len) return;
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  const int grp = threadIdx.x / 8, l8 = threadIdx.x % 8;
  for (int idx = grp; idx < kBlk * kBlk * 2; idx += 32) {
    const int kind = idx & 1, i = (idx >> 1) % kBlk, j = (idx >> 1) / kBlk;
    const bool need = i <= j && t0 + j < len;                                // uniform over the group
    float s_ = 0.f;
    if (need) {
      const float* x = a.u + (int64_t) (row0 + t0 + i) * C + (a.G + g) * a.dim;
      const float* y = a.u + (int64_t) (row0 + t0 + j) * C + (kind ? g : a.G + g) * a.dim;
      for (int d = l8; d < a.dim; d += 8) s_ = fmaf(x[d], y[d], s_);
    }
    s_ += __shfl_xor_sync(0xffffffffu, s_, 4);
    s_ += __shfl_xor_sync(0xffffffffu, s_, 2);
    s_ += __shfl_xor_sync(0xffffffffu, s_, 1);
    if (need && l8 == 0) gram[(((int64_t) (row0 + t0 + j) * a.G + g) * kBlk + i) * 2 + kind] = s_;
  }
}

constexpr int kMatRow = 20;      // floats per (row, head): M_j. [8] | W_j. [8] | D_j | D_last / D_j | pad

// mats [rows][H][20]; one thread per (block of 8 rows, head, sequence).  R_ji = D_j / D_i is kept as a running product (no division).
__global__ void __launch_bounds__(128) delta_block_matrices_kernel(float* mats, const float* gram, ScanArgs a, int nblk, int seqs) {
  constexpr int T = kBlk;
  const int64_t id = (int64_t) blockIdx.x * 128 + threadIdx.x;
  if (id >= (int64_t) seqs * a.H * nblk) return;
  const int blk = (int) (id % nblk), h = (int) ((id / nblk) % a.H), e = (int) (id / ((int64_t) nblk * a.H));
  const int len = a.seq_len[e], row0 = a.seq_start[e], t0 = blk * T;
  if (t0 >= len) return;
  const int nv = min(T, len - t0), g = h / (a.H / a.G);
  float beta[T], dec[T], D[T], N[T][T], R[T][T];
#pragma unroll
  for (int j = 0; j < T; ++j) {
    const bool in = j < nv;
    beta[j] = in ? a.bg[(int64_t) (row0 + t0 + j) * 2 * a.H + h] : 0.f;
    dec[j] = in ? a.bg[(int64_t) (row0 + t0 + j) * 2 * a.H + a.H + h] : 1.f;
    D[j] = j ? D[j - 1] * dec[j] : dec[j];
  }
#pragma unroll
  for (int j = 0; j < T; ++j) {
    const float* gj = gram + ((int64_t) (row0 + t0 + (j < nv ? j : 0)) * a.G + g) * T * 2;      // [i][kk, kq] of row j
#pragma unroll
    for (int i = 0; i < T; ++i) {
      R[j][i] = i == j ? 1.f : (i < j ? R[j - 1 > i ? j - 1 : i][i] * dec[j] : 0.f);
      N[j][i] = i == j ? 1.f : 0.f;
    }
    // row j of (I + diag(beta) L)^-1:  N_j = e_j - beta_j sum_{i<j} L_ji N_i
#pragma unroll
    for (int i = 0; i < j; ++i) {
      const float l = j < nv ? beta[j] * R[j][i] * gj[i * 2] : 0.f;
#pragma unroll
      for (int c = 0; c <= i; ++c) N[j][c] = fmaf(-l, N[i][c], N[j][c]);
    }
    if (j < nv) {
      float* dst = mats + ((int64_t) (row0 + t0 + j) * a.H + h) * kMatRow;
#pragma unroll
      for (int i = 0; i < T; ++i) {
        dst[i] = i <= j ? N[j][i] * beta[i] : 0.f;
        dst[T + i] = i <= j ? R[j][i] * gj[i * 2 + 1] : 0.f;
      }
      dst[2 * T] = D[j];
    }
  }
#pragma unroll
  for (int j = 0; j < T; ++j) {
    if (j < nv) {
      // D_last / D_j as the product of the decays behind j
      float f = 1.f;
#pragma unroll
      for (int m = 0; m < T; ++m) f *= (m > j && m < nv) ? dec[m] : 1.f;
      mats[((int64_t) (row0 + t0 + j) * a.H + h) * kMatRow + 2 * T + 1] = f;
    }
  }
}

// One CTA = NW warps = NW * (32 / LPC) value columns of one (sequence, head).  A thread holds DPL state elements of its column:
// element i is dim index ((i / VEC) * LPC + sub) * VEC + i % VEC (VEC = 4 when DPL allows 16-byte shared loads), so that the
// lanes of a column read neighbouring pieces of a staged key row.  Staged rows are LDK = LPC * DPL >= dim floats wide, zero behind dim.
// Shared memory per stage: k [16][LDK] | q [16][LDK] | block matrices [16][20] | v [16][COLS].
template <int LPC, int DPL, int NW>
__global__ void __launch_bounds__(NW * 32) delta_scan_blocked_kernel(float* out, ScanArgs a, const float* mats, int vec4) {
  constexpr int T = kBlk, TCH = kBlkChunk, CPW = 32 / LPC, COLS = NW * CPW, LDK = LPC * DPL, VEC = DPL % 4 == 0 ? 4 : 1, NT = NW * 32;
  constexpr int MR = kMatRow, STAGE = 2 * TCH * LDK + TCH * MR + TCH * COLS;
  extern __shared__ __align__(16) float smem[];
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, sub = lane % LPC;
  const int cc = warp * CPW + lane / LPC, col = c0 + cc;
  const bool live = col < a.vdim;
  const int len = a.seq_len[e], past = a.seq_past[e], row0 = a.seq_start[e];
  const int jh = h / (a.H / a.G);                                            // the head's query / key head
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  auto dmap = [&](int i) { return ((i / VEC) * LPC + sub) * VEC + i % VEC; };
  float* sp = a.state + (((int64_t) a.seq_slot[e] * a.H + h) * a.vdim + (live ? col : 0)) * a.dim;
  float S[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = dmap(i);
    S[i] = (live && past > 0 && d < a.dim) ? sp[d] : 0.f;                    // a sequence at position 0 starts from zeros
  }
  // the padding behind dim is never written by the copies: zero it once in both stages
  for (int i = threadIdx.x; i < 2 * STAGE; i += NT) smem[i] = 0.f;
  __syncthreads();
  auto stage_in = [&](int c, int buf) {
    float* ks = smem + buf * STAGE;
    float* qs = ks + TCH * LDK;
    float* mw = qs + TCH * LDK;
    float* vs = mw + TCH * MR;
    const int t0 = c * TCH, nt = min(TCH, len - t0);
    const float* ub = a.u + (int64_t) (row0 + t0) * C;
    if (vec4) {
      const int per = a.dim / 4;
      for (int i = threadIdx.x; i < TCH * per; i += NT) {
        const int t = i / per, d = (i % per) * 4;
        const bool ok = t < nt;
        cp_async_f4(qs + t * LDK + d, ok ? ub + (int64_t) t * C + jh * a.dim + d : a.u, ok);
        cp_async_f4(ks + t * LDK + d, ok ? ub + (int64_t) t * C + (a.G + jh) * a.dim + d : a.u, ok);
      }
    } else {
      for (int i = threadIdx.x; i < TCH * a.dim; i += NT) {
        const int t = i / a.dim, d = i % a.dim;
        const bool ok = t < nt;
        cp_async_f(qs + t * LDK + d, ok ? ub + (int64_t) t * C + jh * a.dim + d : a.u, ok);
        cp_async_f(ks + t * LDK + d, ok ? ub + (int64_t) t * C + (a.G + jh) * a.dim + d : a.u, ok);
      }
    }
    for (int i = threadIdx.x; i < TCH * COLS; i += NT) {
      const int t = i / COLS, c_ = c0 + i % COLS;
      const bool ok = t < nt && c_ < a.vdim;
      cp_async_f(vs + i, ok ? ub + (int64_t) t * C + 2 * a.G * a.dim + h * a.vdim + c_ : a.u, ok);
    }
    for (int i = threadIdx.x; i < TCH * (MR / 4); i += NT) {                 // a row's block matrices: 20 floats, 16-byte aligned
      const int t = i / (MR / 4), p4 = (i % (MR / 4)) * 4;
      const bool ok = t < nt;
      cp_async_f4(mw + t * MR + p4, ok ? mats + ((int64_t) (row0 + t0 + t) * a.H + h) * MR + p4 : mats, ok);
    }
    cp_async_commit_wait_all(true);
  };
  const int nch = (len + TCH - 1) / TCH;
  if (nch > 0) stage_in(0, 0);
  for (int c = 0; c < nch; ++c) {
    // behind this barrier chunk c has landed (every thread waited for its own copies) and every warp has left the other stage
    cp_async_commit_wait_all(false);
    __syncthreads();
    if (c + 1 < nch) stage_in(c + 1, (c + 1) & 1);
    const float* ks = smem + (c & 1) * STAGE;
    const float* qs = ks + TCH * LDK;
    const float* mws = qs + TCH * LDK;
    const float* vs = mws + TCH * MR;
    const int t0 = c * TCH;
#pragma unroll 1
    for (int b = 0; b < TCH / T; ++b) {
      const int tb = t0 + b * T;
      if (tb >= len) break;
      const float* kb = ks + b * T * LDK;
      const float* qb = qs + b * T * LDK;
      // sixteen independent sums advance together: the tokens are the inner loop
      float A[T], B[T];
#pragma unroll
      for (int j = 0; j < T; ++j) A[j] = B[j] = 0.f;
      if constexpr (VEC == 4) {
#pragma unroll
        for (int v4 = 0; v4 < DPL / 4; ++v4) {
#pragma unroll
          for (int j = 0; j < T; ++j) {
            const float4 kv = *reinterpret_cast<const float4*>(kb + j * LDK + (v4 * LPC + sub) * 4);
            const float4 qv = *reinterpret_cast<const float4*>(qb + j * LDK + (v4 * LPC + sub) * 4);
            A[j] = fmaf(S[4 * v4], kv.x, A[j]); B[j] = fmaf(S[4 * v4], qv.x, B[j]);
            A[j] = fmaf(S[4 * v4 + 1], kv.y, A[j]); B[j] = fmaf(S[4 * v4 + 1], qv.y, B[j]);
            A[j] = fmaf(S[4 * v4 + 2], kv.z, A[j]); B[j] = fmaf(S[4 * v4 + 2], qv.z, B[j]);
            A[j] = fmaf(S[4 * v4 + 3], kv.w, A[j]); B[j] = fmaf(S[4 * v4 + 3], qv.w, B[j]);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
#pragma unroll
          for (int j = 0; j < T; ++j) {
            A[j] = fmaf(S[i], kb[j * LDK + dmap(i)], A[j]);
            B[j] = fmaf(S[i], qb[j * LDK + dmap(i)], B[j]);
          }
        }
      }
#pragma unroll
      for (int o = LPC / 2; o > 0; o >>= 1) {
#pragma unroll
        for (int j = 0; j < T; ++j) {
          A[j] += __shfl_xor_sync(0xffffffffu, A[j], o);
          B[j] += __shfl_xor_sync(0xffffffffu, B[j], o);
        }
      }
      // per column: r = v - D (S^T k), u = M r, o = D (S^T q) + W u, and the updates' weights u_j D_last / D_j.  Rows behind the
      // portion's end were staged as zeros: they give u = 0 and are not stored.
      const float* mw = mws + b * T * MR;
      const int nv = min(T, len - tb);
      float r[T], ut[T];
      float2 df[T];
#pragma unroll
      for (int j = 0; j < T; ++j) {
        df[j] = *reinterpret_cast<const float2*>(mw + j * MR + 2 * T);        // D_j, D_last / D_j
        r[j] = fmaf(-df[j].x, A[j], vs[(b * T + j) * COLS + cc]);
      }
#pragma unroll
      for (int j = 0; j < T; ++j) {
        const float4 m0 = *reinterpret_cast<const float4*>(mw + j * MR), m1 = *reinterpret_cast<const float4*>(mw + j * MR + 4);
        const float m[T] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float uj = 0.f;
#pragma unroll
        for (int i = 0; i <= j; ++i) uj = fmaf(m[i], r[i], uj);
        ut[j] = uj;
      }
#pragma unroll
      for (int j = 0; j < T; ++j) {
        const float4 w0 = *reinterpret_cast<const float4*>(mw + j * MR + T), w1 = *reinterpret_cast<const float4*>(mw + j * MR + T + 4);
        const float w[T] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float oj = df[j].x * B[j];
#pragma unroll
        for (int i = 0; i <= j; ++i) oj = fmaf(w[i], ut[i], oj);
        if (j < nv && live && sub == 0) out[((int64_t) (row0 + tb + j) * a.H + h) * a.vdim + col] = oj;
      }
      const float D = mw[(nv - 1) * MR + 2 * T];                              // all of the block's decays
#pragma unroll
      for (int j = 0; j < T; ++j) ut[j] *= df[j].y;
      if constexpr (VEC == 4) {
#pragma unroll
        for (int v4 = 0; v4 < DPL / 4; ++v4) {
          float s0 = D * S[4 * v4], s1 = D * S[4 * v4 + 1], s2 = D * S[4 * v4 + 2], s3 = D * S[4 * v4 + 3];
#pragma unroll
          for (int j = 0; j < T; ++j) {
            const float4 kv = *reinterpret_cast<const float4*>(kb + j * LDK + (v4 * LPC + sub) * 4);
            s0 = fmaf(ut[j], kv.x, s0); s1 = fmaf(ut[j], kv.y, s1); s2 = fmaf(ut[j], kv.z, s2); s3 = fmaf(ut[j], kv.w, s3);
          }
          S[4 * v4] = s0; S[4 * v4 + 1] = s1; S[4 * v4 + 2] = s2; S[4 * v4 + 3] = s3;
        }
      } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
          float acc = D * S[i];
#pragma unroll
          for (int j = 0; j < T; ++j) acc = fmaf(ut[j], kb[j * LDK + dmap(i)], acc);
          S[i] = acc;
        }
      }
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = dmap(i);
      if (d < a.dim) sp[d] = S[i];
    }
  }
}

// The form for steps with columns enough to fill the chip: a warp carries FOUR value columns, every lane holding DPL elements of
// each (a column's `dim` elements spread over all 32 lanes), so a staged key or query element is read from shared memory once per
// warp and used for four columns.  The 64 partial sums of a block (4 columns x 8 rows x {S^T k, S^T q}) are folded over the lanes
// — each stage halves the values a lane keeps — so that after five stages lane 8 c + j holds the two sums of column c, row j;
// u = M r and o = D (S^T q) + W u then run across the eight lanes of a column with shuffles, and the weights of the rank-one updates
// are handed back to all lanes.
template <int DPL>
__global__ void __launch_bounds__(128) delta_scan_tiled_kernel(float* out, ScanArgs a, const float* mats, int vec4) {
  constexpr int T = kBlk, TCH = kBlkChunk, CT = 4, NW = 4, COLS = NW * CT, LDK = 32 * DPL, VEC = DPL % 4 == 0 ? 4 : 1, NT = NW * 32;
  constexpr int MR = kMatRow, STAGE = 2 * TCH * LDK + TCH * MR + TCH * COLS;
  extern __shared__ __align__(16) float smem[];
  const int e = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int len = a.seq_len[e], past = a.seq_past[e], row0 = a.seq_start[e];
  const int jh = h / (a.H / a.G);
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  auto dmap = [&](int i) { return ((i / VEC) * 32 + lane) * VEC + i % VEC; };
  float* sp = a.state + ((int64_t) a.seq_slot[e] * a.H + h) * a.vdim * a.dim;
  float S[CT][DPL];
#pragma unroll
  for (int c = 0; c < CT; ++c) {
    const int col = c0 + warp * CT + c;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = dmap(i);
      S[c][i] = (col < a.vdim && past > 0 && d < a.dim) ? sp[(int64_t) col * a.dim + d] : 0.f;
    }
  }
  for (int i = threadIdx.x; i < 2 * STAGE; i += NT) smem[i] = 0.f;
  __syncthreads();
  auto stage_in = [&](int c, int buf) {
    float* ks = smem + buf * STAGE;
    float* qs = ks + TCH * LDK;
    float* mw = qs + TCH * LDK;
    float* vs = mw + TCH * MR;
    const int t0 = c * TCH, nt = min(TCH, len - t0);
    const float* ub = a.u + (int64_t) (row0 + t0) * C;
    if (vec4) {
      const int per = a.dim / 4;
      for (int i = threadIdx.x; i < TCH * per; i += NT) {
        const int t = i / per, d = (i % per) * 4;
        const bool ok = t < nt;
        cp_async_f4(qs + t * LDK + d, ok ? ub + (int64_t) t * C + jh * a.dim + d : a.u, ok);
        cp_async_f4(ks + t * LDK + d, ok ? ub + (int64_t) t * C + (a.G + jh) * a.dim + d : a.u, ok);
      }
    } else {
      for (int i = threadIdx.x; i < TCH * a.dim; i += NT) {
        const int t = i / a.dim, d = i % a.dim;
        const bool ok = t < nt;
        cp_async_f(qs + t * LDK + d, ok ? ub + (int64_t) t * C + jh * a.dim + d : a.u, ok);
        cp_async_f(ks + t * LDK + d, ok ? ub + (int64_t) t * C + (a.G + jh) * a.dim + d : a.u, ok);
      }
    }
    for (int i = threadIdx.x; i < TCH * COLS; i += NT) {
      const int t = i / COLS, c_ = c0 + i % COLS;
      const bool ok = t < nt && c_ < a.vdim;
      cp_async_f(vs + i, ok ? ub + (int64_t) t * C + 2 * a.G * a.dim + h * a.vdim + c_ : a.u, ok);
    }
    for (int i = threadIdx.x; i < TCH * (MR / 4); i += NT) {
      const int t = i / (MR / 4), p4 = (i % (MR / 4)) * 4;
      const bool ok = t < nt;
      cp_async_f4(mw + t * MR + p4, ok ? mats + ((int64_t) (row0 + t0 + t) * a.H + h) * MR + p4 : mats, ok);
    }
    cp_async_commit_wait_all(true);
  };
  const int nch = (len + TCH - 1) / TCH;
  if (nch > 0) stage_in(0, 0);
  const int cl = lane >> 3, jl = lane & 7;                                   // after the fold this lane owns (column cl, row jl)
  for (int c = 0; c < nch; ++c) {
    cp_async_commit_wait_all(false);
    __syncthreads();
    if (c + 1 < nch) stage_in(c + 1, (c + 1) & 1);
    const float* ks = smem + (c & 1) * STAGE;
    const float* qs = ks + TCH * LDK;
    const float* mws = qs + TCH * LDK;
    const float* vs = mws + TCH * MR;
    const int t0 = c * TCH;
#pragma unroll 1
    for (int b = 0; b < TCH / T; ++b) {
      const int tb = t0 + b * T;
      if (tb >= len) break;
      const float* kb = ks + b * T * LDK;
      const float* qb = qs + b * T * LDK;
      float x[CT * T * 2];                                                   // index (c * 8 + j) * 2 + {S^T k, S^T q}
#pragma unroll
      for (int v = 0; v < CT * T * 2; ++v) x[v] = 0.f;
#pragma unroll
      for (int i0 = 0; i0 < DPL; i0 += VEC) {
#pragma unroll
        for (int j = 0; j < T; ++j) {
          float kv[VEC], qv[VEC];
          if constexpr (VEC == 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kb + j * LDK + ((i0 / 4) * 32 + lane) * 4);
            const float4 q4 = *reinterpret_cast<const float4*>(qb + j * LDK + ((i0 / 4) * 32 + lane) * 4);
            kv[0] = k4.x; kv[1] = k4.y; kv[2] = k4.z; kv[3] = k4.w;
            qv[0] = q4.x; qv[1] = q4.y; qv[2] = q4.z; qv[3] = q4.w;
          } else {
            kv[0] = kb[j * LDK + dmap(i0)];
            qv[0] = qb[j * LDK + dmap(i0)];
          }
#pragma unroll
          for (int cc = 0; cc < CT; ++cc)
#pragma unroll
            for (int w = 0; w < VEC; ++w) {
              x[(cc * T + j) * 2] = fmaf(S[cc][i0 + w], kv[w], x[(cc * T + j) * 2]);
              x[(cc * T + j) * 2 + 1] = fmaf(S[cc][i0 + w], qv[w], x[(cc * T + j) * 2 + 1]);
            }
        }
      }
      // fold: a lane whose bit is set keeps the upper half of its values, hands the lower half over, and adds what it receives
#pragma unroll
      for (int st = 0; st < 5; ++st) {
        const int o = 16 >> st, half = (CT * T * 2) >> (st + 1);
        const bool up = lane & o;
#pragma unroll
        for (int m = 0; m < half; ++m) {
          const float send = up ? x[m] : x[m + half];
          const float keep = up ? x[m + half] : x[m];
          x[m] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
      }
      const float* mw = mws + b * T * MR;
      const int nv = min(T, len - tb);
      const float2 df = *reinterpret_cast<const float2*>(mw + jl * MR + 2 * T);        // D_j, D_last / D_j of this lane's row
      const float r = fmaf(-df.x, x[0], vs[(b * T + jl) * COLS + warp * CT + cl]);
      const float4 m0 = *reinterpret_cast<const float4*>(mw + jl * MR), m1 = *reinterpret_cast<const float4*>(mw + jl * MR + 4);
      const float4 w0 = *reinterpret_cast<const float4*>(mw + jl * MR + T), w1 = *reinterpret_cast<const float4*>(mw + jl * MR + T + 4);
      const float mr[T] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
      const float wr[T] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float uj = 0.f;
#pragma unroll
      for (int i = 0; i < T; ++i) uj = fmaf(mr[i], __shfl_sync(0xffffffffu, r, (lane & 24) | i), uj);      // entries behind the row are zero
      float oj = df.x * x[1];
#pragma unroll
      for (int i = 0; i < T; ++i) oj = fmaf(wr[i], __shfl_sync(0xffffffffu, uj, (lane & 24) | i), oj);
      const int col = c0 + warp * CT + cl;
      if (jl < nv && col < a.vdim) out[((int64_t) (row0 + tb + jl) * a.H + h) * a.vdim + col] = oj;
      const float ut = uj * df.y;
      const float D = mw[(nv - 1) * MR + 2 * T];
#pragma unroll
      for (int cc = 0; cc < CT; ++cc)
#pragma unroll
        for (int i = 0; i < DPL; ++i) S[cc][i] *= D;
#pragma unroll
      for (int j = 0; j < T; ++j) {
        float uc[CT];
#pragma unroll
        for (int cc = 0; cc < CT; ++cc) uc[cc] = __shfl_sync(0xffffffffu, ut, cc * 8 + j);
#pragma unroll
        for (int i0 = 0; i0 < DPL; i0 += VEC) {
          float kv[VEC];
          if constexpr (VEC == 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kb + j * LDK + ((i0 / 4) * 32 + lane) * 4);
            kv[0] = k4.x; kv[1] = k4.y; kv[2] = k4.z; kv[3] = k4.w;
          } else {
            kv[0] = kb[j * LDK + dmap(i0)];
          }
#pragma unroll
          for (int cc = 0; cc < CT; ++cc)
#pragma unroll
            for (int w = 0; w < VEC; ++w) S[cc][i0 + w] = fmaf(uc[cc], kv[w], S[cc][i0 + w]);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < CT; ++c) {
    const int col = c0 + warp * CT + c;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = dmap(i);
      if (col < a.vdim && d < a.dim) sp[(int64_t) col * a.dim + d] = S[c][i];
    }
  }
}

template <int DPL>
int launch_scan_tiled(float* out, const ScanArgs& a, const float* mats, int seqs, cudaStream_t s) {
  constexpr int COLS = 16, LDK = 32 * DPL;
  constexpr size_t smem = (size_t) 2 * (2 * kBlkChunk * LDK + kBlkChunk * kMatRow + kBlkChunk * COLS) * sizeof(float);
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(delta_scan_tiled_kernel<DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = true;
  }
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  const int vec4 = a.dim % 4 == 0 && C % 4 == 0 && (uintptr_t) a.u % 16 == 0;
  dim3 grid((a.vdim + COLS - 1) / COLS, a.H, seqs);
  delta_scan_tiled_kernel<DPL><<<grid, 128, smem, s>>>(out, a, mats, vec4);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// the blocks' products and inverted systems (workspace: gram [rows][G][16], then mats [rows][H][20]) -> mats
const float* prepare_blocks(const ScanArgs& a, float* workspace, int rows, int seqs, int max_len, cudaStream_t s) {
  const int nblk = (max_len + kBlk - 1) / kBlk;
  float* mats = workspace + (int64_t) rows * a.G * kBlk * 2;
  delta_gram_kernel<<<dim3(nblk, a.G, seqs), 256, 0, s>>>(workspace, a);
  const int64_t items = (int64_t) seqs * a.H * nblk;
  delta_block_matrices_kernel<<<(unsigned) ((items + 127) / 128), 128, 0, s>>>(mats, workspace, a, nblk, seqs);
  return mats;
}

template <int LPC, int DPL, int NW>
int launch_scan_blocked(float* out, const ScanArgs& a, const float* mats, int seqs, cudaStream_t s) {
  constexpr int COLS = NW * (32 / LPC), LDK = LPC * DPL;
  constexpr size_t smem = (size_t) 2 * (2 * kBlkChunk * LDK + kBlkChunk * kMatRow + kBlkChunk * COLS) * sizeof(float);
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(delta_scan_blocked_kernel<LPC, DPL, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = true;
  }
  const int C = 2 * a.G * a.dim + a.H * a.vdim;
  const int vec4 = a.dim % 4 == 0 && C % 4 == 0 && LDK % 4 == 0 && (uintptr_t) a.u % 16 == 0;
  dim3 grid((a.vdim + COLS - 1) / COLS, a.H, seqs);
  delta_scan_blocked_kernel<LPC, DPL, NW><<<grid, NW * 32, smem, s>>>(out, a, mats, vec4);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
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
static int g_scan_mode = 0;
extern "C" int tb_delta_scan_set_mode(int mode) { g_scan_mode = mode; return 0; }

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
  // one CTA per row when the rows alone fill the chip; a step of few rows also spreads a row's channels over CTAs
  const int C = 2 * kv_heads * dim + heads * vdim;
  const int ysplit = rows >= 296 ? 1 : std::max(1, std::min((C + 511) / 512, (296 + rows - 1) / rows));
  delta_prepare_kernel<<<dim3(rows, ysplit), 256, 0, (cudaStream_t) stream>>>(u, bg, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_delta_rule_scan(float* out, const float* u, const float* bg, float* state, const int* seq_start, const int* seq_len,
                                  const int* seq_past, const int* seq_slot, int rows, int seqs, int heads, int kv_heads, int dim,
                                  int vdim, int max_len, float* workspace, tb_stream_t stream) {
  if (!out || !u || !bg || !state || !seq_start || !seq_len || !seq_past || !seq_slot) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || dim > 512 || vdim <= 0 || seqs < 0 || seqs > 65535 || heads > 65535)
    return -1;
  if (seqs == 0) return 0;
  ScanArgs a{u, bg, state, seq_start, seq_len, seq_past, seq_slot, heads, kv_heads, dim, vdim};
  cudaStream_t s = (cudaStream_t) stream;
  if (max_len >= 3 && workspace) {
    // prompt portions: eight rows at a time; four columns per warp when there are columns enough to fill the chip that way
    const float* mats = prepare_blocks(a, workspace, rows, seqs, max_len, s);
    TB_CHECK_CUDA(cudaGetLastError());
    const bool tiled = dim <= 256 && (g_scan_mode == 1 || (g_scan_mode == 0 && (int64_t) seqs * heads * vdim >= 1200));
    if (tiled) {
      if (dim <= 32) return launch_scan_tiled<1>(out, a, mats, seqs, s);
      if (dim <= 64) return launch_scan_tiled<2>(out, a, mats, seqs, s);
      if (dim <= 128) return launch_scan_tiled<4>(out, a, mats, seqs, s);
      return launch_scan_tiled<8>(out, a, mats, seqs, s);
    }
    if (dim <= 32) return launch_scan_blocked<32, 1, 8>(out, a, mats, seqs, s);
    if (dim <= 64) return launch_scan_blocked<32, 2, 8>(out, a, mats, seqs, s);
    if (dim <= 128) return launch_scan_blocked<32, 4, 8>(out, a, mats, seqs, s);
    if (dim <= 256) return launch_scan_blocked<32, 8, 8>(out, a, mats, seqs, s);
    return launch_scan_blocked<32, 16, 8>(out, a, mats, seqs, s);
  }
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
