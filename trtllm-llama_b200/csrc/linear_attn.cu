// Linear attention with a scalar decay per head and token over a ragged in-flight batch — the recurrence behind a retention
// (fixed decay per head) and behind the matrix memory of an mLSTM (decay and input weight from exponential gates kept in range
// by a running maximum) — with the steps around it: rotation of projected heads in either pairing, the gates of the matrix
// memory, and the per-head normalisation + output gate.
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T,   o_t = S_t^T q_t          S [dim, vcols] fp32 per (sequence, head)
//
// Everything here is fp32: the state, the decays and their logarithms, the products that enter the state.
//
//   rope_heads_kernel        a thread per rotated pair: (2i, 2i + 1) or (i, i + dims / 2), with an output factor per head range
//   mlstm_gates_kernel       a CTA per (sequence, head): capped gates, then the running maximum m_t = max(f_t + m_(t-1), i_t) as a
//                            max-plus prefix scan over 256 rows at a time; emits ln a_t = f_t + m_(t-1) - m_t, ln b_t = i_t - m_t, m_t
//   decay_scan_rows_kernel   row by row, a warp per value column with dim over its lanes (generation steps, any dim <= 1024)
//   decay_scan_chunk_kernel  prompt portions, 32 rows at a time: the chunk's own products A[t, s] = (q_t . k_s) a_(s+1..t) b_s, then
//                            o = a_(..t) S0^T q_t + A V and S <- a_(..n) S0 + K^T (w V) as register-tiled fp32 products: a thread owns
//                            one value column and an eighth of dim, partial read-outs meet in shared memory
//   head_norm_gate_kernel    a warp per (row, head): optional division by max(|n . q|, exp(-m)) + tiny, RMS norm over vdim, weight,
//                            silu or sigmoid gate
#include <cuda_bf16.h>

#include <algorithm>

#include "common.cuh"
#include "../../include/trtllm_b200_ragged.h"

namespace tb {
namespace {

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------------------------------------
__global__ void rope_heads_kernel(float* out, int64_t ldo, const float* x, int64_t ldx, const float* table, int rows, int heads,
                                  int dim, int dims, int layout, int split, float scale_lo, float scale_hi) {
  const int half = dims / 2, rest = dim - dims;
  const int per_head = half + rest;                       // work items of a head: rotated pairs, then untouched elements
  const int64_t n = (int64_t) rows * heads * per_head;
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < n; i += (int64_t) gridDim.x * blockDim.x) {
    const int w = (int) (i % per_head);
    const int h = (int) ((i / per_head) % heads);
    const int64_t row = i / ((int64_t) per_head * heads);
    const float sc = h < split ? scale_lo : scale_hi;
    const float* src = x + row * ldx + (int64_t) h * dim;
    float* dst = out + row * ldo + (int64_t) h * dim;
    if (w >= half) { dst[dims + w - half] = src[dims + w - half] * sc; continue; }
    const int i0 = layout == TB_ROPE_HALF ? w : 2 * w, i1 = layout == TB_ROPE_HALF ? w + half : 2 * w + 1;
    const float c = table[(row * half + w) * 2], s = table[(row * half + w) * 2 + 1];
    const float u = src[i0], v = src[i1];
    dst[i0] = fmaf(u, c, -v * s) * sc;
    dst[i1] = fmaf(v, c, u * s) * sc;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
struct GateArgs {
  const float* proj; int64_t ldp; int col_i, col_f;
  const void *bias_i, *bias_f; int w_dtype; float cap;
  float* m_state; int64_t m_stride;                 // running maximum per (slot, head): m_state[slot * m_stride + head]
  const int *seq_start, *seq_len, *seq_past, *seq_slot;
  int heads;
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// one CTA of 8 warps per (sequence, head), 256 rows per trip: a warp scans its 32 rows, the warps' maps meet in shared memory
__global__ void __launch_bounds__(256) mlstm_gates_kernel(float* log_ab, float* m_out, GateArgs a) {
  __shared__ float wF[8], wI[8];
  __shared__ float m_carry;
  const int h = blockIdx.x, e = blockIdx.y, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int len = a.seq_len[e], start = a.seq_start[e], past = a.seq_past[e];
  float* ms = a.m_state + (int64_t) a.seq_slot[e] * a.m_stride + h;
  float m = past > 0 ? *ms : 0.f;                      // the maximum starts at 0, not at -inf
  const float bi = a.bias_i ? ld_w(a.bias_i, a.w_dtype, h) : 0.f, bf = a.bias_f ? ld_w(a.bias_f, a.w_dtype, h) : 0.f;
  for (int c0 = 0; c0 < len; c0 += 256) {
    const int t = c0 + threadIdx.x;
    const bool live = t < len;
    float ig = -INFINITY, fg = 0.f;                    // a dead lane is the identity map m -> max(m + 0, -inf)
    if (live) {
      const float* pr = a.proj + (int64_t) (start + t) * a.ldp;
      float zi = pr[a.col_i + h] + bi, zf = pr[a.col_f + h] + bf;
      if (a.cap > 0.f) { zi = a.cap * tanhf(zi / a.cap); zf = a.cap * tanhf(zf / a.cap); }
      ig = zi;
      fg = log_sigmoid(zf);
    }
    // inclusive max-plus scan: lane t ends with the map of its warp's rows up to t in a row, m -> max(m + F, I)
    float F = fg, I = ig;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, o), Ip = __shfl_up_sync(0xffffffffu, I, o);
      if (lane >= o) { I = fmaxf(Ip + F, I); F = Fp + F; }
    }
    if (lane == 31) { wF[warp] = F; wI[warp] = I; }
    __syncthreads();
    float PF = 0.f, PI = -INFINITY;                    // the map of the warps in front of this one
    for (int w = 0; w < warp; ++w) { PI = fmaxf(PI + wF[w], wI[w]); PF += wF[w]; }
    const float mt = fmaxf(m + (PF + F), fmaxf(PI + F, I));
    float mp = __shfl_up_sync(0xffffffffu, mt, 1);
    if (lane == 0) mp = fmaxf(m + PF, PI);             // the row in front of this warp's first
    if (live) {
      const int64_t o = (int64_t) (start + t) * a.heads + h;
      log_ab[2 * o] = fminf(fg + mp - mt, 0.f);        // m_t >= f_t + m_(t-1); the scan's sums may round it a few ulp the other way
      log_ab[2 * o + 1] = ig - mt;
      m_out[o] = mt;
    }
    if (threadIdx.x == 255) m_carry = mt;
    __syncthreads();
    m = m_carry;
  }
  if (threadIdx.x == 0) *ms = m;
}

// ---------------------------------------------------------------------------------------------------------------------
struct ScanArgs {
  const float *q, *k, *v; int64_t ldq, ldk, ldv;      // rows of [heads, dim] / [heads, vdim] behind these strides
  const float* log_ab;                                // [rows, heads, 2] or NULL
  const float* head_decay;                            // [heads] when log_ab is NULL
  float* state; int64_t state_stride;                 // state + slot * state_stride: [heads, vcols, dim]
  const int *seq_start, *seq_len, *seq_past, *seq_slot;
  int heads, dim, vdim, vcols;                        // vcols = vdim + 1 when a column of ones follows the values
  float q_scale;                                      // every query is multiplied by it as it is read
  // long portions are cut into segments of seg_rows rows (a multiple of 32) that run side by side: ws [seqs, max_segs, heads, vcols,
  // dim] holds at index sg + 1 segment sg's own end state from zero and then, after the carry kernel, at index sg the state segment
  // sg starts from (index 0: a copy of the slot's — the last segment overwrites the slot while the first may still be reading);
  // lseg [seqs, max_segs, heads] the sum of ln a over the segment.  ws NULL: one segment.
  float* ws; float* lseg; int max_segs, seg_rows;
};

constexpr int kRowWarps = 4;

template <int DPL>
__global__ void __launch_bounds__(kRowWarps * 32) decay_scan_rows_kernel(float* out, ScanArgs a) {
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int col = blockIdx.x * kRowWarps + warp, h = blockIdx.y, e = blockIdx.z;
  if (col >= a.vcols) return;
  const int len = a.seq_len[e], start = a.seq_start[e], past = a.seq_past[e];
  float* sp = a.state + (int64_t) a.seq_slot[e] * a.state_stride + ((int64_t) h * a.vcols + col) * a.dim;
  float s[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    s[i] = past > 0 && d < a.dim ? sp[d] : 0.f;
  }
  const float fixed = a.log_ab ? 0.f : a.head_decay[h];
  for (int t = 0; t < len; ++t) {
    const int64_t row = start + t;
    float at = fixed, bt = 1.f;
    if (a.log_ab) { at = expf(a.log_ab[2 * (row * a.heads + h)]); bt = expf(a.log_ab[2 * (row * a.heads + h) + 1]); }
    const float vv = (col < a.vdim ? a.v[row * a.ldv + (int64_t) h * a.vdim + col] : 1.f) * bt;
    const float* qr = a.q + row * a.ldq + (int64_t) h * a.dim;
    const float* kr = a.k + row * a.ldk + (int64_t) h * a.dim;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int d = lane + 32 * i;
      if (d < a.dim) {
        s[i] = fmaf(at, s[i], vv * kr[d]);
        o = fmaf(s[i], qr[d], o);
      }
    }
    o = warp_sum(o) * a.q_scale;
    if (lane == 0) out[(row * a.heads + h) * a.vcols + col] = o;
  }
#pragma unroll
  for (int i = 0; i < DPL; ++i) {
    const int d = lane + 32 * i;
    if (d < a.dim) sp[d] = s[i];
  }
}

// Prompt portions, 32 rows at a time.  CTA = (32 value columns, head, sequence), 8 warps: lane = column, warp = an eighth of
// dim (DPT elements, dim padded to 8 DPT with zeros).  The chunk's q, k, v tiles arrive through a two-stage cp.async ring (the next
// chunk's copies fly while this one is worked on) when the rows are 16-byte aligned, through plain loads otherwise.  Shared memory (floats):
//   Q [2][32][LD] | K [2][32][LD] | V [2][32][32] | A [32][33] | part [8][32][32] | L [32] | lbs [32] | eL [32] | wS [32]      LD = 8 DPT + 4
constexpr int kChunk = 32;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;                       // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;"); }

template <int DPT>
__global__ void __launch_bounds__(256) decay_scan_chunk_kernel(float* out, ScanArgs a, int vec) {
  constexpr int DP = 8 * DPT, LD = DP + 4;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                                       // [2][kChunk][LD]
  float* Ks = Qs + 2 * kChunk * LD;
  float* Vs = Ks + 2 * kChunk * LD;                     // [2][kChunk][32]
  float* As = Vs + 2 * kChunk * 32;
  float* part = As + kChunk * 33;
  float* Ls = part + 8 * kChunk * 32;
  float* lbs = Ls + kChunk;
  float* eL = lbs + kChunk;
  float* wS = eL + kChunk;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int cg = blockIdx.x, h = blockIdx.y;
  const int e = a.ws ? blockIdx.z / a.max_segs : blockIdx.z, sg = a.ws ? blockIdx.z % a.max_segs : 0;
  const int len_all = a.seq_len[e], past = a.seq_past[e];
  const int r0 = sg * a.seg_rows;                       // this CTA's rows of the portion: [r0, r1)
  if (r0 >= len_all) return;
  const int r1 = a.ws ? min(len_all, r0 + a.seg_rows) : len_all;
  const int len = r1 - r0, start = a.seq_start[e] + r0;
  const int col = cg * 32 + lane;
  const bool col_ok = col < a.vcols;
  const bool ones_here = col_ok && col >= a.vdim;       // the column of ones: its value is 1 at every live row
  float* sp = a.state + (int64_t) a.seq_slot[e] * a.state_stride + ((int64_t) h * a.vcols + (col_ok ? col : 0)) * a.dim;
  // the state in front of the first row: the slot's (zeros at a sequence's start), or what the carry kernel left for this segment
  const bool cut = a.ws && len_all > a.seg_rows;         // this sequence runs as several segments
  const float* s0 = cut ? a.ws + (((int64_t) e * a.max_segs + sg) * a.heads + h) * a.vcols * a.dim + (int64_t) (col_ok ? col : 0) * a.dim
                        : (past > 0 ? sp : nullptr);
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = warp * DPT + i;
    s[i] = s0 && col_ok && d < a.dim ? s0[d] : 0.f;
  }
  const float fixed_la = a.log_ab ? 0.f : logf(a.head_decay[h]);

  auto load_chunk = [&](int c0, int buf) {
    const int n = min(kChunk, len - c0);
    const int64_t row0 = start + c0;
    float* Qb = Qs + buf * kChunk * LD;
    float* Kb = Ks + buf * kChunk * LD;
    float* Vb = Vs + buf * kChunk * 32;
    if (vec) {
      for (int idx = threadIdx.x; idx < kChunk * (DP / 4); idx += 256) {
        const int t = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
        const bool ok = t < n && d < a.dim;            // dim is a multiple of 4 here: the four elements are in or out together
        cp_async16(Qb + t * LD + d, ok ? a.q + (row0 + t) * a.ldq + (int64_t) h * a.dim + d : a.q, ok);
        cp_async16(Kb + t * LD + d, ok ? a.k + (row0 + t) * a.ldk + (int64_t) h * a.dim + d : a.k, ok);
      }
      {
        const int t = threadIdx.x / 8, c = cg * 32 + (threadIdx.x % 8) * 4;
        const bool ok = t < n && c < a.vdim;
        cp_async16(Vb + t * 32 + (threadIdx.x % 8) * 4, ok ? a.v + (row0 + t) * a.ldv + (int64_t) h * a.vdim + c : a.v, ok);
      }
    } else {
      for (int idx = threadIdx.x; idx < kChunk * DP; idx += 256) {
        const int t = idx / DP, d = idx % DP;
        const bool ok = t < n && d < a.dim;
        Qb[t * LD + d] = ok ? a.q[(row0 + t) * a.ldq + (int64_t) h * a.dim + d] : 0.f;
        Kb[t * LD + d] = ok ? a.k[(row0 + t) * a.ldk + (int64_t) h * a.dim + d] : 0.f;
      }
      for (int idx = threadIdx.x; idx < kChunk * 32; idx += 256) {
        const int t = idx / 32, c = cg * 32 + idx % 32;
        Vb[idx] = t < n && c < a.vdim ? a.v[(row0 + t) * a.ldv + (int64_t) h * a.vdim + c] : 0.f;
      }
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < len; c0 += kChunk, buf ^= 1) {
    const int n = min(kChunk, len - c0);
    const int64_t row0 = start + c0;
    const float* Qb = Qs + buf * kChunk * LD;
    const float* Kb = Ks + buf * kChunk * LD;
    const float* Vb = Vs + buf * kChunk * 32;
    cp_async_wait_all();
    __syncthreads();                                   // this chunk's tiles have landed; the other stage and part / A are free
    if (c0 + kChunk < len) load_chunk(c0 + kChunk, buf ^ 1);
    if (warp == 0) {
      float la = 0.f, lb = -INFINITY;
      if (lane < n) {
        if (a.log_ab) { la = a.log_ab[2 * ((row0 + lane) * a.heads + h)]; lb = a.log_ab[2 * ((row0 + lane) * a.heads + h) + 1]; }
        else { la = fixed_la; lb = 0.f; }
      }
      float L = la;                                    // inclusive sum of ln a over the chunk's rows
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float p = __shfl_up_sync(0xffffffffu, L, o);
        if (lane >= o) L += p;
      }
      const float Ltot = __shfl_sync(0xffffffffu, L, n - 1);
      Ls[lane] = L;
      lbs[lane] = lb - L;                              // weight of key s for row t: exp(L_t - L_s + ln b_s)
      eL[lane] = expf(L);                              // weight of the carried state for row t
      wS[lane] = lane < n ? expf(Ltot - L + lb) : 0.f;  // weight of key s in the state after the chunk
    }
    __syncthreads();
    // the chunk's own products: thread -> rows t = warp * 4 + j, key s = lane
    {
      float dot[4] = {0.f, 0.f, 0.f, 0.f};
      const float* kr = Kb + lane * LD;
#pragma unroll 4
      for (int d = 0; d < DP; d += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 qv = *reinterpret_cast<const float4*>(Qb + (warp * 4 + j) * LD + d);
          dot[j] = fmaf(qv.x, kv.x, dot[j]);
          dot[j] = fmaf(qv.y, kv.y, dot[j]);
          dot[j] = fmaf(qv.z, kv.z, dot[j]);
          dot[j] = fmaf(qv.w, kv.w, dot[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = warp * 4 + j;
        As[t * 33 + lane] = (lane <= t && t < n) ? dot[j] * a.q_scale * expf(Ls[t] + lbs[lane]) : 0.f;
      }
    }
    __syncthreads();
    // read-out against the carried state: 32 independent sums per thread, the state's elements outermost
    float acc[kChunk];
#pragma unroll
    for (int t = 0; t < kChunk; ++t) acc[t] = 0.f;
    if constexpr (DPT % 4 == 0) {
#pragma unroll
      for (int i = 0; i < DPT; i += 4) {
#pragma unroll
        for (int t = 0; t < kChunk; ++t) {
          const float4 qv = *reinterpret_cast<const float4*>(Qb + t * LD + warp * DPT + i);
          acc[t] = fmaf(s[i], qv.x, acc[t]); acc[t] = fmaf(s[i + 1], qv.y, acc[t]);
          acc[t] = fmaf(s[i + 2], qv.z, acc[t]); acc[t] = fmaf(s[i + 3], qv.w, acc[t]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < DPT; i += 2) {
#pragma unroll
        for (int t = 0; t < kChunk; ++t) {
          const float2 qv = *reinterpret_cast<const float2*>(Qb + t * LD + warp * DPT + i);
          acc[t] = fmaf(s[i], qv.x, acc[t]); acc[t] = fmaf(s[i + 1], qv.y, acc[t]);
        }
      }
    }
#pragma unroll
    for (int t = 0; t < kChunk; ++t) acc[t] *= eL[t] * a.q_scale;
    for (int sk = warp; sk < n; sk += 8) {             // this warp's share of the chunk's keys
      const float vv = ones_here ? 1.f : Vb[sk * 32 + lane];
#pragma unroll
      for (int t = 0; t < kChunk; ++t) acc[t] = fmaf(As[t * 33 + sk], vv, acc[t]);
    }
#pragma unroll
    for (int t = 0; t < kChunk; ++t) part[(warp * kChunk + t) * 32 + lane] = acc[t];
    // the state after the chunk
    const float dec = eL[n - 1];
#pragma unroll
    for (int i = 0; i < DPT; ++i) s[i] *= dec;
    for (int sk = 0; sk < n; ++sk) {
      const float wv = wS[sk] * (ones_here ? 1.f : Vb[sk * 32 + lane]);
      const float* kr = Kb + sk * LD + warp * DPT;
      if constexpr (DPT % 4 == 0) {
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + i);
          s[i] = fmaf(wv, kv.x, s[i]); s[i + 1] = fmaf(wv, kv.y, s[i + 1]); s[i + 2] = fmaf(wv, kv.z, s[i + 2]); s[i + 3] = fmaf(wv, kv.w, s[i + 3]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < DPT; i += 2) {
          const float2 kv = *reinterpret_cast<const float2*>(kr + i);
          s[i] = fmaf(wv, kv.x, s[i]); s[i + 1] = fmaf(wv, kv.y, s[i + 1]);
        }
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kChunk * 32; idx += 256) {
      const int t = idx / 32, c = idx % 32;
      if (t >= n || cg * 32 + c >= a.vcols) continue;
      float o = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) o += part[(w * kChunk + t) * 32 + c];      // fixed order
      out[((row0 + t) * a.heads + h) * a.vcols + cg * 32 + c] = o;
    }
  }
  if (col_ok && r1 == len_all) {                       // the portion's last rows: the sequence's state
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = warp * DPT + i;
      if (d < a.dim) sp[d] = s[i];
    }
  }
}

// A segment's own end state, from zero: S <- a_(..n) S + K^T (w V) chunk by chunk, nothing read out.  Same CTA shape and ring as above
// (keys and values only).  Shared memory (floats): K [2][32][LD] | V [2][32][32] | wS [32] | dec
template <int DPT>
__global__ void __launch_bounds__(256) decay_segment_state_kernel(ScanArgs a, int vec) {
  constexpr int DP = 8 * DPT, LD = DP + 4;
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;
  float* Vs = Ks + 2 * kChunk * LD;
  float* wS = Vs + 2 * kChunk * 32;
  float* dec_s = wS + kChunk;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int cg = blockIdx.x, h = blockIdx.y, e = blockIdx.z / a.max_segs, sg = blockIdx.z % a.max_segs;
  const int len_all = a.seq_len[e];
  const int r0 = sg * a.seg_rows;
  if (r0 + a.seg_rows >= len_all) return;                // the last segment's end state is the sequence's: the main kernel writes it
  const int start = a.seq_start[e] + r0, len = a.seg_rows;   // whole chunks: seg_rows is a multiple of 32
  const int col = cg * 32 + lane;
  const bool col_ok = col < a.vcols;
  const bool ones_here = col_ok && col >= a.vdim;
  float s[DPT];
#pragma unroll
  for (int i = 0; i < DPT; ++i) s[i] = 0.f;
  const float fixed_la = a.log_ab ? 0.f : logf(a.head_decay[h]);
  float Lsum = 0.f;

  auto load_chunk = [&](int c0, int buf) {
    const int64_t row0 = start + c0;
    float* Kb = Ks + buf * kChunk * LD;
    float* Vb = Vs + buf * kChunk * 32;
    if (vec) {
      for (int idx = threadIdx.x; idx < kChunk * (DP / 4); idx += 256) {
        const int t = idx / (DP / 4), d = (idx % (DP / 4)) * 4;
        const bool ok = d < a.dim;
        cp_async16(Kb + t * LD + d, ok ? a.k + (row0 + t) * a.ldk + (int64_t) h * a.dim + d : a.k, ok);
      }
      {
        const int t = threadIdx.x / 8, c = cg * 32 + (threadIdx.x % 8) * 4;
        const bool ok = c < a.vdim;
        cp_async16(Vb + t * 32 + (threadIdx.x % 8) * 4, ok ? a.v + (row0 + t) * a.ldv + (int64_t) h * a.vdim + c : a.v, ok);
      }
    } else {
      for (int idx = threadIdx.x; idx < kChunk * DP; idx += 256) {
        const int t = idx / DP, d = idx % DP;
        Kb[t * LD + d] = d < a.dim ? a.k[(row0 + t) * a.ldk + (int64_t) h * a.dim + d] : 0.f;
      }
      for (int idx = threadIdx.x; idx < kChunk * 32; idx += 256) {
        const int t = idx / 32, c = cg * 32 + idx % 32;
        Vb[idx] = c < a.vdim ? a.v[(row0 + t) * a.ldv + (int64_t) h * a.vdim + c] : 0.f;
      }
    }
    cp_async_commit();
  };

  load_chunk(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < len; c0 += kChunk, buf ^= 1) {
    const int64_t row0 = start + c0;
    const float* Kb = Ks + buf * kChunk * LD;
    const float* Vb = Vs + buf * kChunk * 32;
    cp_async_wait_all();
    __syncthreads();
    if (c0 + kChunk < len) load_chunk(c0 + kChunk, buf ^ 1);
    if (warp == 0) {
      float la = fixed_la, lb = 0.f;
      if (a.log_ab) { la = a.log_ab[2 * ((row0 + lane) * a.heads + h)]; lb = a.log_ab[2 * ((row0 + lane) * a.heads + h) + 1]; }
      float L = la;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float p = __shfl_up_sync(0xffffffffu, L, o);
        if (lane >= o) L += p;
      }
      const float Ltot = __shfl_sync(0xffffffffu, L, 31);
      wS[lane] = expf(Ltot - L + lb);
      if (lane == 0) { dec_s[0] = expf(Ltot); dec_s[1] = Ltot; }
    }
    __syncthreads();
    const float dec = dec_s[0];
    Lsum += dec_s[1];
#pragma unroll
    for (int i = 0; i < DPT; ++i) s[i] *= dec;
    for (int sk = 0; sk < kChunk; ++sk) {
      const float wv = wS[sk] * (ones_here ? 1.f : Vb[sk * 32 + lane]);
      const float* kr = Kb + sk * LD + warp * DPT;
      if constexpr (DPT % 4 == 0) {
#pragma unroll
        for (int i = 0; i < DPT; i += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + i);
          s[i] = fmaf(wv, kv.x, s[i]); s[i + 1] = fmaf(wv, kv.y, s[i + 1]); s[i + 2] = fmaf(wv, kv.z, s[i + 2]); s[i + 3] = fmaf(wv, kv.w, s[i + 3]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < DPT; i += 2) {
          const float2 kv = *reinterpret_cast<const float2*>(kr + i);
          s[i] = fmaf(wv, kv.x, s[i]); s[i + 1] = fmaf(wv, kv.y, s[i + 1]);
        }
      }
    }
  }
  if (col_ok) {
    float* dst = a.ws + (((int64_t) e * a.max_segs + sg + 1) * a.heads + h) * a.vcols * a.dim + (int64_t) col * a.dim;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
      const int d = warp * DPT + i;
      if (d < a.dim) dst[d] = s[i];
    }
  }
  if (cg == 0 && threadIdx.x == 0) a.lseg[((int64_t) e * a.max_segs + sg) * a.heads + h] = Lsum;
}

// ws[sg + 1] (segment sg's own end state) -> the state segment sg + 1 starts from: run <- exp(sum of ln a over sg) * run + own, in
// order; ws[0] <- the state the sequence brings
__global__ void decay_segment_carry_kernel(ScanArgs a) {
  const int e = blockIdx.y;
  const int64_t per = (int64_t) a.heads * a.vcols * a.dim;
  const int64_t idx = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
  if (idx >= per) return;
  const int len = a.seq_len[e];
  const int nseg = (len + a.seg_rows - 1) / a.seg_rows;
  if (nseg <= 1) return;
  const int h = (int) (idx / ((int64_t) a.vcols * a.dim));
  float run = a.seq_past[e] > 0 ? a.state[(int64_t) a.seq_slot[e] * a.state_stride + idx] : 0.f;
  a.ws[(int64_t) e * a.max_segs * per + idx] = run;
  for (int sg = 0; sg + 1 < nseg; ++sg) {
    float* p = a.ws + ((int64_t) e * a.max_segs + sg + 1) * per + idx;
    run = fmaf(expf(a.lseg[((int64_t) e * a.max_segs + sg) * a.heads + h]), run, *p);
    *p = run;
  }
}

template <int DPT>
int launch_chunk(float* out, const ScanArgs& a, int seqs, cudaStream_t st) {
  constexpr int DP = 8 * DPT, LD = DP + 4;
  constexpr size_t smem = ((size_t) 4 * kChunk * LD + 2 * kChunk * 32 + kChunk * 33 + 8 * kChunk * 32 + 4 * kChunk) * sizeof(float);
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(decay_scan_chunk_kernel<DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = true;
  }
  // cp.async moves 16 bytes: every row of q, k, v and every head and column group inside it must start on such a boundary
  const int vec = a.dim % 4 == 0 && a.vdim % 4 == 0 && a.ldq % 4 == 0 && a.ldk % 4 == 0 && a.ldv % 4 == 0 &&
                  (uintptr_t) a.q % 16 == 0 && (uintptr_t) a.k % 16 == 0 && (uintptr_t) a.v % 16 == 0;
  if (a.ws) {
    constexpr size_t smem_a = ((size_t) 2 * kChunk * LD + 2 * kChunk * 32 + kChunk + 2) * sizeof(float);
    static bool raised_a = false;
    if (!raised_a && smem_a > 48 * 1024) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(decay_segment_state_kernel<DPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_a));
      raised_a = true;
    }
    dim3 grid((a.vcols + 31) / 32, a.heads, seqs * a.max_segs);
    decay_segment_state_kernel<DPT><<<grid, 256, smem_a, st>>>(a, vec);
    const int64_t per = (int64_t) a.heads * a.vcols * a.dim;
    decay_segment_carry_kernel<<<dim3((unsigned) ((per + 255) / 256), seqs), 256, 0, st>>>(a);
    decay_scan_chunk_kernel<DPT><<<grid, 256, smem, st>>>(out, a, vec);
    return 0;
  }
  dim3 grid((a.vcols + 31) / 32, a.heads, seqs);
  decay_scan_chunk_kernel<DPT><<<grid, 256, smem, st>>>(out, a, vec);
  return 0;
}

template <int DPL>
void launch_rows(float* out, const ScanArgs& a, int seqs, cudaStream_t st) {
  dim3 grid((a.vcols + kRowWarps - 1) / kRowWarps, a.heads, seqs);
  decay_scan_rows_kernel<DPL><<<grid, kRowWarps * 32, 0, st>>>(out, a);
}

// ---------------------------------------------------------------------------------------------------------------------
struct HeadNormArgs {
  const float* o; int vcols;                         // [rows, heads, vcols]; the first vdim columns are the read-out
  const float* m;                                    // [rows, heads] running maxima, or NULL: no division
  float den_eps;
  const float* gate; int64_t ldg; int gate_act;      // logits [rows, >= heads * vdim]; 0 none, 1 silu, 2 sigmoid
  const void* w; int w_dtype; int w_per_head;        // [vdim] shared by the heads, or [heads * vdim]
  float eps; int rows, heads, vdim;
};

template <typename T>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(T* out, HeadNormArgs a) {
  const int lane = threadIdx.x % 32;
  const int64_t item = (int64_t) blockIdx.x * 4 + threadIdx.x / 32;
  if (item >= (int64_t) a.rows * a.heads) return;
  const int h = (int) (item % a.heads);
  const int64_t row = item / a.heads;
  const float* src = a.o + item * a.vcols;
  float f = 1.f;
  if (a.m) f = 1.f / (fmaxf(fabsf(src[a.vdim]), expf(-a.m[item])) + a.den_eps);
  float ss = 0.f;
  for (int c = lane; c < a.vdim; c += 32) { const float v = src[c] * f; ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float inv = f / sqrtf(ss / (float) a.vdim + a.eps);
  for (int c = lane; c < a.vdim; c += 32) {
    float v = src[c] * inv;
    if (a.w) v *= ld_w(a.w, a.w_dtype, a.w_per_head ? (int64_t) h * a.vdim + c : c);
    if (a.gate_act) {
      const float z = a.gate[row * a.ldg + (int64_t) h * a.vdim + c], sg = 1.f / (1.f + expf(-z));
      v *= a.gate_act == 1 ? z * sg : sg;
    }
    out[item * a.vdim + c] = from_f<T>(v);
  }
}

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_rope_heads(float* out, int64_t ldo, const float* x, int64_t ldx, const float* table, int rows, int heads, int dim,
                             int dims, int layout, int split, float scale_lo, float scale_hi, tb_stream_t stream) {
  if (!out || !x || rows < 0 || heads <= 0 || dim <= 0 || dims < 0 || dims % 2 || dims > dim || (dims > 0 && !table) ||
      (layout != TB_ROPE_INTERLEAVED && layout != TB_ROPE_HALF))
    return -1;
  if (rows == 0) return 0;
  const int64_t n = (int64_t) rows * heads * (dim - dims / 2);
  const int grid = (int) std::min<int64_t>((n + 255) / 256, 148 * 16);
  rope_heads_kernel<<<grid, 256, 0, (cudaStream_t) stream>>>(out, ldo, x, ldx, table, rows, heads, dim, dims, layout, split, scale_lo,
                                                             scale_hi);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_mlstm_gates(float* log_ab, float* m_out, const float* proj, int64_t ldp, int col_i, int col_f, const void* bias_i,
                              const void* bias_f, int w_dtype, float cap, float* m_state, int64_t m_stride, const int* seq_start,
                              const int* seq_len, const int* seq_past, const int* seq_slot, int seqs, int heads, tb_stream_t stream) {
  if (!log_ab || !m_out || !proj || !m_state || !seq_start || !seq_len || !seq_past || !seq_slot || heads <= 0 || seqs < 0 ||
      col_i < 0 || col_f < 0 || seqs > 65535)
    return -1;
  if ((bias_i || bias_f) && w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16) return -1;
  if (seqs == 0) return 0;
  GateArgs a{proj, ldp, col_i, col_f, bias_i, bias_f, w_dtype, cap, m_state, m_stride, seq_start, seq_len, seq_past, seq_slot, heads};
  mlstm_gates_kernel<<<dim3(heads, seqs), 256, 0, (cudaStream_t) stream>>>(log_ab, m_out, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

static int g_decay_scan_mode = 0;
extern "C" int tb_decay_scan_set_mode(int mode) { g_decay_scan_mode = mode; return 0; }

// Segments a long portion is cut into so that the chip is filled: as many as still run as ONE wave of two CTAs per SM (a second,
// partly filled wave would cost a whole segment's time), at least two chunks of 32 rows per segment, at most 16 (the workspace
// holds a state per segment).  1: the portion runs as one.
extern "C" int tb_decay_scan_segments(int seqs, int heads, int vcols, int max_len) {
  if (seqs <= 0 || heads <= 0 || vcols <= 0 || max_len <= 0 || g_decay_scan_mode == 2) return 1;
  const int64_t base = (int64_t) ((vcols + 31) / 32) * heads * seqs;
  int64_t segs = (2 * kNumSMs) / base;
  segs = std::min<int64_t>(segs, std::min(16, max_len / 64));
  return segs < 2 ? 1 : (int) segs;
}

extern "C" int tb_decay_attention_scan(float* out, const float* q, int64_t ldq, const float* k, int64_t ldk, const float* v, int64_t ldv,
                                       const float* log_ab, const float* head_decay, float* state, int64_t state_stride,
                                       const int* seq_start, const int* seq_len, const int* seq_past, const int* seq_slot, int rows,
                                       int seqs, int heads, int dim, int vdim, int ones_col, float q_scale, int max_len,
                                       float* workspace, int segments, tb_stream_t stream) {
  if (!out || !q || !k || !v || !state || !seq_start || !seq_len || !seq_past || !seq_slot || (!log_ab && !head_decay)) return -1;
  if (heads <= 0 || dim <= 0 || dim > 1024 || vdim <= 0 || rows < 0 || seqs < 0 || seqs > 65535 || heads > 65535) return -1;
  if (rows == 0 || seqs == 0) return 0;
  ScanArgs a{q, k, v, ldq, ldk, ldv, log_ab, head_decay, state, state_stride, seq_start, seq_len, seq_past, seq_slot, heads, dim, vdim,
             vdim + (ones_col ? 1 : 0), q_scale, nullptr, nullptr, 1, 0};
  cudaStream_t st = (cudaStream_t) stream;
  if (segments > 1 && workspace && max_len >= 64 * segments) {
    // workspace: [seqs, segments, heads, vcols, dim] states, then [seqs, segments, heads] sums of ln a
    a.max_segs = segments;
    a.seg_rows = (((max_len + segments - 1) / segments + kChunk - 1) / kChunk) * kChunk;
    a.ws = workspace;
    a.lseg = workspace + (int64_t) seqs * segments * heads * a.vcols * dim;
  }
  if (g_decay_scan_mode != 1 && max_len >= 4 && dim <= 256) {
    const int dpt = (dim + 7) / 8;
    int rc;
    if (dpt <= 2) rc = launch_chunk<2>(out, a, seqs, st);
    else if (dpt <= 4) rc = launch_chunk<4>(out, a, seqs, st);
    else if (dpt <= 6) rc = launch_chunk<6>(out, a, seqs, st);
    else if (dpt <= 8) rc = launch_chunk<8>(out, a, seqs, st);
    else if (dpt <= 12) rc = launch_chunk<12>(out, a, seqs, st);
    else if (dpt <= 16) rc = launch_chunk<16>(out, a, seqs, st);
    else if (dpt <= 24) rc = launch_chunk<24>(out, a, seqs, st);
    else rc = launch_chunk<32>(out, a, seqs, st);
    if (rc) return rc;
    TB_CHECK_CUDA(cudaGetLastError());
    return 0;
  }
  const int dpl = (dim + 31) / 32;
  if (dpl <= 1) launch_rows<1>(out, a, seqs, st);
  else if (dpl <= 2) launch_rows<2>(out, a, seqs, st);
  else if (dpl <= 4) launch_rows<4>(out, a, seqs, st);
  else if (dpl <= 8) launch_rows<8>(out, a, seqs, st);
  else if (dpl <= 16) launch_rows<16>(out, a, seqs, st);
  else launch_rows<32>(out, a, seqs, st);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_head_norm_gate(void* out, int dtype, const float* o, int vcols, const float* m, float den_eps, const float* gate,
                                 int64_t ldg, int gate_act, const void* w, int w_dtype, int w_per_head, float eps, int rows, int heads,
                                 int vdim, tb_stream_t stream) {
  if (!out || !o || (dtype != TB_DT_F32 && dtype != TB_DT_BF16) || rows < 0 || heads <= 0 || vdim <= 0 || vcols < vdim ||
      (m && vcols < vdim + 1) || gate_act < 0 || gate_act > 2 || (gate_act && !gate))
    return -1;
  if (w && w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16) return -1;
  if (rows == 0) return 0;
  HeadNormArgs a{o, vcols, m, den_eps, gate, ldg, gate_act, w, w_dtype, w_per_head, eps, rows, heads, vdim};
  const int64_t items = (int64_t) rows * heads;
  const unsigned grid = (unsigned) ((items + 3) / 4);
  if (dtype == TB_DT_F32) head_norm_gate_kernel<float><<<grid, 128, 0, (cudaStream_t) stream>>>((float*) out, a);
  else head_norm_gate_kernel<__nv_bfloat16><<<grid, 128, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) out, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
