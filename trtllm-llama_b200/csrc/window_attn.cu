// Grouped-query attention over a sliding window of a paged key/value pool, with a softmax sink and per-head output
// gates, for a ragged in-flight batch; and the step in front of it that turns projected rows into queries and cache
// entries (short causal convolution -> rotation -> paged store).
//
// Pool entry of one position: [G][dim] rotated keys, then [G][vdim] values (G key/value heads).  Query head h reads
// key/value head h / (H / G).
//
//   qkv_conv_rope_append_kernel   one CTA per row, threads walk pairs of channels of the concatenated q | k | v projection: the causal
//                                 convolution over the row's own portion and the sequence's carried inputs, the
//                                 rotation of the head's leading `dims` elements (interleaved pairs; the partner's
//                                 convolution is recomputed), and the store: queries to their buffer, keys and values
//                                 to the row's place in its sequence's pages.
//   window_attention_kernel       any sizes, fp32 or bf16: one CTA per (row, key/value head, 4 query heads of its group);
//                                 key blocks of 32 positions aligned to absolute positions, from the window's first block,
//                                 staged as fp32; lane = key for the scores, lane = value column for the weighted sum.
//   window_attention_mma_kernel   bf16 and the head sizes it is built for: tensor cores, 64 (token, head) rows of one
//                                 sequence and key/value head per CTA — see its own comment below.
//
// The softmax runs online in fp32 and starts from the sink: m = sink_h, l = 1, no value — so the sink is counted once,
// unscaled, whatever the number of key blocks.  Keys are visited in an order fixed by the row's position alone.
#include <cuda_bf16.h>

#include <algorithm>
#include <cstdlib>

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

__device__ __forceinline__ float ld_w(const void* p, int dtype, int64_t i) {
  return dtype == TB_DT_F32 ? reinterpret_cast<const float*>(p)[i]
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

constexpr int kMaxTaps = 16;

struct QkvArgs {
  const float* proj; int64_t ldp;            // [rows, >= C] : q (H dim) | k (G dim) | v (G vdim)
  const void* conv_w; int w_dtype;           // [C, taps]
  const float* state;                        // [slots, taps - 1, C] carried inputs, oldest first
  const float* table;                        // [rows, dims / 2, 2] cos, sin
  const int *tok_seq, *tok_pos, *seq_start, *seq_past, *seq_slot, *block_table;
  int max_blocks, page, rows, H, G, dim, vdim, dims, taps;
  float* state_rw;                           // == state when a sequence that brings ONE row moves its carried inputs on here
  const int* seq_len;                        // (then tb_causal_conv1d_update skips such sequences)
};

// convolution output of channel ch at the row's position
__device__ __forceinline__ float conv_at(const QkvArgs& a, const float* st, int C, int ch, int pos, int past, int start) {
  float acc = 0.f;
  for (int k = 0; k < a.taps; ++k) {
    const int p = pos - (a.taps - 1 - k);
    float v = 0.f;
    if (p >= past) v = a.proj[(int64_t) (start + (p - past)) * a.ldp + ch];
    else if (p >= 0) v = st[(int64_t) (a.taps - 1 - (past - p)) * C + ch];     // state row j holds position past - (taps-1) + j
    acc = fmaf(ld_w(a.conv_w, a.w_dtype, (int64_t) ch * a.taps + k), v, acc);
  }
  return acc;
}

// one CTA (or a few, for steps of few rows) per row; a thread walks pairs of neighbouring channels (both convolutions once, the rotation, the two stores),
// the row's place in its sequence and its page looked up once per thread
template <typename T>
__global__ void __launch_bounds__(256) qkv_conv_rope_append_kernel(T* q_out, T* pool, QkvArgs a) {
  const int Cq = a.H * a.dim, Ck = a.G * a.dim, Cv = a.G * a.vdim, C = Cq + Ck + Cv;
  const int row = blockIdx.x;
  const int e = a.tok_seq[row], pos = a.tok_pos[row], past = a.seq_past[e], start = a.seq_start[e];
  const float* st = a.state + (int64_t) a.seq_slot[e] * (a.taps - 1) * C;
  const int64_t slot = (int64_t) a.block_table[(int64_t) e * a.max_blocks + pos / a.page] * a.page + pos % a.page;
  T* q_row = q_out + (int64_t) row * Cq;
  T* kv_row = pool + slot * (Ck + Cv);
  // a sequence that brings one row: nobody else reads its carried inputs in this step, and this thread is the only one that
  // touches its channels — it moves them on itself, after it has read them
  const bool carry = a.state_rw && a.taps > 1 && a.seq_len[e] == 1;
  float* st_rw = carry ? a.state_rw + (int64_t) a.seq_slot[e] * (a.taps - 1) * C : nullptr;
  const float* cs_row = a.dims > 0 ? a.table + (int64_t) row * a.dims : nullptr;      // [dims / 2][cos, sin]
#pragma unroll 2
  for (int ch = 2 * (blockIdx.y * 256 + threadIdx.x); ch < C; ch += 2 * 256 * gridDim.y) {
    const bool two = ch + 1 < C;
    float y0 = conv_at(a, st, C, ch, pos, past, start), y1 = two ? conv_at(a, st, C, ch + 1, pos, past, start) : 0.f;
    if (ch < Cq + Ck) {
      const int d = (ch < Cq ? ch : ch - Cq) % a.dim;    // even: a.dim is even whenever anything is rotated
      if (d < a.dims) {
        const float c = cs_row[d], sn = cs_row[d + 1];
        const float u = y0, v = y1;
        y0 = fmaf(u, c, -v * sn);
        y1 = fmaf(v, c, u * sn);
      }
    }
    // the q | k | v boundaries can be odd only when nothing is rotated: the two elements are stored one by one
    if (ch < Cq) q_row[ch] = from_f<T>(y0); else kv_row[ch - Cq] = from_f<T>(y0);
    if (two) {
      if (ch + 1 < Cq) q_row[ch + 1] = from_f<T>(y1); else kv_row[ch + 1 - Cq] = from_f<T>(y1);
    }
    if (carry) {
      const int n = a.taps - 1;
      for (int i = 0; i < (two ? 2 : 1); ++i) {
        const int c = ch + i;
        // row j of the new state holds position pos - n + 1 + j: the old row j + 1 (zero before the sequence's start), then this row's input
        for (int j = 0; j + 1 < n; ++j) st_rw[(int64_t) j * C + c] = pos - n + 1 + j >= 0 ? st_rw[(int64_t) (j + 1) * C + c] : 0.f;
        st_rw[(int64_t) (n - 1) * C + c] = a.proj[(int64_t) row * a.ldp + c];
      }
    }
  }
}


// The same step for an attention whose queries and keys are RMS-normalised over the WHOLE projection (all heads at once, one
// weight per channel) between the convolution and the rotation, and whose values may be the keys themselves as they leave the
// convolution (before norm and rotation): proj holds q (H dim) | k (G dim) [| v (G vdim) when the values are projected].
// One CTA per row: pass 1 convolves every channel into shared memory and sums the squares of the q part and of the k part,
// pass 2 normalises, rotates pairs and stores.  Shared memory: the row's C convolved channels (fp32).
struct QkNormArgs {
  QkvArgs a;
  const void *norm_q, *norm_k;               // [H dim], [G dim] in w_dtype, or NULL
  float eps;
  int tied;                                  // values = convolved keys (vdim == dim, no v columns in proj)
};

template <typename T>
__global__ void __launch_bounds__(256) qk_conv_norm_rope_append_kernel(T* q_out, T* pool, QkNormArgs n) {
  extern __shared__ float ys[];
  __shared__ float red[2][8];
  __shared__ float inv_s[2];
  const QkvArgs& a = n.a;
  const int Cq = a.H * a.dim, Ck = a.G * a.dim, Cv = a.G * a.vdim, C = Cq + Ck + (n.tied ? 0 : Cv);
  const int row = blockIdx.x;
  const int e = a.tok_seq[row], pos = a.tok_pos[row], past = a.seq_past[e], start = a.seq_start[e];
  const float* st = a.taps > 1 ? a.state + (int64_t) a.seq_slot[e] * (a.taps - 1) * C : nullptr;
  const int64_t slot = (int64_t) a.block_table[(int64_t) e * a.max_blocks + pos / a.page] * a.page + pos % a.page;
  T* q_row = q_out + (int64_t) row * Cq;
  T* kv_row = pool + slot * (Ck + Cv);
  const bool carry = a.state_rw && a.taps > 1 && a.seq_len[e] == 1;
  float* st_rw = carry ? a.state_rw + (int64_t) a.seq_slot[e] * (a.taps - 1) * C : nullptr;
  float sq = 0.f, sk = 0.f;
  for (int ch = threadIdx.x; ch < C; ch += 256) {
    const float y = a.conv_w ? conv_at(a, st, C, ch, pos, past, start) : a.proj[(int64_t) row * a.ldp + ch];
    ys[ch] = y;
    if (ch < Cq) sq = fmaf(y, y, sq); else if (ch < Cq + Ck) sk = fmaf(y, y, sk);
    if (carry) {
      const int m = a.taps - 1;
      for (int j = 0; j + 1 < m; ++j) st_rw[(int64_t) j * C + ch] = pos - m + 1 + j >= 0 ? st_rw[(int64_t) (j + 1) * C + ch] : 0.f;
      st_rw[(int64_t) (m - 1) * C + ch] = a.proj[(int64_t) row * a.ldp + ch];
    }
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (threadIdx.x % 32 == 0) { red[0][threadIdx.x / 32] = sq; red[1][threadIdx.x / 32] = sk; }
  __syncthreads();
  if (threadIdx.x < 64) {
    const int w = threadIdx.x / 32, l = threadIdx.x % 32;
    float v = l < 8 ? red[w][l] : 0.f;
    v = warp_sum(v);
    if (l == 0) inv_s[w] = 1.f / sqrtf(v / (float) (w == 0 ? Cq : Ck) + n.eps);
  }
  __syncthreads();
  const bool normed = n.norm_q != nullptr;
  const float iq = normed ? inv_s[0] : 1.f, ik = normed ? inv_s[1] : 1.f;
  const float* cs_row = a.dims > 0 ? a.table + (int64_t) row * a.dims : nullptr;      // [dims / 2][cos, sin]
  // pairs of neighbouring channels of q | k: norm, weight, rotation, store (dim is even whenever anything is rotated)
  for (int ch = 2 * threadIdx.x; ch < Cq + Ck; ch += 512) {
    const bool two = ch + 1 < Cq + Ck;
    const bool isq = ch < Cq;
    const int c0 = isq ? ch : ch - Cq;
    float y0 = ys[ch] * (isq ? iq : ik), y1 = two ? ys[ch + 1] * (ch + 1 < Cq ? iq : ik) : 0.f;
    if (normed) {
      y0 *= ld_w(isq ? n.norm_q : n.norm_k, a.w_dtype, c0);
      if (two) y1 *= (ch + 1 < Cq) ? ld_w(n.norm_q, a.w_dtype, ch + 1) : ld_w(n.norm_k, a.w_dtype, ch + 1 - Cq);
    }
    const int d = c0 % a.dim;
    if (d < a.dims) {
      const float c = cs_row[d], sn = cs_row[d + 1];
      const float u = y0, v = y1;
      y0 = fmaf(u, c, -v * sn);
      y1 = fmaf(v, c, u * sn);
    }
    if (isq) q_row[ch] = from_f<T>(y0); else kv_row[ch - Cq] = from_f<T>(y0);
    if (two) {
      if (ch + 1 < Cq) q_row[ch + 1] = from_f<T>(y1); else kv_row[ch + 1 - Cq] = from_f<T>(y1);
    }
  }
  // values: the convolved keys as they are, or the convolved value channels
  for (int c = threadIdx.x; c < Cv; c += 256) kv_row[Ck + c] = from_f<T>(ys[n.tied ? Cq + c : Cq + Ck + c]);
}

constexpr int kWarps = 4;
constexpr int kTile = 32;
constexpr int kMaxVPerLane = 16;         // vdim <= 512

struct AttnArgs {
  const float* gate; int64_t ldg;          // gate logits [rows, >= H] or NULL
  const void* sink; int sink_dtype;        // [H] or NULL
  const int *tok_seq, *tok_pos, *block_table;
  int max_blocks, page, H, G, dim, vdim, window;
  float scale;
  int vsh, GV;                             // key heads per value head (key head g reads value head g / vsh), GV = G / vsh value heads
  int out_f32;                             // the result is stored as fp32 whatever the storage type
  int keep;                                // with a window: positions below `keep` stay visible to every later row
};

// shared memory (fp32): keys [32][dim + 1] | values [32][vdim] | per warp q [dim]
template <typename T>
__global__ void __launch_bounds__(kWarps * 32) window_attention_kernel(T* out, const T* q, const T* pool, AttnArgs a) {
  extern __shared__ float smem[];
  const int LDK = a.dim + 1, E = a.G * a.dim + a.GV * a.vdim, per = a.H / a.G;
  float* keys = smem;
  float* vals = keys + kTile * LDK;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  float* qs = vals + kTile * a.vdim + warp * a.dim;
  const int row = blockIdx.x, g = blockIdx.y;
  const int hl = blockIdx.z * kWarps + warp;            // head within the group
  const bool live = hl < per;
  const int head = g * per + (live ? hl : 0);
  const int pos = a.tok_pos[row];
  const int* bt = a.block_table + (int64_t) a.tok_seq[row] * a.max_blocks;
  const int lo = a.window > 0 && pos - a.window + 1 > 0 ? pos - a.window + 1 : 0;      // first visible position
  if (live) {
    const T* qsrc = q + ((int64_t) row * a.H + head) * a.dim;
    for (int d = lane; d < a.dim; d += 32) qs[d] = to_f<T>(qsrc[d]) * a.scale;
  }
  float acc[kMaxVPerLane];
#pragma unroll
  for (int c = 0; c < kMaxVPerLane; ++c) acc[c] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (a.sink) { m = ld_w(a.sink, a.sink_dtype, head); l = 1.f; }
  // kept first positions below the window: their blocks come first, then the window's blocks (an order fixed by pos alone)
  const int keep_lo = a.keep < lo ? a.keep : lo;                       // kept positions that the window does not cover
  const int kept_blocks = min((keep_lo + kTile - 1) / kTile, lo / kTile);
  const int first_block = lo / kTile - kept_blocks;
  for (int jb = first_block; jb * kTile <= pos; ++jb) {
    const int j0 = (jb < lo / kTile ? jb - first_block : jb) * kTile;
    __syncthreads();
    for (int e = threadIdx.x; e < kTile * a.dim; e += kWarps * 32) {
      const int jj = e / a.dim, d = e % a.dim, j = j0 + jj;
      float v = 0.f;
      if ((j >= lo || j < a.keep) && j <= pos) v = to_f<T>(pool[((int64_t) bt[j / a.page] * a.page + j % a.page) * E + g * a.dim + d]);
      keys[jj * LDK + d] = v;
    }
    for (int e = threadIdx.x; e < kTile * a.vdim; e += kWarps * 32) {
      const int jj = e / a.vdim, d = e % a.vdim, j = j0 + jj;
      float v = 0.f;
      if ((j >= lo || j < a.keep) && j <= pos)
        v = to_f<T>(pool[((int64_t) bt[j / a.page] * a.page + j % a.page) * E + a.G * a.dim + (g / a.vsh) * a.vdim + d]);
      vals[jj * a.vdim + d] = v;
    }
    __syncthreads();
    if (!live) continue;
    float s = 0.f;
    const float* kr = keys + lane * LDK;
    for (int d = 0; d < a.dim; ++d) s = fmaf(qs[d], kr[d], s);
    const bool vis = (j0 + lane >= lo || j0 + lane < a.keep) && j0 + lane <= pos;
    s = vis ? s : -INFINITY;
    const float m_new = fmaxf(m, warp_max(s));          // finite: every visited block holds a visible key
    const float p = vis ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);                 // 0 when m is still -inf
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
      const int col = c * 32 + lane;
      if (c * 32 >= a.vdim) break;                      // uniform over the warp
      const int cc = col < a.vdim ? col : a.vdim - 1;
      float v = acc[c] * corr;
#pragma unroll 8
      for (int jj = 0; jj < kTile; ++jj) v = fmaf(__shfl_sync(0xffffffffu, p, jj), vals[jj * a.vdim + cc], v);
      acc[c] = v;
    }
  }
  if (live) {
    float f = 1.f / l;
    if (a.gate) f *= 1.f / (1.f + expf(-a.gate[(int64_t) row * a.ldg + head]));
    const int64_t dst = ((int64_t) row * a.H + head) * a.vdim;
#pragma unroll
    for (int c = 0; c < kMaxVPerLane; ++c) {
      const int col = c * 32 + lane;
      if (col >= a.vdim) continue;
      if (a.out_f32) reinterpret_cast<float*>(out)[dst + col] = acc[c] * f;
      else out[dst + col] = from_f<T>(acc[c] * f);
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Tensor-core form (bf16 storage).  One CTA = 64 query rows of ONE sequence and ONE key/value head, where a "row" is a
// (token, query head of the group) pair, r = token * group + head: the heads that share a key/value head sit side by
// side in the MMA's M, so a key tile is loaded once for all of them and a generation step of one token still fills
// `group` rows.  Four warps of 16 rows.  Per key tile of 64 absolute positions (tile index = position / 64):
//   S [16 x 64] = Q [16 x DIM] . K^T            mma.sync m16n8k16 bf16, fp32 accumulators, fragments through ldmatrix
//   online softmax in fp32 in registers          window / causal mask per row; starts from the sink (m = sink, l = 1)
//   O [16 x VDIM] += P [16 x 64] . V             P reused from the S registers as the A operand, V through ldmatrix.trans
// K and V tiles arrive through a two-stage cp.async ring (one barrier per tile); positions outside [first visible of the CTA, last position of the
// CTA] are zero-filled, so nothing unwritten in the pool reaches an accumulator.  A tile that is wholly masked for a row
// adds exact zeros and rescales by exactly 1, so a row's result does not depend on the rows it shares a CTA with.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t) __cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t) __cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;                       // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x in one instruction (ex2.approx: 2 ulp, -inf -> +0): the probabilities are rounded to bf16 right after
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

constexpr int kMmaRows = 64, kMmaKeys = 64;

struct MmaArgs {
  AttnArgs a;
  const int *seq_start, *seq_len, *seq_past;
  int nsplit;              // > 1: the key tiles of a row block are dealt round-robin to nsplit CTAs (blockIdx.x = block * nsplit + split)
  float* partial;          // nsplit > 1: [rows, H, nsplit, VDIM + 2] = m (log2 units), l, unnormalised o — merged by a second kernel
};

template <int DIM, int VDIM>
__global__ void __launch_bounds__(128, 3) window_attention_mma_kernel(__nv_bfloat16* out, const __nv_bfloat16* q,
                                                                   const __nv_bfloat16* pool, MmaArgs m) {
  constexpr int LDQ = DIM + 8, LDV = VDIM + 8;        // +16 bytes per row: ldmatrix rows fall into distinct banks
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // K [2][64][LDQ] | V [2][64][LDV]; the query tile [64][LDQ] borrows the K ring's second stage until its fragments sit in
  // registers (that stage is first filled inside the key loop)
  __nv_bfloat16* ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* vs = ks + 2 * kMmaKeys * LDQ;
  __nv_bfloat16* qs = ks + kMmaKeys * LDQ;
  __shared__ int64_t key_row[2][kMmaKeys];            // pool row of every key of a stage (-1: zero-fill)
  const AttnArgs& a = m.a;
  const int e = blockIdx.y, g = blockIdx.z;
  const int per = a.H / a.G, len = m.seq_len[e], past = m.seq_past[e], row0 = m.seq_start[e];
  const int split = m.nsplit > 1 ? blockIdx.x % m.nsplit : 0, nsplit = m.nsplit > 1 ? m.nsplit : 1;
  // row blocks are dealt from the END of the portion: the blocks at its start see the fewest keys, so the cheap CTAs
  // fill the last, partial wave of the grid instead of the expensive ones
  const int r0 = ((int) (gridDim.x / nsplit) - 1 - (int) (blockIdx.x / nsplit)) * kMmaRows;   // first (token, head) row of this CTA
  if (r0 >= len * per) return;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, gq = lane / 4, tq = lane % 4;
  const int t_first = r0 / per;
  const int r_last = min(r0 + kMmaRows, len * per) - 1, t_last = r_last / per;
  const int p_last = past + t_last;                     // last position any row of the CTA sees
  const int p_first = past + t_first;
  const int lo_cta = a.window > 0 && p_first - a.window + 1 > 0 ? p_first - a.window + 1 : 0;
  const int E = a.G * DIM + a.GV * VDIM;
  const int* bt = a.block_table + (int64_t) e * a.max_blocks;

  // queries of the CTA's rows (zeros for rows past the sequence's portion)
  for (int i = threadIdx.x; i < kMmaRows * (DIM / 8); i += 128) {
    const int r = i / (DIM / 8), c = (i % (DIM / 8)) * 8;
    const int R = r0 + r, t = R / per, hl = R % per;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < len) v = *reinterpret_cast<const uint4*>(q + ((int64_t) (row0 + t) * a.H + g * per + hl) * DIM + c);
    *reinterpret_cast<uint4*>(qs + r * LDQ + c) = v;
  }
  // the page arithmetic runs once per key and tile (64 threads), not once per 16-byte chunk
  auto locate_tile = [&](int kt, int stage) {
    if (threadIdx.x < kMmaKeys) {
      const int j = kt * kMmaKeys + threadIdx.x;
      key_row[stage][threadIdx.x] = ((j >= lo_cta || j < a.keep) && j <= p_last) ? ((int64_t) bt[j / a.page] * a.page + j % a.page) * E : -1;
    }
  };
  auto load_tile = [&](int stage) {
    __nv_bfloat16* kd = ks + stage * kMmaKeys * LDQ;
    __nv_bfloat16* vd = vs + stage * kMmaKeys * LDV;
    for (int i = threadIdx.x; i < kMmaKeys * (DIM / 8); i += 128) {
      const int jj = i / (DIM / 8), c = (i % (DIM / 8)) * 8;
      const int64_t r = key_row[stage][jj];
      cp_async16(kd + jj * LDQ + c, r >= 0 ? pool + r + g * DIM + c : pool, r >= 0);
    }
    for (int i = threadIdx.x; i < kMmaKeys * (VDIM / 8); i += 128) {
      const int jj = i / (VDIM / 8), c = (i % (VDIM / 8)) * 8;
      const int64_t r = key_row[stage][jj];
      cp_async16(vd + jj * LDV + c, r >= 0 ? pool + r + a.G * DIM + (g / a.vsh) * VDIM + c : pool, r >= 0);
    }
  };
  // the CTA's key tiles in visiting order: those of kept first positions that lie below the window's first tile, then the
  // window's tiles; index i of that list is tile (i < n_kept ? i : wt0 + i - n_kept)
  const int wt0 = lo_cta / kMmaKeys;
  const int keep_lo = a.keep < lo_cta ? a.keep : lo_cta;
  const int n_kept = min((keep_lo + kMmaKeys - 1) / kMmaKeys, wt0);
  const int n_tiles = n_kept + p_last / kMmaKeys - wt0 + 1;
  auto tile_at = [&](int i) { return i < n_kept ? i : wt0 + i - n_kept; };
  const int kt0 = split, kt1 = n_tiles - 1;              // indices into the list from here on
  locate_tile(tile_at(kt0 < n_tiles ? kt0 : 0), 0);

  // the two rows of this thread: warp * 16 + gq and + 8
  int pos_r[2], lo_r[2], head_r[2];
  bool live_r[2];
  float m_r[2], l_r[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int R = r0 + warp * 16 + gq + h * 8, t = R / per;
    live_r[h] = t < len;
    head_r[h] = g * per + R % per;
    pos_r[h] = live_r[h] ? past + t : -1;               // a dead row sees nothing
    lo_r[h] = a.window > 0 && pos_r[h] - a.window + 1 > 0 ? pos_r[h] - a.window + 1 : 0;
    m_r[h] = -INFINITY;
    l_r[h] = 0.f;
    // the sink: a term exp(sink - m) of the denominator without a value; one thread of the row's quad carries it
    // (with the keys split over CTAs the merge kernel adds it instead)
    if (a.sink && live_r[h] && nsplit == 1) { m_r[h] = ld_w(a.sink, a.sink_dtype, head_r[h]) * 1.4426950408889634f; l_r[h] = tq == 0 ? 1.f : 0.f; }
  }
  const float scale2 = a.scale * 1.4426950408889634f;   // scores in units of log 2: exp2f below
  float o[VDIM / 8][4];
#pragma unroll
  for (int n = 0; n < VDIM / 8; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
  __syncthreads();                                      // qs and key_row[0] are written
  if (kt0 <= kt1) load_tile(0);
  cp_async_commit();
  uint32_t qf[DIM / 16][4];
#pragma unroll
  for (int kk = 0; kk < DIM / 16; ++kk)
    ldsm_x4(qf[kk], qs + (warp * 16 + lane % 16) * LDQ + kk * 16 + (lane / 16) * 8);
  if (kt0 + nsplit <= kt1) locate_tile(tile_at(kt0 + nsplit), 1);   // visible behind the loop's first barrier, like the end of the
                                                           // fragment loads from the stage the query tile borrows
  int stage = 0;
  for (int kt = kt0; kt <= kt1; kt += nsplit, stage ^= 1) {
    // ONE barrier per tile: behind it this tile's copies have landed (every thread waited for its own), the other stage
    // has been consumed by every warp, and the pool rows located last trip are visible — so the next tile's copies start here
    cp_async_wait<0>();
    __syncthreads();
    if (kt + nsplit <= kt1) { load_tile(stage ^ 1); cp_async_commit(); }
    if (kt + 2 * nsplit <= kt1) locate_tile(tile_at(kt + 2 * nsplit), stage);   // read by load_tile behind the next barrier
    const __nv_bfloat16* kd = ks + stage * kMmaKeys * LDQ;
    const __nv_bfloat16* vd = vs + stage * kMmaKeys * LDV;
    const int j0 = tile_at(kt) * kMmaKeys;
    float s[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[n][c] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DIM / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {                  // two key groups of 8 per ldmatrix.x4
        uint32_t b[4];
        ldsm_x4(b, kd + (np * 16 + lane % 8 + (lane / 16) * 8) * LDQ + kk * 16 + ((lane / 8) % 2) * 8);
        mma_bf16_16816(s[2 * np], qf[kk], b[0], b[1]);
        mma_bf16_16816(s[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }
    // mask, running maximum
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int h = c >> 1, j = j0 + n * 8 + 2 * tq + (c & 1);
        const float v = ((j >= lo_r[h] || j < a.keep) && j <= pos_r[h]) ? s[n][c] * scale2 : -INFINITY;
        s[n][c] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_r[h], mx[h]);
      corr[h] = m_new == -INFINITY ? 1.f : exp2_fast(m_r[h] - m_new); // nothing seen yet: nothing to rescale
      m_r[h] = m_new;
      mx[h] = m_new == -INFINITY ? 0.f : m_new;                       // exp2f(-inf - 0) = 0 below
    }
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2_fast(s[n][c] - mx[c >> 1]);
        s[n][c] = p;
        rs[c >> 1] += p;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_r[h] = l_r[h] * corr[h] + rs[h];    // per-thread partial sums; the quad is added at the end
    if (corr[0] != 1.f || corr[1] != 1.f) {             // once the running maxima have settled nothing is rescaled
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n) {
        o[n][0] *= corr[0]; o[n][1] *= corr[0]; o[n][2] *= corr[1]; o[n][3] *= corr[1];
      }
    }
#pragma unroll
    for (int kk = 0; kk < kMmaKeys / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int np = 0; np < VDIM / 16; ++np) {
        uint32_t b[4];
        ldsm_x4_trans(b, vd + (kk * 16 + lane % 8 + ((lane / 8) % 2) * 8) * LDV + np * 16 + (lane / 16) * 8);
        mma_bf16_16816(o[2 * np], pa, b[0], b[1]);
        mma_bf16_16816(o[2 * np + 1], pa, b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();
  if (nsplit > 1) {
    // unnormalised partial result of this CTA's share of the keys
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float l = l_r[h];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      if (!live_r[h]) continue;
      const int R = r0 + warp * 16 + gq + h * 8, t = R / per;
      float* dst = m.partial + (((int64_t) (row0 + t) * a.H + head_r[h]) * nsplit + split) * (VDIM + 2);
      if (tq == 0) { dst[0] = m_r[h]; dst[1] = l; }
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n) {
        dst[2 + n * 8 + 2 * tq] = o[n][2 * h];
        dst[2 + n * 8 + 2 * tq + 1] = o[n][2 * h + 1];
      }
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = l_r[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    l_r[h] = l;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!live_r[h]) continue;
    const int R = r0 + warp * 16 + gq + h * 8, t = R / per;
    float f = 1.f / l_r[h];
    if (a.gate) f *= 1.f / (1.f + expf(-a.gate[(int64_t) (row0 + t) * a.ldg + head_r[h]]));
    const int64_t dst = ((int64_t) (row0 + t) * a.H + head_r[h]) * VDIM;
    if (a.out_f32) {
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n)
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + dst + n * 8 + 2 * tq) = make_float2(o[n][2 * h] * f, o[n][2 * h + 1] * f);
    } else {
#pragma unroll
      for (int n = 0; n < VDIM / 8; ++n)
        *reinterpret_cast<__nv_bfloat162*>(out + dst + n * 8 + 2 * tq) = __floats2bfloat162_rn(o[n][2 * h] * f, o[n][2 * h + 1] * f);
    }
  }
}

// one CTA per (row, head): splits merged in index order, the sink added once, gate applied
__global__ void window_attention_merge_kernel(__nv_bfloat16* out, const float* partial, AttnArgs a, int nsplit, int vdim) {
  __shared__ float w_s[32];                    // weight of every split: 2^(m_s - M), 0 for a split that saw nothing
  __shared__ float f_s;
  const int row = blockIdx.x, head = blockIdx.y;
  const float* src = partial + ((int64_t) row * a.H + head) * nsplit * (vdim + 2);
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const float ms = s < nsplit ? src[s * (vdim + 2)] : -INFINITY, ls = s < nsplit ? src[s * (vdim + 2) + 1] : 0.f;
    const float sink2 = a.sink ? ld_w(a.sink, a.sink_dtype, head) * 1.4426950408889634f : -INFINITY;
    const float M = fmaxf(warp_max(ms), sink2);                  // finite: the row sees at least itself
    const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
    w_s[s] = w;
    float l = ls * w;
    // fixed order: lanes are added in a tree whose shape does not depend on the data
    l = warp_sum(l) + (a.sink ? exp2f(sink2 - M) : 0.f);
    if (s == 0) {
      float f = 1.f / l;
      if (a.gate) f *= 1.f / (1.f + expf(-a.gate[(int64_t) row * a.ldg + head]));
      f_s = f;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) acc = fmaf(src[s * (vdim + 2) + 2 + c], w_s[s], acc);
    const int64_t o = ((int64_t) row * a.H + head) * vdim + c;
    if (a.out_f32) reinterpret_cast<float*>(out)[o] = acc * f_s;
    else out[o] = __float2bfloat16_rn(acc * f_s);
  }
}

template <int DIM, int VDIM>
int launch_window_mma(__nv_bfloat16* out, const __nv_bfloat16* q, const __nv_bfloat16* pool, const MmaArgs& m, int seqs,
                      int max_len, cudaStream_t s) {
  constexpr size_t smem = ((size_t) 2 * kMmaKeys * (DIM + 8) + 2 * kMmaKeys * (VDIM + 8)) * 2;
  static bool raised = false;
  if (!raised && smem > 48 * 1024) {
    TB_CHECK_CUDA(cudaFuncSetAttribute(window_attention_mma_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    raised = true;
  }
  const int per = m.a.H / m.a.G;
  const int nsplit = m.nsplit > 1 ? m.nsplit : 1;
  dim3 grid((((int64_t) max_len * per + kMmaRows - 1) / kMmaRows) * nsplit, seqs, m.a.G);
  window_attention_mma_kernel<DIM, VDIM><<<grid, 128, smem, s>>>(out, q, pool, m);
  return 0;
}

// the (dim, vdim) pairs the tensor-core kernel is built for
#define TB_WINDOW_MMA_SHAPES(X) X(32, 16) X(32, 32) X(64, 32) X(64, 64) X(64, 128) X(96, 96) X(128, 64) X(128, 128)

}  // namespace
}  // namespace tb

using namespace tb;

extern "C" int tb_qkv_conv_rope_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* conv_w,
                                       int w_dtype, const float* state, const float* table, int dims, const int* tok_seq,
                                       const int* tok_pos, const int* seq_start, const int* seq_past, const int* seq_slot,
                                       const int* block_table, int max_blocks, int page, int rows, int heads, int kv_heads,
                                       int dim, int vdim, int taps, float* state_rw, const int* seq_len, tb_stream_t stream) {
  if (!q_out || !pool || !proj || !conv_w || !tok_seq || !tok_pos || !seq_start || !seq_past || !seq_slot || !block_table)
    return -1;
  if ((dtype != TB_DT_F32 && dtype != TB_DT_BF16) || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16)) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || taps < 1 || taps > kMaxTaps || page <= 0 ||
      rows < 0 || dims < 0 || dims % 2 || dims > dim || (dims > 0 && (dim % 2 || !table)) || (taps > 1 && !state))
    return -1;
  if (rows == 0) return 0;
  if (state_rw && (state_rw != state || !seq_len)) return -1;
  QkvArgs a{proj, ldp, conv_w, w_dtype, state, table, tok_seq, tok_pos, seq_start, seq_past, seq_slot, block_table,
            max_blocks, page, rows, heads, kv_heads, dim, vdim, dims, taps, state_rw, seq_len};
  // one CTA per row when the rows alone fill the chip; a step of few rows also spreads a row's channels over CTAs
  const int C = heads * dim + kv_heads * (dim + vdim);
  const int ysplit = rows >= 296 ? 1 : std::min((C + 511) / 512, (296 + rows - 1) / rows);
  const dim3 grid(rows, ysplit);
  if (dtype == TB_DT_F32) qkv_conv_rope_append_kernel<float><<<grid, 256, 0, (cudaStream_t) stream>>>((float*) q_out, (float*) pool, a);
  else qkv_conv_rope_append_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t) stream>>>((__nv_bfloat16*) q_out, (__nv_bfloat16*) pool, a);
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_qk_conv_norm_rope_append(void* q_out, void* pool, int dtype, const float* proj, int64_t ldp, const void* conv_w,
                                           const void* norm_q, const void* norm_k, int w_dtype, float eps, const float* state,
                                           const float* table, int dims, const int* tok_seq, const int* tok_pos, const int* seq_start,
                                           const int* seq_past, const int* seq_slot, const int* block_table, int max_blocks, int page,
                                           int rows, int heads, int kv_heads, int dim, int vdim, int taps, int tied_values,
                                           float* state_rw, const int* seq_len, tb_stream_t stream) {
  if (!q_out || !pool || !proj || !tok_seq || !tok_pos || !seq_start || !seq_past || !seq_slot || !block_table) return -1;
  if ((dtype != TB_DT_F32 && dtype != TB_DT_BF16) || (w_dtype != TB_DT_F32 && w_dtype != TB_DT_BF16)) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || taps < 1 || taps > kMaxTaps || page <= 0 ||
      rows < 0 || dims < 0 || dims % 2 || dims > dim || (dims > 0 && (dim % 2 || !table)) || (taps > 1 && (!state || !conv_w)) ||
      (tied_values && vdim != dim) || (!norm_q != !norm_k))
    return -1;
  if (rows == 0) return 0;
  if (state_rw && (state_rw != state || !seq_len)) return -1;
  const int C = (heads + kv_heads) * dim + (tied_values ? 0 : kv_heads * vdim);
  const size_t smem = (size_t) C * sizeof(float);
  if (smem > 200 * 1024) return -2;
  QkNormArgs n{{proj, ldp, conv_w, w_dtype, state, table, tok_seq, tok_pos, seq_start, seq_past, seq_slot, block_table, max_blocks,
                page, rows, heads, kv_heads, dim, vdim, dims, taps, state_rw, seq_len},
               norm_q, norm_k, eps, tied_values ? 1 : 0};
  static size_t raised_f = 48 * 1024, raised_b = 48 * 1024;
  if (dtype == TB_DT_F32) {
    if (smem > raised_f) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(qk_conv_norm_rope_append_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_f = smem;
    }
    qk_conv_norm_rope_append_kernel<float><<<rows, 256, smem, (cudaStream_t) stream>>>((float*) q_out, (float*) pool, n);
  } else {
    if (smem > raised_b) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(qk_conv_norm_rope_append_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_b = smem;
    }
    qk_conv_norm_rope_append_kernel<__nv_bfloat16><<<rows, 256, smem, (cudaStream_t) stream>>>((__nv_bfloat16*) q_out, (__nv_bfloat16*) pool, n);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int tb_window_attention_tensor_cores(int dtype, int heads, int kv_heads, int dim, int vdim) {
  if (dtype != TB_DT_BF16 || heads <= 0 || kv_heads <= 0 || heads % kv_heads) return 0;
#define X(D, V) if (dim == D && vdim == V) return 1;
  TB_WINDOW_MMA_SHAPES(X)
#undef X
  return 0;
}

extern "C" int tb_window_attention(void* out, const void* q, const void* pool, int dtype, const float* gate, int64_t ldg,
                                   const void* sink, int sink_dtype, const int* tok_seq, const int* tok_pos,
                                   const int* block_table, const int* seq_start, const int* seq_len, const int* seq_past,
                                   int seqs, int max_len, int max_blocks, int page, int rows, int heads, int kv_heads,
                                   int dim, int vdim, float scale, int window, int mode, int nsplit, float* workspace,
                                   tb_stream_t stream) {
  return tb_window_attention_shared_values(out, 0, q, pool, dtype, gate, ldg, sink, sink_dtype, tok_seq, tok_pos, block_table,
                                           seq_start, seq_len, seq_past, seqs, max_len, max_blocks, page, rows, heads, kv_heads, 1,
                                           dim, vdim, scale, window, 0, mode, nsplit, workspace, stream);
}

extern "C" int tb_window_attention_shared_values(void* out, int out_f32, const void* q, const void* pool, int dtype,
                                                 const float* gate, int64_t ldg, const void* sink, int sink_dtype,
                                                 const int* tok_seq, const int* tok_pos, const int* block_table,
                                                 const int* seq_start, const int* seq_len, const int* seq_past, int seqs,
                                                 int max_len, int max_blocks, int page, int rows, int heads, int kv_heads,
                                                 int v_share, int dim, int vdim, float scale, int window, int keep_first, int mode,
                                                 int nsplit, float* workspace, tb_stream_t stream) {
  if (!out || !q || !pool || !tok_seq || !tok_pos || !block_table || keep_first < 0) return -1;
  if (v_share <= 0 || kv_heads % v_share) return -1;
  if (dtype != TB_DT_F32 && dtype != TB_DT_BF16) return -1;
  if (sink && sink_dtype != TB_DT_F32 && sink_dtype != TB_DT_BF16) return -1;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 || vdim > 32 * kMaxVPerLane || page <= 0 ||
      rows < 0 || window < 0 || kv_heads > 65535)
    return -1;
  if (rows == 0) return 0;
  AttnArgs a{gate, ldg, sink, sink_dtype, tok_seq, tok_pos, block_table, max_blocks, page, heads, kv_heads, dim, vdim,
             window, scale, v_share, kv_heads / v_share, out_f32 ? 1 : 0, window > 0 ? keep_first : 0};
  cudaStream_t s = (cudaStream_t) stream;
  if (mode == 0 && seq_start && seq_len && seq_past && seqs > 0 && max_len > 0 && seqs <= 65535 &&
      tb_window_attention_tensor_cores(dtype, heads, kv_heads, dim, vdim) && (uintptr_t) q % 16 == 0 && (uintptr_t) pool % 16 == 0) {
    if (nsplit > 1 && !workspace) return -1;
    MmaArgs m{a, seq_start, seq_len, seq_past, nsplit > 1 ? nsplit : 1, workspace};
#define X(D, V)                                                                                                     \
  if (dim == D && vdim == V) {                                                                                      \
    const int rc = launch_window_mma<D, V>((__nv_bfloat16*) out, (const __nv_bfloat16*) q, (const __nv_bfloat16*) pool, m, \
                                           seqs, max_len, s);                                                       \
    if (rc) return rc;                                                                                              \
  }
    TB_WINDOW_MMA_SHAPES(X)
#undef X
    TB_CHECK_CUDA(cudaGetLastError());
    if (nsplit > 1) {
      window_attention_merge_kernel<<<dim3(rows, heads), vdim < 128 ? 64 : 128, 0, s>>>((__nv_bfloat16*) out, workspace, a, nsplit, vdim);
      TB_CHECK_CUDA(cudaGetLastError());
    }
    return 0;
  }
  const size_t smem = ((size_t) kTile * (dim + 1) + (size_t) kTile * vdim + (size_t) kWarps * dim) * sizeof(float);
  if (smem > 220 * 1024) return -2;
  dim3 grid(rows, kv_heads, (heads / kv_heads + kWarps - 1) / kWarps);
  static size_t raised_f = 48 * 1024, raised_b = 48 * 1024;
  if (dtype == TB_DT_F32) {
    if (smem > raised_f) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(window_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_f = smem;
    }
    window_attention_kernel<float><<<grid, kWarps * 32, smem, s>>>((float*) out, (const float*) q, (const float*) pool, a);
  } else {
    if (smem > raised_b) {
      TB_CHECK_CUDA(cudaFuncSetAttribute(window_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
      raised_b = smem;
    }
    window_attention_kernel<__nv_bfloat16><<<grid, kWarps * 32, smem, s>>>((__nv_bfloat16*) out, (const __nv_bfloat16*) q,
                                                                             (const __nv_bfloat16*) pool, a);
  }
  TB_CHECK_CUDA(cudaGetLastError());
  return 0;
}
