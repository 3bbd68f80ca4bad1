// attn_heads.cu -- softmax attention with per-head keys and values for the layer-list families, any head width, fp32 or
// bf16 cache.  What is optional is a parameter (HeadsGeom), so that one set of kernels serves every mixer of this kind:
//   rotary positions on interleaved pairs of the first rot_dims entries of every query / key head,
//   a short causal convolution over time on every q / k / v channel (the last projected rows of a sequence live in a
//     ring of `taps` rows per sequence slot, indexed by position mod taps: nothing is shifted, a slot that is used again
//     needs no clearing since positions below 0 read as zero, and a token never overwrites a row it reads, so a step
//     that is run twice from the same bookkeeping -- the warm-up ahead of a graph capture -- leaves the same state),
//   q and k heads divided by their root mean square,
//   a linear distance penalty slope_a * (i - j) with slope_a = 2^(-slope_exp (a + 1) / heads),
//   a sliding window that also keeps the first tokens of the sequence,
//   value mixing v <- (1 - lam) v + lam v_first with the values another layer computed for the same token,
//   mixing of the heads' softmax weights by a heads x heads matrix, and a sigmoid gate per head.
//
// Cache: two regions per layer, K rows [kv_heads * dim] and V rows [kv_heads * vdim] per token, in pages of block_size
// tokens; the element type is the engine's operand type.
//
// Arithmetic is fp32 everywhere (angles in fp64 before one rounding): scores, softmax, weights, norms, the convolution and
// its ring.  Only what is stored in a bf16 cache or handed to a bf16 product is rounded.
//
// Kernels:
//   heads_finish      what follows the fused q | k | v (| gate) projection, one CTA per (token, head): bias, convolution, rotary or
//                     unit-RMS norm, value mixing, cache row write, fp32 queries
//   conv_tail_store   the ring update, after every token of the step has read the ring
//   heads_attention   one warp per (query token, head) for prompt portions; for a decode step the eight warps of a CTA
//                     split the keys of one (sequence, head) and merge.  Tiles of 32 keys: lane j scores key j, then lane
//                     c accumulates value columns c, c + 32, ...  Key tiles that the window hides are never visited.
//                     With weight mixing ("cross") a query head's weights are applied to the values of EVERY key/value head
//                     (out [heads][kv_heads * vdim], normalised per head), because the mixed output of head a is
//                     sum_b talk[a][b] * (weights of head b applied to the values of a's key/value head)
//   heads_attention_mma   bf16 caches and prompt portions, head sizes in multiples of 16 / 8: the same pass on warp-level tensor-core
//                     MMAs, 64 query tokens of one head per CTA (see at the kernel)
//   talk_gate         that sum, times the gate, rounded to the operand type
#include <mma.h>

#include "kernels.h"

#define B2_TRY_RC(expr)      \
  do {                      \
    int _r = (expr);        \
    if (_r != 0) return _r; \
  } while (0)

namespace b2 {

namespace {

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ void pair_cos_sin(int pos, int i, int dims, float base, float* c, float* s) {
  const double f = exp2(-2.0 * (double)i / (double)dims * log2((double)base));
  double sd, cd;
  sincos((double)pos * f, &sd, &cd);
  *c = (float)cd;
  *s = (float)sd;
}

// Element index of (slot, key/value head, dim) in the page layout of the GQA kernels (attn_decode.cu, attn_prefill_tc.cu): pages of 16
// tokens, [page][kv_head][16][128], the 16-byte chunks of a token row XOR-swizzled by the row (kv_swizzled_chunk).
__device__ __forceinline__ size_t swizzled_index(int slot, int kvh, int kv_heads, int d) {
  const int page = slot >> 4, r = slot & 15;
  return (((size_t)page * kv_heads + kvh) * 16 + r) * 128 + (size_t)kv_swizzled_chunk(r, d >> 3) * 8 + (d & 7);
}

// A CTA takes `upc` heads of one token, counted through the query heads, then the key heads, then the value heads, one warp per
// head at a time: all of them for prompt-sized steps (the token's cosines and sines are formed once), four when the step has few
// tokens.  proj [T][ld] fp32: q (heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim) | anything else.
template <typename TC>
__global__ void __launch_bounds__(128) heads_finish_kernel(const float* __restrict__ proj, int ld, HeadsGeom g, const float* __restrict__ bias,
                                                           const float* __restrict__ conv_w, const float* __restrict__ ring,
                                                           const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_first,
                                                           const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                                                           int vmix_mode, const float* __restrict__ vmix_lambda, float* __restrict__ v_first,
                                                           float* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache, int upc,
                                                           bf16* __restrict__ q_bf16) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = slots[t];
  if (slot < 0) return;  // padding row of a decode bucket
  const int pos = positions[t];
  const int nq = g.heads * g.dim, nk = g.kv_heads * g.dim, nv = g.kv_heads * g.vdim, C = nq + nk + nv;
  const int units = g.heads + 2 * g.kv_heads, u_lo = blockIdx.y * upc, u_hi = min(units, u_lo + upc);
  const int maxw = max(g.dim, g.vdim);
  float* y = sm + (size_t)warp * maxw;      // this warp's head after bias and convolution
  float* cs = sm + (size_t)4 * maxw;        // [rot_dims] cos | sin
  const int rhalf = g.rot_dims / 2;
  if (u_lo < g.heads + g.kv_heads)
    for (int i = threadIdx.x; i < rhalf; i += 128) pair_cos_sin(pos, i, g.rot_dims, g.rot_base, &cs[i], &cs[rhalf + i]);
  __syncthreads();
  const float* row = proj + (size_t)t * ld;
  for (int u = u_lo + warp; u < u_hi; u += 4) {
    const bool is_v = u >= g.heads + g.kv_heads;
    const int width = is_v ? g.vdim : g.dim;
    const int c0 = is_v ? nq + nk + (u - g.heads - g.kv_heads) * g.vdim : u * g.dim;   // first channel of this head in q | k | v
    const int half = is_v ? 0 : rhalf;
    __syncwarp();   // the head before this one is out of y
    if (g.conv_taps > 0) {
      const int taps = g.conv_taps, back = t - row_first[t];
      const float* rg = ring + (size_t)row_seq[t] * taps * C;
      for (int i = lane; i < width; i += 32) {
        const int c = c0 + i;
        const float b = bias ? bias[c] : 0.f;
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {          // y_t = sum_j w[c][j] * u_(t - taps + 1 + j), oldest first
          const int d = taps - 1 - j;             // how far back
          float uu = 0.f;
          if (d <= back) uu = (row - (size_t)d * ld)[c] + b;
          else if (pos - d >= 0) uu = rg[(size_t)((pos - d) % taps) * C + c];
          acc = fmaf(conv_w[(size_t)c * taps + j], uu, acc);
        }
        y[i] = acc;
      }
    } else {
      for (int i = lane; i < width; i += 32) y[i] = row[c0 + i] + (bias ? bias[c0 + i] : 0.f);
    }
    __syncwarp();
    if (is_v) {
      const int vc = c0 - nq - nk;   // first column of this head among the values
      float* vf = v_first ? v_first + (size_t)t * nv + vc : nullptr;
      TC* vr = v_cache + (size_t)slot * nv + vc;
      const float lam = vmix_mode == 2 ? *vmix_lambda : 0.f;
      for (int i = lane; i < width; i += 32) {
        float v = y[i];
        if (vmix_mode == 1) vf[i] = v;
        else if (vmix_mode == 2) v = (1.0f - lam) * v + lam * vf[i];
        if (g.swizzled) stf(v_cache + swizzled_index(slot, u - g.heads - g.kv_heads, g.kv_heads, i), v);
        else stf(vr + i, v);
      }
      continue;
    }
    float r = 1.0f;
    if (g.unit_qk) {
      float ss = 0.f;
      for (int i = lane; i < width; i += 32) ss = fmaf(y[i], y[i], ss);
      ss = warp_sum(ss);
      r = 1.0f / sqrtf(ss / (float)width + g.eps);
    }
    // pairs below rot_dims turn, the rest passes; one lane per pair (an odd last element passes alone)
    const bool is_q = u < g.heads;
    float* qo = q_out + (size_t)t * nq + c0;
    TC* kr = k_cache + (size_t)slot * nk + (c0 - nq);
    for (int p = lane; p < (width + 1) / 2; p += 32) {
      const bool two = 2 * p + 1 < width;
      float a = y[2 * p] * r, b = two ? y[2 * p + 1] * r : 0.f;
      if (p < half) {
        const float ra = a * cs[p] - b * cs[half + p], rb = b * cs[p] + a * cs[half + p];
        a = ra;
        b = rb;
      }
      if (is_q) {
        if (q_bf16 != nullptr) {   // the GQA tensor-core kernels take bf16 queries
          *reinterpret_cast<uint32_t*>(q_bf16 + (size_t)t * nq + c0 + 2 * p) = pack_bf16x2(a, b);
        } else {
          qo[2 * p] = a;
          if (two) qo[2 * p + 1] = b;
        }
      } else if (g.swizzled) {
        const size_t at = swizzled_index(slot, u - g.heads, g.kv_heads, 2 * p);
        stf(k_cache + at, a);
        stf(k_cache + at + 1, b);
      } else {
        stf(kr + 2 * p, a);
        if (two) stf(kr + 2 * p + 1, b);
      }
    }
  }
}

// Whole-row norms: q (all heads at once) and k (all key heads at once) are each divided by the root mean square of the row and
// multiplied by a gain per entry; v passes.  One CTA of NT threads per token (wide CTAs for steps of few tokens).
template <typename TC, int NT>
__global__ void __launch_bounds__(NT) heads_finish_rownorm_kernel(const float* __restrict__ proj, int ld, HeadsGeom g, const float* __restrict__ bias,
                                                                   const float* __restrict__ qk_gain, const int32_t* __restrict__ slots,
                                                                   float* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                                                   bf16* __restrict__ q_bf16) {
  __shared__ float red[2][NT / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = slots[t];
  if (slot < 0) return;
  const int nq = g.heads * g.dim, nk = g.kv_heads * g.dim, nv = g.kv_heads * g.vdim;
  const float* row = proj + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += NT) {
    const float v = row[i] + (bias ? bias[i] : 0.f);
    sq = fmaf(v, v, sq);
  }
  for (int i = threadIdx.x; i < nk; i += NT) {
    const float v = row[nq + i] + (bias ? bias[nq + i] : 0.f);
    sk = fmaf(v, v, sk);
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) {
    red[0][warp] = sq;
    red[1][warp] = sk;
  }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) {
    tq += red[0][w];
    tk += red[1][w];
  }
  const float rq = 1.0f / sqrtf(tq / (float)nq + g.eps);
  const float rk = 1.0f / sqrtf(tk / (float)nk + g.eps);
  if (g.swizzled) {   // the page layout of the GQA kernels (128-wide heads), queries as bf16
    for (int i = threadIdx.x; i < nq; i += NT) q_bf16[(size_t)t * nq + i] = __float2bfloat16_rn((row[i] + (bias ? bias[i] : 0.f)) * rq * qk_gain[i]);
    for (int i = threadIdx.x; i < nk; i += NT)
      stf(k_cache + swizzled_index(slot, i >> 7, g.kv_heads, i & 127), (row[nq + i] + (bias ? bias[nq + i] : 0.f)) * rk * qk_gain[nq + i]);
    for (int i = threadIdx.x; i < nv; i += NT) stf(v_cache + swizzled_index(slot, i >> 7, g.kv_heads, i & 127), row[nq + nk + i] + (bias ? bias[nq + nk + i] : 0.f));
    return;
  }
  for (int i = threadIdx.x; i < nq; i += NT) q_out[(size_t)t * nq + i] = (row[i] + (bias ? bias[i] : 0.f)) * rq * qk_gain[i];
  for (int i = threadIdx.x; i < nk; i += NT) stf(k_cache + (size_t)slot * nk + i, (row[nq + i] + (bias ? bias[nq + i] : 0.f)) * rk * qk_gain[nq + i]);
  for (int i = threadIdx.x; i < nv; i += NT) stf(v_cache + (size_t)slot * nv + i, row[nq + nk + i] + (bias ? bias[nq + nk + i] : 0.f));
}

__global__ void __launch_bounds__(128) conv_tail_store_kernel(const float* __restrict__ proj, int ld, int C, int taps,
                                                              const float* __restrict__ bias, float* __restrict__ ring,
                                                              const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_end,
                                                              const int32_t* __restrict__ positions, const int32_t* __restrict__ slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (slots[t] < 0) return;
  if (row_end[t] - 1 - t >= taps) return;  // a later token of the same portion owns this ring row
  float* dst = ring + ((size_t)row_seq[t] * taps + positions[t] % taps) * C;
  const float* row = proj + (size_t)t * ld;
  for (int c = threadIdx.x; c < C; c += 128) dst[c] = row[c] + (bias ? bias[c] : 0.f);
}

constexpr int HA_WARPS = 8;

// Visible key tiles of query position i: tiles [0, nA) cover the kept first tokens, tiles [tB, i / 32] the window.
struct TileRange {
  int nA, tB, total;
};
__device__ __forceinline__ TileRange visible_tiles(int i, int window, int keep_first) {
  TileRange r;
  const int last = i >> 5;
  if (window <= 0) {
    r.nA = 0; r.tB = 0; r.total = last + 1;
    return r;
  }
  const int lo = max(i - window + 1, 0);
  const int endA = min(keep_first, lo);  // kept keys below the window
  r.nA = (endA + 31) >> 5;
  r.tB = max(lo >> 5, r.nA);
  r.total = r.nA + (last - r.tB + 1);
  return r;
}

// NV = ceil(value columns / 32).  DECODE: a CTA is one (sequence, head), its warps take the visible key tiles round robin;
// else a CTA is eight query tokens of one tile and one head, a warp per token.
// VEC (bf16 caches, dim a multiple of 8, value columns a multiple of 64): a lane reads its key's row 16 bytes at a time and owns
// value columns in pairs (64 n + 2 lane, + 1), one 4-byte load per pair; otherwise element by element, columns lane + 32 n.
template <bool VEC>
__device__ __forceinline__ int ha_col(int n, int lane) { return VEC ? 64 * (n >> 1) + 2 * lane + (n & 1) : lane + 32 * n; }

template <typename TC, typename TO, int NV, bool DECODE, bool VEC>
__global__ void __launch_bounds__(HA_WARPS * 32) heads_attention_kernel(const float* __restrict__ q, const TC* __restrict__ k_cache,
                                                                        const TC* __restrict__ v_cache, HeadsGeom g,
                                                                        const int32_t* __restrict__ block_table, int bt_stride, int block_size,
                                                                        const PrefillTile* __restrict__ tiles, const int32_t* __restrict__ positions,
                                                                        const int32_t* __restrict__ seq_lens, TO* __restrict__ out, int cross_cols) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a = blockIdx.y, kvh = a / (g.heads / g.kv_heads);
  const int D = g.dim, krow = g.kv_heads * g.dim, vrow = g.kv_heads * g.vdim;
  // the value columns this CTA weights: its key/value head's, or with cross a run of cross_cols columns of the whole value row
  const int voff = g.cross ? (int)blockIdx.z * cross_cols : kvh * g.vdim;
  const int VW = g.cross ? min(cross_cols, vrow - voff) : g.vdim;
  int t, pos, bt_row;
  bool live;
  if (DECODE) {
    t = blockIdx.x;
    bt_row = t;
    live = seq_lens[t] > 0;
    pos = live ? positions[t] : 0;
  } else {
    const PrefillTile tl = tiles[blockIdx.x >> 3];
    const int r = ((blockIdx.x & 7) << 3) + warp;
    live = r < tl.nrows;
    t = tl.q_row0 + r;
    pos = tl.q_pos0 + r;
    bt_row = tl.bt_row;
    if (((blockIdx.x & 7) << 3) >= tl.nrows) return;
  }
  float* qs = sm + (DECODE ? 0 : (size_t)warp * D);
  if (live) {
    const float* qr = q + ((size_t)t * g.heads + a) * D;
    if (DECODE) {
      for (int d = threadIdx.x; d < D; d += HA_WARPS * 32) qs[d] = qr[d];
    } else {
      for (int d = lane; d < D; d += 32) qs[d] = qr[d];
    }
  }
  if (DECODE) __syncthreads();
  else __syncwarp();
  const float slope = g.slopes ? (float)exp2(-(double)g.slope_exp * (double)(a + 1) / (double)g.heads) : 0.f;
  float m = -INFINITY, l = 0.f, acc[NV];
#pragma unroll
  for (int n = 0; n < NV; ++n) acc[n] = 0.f;
  if (live) {
    const TileRange tr = visible_tiles(pos, g.window, g.keep_first);
    const int32_t* bt = block_table + (size_t)bt_row * bt_stride;
    const int lo = g.window > 0 ? pos - g.window + 1 : 0;
    for (int vi = DECODE ? warp : 0; vi < tr.total; vi += DECODE ? HA_WARPS : 1) {
      const int tile = vi < tr.nA ? vi : tr.tB + (vi - tr.nA);
      const int j = (tile << 5) + lane;
      const bool vis = j <= pos && (g.window <= 0 || j >= lo || j < g.keep_first);
      float s = -INFINITY;
      size_t slot = 0;
      if (vis) {
        slot = (size_t)bt[j / block_size] * block_size + j % block_size;
        const TC* kr = k_cache + slot * krow + (size_t)kvh * D;
        float dot = 0.f;
        if (VEC) {
          const uint4* kp = reinterpret_cast<const uint4*>(kr);
          for (int d8 = 0; d8 < D / 8; ++d8) {
            const uint4 u = kp[d8];
            const float4 qa = *reinterpret_cast<const float4*>(qs + 8 * d8), qb = *reinterpret_cast<const float4*>(qs + 8 * d8 + 4);
            dot = fmaf(qa.x, bf16lo(u.x), dot); dot = fmaf(qa.y, bf16hi(u.x), dot);
            dot = fmaf(qa.z, bf16lo(u.y), dot); dot = fmaf(qa.w, bf16hi(u.y), dot);
            dot = fmaf(qb.x, bf16lo(u.z), dot); dot = fmaf(qb.y, bf16hi(u.z), dot);
            dot = fmaf(qb.z, bf16lo(u.w), dot); dot = fmaf(qb.w, bf16hi(u.w), dot);
          }
        } else {
          for (int d = 0; d < D; ++d) dot = fmaf(qs[d], ldf(kr + d), dot);
        }
        s = dot * g.scale - slope * (float)(pos - j);
      }
      const float mt = warp_max(s);  // finite: a visited tile holds at least one visible key
      const float mn = fmaxf(m, mt);
      const float corr = expf(m - mn);  // exp(-inf) = 0 on the first tile
      const float p = vis ? expf(s - mn) : 0.f;
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int n = 0; n < NV; ++n) acc[n] *= corr;
      m = mn;
      unsigned mask = __ballot_sync(0xffffffffu, vis);
      if (VEC) {
        // every key of the tile, eight at a time so that their loads are in flight together; a key that is not seen has
        // weight 0 and slot 0 (the null page: zeros)
        const unsigned slot32 = (unsigned)slot;
#pragma unroll 1
        for (int j0 = 0; j0 < 32; j0 += 8) {
          if (((mask >> j0) & 0xffu) == 0) continue;
          uint32_t u[8][(NV + 1) / 2];
          float pj[8];
#pragma unroll
          for (int x = 0; x < 8; ++x) {
            pj[x] = __shfl_sync(0xffffffffu, p, j0 + x);
            const size_t sj = __shfl_sync(0xffffffffu, slot32, j0 + x);
            const TC* vr = v_cache + sj * vrow + voff;
#pragma unroll
            for (int n = 0; n < NV; n += 2) u[x][n >> 1] = *reinterpret_cast<const uint32_t*>(vr + 32 * n + 2 * lane);
          }
#pragma unroll
          for (int x = 0; x < 8; ++x) {
#pragma unroll
            for (int n = 0; n < NV; n += 2) {
              acc[n] = fmaf(pj[x], bf16lo(u[x][n >> 1]), acc[n]);
              if (n + 1 < NV) acc[n + 1] = fmaf(pj[x], bf16hi(u[x][n >> 1]), acc[n + 1]);
            }
          }
        }
        mask = 0;
      }
      while (mask) {
        const int jj = __ffs(mask) - 1;
        mask &= mask - 1;
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const size_t sj = __shfl_sync(0xffffffffu, (unsigned long long)slot, jj);
        const TC* vr = v_cache + sj * vrow + voff;
        {
#pragma unroll
          for (int n = 0; n < NV; ++n) {
            const int c = lane + 32 * n;
            if (c < VW) acc[n] = fmaf(pj, ldf(vr + c), acc[n]);
          }
        }
      }
    }
  }
  TO* orow = g.cross ? out + ((size_t)t * g.heads + a) * vrow + voff : out + ((size_t)t * g.heads + a) * g.vdim;
  if (!DECODE) {
    if (!live) return;
    const float inv = 1.0f / l;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int c = ha_col<VEC>(n, lane);
      if (c < VW) stf(orow + c, acc[n] * inv);
    }
    return;
  }
  // merge the warps' partial sums in warp order
  float* ms = sm + D;            // [8] maxima, [8] sums, [8][VW] accumulators
  float* ls = ms + HA_WARPS;
  float* as = ls + HA_WARPS;
  if (lane == 0) {
    ms[warp] = m;
    ls[warp] = l;
  }
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int c = ha_col<VEC>(n, lane);
    if (c < VW) as[(size_t)warp * VW + c] = acc[n];
  }
  __syncthreads();
  float M = -INFINITY;
  for (int w = 0; w < HA_WARPS; ++w) M = fmaxf(M, ms[w]);
  float L = 0.f;
  float f[HA_WARPS];
  for (int w = 0; w < HA_WARPS; ++w) {
    f[w] = ms[w] == -INFINITY ? 0.f : expf(ms[w] - M);
    L = fmaf(ls[w], f[w], L);
  }
  const float inv = live && L > 0.f ? 1.0f / L : 0.f;
  for (int c = threadIdx.x; c < VW; c += HA_WARPS * 32) {
    float o = 0.f;
    for (int w = 0; w < HA_WARPS; ++w) o = fmaf(as[(size_t)w * VW + c], f[w], o);
    stf(orow + c, o * inv);
  }
}

// out[t][a][d] = sigmoid(gate[t][a]) * sum_b talk[a][b] * cross[t][b][kv(a) * vdim + d]
template <typename TX>
__global__ void __launch_bounds__(128) talk_gate_kernel(const float* __restrict__ cross, const float* __restrict__ talk,
                                                        const float* __restrict__ gate, int gate_ld, TX* __restrict__ out, int heads,
                                                        int kv_heads, int vdim) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, rep = heads / kv_heads, vrow = kv_heads * vdim;
  const float* cr = cross + (size_t)t * heads * vrow;
  for (int i = blockIdx.y * 128 + threadIdx.x; i < heads * vdim; i += 128 * gridDim.y) {
    const int a = i / vdim, d = i - a * vdim, col = (a / rep) * vdim + d;
    float o = 0.f;
    for (int b = 0; b < heads; ++b) o = fmaf(talk[a * heads + b], cr[(size_t)b * vrow + col], o);
    const float gl = gate ? gate[(size_t)t * gate_ld + a] : 0.f;
    const float gv = gate ? 1.0f / (1.0f + expf(-gl)) : 1.0f;
    stf(out + (size_t)t * heads * vdim + i, o * gv);
  }
}


// ---- bf16 caches, prompt portions: 64 query tokens of one head per CTA on warp-level tensor-core MMAs ----
// Four warps of 16 query rows; key tiles of 64 in shared memory.  S = Q.K^T (m16n8k16, fp32 accumulators), the scale, the
// distance penalty and the mask in fp32 on the accumulator fragments, online softmax with the row statistics in registers, P rounded
// to bf16 as the A operand of O += P.V (V fragments through ldmatrix.trans), row sums from the unrounded weights.  Key tiles
// run from position 0 upwards whatever the batch holds, and tiles that no row of the CTA can see (between the kept first
// tokens and the window) are skipped.  cross: blockIdx.z names the key/value head whose values the weights are applied to.
// KD = dim / 16, NO = vdim / 8.
constexpr int HM_ROWS = 64, HM_KEYS = 64, HM_PAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// HPC query heads of one key/value head per CTA (four warps each) share the staged key and value tiles.
template <int KD, int NO, int HPC, typename TO>
__global__ void __launch_bounds__(128 * HPC, 2) heads_attention_mma_kernel(const float* __restrict__ q, const bf16* __restrict__ k_cache,
                                                                  const bf16* __restrict__ v_cache, HeadsGeom g,
                                                                  const int32_t* __restrict__ block_table, int bt_stride, int block_size,
                                                                  const PrefillTile* __restrict__ tiles, TO* __restrict__ out) {
  constexpr int D = KD * 16, DV = NO * 8, QS = D + HM_PAD, VS = DV + HM_PAD;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);       // [HPC][64][QS]
  bf16* Ks = Qs + HPC * HM_ROWS * QS;              // [2][64][QS]: a tile is loaded while the one before it is used
  bf16* Vs = Ks + 2 * HM_KEYS * QS;                // [2][64][VS]
  pdl_wait();
  pdl_launch_dependents();
  const PrefillTile tl = tiles[gridDim.x - 1 - blockIdx.x];   // the tiles late in a sequence see the most keys: they start first
  if (tl.nrows <= 0) return;
  constexpr int NT = 128 * HPC;
  const int warp = (threadIdx.x >> 5) & 3, hl = threadIdx.x >> 7, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  const int a = blockIdx.y * HPC + hl, kvh = (blockIdx.y * HPC) / (g.heads / g.kv_heads), vh = g.cross ? (int)blockIdx.z : kvh;
  const int krow = g.kv_heads * D, vrow = g.kv_heads * DV;
  // queries: fp32 -> bf16, rows past the tile's end are zero
  for (int i = threadIdx.x; i < HPC * HM_ROWS * (D / 4); i += NT) {
    const int hr = i / (D / 4), c4 = (i - hr * (D / 4)) * 4, h2 = hr / HM_ROWS, r = hr - h2 * HM_ROWS;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < tl.nrows) v = *reinterpret_cast<const float4*>(q + ((size_t)(tl.q_row0 + r) * g.heads + blockIdx.y * HPC + h2) * D + c4);
    uint2 pk;
    pk.x = pack_bf16x2(v.x, v.y);
    pk.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(Qs + hr * QS + c4) = pk;
  }
  __syncthreads();
  // the query fragments stay in shared memory and are read again for every key tile (32 registers less per thread)
  const uint32_t qbase = smem_u32(Qs + (hl * HM_ROWS + warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + (lane >> 4) * 8);
  const float slope = g.slopes ? (float)exp2(-(double)g.slope_exp * (double)(a + 1) / (double)g.heads) : 0.f;
  const int r0 = warp * 16 + gq, r1 = r0 + 8;                 // this thread's two query rows
  const int p0 = tl.q_pos0 + r0, p1 = tl.q_pos0 + r1;
  const bool live0 = r0 < tl.nrows, live1 = r1 < tl.nrows;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[NO][4];
#pragma unroll
  for (int n = 0; n < NO; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  // key tiles some row of the CTA sees
  const int last_key = tl.q_pos0 + tl.nrows - 1, last_tile = last_key / HM_KEYS;
  int nA = 0, tB = 0;
  if (g.window > 0) {
    const int lo_min = max(tl.q_pos0 - g.window + 1, 0);
    nA = (min(g.keep_first, lo_min) + HM_KEYS - 1) / HM_KEYS;
    tB = max(lo_min / HM_KEYS, nA);
  }
  const int total = nA + (last_tile - tB + 1);
  const int32_t* bt = block_table + (size_t)tl.bt_row * bt_stride;
  constexpr float LOG2E = 1.4426950408889634f;
  // 16-byte asynchronous copies; rows past the sequence's end are filled with zeros (source size 0)
  auto stage = [&](int vi, int buf) {
    const int key0 = (vi < nA ? vi : tB + (vi - nA)) * HM_KEYS;
    bf16* kd = Ks + buf * HM_KEYS * QS;
    bf16* vd = Vs + buf * HM_KEYS * VS;
    for (int i = threadIdx.x; i < HM_KEYS * (D / 8); i += NT) {
      const int r = i / (D / 8), c8 = (i - r * (D / 8)) * 8, j = key0 + r;
      const bool in = j <= last_key;
      const bf16* src = k_cache + ((size_t)(in ? bt[j / block_size] : 0) * block_size + j % block_size) * krow + (size_t)kvh * D + c8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(kd + r * QS + c8)), "l"(src), "r"(in ? 16 : 0));   // ordered by the commit / wait below, which do clobber memory
    }
    for (int i = threadIdx.x; i < HM_KEYS * (DV / 8); i += NT) {
      const int r = i / (DV / 8), c8 = (i - r * (DV / 8)) * 8, j = key0 + r;
      const bool in = j <= last_key;
      const bf16* src = v_cache + ((size_t)(in ? bt[j / block_size] : 0) * block_size + j % block_size) * vrow + (size_t)vh * DV + c8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(vd + r * VS + c8)), "l"(src), "r"(in ? 16 : 0));   // ordered by the commit / wait below, which do clobber memory
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(0, 0);
  for (int vi = 0; vi < total; ++vi) {
    const int key0 = (vi < nA ? vi : tB + (vi - nA)) * HM_KEYS;
    const bf16* Kt = Ks + (vi & 1) * HM_KEYS * QS;
    const bf16* Vt = Vs + (vi & 1) * HM_KEYS * VS;
    if (vi + 1 < total) {
      stage(vi + 1, (vi + 1) & 1);   // its buffer was last read two tiles ago (the barrier at the end of that iteration)
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    float sc[HM_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < HM_KEYS / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
    {
      const uint32_t kb = smem_u32(Kt + (lane & 7) * QS + (lane >> 3) * 8);   // four 8 x 8 blocks: two k-steps of one key group
#pragma unroll
      for (int kk = 0; kk < KD; kk += 2) {       // k-steps outside, key groups inside: neighbouring MMAs feed different accumulators
        uint32_t qa0[4], qa1[4];
        ldmatrix_x4(qa0, qbase + kk * 16 * 2);
        ldmatrix_x4(qa1, qbase + (kk + 1) * 16 * 2);
#pragma unroll
        for (int n = 0; n < HM_KEYS / 8; ++n) {
          uint32_t kf[4];
          ldmatrix_x4(kf, kb + (n * 8 * QS + kk * 16) * 2);
          mma_bf16_16816(sc[n], qa0, kf[0], kf[1]);
          mma_bf16_16816(sc[n], qa1, kf[2], kf[3]);
        }
      }
    }
    // scale, distance penalty, mask; row maxima over the quad.  A tile that every row of the CTA sees whole needs no mask.
    float t0 = -INFINITY, t1 = -INFINITY;
    const bool whole = tl.nrows == HM_ROWS && key0 + HM_KEYS - 1 <= tl.q_pos0 &&
                       (g.window <= 0 || last_key - key0 < g.window || key0 + HM_KEYS - 1 < g.keep_first);
    if (whole) {
#pragma unroll
      for (int n = 0; n < HM_KEYS / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + n * 8 + 2 * tq + (e & 1);
          const float v = sc[n][e] * g.scale - slope * (float)(((e & 2) ? p1 : p0) - j);
          sc[n][e] = v;
          if (e & 2) t1 = fmaxf(t1, v);
          else t0 = fmaxf(t0, v);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < HM_KEYS / 8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + n * 8 + 2 * tq + (e & 1);
          const int p = (e & 2) ? p1 : p0;
          const bool ok = ((e & 2) ? live1 : live0) && j <= p && (g.window <= 0 || p - j < g.window || j < g.keep_first);
          const float v = ok ? sc[n][e] * g.scale - slope * (float)(p - j) : -INFINITY;
          sc[n][e] = v;
          if (e & 2) t1 = fmaxf(t1, v);
          else t0 = fmaxf(t0, v);
        }
      }
    }
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
    t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;   // a row that has seen no key yet
    const float c0 = exp2f((m0 - u0) * LOG2E), c1 = exp2f((m1 - u1) * LOG2E);
    m0 = n0;
    m1 = n1;
    float s0 = 0.f, s1 = 0.f;
    uint32_t pa[HM_KEYS / 16][4];
#pragma unroll
    for (int n = 0; n < HM_KEYS / 8; ++n) {
      const float e0 = exp2f((sc[n][0] - u0) * LOG2E), e1 = exp2f((sc[n][1] - u0) * LOG2E);
      const float e2 = exp2f((sc[n][2] - u1) * LOG2E), e3 = exp2f((sc[n][3] - u1) * LOG2E);
      s0 += e0 + e1;
      s1 += e2 + e3;
      pa[n >> 1][(n & 1) * 2] = pack_bf16x2(e0, e1);
      pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16x2(e2, e3);
    }
    l0 = l0 * c0 + s0;
    l1 = l1 * c1 + s1;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      o[n][0] *= c0; o[n][1] *= c0;
      o[n][2] *= c1; o[n][3] *= c1;
    }
#pragma unroll
    for (int kk = 0; kk < HM_KEYS / 16; ++kk) {
      const uint32_t vbase = smem_u32(Vt + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + (lane >> 4) * 8);
#pragma unroll
      for (int n = 0; n < NO; n += 2) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vbase + n * 8 * 2);
        mma_bf16_16816(o[n], pa[kk], vb[0], vb[1]);
        mma_bf16_16816(o[n + 1], pa[kk], vb[2], vb[3]);
      }
    }
    __syncthreads();  // every warp is done with this buffer before the tile after the next is copied into it
  }
  // row sums over the quad, then the output
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const int ow = g.cross ? vrow : DV, ooff = g.cross ? vh * DV : 0;
  if (live0) {
    const float inv = 1.0f / l0;
    TO* orow = out + ((size_t)(tl.q_row0 + r0) * g.heads + a) * ow + ooff + 2 * tq;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      stf(orow + n * 8, o[n][0] * inv);
      stf(orow + n * 8 + 1, o[n][1] * inv);
    }
  }
  if (live1) {
    const float inv = 1.0f / l1;
    TO* orow = out + ((size_t)(tl.q_row0 + r1) * g.heads + a) * ow + ooff + 2 * tq;
#pragma unroll
    for (int n = 0; n < NO; ++n) {
      stf(orow + n * 8, o[n][2] * inv);
      stf(orow + n * 8 + 1, o[n][3] * inv);
    }
  }
}

template <int KD, int NO, int HPC, typename TO>
int launch_attention_mma_h(const float* q, const bf16* k, const bf16* v, const HeadsGeom& g, const int32_t* bt, int bt_stride, int block_size,
                           const PrefillTile* tiles, int ntiles, TO* out, cudaStream_t s) {
  const size_t smem = ((size_t)(HPC + 2) * HM_ROWS * (KD * 16 + HM_PAD) + (size_t)2 * HM_KEYS * (NO * 8 + HM_PAD)) * sizeof(bf16);
  auto kern = heads_attention_mma_kernel<KD, NO, HPC, TO>;
  if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  B2_CUDA_OK(b2_launch(kern, dim3(ntiles, g.heads / HPC, g.cross ? g.kv_heads : 1), dim3(128 * HPC), smem, s, q, k, v, g, bt, bt_stride, block_size,
                       tiles, out));
  return 0;
}
template <int KD, int NO, typename TO>
int launch_attention_mma_t(const float* q, const bf16* k, const bf16* v, const HeadsGeom& g, const int32_t* bt, int bt_stride, int block_size,
                           const PrefillTile* tiles, int ntiles, TO* out, cudaStream_t s) {
  if ((g.heads / g.kv_heads) % 2 == 0)   // two query heads of a key/value head share its staged tiles
    return launch_attention_mma_h<KD, NO, 2, TO>(q, k, v, g, bt, bt_stride, block_size, tiles, ntiles, out, s);
  return launch_attention_mma_h<KD, NO, 1, TO>(q, k, v, g, bt, bt_stride, block_size, tiles, ntiles, out, s);
}

// 1 = launched; 0 = the sizes have no tensor-core form (the caller takes the plain kernel)
template <typename TO>
int launch_attention_mma(const float* q, const bf16* k, const bf16* v, const HeadsGeom& g, const int32_t* bt, int bt_stride, int block_size,
                         const PrefillTile* tiles, int ntiles, TO* out, cudaStream_t s, int* rc) {
#define HM_CASE(DD, VV)                                                                                                            \
  if (g.dim == DD && g.vdim == VV) {                                                                                               \
    *rc = launch_attention_mma_t<DD / 16, VV / 8, TO>(q, k, v, g, bt, bt_stride, block_size, tiles, ntiles, out, s);                 \
    return 1;                                                                                                                      \
  }
  HM_CASE(32, 32) HM_CASE(64, 32) HM_CASE(64, 64) HM_CASE(96, 64) HM_CASE(96, 96) HM_CASE(128, 64) HM_CASE(128, 128) HM_CASE(192, 128) HM_CASE(256, 128)
#undef HM_CASE
  return 0;
}

template <typename TC, typename TO, bool DECODE, bool VEC>
int launch_attention_nv(int nv, dim3 grid, size_t smem, cudaStream_t s, const float* q, const TC* k, const TC* v, const HeadsGeom& g,
                        const int32_t* bt, int bt_stride, int block_size, const PrefillTile* tiles, const int32_t* positions,
                        const int32_t* seq_lens, TO* out, int cross_cols) {
#define HA_CASE(NVV)                                                                                                                   \
  if (nv <= NVV) {                                                                                                                     \
    auto kern = heads_attention_kernel<TC, TO, NVV, DECODE, VEC>;                                                                      \
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));              \
    B2_CUDA_OK(b2_launch(kern, grid, dim3(HA_WARPS * 32), smem, s, q, k, v, g, bt, bt_stride, block_size, tiles, positions, seq_lens, out, cross_cols)); \
    return 0;                                                                                                                          \
  }
  HA_CASE(1) HA_CASE(2) HA_CASE(4) HA_CASE(8) HA_CASE(16) HA_CASE(32)
#undef HA_CASE
  b2_set_error("heads_attention: %d value columns per head exceed 1024", nv * 32);
  return -22;
}

template <typename TC, typename TO>
int launch_attention_t(const float* q, const void* k, const void* v, const HeadsGeom& g, const int32_t* bt, int bt_stride, int block_size,
                       const PrefillTile* tiles, int ntiles, const int32_t* positions, const int32_t* seq_lens, void* out, int T,
                       cudaStream_t s) {
  // with cross a CTA takes as many whole value heads as fit 512 columns; the others go to further CTAs (blockIdx.z)
  const int vrow = g.kv_heads * g.vdim;
  const int cross_cols = g.cross ? g.vdim * std::max(1, std::min(g.kv_heads, 512 / std::max(g.vdim, 1))) : 0;
  const int zs = g.cross ? (vrow + cross_cols - 1) / cross_cols : 1;
  const int VW = g.cross ? cross_cols : g.vdim, nv = (VW + 31) / 32;
  constexpr bool can_vec = sizeof(TC) == 2;
  const bool vec = can_vec && g.dim % 8 == 0 && g.vdim % 64 == 0;
  if (tiles != nullptr) {
    const size_t smem = (size_t)HA_WARPS * g.dim * sizeof(float);
    const dim3 grid(ntiles * 8, g.heads, zs);
    if (vec)
      return launch_attention_nv<TC, TO, false, can_vec>(nv, grid, smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride, block_size, tiles,
                                                         positions, seq_lens, (TO*)out, cross_cols);
    return launch_attention_nv<TC, TO, false, false>(nv, grid, smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride, block_size, tiles, positions,
                                                     seq_lens, (TO*)out, cross_cols);
  }
  const size_t smem = ((size_t)g.dim + 2 * HA_WARPS + (size_t)HA_WARPS * VW) * sizeof(float);
  const dim3 grid(T, g.heads, zs);
  if (vec)
    return launch_attention_nv<TC, TO, true, can_vec>(nv, grid, smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride, block_size, nullptr,
                                                      positions, seq_lens, (TO*)out, cross_cols);
  return launch_attention_nv<TC, TO, true, false>(nv, grid, smem, s, q, (const TC*)k, (const TC*)v, g, bt, bt_stride, block_size, nullptr, positions,
                                                  seq_lens, (TO*)out, cross_cols);
}

// ---- mixers whose scores are mixed over the heads before the softmax ----
// One CTA per token (128 threads in long steps; 512 in short ones, where a token's heads should all be in flight at once), a warp per head
// at a time (query heads, then key heads, then value heads).  The token's cosines and
// sines are formed once: [rot_dims/2] for q and k (angles divided by rot_factor), [vdim/2] for the values.
template <typename TC>
__global__ void __launch_bounds__(512) heads_finish_halves_kernel(const float* __restrict__ proj, int ld, HeadsGeom g, const float* __restrict__ q_gain,
                                                                  const float* __restrict__ k_gain, const int32_t* __restrict__ positions,
                                                                  const int32_t* __restrict__ slots, float* __restrict__ q_out, TC* __restrict__ k_cache,
                                                                  TC* __restrict__ v_cache) {
  extern __shared__ float cs[];   // qk: cos [half] | sin [half]; then v: cos [vhalf] | sin [vhalf]
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t], slot = slots[t];
  const int nthr = blockDim.x, nwarp = nthr >> 5;
  const int half = g.rot_dims / 2, vhalf = g.rot_values ? g.vdim / 2 : 0;
  float* vcs = cs + 2 * half;
  const double inv_factor = g.rot_factor > 0.f ? 1.0 / (double)g.rot_factor : 1.0;
  for (int i = threadIdx.x; i < half; i += nthr) {
    const double f = exp2(-2.0 * (double)i / (double)g.rot_dims * log2((double)g.rot_base)) * inv_factor;
    double sd, cd;
    sincos((double)pos * f, &sd, &cd);
    cs[i] = (float)cd;
    cs[half + i] = (float)sd;
  }
  for (int i = threadIdx.x; i < vhalf; i += nthr) pair_cos_sin(pos, i, g.vdim, g.rot_base, &vcs[i], &vcs[vhalf + i]);
  __syncthreads();
  const float* row = proj + (size_t)t * ld;
  const int nqk = g.heads + g.kv_heads;
  for (int u = warp; u < nqk + g.kv_heads; u += nwarp) {
    if (u < nqk) {
      const bool is_q = u < g.heads;
      const int a = is_q ? u : u - g.heads;
      const float* src = row + (is_q ? a * g.dim : g.heads * g.dim + a * g.dim);
      const float* gain = is_q ? q_gain : k_gain;
      float r = 1.0f;
      if (gain != nullptr) {
        float ss = 0.f;
        for (int d = lane; d < g.dim; d += 32) ss = fmaf(src[d], src[d], ss);
        r = 1.0f / sqrtf(warp_sum(ss) / (float)g.dim + g.eps);
      }
      if (!is_q && slot < 0) continue;
      float* qd = q_out + (size_t)t * g.heads * g.dim + (size_t)a * g.dim;
      TC* kd = k_cache + ((size_t)(slot < 0 ? 0 : slot) * g.kv_heads + a) * g.dim;
      for (int d = lane; d < g.dim; d += 32) {
        float y = gain != nullptr ? src[d] * r * gain[d] : src[d];
        if (d < g.rot_dims) {
          const int i = d < half ? d : d - half, o = d < half ? d + half : d - half;
          const float z = gain != nullptr ? src[o] * r * gain[o] : src[o];
          y = d < half ? y * cs[i] - z * cs[half + i] : y * cs[i] + z * cs[half + i];
        }
        if (is_q) qd[d] = y;
        else stf(kd + d, y);
      }
    } else {
      if (slot < 0) continue;
      const int a = u - nqk;
      const float* src = row + (g.heads + g.kv_heads) * g.dim + a * g.vdim;
      TC* vd = v_cache + ((size_t)slot * g.kv_heads + a) * g.vdim;
      for (int d = lane; d < g.vdim; d += 32) {
        float y = src[d];
        if (d < 2 * vhalf) {
          const int i = d < vhalf ? d : d - vhalf;
          const float z = src[d < vhalf ? d + vhalf : d - vhalf];
          y = d < vhalf ? y * vcs[i] - z * vcs[vhalf + i] : y * vcs[i] + z * vcs[vhalf + i];
        }
        stf(vd + d, y);
      }
    }
  }
}

// All heads of `qt` query tokens of one sequence per CTA (eight warps), because a mixed score of one head needs the scores of every head
// for the same (query, key) pair.  Keys go by in tiles of 32, upwards from the first visible one.  Per tile: for every key/value head its
// K rows are staged and the group's query heads score them (lane j scores key j; scale, cap); then every (token, head) mixes its row of
// scores over the heads, masks it and updates its running maximum, sum and weights; then for every key/value head its V rows are staged
// and the group's heads accumulate (lane c holds value columns c, c + 32, ...; the running sums live in shared memory).  The end divides,
// turns the sum back by the query's position when the values were rotated, and rounds to the output type.
constexpr int PM_WARPS = 8, PM_KEYS = 32;
struct PremixArgs {
  const float* q;
  const void* k_cache;
  const void* v_cache;
  HeadsGeom g;
  const float* mix;
  const int32_t* block_table;
  int bt_stride, block_size;
  const PrefillTile* tiles;
  const int32_t* positions;
  const int32_t* seq_lens;
  void* out;
  int qt;
};
__host__ __device__ inline int premix_kv_stride(const HeadsGeom& g) { return (g.dim > g.vdim ? g.dim : g.vdim) | 1; }
__host__ __device__ inline size_t premix_smem_floats(const HeadsGeom& g, int qt) {
  return (size_t)qt * g.heads * (g.dim + g.vdim + 2 * PM_KEYS + 3) + (size_t)PM_KEYS * premix_kv_stride(g) + (size_t)g.heads * g.heads;
}

template <typename TC, typename TX>
__global__ void __launch_bounds__(PM_WARPS * 32) heads_attention_premix_kernel(PremixArgs a) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const HeadsGeom& g = a.g;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = g.heads, G = g.kv_heads, rep = H / G, D = g.dim, V = g.vdim, SD = premix_kv_stride(g);
  int q_row0, q_pos0, nrows, bt_row;
  if (a.tiles != nullptr) {
    const PrefillTile tl = a.tiles[blockIdx.x];
    q_row0 = tl.q_row0; q_pos0 = tl.q_pos0; nrows = tl.nrows; bt_row = tl.bt_row;
  } else {
    q_row0 = blockIdx.x; q_pos0 = a.positions[blockIdx.x]; nrows = a.seq_lens[blockIdx.x] > 0 ? 1 : 0; bt_row = blockIdx.x;
  }
  const int tok0 = blockIdx.y * a.qt;
  const int ntok = min(a.qt, nrows - tok0);
  TX* out = reinterpret_cast<TX*>(a.out);
  if (ntok <= 0) {
    if (a.tiles == nullptr && blockIdx.y == 0)   // an empty row of a padded decode batch: zeros
      for (int i = threadIdx.x; i < H * V; i += PM_WARPS * 32) stf(out + (size_t)q_row0 * H * V + i, 0.f);
    return;
  }
  float* Qs = sm;                                  // [qt][H][D]
  float* Os = Qs + (size_t)a.qt * H * D;           // [qt][H][V]
  float* Ss = Os + (size_t)a.qt * H * V;           // [qt][H][32] capped scores
  float* Ps = Ss + (size_t)a.qt * H * PM_KEYS;     // [qt][H][32] weights
  float* Ms = Ps + (size_t)a.qt * H * PM_KEYS;     // [qt][H] running maximum
  float* Ls = Ms + (size_t)a.qt * H;               // [qt][H] running sum
  float* Cs = Ls + (size_t)a.qt * H;               // [qt][H] this tile's rescale factor
  float* KV = Cs + (size_t)a.qt * H;               // [32][SD]
  float* Tk = KV + (size_t)PM_KEYS * SD;           // [H][H]
  const int pos_lo = q_pos0 + tok0, pos_hi = pos_lo + ntok - 1;
  const int items = ntok * H;
  {
    const float* qsrc = a.q + (size_t)(q_row0 + tok0) * H * D;
    for (int i = threadIdx.x; i < items * D; i += PM_WARPS * 32) Qs[i] = qsrc[i];
    for (int i = threadIdx.x; i < items * V; i += PM_WARPS * 32) Os[i] = 0.f;
    for (int i = threadIdx.x; i < items; i += PM_WARPS * 32) {
      Ms[i] = -INFINITY;
      Ls[i] = 0.f;
    }
    if (a.mix != nullptr)
      for (int i = threadIdx.x; i < H * H; i += PM_WARPS * 32) Tk[i] = a.mix[i];
  }
  const TC* kc = reinterpret_cast<const TC*>(a.k_cache);
  const TC* vc = reinterpret_cast<const TC*>(a.v_cache);
  const int32_t* bt = a.block_table + (size_t)bt_row * a.bt_stride;
  const int k_first = g.window > 0 ? max(0, pos_lo - g.window + 1) / PM_KEYS * PM_KEYS : 0;
  for (int k0 = k_first; k0 <= pos_hi; k0 += PM_KEYS) {
    const int nk = min(PM_KEYS, pos_hi + 1 - k0);
    for (int kvh = 0; kvh < G; ++kvh) {
      __syncthreads();   // the staged rows' last readers are done (first time: Qs is in place)
      for (int j = warp; j < nk; j += PM_WARPS) {
        const int kp = k0 + j;
        const TC* src = kc + (((size_t)bt[kp / a.block_size] * a.block_size + kp % a.block_size) * G + kvh) * D;
        for (int d = lane; d < D; d += 32) KV[j * SD + d] = ldf(src + d);
      }
      __syncthreads();
      for (int it = warp; it < ntok * rep; it += PM_WARPS) {
        const int tok = it / rep, h = kvh * rep + (it - tok * rep);
        if (lane < nk) {
          const float* qv = Qs + ((size_t)tok * H + h) * D;
          const float* kr = KV + lane * SD;
          float acc = 0.f;
          for (int d = 0; d < D; ++d) acc = fmaf(qv[d], kr[d], acc);
          acc *= g.scale;
          if (g.softcap > 0.f) acc = g.softcap * tanhf(acc / g.softcap);
          Ss[((size_t)tok * H + h) * PM_KEYS + lane] = acc;
        }
      }
    }
    __syncthreads();
    for (int it = warp; it < items; it += PM_WARPS) {
      const int tok = it / H, h = it - tok * H;
      const int my_pos = pos_lo + tok, kp = k0 + lane;
      const bool vis = lane < nk && kp <= my_pos && (g.window <= 0 || my_pos - kp < g.window);
      float sc = -INFINITY;
      if (vis) {
        if (a.mix != nullptr) {
          sc = 0.f;
          for (int b = 0; b < H; ++b) sc = fmaf(Tk[h * H + b], Ss[((size_t)tok * H + b) * PM_KEYS + lane], sc);
        } else {
          sc = Ss[(size_t)it * PM_KEYS + lane];
        }
      }
      const float m_old = Ms[it];
      const float m_new = fmaxf(m_old, warp_max(sc));
      const float p = vis ? expf(sc - m_new) : 0.f;
      const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
      const float psum = warp_sum(p);
      Ps[(size_t)it * PM_KEYS + lane] = p;
      if (lane == 0) {
        Ms[it] = m_new;
        Ls[it] = Ls[it] * corr + psum;
        Cs[it] = corr;
      }
    }
    for (int kvh = 0; kvh < G; ++kvh) {
      __syncthreads();   // the weights are written / the staged rows' last readers are done
      for (int j = warp; j < nk; j += PM_WARPS) {
        const int kp = k0 + j;
        const TC* src = vc + (((size_t)bt[kp / a.block_size] * a.block_size + kp % a.block_size) * G + kvh) * V;
        for (int d = lane; d < V; d += 32) KV[j * SD + d] = ldf(src + d);
      }
      __syncthreads();
      for (int it = warp; it < ntok * rep; it += PM_WARPS) {
        const int tok = it / rep, h = kvh * rep + (it - tok * rep);
        const size_t row = (size_t)tok * H + h;
        const float corr = Cs[row];
        const float* pw = Ps + row * PM_KEYS;
        for (int d = lane; d < V; d += 32) {
          float acc = Os[row * V + d] * corr;
          for (int j = 0; j < nk; ++j) acc = fmaf(pw[j], KV[j * SD + d], acc);
          Os[row * V + d] = acc;
        }
      }
    }
  }
  __syncthreads();
  const int vhalf = g.rot_values ? V / 2 : 0;
  for (int it = warp; it < items; it += PM_WARPS) {
    const int tok = it / H;
    const float inv = 1.0f / Ls[it];
    const float* o = Os + (size_t)it * V;
    TX* dst = out + (size_t)(q_row0 + tok0) * H * V + (size_t)it * V;
    for (int d = lane; d < V; d += 32) {
      float y = o[d];
      if (d < 2 * vhalf) {   // turned back by the query's position: the pair (u, v) by minus the angle
        const int i = d < vhalf ? d : d - vhalf;
        float c, sn;
        pair_cos_sin(pos_lo + tok, i, V, g.rot_base, &c, &sn);
        const float z = o[d < vhalf ? d + vhalf : d - vhalf];
        y = d < vhalf ? y * c + z * sn : y * c - z * sn;
      }
      stf(dst + d, y * inv);
    }
  }
}

// ---- the same pass on warp-level tensor-core MMAs (bf16 caches, prompt portions, head sizes in multiples of 16) ----
// One CTA of sixteen warps per 16 query tokens and ALL heads; keys go by in tiles of 32.  Per tile: the K rows of every key/value head are
// staged (bf16, asynchronous copies) and every query head forms S = Q K^T, one 16 x 16 block per warp at a time (ldmatrix + mma.sync), into
// an fp32 slab [heads][16][32]; the V rows take the K rows' place while every thread takes one (token, key) pair, reads the pair's scores
// head by head (scale, cap), mixes them (two heads per packed fp32 multiply-add, each head's sum in the order of the heads) and writes them
// back masked; then two threads per (token, head) row update the row's maximum and sum and write the weights as bf16; then the warps
// accumulate P V into the output blocks they own (unit u = head * (vdim / 16) + column block belongs to warp u mod 16), rescaled once per
// tile by the rows' factors.  The end goes through shared memory: division, the turn back by the query's position (cosines and sines of the
// sixteen positions are formed once), rounding.
constexpr int PX_ROWS = 16, PX_KEYS = 32, PX_WARPS = 16, PX_THREADS = 32 * PX_WARPS, PX_SLD = 36, PX_PLD = 40;
struct PremixMmaArgs {
  const float* q;
  const bf16* k_cache;
  const bf16* v_cache;
  HeadsGeom g;
  const float* mix;
  const int32_t* block_table;
  int bt_stride, block_size;
  const PrefillTile* tiles;
  bf16* out;
};
struct PremixMmaLayout {
  int QP, KP, OP;            // row strides: queries (bf16), staged K / V rows (bf16), the output slab (fp32)
  size_t q_off, k_off, s_off, p_off, misc_off, cs_off, total;   // bytes
};
__host__ __device__ inline PremixMmaLayout premix_mma_layout(const HeadsGeom& g) {
  PremixMmaLayout L;
  const int H = g.heads, D = g.dim, V = g.vdim;
  L.QP = D + 8;
  L.KP = (D > V ? D : V) + 8;
  L.OP = V + 4;
  L.q_off = 0;
  L.k_off = L.q_off + (size_t)H * PX_ROWS * L.QP * 2;
  L.s_off = L.k_off + (size_t)g.kv_heads * PX_KEYS * L.KP * 2;
  L.p_off = L.s_off + (size_t)H * PX_ROWS * PX_SLD * 4;
  const size_t main_end = L.p_off + (size_t)H * PX_ROWS * PX_PLD * 2;
  const size_t out_end = (size_t)H * PX_ROWS * L.OP * 4;              // the output slab reuses everything from the start
  L.misc_off = ((main_end > out_end ? main_end : out_end) + 127) / 128 * 128;
  // misc: running maximum, sum, this tile's factor [heads * 16] each, the mixing matrix [heads][up to 32], positions [16], cache rows [2][32]
  L.cs_off = L.misc_off + ((size_t)3 * H * PX_ROWS + (size_t)H * 32 + PX_ROWS + 2 * PX_KEYS) * 4;
  L.total = L.cs_off + (size_t)PX_ROWS * V * 4;                        // cos [16][V/2] | sin [16][V/2]
  return L;
}

// HMAX: register slots for one pair's mixed scores (heads <= HMAX); NU: 16 x 16 output blocks per warp (heads * vdim / 16 <= PX_WARPS * NU)
template <int HMAX, int NU>
__global__ void __launch_bounds__(PX_THREADS, 1) heads_attention_premix_mma_kernel(PremixMmaArgs a) {
  extern __shared__ __align__(128) unsigned char smraw[];
  pdl_wait();
  pdl_launch_dependents();
  const HeadsGeom& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int H = g.heads, G = g.kv_heads, rep = H / G, D = g.dim, V = g.vdim, VB = V / 16;
  const PremixMmaLayout L = premix_mma_layout(g);
  bf16* Qs = reinterpret_cast<bf16*>(smraw + L.q_off);      // [H][16][QP]
  bf16* Ks = reinterpret_cast<bf16*>(smraw + L.k_off);      // [G][32][KP]: the tile's K rows, then its V rows
  float* Ss = reinterpret_cast<float*>(smraw + L.s_off);    // [H][16][36]
  bf16* Ps = reinterpret_cast<bf16*>(smraw + L.p_off);      // [H][16][40]
  float* Os = reinterpret_cast<float*>(smraw);              // at the end: [H][16][OP]
  float* row_m = reinterpret_cast<float*>(smraw + L.misc_off);   // [H][16]
  float* row_l = row_m + H * PX_ROWS;
  float* row_f = row_l + H * PX_ROWS;
  float* Tk = row_f + H * PX_ROWS;                          // [H][HMAX], transposed: entry [b][h] weighs head b's score in head h's mix
  int* row_pos = reinterpret_cast<int*>(Tk + H * HMAX);     // [16]
  int* key_row = row_pos + PX_ROWS;                         // [2][32]: this tile's cache rows and the next tile's
  float* cs = reinterpret_cast<float*>(smraw + L.cs_off);

  // CTAs start in the order of their index: the list of tiles and the blocks of a tile are walked backwards, so that the late positions of a
  // prompt (the most key tiles) start first and the last CTAs to start are short ones
  const PrefillTile tl = a.tiles[gridDim.x - 1 - blockIdx.x];
  const int tok0 = (gridDim.y - 1 - blockIdx.y) * PX_ROWS;
  const int ntok = min(PX_ROWS, tl.nrows - tok0);
  if (ntok <= 0) return;
  const int q_row0 = tl.q_row0 + tok0, pos_lo = tl.q_pos0 + tok0, pos_hi = pos_lo + ntok - 1;
  // ---- stage Q as bf16 (rows past the portion are zero), the mixing matrix, the rows' bookkeeping ----
  for (int idx = tid; idx < H * PX_ROWS * (D / 4); idx += PX_THREADS) {
    const int c = idx % (D / 4), r = (idx / (D / 4)) % PX_ROWS, h = idx / ((D / 4) * PX_ROWS);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < ntok) v = __ldg(reinterpret_cast<const float4*>(a.q + ((size_t)(q_row0 + r) * H + h) * D) + c);
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<unsigned*>(&lo);
    pk.y = *reinterpret_cast<unsigned*>(&hi);
    *reinterpret_cast<uint2*>(Qs + ((size_t)h * PX_ROWS + r) * L.QP + c * 4) = pk;
  }
  for (int i = tid; i < H * PX_ROWS; i += PX_THREADS) {
    row_m[i] = -INFINITY;
    row_l[i] = 0.f;
  }
  for (int i = tid; i < H * HMAX; i += PX_THREADS) {
    const int b = i / HMAX, h = i - b * HMAX;
    Tk[i] = h >= H ? 0.f : a.mix != nullptr ? a.mix[h * H + b] : (h == b ? 1.f : 0.f);
  }
  if (tid < PX_ROWS) row_pos[tid] = tid < ntok ? pos_lo + tid : -1;
  // ---- output accumulators: unit u = head * (vdim / 16) + column block holds a 16 x 16 block as two m16n8 accumulators (element 0, 1: row
  //      lane / 4, columns 2 (lane % 4) and the next; element 2, 3: row lane / 4 + 8) ----
  float oacc[NU][2][4];
#pragma unroll
  for (int u = 0; u < NU; ++u)
#pragma unroll
    for (int e = 0; e < 4; ++e) oacc[u][0][e] = oacc[u][1][e] = 0.f;
  const int fg = lane >> 2, ft = lane & 3;
  const int units = H * VB;
  const int32_t* bt = a.block_table + (size_t)tl.bt_row * a.bt_stride;
  // a chunk index splits into (key, head, chunk of the head row) by multiplications: q = n / d as the high word of n * ceil(2^32 / d), exact
  // for n < 2^16 and 2 <= d < 2^16 (32 keys of at most a few hundred chunks each)
  struct StageGeom {
    int cpr, per_key;          // 16-byte chunks per head row; per key (a key's cache row holds the heads side by side)
    unsigned m_cpr, m_key;
  };
  auto stage_geom = [&](int width) {
    StageGeom sg;
    sg.cpr = width / 8;
    sg.per_key = G * sg.cpr;
    sg.m_cpr = (unsigned)((0x100000000ull + sg.cpr - 1) / sg.cpr);
    sg.m_key = (unsigned)((0x100000000ull + sg.per_key - 1) / sg.per_key);
    return sg;
  };
  const StageGeom sg_k = stage_geom(D), sg_v = stage_geom(V);
  auto stage_rows = [&](const bf16* cache, int width, const StageGeom& sg, const int* key_row) {   // the tile's rows of every key/value head, zeros past the last key
    const int total = PX_KEYS * sg.per_key;
#pragma unroll 4
    for (int idx = tid; idx < total; idx += PX_THREADS) {
      const int j = (int)__umulhi((unsigned)idx, sg.m_key), rest = idx - j * sg.per_key;
      const int kvh = (int)__umulhi((unsigned)rest, sg.m_cpr), c = rest - kvh * sg.cpr;
      const int kr = key_row[j];
      // asynchronous 16-byte copies (zero-filled past the last key): every chunk of a thread is in flight at once
      const bf16* src = cache + (size_t)(kr >= 0 ? kr : 0) * G * width + (size_t)rest * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(Ks + ((size_t)kvh * PX_KEYS + j) * L.KP + c * 8)), "l"(src), "r"(kr >= 0 ? 16 : 0));
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto stage_wait = [&]() { asm volatile("cp.async.wait_group 0;" ::: "memory"); };
  const int k_first = g.window > 0 ? max(0, pos_lo - g.window + 1) / PX_KEYS * PX_KEYS : 0;
  // the cache rows of a tile's keys are looked up a tile ahead (thirty-two threads, beside the mix), so that no tile waits for its block table
  auto cache_row = [&](int kp) { return kp <= pos_hi ? bt[kp / a.block_size] * a.block_size + kp % a.block_size : -1; };
  if (tid < PX_KEYS) key_row[tid] = cache_row(k_first + tid);
  int cur = 0;
  for (int k0 = k_first; k0 <= pos_hi; k0 += PX_KEYS, cur ^= 1) {
    const int* rows_now = key_row + cur * PX_KEYS;
    int row_ahead = -1;   // (read here, stored behind the mix: its latency hides behind this tile's work)
    if (tid < PX_KEYS && k0 + PX_KEYS <= pos_hi) row_ahead = cache_row(k0 + PX_KEYS + tid);
    __syncthreads();   // the tile before is consumed; this tile's cache rows are in place
    stage_rows(a.k_cache, D, sg_k, rows_now);
    stage_wait();
    __syncthreads();
    // ---- S = Q K^T: unit u = head * 2 + key block; per 16 entries of the heads one ldmatrix for the queries' 16 x 16 block, one for the
    //      two 8-key groups' blocks, two MMAs ----
    for (int u = warp; u < H * 2; u += PX_WARPS) {
      const int h = u >> 1, kb = u & 1;
      float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      const uint32_t qaddr = smem_u32(Qs + ((size_t)h * PX_ROWS + (lane & 15)) * L.QP + (lane >> 4) * 8);
      const uint32_t kaddr = smem_u32(Ks + ((size_t)(h / rep) * PX_KEYS + 16 * kb + (lane & 7) + ((lane >> 4) & 1) * 8) * L.KP + ((lane >> 3) & 1) * 8);
#pragma unroll 4
      for (int d = 0; d < D; d += 16) {
        uint32_t qa[4], kf[4];
        ldmatrix_x4(qa, qaddr + d * 2);
        ldmatrix_x4(kf, kaddr + d * 2);
        mma_bf16_16816(acc[0], qa, kf[0], kf[1]);
        mma_bf16_16816(acc[1], qa, kf[2], kf[3]);
      }
      float* srow = Ss + ((size_t)h * PX_ROWS + fg) * PX_SLD + 16 * kb + 2 * ft;
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        *reinterpret_cast<float2*>(srow + 8 * n) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2*>(srow + 8 * PX_SLD + 8 * n) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    __syncthreads();
    stage_rows(a.v_cache, V, sg_v, rows_now);   // (the K rows are consumed; the loads fly while the scores are mixed)
    if (tid < PX_KEYS) key_row[(cur ^ 1) * PX_KEYS + tid] = row_ahead;
    // ---- scale, cap, mix over the heads, mask: a thread takes ONE (token, key) pair.  It walks the heads b in their order, reads the pair's
    //      score of head b (scale, cap) and adds its share to the mixed score of every head h, two heads per packed fp32 multiply-add with
    //      the matrix column b read four entries a load; every sum therefore runs over b upwards, as the plain kernel's does ----
    {
      const int r0 = tid >> 5, j = tid & 31, kp = k0 + j;
      unsigned long long mixed[HMAX / 2];
#pragma unroll
      for (int h2 = 0; h2 < HMAX / 2; ++h2) mixed[h2] = 0ull;
      const float* scol = Ss + (size_t)r0 * PX_SLD + j;
      const float exp_scale = g.softcap > 0.f ? g.scale * 2.0f * 1.4426950408889634f / g.softcap : 0.f, minus_two_cap = -2.0f * g.softcap;
#pragma unroll 4
      for (int b = 0; b < H; ++b) {
        float v = scol[(size_t)b * PX_ROWS * PX_SLD];
        // cap * tanh(s / cap) with s = v * scale as cap - 2 cap / (2^(s * 2 log2(e) / cap) + 1): the operands of this kernel are bf16, its fast
        // exponential and reciprocal are not what bounds it
        if (g.softcap > 0.f) {
          float ex;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(v * exp_scale));
          v = g.softcap + __fdividef(minus_two_cap, ex + 1.0f);
        } else {
          v *= g.scale;
        }
        unsigned long long vv;
        asm("mov.b64 %0, {%1, %1};" : "=l"(vv) : "f"(v));
        const float* tcol = Tk + b * HMAX;   // (padded to HMAX entries, zeros behind the heads)
#pragma unroll
        for (int h4 = 0; h4 < HMAX / 4; ++h4) {
          const ulonglong2 t4 = *reinterpret_cast<const ulonglong2*>(tcol + 4 * h4);
          asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(mixed[2 * h4]) : "l"(t4.x), "l"(vv));
          asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(mixed[2 * h4 + 1]) : "l"(t4.y), "l"(vv));
        }
      }
      const int p0 = row_pos[r0];
      const bool vis = kp <= p0 && (g.window <= 0 || p0 - kp < g.window);
      float* dcol = Ss + (size_t)r0 * PX_SLD + j;
#pragma unroll
      for (int h2 = 0; h2 < HMAX / 2; ++h2) {
        float lo, hi;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(mixed[h2]));
        if (2 * h2 < H) dcol[(size_t)(2 * h2) * PX_ROWS * PX_SLD] = vis ? lo : -INFINITY;
        if (2 * h2 + 1 < H) dcol[(size_t)(2 * h2 + 1) * PX_ROWS * PX_SLD] = vis ? hi : -INFINITY;
      }
    }
    stage_wait();   // this thread's V chunks have landed
    __syncthreads();
    // ---- two threads per (head, token) row, sixteen keys each: maximum, weights (bf16: what is summed is what multiplies the values), sum,
    //      this tile's factor ----
    for (int idx = tid; idx < 2 * H * PX_ROWS; idx += PX_THREADS) {
      const int row = idx >> 1, part = idx & 1;
      float sv[16];
      const float4* s4 = reinterpret_cast<const float4*>(Ss + (size_t)row * PX_SLD + 16 * part);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 x = s4[i];
        sv[4 * i] = x.x; sv[4 * i + 1] = x.y; sv[4 * i + 2] = x.z; sv[4 * i + 3] = x.w;
      }
      float mx = sv[0];
#pragma unroll
      for (int i = 1; i < 16; ++i) mx = fmaxf(mx, sv[i]);
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      const float m_old = row_m[row];
      const float m_new = fmaxf(m_old, mx);
      float psum = 0.f;
      unsigned pk[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // (the weights are rounded to bf16 next: the approximate exponential loses nothing)
        float e0, e1;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"((sv[2 * i] - m_new) * 1.4426950408889634f));
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"((sv[2 * i + 1] - m_new) * 1.4426950408889634f));
        if (sv[2 * i] == -INFINITY) e0 = 0.f;
        if (sv[2 * i + 1] == -INFINITY) e1 = 0.f;
        const __nv_bfloat162 pp = __floats2bfloat162_rn(e0, e1);
        pk[i] = *reinterpret_cast<const unsigned*>(&pp);
        psum += __low2float(pp) + __high2float(pp);
      }
      uint4* pd = reinterpret_cast<uint4*>(Ps + (size_t)row * PX_PLD + 16 * part);
      pd[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      pd[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      psum += __shfl_xor_sync(0xffffffffu, psum, 1);
      __syncwarp();   // (both threads of a row have read its old maximum)
      if (part == 0) {
        const float corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        row_m[row] = m_new;
        row_l[row] = row_l[row] * corr + psum;
        row_f[row] = corr;
      }
    }
    __syncthreads();   // weights, factors and the V rows are in place
    // ---- O = O * factor + P V: per 16 keys one ldmatrix for the weights' block, one (transposing) for the values' two 8-column groups ----
#pragma unroll
    for (int i = 0; i < NU; ++i) {
      const int u = warp + PX_WARPS * i;
      if (u >= units) continue;
      const int h = u / VB, cb = u - h * VB;
      const float f0 = row_f[h * PX_ROWS + fg], f1 = row_f[h * PX_ROWS + fg + 8];
#pragma unroll
      for (int n = 0; n < 2; ++n) {
        oacc[i][n][0] *= f0; oacc[i][n][1] *= f0;
        oacc[i][n][2] *= f1; oacc[i][n][3] *= f1;
      }
      const uint32_t paddr = smem_u32(Ps + ((size_t)h * PX_ROWS + (lane & 15)) * PX_PLD + (lane >> 4) * 8);
      const uint32_t vaddr = smem_u32(Ks + ((size_t)(h / rep) * PX_KEYS + (lane & 7) + ((lane >> 3) & 1) * 8) * L.KP + 16 * cb + (lane >> 4) * 8);
#pragma unroll
      for (int kk = 0; kk < PX_KEYS; kk += 16) {
        uint32_t pa[4], vb[4];
        ldmatrix_x4(pa, paddr + kk * 2);
        ldmatrix_x4_trans(vb, vaddr + (uint32_t)(kk * L.KP) * 2);
        mma_bf16_16816(oacc[i][0], pa, vb[0], vb[1]);
        mma_bf16_16816(oacc[i][1], pa, vb[2], vb[3]);
      }
    }
  }
  __syncthreads();   // every warp is done with the operand slabs: they become the output slab
#pragma unroll
  for (int i = 0; i < NU; ++i) {
    const int u = warp + PX_WARPS * i;
    if (u >= units) continue;
    const int h = u / VB, cb = u - h * VB;
    float* orow = Os + ((size_t)h * PX_ROWS + fg) * L.OP + 16 * cb + 2 * ft;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      *reinterpret_cast<float2*>(orow + 8 * n) = make_float2(oacc[i][n][0], oacc[i][n][1]);
      *reinterpret_cast<float2*>(orow + (size_t)8 * L.OP + 8 * n) = make_float2(oacc[i][n][2], oacc[i][n][3]);
    }
  }
  const int vhalf = g.rot_values ? V / 2 : 0;
  for (int i = tid; i < ntok * vhalf; i += PX_THREADS) {
    const int r = i / vhalf, m = i - r * vhalf;
    pair_cos_sin(pos_lo + r, m, V, g.rot_base, &cs[r * V + m], &cs[r * V + vhalf + m]);
  }
  __syncthreads();
  for (int row = warp; row < H * PX_ROWS; row += PX_WARPS) {
    const int h = row / PX_ROWS, r = row - h * PX_ROWS;
    if (r >= ntok) continue;
    const float inv = 1.0f / row_l[row];
    const float* o = Os + (size_t)row * L.OP;
    bf16* dst = a.out + ((size_t)(q_row0 + r) * H + h) * V;
    for (int d = lane; d < V; d += 32) {
      float y = o[d];
      if (d < 2 * vhalf) {   // turned back by the query's position: the pair (u, v) by minus the angle
        const int m = d < vhalf ? d : d - vhalf;
        const float c = cs[r * V + m], sn = cs[r * V + vhalf + m];
        const float z = o[d < vhalf ? d + vhalf : d - vhalf];
        y = d < vhalf ? y * c + z * sn : y * c - z * sn;
      }
      dst[d] = __float2bfloat16_rn(y * inv);
    }
  }
}

template <int HMAX, int NU>
int launch_premix_mma_t(const PremixMmaArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
  static B2PerDeviceOnce once;
  static size_t set_to = 0;
  if (once.need() || smem > set_to) {
    B2_CUDA_OK(cudaFuncSetAttribute(heads_attention_premix_mma_kernel<HMAX, NU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, set_to)));
    set_to = std::max(smem, set_to);
  }
  B2_CUDA_OK(b2_launch(heads_attention_premix_mma_kernel<HMAX, NU>, grid, dim3(PX_THREADS), smem, s, a));
  return 0;
}
template <int HMAX>
int launch_premix_mma_h(int nu, const PremixMmaArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
  if (nu <= 1) return launch_premix_mma_t<HMAX, 1>(a, grid, smem, s);
  if (nu <= 2) return launch_premix_mma_t<HMAX, 2>(a, grid, smem, s);
  if (nu <= 4) return launch_premix_mma_t<HMAX, 4>(a, grid, smem, s);
  return launch_premix_mma_t<HMAX, 8>(a, grid, smem, s);   // (premix_mma_fits admits no more: sixteen fragments a thread would spill)
}
// whether the tensor-core form serves this geometry (else the plain kernel does)
bool premix_mma_fits(const HeadsGeom& g) {
  return g.dim % 16 == 0 && g.vdim % 16 == 0 && g.heads <= 32 && (g.heads * (g.vdim / 16) + PX_WARPS - 1) / PX_WARPS <= 8 && premix_mma_layout(g).total <= 224 * 1024;
}

// ---- decode steps: one new token per sequence against a long cache ----
// A CTA takes one sequence and one split of its visible keys, with a warp per head; the splits' partial sums (maximum, sum, unnormalised
// weighted values) go to a scratch buffer and premix_merge folds them in split order, turns the result back and rounds.  Per tile of 32
// keys: warp h scores the tile for head h straight from the cache (lane j reads key j's row; the heads of a group hit the same lines),
// a barrier, then warp h mixes its row over the heads, updates its running maximum and sum in registers and accumulates the values
// (lane c holds columns c, c + 32, ...), a barrier.  The number of splits depends on the batch size and the engine's longest sequence
// only, never on the lengths in the batch, so that a captured step serves every length.
constexpr int PD_KEYS = 32;
struct PremixDecodeArgs {
  const float* q;
  const void* k_cache;
  const void* v_cache;
  HeadsGeom g;
  const float* mix;
  const int32_t* block_table;
  int bt_stride, block_size;
  const int32_t* positions;
  const int32_t* seq_lens;
  float* partial;   // [row][split][head][vdim + 2]
  int nsplit;
};

template <typename TC>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const TC* __restrict__ k, int D) {
  float acc = 0.f;
  for (int d = 0; d < D; ++d) acc = fmaf(q[d], ldf(k + d), acc);
  return acc;
}
template <>
__device__ __forceinline__ float dot_row<bf16>(const float* __restrict__ q, const bf16* __restrict__ k, int D) {
  float acc = 0.f;
  int d = 0;
  if ((D & 7) == 0 && (reinterpret_cast<size_t>(k) & 15) == 0) {
    for (; d < D; d += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(k + d);
      const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc = fmaf(q[d + 2 * i], __uint_as_float(w[i] << 16), acc);
        acc = fmaf(q[d + 2 * i + 1], __uint_as_float(w[i] & 0xffff0000u), acc);
      }
    }
    return acc;
  }
  for (; d < D; ++d) acc = fmaf(q[d], __bfloat162float(k[d]), acc);
  return acc;
}

// NV = ceil(vdim / 32): value columns per lane
template <typename TC, int NV>
__global__ void __launch_bounds__(1024) heads_attention_premix_decode_kernel(PremixDecodeArgs a) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const HeadsGeom& g = a.g;
  const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = g.heads, G = g.kv_heads, D = g.dim, V = g.vdim, kvh = h / (H / G);
  const int b = blockIdx.x, split = blockIdx.y;
  float* Qs = sm;                 // [H][D]
  float* Ss = Qs + H * D;         // [H][32]
  float* Tk = Ss + H * PD_KEYS;   // [H][H]
  float* dst = a.partial + (((size_t)b * a.nsplit + split) * H + h) * (V + 2);
  const int pos = a.positions[b];
  int first = 0, k_end = 0;
  if (a.seq_lens[b] > 0) {
    const int lo = g.window > 0 ? max(0, pos - g.window + 1) : 0;
    const int per = ((pos + 1 - lo + a.nsplit - 1) / a.nsplit + PD_KEYS - 1) / PD_KEYS * PD_KEYS;
    first = lo + split * per;
    k_end = min(pos + 1, first + per);
  }
  float o[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  if (first < k_end) {   // (uniform over the CTA)
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) Qs[i] = a.q[(size_t)b * H * D + i];
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) Tk[i] = a.mix != nullptr ? a.mix[i] : ((i / H) == (i % H) ? 1.f : 0.f);
    const TC* kc = reinterpret_cast<const TC*>(a.k_cache);
    const TC* vc = reinterpret_cast<const TC*>(a.v_cache);
    const int32_t* bt = a.block_table + (size_t)b * a.bt_stride;
    for (int k0 = first; k0 < k_end; k0 += PD_KEYS) {
      __syncthreads();   // the tile before is consumed (first time: q and the mixing matrix are staged)
      const int kp = k0 + lane;
      const bool live = kp < k_end;
      const int row = live ? bt[kp / a.block_size] * a.block_size + kp % a.block_size : 0;
      float sc = 0.f;
      if (live) {
        sc = dot_row<TC>(Qs + h * D, kc + ((size_t)row * G + kvh) * D, D) * g.scale;
        if (g.softcap > 0.f) sc = g.softcap * tanhf(sc / g.softcap);
      }
      Ss[h * PD_KEYS + lane] = sc;
      __syncthreads();
      float mixed = -INFINITY;
      if (live) {
        mixed = 0.f;
        for (int c = 0; c < H; ++c) mixed = fmaf(Tk[h * H + c], Ss[c * PD_KEYS + lane], mixed);
      }
      const float m_new = fmaxf(m, warp_max(mixed));
      const float p = live ? expf(mixed - m_new) : 0.f;
      const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NV; ++i) o[i] *= corr;
      const int nk = min(PD_KEYS, k_end - k0);
      for (int j = 0; j < nk; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const int rj = __shfl_sync(0xffffffffu, row, j);
        const TC* vr = vc + ((size_t)rj * G + kvh) * V;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int d = lane + 32 * i;
          if (d < V) o[i] = fmaf(pj, ldf(vr + d), o[i]);
        }
      }
    }
  }
  if (lane == 0) {
    dst[0] = m;
    dst[1] = l;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int d = lane + 32 * i;
    if (d < V) dst[2 + d] = o[i];
  }
}

// folds the splits of every (row, head) in split order, divides, turns the sum back by the row's position, rounds; a CTA per row, a warp
// per head at a time (lane s holds split s: at most 32 splits; the CTA has as many warps as heads, up to sixteen, so that every head's
// partial sums are in flight at once, eight splits a batch); the row's cosines and sines are formed once for all heads
template <typename TX>
__global__ void __launch_bounds__(512) premix_merge_kernel(const float* __restrict__ partial, int nsplit, HeadsGeom g, const int32_t* __restrict__ positions,
                                                           const int32_t* __restrict__ seq_lens, TX* __restrict__ out) {
  extern __shared__ float sm[];   // [warps][vdim], then cos [vdim/2] | sin [vdim/2]
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nthr = blockDim.x, nwarp = nthr >> 5;
  const int H = g.heads, V = g.vdim, vhalf = g.rot_values ? V / 2 : 0;
  const bool empty = seq_lens[b] <= 0;
  float* row = sm + warp * V;
  float* cs = sm + nwarp * V;
  if (!empty) {
    const int pos = positions[b];
    for (int i = threadIdx.x; i < vhalf; i += nthr) pair_cos_sin(pos, i, V, g.rot_base, &cs[i], &cs[vhalf + i]);
  }
  __syncthreads();
  for (int h = warp; h < H; h += nwarp) {
    TX* dst = out + ((size_t)b * H + h) * V;
    if (empty) {
      for (int d = lane; d < V; d += 32) stf(dst + d, 0.f);
      continue;
    }
    const float* p = partial + ((size_t)b * nsplit * H + h) * (V + 2);
    const size_t stride = (size_t)H * (V + 2);
    const float ms = lane < nsplit ? p[lane * stride] : -INFINITY;
    const float ls = lane < nsplit ? p[lane * stride + 1] : 0.f;
    const float m = warp_max(ms);
    const float wgt = ms == -INFINITY ? 0.f : expf(ms - m);
    const float inv = 1.0f / warp_sum(ls * wgt);
    for (int d0 = 0; d0 < V; d0 += 32) {
      const int d = d0 + lane;
      float acc = 0.f;
      for (int s2 = 0; s2 < nsplit; s2 += 8) {
        float w2[8], x[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {   // (a split without keys left its sums unwritten: weight 0 reads nothing)
          const float w = __shfl_sync(0xffffffffu, wgt, (s2 + k) & 31);
          w2[k] = s2 + k < nsplit ? w : 0.f;
          x[k] = d < V && w2[k] != 0.f ? p[(s2 + k) * stride + 2 + d] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (w2[k] != 0.f) acc = fmaf(x[k], w2[k], acc);
      }
      if (d < V) row[d] = acc * inv;
    }
    __syncwarp();
    for (int d = lane; d < V; d += 32) {
      float y = row[d];
      if (d < 2 * vhalf) {
        const int i = d < vhalf ? d : d - vhalf;
        const float z = row[d < vhalf ? d + vhalf : d - vhalf];
        y = d < vhalf ? y * cs[i] + z * cs[vhalf + i] : y * cs[i] - z * cs[vhalf + i];
      }
      stf(dst + d, y);
    }
    __syncwarp();
  }
}

int premix_decode_splits(int rows, int max_context) {
  int ns = (2 * 148 + rows - 1) / std::max(rows, 1);   // about two CTAs per SM
  ns = std::min(std::min(ns, 32), std::max(1, (max_context + 2 * PD_KEYS - 1) / (2 * PD_KEYS)));
  return std::max(ns, 1);
}

template <typename TC, int NV>
int launch_premix_decode_nv(const PremixDecodeArgs& a, int T, size_t smem, cudaStream_t s) {
  static B2PerDeviceOnce once;
  static size_t set_to = 0;
  if (smem > 48 * 1024 && (once.need() || smem > set_to)) {
    B2_CUDA_OK(cudaFuncSetAttribute(heads_attention_premix_decode_kernel<TC, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, set_to)));
    set_to = std::max(smem, set_to);
  }
  B2_CUDA_OK(b2_launch(heads_attention_premix_decode_kernel<TC, NV>, dim3(T, a.nsplit), dim3(32 * a.g.heads), smem, s, a));
  return 0;
}
template <typename TC>
int launch_premix_decode_t(const PremixDecodeArgs& a, int T, size_t smem, cudaStream_t s) {
  const int nv = (a.g.vdim + 31) / 32;
  if (nv <= 1) return launch_premix_decode_nv<TC, 1>(a, T, smem, s);
  if (nv <= 2) return launch_premix_decode_nv<TC, 2>(a, T, smem, s);
  if (nv <= 4) return launch_premix_decode_nv<TC, 4>(a, T, smem, s);
  if (nv <= 8) return launch_premix_decode_nv<TC, 8>(a, T, smem, s);
  return launch_premix_decode_nv<TC, 16>(a, T, smem, s);
}

template <typename TC, typename TX>
int launch_premix_t(const PremixArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
  static B2PerDeviceOnce once;
  static size_t set_to = 0;
  if (smem > 48 * 1024 && (once.need() || smem > set_to)) {
    B2_CUDA_OK(cudaFuncSetAttribute(heads_attention_premix_kernel<TC, TX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, set_to)));
    set_to = std::max(smem, set_to);
  }
  B2_CUDA_OK(b2_launch(heads_attention_premix_kernel<TC, TX>, grid, dim3(PM_WARPS * 32), smem, s, a));
  return 0;
}

}  // namespace

int launch_heads_finish_halves(const float* proj, int ld, const HeadsGeom& g, const float* q_gain, const float* k_gain, const int32_t* positions,
                               const int32_t* slots, float* q_out, void* k_cache, void* v_cache, int cache_f32, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(g.rot_dims >= 0 && g.rot_dims <= g.dim && g.rot_dims % 2 == 0, "heads_finish_halves: rot dims %d must be even and <= dim %d", g.rot_dims, g.dim);
  B2_REQUIRE(!g.rot_values || g.vdim % 2 == 0, "heads_finish_halves: rotated values need an even vdim (%d)", g.vdim);
  const size_t smem = (size_t)(g.rot_dims + (g.rot_values ? g.vdim : 0) + 2) * sizeof(float);
  const dim3 block(T <= 4 * 148 ? 512 : 128);   // few tokens: every head of a token gets a warp of its own
  if (cache_f32)
    B2_CUDA_OK(b2_launch(heads_finish_halves_kernel<float>, dim3(T), block, smem, s, proj, ld, g, q_gain, k_gain, positions, slots, q_out,
                         (float*)k_cache, (float*)v_cache));
  else
    B2_CUDA_OK(b2_launch(heads_finish_halves_kernel<bf16>, dim3(T), block, smem, s, proj, ld, g, q_gain, k_gain, positions, slots, q_out,
                         (bf16*)k_cache, (bf16*)v_cache));
  return 0;
}

int launch_heads_attention_premix(const float* q, const void* k_cache, const void* v_cache, int cache_f32, const HeadsGeom& g, const float* mix,
                                  const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                                  const int32_t* positions, const int32_t* seq_lens, void* out, int out_f32, int T, cudaStream_t s, float* scratch,
                                  size_t scratch_floats, int max_context) {
  if (T <= 0 || (tiles != nullptr && ntiles <= 0)) return 0;
  B2_REQUIRE(g.heads >= 1 && g.kv_heads >= 1 && g.heads % g.kv_heads == 0, "heads_attention_premix: %d heads over %d key/value heads", g.heads, g.kv_heads);
  B2_REQUIRE(cache_f32 == out_f32, "heads_attention_premix: cache and output have one element type");
  static const bool use_mma = [] { const char* e = getenv("B2_PREMIX_MMA"); return !(e && *e == '0'); }();
  if (use_mma && !cache_f32 && tiles != nullptr && premix_mma_fits(g)) {
    PremixMmaArgs a{q, (const bf16*)k_cache, (const bf16*)v_cache, g, mix, block_table, bt_stride, block_size, tiles, (bf16*)out};
    const dim3 grid(ntiles, 64 / PX_ROWS);
    const size_t smem = premix_mma_layout(g).total;
    const int nu = (g.heads * (g.vdim / 16) + PX_WARPS - 1) / PX_WARPS;
    if (g.heads <= 8) return launch_premix_mma_h<8>(nu, a, grid, smem, s);
    if (g.heads <= 16) return launch_premix_mma_h<16>(nu, a, grid, smem, s);
    return launch_premix_mma_h<32>(nu, a, grid, smem, s);
  }
  if (tiles == nullptr && scratch != nullptr && g.heads <= 32 && g.vdim <= 512) {   // a decode step: key splits with a warp per head, then the merge
    int ns = premix_decode_splits(T, max_context);
    while (ns > 1 && (size_t)T * ns * g.heads * (g.vdim + 2) > scratch_floats) --ns;
    const size_t smem = ((size_t)g.heads * (g.dim + PD_KEYS) + (size_t)g.heads * g.heads) * sizeof(float);
    if ((size_t)T * ns * g.heads * (g.vdim + 2) <= scratch_floats && smem <= 200 * 1024) {
      PremixDecodeArgs a{q, k_cache, v_cache, g, mix, block_table, bt_stride, block_size, positions, seq_lens, scratch, ns};
      if (cache_f32) B2_TRY_RC(launch_premix_decode_t<float>(a, T, smem, s));
      else B2_TRY_RC(launch_premix_decode_t<bf16>(a, T, smem, s));
      const int mw = std::min(16, std::max(4, g.heads));   // warps of a merge CTA
      const size_t msm = (size_t)(mw + 1) * g.vdim * sizeof(float);
      if (out_f32) B2_CUDA_OK(b2_launch(premix_merge_kernel<float>, dim3(T), dim3(32 * mw), msm, s, (const float*)scratch, ns, g, positions, seq_lens, (float*)out));
      else B2_CUDA_OK(b2_launch(premix_merge_kernel<bf16>, dim3(T), dim3(32 * mw), msm, s, (const float*)scratch, ns, g, positions, seq_lens, (bf16*)out));
      return 0;
    }
  }
  // query tokens per CTA: as many as fit beside a second CTA on the SM, at least one
  int qt = tiles != nullptr ? 16 : 1;
  while (qt > 1 && premix_smem_floats(g, qt) * 4 > 100 * 1024) qt >>= 1;
  const size_t smem = premix_smem_floats(g, qt) * sizeof(float);
  B2_REQUIRE(smem <= 200 * 1024, "heads_attention_premix: %d heads of %d + %d numbers need %zu bytes of shared memory for one token", g.heads, g.dim, g.vdim, smem);
  PremixArgs a{q, k_cache, v_cache, g, mix, block_table, bt_stride, block_size, tiles, positions, seq_lens, out, qt};
  const dim3 grid(tiles != nullptr ? ntiles : T, tiles != nullptr ? (64 + qt - 1) / qt : 1);
  if (cache_f32) return launch_premix_t<float, float>(a, grid, smem, s);
  return launch_premix_t<bf16, bf16>(a, grid, smem, s);
}

int launch_heads_finish(const float* proj, int ld, const HeadsGeom& g, const float* bias, const float* conv_w, float* ring,
                        const int32_t* row_seq, const int32_t* row_first, const int32_t* row_end, const int32_t* positions,
                        const int32_t* slots, int vmix_mode, const float* vmix_lambda, float* v_first, float* q_out, void* k_cache,
                        void* v_cache, int cache_f32, int T, cudaStream_t s, void* q_bf16) {
  if (T <= 0) return 0;
  B2_REQUIRE(!g.swizzled || (!cache_f32 && g.dim == 128 && g.vdim == 128 && q_bf16 != nullptr), "heads_finish: the swizzled page layout is bf16, 128 wide");
  B2_REQUIRE(g.rot_dims >= 0 && g.rot_dims <= g.dim && g.rot_dims % 2 == 0, "heads_finish: rot dims %d must be even and <= dim %d", g.rot_dims,
             g.dim);
  B2_REQUIRE(g.conv_taps == 0 || (conv_w && ring && row_seq && row_first && row_end), "heads_finish: the convolution needs its weights and state");
  B2_REQUIRE(vmix_mode == 0 || v_first != nullptr, "heads_finish: value mixing needs the first layer's values");
  const int C = g.heads * g.dim + g.kv_heads * (g.dim + g.vdim);
  const size_t smem = ((size_t)4 * std::max(g.dim, g.vdim) + std::max(g.rot_dims, 2)) * sizeof(float);
  B2_REQUIRE(smem <= 200 * 1024, "heads_finish: a head of %d numbers exceeds shared memory", std::max(g.dim, g.vdim));
  const int units = g.heads + 2 * g.kv_heads, upc = T >= 256 ? units : 4;   // prompt-sized steps: a CTA per token
  const dim3 fgrid(T, (units + upc - 1) / upc);
  if (cache_f32) {
    auto kern = heads_finish_kernel<float>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B2_CUDA_OK(b2_launch(kern, fgrid, dim3(128), smem, s, proj, ld, g, bias, conv_w, (const float*)ring, row_seq, row_first, positions, slots,
                         vmix_mode, vmix_lambda, v_first, q_out, (float*)k_cache, (float*)v_cache, upc, (bf16*)nullptr));
  } else {
    auto kern = heads_finish_kernel<bf16>;
    if (smem > 48 * 1024) B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    B2_CUDA_OK(b2_launch(kern, fgrid, dim3(128), smem, s, proj, ld, g, bias, conv_w, (const float*)ring, row_seq, row_first, positions, slots,
                         vmix_mode, vmix_lambda, v_first, q_out, (bf16*)k_cache, (bf16*)v_cache, upc, (bf16*)q_bf16));
  }
  if (g.conv_taps > 1)
    B2_CUDA_OK(b2_launch(conv_tail_store_kernel, dim3(T), dim3(128), 0, s, proj, ld, C, g.conv_taps, bias, ring, row_seq, row_end, positions, slots));
  return 0;
}

int launch_heads_finish_rownorm(const float* proj, int ld, const HeadsGeom& g, const float* bias, const float* qk_gain, const int32_t* slots,
                                float* q_out, void* k_cache, void* v_cache, int cache_f32, int T, cudaStream_t s, void* q_bf16) {
  if (T <= 0) return 0;
  B2_REQUIRE(qk_gain != nullptr, "heads_finish_rownorm: the row norms need their gains");
  B2_REQUIRE(!g.swizzled || (!cache_f32 && g.dim == 128 && g.vdim == 128 && q_bf16 != nullptr), "heads_finish_rownorm: the swizzled page layout is bf16, 128 wide");
  const bool wide = T < 1024 && g.heads * g.dim >= 1024;
#define B2_ROWNORM(TC, NT, QB)                                                                                                                         \
  B2_CUDA_OK(b2_launch(heads_finish_rownorm_kernel<TC, NT>, dim3(T), dim3(NT), 0, s, proj, ld, g, bias, qk_gain, slots, q_out, (TC*)k_cache, (TC*)v_cache, \
                       (bf16*)(QB)))
  if (cache_f32) {
    if (wide) B2_ROWNORM(float, 512, nullptr);
    else B2_ROWNORM(float, 128, nullptr);
  } else {
    if (wide) B2_ROWNORM(bf16, 512, q_bf16);
    else B2_ROWNORM(bf16, 128, q_bf16);
  }
#undef B2_ROWNORM
  return 0;
}

int launch_heads_attention(const float* q, const void* k_cache, const void* v_cache, int cache_f32, const HeadsGeom& g,
                           const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                           const int32_t* positions, const int32_t* seq_lens, void* out, int out_f32, int T, cudaStream_t s) {
  if (T <= 0 || (tiles != nullptr && ntiles <= 0)) return 0;
  B2_REQUIRE(g.heads >= 1 && g.kv_heads >= 1 && g.heads % g.kv_heads == 0, "heads_attention: %d query heads over %d key/value heads", g.heads,
             g.kv_heads);
  B2_REQUIRE(!g.cross || out_f32, "heads_attention: the per-head sums that are mixed afterwards are fp32");
  if (cache_f32) {
    B2_REQUIRE(out_f32, "heads_attention: an fp32 cache goes with fp32 operands");
    return launch_attention_t<float, float>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
  }
  static const bool use_mma = [] { const char* e = getenv("B2_HEADS_MMA"); return !(e && *e == '0'); }();
  if (use_mma && tiles != nullptr && block_size > 0) {   // prompt portions on tensor-core MMAs when the head sizes have that form
    int rc = 0;
    if (out_f32 ? launch_attention_mma<float>(q, (const bf16*)k_cache, (const bf16*)v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, (float*)out, s, &rc)
                : launch_attention_mma<bf16>(q, (const bf16*)k_cache, (const bf16*)v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, (bf16*)out, s, &rc))
      return rc;
  }
  if (out_f32)
    return launch_attention_t<bf16, float>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
  return launch_attention_t<bf16, bf16>(q, k_cache, v_cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, out, T, s);
}

size_t heads_attention_premix_scratch_floats(int max_rows, int heads, int vdim) {
  // rows * splits stays below two CTAs per SM plus one split per row
  return ((size_t)2 * 148 + 2 * (size_t)max_rows) * heads * ((size_t)vdim + 2);
}

int launch_talk_gate(const float* cross, const float* talk, const float* gate, int gate_ld, void* out, int out_f32, int heads, int kv_heads,
                     int vdim, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  const dim3 grid(T, T >= 1024 ? 1 : std::max(1, std::min((heads * vdim + 127) / 128, 1024 / T)));   // few tokens: several CTAs per row
  if (out_f32) B2_CUDA_OK(b2_launch(talk_gate_kernel<float>, grid, dim3(128), 0, s, cross, talk, gate, gate_ld, (float*)out, heads, kv_heads, vdim));
  else B2_CUDA_OK(b2_launch(talk_gate_kernel<bf16>, grid, dim3(128), 0, s, cross, talk, gate, gate_ld, (bf16*)out, heads, kv_heads, vdim));
  return 0;
}

}  // namespace b2
