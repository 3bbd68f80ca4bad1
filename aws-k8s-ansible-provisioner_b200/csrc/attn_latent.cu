// attn_latent.cu -- attention over a low-rank latent that all heads share, with a per-head softmax sink.
//
// Per token the cache holds ONE row: the normalised latent c [kv_rank] and one rotated key piece k_r [rot_dim] (not one
// key and one value per head).  Head a's key would be (U_k[a] c | k_r) and its value U_v[a] c; instead of rebuilding them
// for every cached token, the query is pulled through U_k once ("absorbed"):
//     score(a, j)   = ((U_k[a]^T q_nope[a]) . c_j + q_rot[a] . k_r_j) * scale
//     out_lat[a]    = sum_j p(a, j) c_j / (sum_j exp(score - m) + exp(sink[a] - m))
// and U_v[a] is applied to out_lat afterwards (gemm_any.cu, one strided batch over the heads).  The pass therefore reads
// kv_rank + rot_dim numbers per cached token for ALL heads, which is what makes this cache small.
// The sink is one more term of the softmax denominator with no key and no value: unscaled, counted once.
//
// Everything here is fp32 arithmetic (scores, softmax, rotary angles in fp64 before the rounding, norms); the cache and
// the operands handed on are fp32 or bf16.  Kernels:
//   latent_finish     what follows the fused q | latent projection: rotary on the query's rotated piece, unit-RMS norm of
//                     the latent with a plain gain, rotary on the shared key piece, cache row write
//   latent_attention_mma   bf16 cache: 64 (token, head) rows x 64-key tiles on warp-level bf16 MMAs with fp32 accumulators.  Two
//                     sweeps over the keys: the first finds every row's maximum (Q.K^T only), the second forms
//                     P = exp(s - max) and accumulates P.C with no rescaling in between, so the accumulators never
//                     leave the MMA fragments.  The keys of a row block may be cut into splits that run as CTAs of their
//                     own (decode steps: few rows, long caches); splits leave (max, sum, unnormalised sum of latents) and
//                     latent_merge folds them, and the sink, into the output
//   latent_attention  fp32 cache (and latents wider than 512): one warp per (query token, head); a CTA's eight rows share 32-key tiles staged in shared memory; lane j
//                     scores key j, then lane d accumulates latent dims d, d + 32, ...; the same kernel serves prompt
//                     portions (64-token tiles over the block table) and decode steps (one row per sequence)
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

// (u, v) of pair i at position p turns by p * base^(-2 i / dims); angle formed in fp64, rounded once
__device__ __forceinline__ void pair_cos_sin(int pos, int i, int dims, float base, float* c, float* s) {
  const double f = exp2(-2.0 * (double)i / (double)dims * log2((double)base));
  double sd, cd;
  sincos((double)pos * f, &sd, &cd);
  *c = (float)cd;
  *s = (float)sd;
}

template <typename TX, typename TC>
__global__ void __launch_bounds__(128) latent_finish_kernel(const float* __restrict__ qd, int ld, LatentGeom g, int has_kv,
                                                            const float* __restrict__ latent_gain, const int32_t* __restrict__ positions,
                                                            const int32_t* __restrict__ slots, TX* __restrict__ q_nope,
                                                            float* __restrict__ q_rot, TC* __restrict__ cache) {
  extern __shared__ float cs[];  // [rot_dims / 2] cos | sin
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = g.rot_dims / 2;
  for (int i = threadIdx.x; i < half; i += 128) pair_cos_sin(pos, i, g.rot_dims, g.rot_base, &cs[i], &cs[half + i]);
  __syncthreads();
  const float* row = qd + (size_t)t * ld;
  const int hw = g.dim + g.rot_dim;
  for (int i = threadIdx.x; i < g.heads * g.dim; i += 128) {
    const int a = i / g.dim, d = i - a * g.dim;
    stf(q_nope + (size_t)t * g.heads * g.dim + i, row[a * hw + d]);
  }
  // rotated piece: pairs below rot_dims turn, the rest passes (one thread per pair; an odd last element passes alone)
  const int pairs_per = (g.rot_dim + 1) / 2;
  for (int i = threadIdx.x; i < g.heads * pairs_per; i += 128) {
    const int a = i / pairs_per, p = i - a * pairs_per;
    const float* src = row + a * hw + g.dim + 2 * p;
    float* dst = q_rot + (size_t)t * g.heads * g.rot_dim + a * g.rot_dim + 2 * p;
    const bool has_v = 2 * p + 1 < g.rot_dim;
    const float u = src[0], v = has_v ? src[1] : 0.f;
    if (p < half && has_v) {
      dst[0] = u * cs[p] - v * cs[half + p];
      dst[1] = v * cs[p] + u * cs[half + p];
    } else {
      dst[0] = u;
      if (has_v) dst[1] = v;
    }
  }
  if (!has_kv) return;
  const int slot = slots[t];
  if (slot < 0) return;
  const float* lat = row + g.heads * hw;
  float ss = 0.f;
  for (int i = threadIdx.x; i < g.kv_rank; i += 128) ss = fmaf(lat[i], lat[i], ss);
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = red[0] + red[1] + red[2] + red[3];
  const float r = 1.0f / sqrtf(ss / (float)g.kv_rank + g.eps);
  TC* crow = cache + (size_t)slot * (g.kv_rank + g.rot_dim);
  for (int i = threadIdx.x; i < g.kv_rank; i += 128) stf(crow + i, lat[i] * r * latent_gain[i]);
  const float* kr = lat + g.kv_rank;
  for (int p = threadIdx.x; p < pairs_per; p += 128) {
    const bool has_v = 2 * p + 1 < g.rot_dim;
    const float u = kr[2 * p], v = has_v ? kr[2 * p + 1] : 0.f;
    TC* dst = crow + g.kv_rank + 2 * p;
    if (p < half && has_v) {
      stf(dst, u * cs[p] - v * cs[half + p]);
      stf(dst + 1, v * cs[p] + u * cs[half + p]);
    } else {
      stf(dst, u);
      if (has_v) stf(dst + 1, v);
    }
  }
}

// What follows a fused projection whose output holds a query latent and a key/value latent (proj [T][ld] fp32, the query latent of
// q_rank entries at column off_q, the other of kv_rank entries at off_c): both are RMS-normed with a plain gain; the first goes out as the
// operand of the query up-projection, the second is the token's cache row.  One CTA of 128 threads per token.
template <typename TX, typename TC>
__global__ void __launch_bounds__(128) latent_pair_finish_kernel(const float* __restrict__ proj, int ld, int off_q, int q_rank, int off_c, int kv_rank,
                                                                 const float* __restrict__ gain_q, const float* __restrict__ gain_c, float eps,
                                                                 const int32_t* __restrict__ slots, TX* __restrict__ xq, TC* __restrict__ cache) {
  __shared__ float red[2][4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += 128) sq = fmaf(row[off_q + i], row[off_q + i], sq);
  for (int i = threadIdx.x; i < kv_rank; i += 128) sc = fmaf(row[off_c + i], row[off_c + i], sc);
  sq = warp_sum(sq);
  sc = warp_sum(sc);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = sq;
    red[1][threadIdx.x >> 5] = sc;
  }
  __syncthreads();
  const float rq = 1.0f / sqrtf((red[0][0] + red[0][1] + red[0][2] + red[0][3]) / (float)q_rank + eps);
  const float rc = 1.0f / sqrtf((red[1][0] + red[1][1] + red[1][2] + red[1][3]) / (float)kv_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += 128) stf(xq + (size_t)t * q_rank + i, row[off_q + i] * rq * gain_q[i]);
  const int slot = slots[t];
  if (slot < 0) return;
  TC* crow = cache + (size_t)slot * kv_rank;
  for (int i = threadIdx.x; i < kv_rank; i += 128) stf(crow + i, row[off_c + i] * rc * gain_c[i]);
}

constexpr int LA_WARPS = 8, LA_KEYS = 32;

// NR = ceil(kv_rank / 32): latent dims per lane
template <typename TC, typename TX, int NR>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attention_kernel(const float* __restrict__ q_abs, const float* __restrict__ q_rot,
                                                                         const TC* __restrict__ cache, LatentGeom g,
                                                                         const int32_t* __restrict__ block_table, int bt_stride, int block_size,
                                                                         const PrefillTile* __restrict__ tiles, const int32_t* __restrict__ positions,
                                                                         const int32_t* __restrict__ seq_lens, const float* __restrict__ sink,
                                                                         TX* __restrict__ out_lat) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = g.kv_rank, D = g.kv_rank + g.rot_dim, SD = D | 1;  // odd row stride: lanes that walk down a column hit 32 banks
  float* qs = sm;                       // [LA_WARPS][D]
  float* ks = sm + LA_WARPS * D;        // [LA_KEYS][SD]
  int q_row0, q_pos0, nrows, bt_row;
  if (tiles != nullptr) {
    const PrefillTile tl = tiles[blockIdx.x];
    q_row0 = tl.q_row0; q_pos0 = tl.q_pos0; nrows = tl.nrows; bt_row = tl.bt_row;
  } else {
    q_row0 = blockIdx.x; q_pos0 = positions[blockIdx.x]; nrows = seq_lens[blockIdx.x] > 0 ? 1 : 0; bt_row = blockIdx.x;
  }
  const int total = nrows * g.heads;
  const int first = blockIdx.y * LA_WARPS;
  if (first >= total) return;
  const int my = first + warp;
  const bool active = my < total;
  const int tok = active ? my / g.heads : 0, head = active ? my - tok * g.heads : 0;
  const int my_pos = q_pos0 + tok;
  const int last_row = min(first + LA_WARPS, total) - 1;
  const int max_pos = q_pos0 + last_row / g.heads;
  if (active) {
    const float* qa = q_abs + ((size_t)(q_row0 + tok) * g.heads + head) * R;
    const float* qr = q_rot + ((size_t)(q_row0 + tok) * g.heads + head) * g.rot_dim;
    for (int d = lane; d < R; d += 32) qs[warp * D + d] = qa[d];
    for (int d = lane; d < g.rot_dim; d += 32) qs[warp * D + R + d] = qr[d];
  }
  float o[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) o[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const int32_t* bt = block_table + (size_t)bt_row * bt_stride;
  // with a window the keys below the first row's window are hidden from every row of the CTA
  const int k_first = g.window > 0 ? max(0, q_pos0 + first / g.heads - g.window + 1) / LA_KEYS * LA_KEYS : 0;
  for (int k0 = k_first; k0 <= max_pos; k0 += LA_KEYS) {
    __syncthreads();  // previous tile consumed (and, first time, q staged)
    const int nk = min(LA_KEYS, max_pos + 1 - k0);
    for (int j = warp; j < nk; j += LA_WARPS) {
      const int kp = k0 + j;
      const TC* src = cache + ((size_t)bt[kp / block_size] * block_size + kp % block_size) * D;
      for (int d = lane; d < D; d += 32) ks[j * SD + d] = ldf(src + d);
    }
    __syncthreads();
    if (!active || k0 > my_pos) continue;
    // lane j scores key k0 + j
    float s = -INFINITY;
    if (lane < nk && k0 + lane <= my_pos && (g.window <= 0 || my_pos - (k0 + lane) < g.window)) {
      const float* kr = ks + lane * SD;
      const float* q = qs + warp * D;
      float acc = 0.f;
      for (int d = 0; d < D; ++d) acc = fmaf(q[d], kr[d], acc);
      s = acc * g.scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = s == -INFINITY ? 0.f : expf(s - m_new);
    const float corr = m == -INFINITY ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < NR; ++i) o[i] *= corr;
    m = m_new;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      if (pj == 0.f) continue;  // warp-uniform
      const float* c = ks + j * SD;
#pragma unroll
      for (int i = 0; i < NR; ++i) {
        const int d = lane + 32 * i;
        if (d < R) o[i] = fmaf(pj, c[d], o[i]);
      }
    }
  }
  if (!active) return;
  // the sink: one more term of the denominator (none: its weight is zero)
  const float sk = sink != nullptr ? sink[head] : -INFINITY;
  const float mf = fmaxf(m, sk);
  const float corr = expf(m - mf);
  const float den = l * corr + expf(sk - mf);
  const float inv = corr / den;
  TX* dst = out_lat + ((size_t)(q_row0 + tok) * g.heads + head) * R;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int d = lane + 32 * i;
    if (d < R) stf(dst + d, o[i] * inv);
  }
}

// ---- tensor-core form -----------------------------------------------------------------------------------------------
constexpr int MA_ROWS = 64, MA_KEYS = 64, MA_THREADS = 256;

struct MmaAttnArgs {
  const float* q_abs;
  const float* q_rot;
  const bf16* cache;
  LatentGeom g;
  const int32_t* block_table;
  int bt_stride, block_size;
  const PrefillTile* tiles;
  const int32_t* positions;
  const int32_t* seq_lens;
  const float* sink;
  bf16* out_lat;
  float* partial;   // nsplit > 1: [(token row * heads + head) * nsplit + split][kv_rank + 2] = max, sum, sum of p * latent
  int nsplit;
};

// NF: 16-wide output column fragments per warp (8 warps): kv_rank <= 128 * NF
template <int NF>
__global__ void __launch_bounds__(MA_THREADS, 1) latent_attention_mma_kernel(MmaAttnArgs a) {
  using namespace nvcuda;
  extern __shared__ __align__(128) unsigned char smraw[];
  pdl_wait();
  pdl_launch_dependents();
  const LatentGeom& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int R = g.kv_rank, D = R + g.rot_dim, D16 = (D + 15) & ~15, DP = D16 + 8, R16 = (R + 15) & ~15;
  bf16* Qs = reinterpret_cast<bf16*>(smraw);                 // [64][DP]
  bf16* Ks = Qs + MA_ROWS * DP;                              // [64][DP]
  float* Ss = reinterpret_cast<float*>(Ks + MA_KEYS * DP);   // [64][68]
  bf16* Ps = reinterpret_cast<bf16*>(Ss + MA_ROWS * 68);     // [64][72]
  float* row_m = reinterpret_cast<float*>(Ps + MA_ROWS * 72);  // [64]
  float* row_l = row_m + MA_ROWS;                            // [64]
  int* row_pos = reinterpret_cast<int*>(row_l + MA_ROWS);    // [64]
  int* key_row = row_pos + MA_ROWS;                          // [64] cache rows of the staged keys
  float* Os = reinterpret_cast<float*>(smraw);               // after the sweeps: [64][R16 + 4] over Qs / Ks

  int q_row0, q_pos0, nrows, bt_row;
  if (a.tiles != nullptr) {
    const PrefillTile tl = a.tiles[blockIdx.x];
    q_row0 = tl.q_row0; q_pos0 = tl.q_pos0; nrows = tl.nrows; bt_row = tl.bt_row;
  } else {
    q_row0 = blockIdx.x; q_pos0 = a.positions[blockIdx.x]; nrows = a.seq_lens[blockIdx.x] > 0 ? 1 : 0; bt_row = blockIdx.x;
  }
  const int total = nrows * g.heads;
  const int first = blockIdx.y * MA_ROWS;
  if (first >= total) return;
  const int split = blockIdx.z;
  const int last_row = min(first + MA_ROWS, total) - 1;
  const int max_pos = q_pos0 + last_row / g.heads;
  // this split's keys: whole 64-key tiles [t_lo, t_hi)
  const int ntile = max_pos / MA_KEYS + 1;
  // with a window the tiles below the first row's window are hidden from every row of the block
  const int t_first = g.window > 0 ? max(0, q_pos0 + first / g.heads - g.window + 1) / MA_KEYS : 0;
  const int per = (ntile - t_first + a.nsplit - 1) / a.nsplit;
  const int t_lo = t_first + split * per, t_hi = min(ntile, t_lo + per);

  // ---- stage Q (bf16), zero the padding columns of both operand slabs ----
  if (R % 4 == 0 && g.rot_dim % 4 == 0) {   // one flat loop over (row, four floats): many independent loads per thread
    const int qc = R >> 2, per_row = qc + (g.rot_dim >> 2);
#pragma unroll 8
    for (int idx = tid; idx < MA_ROWS * per_row; idx += MA_THREADS) {
      const int r = idx / per_row, c = idx - r * per_row, row = first + r;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row < total) {
        const int tok = row / g.heads, head = row - tok * g.heads;
        const size_t base = (size_t)(q_row0 + tok) * g.heads + head;
        v = c < qc ? __ldg(reinterpret_cast<const float4*>(a.q_abs + base * R) + c)
                   : __ldg(reinterpret_cast<const float4*>(a.q_rot + base * g.rot_dim) + (c - qc));
      }
      __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
      uint2 pk;
      pk.x = *reinterpret_cast<unsigned*>(&lo);
      pk.y = *reinterpret_cast<unsigned*>(&hi);
      *reinterpret_cast<uint2*>(Qs + r * DP + c * 4) = pk;   // the rotated piece follows the latent part: column R + 4 (c - qc) = 4 c
    }
    for (int idx = tid; idx < MA_ROWS * (DP - D); idx += MA_THREADS) {
      const int r = idx / (DP - D), d = D + idx - r * (DP - D);
      Qs[r * DP + d] = __float2bfloat16_rn(0.f);
      Ks[r * DP + d] = __float2bfloat16_rn(0.f);
    }
  } else {
    for (int r = warp; r < MA_ROWS; r += MA_THREADS / 32) {
      const int row = first + r, lane = tid & 31;
      if (row < total) {
        const int tok = row / g.heads, head = row - tok * g.heads;
        const size_t base = (size_t)(q_row0 + tok) * g.heads + head;
        const float* qa = a.q_abs + base * R;
        const float* qr = a.q_rot + base * g.rot_dim;
        for (int d = lane; d < R; d += 32) Qs[r * DP + d] = __float2bfloat16_rn(qa[d]);
        for (int d = lane; d < g.rot_dim; d += 32) Qs[r * DP + R + d] = __float2bfloat16_rn(qr[d]);
        for (int d = D + lane; d < DP; d += 32) Qs[r * DP + d] = __float2bfloat16_rn(0.f);
      } else {
        for (int d = lane; d < DP; d += 32) Qs[r * DP + d] = __float2bfloat16_rn(0.f);
      }
      // key slab: only the padding columns need zeros (the copies write [0, D) of every row, zeros past the last key)
      for (int d = D + lane; d < DP; d += 32) Ks[r * DP + d] = __float2bfloat16_rn(0.f);
    }
  }
  if (tid < MA_ROWS) {
    const int row = first + tid;
    row_pos[tid] = row < total ? q_pos0 + row / g.heads : -1;
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }
  const int32_t* bt = a.block_table + (size_t)bt_row * a.bt_stride;
  // 16-row groups of the tile that hold real rows: a decode step brings `heads` rows, and the groups past them are zero
  // queries whose weights are all zero, so neither product needs to touch them
  const int live_groups = (min(MA_ROWS, total - first) + 15) >> 4;
  const bool vec = (D % 8 == 0);
  auto load_keys = [&](int k0) {
    __syncthreads();  // the previous tile's reads of Ks / Ss / Ps are done
    // cache row of every key of the tile first (one block-table lookup per key), so that the copies below are independent loads
    if (tid < MA_KEYS) {
      const int kp = k0 + tid;
      key_row[tid] = kp <= max_pos ? bt[kp / a.block_size] * a.block_size + kp % a.block_size : -1;
    }
    __syncthreads();
    if (vec) {
      const int cpr = D / 8;  // 16-byte chunks per key row
#pragma unroll 8
      for (int idx = tid; idx < MA_KEYS * cpr; idx += MA_THREADS) {
        const int j = idx / cpr, c = idx - j * cpr;
        const int kr = key_row[j];
        uint4 v = make_uint4(0, 0, 0, 0);
        if (kr >= 0) v = ld_stream(a.cache + (size_t)kr * D + c * 8);
        *reinterpret_cast<uint4*>(Ks + j * DP + c * 8) = v;
      }
    } else {
      for (int idx = tid; idx < MA_KEYS * D; idx += MA_THREADS) {
        const int j = idx / D, d = idx - j * D;
        const int kr = key_row[j];
        Ks[j * DP + d] = kr >= 0 ? a.cache[(size_t)kr * D + d] : __float2bfloat16_rn(0.f);
      }
    }
    __syncthreads();
  };
  // S = Q . K^T for the staged tile: warp w computes rows 16 * (w / 2) .., keys 32 * (w % 2) ..
  auto scores = [&]() {
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[2];
    wmma::fill_fragment(acc[0], 0.f);
    wmma::fill_fragment(acc[1], 0.f);
    if (live_groups == 1) {   // sixteen rows: warps 0..3 take sixteen keys each (the other row groups are never read)
      if (warp < 4) {
        for (int d = 0; d < D16; d += 16) {
          wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fq;
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fk;
          wmma::load_matrix_sync(fq, Qs + d, DP);
          wmma::load_matrix_sync(fk, Ks + (16 * warp) * DP + d, DP);
          wmma::mma_sync(acc[0], fq, fk, acc[0]);
        }
        wmma::store_matrix_sync(Ss + 16 * warp, acc[0], 68, wmma::mem_row_major);
      }
      __syncthreads();
      return;
    }
    const int rm = (warp >> 1) * 16, kn = (warp & 1) * 32;
    if (rm < 16 * live_groups) {
      for (int d = 0; d < D16; d += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fq;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fk;
        wmma::load_matrix_sync(fq, Qs + rm * DP + d, DP);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          wmma::load_matrix_sync(fk, Ks + (kn + 16 * j) * DP + d, DP);
          wmma::mma_sync(acc[j], fq, fk, acc[j]);
        }
      }
      wmma::store_matrix_sync(Ss + rm * 68 + kn, acc[0], 68, wmma::mem_row_major);
      wmma::store_matrix_sync(Ss + rm * 68 + kn + 16, acc[1], 68, wmma::mem_row_major);
    }
    __syncthreads();
  };
  // ---- which row of its 16 x 16 tile each accumulator element of this thread belongs to: read back from a tile that holds
  //      its own row numbers (the layout of a fragment is the compiler's business) ----
  using OFrag = wmma::fragment<wmma::accumulator, 16, 16, 16, float>;
  constexpr int NE = OFrag::num_elements;
  OFrag oacc[4][NF];   // warp w: every row, columns [w * NF * 16, (w + 1) * NF * 16)
  int frag_row[NE];
  {
    __syncthreads();
    Ss[tid] = (float)(tid >> 4);   // 256 threads: a 16 x 16 tile, row-major
    __syncthreads();
    wmma::load_matrix_sync(oacc[0][0], Ss, 16, wmma::mem_row_major);
#pragma unroll
    for (int e = 0; e < NE; ++e) frag_row[e] = (int)oacc[0][0].x[e];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < NF; ++j) wmma::fill_fragment(oacc[i][j], 0.f);
  // ---- one sweep over the keys.  Weights are exp(s - ref) against a per-row reference that follows the running maximum
  //      lazily: it moves (and the row's sums are rescaled) only when a tile's maximum exceeds it by more than REF_SLACK, so
  //      most tiles leave the accumulators alone.  Sum, accumulator and reference stay consistent, which is all the final
  //      division needs; weights stay below e^REF_SLACK, well inside bf16's range ----
  constexpr float REF_SLACK = 8.0f;
  const int r4 = tid >> 2, q4 = tid & 3;  // four threads per row, 16 keys each
  float m_ref = -INFINITY, mysum = 0.f;
  const int col0 = warp * NF * 16;
  float* row_f = row_m;   // per-row rescale factor of the current tile (row_m itself is written after the sweep)
  for (int t = t_lo; t < t_hi; ++t) {
    const int k0 = t * MA_KEYS;
    load_keys(k0);
    scores();
    const int lim = row_pos[r4] - k0;  // keys j <= lim are visible ...
    const int low = g.window > 0 ? lim - g.window + 1 : -(1 << 30);   // ... from j = low on
    float tmax = -INFINITY;
    for (int j = q4 * 16; j < q4 * 16 + 16; ++j)
      if (j <= lim && j >= low) tmax = fmaxf(tmax, Ss[r4 * 68 + j] * g.scale);
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
    tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
    const bool move = tmax > m_ref + REF_SLACK || (m_ref == -INFINITY && tmax > -INFINITY);
    float f = 1.f;
    if (move) {
      f = m_ref == -INFINITY ? 0.f : expf(m_ref - tmax);
      mysum *= f;
      m_ref = tmax;
    }
    if (q4 == 0) row_f[r4] = f;
    if (__syncthreads_or(move ? 1 : 0) && t != t_lo) {   // (before the first tile the accumulators are zero)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float fr[NE];
#pragma unroll
        for (int e = 0; e < NE; ++e) fr[e] = row_f[16 * i + frag_row[e]];
#pragma unroll
        for (int j = 0; j < NF; ++j)
#pragma unroll
          for (int e = 0; e < NE; ++e) oacc[i][j].x[e] *= fr[e];
      }
    }
    for (int j = q4 * 16; j < q4 * 16 + 16; ++j) {
      float p = 0.f;
      if (j <= lim && j >= low) p = expf(Ss[r4 * 68 + j] * g.scale - m_ref);
      const bf16 pb = __float2bfloat16_rn(p);
      Ps[r4 * 72 + j] = pb;
      mysum += __bfloat162float(pb);   // the weights that are summed are the weights that multiply the latents
    }
    __syncthreads();
    for (int kk = 0; kk < MA_KEYS; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fp[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (i < live_groups) wmma::load_matrix_sync(fp[i], Ps + (16 * i) * 72 + kk, 72);
#pragma unroll
      for (int j = 0; j < NF; ++j) {
        if (col0 + 16 * j >= R16) continue;  // warp-uniform
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> fv;
        wmma::load_matrix_sync(fv, Ks + kk * DP + col0 + 16 * j, DP);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (i < live_groups) wmma::mma_sync(oacc[i][j], fp[i], fv, oacc[i][j]);
      }
    }
  }
  mysum += __shfl_xor_sync(0xffffffffu, mysum, 1);
  mysum += __shfl_xor_sync(0xffffffffu, mysum, 2);
  __syncthreads();  // every warp is done with Qs / Ks: they become the output tile
  if (q4 == 0) {
    row_l[r4] = mysum;
    row_m[r4] = m_ref;
  }
  const int OLD = R16 + 4;
#pragma unroll
  for (int j = 0; j < NF; ++j) {
    if (col0 + 16 * j >= R16) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) wmma::store_matrix_sync(Os + (16 * i) * OLD + col0 + 16 * j, oacc[i][j], OLD, wmma::mem_row_major);
  }
  __syncthreads();
  for (int r = warp; r < MA_ROWS; r += MA_THREADS / 32) {
    const int row = first + r;
    if (row >= total) continue;
    const int tok = row / g.heads, head = row - tok * g.heads, lane = tid & 31;
    const size_t base = (size_t)(q_row0 + tok) * g.heads + head;
    const float m = row_m[r], l = row_l[r];
    if (a.nsplit == 1) {
      const float sk = a.sink != nullptr ? a.sink[head] : -INFINITY;
      const float mf = fmaxf(m, sk);
      const float corr = m == -INFINITY ? 0.f : expf(m - mf);
      const float inv = corr / (l * corr + expf(sk - mf));
      for (int d = lane; d < R; d += 32) a.out_lat[base * R + d] = __float2bfloat16_rn(Os[r * OLD + d] * inv);
    } else {
      float* dst = a.partial + (base * a.nsplit + split) * (R + 2);
      if (lane == 0) {
        dst[0] = m;
        dst[1] = l;
      }
      for (int d = lane; d < R; d += 32) dst[2 + d] = Os[r * OLD + d];
    }
  }
}

// folds the splits of every (token, head) row and the sink into the output; one CTA per row, thread d owns latent dims d, d + 128, ...
__global__ void __launch_bounds__(128) latent_merge_kernel(const float* __restrict__ partial, int nsplit, int R, int heads,
                                                           const int32_t* __restrict__ seq_lens, const float* __restrict__ sink,
                                                           bf16* __restrict__ out_lat, int nrows) {
  __shared__ float w_s[32];
  __shared__ float inv_s;
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x, lane = threadIdx.x & 31;
  const int tok = row / heads, head = row - tok * heads;
  if (seq_lens != nullptr && seq_lens[tok] <= 0) return;
  const float* p = partial + (size_t)row * nsplit * (R + 2);
  if (threadIdx.x < 32) {   // lane s holds split s (nsplit <= 32): its maximum, then its weight exp(m_s - m)
    const float sk = sink != nullptr ? sink[head] : -INFINITY;
    const float m = lane < nsplit ? p[(size_t)lane * (R + 2)] : -INFINITY;
    const float l = lane < nsplit ? p[(size_t)lane * (R + 2) + 1] : 0.f;
    const float mf = fmaxf(warp_max(m), sk);
    const float w = m == -INFINITY ? 0.f : expf(m - mf);
    const float den = warp_sum(l * w) + expf(sk - mf);
    w_s[lane] = w;
    if (lane == 0) inv_s = 1.0f / den;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < R; d += 128) {
    float acc = 0.f;
#pragma unroll 8
    for (int s = 0; s < nsplit; ++s) acc = fmaf(p[(size_t)s * (R + 2) + 2 + d], w_s[s], acc);
    out_lat[(size_t)row * R + d] = __float2bfloat16_rn(acc * inv_s);
  }
}

size_t mma_attn_smem(const LatentGeom& g) {
  const int D = g.kv_rank + g.rot_dim, DP = ((D + 15) & ~15) + 8;
  return (size_t)2 * MA_ROWS * DP * 2 + (size_t)MA_ROWS * 68 * 4 + (size_t)MA_ROWS * 72 * 2 + 4 * MA_ROWS * 4;
}

template <int NF>
int launch_mma(const MmaAttnArgs& a, dim3 grid, size_t smem, cudaStream_t s) {
  static B2PerDeviceOnce once;
  static size_t set_to = 0;
  if (once.need() || smem > set_to) {
    B2_CUDA_OK(cudaFuncSetAttribute(latent_attention_mma_kernel<NF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)std::max(smem, set_to)));
    set_to = std::max(smem, set_to);
  }
  B2_CUDA_OK(b2_launch(latent_attention_mma_kernel<NF>, grid, dim3(MA_THREADS), smem, s, a));
  return 0;
}

template <typename TC, typename TX, int NR>
int launch_la(const float* q_abs, const float* q_rot, const void* cache, const LatentGeom& g, const int32_t* block_table, int bt_stride,
              int block_size, const PrefillTile* tiles, int ntiles, const int32_t* positions, const int32_t* seq_lens, const float* sink,
              void* out_lat, int T, cudaStream_t s) {
  const int D = g.kv_rank + g.rot_dim;
  const size_t smem = ((size_t)LA_WARPS * D + (size_t)LA_KEYS * (D | 1)) * sizeof(float);
  auto kern = latent_attention_kernel<TC, TX, NR>;
  if (smem > 48 * 1024) {
    static B2PerDeviceOnce once;
    static size_t set_to = 0;
    if (once.need() || smem > set_to) {
      B2_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      set_to = smem;
    }
  }
  const int rows_per_tile = tiles != nullptr ? 64 : 1;
  dim3 grid(tiles != nullptr ? ntiles : T, (rows_per_tile * g.heads + LA_WARPS - 1) / LA_WARPS);
  B2_CUDA_OK(b2_launch(kern, grid, dim3(LA_WARPS * 32), smem, s, q_abs, q_rot, (const TC*)cache, g, block_table, bt_stride, block_size, tiles,
                       positions, seq_lens, sink, (TX*)out_lat));
  return 0;
}

template <typename TC, typename TX>
int launch_la_nr(int nr, const float* q_abs, const float* q_rot, const void* cache, const LatentGeom& g, const int32_t* block_table,
                 int bt_stride, int block_size, const PrefillTile* tiles, int ntiles, const int32_t* positions, const int32_t* seq_lens,
                 const float* sink, void* out_lat, int T, cudaStream_t s) {
#define LA(N) return launch_la<TC, TX, N>(q_abs, q_rot, cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, sink, out_lat, T, s)
  if (nr <= 1) LA(1);
  if (nr <= 2) LA(2);
  if (nr <= 4) LA(4);
  if (nr <= 8) LA(8);
  if (nr <= 16) LA(16);
  LA(32);
#undef LA
}

}  // namespace

int launch_latent_finish(const float* qd, int ld, const LatentGeom& g, int has_kv, const float* latent_gain, const int32_t* positions,
                         const int32_t* slots, void* q_nope, int x_f32, float* q_rot, void* cache, int cache_f32, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(g.rot_dims >= 0 && g.rot_dims <= g.rot_dim && g.rot_dims % 2 == 0, "latent_finish: rot_dims %d must be even and <= rot_dim %d",
             g.rot_dims, g.rot_dim);
  B2_REQUIRE(x_f32 == cache_f32, "latent_finish: operands and cache have one element type");
  const size_t smem = (size_t)std::max(g.rot_dims, 2) * sizeof(float);
  if (x_f32)
    B2_CUDA_OK(b2_launch(latent_finish_kernel<float, float>, dim3(T), dim3(128), smem, s, qd, ld, g, has_kv, latent_gain, positions, slots,
                         (float*)q_nope, q_rot, (float*)cache));
  else
    B2_CUDA_OK(b2_launch(latent_finish_kernel<bf16, bf16>, dim3(T), dim3(128), smem, s, qd, ld, g, has_kv, latent_gain, positions, slots,
                         (bf16*)q_nope, q_rot, (bf16*)cache));
  return 0;
}

int launch_latent_pair_finish(const float* proj, int ld, int off_q, int q_rank, int off_c, int kv_rank, const float* gain_q, const float* gain_c,
                              float eps, const int32_t* slots, void* xq, void* cache, int x_f32, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  if (x_f32)
    B2_CUDA_OK(b2_launch(latent_pair_finish_kernel<float, float>, dim3(T), dim3(128), 0, s, proj, ld, off_q, q_rank, off_c, kv_rank, gain_q, gain_c, eps,
                         slots, (float*)xq, (float*)cache));
  else
    B2_CUDA_OK(b2_launch(latent_pair_finish_kernel<bf16, bf16>, dim3(T), dim3(128), 0, s, proj, ld, off_q, q_rank, off_c, kv_rank, gain_q, gain_c, eps,
                         slots, (bf16*)xq, (bf16*)cache));
  return 0;
}

size_t latent_attention_scratch_floats(int max_rows, int max_heads, int max_rank) {
  // decode steps cut the keys into splits until every SM has a CTA; every (row block, split) leaves up to 64 rows
  return ((size_t)2 * 148 + (size_t)max_rows * ((max_heads + MA_ROWS - 1) / MA_ROWS)) * MA_ROWS * ((size_t)max_rank + 2);
}

int launch_latent_attention(const float* q_abs, const float* q_rot, const void* cache, int cache_f32, const LatentGeom& g,
                            const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                            const int32_t* positions, const int32_t* seq_lens, const float* sink, void* out_lat, int x_f32, int T,
                            cudaStream_t s, float* scratch, size_t scratch_floats, int max_context) {
  if (T <= 0 || (tiles != nullptr && ntiles <= 0)) return 0;
  static const bool use_mma = [] { const char* e = getenv("B2_LATENT_MMA"); return !(e && *e == '0'); }();
  const size_t mma_smem = mma_attn_smem(g);
  if (!cache_f32 && use_mma && g.kv_rank <= 512 && mma_smem <= 200 * 1024) {
    B2_REQUIRE(x_f32 == 0, "latent_attention: operands and cache have one element type");
    MmaAttnArgs a{q_abs, q_rot, (const bf16*)cache, g, block_table, bt_stride, block_size, tiles, positions, seq_lens, sink, (bf16*)out_lat, scratch, 1};
    const int blocks_y = ((tiles != nullptr ? 64 : 1) * g.heads + MA_ROWS - 1) / MA_ROWS;
    const int blocks = (tiles != nullptr ? ntiles : T) * blocks_y;
    if (tiles == nullptr && scratch != nullptr) {   // decode: few rows, long caches -> cut the keys
      int ns = 148 / std::max(blocks, 1);   // one CTA per SM fits (the operand slabs fill its shared memory): one wave
      ns = std::min(std::min(ns, 32), std::max(1, (max_context + MA_KEYS - 1) / MA_KEYS));
      while (ns > 1 && (size_t)T * g.heads * ns * (g.kv_rank + 2) > scratch_floats) --ns;
      a.nsplit = std::max(ns, 1);
    }
    const dim3 grid(tiles != nullptr ? ntiles : T, blocks_y, a.nsplit);
    const int nf = (g.kv_rank + 127) / 128;
    if (nf <= 1) B2_TRY_RC(launch_mma<1>(a, grid, mma_smem, s));
    else if (nf == 2) B2_TRY_RC(launch_mma<2>(a, grid, mma_smem, s));
    else B2_TRY_RC(launch_mma<4>(a, grid, mma_smem, s));
    if (a.nsplit > 1)
      B2_CUDA_OK(b2_launch(latent_merge_kernel, dim3(T * g.heads), dim3(128), 0, s, (const float*)scratch, a.nsplit, g.kv_rank, g.heads,
                           seq_lens, sink, (bf16*)out_lat, T * g.heads));
    return 0;
  }
  B2_REQUIRE(g.kv_rank >= 1 && g.kv_rank <= 1024, "latent_attention: kv_rank %d outside [1, 1024]", g.kv_rank);
  B2_REQUIRE(x_f32 == cache_f32, "latent_attention: operands and cache have one element type");
  const size_t smem = ((size_t)LA_WARPS * (g.kv_rank + g.rot_dim) + (size_t)LA_KEYS * ((g.kv_rank + g.rot_dim) | 1)) * sizeof(float);
  B2_REQUIRE(smem <= 200 * 1024, "latent_attention: kv_rank + rot_dim = %d needs %zu bytes of shared memory", g.kv_rank + g.rot_dim, smem);
  const int nr = (g.kv_rank + 31) / 32;
  if (cache_f32)
    return launch_la_nr<float, float>(nr, q_abs, q_rot, cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, sink,
                                      out_lat, T, s);
  return launch_la_nr<bf16, bf16>(nr, q_abs, q_rot, cache, g, block_table, bt_stride, block_size, tiles, ntiles, positions, seq_lens, sink,
                                  out_lat, T, s);
}

}  // namespace b2
