// attn_state.cu -- mixers whose memory is a matrix state per head instead of a cache of keys and values: a head keeps
// S [dim][vdim] in fp32, every token updates it and reads it out, and the state of a sequence lives in a slot of the
// engine's sequence table.  Two update rules share the kernels (StateGeom.rule):
//
//   STATE_RULE_DECAY   S <- diag(a_t) S + k_t v_t^T;                                  o_t = S^T q_t     (gated linear attention)
//   STATE_RULE_DELTA   S <- diag(a_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t     (gated delta rule)
//
// a_t is a decay per head and key channel in (0, 1); it scales the rows of S.  Query/key head of state head a is
// a / (heads / kv_heads).
//
// Everything here is fp32: the state, the decays (formed as exp(-rate * softplus(.)), never as a power of a rounded
// sigmoid), the step sizes, the unit norms, the read-out and its norm.  The inputs are the fp32 sums of the fused
// projection; only the gated read-out handed to the output projection is rounded to the operand type.
//
// A step must leave the same state when it is run twice from the same bookkeeping (the eager warm-up ahead of a graph
// capture): the state of a slot is kept twice, indexed by the parity of the last position it includes.  A portion that
// starts at position p reads copy (p - 1) & 1 (nothing when p == 0: a sequence starts from zero, so a slot that is
// used again needs no clearing) and writes copy (p + n - 1) & 1; a decode step therefore never overwrites what it
// reads.  The convolution keeps its last inputs in a ring of `taps` rows per slot indexed by position mod taps, for the
// same reason.
//
// The scan is sequential in time and parallel over (sequence, head, value column): a CTA owns up to 128 columns of one
// head's state for one portion, eight lanes share four neighbouring columns and split the key channels (channel i * 8 + j
// belongs to lane j), each lane keeps its channels of its columns in registers for the whole portion.  Tokens are staged through shared memory by asynchronous copies, a chunk ahead.  The arithmetic of a token does
// not depend on where the portion was cut, so prefill, chunked prefill and token-by-token decoding give the same bits.
//
// Kernels:
//   lowrank_act        y = act(W2 . lr + bias) for the low-rank second stages (decays, output gates), fp32
//   conv_unit_finish   delta rule: causal convolution + silu on q | k | v (a thread per channel), then unit vectors and the query scale
//                      (a warp per head), beta
//   conv_ring_store    the ring update, after every token of the step has read the ring
//   state_scan         the recurrence
//   state_out_gate     per-head RMS norm of the read-out with a gain, times the gate (silu or given), operand type out
#include "kernels.h"

namespace b2 {

namespace {

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// A CTA takes LR_TOKENS tokens and 256 output channels; a thread owns one channel, reads its row of w2 once (sixteen numbers at a
// time) and applies it to every token of the tile.  lr [T][ld] fp32 (rank numbers per token at column lr_off), staged in shared memory.
constexpr int LR_TOKENS = 8;
__global__ void __launch_bounds__(256) lowrank_act_kernel(const float* __restrict__ lr, int ld, int lr_off, int rank, const float* __restrict__ w2,
                                                          const float* __restrict__ bias, const float* __restrict__ rate_log, float rate,
                                                          int per_head, int mode, float* __restrict__ out, int C, int T) {
  extern __shared__ __align__(16) float lrs[];   // [LR_TOKENS][rank]
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * LR_TOKENS, tn = min(LR_TOKENS, T - t0);
  for (int i = threadIdx.x; i < tn * rank; i += 256) lrs[i] = lr[(size_t)(t0 + i / rank) * ld + lr_off + i % rank];
  __syncthreads();
  const int c = blockIdx.y * 256 + threadIdx.x;
  if (c >= C) return;
  const float* wr = w2 + (size_t)c * rank;
  float z[LR_TOKENS];
#pragma unroll
  for (int tt = 0; tt < LR_TOKENS; ++tt) z[tt] = 0.f;
  for (int r0 = 0; r0 < rank; r0 += 16) {
    float w[16];
#pragma unroll
    for (int x = 0; x < 16; ++x) w[x] = r0 + x < rank ? wr[r0 + x] : 0.f;
#pragma unroll
    for (int tt = 0; tt < LR_TOKENS; ++tt) {
      if (tt < tn) {
        const float* l = lrs + tt * rank + r0;
        if ((rank & 3) == 0) {     // sixteen bytes of the token's low-rank values at a time
#pragma unroll
          for (int x = 0; x < 16; x += 4)
            if (r0 + x < rank) {
              const float4 lv = *reinterpret_cast<const float4*>(l + x);
              z[tt] = fmaf(w[x], lv.x, z[tt]);
              z[tt] = fmaf(w[x + 1], lv.y, z[tt]);
              z[tt] = fmaf(w[x + 2], lv.z, z[tt]);
              z[tt] = fmaf(w[x + 3], lv.w, z[tt]);
            }
        } else {
#pragma unroll
          for (int x = 0; x < 16; ++x)
            if (r0 + x < rank) z[tt] = fmaf(w[x], l[x], z[tt]);
        }
      }
    }
  }
  const float b = bias ? bias[c] : 0.f;
  const float rt = mode == LOWRANK_DECAY_SOFTPLUS ? expf(rate_log[c / per_head]) : rate;
#pragma unroll
  for (int tt = 0; tt < LR_TOKENS; ++tt) {
    if (tt >= tn) break;
    const float zz = z[tt] + b;
    float y;
    if (mode == LOWRANK_SIGMOID) y = sigmoid_f(zz);
    else if (mode == LOWRANK_DECAY_SIGMOID_POW) y = expf(-rt * softplus_f(-zz));               // sigmoid(z)^rate
    else y = expf(-rt * softplus_f(zz));                                                       // exp(-exp(A) softplus(z))
    out[(size_t)(t0 + tt) * C + c] = y;
  }
}

// A CTA takes `upc` head units of one token (query heads, key heads, value heads, in the order of the projection's columns): first every
// thread convolves and activates channels of the CTA's range, then a warp per query / key head turns the head into a unit vector.
// proj [T][ld] fp32 = q (kv_heads*dim) | k (kv_heads*dim) | v (heads*vdim) | beta logits (heads) | ...; out [T][C] = the finished q | k | v,
// beta_out [T][heads].
template <int TAPS>   // 0: any number of taps
__global__ void __launch_bounds__(256) conv_unit_finish_kernel(const float* __restrict__ proj, int ld, StateGeom g, int taps_any,
                                                               const float* __restrict__ conv_w, const float* __restrict__ ring,
                                                               const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_first,
                                                               const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                                                               float unit_eps, float* __restrict__ out, float* __restrict__ beta_out, int upc) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (slots[t] < 0) return;
  const int taps = TAPS > 0 ? TAPS : taps_any;
  const int pos = positions[t];
  const int nqk = g.kv_heads * g.dim, nv = g.heads * g.vdim, C = 2 * nqk + nv;
  const int units = 2 * g.kv_heads + g.heads, u_lo = blockIdx.y * upc, u_hi = min(units, u_lo + upc);
  auto unit_c0 = [&](int u) { return u < 2 * g.kv_heads ? u * g.dim : 2 * nqk + (u - 2 * g.kv_heads) * g.vdim; };
  const int c_lo = unit_c0(u_lo), c_hi = u_hi == units ? C : unit_c0(u_hi);
  const int back = t - row_first[t];
  const float* row = proj + (size_t)t * ld;
  const float* rg = ring + (size_t)row_seq[t] * taps * C;
  float* orow = out + (size_t)t * C;
  for (int c = c_lo + threadIdx.x; c < c_hi; c += 256) {
    float acc = 0.f;
    if constexpr (TAPS > 0) {                 // every load of the channel in flight at once
      float xx[TAPS], ww[TAPS];
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const int d = TAPS - 1 - j;
        ww[j] = conv_w[(size_t)c * TAPS + j];
        xx[j] = d <= back ? (row - (size_t)d * ld)[c] : (pos - d >= 0 ? rg[(size_t)((pos - d) % TAPS) * C + c] : 0.f);
      }
#pragma unroll
      for (int j = 0; j < TAPS; ++j) acc = fmaf(ww[j], xx[j], acc);
    } else {
      for (int j = 0; j < taps; ++j) {        // y_t = sum_j w[c][j] * x_(t - taps + 1 + j), the last column is the current token's
        const int d = taps - 1 - j;
        float xx = 0.f;
        if (d <= back) xx = (row - (size_t)d * ld)[c];
        else if (pos - d >= 0) xx = rg[(size_t)((pos - d) % taps) * C + c];
        acc = fmaf(conv_w[(size_t)c * taps + j], xx, acc);
      }
    }
    orow[c] = silu_f(acc);
  }
  __syncthreads();   // (the CTA reads back only what it wrote itself)
  const float qscale = rsqrtf((float)g.dim);
  for (int u = u_lo + warp; u < min(u_hi, 2 * g.kv_heads); u += 8) {
    float* h = orow + u * g.dim;
    float ss = 0.f;
    for (int i = lane; i < g.dim; i += 32) ss = fmaf(h[i], h[i], ss);
    ss = warp_sum(ss);
    const float r = (1.0f / sqrtf(ss + unit_eps)) * (u < g.kv_heads ? qscale : 1.0f);
    for (int i = lane; i < g.dim; i += 32) h[i] *= r;
  }
  if (blockIdx.y == 0)
    for (int a = threadIdx.x; a < g.heads; a += 256) beta_out[(size_t)t * g.heads + a] = sigmoid_f(row[C + a]);
}

__global__ void __launch_bounds__(128) conv_ring_store_kernel(const float* __restrict__ proj, int ld, int C, int taps, float* __restrict__ ring,
                                                              const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_end,
                                                              const int32_t* __restrict__ positions, const int32_t* __restrict__ slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  if (slots[t] < 0) return;
  if (row_end[t] - 1 - t >= taps) return;  // a later token of the same portion owns this ring row
  float* dst = ring + ((size_t)row_seq[t] * taps + positions[t] % taps) * C;
  const float* row = proj + (size_t)t * ld;
  for (int c = threadIdx.x; c < C; c += 128) dst[c] = row[c];
}

constexpr int SC_LANES = 8;     // lanes that share a group of state columns and split the key channels
constexpr int SC_CHUNK = 8;     // tokens of one stage (two stages)

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// grid (portions, heads, column tiles); block (cols / NC) * 8.  Eight lanes share NC neighbouring columns of the state and split the key
// channels (channel i * 8 + j belongs to lane j; DPT channels per lane, dim <= 8 * DPT), so a value of q, k or the decay read from shared
// memory serves NC columns.  Shared-memory rows hold lane j's channels side by side (at j * (DPT + 4) + i; the pad of four words spreads the
// eight lanes over the banks) and are read sixteen bytes at a time.  Tokens arrive by asynchronous copies, the chunk after the one being
// worked on always in flight.  q is scaled at the read-out (S^T (c q) = c S^T q).
template <int DPT, int NC, int RULE>
__global__ void __launch_bounds__(256) state_scan_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ k, int ldk,
                                                         const float* __restrict__ v, int ldv, const float* __restrict__ decay,
                                                         const float* __restrict__ beta, StateGeom g, float qscale, float* __restrict__ state,
                                                         const int32_t* __restrict__ last_rows, const int32_t* __restrict__ row_seq,
                                                         const int32_t* __restrict__ row_first, const int32_t* __restrict__ row_end,
                                                         const int32_t* __restrict__ positions, const int32_t* __restrict__ slots,
                                                         float* __restrict__ out, int cols) {
  constexpr int LS = DPT + 4;               // words of one lane's channels in a staged row
  constexpr int RS = LS * SC_LANES;         // words of a staged row
  constexpr int CH = DPT >= 32 ? SC_CHUNK / 2 : SC_CHUNK;   // (static shared memory ends at 48 KB)
  constexpr int VW = DPT >= 4 ? 4 : DPT;    // channels per shared-memory load
  constexpr int DP = DPT * SC_LANES;
  constexpr int MAXC = 32 * NC;             // columns of a CTA at most
  __shared__ __align__(16) float qs[2][CH][RS], ks[2][CH][RS], as[2][CH][RS];
  __shared__ __align__(16) float vs[2][CH][MAXC];
  __shared__ float bs[2][CH];
  pdl_wait();
  pdl_launch_dependents();
  const int r_last = last_rows ? last_rows[blockIdx.x] : (int)blockIdx.x;
  const int first = row_first[r_last], end = row_end[r_last];
  if (slots[first] < 0) return;   // padding row of a decode bucket
  const int a = blockIdx.y, kh = a / (g.heads / g.kv_heads);
  const int col0 = blockIdx.z * cols;
  const int grp = threadIdx.x / SC_LANES, j = threadIdx.x % SC_LANES;
  const int cl = grp * NC;                  // first of this thread's columns within the CTA's tile
  const int pos0 = positions[first], n = end - first;
  const int nthreads = blockDim.x;
  const size_t head_floats = (size_t)g.dim * g.vdim;
  float* sbase = state + ((size_t)row_seq[first] * 2 * g.heads) * head_floats;
  const float* s_in = sbase + ((size_t)((pos0 + 1) & 1) * g.heads + a) * head_floats;
  float* s_out = sbase + ((size_t)((pos0 + n - 1) & 1) * g.heads + a) * head_floats;
  // channels past dim and columns past vdim never change: zero keys, queries and values, a decay of one
  for (int i = threadIdx.x; i < 2 * CH * (DP - g.dim); i += nthreads) {
    const int st = i / (CH * (DP - g.dim)), rem = i % (CH * (DP - g.dim)), tt = rem / (DP - g.dim), d = g.dim + rem % (DP - g.dim);
    const int at = (d % SC_LANES) * LS + d / SC_LANES;
    qs[st][tt][at] = 0.f;
    ks[st][tt][at] = 0.f;
    as[st][tt][at] = 1.f;
  }
  const int vcols = min(cols, g.vdim - col0);
  for (int i = threadIdx.x; i < 2 * CH * MAXC; i += nthreads) (&vs[0][0][0])[i] = 0.f;
  __syncthreads();
  // (flat loops over a chunk's numbers keep every thread's copies in flight together; sizes that are powers of two -- the usual case --
  // index by shifts instead of divisions)
  const int dsh = (g.dim & (g.dim - 1)) == 0 ? 31 - __clz(g.dim) : -1, vsh = (vcols & (vcols - 1)) == 0 ? 31 - __clz(vcols) : -1;
  const float* qb = q + (size_t)first * ldq + kh * g.dim;
  const float* kb = k + (size_t)first * ldk + kh * g.dim;
  const float* ab = decay + (size_t)first * ((size_t)g.heads * g.dim) + a * g.dim;
  const float* vb = v + (size_t)first * ldv + a * g.vdim + col0;
  const int lda = g.heads * g.dim;
  auto issue = [&](int c0, int st) {
    const int cn = min(CH, n - c0);
    for (int i = threadIdx.x; i < cn * g.dim; i += nthreads) {
      const int tt = dsh >= 0 ? i >> dsh : i / g.dim, d = dsh >= 0 ? i & (g.dim - 1) : i % g.dim, at = (d % SC_LANES) * LS + d / SC_LANES;
      const int row = c0 + tt;
      cp_async_f32(&qs[st][tt][at], qb + (size_t)row * ldq + d);
      cp_async_f32(&ks[st][tt][at], kb + (size_t)row * ldk + d);
      cp_async_f32(&as[st][tt][at], ab + (size_t)row * lda + d);
    }
    for (int i = threadIdx.x; i < cn * vcols; i += nthreads) {
      const int tt = vsh >= 0 ? i >> vsh : i / vcols, c = vsh >= 0 ? i & (vcols - 1) : i % vcols;
      cp_async_f32(&vs[st][tt][c], vb + (size_t)(c0 + tt) * ldv + c);
    }
    if (RULE == STATE_RULE_DELTA)
      for (int i = threadIdx.x; i < cn; i += nthreads) cp_async_f32(&bs[st][i], beta + (size_t)(first + c0 + i) * g.heads + a);
    cp_async_commit();
  };
  issue(0, 0);
  float s[DPT][NC];
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = i * SC_LANES + j;
#pragma unroll
    for (int c = 0; c < NC; ++c) s[i][c] = (pos0 > 0 && d < g.dim && col0 + cl + c < g.vdim) ? s_in[(size_t)d * g.vdim + col0 + cl + c] : 0.f;
  }
  auto load = [&](const float* p, int i, float* dst) {
    if constexpr (VW == 4) {
      const float4 x = *reinterpret_cast<const float4*>(p + i);
      dst[0] = x.x; dst[1] = x.y; dst[2] = x.z; dst[3] = x.w;
    } else if constexpr (VW == 2) {
      const float2 x = *reinterpret_cast<const float2*>(p + i);
      dst[0] = x.x; dst[1] = x.y;
    } else {
      dst[0] = p[i];
    }
  };
  int st = 0;
  for (int c0 = 0; c0 < n; c0 += CH, st ^= 1) {
    const int cn = min(CH, n - c0);
    if (c0 + CH < n) {
      issue(c0 + CH, st ^ 1);     // (every thread left that stage at the barrier that ended the chunk before this one)
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      float vc[NC];
      if constexpr (NC == 4) {
        const float4 x = *reinterpret_cast<const float4*>(&vs[st][tt][cl]);
        vc[0] = x.x; vc[1] = x.y; vc[2] = x.z; vc[3] = x.w;
      } else {
#pragma unroll
        for (int c = 0; c < NC; ++c) vc[c] = vs[st][tt][cl + c];
      }
      const float* ap = &as[st][tt][j * LS];
      const float* kp = &ks[st][tt][j * LS];
      const float* qp = &qs[st][tt][j * LS];
      float av[VW], kw[VW], qv[VW], acc[NC];
#pragma unroll
      for (int c = 0; c < NC; ++c) acc[c] = 0.f;
      if (RULE == STATE_RULE_DECAY) {
#pragma unroll
        for (int i = 0; i < DPT; i += VW) {
          load(ap, i, av);
          load(kp, i, kw);
          load(qp, i, qv);
#pragma unroll
          for (int x = 0; x < VW; ++x)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              s[i + x][c] = fmaf(av[x], s[i + x][c], kw[x] * vc[c]);
              acc[c] = fmaf(s[i + x][c], qv[x], acc[c]);
            }
        }
      } else {
        float kv[NC];
#pragma unroll
        for (int c = 0; c < NC; ++c) kv[c] = 0.f;
#pragma unroll
        for (int i = 0; i < DPT; i += VW) {
          load(ap, i, av);
          load(kp, i, kw);
#pragma unroll
          for (int x = 0; x < VW; ++x)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              s[i + x][c] *= av[x];
              kv[c] = fmaf(s[i + x][c], kw[x], kv[c]);
            }
        }
        const float bt = bs[st][tt];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          kv[c] += __shfl_xor_sync(0xffffffffu, kv[c], 1);
          kv[c] += __shfl_xor_sync(0xffffffffu, kv[c], 2);
          kv[c] += __shfl_xor_sync(0xffffffffu, kv[c], 4);
          kv[c] = bt * (vc[c] - kv[c]);     // u
        }
#pragma unroll
        for (int i = 0; i < DPT; i += VW) {
          load(kp, i, kw);
          load(qp, i, qv);
#pragma unroll
          for (int x = 0; x < VW; ++x)
#pragma unroll
            for (int c = 0; c < NC; ++c) {
              s[i + x][c] = fmaf(kw[x], kv[c], s[i + x][c]);
              acc[c] = fmaf(s[i + x][c], qv[x], acc[c]);
            }
        }
      }
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 4);
      }
      if (j == 0) {
        float* orow = out + (size_t)(first + c0 + tt) * ((size_t)g.heads * g.vdim) + a * g.vdim + col0 + cl;
#pragma unroll
        for (int c = 0; c < NC; ++c)
          if (col0 + cl + c < g.vdim) orow[c] = acc[c] * qscale;
      }
    }
    __syncthreads();   // the chunk has been consumed: its stage may be filled again
  }
#pragma unroll
  for (int i = 0; i < DPT; ++i) {
    const int d = i * SC_LANES + j;
#pragma unroll
    for (int c = 0; c < NC; ++c)
      if (d < g.dim && col0 + cl + c < g.vdim) s_out[(size_t)d * g.vdim + col0 + cl + c] = s[i][c];
  }
}

// One warp per (token, head): y = o / sqrt(mean(o^2) + eps) * gain * gate, gate = silu(gate_in) or gate_in as it is.
template <typename TX>
__global__ void __launch_bounds__(128) state_out_gate_kernel(const float* __restrict__ o, const float* __restrict__ gain,
                                                             const float* __restrict__ gate, int gate_ld, int gate_silu, TX* __restrict__ out,
                                                             int heads, int vdim, float eps, int T) {
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long unit = (long)blockIdx.x * 4 + warp;
  if (unit >= (long)T * heads) return;
  const int t = (int)(unit / heads), a = (int)(unit % heads);
  const float* orow = o + ((size_t)t * heads + a) * vdim;
  const float* grow = gate + (size_t)t * gate_ld + (size_t)a * vdim;
  float ss = 0.f;
  for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / (float)vdim + eps);
  TX* dst = out + ((size_t)t * heads + a) * vdim;
  for (int i = lane; i < vdim; i += 32) {
    const float gt = gate_silu ? silu_f(grow[i]) : grow[i];
    dst[i] = (TX)(orow[i] * r * gain[i] * gt);
  }
}

template <int RULE>
int launch_scan_rule(int dpt, dim3 grid, dim3 block, cudaStream_t s, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                     const float* decay, const float* beta, const StateGeom& g, float qscale, float* state, const int32_t* last_rows,
                     const int32_t* row_seq, const int32_t* row_first, const int32_t* row_end, const int32_t* positions, const int32_t* slots,
                     float* out, int cols) {
#define B2_SCAN_CASE(D, N)                                                                                                                    \
  case D:                                                                                                                                     \
    B2_CUDA_OK(b2_launch(state_scan_kernel<D, N, RULE>, grid, block, 0, s, q, ldq, k, ldk, v, ldv, decay, beta, g, qscale, state, last_rows,  \
                         row_seq, row_first, row_end, positions, slots, out, cols));                                                          \
    return 0;
  switch (dpt) {
    B2_SCAN_CASE(1, 4)
    B2_SCAN_CASE(2, 4)
    B2_SCAN_CASE(4, 4)
    B2_SCAN_CASE(8, 4)
    B2_SCAN_CASE(16, 4)
    B2_SCAN_CASE(32, 2)
  }
#undef B2_SCAN_CASE
  b2_set_error("state_scan: key width %d not built (at most 256)", g.dim);
  return -22;
}

}  // namespace

int launch_lowrank_act(const float* lr, int ld, int lr_off, int rank, const float* w2, const float* bias, int mode, float rate,
                       const float* rate_log, int per_head, float* out, int T, int C, cudaStream_t s) {
  if (T <= 0 || C <= 0) return 0;
  B2_REQUIRE(rank >= 1 && rank <= 1024, "lowrank_act: rank %d (at most 1024)", rank);
  B2_REQUIRE(mode != LOWRANK_DECAY_SOFTPLUS || (rate_log != nullptr && per_head >= 1), "lowrank_act: the softplus decay needs a rate per head");
  const dim3 grid((T + LR_TOKENS - 1) / LR_TOKENS, (C + 255) / 256);
  B2_CUDA_OK(b2_launch(lowrank_act_kernel, grid, dim3(256), (size_t)LR_TOKENS * rank * 4, s, lr, ld, lr_off, rank, w2, bias, rate_log, rate,
                       per_head > 0 ? per_head : 1, mode, out, C, T));
  return 0;
}

int launch_conv_unit_finish(const float* proj, int ld, const StateGeom& g, int taps, const float* conv_w, float* ring, const int32_t* row_seq,
                            const int32_t* row_first, const int32_t* row_end, const int32_t* positions, const int32_t* slots, float unit_eps,
                            float* out, float* beta_out, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(taps >= 1 && conv_w && (ring || taps == 1) && row_seq && row_first && row_end, "conv_unit_finish: the convolution needs its weights and state");
  const int C = 2 * g.kv_heads * g.dim + g.heads * g.vdim;
  const int units = 2 * g.kv_heads + g.heads, upc = T >= 256 ? units : std::max(1, (units + 15) / 16);   // few tokens: up to sixteen CTAs each
  const dim3 grid(T, (units + upc - 1) / upc);
#define B2_CONV_FINISH(TAPS)                                                                                                                      \
  B2_CUDA_OK(b2_launch(conv_unit_finish_kernel<TAPS>, grid, dim3(256), 0, s, proj, ld, g, taps, conv_w, (const float*)ring, row_seq, row_first, positions, \
                       slots, unit_eps, out, beta_out, upc))
  if (taps == 4) B2_CONV_FINISH(4);
  else if (taps == 3) B2_CONV_FINISH(3);
  else if (taps == 2) B2_CONV_FINISH(2);
  else B2_CONV_FINISH(0);
#undef B2_CONV_FINISH
  if (taps > 1)
    B2_CUDA_OK(b2_launch(conv_ring_store_kernel, dim3(T), dim3(128), 0, s, proj, ld, C, taps, ring, row_seq, row_end, positions, slots));
  return 0;
}

int launch_state_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* decay, const float* beta,
                      const StateGeom& g, float qscale, float* state, int portions, const int32_t* last_rows, const int32_t* row_seq,
                      const int32_t* row_first, const int32_t* row_end, const int32_t* positions, const int32_t* slots, float* out,
                      cudaStream_t s) {
  if (portions <= 0) return 0;
  B2_REQUIRE(g.heads >= 1 && g.kv_heads >= 1 && g.heads % g.kv_heads == 0 && g.dim >= 1 && g.vdim >= 1, "state_scan: bad sizes");
  B2_REQUIRE(g.rule == STATE_RULE_DECAY || (g.rule == STATE_RULE_DELTA && beta != nullptr), "state_scan: rule %d", g.rule);
  int dpt = 1;
  while (dpt * SC_LANES < g.dim) dpt *= 2;
  B2_REQUIRE(dpt <= 32, "state_scan: key width %d not built (at most 256)", g.dim);
  // a warp is four groups of eight lanes, a group owns nc neighbouring columns; as many columns per CTA (at most eight warps) as still
  // leave two CTAs for every SM (a column's arithmetic does not depend on the tile it falls into)
  const int nc = dpt >= 32 ? 2 : 4, step = 4 * nc;
  int cols = std::min(32 * nc, (g.vdim + step - 1) / step * step);
  while (cols > step && (long)portions * g.heads * ((g.vdim + cols - 1) / cols) < 2L * device_num_sms()) cols = (cols / 2 + step - 1) / step * step;
  const dim3 grid(portions, g.heads, (g.vdim + cols - 1) / cols), block(cols / nc * SC_LANES);
  if (g.rule == STATE_RULE_DECAY)
    return launch_scan_rule<STATE_RULE_DECAY>(dpt, grid, block, s, q, ldq, k, ldk, v, ldv, decay, beta, g, qscale, state, last_rows, row_seq,
                                              row_first, row_end, positions, slots, out, cols);
  return launch_scan_rule<STATE_RULE_DELTA>(dpt, grid, block, s, q, ldq, k, ldk, v, ldv, decay, beta, g, qscale, state, last_rows, row_seq,
                                            row_first, row_end, positions, slots, out, cols);
}

size_t state_floats_per_slot(const StateGeom& g) { return (size_t)2 * g.heads * g.dim * g.vdim; }

int launch_state_out_gate(const float* o, const float* gain, const float* gate, int gate_ld, int gate_silu, void* out, int out_f32,
                          int heads, int vdim, float eps, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  const long units = (long)T * heads;
  const dim3 grid((unsigned)((units + 3) / 4));
  if (out_f32) B2_CUDA_OK(b2_launch(state_out_gate_kernel<float>, grid, dim3(128), 0, s, o, gain, gate, gate_ld, gate_silu, (float*)out, heads, vdim, eps, T));
  else B2_CUDA_OK(b2_launch(state_out_gate_kernel<bf16>, grid, dim3(128), 0, s, o, gain, gate, gate_ld, gate_silu, (bf16*)out, heads, vdim, eps, T));
  return 0;
}

}  // namespace b2
