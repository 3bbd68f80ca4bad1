// resid_f32.cu -- element-wise kernels around an fp32 residual stream: the embedding lookup with its norm, the
// unit-offset RMS norm  x / sqrt(mean(x^2) + eps) * (1 + g)  that feeds both branches of a parallel layer from ONE
// statistic, and the tail of the lm_head (greedy token, the sampler's bf16 rows).
//
// The bf16 families keep their residual stream in bf16 (elementwise.cu reproduces HF's rounding points); families that
// ask for an fp32 stream (Lerasun) use these.  Statistics, gains and the stream itself are fp32 throughout; only the
// operand handed to the next projection is rounded to bf16, and not even that when the engine runs in fp32.
// One CTA of 128 threads per token row; any width.
#include "kernels.h"

namespace b2 {

namespace {

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  const float r = red[0] + red[1] + red[2] + red[3];
  __syncthreads();
  return r;
}

// the same for a CTA of NT threads (NT a multiple of 32, at most 1024)
template <int NT>
__device__ __forceinline__ float block_sum_n(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) r += red[w];
  __syncthreads();
  return r;
}

template <typename TT>
__global__ void __launch_bounds__(128) embed_unit_norm_kernel(const int32_t* __restrict__ ids, const TT* __restrict__ table,
                                                              const float* __restrict__ gain1p, float* __restrict__ h, int W, int vocab,
                                                              float eps) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const TT* row = table + (size_t)id * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float v = (float)row[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum_128(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 128) h[(size_t)t * W + i] = (float)row[i] * r * gain1p[i];
}

template <typename TX>
__global__ void __launch_bounds__(128) unit_norm2_kernel(const float* __restrict__ h, const float* __restrict__ gain_a,
                                                         const float* __restrict__ gain_b, TX* __restrict__ x1, TX* __restrict__ x2, int W,
                                                         float eps, const int32_t* __restrict__ rows) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* src = h + (size_t)(rows ? rows[t] : t) * W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float v = src[i];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum_128(ss, red);
  const float r = 1.0f / sqrtf(ss / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 128) {
    const float v = src[i] * r;
    x1[(size_t)t * W + i] = (TX)(v * gain_a[i]);
    if (x2 != nullptr) x2[(size_t)t * W + i] = (TX)(v * gain_b[i]);
  }
}

__global__ void __launch_bounds__(1024) logits_finish_kernel(const float* __restrict__ logits, int32_t* __restrict__ out_tokens,
                                                            bf16* __restrict__ lb, int lb_rows, int V, int v_pad) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= lb_rows) lb = nullptr;
  const float* row = logits + (size_t)r * V;
  float best = -INFINITY;
  int besti = 0x7fffffff;
#pragma unroll 4
  for (int i = threadIdx.x; i < v_pad; i += 1024) {
    const float v = i < V ? row[i] : -INFINITY;
    if (lb != nullptr) lb[(size_t)r * v_pad + i] = __float2bfloat16_rn(v);
    if (i < V && (v > best || (v == best && i < besti))) {
      best = v;
      besti = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) {
      best = ov;
      besti = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    bv[threadIdx.x >> 5] = best;
    bi[threadIdx.x >> 5] = besti;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 32; ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < besti)) {
        best = bv[w];
        besti = bi[w];
      }
    out_tokens[r] = besti == 0x7fffffff ? 0 : besti;
  }
}

// ---- grouped RMS norm with a plain gain (Kedasun): the vector is `groups` equal pieces, each with its own statistic ----
template <typename TT>
__global__ void __launch_bounds__(128) embed_scaled_kernel(const int32_t* __restrict__ ids, const TT* __restrict__ table, float scale,
                                                           float* __restrict__ h, int W, int vocab) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  const TT* row = table + (size_t)id * W;
  for (int i = threadIdx.x; i < W; i += 128) h[(size_t)t * W + i] = (float)row[i] * scale;
}

// One warp per piece; a token's pieces are spread over the warps of one CTA, or of several when the step has few tokens.  ADD: h += norm(y + bias) * gain, and when
// gain_next is given the norm in front of the next sublayer follows at once, x = norm(h) * gain_next (the pieces of both
// norms are the same, so the warp that updated a piece normalises it).
constexpr int GN_REG = 16;   // values of a piece a lane keeps in registers (pieces up to 512 wide)
// EARLY (steps of few tokens, where a launch is all latency): every operand is loaded before the first reduction -- one round trip
// to memory instead of one per phase; prompt-sized steps load late and keep the registers for occupancy.
template <typename TX, bool ADD, bool EARLY>
__global__ void __launch_bounds__(128) group_norm_kernel(const float* __restrict__ src, const float* __restrict__ bias,
                                                         const float* __restrict__ gain, TX* __restrict__ x, float* __restrict__ h, int W,
                                                         int groups, float eps, const int32_t* __restrict__ rows,
                                                         const float* __restrict__ gain_next) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int piece = W / groups;
  const float* row = src + (size_t)(rows ? rows[t] : t) * W;
  // pieces round robin over the warps of the token's CTAs (gridDim.y CTAs of four warps: few tokens get more CTAs each)
  for (int gi = blockIdx.y * 4 + warp; gi < groups; gi += 4 * gridDim.y) {
    const int o = gi * piece;
    if (piece <= 32 * GN_REG) {
      // the piece fits the warp's registers: every load of a pass is in flight at once, and nothing is read twice
      float v[GN_REG], gv[GN_REG], hv[GN_REG], gn[GN_REG], ss = 0.f;
#pragma unroll
      for (int k = 0; k < GN_REG; ++k) {
        const int i = lane + 32 * k;
        const bool in = i < piece;
        v[k] = in ? row[o + i] + (bias ? bias[o + i] : 0.f) : 0.f;
        gv[k] = (EARLY && in) ? gain[o + i] : 0.f;
        hv[k] = (EARLY && ADD && in) ? h[(size_t)t * W + o + i] : 0.f;
        gn[k] = (EARLY && ADD && in && gain_next != nullptr) ? gain_next[o + i] : 0.f;
        ss = fmaf(v[k], v[k], ss);
      }
      ss = warp_sum(ss);
      const float r = 1.0f / sqrtf(ss / (float)piece + eps);
      float ss2 = 0.f;
#pragma unroll
      for (int k = 0; k < GN_REG; ++k) {
        const int i = lane + 32 * k;
        if (i < piece) {
          v[k] = v[k] * r * (EARLY ? gv[k] : gain[o + i]);
          if (ADD) {
            v[k] += EARLY ? hv[k] : h[(size_t)t * W + o + i];
            h[(size_t)t * W + o + i] = v[k];
            ss2 = fmaf(v[k], v[k], ss2);
          } else {
            x[(size_t)t * W + o + i] = (TX)v[k];
          }
        }
      }
      if (ADD && gain_next != nullptr) {
        ss2 = warp_sum(ss2);
        const float r2 = 1.0f / sqrtf(ss2 / (float)piece + eps);
#pragma unroll
        for (int k = 0; k < GN_REG; ++k) {
          const int i = lane + 32 * k;
          if (i < piece) x[(size_t)t * W + o + i] = (TX)(v[k] * r2 * (EARLY ? gn[k] : gain_next[o + i]));
        }
      }
      continue;
    }
    float ss = 0.f;
    for (int i = lane; i < piece; i += 32) {
      const float v = row[o + i] + (bias ? bias[o + i] : 0.f);
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)piece + eps);
    float ss2 = 0.f;
    for (int i = lane; i < piece; i += 32) {
      const float v = (row[o + i] + (bias ? bias[o + i] : 0.f)) * r * gain[o + i];
      if (ADD) {
        const float hn = h[(size_t)t * W + o + i] + v;
        h[(size_t)t * W + o + i] = hn;
        ss2 = fmaf(hn, hn, ss2);
      } else {
        x[(size_t)t * W + o + i] = (TX)v;
      }
    }
    if (ADD && gain_next != nullptr) {
      ss2 = warp_sum(ss2);
      const float r2 = 1.0f / sqrtf(ss2 / (float)piece + eps);
      for (int i = lane; i < piece; i += 32) x[(size_t)t * W + o + i] = (TX)(h[(size_t)t * W + o + i] * r2 * gain_next[o + i]);  // its own writes
    }
  }
}

template <typename TX>
__global__ void __launch_bounds__(256) clamped_gate_kernel(const float* __restrict__ gu, TX* __restrict__ act, int F, float limit, float sharp) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* row = gu + (size_t)t * 2 * F;
  if (F % 4 == 0) {   // four features per thread: 16-byte loads of gate and up, one 8-byte (bf16) or 16-byte (fp32) store
    for (int i = (blockIdx.y * 256 + threadIdx.x) * 4; i < F; i += 1024 * gridDim.y) {
      const float4 gq = *reinterpret_cast<const float4*>(row + i), uq = *reinterpret_cast<const float4*>(row + F + i);
      const float gs[4] = {gq.x, gq.y, gq.z, gq.w}, us[4] = {uq.x, uq.y, uq.z, uq.w};
      float y[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float g = fminf(gs[k], limit), u = fminf(fmaxf(us[k], -limit), limit);
        y[k] = g / (1.0f + expf(-sharp * g)) * (u + 1.0f);
      }
      TX* dst = act + (size_t)t * F + i;
      if constexpr (sizeof(TX) == 4) {
        *reinterpret_cast<float4*>(dst) = make_float4(y[0], y[1], y[2], y[3]);
      } else {
        uint2 pk;
        pk.x = pack_bf16x2(y[0], y[1]);
        pk.y = pack_bf16x2(y[2], y[3]);
        *reinterpret_cast<uint2*>(dst) = pk;
      }
    }
    return;
  }
  for (int i = blockIdx.y * 256 + threadIdx.x; i < F; i += 256 * gridDim.y) {
    const float g = fminf(row[i], limit);
    const float u = fminf(fmaxf(row[F + i], -limit), limit);
    act[(size_t)t * F + i] = (TX)(g / (1.0f + expf(-sharp * g)) * (u + 1.0f));
  }
}

// ---- a parallel layer with ONE norm and several branches (Bumalix) ----
template <typename TX>
__global__ void __launch_bounds__(256) store_rows_kernel(const float* __restrict__ src, TX* __restrict__ x, int ldx, int col0, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W; i += 256) x[(size_t)t * ldx + col0 + i] = (TX)src[(size_t)t * W + i];
}

// One CTA of 128 threads per token row: three power sums in one pass, then the polynomial of the three unit-RMS vectors.
template <typename TX>
__global__ void __launch_bounds__(128) poly_norm_kernel(const float* __restrict__ z, const float* __restrict__ coef, TX* __restrict__ act, int F,
                                                        float eps) {
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* row = z + (size_t)t * F;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < F; i += 128) {
    const float v = row[i], v2 = v * v, v3 = v2 * v;
    s2 = fmaf(v, v, s2);
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  s2 = block_sum_128(s2, red);
  s4 = block_sum_128(s4, red);
  s6 = block_sum_128(s6, red);
  const float r1 = coef[0] / sqrtf(s2 / (float)F + eps), r2 = coef[1] / sqrtf(s4 / (float)F + eps), r3 = coef[2] / sqrtf(s6 / (float)F + eps);
  const float e = coef[3];
  for (int i = threadIdx.x; i < F; i += 128) {
    const float v = row[i], v2 = v * v;
    act[(size_t)t * F + i] = (TX)(r1 * v + r2 * v2 + r3 * (v2 * v) + e);
  }
}

template <typename TX>
__global__ void __launch_bounds__(256) silu_gate_kernel(const float* __restrict__ gu, const float* __restrict__ row_scale,
                                                        const int32_t* __restrict__ row_of, TX* __restrict__ act, int F) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const float sc = row_scale ? row_scale[row_of ? row_of[r] : r] : 1.0f;
  const float* row = gu + (size_t)r * 2 * F;
  for (int i = blockIdx.y * 256 + threadIdx.x; i < F; i += 256 * gridDim.y) {
    const float g = sc * row[i], u = sc * row[F + i];
    act[(size_t)r * F + i] = (TX)(g / (1.0f + expf(-g)) * u);
  }
}

// h[t] += coef * (n(a) ga + n(b) gb) + d1 + sum_k y[slot_k]; then optionally x_next = n(h) * gain_next.  One CTA of NT threads per row
// (steps of few tokens take wide CTAs: a row is then two or three rounds of loads instead of sixteen).
constexpr int BA_MAX_TOP = 16;
template <typename TX, int NT>
__global__ void __launch_bounds__(NT) branch_add_kernel(float* __restrict__ h, const float* __restrict__ a, const float* __restrict__ gain_a,
                                                        const float* __restrict__ b, const float* __restrict__ gain_b, float coef,
                                                        const float* __restrict__ d1, const float* __restrict__ y,
                                                        const int32_t* __restrict__ pair_slot, int top, int W, float eps,
                                                        const float* __restrict__ gain_next, TX* __restrict__ x_next) {
  __shared__ float red[NT / 32];
  __shared__ int slot_s[BA_MAX_TOP];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* ar = a ? a + (size_t)t * W : nullptr;
  const float* br = b ? b + (size_t)t * W : nullptr;
  const float* dr = d1 ? d1 + (size_t)t * W : nullptr;
  float* hr = h + (size_t)t * W;
  if (y != nullptr && (int)threadIdx.x < min(top, BA_MAX_TOP)) slot_s[threadIdx.x] = pair_slot[(size_t)t * top + threadIdx.x];
  float ra = 1.0f, rb = 1.0f;
  {
    float sa = 0.f, sb = 0.f;
    if (ar && gain_a)
      for (int i = threadIdx.x; i < W; i += NT) sa = fmaf(ar[i], ar[i], sa);
    if (br && gain_b)
      for (int i = threadIdx.x; i < W; i += NT) sb = fmaf(br[i], br[i], sb);
    if (ar && gain_a) ra = 1.0f / sqrtf(block_sum_n<NT>(sa, red) / (float)W + eps);
    if (br && gain_b) rb = 1.0f / sqrtf(block_sum_n<NT>(sb, red) / (float)W + eps);
  }
  __syncthreads();
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < W; i += NT) {
    float m = 0.f;
    if (ar) m = ar[i] * ra * (gain_a ? gain_a[i] : 1.0f);
    if (br) m += br[i] * rb * (gain_b ? gain_b[i] : 1.0f);
    m *= coef;
    float ff = dr ? dr[i] : 0.f;
    if (y != nullptr)
      for (int k = 0; k < top; ++k) ff += y[(size_t)(k < BA_MAX_TOP ? slot_s[k] : pair_slot[(size_t)t * top + k]) * W + i];   // choice order
    const float hn = hr[i] + (m + ff);
    hr[i] = hn;
    ss2 = fmaf(hn, hn, ss2);
  }
  if (gain_next != nullptr) {
    const float r2 = 1.0f / sqrtf(block_sum_n<NT>(ss2, red) / (float)W + eps);
    for (int i = threadIdx.x; i < W; i += NT) x_next[(size_t)t * W + i] = (TX)(hr[i] * r2 * gain_next[i]);   // its own writes
  }
}

__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ logits, size_t n, float cap) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) logits[i] = cap * tanhf(logits[i] / cap);
}

// ---- layer norms with gain and bias in front of and behind every sublayer (Tinevik) ----
// (x - mean) / sqrt(variance + eps) * w + b, the variance as the mean of the squared deviations (two passes over a row staged in shared
// memory).  One CTA of 128 threads per row, any width.
template <typename TX>
__global__ void __launch_bounds__(128) layer_norm_kernel(const float* __restrict__ h, const float* __restrict__ w, const float* __restrict__ b,
                                                         TX* __restrict__ x, int W, float eps, const int32_t* __restrict__ rows) {
  extern __shared__ float lrow[];
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float* src = h + (size_t)(rows ? rows[t] : t) * W;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float v = src[i];
    lrow[i] = v;
    s += v;
  }
  const float mean = block_sum_128(s, red) / (float)W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float d = lrow[i] - mean;
    q = fmaf(d, d, q);
  }
  const float r = 1.0f / sqrtf(block_sum_128(q, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 128) x[(size_t)t * W + i] = (TX)((lrow[i] - mean) * r * w[i] + b[i]);
}

// h[t] += ln(y[t]) (gain w, bias b); with pair_slot the sublayer's output is the sum of the token's `top` routed rows times coef,
// y[t] = coef * sum_k y[pair_slot[t * top + k]].  With w_next the norm in front of the next sublayer follows, x_next[t] = ln(h[t]).
template <typename TX>
__global__ void __launch_bounds__(128) layer_norm_add_kernel(float* __restrict__ h, const float* __restrict__ y, const int32_t* __restrict__ pair_slot,
                                                             int top, float coef, const float* __restrict__ w, const float* __restrict__ b, int W,
                                                             float eps, const float* __restrict__ w_next, const float* __restrict__ b_next,
                                                             TX* __restrict__ x_next) {
  extern __shared__ float lrow[];
  __shared__ float red[4];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    float v;
    if (pair_slot != nullptr) {
      v = 0.f;
      for (int k = 0; k < top; ++k) v += y[(size_t)pair_slot[t * top + k] * W + i];
      v *= coef;
    } else {
      v = y[(size_t)t * W + i];
    }
    lrow[i] = v;
    s += v;
  }
  const float mean = block_sum_128(s, red) / (float)W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float d = lrow[i] - mean;
    q = fmaf(d, d, q);
  }
  const float r = 1.0f / sqrtf(block_sum_128(q, red) / (float)W + eps);
  float s2 = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float hn = h[(size_t)t * W + i] + ((lrow[i] - mean) * r * w[i] + b[i]);
    h[(size_t)t * W + i] = hn;
    lrow[i] = hn;   // (each thread re-reads only what it wrote)
    s2 += hn;
  }
  if (w_next == nullptr) return;
  const float mean2 = block_sum_128(s2, red) / (float)W;
  float q2 = 0.f;
  for (int i = threadIdx.x; i < W; i += 128) {
    const float d = lrow[i] - mean2;
    q2 = fmaf(d, d, q2);
  }
  const float r2 = 1.0f / sqrtf(block_sum_128(q2, red) / (float)W + eps);
  for (int i = threadIdx.x; i < W; i += 128) x_next[(size_t)t * W + i] = (TX)((lrow[i] - mean2) * r2 * w_next[i] + b_next[i]);
}

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// act = a(z), a(z) = softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise; pq (device) = p, q
template <typename TX>
__global__ void __launch_bounds__(256) xielu_kernel(const float* __restrict__ z, const float* __restrict__ pq, TX* __restrict__ act, size_t n) {
  pdl_wait();
  pdl_launch_dependents();
  const float ap = softplus_f(pq[0]), an = 0.5f + softplus_f(pq[1]);
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
    const float v = z[i];
    act[i] = (TX)(v > 0.f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v));
  }
}

// out[t][i] = a[t][i] * sigmoid(gate[t * gate_ld + i])
template <typename TX>
__global__ void __launch_bounds__(256) sigmoid_gate_kernel(const float* __restrict__ a, const float* __restrict__ gate, int gate_ld, TX* __restrict__ out,
                                                           int N) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * 256 + threadIdx.x; i < N; i += 256 * gridDim.y)
    out[(size_t)t * N + i] = (TX)(a[(size_t)t * N + i] / (1.0f + expf(-gate[(size_t)t * gate_ld + i])));
}

}  // namespace

constexpr int GN_EARLY_ROWS = 1024;
static dim3 gn_grid(int T, int groups) { return dim3(T, T >= 1024 ? 1 : std::max(1, (groups + 3) / 4)); }

int launch_embed_scaled(const int32_t* ids, const void* table, int table_f32, float scale, float* h, int T, int W, int vocab, cudaStream_t s) {
  if (T <= 0) return 0;
  if (table_f32) B2_CUDA_OK(b2_launch(embed_scaled_kernel<float>, dim3(T), dim3(128), 0, s, ids, (const float*)table, scale, h, W, vocab));
  else B2_CUDA_OK(b2_launch(embed_scaled_kernel<bf16>, dim3(T), dim3(128), 0, s, ids, (const bf16*)table, scale, h, W, vocab));
  return 0;
}

int launch_group_norm(const float* h, const float* gain, void* x, int x_f32, int T, int W, int groups, float eps, const int32_t* rows,
                      cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(groups >= 1 && W % groups == 0, "group_norm: width %d is not %d equal pieces", W, groups);
  if (x_f32)
    B2_CUDA_OK(b2_launch(T < GN_EARLY_ROWS ? group_norm_kernel<float, false, true> : group_norm_kernel<float, false, false>, gn_grid(T, groups), dim3(128), 0, s, h,
                         (const float*)nullptr, gain, (float*)x, (float*)nullptr, W, groups, eps, rows, (const float*)nullptr));
  else
    B2_CUDA_OK(b2_launch(T < GN_EARLY_ROWS ? group_norm_kernel<bf16, false, true> : group_norm_kernel<bf16, false, false>, gn_grid(T, groups), dim3(128), 0, s, h,
                         (const float*)nullptr, gain, (bf16*)x, (float*)nullptr, W, groups, eps, rows, (const float*)nullptr));
  return 0;
}

int launch_group_norm_add(float* h, const float* y, const float* bias, const float* gain, int T, int W, int groups, float eps, cudaStream_t s,
                          const float* gain_next, void* x_next, int x_f32) {
  if (T <= 0) return 0;
  B2_REQUIRE(groups >= 1 && W % groups == 0, "group_norm: width %d is not %d equal pieces", W, groups);
  B2_REQUIRE((gain_next == nullptr) == (x_next == nullptr), "group_norm_add: the following norm needs its gain and its output");
  if (x_f32 || x_next == nullptr)
    B2_CUDA_OK(b2_launch(T < GN_EARLY_ROWS ? group_norm_kernel<float, true, true> : group_norm_kernel<float, true, false>, gn_grid(T, groups), dim3(128), 0, s, y, bias, gain,
                         (float*)x_next, h, W, groups, eps, (const int32_t*)nullptr, gain_next));
  else
    B2_CUDA_OK(b2_launch(T < GN_EARLY_ROWS ? group_norm_kernel<bf16, true, true> : group_norm_kernel<bf16, true, false>, gn_grid(T, groups), dim3(128), 0, s, y, bias, gain,
                         (bf16*)x_next, h, W, groups, eps, (const int32_t*)nullptr, gain_next));
  return 0;
}

int launch_clamped_gate(const float* gu, void* act, int act_f32, int T, int F, float limit, float sharp, cudaStream_t s) {
  if (T <= 0) return 0;
  const dim3 grid(T, T >= 1024 ? 1 : std::max(1, std::min((F + 1023) / 1024, 1024 / T)));   // few tokens: several CTAs per row
  if (act_f32) B2_CUDA_OK(b2_launch(clamped_gate_kernel<float>, grid, dim3(256), 0, s, gu, (float*)act, F, limit, sharp));
  else B2_CUDA_OK(b2_launch(clamped_gate_kernel<bf16>, grid, dim3(256), 0, s, gu, (bf16*)act, F, limit, sharp));
  return 0;
}

int launch_embed_unit_norm(const int32_t* ids, const void* table, int table_f32, const float* gain1p, float* h, int T, int W, int vocab,
                           float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  if (table_f32)
    B2_CUDA_OK(b2_launch(embed_unit_norm_kernel<float>, dim3(T), dim3(128), 0, s, ids, (const float*)table, gain1p, h, W, vocab, eps));
  else
    B2_CUDA_OK(b2_launch(embed_unit_norm_kernel<bf16>, dim3(T), dim3(128), 0, s, ids, (const bf16*)table, gain1p, h, W, vocab, eps));
  return 0;
}

int launch_unit_norm2(const float* h, const float* gain_a, const float* gain_b, void* x1, void* x2, int x_f32, int T, int W, float eps,
                      const int32_t* rows, cudaStream_t s) {
  if (T <= 0) return 0;
  if (x_f32)
    B2_CUDA_OK(b2_launch(unit_norm2_kernel<float>, dim3(T), dim3(128), 0, s, h, gain_a, gain_b, (float*)x1, (float*)x2, W, eps, rows));
  else
    B2_CUDA_OK(b2_launch(unit_norm2_kernel<bf16>, dim3(T), dim3(128), 0, s, h, gain_a, gain_b, (bf16*)x1, (bf16*)x2, W, eps, rows));
  return 0;
}

int launch_logits_finish(const float* logits, int32_t* out_tokens, bf16* logits_bf16, int bf16_rows, int rows, int V, int v_pad, cudaStream_t s) {
  if (rows <= 0) return 0;
  B2_CUDA_OK(b2_launch(logits_finish_kernel, dim3(rows), dim3(1024), 0, s, logits, out_tokens, logits_bf16, bf16_rows, V, v_pad));
  return 0;
}

int launch_store_rows(const float* src, void* x, int x_f32, int ldx, int col0, int T, int W, cudaStream_t s) {
  if (T <= 0) return 0;
  if (x_f32) B2_CUDA_OK(b2_launch(store_rows_kernel<float>, dim3(T), dim3(256), 0, s, src, (float*)x, ldx, col0, W));
  else B2_CUDA_OK(b2_launch(store_rows_kernel<bf16>, dim3(T), dim3(256), 0, s, src, (bf16*)x, ldx, col0, W));
  return 0;
}

int launch_poly_norm(const float* z, const float* coef, void* act, int act_f32, int T, int F, float eps, cudaStream_t s) {
  if (T <= 0) return 0;
  if (act_f32) B2_CUDA_OK(b2_launch(poly_norm_kernel<float>, dim3(T), dim3(128), 0, s, z, coef, (float*)act, F, eps));
  else B2_CUDA_OK(b2_launch(poly_norm_kernel<bf16>, dim3(T), dim3(128), 0, s, z, coef, (bf16*)act, F, eps));
  return 0;
}

int launch_silu_gate(const float* gu, const float* row_scale, const int32_t* row_of, void* act, int act_f32, int rows, int F, cudaStream_t s) {
  if (rows <= 0) return 0;
  const dim3 grid(rows, rows >= 1024 ? 1 : std::max(1, std::min((F + 255) / 256, 1024 / rows)));
  if (act_f32) B2_CUDA_OK(b2_launch(silu_gate_kernel<float>, grid, dim3(256), 0, s, gu, row_scale, row_of, (float*)act, F));
  else B2_CUDA_OK(b2_launch(silu_gate_kernel<bf16>, grid, dim3(256), 0, s, gu, row_scale, row_of, (bf16*)act, F));
  return 0;
}

int launch_branch_add(float* h, const float* a, const float* gain_a, const float* b, const float* gain_b, float coef, const float* d1,
                      const float* y, const int32_t* pair_slot, int top, int T, int W, float eps, cudaStream_t s, const float* gain_next,
                      void* x_next, int x_f32) {
  if (T <= 0) return 0;
  B2_REQUIRE((gain_next == nullptr) == (x_next == nullptr), "branch_add: the following norm needs its gain and its output");
  B2_REQUIRE(y == nullptr || (pair_slot != nullptr && top >= 1), "branch_add: routed rows need their slots");
  const bool wide = T < 1024 && W >= 1024;
  if (x_f32 || x_next == nullptr) {
    if (wide) B2_CUDA_OK(b2_launch(branch_add_kernel<float, 512>, dim3(T), dim3(512), 0, s, h, a, gain_a, b, gain_b, coef, d1, y, pair_slot, top, W, eps, gain_next, (float*)x_next));
    else B2_CUDA_OK(b2_launch(branch_add_kernel<float, 128>, dim3(T), dim3(128), 0, s, h, a, gain_a, b, gain_b, coef, d1, y, pair_slot, top, W, eps, gain_next, (float*)x_next));
  } else {
    if (wide) B2_CUDA_OK(b2_launch(branch_add_kernel<bf16, 512>, dim3(T), dim3(512), 0, s, h, a, gain_a, b, gain_b, coef, d1, y, pair_slot, top, W, eps, gain_next, (bf16*)x_next));
    else B2_CUDA_OK(b2_launch(branch_add_kernel<bf16, 128>, dim3(T), dim3(128), 0, s, h, a, gain_a, b, gain_b, coef, d1, y, pair_slot, top, W, eps, gain_next, (bf16*)x_next));
  }
  return 0;
}

int launch_softcap(float* logits, size_t n, float cap, cudaStream_t s) {
  if (n == 0 || !(cap > 0.f)) return 0;
  const unsigned blocks = (unsigned)std::min<size_t>((n + 255) / 256, 4096);
  B2_CUDA_OK(b2_launch(softcap_kernel, dim3(blocks), dim3(256), 0, s, logits, n, cap));
  return 0;
}

int launch_layer_norm(const float* h, const float* w, const float* b, void* x, int x_f32, int T, int W, float eps, const int32_t* rows, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE((size_t)W * 4 <= 160 * 1024, "layer_norm: a row of %d numbers does not fit in shared memory", W);
  const size_t smem = (size_t)W * 4;
  if (x_f32) {
    static B2PerDeviceOnce once;
    if (smem > 48 * 1024) b2_prefer_max_smem(layer_norm_kernel<float>, once);
    B2_CUDA_OK(b2_launch(layer_norm_kernel<float>, dim3(T), dim3(128), smem, s, h, w, b, (float*)x, W, eps, rows));
  } else {
    static B2PerDeviceOnce once;
    if (smem > 48 * 1024) b2_prefer_max_smem(layer_norm_kernel<bf16>, once);
    B2_CUDA_OK(b2_launch(layer_norm_kernel<bf16>, dim3(T), dim3(128), smem, s, h, w, b, (bf16*)x, W, eps, rows));
  }
  return 0;
}

int launch_layer_norm_add(float* h, const float* y, const int32_t* pair_slot, int top, float coef, const float* w, const float* b, int T, int W, float eps,
                          cudaStream_t s, const float* w_next, const float* b_next, void* x_next, int x_f32) {
  if (T <= 0) return 0;
  B2_REQUIRE((size_t)W * 4 <= 160 * 1024, "layer_norm_add: a row of %d numbers does not fit in shared memory", W);
  B2_REQUIRE((w_next == nullptr) == (x_next == nullptr) && (w_next == nullptr) == (b_next == nullptr), "layer_norm_add: the following norm needs gain, bias and output");
  const size_t smem = (size_t)W * 4;
  if (x_f32 || x_next == nullptr) {
    static B2PerDeviceOnce once;
    if (smem > 48 * 1024) b2_prefer_max_smem(layer_norm_add_kernel<float>, once);
    B2_CUDA_OK(b2_launch(layer_norm_add_kernel<float>, dim3(T), dim3(128), smem, s, h, y, pair_slot, top, coef, w, b, W, eps, w_next, b_next, (float*)x_next));
  } else {
    static B2PerDeviceOnce once;
    if (smem > 48 * 1024) b2_prefer_max_smem(layer_norm_add_kernel<bf16>, once);
    B2_CUDA_OK(b2_launch(layer_norm_add_kernel<bf16>, dim3(T), dim3(128), smem, s, h, y, pair_slot, top, coef, w, b, W, eps, w_next, b_next, (bf16*)x_next));
  }
  return 0;
}

int launch_xielu(const float* z, const float* pq, void* act, int act_f32, size_t n, cudaStream_t s) {
  if (n == 0) return 0;
  const int blocks = (int)std::min<size_t>((n + 255) / 256, 148 * 16);
  if (act_f32) B2_CUDA_OK(b2_launch(xielu_kernel<float>, dim3(blocks), dim3(256), 0, s, z, pq, (float*)act, n));
  else B2_CUDA_OK(b2_launch(xielu_kernel<bf16>, dim3(blocks), dim3(256), 0, s, z, pq, (bf16*)act, n));
  return 0;
}

int launch_sigmoid_gate(const float* a, const float* gate, int gate_ld, void* out, int out_f32, int T, int N, cudaStream_t s) {
  if (T <= 0) return 0;
  const dim3 grid(T, T >= 1024 ? 1 : std::max(1, std::min((N + 255) / 256, 1024 / T)));
  if (out_f32) B2_CUDA_OK(b2_launch(sigmoid_gate_kernel<float>, grid, dim3(256), 0, s, a, gate, gate_ld, (float*)out, N));
  else B2_CUDA_OK(b2_launch(sigmoid_gate_kernel<bf16>, grid, dim3(256), 0, s, a, gate, gate_ld, (bf16*)out, N));
  return 0;
}

}  // namespace b2
