// moe_route.cu -- the router of a routed-experts feed-forward, and the bookkeeping that turns its choices into ragged
// groups for gemm_any.cu.
//
// Router (all fp32): z = R x, s = sigmoid(z).  The CHOICE uses s + correction (a per-expert offset that steers load and
// may make a choice score negative); the mixing WEIGHTS use s alone.  Experts are `groups` equal runs of neighbours; a
// group's score is the sum of its two best choice scores and only the `keep` best groups may supply experts (the others
// are out, not zero).  Of the allowed experts the `top` with the best choice scores are taken; their s, divided by their
// sum (+ 1e-20), are the weights.  Ties go to the lower index.
//
// route_permute is a counting sort of the (token, choice) pairs by expert: slots of expert e are [offsets[e], offsets[e+1]).
// Which slot of its expert a pair gets depends on the order of atomic arrivals, and that is harmless: gemm_any.cu sums every
// output row on its own, so a row's result does not depend on its slot or on its tile mates -- nor, therefore, on the other
// requests of the batch.  route_combine adds the weighted expert outputs (and the mixer branch) onto the fp32 residual
// stream in choice order.
#include "kernels.h"

namespace b2 {

namespace {

constexpr int RT_WARPS = 16;

// one CTA per token: the row is staged once as fp32, warp w takes experts w, w + 16, ...; thread 0 then selects
template <typename TX>
__global__ void __launch_bounds__(RT_WARPS * 32) route_kernel(const TX* __restrict__ x, const float* __restrict__ router,
                                                              const float* __restrict__ correction, RouteGeom g, int32_t* __restrict__ idx,
                                                              float* __restrict__ weight, int T, int W) {
  extern __shared__ __align__(16) float sm[];  // x row [W rounded up to 4] (read as float4), s [E], choice [E]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int E = g.experts;
  float* xs = sm;
  float* s = xs + ((W + 3) & ~3);
  float* ch = s + E;
  const TX* xr = x + (size_t)t * W;
  for (int i = threadIdx.x; i < W; i += RT_WARPS * 32) xs[i] = (float)xr[i];
  __syncthreads();
  const bool vec = (W % 4 == 0);
  for (int e = warp; e < E; e += RT_WARPS) {
    const float* rr = router + (size_t)e * W;
    float acc = 0.f;
    if (vec) {
#pragma unroll 8
      for (int i = lane * 4; i < W; i += 128) {
        const float4 r4 = *reinterpret_cast<const float4*>(rr + i);
        const float4 x4 = *reinterpret_cast<const float4*>(xs + i);
        acc = fmaf(x4.x, r4.x, acc); acc = fmaf(x4.y, r4.y, acc); acc = fmaf(x4.z, r4.z, acc); acc = fmaf(x4.w, r4.w, acc);
      }
    } else {
      for (int i = lane; i < W; i += 32) acc = fmaf(xs[i], rr[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const float sg = 1.0f / (1.0f + expf(-acc));
      s[e] = sg;
      ch[e] = sg + (correction ? correction[e] : 0.f);
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  // groups: score = sum of the two best choice scores; all but the `keep` best are out (choice = -inf).  Ranks are formed
  // from the untouched scores first (a 64-bit mask remembers who is out), then applied.
  const int per = E / g.groups;
  if (g.keep < g.groups) {
    auto group_score = [&](int gi) {
      float b1 = -INFINITY, b2 = -INFINITY;
      for (int e = gi * per; e < (gi + 1) * per; ++e) {
        const float v = ch[e];
        if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
      }
      return per >= 2 ? b1 + b2 : b1;
    };
    unsigned long long out_mask = 0ull;
    for (int gi = 0; gi < g.groups; ++gi) {
      const float my = group_score(gi);
      int beat = 0;  // groups ranked ahead of gi (lower index wins a tie)
      for (int gj = 0; gj < g.groups; ++gj) {
        if (gj == gi) continue;
        const float other = group_score(gj);
        if (other > my || (other == my && gj < gi)) ++beat;
      }
      if (beat >= g.keep) out_mask |= 1ull << gi;
    }
    for (int gi = 0; gi < g.groups; ++gi)
      if ((out_mask >> gi) & 1ull)
        for (int e = gi * per; e < (gi + 1) * per; ++e) ch[e] = -INFINITY;
  }
  float sum = 0.f;
  for (int k = 0; k < g.top; ++k) {
    int best = -1;
    float bv = -INFINITY;
    for (int e = 0; e < E; ++e)
      if (ch[e] > bv) { best = e; bv = ch[e]; }   // -inf = out or already taken; first index wins a tie
    if (best < 0) best = k < E ? k : 0;  // only for rows that hold no numbers (padding rows of a graph bucket): keep the index valid
    idx[(size_t)t * g.top + k] = best;
    weight[(size_t)t * g.top + k] = s[best];
    sum += s[best];
    ch[best] = -INFINITY;
  }
  if (g.raw_weights) return;   // the scores as they are
  const float inv = 1.0f / (sum + 1e-20f);
  for (int k = 0; k < g.top; ++k) weight[(size_t)t * g.top + k] *= inv;
}

// the permutation in three steps: histogram (any number of CTAs), scan (one thread; experts are few), placement
__global__ void __launch_bounds__(256) route_count_kernel(const int32_t* __restrict__ idx, int npairs, int E, int* __restrict__ counts) {
  extern __shared__ int hist[];
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += 256) hist[e] = 0;
  __syncthreads();
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p < npairs) atomicAdd(&hist[idx[p]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += 256)
    if (hist[e]) atomicAdd(&counts[e], hist[e]);
}
__global__ void route_scan_kernel(int* __restrict__ counts, int E, int32_t* __restrict__ offsets, int* __restrict__ cursor) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x != 0) return;
  int run = 0;
  for (int e = 0; e < E; ++e) {
    offsets[e] = run;
    cursor[e] = run;
    run += counts[e];
    counts[e] = 0;  // ready for the next call
  }
  offsets[E] = run;
}
__global__ void __launch_bounds__(256) route_place_kernel(const int32_t* __restrict__ idx, int npairs, int top, int* __restrict__ cursor,
                                                          int32_t* __restrict__ slot_token, int32_t* __restrict__ pair_slot) {
  pdl_wait();
  pdl_launch_dependents();
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p >= npairs) return;
  const int slot = atomicAdd(&cursor[idx[p]], 1);
  slot_token[slot] = p / top;
  pair_slot[p] = slot;
}

// few pairs (a decode step): the three steps in one CTA, histogram and cursors in shared memory
__global__ void __launch_bounds__(1024) route_permute_small_kernel(const int32_t* __restrict__ idx, int npairs, int top, int E,
                                                                   int32_t* __restrict__ offsets, int32_t* __restrict__ slot_token,
                                                                   int32_t* __restrict__ pair_slot) {
  extern __shared__ int cur[];  // [E]
  pdl_wait();
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += 1024) cur[e] = 0;
  __syncthreads();
  const int p = threadIdx.x;
  const int mine = p < npairs ? idx[p] : -1;
  if (mine >= 0) atomicAdd(&cur[mine], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cur[e];
      offsets[e] = run;
      cur[e] = run;
      run += c;
    }
    offsets[E] = run;
  }
  __syncthreads();
  if (mine >= 0) {
    const int slot = atomicAdd(&cur[mine], 1);
    slot_token[slot] = p / top;
    pair_slot[p] = slot;
  }
}

constexpr int COMBINE_MAX_TOP = 16;   // choices staged in shared memory; wider routers read them from global memory
__global__ void __launch_bounds__(256) route_combine_kernel(float* __restrict__ h, const float* __restrict__ mix, const float* __restrict__ y,
                                                            const float* __restrict__ weight, const int32_t* __restrict__ pair_slot, int W,
                                                            int top) {
  __shared__ float w_s[COMBINE_MAX_TOP];
  __shared__ int slot_s[COMBINE_MAX_TOP];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const bool staged = top <= COMBINE_MAX_TOP;
  if (staged && (int)threadIdx.x < top) {
    w_s[threadIdx.x] = weight[(size_t)t * top + threadIdx.x];
    slot_s[threadIdx.x] = pair_slot[(size_t)t * top + threadIdx.x];
  }
  __syncthreads();
  if (staged && W % 4 == 0) {   // (rows of h, mix and y start on 16-byte boundaries: W * 4 bytes apart from aligned bases)
    float4* hr = reinterpret_cast<float4*>(h + (size_t)t * W);
    const float4* mr = mix != nullptr ? reinterpret_cast<const float4*>(mix + (size_t)t * W) : nullptr;
    for (int i = threadIdx.x; i < W / 4; i += 256) {
      float4 acc = mr != nullptr ? mr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int k = 0; k < top; ++k) {   // choice order
        const float4 v = reinterpret_cast<const float4*>(y + (size_t)slot_s[k] * W)[i];
        const float w = w_s[k];
        acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y); acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
      }
      float4 o = hr[i];
      o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
      hr[i] = o;
    }
    return;
  }
  for (int i = threadIdx.x; i < W; i += 256) {
    float acc = mix != nullptr ? mix[(size_t)t * W + i] : 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weight[(size_t)t * top + k], y[(size_t)pair_slot[(size_t)t * top + k] * W + i], acc);
    h[(size_t)t * W + i] += acc;
  }
}

// slot_weight[pair_slot[p]] = weight[p]: the pairs' weights in expert (slot) order, for experts whose INPUT the weight multiplies
__global__ void __launch_bounds__(256) route_slot_weights_kernel(const float* __restrict__ weight, const int32_t* __restrict__ pair_slot,
                                                                 float* __restrict__ slot_weight, int npairs) {
  pdl_wait();
  pdl_launch_dependents();
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p < npairs) slot_weight[pair_slot[p]] = weight[p];
}

// No router: a table row per token id names the token's experts, each weighted 1 / top.  idx [T][top], weight [T][top].
__global__ void __launch_bounds__(256) route_table_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ table, int vocab, int experts,
                                                          int top, int32_t* __restrict__ idx, float* __restrict__ weight, int npairs) {
  pdl_wait();
  pdl_launch_dependents();
  const int p = blockIdx.x * 256 + threadIdx.x;
  if (p >= npairs) return;
  const int t = p / top, k = p - t * top;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  int x = table[(size_t)id * top + k];
  x = x < 0 ? 0 : (x >= experts ? experts - 1 : x);
  idx[p] = x;
  weight[p] = 1.0f / (float)top;
}

// act = bf16(max(up, 0)^2): the experts' activation between the two dense products of a prompt-sized step
__global__ void __launch_bounds__(256) relu2_round_kernel(const float4* __restrict__ up, uint2* __restrict__ act, size_t n4) {
  pdl_wait();
  pdl_launch_dependents();
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
    const float4 v = up[i];
    const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a * a, b * b), hi = __floats2bfloat162_rn(c * c, d * d);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    act[i] = o;
  }
}

}  // namespace

int launch_relu2_round(const float* up, bf16* act, size_t n, cudaStream_t s) {
  if (n == 0) return 0;
  if (n % 4 != 0) return -22;   // (rows are multiples of 64 wide on this path)
  const size_t n4 = n / 4;
  const int grid = (int)std::min<size_t>((n4 + 255) / 256, 148 * 16);
  B2_CUDA_OK(b2_launch(relu2_round_kernel, dim3(grid), dim3(256), 0, s, (const float4*)up, (uint2*)act, n4));
  return 0;
}

int launch_route(const void* x, int x_f32, const float* router, const float* correction, const RouteGeom& g, int32_t* idx, float* weight,
                 int T, int W, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(g.experts >= 1 && g.groups >= 1 && g.groups <= 64 && g.experts % g.groups == 0, "route: %d experts do not form %d equal groups", g.experts, g.groups);
  B2_REQUIRE(g.keep >= 1 && g.keep <= g.groups, "route: keep %d outside [1, %d]", g.keep, g.groups);
  B2_REQUIRE(g.top >= 1 && g.top <= g.keep * (g.experts / g.groups), "route: top %d exceeds the %d experts of the kept groups", g.top,
             g.keep * (g.experts / g.groups));
  const size_t smem = ((size_t)2 * g.experts + ((W + 3) & ~3)) * sizeof(float);
  B2_REQUIRE(smem <= 48 * 1024, "route: %d experts and width %d need %zu bytes of shared memory", g.experts, W, smem);
  const dim3 grid(T);
  if (x_f32)
    B2_CUDA_OK(b2_launch(route_kernel<float>, grid, dim3(RT_WARPS * 32), smem, s, (const float*)x, router, correction, g, idx, weight, T, W));
  else
    B2_CUDA_OK(b2_launch(route_kernel<bf16>, grid, dim3(RT_WARPS * 32), smem, s, (const bf16*)x, router, correction, g, idx, weight, T, W));
  return 0;
}

int launch_route_permute(const int32_t* idx, int T, int top, int experts, int32_t* offsets, int stride, int32_t* slot_token,
                         int32_t* pair_slot, cudaStream_t s) {
  if (T <= 0) return 0;
  B2_REQUIRE(stride >= experts + 1, "route_permute: stride %d < experts + 1", stride);
  int* counts = offsets + stride;   // zero between calls (the scan step clears what the histogram added)
  int* cursor = counts + stride;
  const int npairs = T * top;
  B2_REQUIRE((size_t)experts * sizeof(int) <= 48 * 1024, "route_permute: %d experts", experts);
  if (npairs <= 1024) {
    B2_CUDA_OK(b2_launch(route_permute_small_kernel, dim3(1), dim3(1024), (size_t)experts * sizeof(int), s, idx, npairs, top, experts, offsets,
                         slot_token, pair_slot));
    return 0;
  }
  B2_CUDA_OK(b2_launch(route_count_kernel, dim3((npairs + 255) / 256), dim3(256), (size_t)experts * sizeof(int), s, idx, npairs, experts, counts));
  B2_CUDA_OK(b2_launch(route_scan_kernel, dim3(1), dim3(32), 0, s, counts, experts, offsets, cursor));
  B2_CUDA_OK(b2_launch(route_place_kernel, dim3((npairs + 255) / 256), dim3(256), 0, s, idx, npairs, top, cursor, slot_token, pair_slot));
  return 0;
}

int launch_route_table(const int32_t* ids, const int32_t* table, int vocab, int experts, int top, int32_t* idx, float* weight, int T, cudaStream_t s) {
  if (T <= 0) return 0;
  const int npairs = T * top;
  B2_CUDA_OK(b2_launch(route_table_kernel, dim3((npairs + 255) / 256), dim3(256), 0, s, ids, table, vocab, experts, top, idx, weight, npairs));
  return 0;
}

int launch_route_slot_weights(const float* weight, const int32_t* pair_slot, float* slot_weight, int npairs, cudaStream_t s) {
  if (npairs <= 0) return 0;
  B2_CUDA_OK(b2_launch(route_slot_weights_kernel, dim3((npairs + 255) / 256), dim3(256), 0, s, weight, pair_slot, slot_weight, npairs));
  return 0;
}

int launch_route_combine(float* h, const float* mix, const float* y, const float* weight, const int32_t* pair_slot, int T, int W, int top,
                         cudaStream_t s) {
  if (T <= 0) return 0;
  B2_CUDA_OK(b2_launch(route_combine_kernel, dim3(T), dim3(256), 0, s, h, mix, y, weight, pair_slot, W, top));
  return 0;
}

}  // namespace b2
