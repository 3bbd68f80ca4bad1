// kernels.h -- internal C++ launch API of the sm_100a kernels (engine.cu and capi.cu call these).
#pragma once
#include "../../include/b2_engine.h"
#include "common.cuh"

namespace b2 {

// step timeline (common.cuh): one setter per .cu file that holds kernels of the decode path
int step_trace_set_elementwise(unsigned long long* dev_buf);
int step_trace_set_gemm(unsigned long long* dev_buf);
int step_trace_set_attn(unsigned long long* dev_buf);

// An activation operand that is either bf16 [T][N] or fp32 split-K partials [nsplit][T][N]
// (summed in split order, then rounded to bf16 -- the rounding point of HF's nn.Linear).
struct ActIn {
  const void* ptr;
  int is_f32;
  int nsplit;
};
inline ActIn act_bf16(const void* p) { return ActIn{p, 0, 1}; }
inline ActIn act_f32(const void* p, int nsplit) { return ActIn{p, 1, nsplit}; }

// ---- elementwise.cu ----
int launch_embed(const int32_t* ids, const bf16* table, bf16* h, int T, int H, int vocab, unsigned long long* zero_buf, int nzero,
                 cudaStream_t s);
int launch_add_rmsnorm(bf16* h, ActIn delta, const bf16* w, bf16* x, int T, int H, float eps, cudaStream_t s, int tag = 0);
// tag: lane marker for the step timeline (common.cuh), no effect on the result
int launch_qknorm_rope_kv(ActIn qkv, const bf16* qw, const bf16* kw, const bf16* cos_sin, const int32_t* positions,
                          const int32_t* slots, bf16* q_out, bf16* k_pages, bf16* v_pages, int T, int nq, int nkv,
                          int hd, int block_size, float eps, cudaStream_t s, int rotary_dim = 128, const bf16* bias = nullptr,
                          float q_mul = 1.0f, int tag = 0);
// qw == kw == nullptr: no QK-norm (Phi-3).  rotary_dim: width of the rotated prefix of each head; heads narrower
// than 128 are stored zero-padded to 128 (see engine.cu, "internal geometry").  bias [(nq + 2 nkv) * 128]: added to the
// fp32 partials before the rounding; q_mul: the query is multiplied by it afterwards (OPT pre-scales q).

// ---- elementwise_opt.cu (OPT variant) ----
int launch_embed_pos(const int32_t* ids, const int32_t* positions, const bf16* table, const bf16* pos_table, bf16* h, int T, int H,
                     int vocab, int pos_rows, unsigned long long* zero_buf, int nzero, cudaStream_t s);
int launch_add_layernorm(bf16* h, ActIn delta, const bf16* delta_bias, const bf16* w, const bf16* b, bf16* x, int T, int H, float eps,
                         cudaStream_t s);
int launch_bias_relu(ActIn fc1, const bf16* bias, bf16* act, int T, int I, cudaStream_t s);
int launch_silu_mul(ActIn gu, bf16* act, int T, int I, cudaStream_t s, int tag = 0);
int launch_gather_rows(const bf16* src, const int32_t* rows, bf16* dst, int n, int H, cudaStream_t s);
int launch_argmax_rows(const bf16* logits, int32_t* out, int T, int V, cudaStream_t s);
int launch_argmax_finalize(const unsigned long long* packed, int32_t* out, int T, cudaStream_t s);
// decode bookkeeping on the device: positions/seq_lens += 1, slots from the block table, and
// the tokens produced by the previous step become this step's input ids.
int launch_decode_advance(int32_t* positions, int32_t* seq_lens, int32_t* slots, const int32_t* block_table,
                          int bt_stride, int block_size, int B, int32_t* frac_q16, long long l2_budget_bytes,
                          long long bytes_per_page_all_heads, cudaStream_t s);
int launch_logits_to_f32(const bf16* in, float* out, size_t n, cudaStream_t s);

// ---- gemm_simt.cu ----
// out = x[T][K] . w[N][K]^T ; bf16 out [T][N] or fp32 [T][N] (single split).
int launch_linear_simt(const bf16* x, const bf16* w, void* out, int out_is_f32, int T, int N, int K, cudaStream_t s);

// Ride-along L2 prefetch of the next attention pass's K/V pages.  The projection kernels are
// latency-bound and leave HBM idle, and B200's L2 (126 MB) holds a good part of one layer's pages,
// so each projection asks the TMA engine to pull a share of them into L2 while it waits for its own
// operands (cp.async.bulk.prefetch.L2; no SM resources, no completion to wait for).
struct KvPrefetch {
  const bf16* k_pages = nullptr;   // target layer's pools (null = no prefetch)
  const bf16* v_pages = nullptr;
  const int32_t* block_table = nullptr;
  const int32_t* seq_lens = nullptr;
  const int32_t* frac_q16 = nullptr;  // device: share of every sequence's pages to pull, in 1/65536
  int bt_stride = 0, B = 0, nkv = 0;
  int part = 0, nparts = 1;           // this launch takes items with (index % nparts == part)
};

// ---- gemm_tc.cu ----
enum TcEpilogue { TC_EPI_BF16 = 0, TC_EPI_F32_PARTIAL = 1, TC_EPI_ARGMAX = 2, TC_EPI_ARGMAX_ROWS = 3 };
struct TcGemmArgs {
  CUtensorMap tmap_w;  // W [N][K], box 64 x 128   (TC_EPI_ARGMAX_ROWS: the operands trade places -- this is X, box 64 x 128)
  CUtensorMap tmap_x;  // X [>=T rows][K], box 64 x bn  (TC_EPI_ARGMAX_ROWS: W [N][K], box 64 x bn)
  int bn;              // token tile: 16, 32, 64, 128 or 256
  int T, N, K;
  int nsplit;          // split-K factor (EPI_F32_PARTIAL when > 1)
  int epilogue;
  void* out;           // bf16 [T][N] | fp32 [nsplit][T][N] | bf16 logits (may be null) for ARGMAX
  unsigned long long* argmax_packed;  // [T] for TC_EPI_ARGMAX (must be zeroed before launch)
  KvPrefetch prefetch;                // optional ride-along K/V prefetch
  int small_smem = 0;                 // F32_PARTIAL, bn <= 64: short stage ring so the CTA fits beside a decode-attention CTA
  int x_row0 = 0;                     // first row of X (tmap_x) this launch reads: a micro-batch of a larger buffer
  const void* resid = nullptr;        // TC_EPI_BF16, bn >= 32: out = bf16(resid[T][N] + bf16(x . W^T)); may be `out` itself (in-place residual add)
  const void* x_raw = nullptr;        // X rows [0, T) as a plain pointer (row stride K), ALREADY offset to the launch's first row:
                                      // lets decode-sized launches fetch X with cp.async instead of the tensor map (gemm_tc.cu, XCP)
};
int launch_linear_tc(const TcGemmArgs& a, cudaStream_t s);
int tc_pick_bn(int T);
int tc_set_trace(unsigned long long* dev_buf);  // diagnostics: per-CTA phase timestamps (null = off)
// choose a split-K factor so that tiles * splits fills the SMs (each split gets >= 1 k-block)
int tc_pick_nsplit(int T, int N, int K, int num_sms);

// ---- gemm_pair.cu: a projection and the element-wise kernel behind it in one launch (clusters of two CTAs split K and
//      exchange accumulator halves through distributed shared memory); at most 64 tokens, K <= 1024 ----
bool pair_shapes_ok(int T, int K);
// gemm_mc.cu: prefill-sized bf16 projection, two CTAs per cluster share the token tile through TMA multicast
bool linear_mc_shapes_ok(int T, int N, int K);
int launch_linear_mc(const CUtensorMap& tm_w, const CUtensorMap& tm_x128, bf16* out, int T, int N, int K, int x_row0, cudaStream_t s);
int launch_qkv_rope_prefill(const CUtensorMap& tm_qkv, const CUtensorMap& tm_x128, const bf16* qw, const bf16* kw, const bf16* cos_sin,
                            const int32_t* positions, const int32_t* slots, bf16* q_out, bf16* k_pages, bf16* v_pages, int T, int nq, int nkv,
                            int K, int block_size, float eps, int x_row0, cudaStream_t s);
// gemm_gateup.cu: the prefill-sized counterpart (two accumulators per tile, SwiGLU in the epilogue)
bool gateup_prefill_shapes_ok(int T, int I, int K);
int launch_gateup_swiglu_prefill(const CUtensorMap& tm_w, const CUtensorMap& tm_x128, bf16* act, int T, int I, int K, int x_row0, cudaStream_t s);
// Normalise-on-load (see gemm_pair.cu): x is the residual stream, ssq [pieces][ld] the per-16-feature sums of squares of
// its rows (gemm_resid.cu writes them), gain the RMSNorm weight.  Default: x is used as given.
struct PairNorm {
  const float* ssq = nullptr;
  const bf16* gain = nullptr;
  int pieces = 0, ld = 0;
  float eps = 0.f;
  L2Prefetch next_w;  // optional: the next projection's weights, prefetched into L2 by this launch's idle lanes
};
int launch_gateup_swiglu(const CUtensorMap& tm_gu64, const bf16* x, bf16* act, int T, int I, int K, cudaStream_t s, int tag = 0,
                         const PairNorm& norm = PairNorm());
// gemm_resid.cu: h += x . W^T for the residual stream (O / down projection), split-K summed inside a cluster of 8;
// also writes the pieces of the next RMSNorm's statistic
bool resid_shapes_ok(int T, int N, int K);
int launch_linear_resid(const CUtensorMap& tm_w, const bf16* x, bf16* h, float* ssq, int T, int N, int K, int ssq_ld, cudaStream_t s, int tag = 0,
                        const L2Prefetch& next_w = L2Prefetch());
int step_trace_set_resid(unsigned long long* buf);
int launch_qkv_rope(const CUtensorMap& tm_qkv, const bf16* x, const bf16* qw, const bf16* kw, const bf16* cos_sin, const int32_t* positions,
                    const int32_t* slots, bf16* q_out, bf16* k_pages, bf16* v_pages, int T, int nq, int nkv, int K, int block_size,
                    float eps, cudaStream_t s, int tag = 0, const PairNorm& norm = PairNorm());
int step_trace_set_pair(unsigned long long* dev_buf);

// ---- chain.cu ----
// The eight dependent steps between two decode-attention passes as one persistent kernel
// (step numbers: 0 O-proj, 1 add+norm, 2 gate-up, 3 SwiGLU, 4 down, 5 add+norm, 6 QKV, 7 QK-norm/RoPE/KV).
struct ChainGemm {
  int N, K, nsplit, kps;  // kps = k-blocks (64 wide) per split
};
struct ChainParams {
  int T, bn, phase_begin, phase_end;  // runs steps [phase_begin, phase_end)
  ChainGemm g[4];                     // O, gate-up, down, QKV(next layer)
  float* partial;                     // split-K partials, reused by every GEMM step
  bf16 *h, *x, *act, *qrot;
  const bf16 *norm_w_a, *norm_w_b;    // gains of step 1 / step 5
  int norm_b_has_delta;               // 0: step 5 only normalises h (first call of a forward, after the embedding)
  const bf16 *qw, *kw, *cos_sin;
  const int32_t *positions, *slots;
  bf16 *k_pages, *v_pages;            // pools of the layer whose QKV step 6 computes
  int H, I, nq, nkv, block_size;
  float eps;
  unsigned long long* gbar;           // grid barrier arrival counter, zero before the first launch; every launch
                                      // that shares it must use the same grid size
};
int chain_set_trace(unsigned long long* dev_buf);  // diagnostics (null = off)
int launch_decode_chain(const CUtensorMap* w_maps4, const CUtensorMap* x_maps4, const ChainParams& p, cudaStream_t s);

// ---- chain_cluster.cu: the chain in four fused steps (0 O + residual, 1 RMSNorm + gate-up + SwiGLU,
//      2 down + residual, 3 RMSNorm + QKV of the next layer + QK-norm/RoPE/KV write) ----
struct FusedChainParams {
  int T, phase_begin, phase_end;      // runs steps [phase_begin, phase_end)
  bf16 *h, *act, *qrot;
  const bf16 *norm_w_a, *norm_w_b;    // gains folded into step 1 (post-attention norm) / step 3 (next layer's input norm)
  const bf16 *qw, *kw, *cos_sin;
  const int32_t *positions, *slots;
  bf16 *k_pages, *v_pages;            // pools of the layer whose QKV step 3 computes
  float *ss_a, *ss_b;                 // [32 slices][64 tokens] sums of squares left by step 0 / step 2
  int H, I, nq, nkv, block_size;
  float eps;
  unsigned long long* gbar;           // grid barrier arrival counter (its own: 128 CTAs)
};
int fused_chain_supported(int H, int I, int nq, int nkv, int hd, int T, int block_size);
int fused_chain_max_clusters();
int fused_chain_set_trace(unsigned long long* dev_buf);
// w_maps4: Wo (box 64x32), Wgu (64x96), Wd (64x32), Wqkv of the next layer (64x128); a_maps2: attention output, SwiGLU
// output (box 64x64)
int launch_decode_fused_chain(const CUtensorMap* w_maps4, const CUtensorMap* a_maps2, const FusedChainParams& p, cudaStream_t s);

// ---- attn_decode.cu ----
// KV page-slice layout ([16 tokens][128 dims] bf16 = 4 KB per (page, kv head)): the 16-byte chunk c
// (8 dims) of token row r is stored at chunk position c ^ (r & 7).  Every kernel that touches the
// pages goes through this one function.
__host__ __device__ inline int kv_swizzled_chunk(int row_in_page, int chunk) { return chunk ^ (row_in_page & 7); }
size_t attn_decode_scratch_floats(int B, int nq, int nkv, int hd);
// scratch counters must be zero at launch (attn_decode_zero_counters once; the kernel re-zeroes them)
int attn_decode_zero_counters(float* scratch, cudaStream_t s);
int launch_attn_decode(const bf16* q, const bf16* k_pages, const bf16* v_pages, const int32_t* block_table,
                       int bt_stride, const int32_t* seq_lens, float* scratch, bf16* out, int B, int nq, int nkv,
                       int hd, int block_size, cudaStream_t s, float softmax_scale = 0.f, int window = 0, int tag = 0);
// softmax_scale 0 = hd^-0.5; a padded head passes the scale of its real width.  window > 0: sliding-window attention,
// each query sees its last `window` keys (itself included).

// ---- attn_prefill.cu ----
struct PrefillTile {  // one 64-query tile of one sequence
  int32_t q_row0;     // first token row of the tile in the batch
  int32_t q_pos0;     // position of that token in its sequence
  int32_t nrows;      // valid rows (<= 64)
  int32_t bt_row;     // row of the sequence in the block table
};
int launch_attn_prefill(const bf16* q, const bf16* k_pages, const bf16* v_pages, const int32_t* block_table,
                        int bt_stride, const PrefillTile* tiles_dev, int ntiles, bf16* out, int nq, int nkv, int hd,
                        int block_size, cudaStream_t s, float softmax_scale = 0.f, int window = 0);

// ---- attn_prefill_tc.cu: the same pass on tcgen05 (S and P.V in TMEM, K/V pages through TMA); num_pages = size of the pool ----
int launch_attn_prefill_tc(const bf16* q, const bf16* k_pages, const bf16* v_pages, int64_t num_pages, const int32_t* block_table,
                           int bt_stride, const PrefillTile* tiles_dev, int ntiles, bf16* out, int nq, int nkv, int hd, int block_size,
                           cudaStream_t s, float softmax_scale = 0.f, int window = 0, int pair_mode = 0);

// ---- sampling.cu ----
struct SampleRow {  // one row to draw from (temperature <= 0: greedy arg-max, lowest index on ties)
  int row;
  float temperature;
  int top_k;
  float top_p;
  unsigned long long seed;
};
int launch_sample_rows(const bf16* logits, const SampleRow* rows_host, SampleRow* stage_dev, int32_t* out, int nrows, int V, uint64_t step,
                       cudaStream_t s);

int device_num_sms();

// ---- gemm_any.cu: C = A . W^T for any shape, bf16 or fp32 operands, strided batch or ragged groups ----
enum AnyEpilogue { ANY_EPI_STORE = 0, ANY_EPI_RELU2 = 1, ANY_EPI_ADD = 2 };
struct AnyGemm {
  const void* A = nullptr;   // [rows][lda]
  const void* W = nullptr;   // [N][ldw]
  void* C = nullptr;         // [rows][ldc]
  int M = 0, N = 0, K = 0;   // dense: M rows; ragged: M unused
  long lda = 0, ldw = 0, ldc = 0;
  long a_bs = 0, w_bs = 0, c_bs = 0;      // element strides between batches (dense) / between groups' weights (ragged: w_bs)
  const int* tile_group = nullptr;        // ragged: device lists built by launch_ragged_tiles
  const int* tile_row0 = nullptr;
  const int* n_tiles = nullptr;
  const int* group_offsets = nullptr;     // [groups + 1] slots of each group
  const int* a_rows = nullptr;            // slot -> row of A (null: the slot itself)
  int epilogue = ANY_EPI_STORE;
  float alpha = 1.f;
};
int any_gemm_tile_rows();
int any_gemm_ragged_rows_limit();
int launch_ragged_tiles(const int* group_offsets, int G, int* tile_group, int* tile_row0, int* n_tiles, int cap, cudaStream_t s);
// *_f32: element type of A / W / C (1 = fp32, 0 = bf16); batch: strided batches (dense); max_tiles: capacity of the tile list (ragged);
// ragged_rows / groups: total rows over all groups and the number of groups (ragged), which let a launch with few rows take the
// weight-streaming form (0 = always tiles)
int launch_gemm_any(const AnyGemm& g, int a_f32, int w_f32, int c_f32, int batch, int max_tiles, cudaStream_t s, int ragged_rows = 0,
                    int groups = 0);

// ---- resid_f32.cu: an fp32 residual stream and the unit-offset RMS norm x / rms(x) * (1 + g) around it ----
// gains are fp32 and hold 1 + g already.  Outputs are fp32 or bf16 (x_f32).
int launch_embed_unit_norm(const int32_t* ids, const void* table, int table_f32, const float* gain1p, float* h, int T, int W, int vocab,
                           float eps, cudaStream_t s);
// x1 = norm(h) * gain_a, x2 = norm(h) * gain_b (x2 / gain_b may be null): both norms of one layer share the statistic.
// rows != null: normalise rows[i] of h into row i of x1 (the final norm over the rows that get logits).
int launch_unit_norm2(const float* h, const float* gain_a, const float* gain_b, void* x1, void* x2, int x_f32, int T, int W, float eps,
                      const int32_t* rows, cudaStream_t s);
// fp32 logits (row stride V) -> greedy token per row (lowest index on ties), and optionally bf16 rows of stride v_pad
// whose tail is -inf (what the sampler reads; only the first bf16_rows rows)
int launch_logits_finish(const float* logits, int32_t* out_tokens, bf16* logits_bf16, int bf16_rows, int rows, int V, int v_pad, cudaStream_t s);

// Grouped RMS norm (the vector is cut into `groups` equal pieces, each divided by its own sqrt(mean(piece^2) + eps)) with a plain
// fp32 gain, around the same fp32 stream:
int launch_embed_scaled(const int32_t* ids, const void* table, int table_f32, float scale, float* h, int T, int W, int vocab, cudaStream_t s);
// x[t] = norm(h[rows ? rows[t] : t]) * gain, x fp32 or bf16
int launch_group_norm(const float* h, const float* gain, void* x, int x_f32, int T, int W, int groups, float eps, const int32_t* rows,
                      cudaStream_t s);
// h[t] += norm(y[t] + bias) * gain  (bias may be null): the norm behind a sublayer and the residual add in one pass; with gain_next
// the norm in front of the next sublayer as well, x_next[t] = norm(h[t]) * gain_next (fp32 or bf16)
int launch_group_norm_add(float* h, const float* y, const float* bias, const float* gain, int T, int W, int groups, float eps, cudaStream_t s,
                          const float* gain_next = nullptr, void* x_next = nullptr, int x_f32 = 0);
// act[t][i] = g * sigmoid(sharp * g) * (u + 1), g = min(gu[t][i], limit), u = clamp(gu[t][F + i], -limit, limit); gu fp32 [T][2F]
int launch_clamped_gate(const float* gu, void* act, int act_f32, int T, int F, float limit, float sharp, cudaStream_t s);

// x[t][col0 .. col0 + W) = src[t][0 .. W) in the operand type (x rows of ldx elements): one half of a concatenated projection input
int launch_store_rows(const float* src, void* x, int x_f32, int ldx, int col0, int T, int W, cudaStream_t s);
// act[t][i] = a N(z)[i] + b N(z^2)[i] + c N(z^3)[i] + e with N(y) = y / sqrt(mean(y^2) + eps) over the row and powers taken
// element by element; coef (device) = a, b, c, e; z fp32 [T][F]
int launch_poly_norm(const float* z, const float* coef, void* act, int act_f32, int T, int F, float eps, cudaStream_t s);
// act[r][i] = silu(s g) * (s u), g = gu[r][i], u = gu[r][F + i], s = row_scale[row_of ? row_of[r] : r] (null = 1): a gated unit whose INPUT was
// multiplied by s, applied behind the products; gu fp32 [rows][2F].  row_of maps a row to the entry of row_scale (an expert slot to its pair).
int launch_silu_gate(const float* gu, const float* row_scale, const int32_t* row_of, void* act, int act_f32, int rows, int F, cudaStream_t s);
// h[t] += coef * (n(a[t]) * gain_a + n(b[t]) * gain_b) + d1[t] + sum_k y[pair_slot[t * top + k]], n = RMS norm over the row; a null gain
// adds the branch as it is, null branches are left out.  With gain_next, x_next[t] = n(h[t]) * gain_next follows in the same pass.
int launch_branch_add(float* h, const float* a, const float* gain_a, const float* b, const float* gain_b, float coef, const float* d1,
                      const float* y, const int32_t* pair_slot, int top, int T, int W, float eps, cudaStream_t s,
                      const float* gain_next = nullptr, void* x_next = nullptr, int x_f32 = 0);
// logits <- cap * tanh(logits / cap), in place
int launch_softcap(float* logits, size_t n, float cap, cudaStream_t s);
// Layer norms with gain and bias, ln(v) = (v - mean) / sqrt(variance + eps) * w + b, around the same fp32 stream:
// x[t] = ln(h[rows ? rows[t] : t]), x fp32 or bf16
int launch_layer_norm(const float* h, const float* w, const float* b, void* x, int x_f32, int T, int W, float eps, const int32_t* rows, cudaStream_t s);
// h[t] += ln(y[t]): the norm behind a sublayer and the residual add in one pass.  pair_slot != null: the sublayer's output is the sum of the
// token's routed rows, y[t] = coef * sum_k y[pair_slot[t * top + k]].  With w_next the norm in front of the next sublayer as well.
int launch_layer_norm_add(float* h, const float* y, const int32_t* pair_slot, int top, float coef, const float* w, const float* b, int T, int W, float eps,
                          cudaStream_t s, const float* w_next = nullptr, const float* b_next = nullptr, void* x_next = nullptr, int x_f32 = 0);
// act[i] = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise; pq (device) = p, q
int launch_xielu(const float* z, const float* pq, void* act, int act_f32, size_t n, cudaStream_t s);
// out[t][i] = a[t][i] * sigmoid(gate[t * gate_ld + i]), out fp32 or bf16 [T][N]
int launch_sigmoid_gate(const float* a, const float* gate, int gate_ld, void* out, int out_f32, int T, int N, cudaStream_t s);

// ---- attn_heads.cu: softmax attention with per-head keys and values, any head width, fp32 or bf16 cache ----
struct HeadsGeom {
  int heads, kv_heads, dim, vdim;   // query head a reads key/value head a / (heads / kv_heads)
  int rot_dims;                     // rotary positions on interleaved pairs of the first rot_dims entries of q and k heads (0 = none)
  float rot_base;
  float scale, eps;
  int conv_taps;                    // causal convolution over time on every q / k / v channel (0 = none)
  int unit_qk;                      // 1: q and k heads are divided by their root mean square
  int slopes;                       // 1: slope_a * (i - j) is taken off the scores, slope_a = 2^(-slope_exp (a + 1) / heads)
  float slope_exp;
  int window, keep_first;           // window > 0: key j is seen from i when i - j < window or j < keep_first
  int cross;                        // 1: every query head's weights are applied to the values of every key/value head (for talk_gate)
  int swizzled;                     // 1: K and V rows go into the page layout of the GQA kernels (bf16, 128 wide, kv_swizzled_chunk) and the
                                    //    queries out as bf16, so that attn_decode.cu / attn_prefill_tc.cu serve the layer
  // mixers whose scores are mixed over the heads before the softmax (heads_finish_halves / heads_attention_premix)
  float rot_factor;                 // rotary angles of q and k are divided by this (0 = 1)
  int rot_values;                   // 1: the value of position j is rotated by j over all of vdim (pairs (m, m + vdim/2), angle j * rot_base^(-2m/vdim))
                                    //    before it is cached, and a query's weighted sum is turned back by its own position
  float softcap;                    // scores <- softcap * tanh(scores / softcap) (0 = none)
};
// proj [T][ld] fp32 = q | k | v (| more) of the fused projection.  bias [heads*dim + kv_heads*(dim+vdim)] or null; conv_w [channels][taps];
// ring [sequence slots][taps][channels] fp32 (row = position mod taps); row_seq / row_first / row_end [T]: the token's sequence slot and the first row / one past
// the last row of its portion in this step.  vmix_mode 0 none, 1 the layer supplies v_first [T][kv_heads*vdim], 2 it blends with it by
// *vmix_lambda.  Writes q_out [T][heads*dim] fp32 and the token's K and V cache rows.
int launch_heads_finish(const float* proj, int ld, const HeadsGeom& g, const float* bias, const float* conv_w, float* ring,
                        const int32_t* row_seq, const int32_t* row_first, const int32_t* row_end, const int32_t* positions,
                        const int32_t* slots, int vmix_mode, const float* vmix_lambda, float* v_first, float* q_out, void* k_cache,
                        void* v_cache, int cache_f32, int T, cudaStream_t s, void* q_bf16 = nullptr);
// tiles == null: decode form (row i is the newest token of block-table row i at positions[i]; seq_lens[i] == 0 rows give zeros).
// out [T][heads][vdim] (fp32 or bf16), or with g.cross [T][heads][kv_heads*vdim] fp32.
int launch_heads_attention(const float* q, const void* k_cache, const void* v_cache, int cache_f32, const HeadsGeom& g,
                           const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                           const int32_t* positions, const int32_t* seq_lens, void* out, int out_f32, int T, cudaStream_t s);
// out[t][a][d] = sigmoid(gate[t*gate_ld + a]) * sum_b talk[a][b] * cross[t][b][(a / (heads/kv_heads)) * vdim + d]; gate may be null
// What follows a fused, biased q | k | v projection when q and k are RMS-normed over the WHOLE row (all heads at once) with a gain per
// entry: proj [T][ld] fp32 = q (heads*dim) | k (kv_heads*dim) | v (kv_heads*vdim) | anything else; bias [nq + nk + nv] or null;
// qk_gain [nq + nk].  Writes q_out [T][heads*dim] fp32 and the token's K and V cache rows (plain layout); with g.swizzled the rows go into
// the GQA kernels' page layout and the queries out as bf16 (q_bf16) instead.
int launch_heads_finish_rownorm(const float* proj, int ld, const HeadsGeom& g, const float* bias, const float* qk_gain, const int32_t* slots,
                                float* q_out, void* k_cache, void* v_cache, int cache_f32, int T, cudaStream_t s, void* q_bf16 = nullptr);
// What follows a fused q | k | v projection (proj [T][ld] fp32) when every q and k head is RMS-normed with one gain of `dim` entries
// (q_gain, k_gain; null = no norm) and then rotated on half-split pairs: entry i of the first rot_dims pairs with entry i + rot_dims/2,
// angle position * rot_base^(-2i/rot_dims) / rot_factor; with g.rot_values the values are rotated over all of vdim the same way (no factor).
// Writes q_out [T][heads*dim] fp32 and the token's K and V cache rows (plain layout).
int launch_heads_finish_halves(const float* proj, int ld, const HeadsGeom& g, const float* q_gain, const float* k_gain, const int32_t* positions,
                               const int32_t* slots, float* q_out, void* k_cache, void* v_cache, int cache_f32, int T, cudaStream_t s);
// Softmax attention whose scaled scores pass the cap and are mixed over the heads, s'_a = sum_b mix[a][b] s_b (mix [heads][heads], null =
// none), BEFORE the softmax; causal, with g.window; with g.rot_values the weighted sum is turned back by the query's position.  All heads of
// a query token are formed together.  tiles == null: decode form.  out [T][heads*vdim] (fp32 or bf16).
int launch_heads_attention_premix(const float* q, const void* k_cache, const void* v_cache, int cache_f32, const HeadsGeom& g, const float* mix,
                                  const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                                  const int32_t* positions, const int32_t* seq_lens, void* out, int out_f32, int T, cudaStream_t s,
                                  float* scratch = nullptr, size_t scratch_floats = 0, int max_context = 0);
// scratch: device floats for the key splits of a decode step (heads_attention_premix_scratch_floats); without it a decode step runs unsplit,
// a CTA per sequence.  max_context: the longest sequence the engine holds (bounds the number of splits).
size_t heads_attention_premix_scratch_floats(int max_rows, int heads, int vdim);
int launch_talk_gate(const float* cross, const float* talk, const float* gate, int gate_ld, void* out, int out_f32, int heads, int kv_heads,
                     int vdim, int T, cudaStream_t s);

// ---- attn_state.cu: mixers with a matrix state per head (gated linear attention, gated delta rule) ----
enum StateRule { STATE_RULE_DECAY = 0, STATE_RULE_DELTA = 1 };
struct StateGeom {
  int heads, kv_heads, dim, vdim;   // state head a reads query/key head a / (heads / kv_heads); S is [dim][vdim] per head
  int rule;                         // StateRule
};
enum LowRankMode {
  LOWRANK_SIGMOID = 0,              // y = sigmoid(z)
  LOWRANK_DECAY_SIGMOID_POW = 1,    // y = sigmoid(z)^rate, formed as exp(-rate * softplus(-z))
  LOWRANK_DECAY_SOFTPLUS = 2        // y = exp(-exp(rate_log[c / per_head]) * softplus(z))
};
// out [T][C] fp32 = act(w2 [C][rank] . lr[t][lr_off .. lr_off + rank) + bias [C] (or null))
int launch_lowrank_act(const float* lr, int ld, int lr_off, int rank, const float* w2, const float* bias, int mode, float rate,
                       const float* rate_log, int per_head, float* out, int T, int C, cudaStream_t s);
// Delta rule, behind the fused projection proj [T][ld] fp32 = q (kv_heads*dim) | k (kv_heads*dim) | v (heads*vdim) | beta logits (heads) | ...:
// causal convolution over time (conv_w [channels][taps], last column = the current token; ring [slots][taps][channels], row = position mod
// taps) and silu on every channel, q and k heads to unit vectors x / sqrt(sum x^2 + unit_eps), q times dim^-1/2; out [T][channels], beta_out
// [T][heads] = sigmoid.  Updates the ring.
int launch_conv_unit_finish(const float* proj, int ld, const StateGeom& g, int taps, const float* conv_w, float* ring, const int32_t* row_seq,
                            const int32_t* row_first, const int32_t* row_end, const int32_t* positions, const int32_t* slots, float unit_eps,
                            float* out, float* beta_out, int T, cudaStream_t s);
// The recurrence over every portion of the step: portion i ends at row last_rows[i] (null: row i is a portion of one token); q / k rows of
// kv_heads*dim at strides ldq / ldk, v rows of heads*vdim at stride ldv, decay [T][heads*dim], beta [T][heads] (delta rule); q is multiplied
// by qscale.  state [slots][2][heads][dim][vdim] fp32 (state_floats_per_slot); out [T][heads*vdim] fp32.  Rows whose slot is negative are skipped.
int launch_state_scan(const float* q, int ldq, const float* k, int ldk, const float* v, int ldv, const float* decay, const float* beta,
                      const StateGeom& g, float qscale, float* state, int portions, const int32_t* last_rows, const int32_t* row_seq,
                      const int32_t* row_first, const int32_t* row_end, const int32_t* positions, const int32_t* slots, float* out,
                      cudaStream_t s);
size_t state_floats_per_slot(const StateGeom& g);
// out[t][a][:] = o[t][a][:] / sqrt(mean(o[t][a]^2) + eps) * gain[:] * (gate_silu ? silu(gate) : gate), gate at gate[t * gate_ld + a * vdim + :]
int launch_state_out_gate(const float* o, const float* gain, const float* gate, int gate_ld, int gate_silu, void* out, int out_f32,
                          int heads, int vdim, float eps, int T, cudaStream_t s);

// ---- attn_latent.cu: attention over a shared per-token latent (absorbed form) ----
// The cache holds, per token, the normalised latent c [kv_rank] and the rotated key piece [rot_dim] side by side
// (row width kv_rank + rot_dim, element type fp32 or bf16), in pages of block_size tokens.
struct LatentGeom {
  int heads, dim, rot_dim, vdim, kv_rank, rot_dims;
  float rot_base, scale, eps;
  int window;   // > 0: query i sees key j only when i - j < window (0 = every earlier key)
};
// qd [T][ld] fp32 = the fused projection's output: per head [dim | rot_dim], then (has_kv) the latent and the key piece.
// Writes q_nope [T][heads*dim] (operand type), q_rot [T][heads*rot_dim] fp32 (rotated) and, when has_kv, the token's cache row.
int launch_latent_finish(const float* qd, int ld, const LatentGeom& g, int has_kv, const float* latent_gain, const int32_t* positions,
                         const int32_t* slots, void* q_nope, int x_f32, float* q_rot, void* cache, int cache_f32, int T, cudaStream_t s);
// proj [T][ld] fp32 holds a query latent (q_rank entries at column off_q) and the key/value latent (kv_rank entries at off_c): both are
// RMS-normed with a plain gain; xq [T][q_rank] (operand type) feeds the query up-projection, the other is the token's cache row (a cache
// without a rotated piece: rows of kv_rank).
int launch_latent_pair_finish(const float* proj, int ld, int off_q, int q_rank, int off_c, int kv_rank, const float* gain_q, const float* gain_c,
                              float eps, const int32_t* slots, void* xq, void* cache, int x_f32, int T, cudaStream_t s);
// scores and weighted latent sum: q_abs [T][heads][kv_rank] fp32 (query pulled through the key up-projection), q_rot as above;
// tiles == null: decode form (token i is the newest token of block-table row i at positions[i]; seq_lens[i] == 0 rows are empty).
// out_lat [T][heads][kv_rank] (operand type).  sink [heads] or null (plain softmax).
int launch_latent_attention(const float* q_abs, const float* q_rot, const void* cache, int cache_f32, const LatentGeom& g,
                            const int32_t* block_table, int bt_stride, int block_size, const PrefillTile* tiles, int ntiles,
                            const int32_t* positions, const int32_t* seq_lens, const float* sink, void* out_lat, int x_f32, int T,
                            cudaStream_t s, float* scratch = nullptr, size_t scratch_floats = 0, int max_context = 0);
// scratch: device floats for the key splits of a decode step (latent_attention_scratch_floats); without it a decode step runs
// unsplit.  max_context: longest cache the engine can hold (bounds the number of splits).
size_t latent_attention_scratch_floats(int max_rows, int max_heads, int max_rank);

// ---- moe_route.cu: sigmoid router with a choice offset and grouped selection, and the token permutation by expert ----
struct RouteGeom {
  int experts, top, groups, keep;
  int raw_weights;   // 1: the weights are the chosen experts' scores as they are; 0: divided by their sum
};
// x [T][W] (operand type), router [experts][W] fp32, correction [experts] fp32 (null = none) -> idx [T][top], weight [T][top]
int launch_route(const void* x, int x_f32, const float* router, const float* correction, const RouteGeom& g, int32_t* idx, float* weight,
                 int T, int W, cudaStream_t s);
// no router: idx[t][k] = table[ids[t]][k] (table [vocab][top] int32, entries clamped into [0, experts)), weight[t][k] = 1 / top
int launch_route_table(const int32_t* ids, const int32_t* table, int vocab, int experts, int top, int32_t* idx, float* weight, int T, cudaStream_t s);
// counting sort of the T*top (token, choice) pairs by expert: offsets [experts + 1] (the buffer holds 3 * stride ints,
// stride >= experts + 1: the kernels keep a histogram and a cursor behind the offsets, at offsets + stride and
// offsets + 2 * stride; zero it once when it is allocated), slot_token [T*top] (slot -> token), pair_slot [T*top] (pair -> slot).
int launch_route_permute(const int32_t* idx, int T, int top, int experts, int32_t* offsets, int stride, int32_t* slot_token,
                         int32_t* pair_slot, cudaStream_t s);
// slot_weight[pair_slot[p]] = weight[p] for the T*top pairs
int launch_route_slot_weights(const float* weight, const int32_t* pair_slot, float* slot_weight, int npairs, cudaStream_t s);
// act[i] = bf16(max(up[i], 0)^2), n a multiple of 4
int launch_relu2_round(const float* up, bf16* act, size_t n, cudaStream_t s);
// h[t] += sum_k weight[t][k] * y[pair_slot[t*top + k]]   (+ mix[t] when given); fp32
int launch_route_combine(float* h, const float* mix, const float* y, const float* weight, const int32_t* pair_slot, int T, int W, int top,
                         cudaStream_t s);

}  // namespace b2
