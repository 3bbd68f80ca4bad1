// engine.cu -- the model engine behind the C ABI (include/b2_engine.h): weights resident in
// HBM, paged KV pool + block allocator, the Qwen3 layer loop (HF:models/qwen3/
// modeling_qwen3.py:378-438, :305-334) as a stream of hand-written kernels, CUDA-graph replay
// of the decode step, and the measurement hooks bench.py uses.
#include <fcntl.h>
#include <math.h>
#include <stdarg.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <list>
#include <map>
#include <unordered_map>
#include <string>
#include <vector>

#include "../../include/b2_engine.h"
#include "json.hpp"
#include "kernels.h"

// ---------------------------------------------------------------------------------------
static thread_local char g_err[1024] = "";
void b2_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
}
extern "C" const char* b2_last_error(void) { return g_err; }
int b2_pdl_early_mask() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B2_PDL_EARLY");
    v = e ? atoi(e) : 7;
  }
  return v;
}
bool b2_pdl_trigger_early() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B2_PDL_TRIGGER");
    v = (e && *e == '0') ? 0 : 1;
  }
  return v != 0;
}
// The next launch of this thread goes out WITHOUT the programmatic attribute (the first kernel after a cross-stream
// fork or join: its predecessors are ordinary full dependencies).
static thread_local int g_pdl_skip_next = 0;
void b2_pdl_skip_next() { g_pdl_skip_next = 1; }
bool b2_pdl_enabled() {
  if (g_pdl_skip_next) {
    g_pdl_skip_next = 0;
    return false;
  }
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B2_PDL");
    v = (e && *e == '0') ? 0 : 1;
  }
  return v != 0;
}
extern "C" int b2_abi_version(void) { return B2_ABI_VERSION; }

using namespace b2;

namespace {

struct LayerW {
  bf16 *ln1 = nullptr, *ln2 = nullptr, *qnorm = nullptr, *knorm = nullptr;
  bf16 *wqkv = nullptr, *wo = nullptr, *wgu = nullptr, *wd = nullptr;
  // OPT only (biased projections, LayerNorm biases); wgu then holds fc1 [I][H] and wd holds fc2
  bf16 *bqkv = nullptr, *bo = nullptr, *ln1_b = nullptr, *ln2_b = nullptr, *b1 = nullptr, *b2 = nullptr;
  CUtensorMap tm_qkv, tm_o, tm_gu, tm_d;
  CUtensorMap tm_o32, tm_gu96, tm_d32;  // narrow-box maps of the fused chain (chain_cluster.cu)
  CUtensorMap tm_gu64;                  // 64-row box: gate rows and up rows of one SwiGLU tile (gemm_pair.cu)
};

// One layer of a layer-list family (Lerasun).  Operand-typed tensors (void*) are bf16, or fp32 when the engine computes in
// fp32; gains, the sink, the router and its correction are always fp32.
struct ListLayer {
  b2_layer_spec sp;
  int nq = 0, nqd = 0;        // rows of the fused q | latent projection: heads * (dim + rot_dim), + kv_rank + rot_dim when the layer has its own latent
  int cache_region = -1;      // which cache region the layer attends over (its own, or layer kv_from's)
  void *wqd = nullptr, *ukT = nullptr, *uv = nullptr, *wo = nullptr, *up = nullptr, *down = nullptr;
  float *gain1 = nullptr, *gain2 = nullptr, *lat_gain = nullptr, *sink = nullptr, *router = nullptr, *corr = nullptr;
  // Mixers with per-head keys and values (Kedasun): wqd holds q | k | v (| the head gates) as one projection of nqd rows, `up` holds
  // gate | up of the dense feed-forward, `down` its output projection; norms before (gain1, gain2) and behind (gain1b, gain2b) each sublayer.
  int nk = 0, nv = 0;         // kv_heads * dim, kv_heads * vdim
  int v_region = -1;          // cache region of the values (cache_region holds the keys)
  int vmix_mode = 0;          // 0 no value mixing, 1 the layer supplies the first values, 2 it blends with them
  bool gqa_tc = false;        // bf16, 128-wide heads in groups of two, plain causal softmax: the layer's cache has the GQA kernels' page
                              // layout and attention runs on attn_prefill_tc.cu / attn_decode.cu
  float *gain1b = nullptr, *gain2b = nullptr, *qkv_bias = nullptr, *o_bias = nullptr, *conv_w = nullptr, *talk = nullptr, *vmix = nullptr;
  float* conv_ring = nullptr; // [sequence slots][taps][q | k | v channels], row = position mod taps: the projected rows a sequence's next convolutions need
  // Mixers with a matrix state (Bumalix): `wqd` is ONE projection of the layer's norm output -- softmax q | k | v, then the state mixer's
  // q | k | v | g, then the low-rank first stage a1 ("parallel"); or q | k | v | b | a1 | g1 (delta rule).  The low-rank widths are the
  // checkpoint tensors' (no config entry names them): a1 / g1 wait on the host until the weights are finalised, when the projection is
  // re-made with their rows behind the n_fixed rows whose count the config gives.  wo / wo2: output projections of the first / second mixer.
  int n_fixed = 0, rank_a = 0, rank_g = 0;
  int off_sq = 0, off_sk = 0, off_sv = 0, off_sg = 0;   // first column of the state mixer's q, k, v, g in the projection's output
  void *wo2 = nullptr, *sh_up = nullptr, *sh_down = nullptr;   // sh_*: the shared expert (gate | up, down)
  float *qk_gain = nullptr, *head_gain = nullptr, *a2 = nullptr, *a2_bias = nullptr, *g2 = nullptr, *a_log = nullptr, *out_gain_l = nullptr,
        *out_gain_r = nullptr, *poly = nullptr;
  size_t a2_floats = 0, g2_floats = 0;
  std::vector<uint16_t> a1_host, g1_host;
  // Layer norms with gain and bias around every sublayer (Tinevik): gain1 / gain1b / gain2 / gain2b hold the gains, these the biases.  Its
  // state mixer projects q | k | v | g (| a1) in `wqd` (off_s*), its softmax mixer q | k | v with one gain per head entry for q and for k
  // (`qk_gain` = [dim] | [dim]) and the score-mixing matrix `talk`, its latent mixer dq | dkv | g in `wqd` (off_sq / off_sk / off_sg), the
  // query up-projection `uq` and the two latent gains (`latq_gain`, `lat_gain`).  `poly` holds the dense activation's two numbers, `table`
  // the experts of every token id [vocab][top].
  float *bias1 = nullptr, *bias1b = nullptr, *bias2 = nullptr, *bias2b = nullptr, *latq_gain = nullptr;
  void* uq = nullptr;
  int32_t* table = nullptr;
};
// One run of a layer.  A looped layer runs once per pass with the same weights (ListLayer) but a cache and state of its own.
struct ListRun {
  int layer = 0;
  bool pass_start = false;     // the loop's input mix x <- W_in [x; x0] comes right before this run
  int k_region = -1, v_region = -1;
  float* state = nullptr;      // [sequence slots][2][heads][dim][vdim] fp32 (attn_state.cu)
  float* ring = nullptr;       // [sequence slots][taps][channels] fp32: the convolutions' last inputs
};
inline bool list_arch(int arch) { return arch == B2_ARCH_LERASUN || arch == B2_ARCH_KEDASUN || arch == B2_ARCH_BUMALIX || arch == B2_ARCH_TINEVIK; }

struct Seq {
  bool active = false;
  int len = 0;        // tokens whose K/V are in the cache
  int reserved = 0;   // token capacity of the pages held
  int32_t next_token = 0;   // greedy token the last forward produced for this sequence (host copy)
  bool next_valid = false;  // false when only the device holds it (no D2H was requested)
  std::vector<int32_t> blocks;
  // prefix cache: chain[j] = hash of the first 16 (j + 1) prompt tokens (one entry per full page whose token ids the
  // host has seen), pending = ids since the last page boundary, chain_open = every token so far came from a prefill
  // call (a decode step's token lives on the device only, so the chain ends there)
  std::vector<uint64_t> chain;
  std::vector<int32_t> pending;
  bool chain_open = false;
};

enum XBuf { XB_X = 0, XB_ATTN = 1, XB_ACT = 2, XB_LAST = 3, XB_COUNT = 4 };
static const int kBnList[5] = {16, 32, 64, 128, 256};
static int bn_index(int bn) { return bn == 16 ? 0 : bn == 32 ? 1 : bn == 64 ? 2 : bn == 128 ? 3 : 4; }

// One stream of dependent launches over a contiguous block of batch rows.  A forward normally has a single lane
// (all rows, the engine's stream); a decode step over a large enough batch runs as TWO lanes -- two half-batches on
// two streams inside one step / one captured graph (see forward()).
struct Lane {
  cudaStream_t stream = nullptr;
  int row0 = 0;                 // first batch row of the lane
  float* partial = nullptr;     // split-K partials of this lane's projections
  size_t partial_floats = 0;
  float* attn_scratch = nullptr;
  bool beside_attention = false;  // projections use the short stage ring so their CTAs fit on an SM next to a
                                  // decode-attention CTA of the OTHER lane
};

struct GraphKey {
  int B, attn_split;
  bool operator<(const GraphKey& o) const { return B != o.B ? B < o.B : attn_split < o.attn_split; }
};

}  // namespace

struct b2_engine {
  b2_config cfg;
  int device = 0;
  int num_sms = 148;
  cudaStream_t stream = nullptr;
  bool finalized = false;
  int q_size = 0, kv_size = 0, qkv_size = 0;
  // Internal geometry.  The attention kernels are built for 128-wide heads in GQA groups of two; a
  // model with narrower heads (Phi-3: 96) or one query head per kv head (MHA) is laid out to fit:
  // every head is zero-padded to 128 dims and, for MHA, every real query head is followed by an
  // all-zero partner head.  The padding lives in the WEIGHTS (zero rows of Wqkv, zero columns of Wo,
  // scattered once at load time), so activations, KV pages and kernels need no special cases and the
  // arithmetic on the real elements is untouched; the cost is wasted bytes, which only matters for the
  // parity configurations that use it.
  int nq = 0, nkv = 0, hd = 128;  // internal (padded) head counts / width handed to the kernels
  int qhead_step = 1;             // real query head h lives at internal head h * qhead_step
  bool native_geom = true;        // cfg geometry == internal geometry (Qwen3): weights copy straight in
  float attn_scale = 0.f;         // real head_dim^-0.5
  int rotary_dim = 128;

  // weights
  bf16* embed = nullptr;
  bf16* lm_head = nullptr;  // == embed when tied
  bf16* final_norm = nullptr;
  bf16* final_norm_b = nullptr;  // OPT
  bf16* pos_embed = nullptr;     // OPT: learned positions [pos_rows][H], row = position + 2
  int pos_rows = 0;
  int gu_rows = 0;               // rows of wgu: 2*I (gate; up) or I (OPT fc1)
  std::vector<LayerW> layers;
  CUtensorMap tm_lm_head;
  std::map<std::string, int> loaded;
  int64_t weight_bytes = 0;
  bf16* cos_sin = nullptr;  // [max_model_len][hd]: cos[hd/2] | sin[hd/2]

  // KV pool
  bf16* kv_pool = nullptr;
  int64_t num_blocks = 0;
  size_t layer_kv_elems = 0;  // elements of one layer's K (or V) pool
  std::vector<int32_t> free_blocks;
  // Prefix cache (B2_TUNE_PREFIX_CACHE; vLLM's --enable-prefix-caching): full pages of PROMPT tokens are registered under
  // the hash of the whole token prefix they end; a new sequence whose prompt starts with the same tokens takes those
  // pages instead of recomputing them (reference-counted; a page nobody holds any more stays registered on an LRU list
  // until the allocator needs it).  A hit is verified against the stored token ids and the parent page, not the hash alone.
  bool prefix_cache = false;
  std::vector<int32_t> blk_ref;       // sequences holding the page
  std::vector<uint64_t> blk_hash;     // 0 = not registered
  std::vector<int32_t> blk_parent;    // registered: the page holding the 16 tokens before it (-1 = first page)
  std::vector<int32_t> blk_tokens;    // registered: its 16 token ids
  std::unordered_map<uint64_t, int32_t> pc_map;
  std::list<int32_t> pc_lru;          // registered pages with no holder, oldest first
  std::vector<std::list<int32_t>::iterator> pc_lru_pos;
  std::vector<char> pc_in_lru;
  int64_t pc_queries = 0, pc_hits = 0;  // prompt tokens looked up / served from the cache
  std::vector<Seq> seqs;
  int bt_stride = 0;

  // activations (capacity rows = cap_tokens)
  int cap_tokens = 0;
  bf16 *h = nullptr, *x = nullptr, *qkv = nullptr, *qrot = nullptr, *attn = nullptr, *gu = nullptr, *act = nullptr,
       *proj = nullptr, *xlast = nullptr;
  float* partial = nullptr;
  size_t partial_floats = 0;
  float* attn_scratch = nullptr;
  size_t attn_scratch_floats = 0;
  CUtensorMap tm_x[XB_COUNT][5];

  // batch state on the device
  int32_t *d_tokens = nullptr, *d_positions = nullptr, *d_seq_lens = nullptr, *d_slots = nullptr, *d_block_table = nullptr,
          *d_last_rows = nullptr, *d_out_tokens = nullptr, *d_token_log = nullptr, *d_step = nullptr;
  unsigned long long* d_argmax = nullptr;
  PrefillTile* d_tiles = nullptr;
  int tiles_cap = 0;
  int log_cap_steps = 0;
  // pinned host staging
  int32_t* h_stage = nullptr;
  size_t h_stage_ints = 0;
  PrefillTile* h_tiles = nullptr;
  int32_t* h_out = nullptr;
  int32_t* h_tok = nullptr;
  cudaEvent_t ev_tok = nullptr;

  std::vector<int32_t> cur_batch;  // sequence ids resident in d_* (decode fast path)
  int cur_B = 0;                   // padded batch (graph bucket)
  int last_n = 0;                  // sequences in the last forward
  int last_tokens = 0;             // tokens in the last forward

  // debug capture
  int debug_flags = 0;
  bf16* dbg_hidden = nullptr;
  int dbg_cap_tokens = 0;
  bf16* logits = nullptr;  // [max_seqs][vocab], allocated on demand

  // graphs
  std::map<GraphKey, cudaGraphExec_t> graphs;
  std::map<GraphKey, int64_t> graph_nodes;
  int64_t launches = 0;

  // profiling
  bool profiling = false;
  std::vector<cudaEvent_t> ev_pool;
  std::vector<std::pair<int, int>> ev_used;  // (class, index of start event)
  int ev_next = 0;

  // tunables (env)
  int simt_max_tokens = 0;  // T <= this -> SIMT GEMV path
  int attn_split_override = 0;
  int force_gemm_impl = -1;
  unsigned skip_mask = 0;
  long long kv_l2_budget = 0;      // B2_KV_L2_MB: bytes of next-layer K/V the projections prefetch into L2 (0 = off)
  int32_t* d_pf_frac = nullptr;
  int32_t* d_sample_out = nullptr;
  SampleRow* d_sample_rows = nullptr;     // per-row sampling parameters of one b2_sample(_rows) call
  std::vector<SampleRow> h_sample_rows;
  unsigned long long* d_gbar = nullptr;  // grid-barrier arrival counter of the decode chain kernel
  float* d_ss = nullptr;                  // fused chain: 2 x [32][64] sums of squares
  unsigned long long* d_gbar2 = nullptr;  // fused chain: its grid-barrier counter
  bool fused_ok = false;                  // shapes + cluster occupancy allow the fused chain
  int o_small_smem = 0;                   // B2_O_SMALL=1: O projection with a short stage ring so that it is resident beside
                                          // attention's CTAs (measured slower: 1.869 vs 1.832 ms/step at C2 -- its weight
                                          // prefetch competes with the tail of the K/V stream)
  int use_chain = 0;  // B2_CHAIN: 0 separate kernels (default, fastest measured), 1 chain.cu, 2 chain_cluster.cu
  int prefill_tc = 1; // B2_PREFILL_TC: prefill attention on tcgen05 (attn_prefill_tc.cu); 0 = the mma.sync kernel (attn_prefill.cu)
  int l2_weight_prefetch = 0;  // B2_WPF: resid path, see forward_layers (measured slower: off)
  int prefill_resid_fused = 0;  // B2_RESID_FUSED: prefill O / down projections add into the residual stream in their epilogue (measured slower: off)
  int qkv_rope_prefill_fused = 1;  // B2_QKV_ROPE_FUSED: prefill QKV projection finishes norm / RoPE / page write itself
  int prefill_pairs = 1;  // B2_PREFILL_PAIRS: see prefill_tile_pairs()
  int prefill_mc = 1;  // B2_MC: prefill projections as multicast CTA pairs (gemm_mc.cu)
  int gu_prefill_fused = 1;  // B2_GU_FUSED: prefill-sized gate/up projection with SwiGLU in its epilogue (gemm_gateup.cu)
  int use_pair = 1;   // B2_PAIR: bit 0 gate/up + SwiGLU, bit 1 QKV + QK-norm/RoPE/KV write as fused cluster-pair launches (gemm_pair.cu)

  // two-lane decode (B2_MB, see forward()): second stream, its own partials and attention scratch, fork/join events
  int mb_min_batch = 0;  // padded decode batches of at least this many rows (and at most 128) run as two lanes; 0 = never
  cudaStream_t stream2 = nullptr;
  float* partial2 = nullptr;
  size_t partial2_floats = 0;
  float* attn_scratch2 = nullptr;
  float* ssq = nullptr;  // [hidden / 16][64]: pieces of the next RMSNorm's sum of squares (gemm_resid.cu -> gemm_pair.cu)
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;

  // Cache regions: one per layer and K/V for the GQA families, one per layer that stores a latent for the layer-list
  // families.  A page p of a region starts at base + p * page_bytes; the allocator, the block tables and the prefix cache are
  // the same for all of them.
  struct PageRegion { char* base; size_t page_bytes; };
  std::vector<PageRegion> regions;

  // ---- layer-list families (Lerasun): fp32 residual stream, per-layer specs ----
  std::vector<b2_layer_spec> specs;
  std::vector<ListLayer> ll;
  bool f32 = false;            // cfg.compute_f32
  size_t esz = 2;              // bytes per operand element
  int v_pad = 0;               // row stride of the bf16 logits the sampler reads (vocab rounded up to 8)
  void *l_embed = nullptr, *l_head = nullptr;
  float *l_embed_gain = nullptr, *l_final_gain = nullptr, *l_final_bias = nullptr;
  char* l_pool = nullptr;      // the latent cache
  float *l_h = nullptr, *l_qd = nullptr, *l_qrot = nullptr, *l_qabs = nullptr, *l_mix = nullptr, *l_y = nullptr, *l_rw = nullptr,
        *l_logits = nullptr;
  void *l_x1 = nullptr, *l_x2 = nullptr, *l_qnope = nullptr, *l_olat = nullptr, *l_av = nullptr, *l_act = nullptr, *l_xl = nullptr;
  int32_t *l_idx = nullptr, *l_offsets = nullptr, *l_slot_token = nullptr, *l_pair_slot = nullptr, *l_tile_group = nullptr,
          *l_tile_row0 = nullptr, *l_ntiles = nullptr;
  int l_max_top = 0, l_tiles_cap = 0, l_rows_cap = 0, l_offsets_stride = 0;
  // per-head attention (Kedasun): fp32 queries, the first value-mixing layer's values of the step's tokens, the per-head sums
  // that weight mixing combines; and, per token row of the step, its sequence slot and the row range of its portion
  float *l_q = nullptr, *l_vfirst = nullptr, *l_cross = nullptr;
  bf16* l_qb = nullptr;              // bf16 queries of the layers the GQA kernels serve
  int32_t *d_row_seq = nullptr, *d_row_first = nullptr, *d_row_end = nullptr;
  bool l_has_state = false;          // some layer keeps per-sequence state besides the cache (convolution rings)
  float* l_attn_scratch = nullptr;   // key splits of a decode step's latent attention
  bf16* l_xperm = nullptr;           // prompt-sized steps: the feed-forward input rows in expert (slot) order
  float* l_upf = nullptr;            // ... and the experts' up-projection sums before the activation
  int32_t* h_offsets = nullptr;      // pinned: the experts' slot ranges of the step, read back for the per-expert launches
  size_t l_attn_scratch_floats = 0;
  float* dbg_hidden_f32 = nullptr;
  int dbg_slots = 0;                 // residual-stream captures per forward: embeddings + one per layer run
  // matrix-state mixers and the layer loop (Bumalix)
  std::vector<ListRun> runs;         // the order the layers run in
  int step_portions = 0;             // sequences in the step being run (each brings one portion of tokens)
  void *l_loop_in = nullptr, *l_cat = nullptr, *l_av2 = nullptr;   // W_in [W][2W]; its input [x | x0]; the second mixer's gated read-out
  float *l_dec = nullptr, *l_beta = nullptr, *l_gate = nullptr, *l_so = nullptr, *l_mix2 = nullptr, *l_ffd = nullptr, *l_slot_scale = nullptr;
  size_t l_qd_cols = 0;
  cudaStream_t l_side[3] = {nullptr, nullptr, nullptr};   // short steps: the second mixer (or the delta rule's low-rank stages), the feed-forward and the shared
                                                          // expert of a layer run beside the first mixer
  cudaEvent_t l_ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  float* l_upf2 = nullptr;           // the shared expert's gate | up sums and activation (its own, so that it can run beside the routed experts)
  void* l_act2 = nullptr;
};

namespace {

template <typename T>
int dalloc(T** p, size_t n) {
  void* q = nullptr;
  cudaError_t e = cudaMalloc(&q, n * sizeof(T));
  if (e != cudaSuccess) {
    b2_set_error("cudaMalloc(%zu bytes) failed: %s", n * sizeof(T), cudaGetErrorString(e));
    return -12;
  }
  *p = reinterpret_cast<T*>(q);
  return 0;
}
#define B2_TRY(expr)      \
  do {                    \
    int _r = (expr);      \
    if (_r != 0) return _r; \
  } while (0)

int env_int(const char* name, int dflt) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : dflt;
}

// kernel-launch bracket: counts launches and, in profile mode, times each one
struct KL {
  b2_engine* e;
  int cls;
  int ev = -1;
  bool skip() const { return (e->skip_mask >> cls) & 1u; }
  KL(b2_engine* e_, int cls_) : e(e_), cls(cls_) {
    if (skip()) return;
    e->launches++;
    if (e->profiling && e->ev_next + 2 <= (int)e->ev_pool.size()) {  // profiled steps are single-lane: the engine's stream
      ev = e->ev_next;
      e->ev_next += 2;
      cudaEventRecord(e->ev_pool[ev], e->stream);
    }
  }
  ~KL() {
    if (ev >= 0) {
      cudaEventRecord(e->ev_pool[ev + 1], e->stream);
      e->ev_used.emplace_back(cls, ev);
    }
  }
};

// Models with one query head per kv head run through the GQA-2 kernels with an all-zero partner head after every real one;
// the tcgen05 prefill attention then pairs two 64-token tiles per CTA instead of (real, zero) heads.
static bool prefill_tile_pairs(const b2_engine* e) {
  return e->prefill_tc && e->qhead_step == 2 && e->cfg.arch != B2_ARCH_OPT && !list_arch(e->cfg.arch) && e->prefill_pairs;
}

int bucket_batch(int B) {
  static const int bk[] = {1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512};
  for (int v : bk)
    if (B <= v) return v;
  return ((B + 127) / 128) * 128;
}

int pick_attn_split(b2_engine* e, int B, int max_len) {
  // The decode-attention kernel balances pages over its persistent warps by itself; there is no
  // host-side split factor any more.  The slot of the graph key now tells the two step variants apart.
  (void)B; (void)max_len;
  return (e->debug_flags & 2) ? 2 : 1;
}

// ---- one Linear layer: picks SIMT GEMV or the tcgen05 kernel, bf16 or split-K partial output
// xptr / out_bf16 are already offset to the lane's first row; the X tensor map covers the whole buffer, so the
// tcgen05 kernel gets the lane's row offset as a coordinate.
ActIn linear(b2_engine* e, const Lane& ln, int cls, XBuf xb, const bf16* xptr, const bf16* w, const CUtensorMap& tm_w, bf16* out_bf16,
             int T, int N, int K, int* rc, const KvPrefetch& pf = KvPrefetch(), bool want_f32 = false, bool after_attention = false,
             bf16* resid = nullptr, bool* resid_done = nullptr) {
  // want_f32: hand the consumer fp32 sums even when K is not split (a bias is added before the rounding)
  // resid: the residual stream rows this projection's output is added to.  When the launch is a single-split tcgen05 GEMM
  // with bf16 output (prefill shapes) the add happens in its epilogue, in place, and *resid_done tells the caller that the
  // norm kernel behind it has no delta to add; otherwise nothing changes.
  *rc = 0;
  if (resid_done) *resid_done = false;
  int impl = e->force_gemm_impl >= 0 ? e->force_gemm_impl : (T <= e->simt_max_tokens ? 0 : 1);
  if (ln.beside_attention && impl == 1 && tc_pick_bn(T) <= 64) want_f32 = true;  // the short ring is built for the partial epilogue
  if (want_f32 && (size_t)T * N > ln.partial_floats) {
    b2_set_error("linear: %d x %d fp32 outputs exceed the partial buffer", T, N);
    *rc = -12;
    return act_bf16(nullptr);
  }
  if (impl == 0) {
    KL k(e, cls);
    if (want_f32) {
      if (!k.skip()) *rc = launch_linear_simt(xptr, w, ln.partial, 1, T, N, K, ln.stream);
      return act_f32(ln.partial, 1);
    }
    if (!k.skip()) *rc = launch_linear_simt(xptr, w, out_bf16, 0, T, N, K, ln.stream);
    return act_bf16(out_bf16);
  }
  TcGemmArgs a;
  a.tmap_w = tm_w;
  a.bn = tc_pick_bn(T);
  a.tmap_x = e->tm_x[xb][bn_index(a.bn)];
  a.T = T; a.N = N; a.K = K;
  a.argmax_packed = nullptr;
  a.prefetch = pf;
  a.x_row0 = ln.row0;
  a.x_raw = xptr;
  a.small_smem = ((after_attention && e->o_small_smem) || ln.beside_attention) ? 1 : 0;
  int ns = tc_pick_nsplit(T, N, K, e->num_sms);
  {  // experiments: B2_NS_<class index>=n forces the split factor of one projection class
    static int forced[B2_NUM_KERNEL_CLASSES];
    static bool init = false;
    if (!init) {
      for (int i = 0; i < B2_NUM_KERNEL_CLASSES; ++i) {
        char name[32];
        snprintf(name, sizeof name, "B2_NS_%d", i);
        forced[i] = env_int(name, 0);
      }
      init = true;
    }
    if (cls >= 0 && cls < B2_NUM_KERNEL_CLASSES && forced[cls] > 0) ns = std::min(forced[cls], K / 64);
  }
  while (ns > 1 && (size_t)ns * T * N > ln.partial_floats) --ns;
  if (ns > 1) {  // re-validate (every split non-empty)
    const int kb = K / 64, kps = (kb + ns - 1) / ns;
    ns = (kb + kps - 1) / kps;
  }
  a.nsplit = ns;
  KL k(e, cls);
  if (ns == 1 && !want_f32) {
    a.epilogue = TC_EPI_BF16;
    a.out = out_bf16;
    if (resid != nullptr && resid_done != nullptr && a.bn >= 32 && !k.skip()) {
      a.out = resid;
      a.resid = resid;
      *rc = launch_linear_tc(a, ln.stream);
      *resid_done = true;
      return act_bf16(nullptr);
    }
    if (e->prefill_mc && a.bn == 256 && linear_mc_shapes_ok(T, N, K) && !pf.k_pages) {
      // prefill shapes: pairs of CTAs share the token tile (gemm_mc.cu); same arithmetic, a third less L2 -> shared-memory traffic
      if (!k.skip()) *rc = launch_linear_mc(tm_w, e->tm_x[xb][bn_index(128)], out_bf16, T, N, K, ln.row0, ln.stream);
      return act_bf16(out_bf16);
    }
    if (!k.skip()) *rc = launch_linear_tc(a, ln.stream);
    return act_bf16(out_bf16);
  }
  a.epilogue = TC_EPI_F32_PARTIAL;
  a.out = ln.partial;
  if (!k.skip()) *rc = launch_linear_tc(a, ln.stream);
  return act_f32(ln.partial, ns);
}

Lane whole_batch_lane(b2_engine* e) {
  Lane ln;
  ln.stream = e->stream;
  ln.row0 = 0;
  ln.partial = e->partial;
  ln.partial_floats = e->partial_floats;
  ln.attn_scratch = e->attn_scratch;
  return ln;
}

void dbg_capture(b2_engine* e, int slot, const bf16* src, int T) {
  if (!(e->debug_flags & 1) || e->dbg_hidden == nullptr || T > e->dbg_cap_tokens) return;
  cudaMemcpyAsync(e->dbg_hidden + (size_t)slot * e->dbg_cap_tokens * e->cfg.hidden, src, (size_t)T * e->cfg.hidden * 2,
                  cudaMemcpyDeviceToDevice, e->stream);
}

// The forward pass over T tokens already described by d_tokens/d_positions/d_slots (and, for
// decode, d_seq_lens/d_block_table rows 0..T-1).  prefill_tiles > 0 selects the causal prefill
// attention; nlast = number of rows that get logits (decode: T; prefill: one per sequence,
// gathered through d_last_rows).
int lm_head_and_argmax(b2_engine* e, int nlast, const bf16* xl, XBuf xb);

// Decode forward (one token per sequence): embedding, then per layer ONE attention launch and ONE
// chain launch (chain.cu) instead of ten separate kernels.
int forward_decode_chain(b2_engine* e, int T) {
  const b2_config& c = e->cfg;
  const int H = c.hidden, I = c.intermediate, L = c.num_layers;
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed(e->d_tokens, e->embed, e->h, T, H, c.vocab, e->d_argmax, T, e->stream));
  }
  const int bn = tc_pick_bn(T), bi = bn_index(bn);
  auto gemm_cfg = [&](int N, int K) {
    ChainGemm g;
    g.N = N; g.K = K;
    // enough splits to give most SMs a tile, but at least 4 k-blocks per split: the weight tile of a
    // split is prefetched a whole step ahead, so fatter splits cost nothing and halve the partials
    int ns = tc_pick_nsplit(T, N, K, e->num_sms);
    const int kb = K / 64;
    if (kb / ns < 4) ns = std::max(1, kb / 4);
    while (ns > 1 && (size_t)ns * T * N > e->partial_floats) --ns;
    g.kps = (kb + ns - 1) / ns;
    g.nsplit = (kb + g.kps - 1) / g.kps;
    return g;
  };
  ChainParams p;
  memset(&p, 0, sizeof p);
  p.T = T; p.bn = bn;
  p.g[0] = gemm_cfg(H, e->q_size);
  p.g[1] = gemm_cfg(2 * I, H);
  p.g[2] = gemm_cfg(H, I);
  p.g[3] = gemm_cfg(e->qkv_size, H);
  p.partial = e->partial;
  p.h = e->h; p.x = e->x; p.act = e->act; p.qrot = e->qrot;
  p.cos_sin = e->cos_sin; p.positions = e->d_positions; p.slots = e->d_slots;
  p.H = H; p.I = I; p.nq = e->nq; p.nkv = e->nkv; p.block_size = c.block_size; p.eps = c.rms_eps;
  p.gbar = e->d_gbar;
  CUtensorMap xm[4] = {e->tm_x[XB_ATTN][bi], e->tm_x[XB_X][bi], e->tm_x[XB_ACT][bi], e->tm_x[XB_X][bi]};
  auto kv_of = [&](int l, bf16** kp, bf16** vp) {
    *kp = e->kv_pool + (size_t)(2 * l) * e->layer_kv_elems;
    *vp = *kp + e->layer_kv_elems;
  };
  {  // head of the forward: ln1 of layer 0 on the embeddings, QKV(0), QK-norm/RoPE/KV(0)
    LayerW& L0 = e->layers[0];
    CUtensorMap wm[4] = {L0.tm_o, L0.tm_gu, L0.tm_d, L0.tm_qkv};
    p.phase_begin = 5; p.phase_end = 8;
    p.norm_w_a = L0.ln2; p.norm_w_b = L0.ln1; p.norm_b_has_delta = 0;
    p.qw = L0.qnorm; p.kw = L0.knorm;
    kv_of(0, &p.k_pages, &p.v_pages);
    KL k(e, B2K_CHAIN);
    if (!k.skip()) B2_TRY(launch_decode_chain(wm, xm, p, e->stream));
  }
  for (int l = 0; l < L; ++l) {
    LayerW& Lw = e->layers[l];
    bf16 *kp, *vp;
    kv_of(l, &kp, &vp);
    {
      KL k(e, B2K_ATTN_DECODE);
      if (!k.skip())
        B2_TRY(launch_attn_decode(e->qrot, kp, vp, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, e->attn, T,
                                  e->nq, e->nkv, e->hd, c.block_size, e->stream, e->attn_scale));
    }
    const bool last = (l + 1 == L);
    LayerW& Ln = e->layers[last ? l : l + 1];
    CUtensorMap wm[4] = {Lw.tm_o, Lw.tm_gu, Lw.tm_d, Ln.tm_qkv};
    p.phase_begin = 0; p.phase_end = last ? 6 : 8;
    p.norm_w_a = Lw.ln2; p.norm_w_b = last ? e->final_norm : Ln.ln1; p.norm_b_has_delta = 1;
    p.qw = Ln.qnorm; p.kw = Ln.knorm;
    kv_of(last ? l : l + 1, &p.k_pages, &p.v_pages);
    KL k(e, B2K_CHAIN);
    if (!k.skip()) B2_TRY(launch_decode_chain(wm, xm, p, e->stream));
  }
  return lm_head_and_argmax(e, T, e->x, XB_X);
}

// Decode through the fused four-step chain (chain_cluster.cu).  The head of the forward (embedding, layer 0's input
// norm, QKV and QK-norm/RoPE) and the tail (final norm, lm_head) use the separate kernels.
int forward_decode_fused(b2_engine* e, int T) {
  const b2_config& c = e->cfg;
  const int H = c.hidden, I = c.intermediate, L = c.num_layers;
  int rc = 0;
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed(e->d_tokens, e->embed, e->h, T, H, c.vocab, e->d_argmax, T, e->stream));
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_add_rmsnorm(e->h, act_bf16(nullptr), e->layers[0].ln1, e->x, T, H, c.rms_eps, e->stream));
  }
  {
    LayerW& L0 = e->layers[0];
    bf16* kp = e->kv_pool;
    bf16* vp = kp + e->layer_kv_elems;
    ActIn qkv = linear(e, whole_batch_lane(e), B2K_GEMM_QKV, XB_X, e->x, L0.wqkv, L0.tm_qkv, e->qkv, T, e->qkv_size, H, &rc);
    B2_TRY(rc);
    KL k(e, B2K_ROPE_KV);
    if (!k.skip()) B2_TRY(launch_qknorm_rope_kv(qkv, L0.qnorm, L0.knorm, e->cos_sin, e->d_positions, e->d_slots, e->qrot, kp, vp, T,
                                 e->nq, e->nkv, e->hd, c.block_size, c.rms_eps, e->stream, e->rotary_dim));
  }
  FusedChainParams p;
  memset(&p, 0, sizeof p);
  p.T = T;
  p.h = e->h; p.act = e->act; p.qrot = e->qrot;
  p.cos_sin = e->cos_sin; p.positions = e->d_positions; p.slots = e->d_slots;
  p.ss_a = e->d_ss; p.ss_b = e->d_ss + 32 * 64;
  p.H = H; p.I = I; p.nq = e->nq; p.nkv = e->nkv; p.block_size = c.block_size; p.eps = c.rms_eps;
  p.gbar = e->d_gbar2;
  const int bi = bn_index(64);
  CUtensorMap am[2] = {e->tm_x[XB_ATTN][bi], e->tm_x[XB_ACT][bi]};
  for (int l = 0; l < L; ++l) {
    LayerW& Lw = e->layers[l];
    bf16* kp = e->kv_pool + (size_t)(2 * l) * e->layer_kv_elems;
    bf16* vp = kp + e->layer_kv_elems;
    {
      KL k(e, B2K_ATTN_DECODE);
      if (!k.skip())
        B2_TRY(launch_attn_decode(e->qrot, kp, vp, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, e->attn, T,
                                  e->nq, e->nkv, e->hd, c.block_size, e->stream, e->attn_scale));
    }
    const bool last = (l + 1 == L);
    LayerW& Ln = e->layers[last ? l : l + 1];
    CUtensorMap wm[4] = {Lw.tm_o32, Lw.tm_gu96, Lw.tm_d32, Ln.tm_qkv};
    p.phase_begin = 0; p.phase_end = last ? 3 : 4;
    p.norm_w_a = Lw.ln2; p.norm_w_b = Ln.ln1;
    p.qw = Ln.qnorm; p.kw = Ln.knorm;
    p.k_pages = e->kv_pool + (size_t)(2 * (last ? l : l + 1)) * e->layer_kv_elems;
    p.v_pages = p.k_pages + e->layer_kv_elems;
    KL k(e, B2K_CHAIN);
    if (!k.skip()) B2_TRY(launch_decode_fused_chain(wm, am, p, e->stream));
  }
  {
    KL k(e, B2K_NORM);  // the last down step has already added the residual: normalise only
    if (!k.skip()) B2_TRY(launch_add_rmsnorm(e->h, act_bf16(nullptr), e->final_norm, e->x, T, H, c.rms_eps, e->stream));
  }
  return lm_head_and_argmax(e, T, e->x, XB_X);
}

// OPT decoder (HF:models/opt/modeling_opt.py:363-391 OPTDecoder.forward, :203-254 OPTDecoderLayer.forward with
// do_layer_norm_before): same GEMM and attention kernels, the elementwise steps of elementwise_opt.cu.
int forward_opt(b2_engine* e, int T, int ntiles, int nlast) {
  const b2_config& c = e->cfg;
  const int H = c.hidden, I = c.intermediate;
  int rc = 0;
  const Lane ln = whole_batch_lane(e);
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed_pos(e->d_tokens, e->d_positions, e->embed, e->pos_embed, e->h, T, H, c.vocab, e->pos_rows,
                                           e->d_argmax, nlast, e->stream));
  }
  dbg_capture(e, 0, e->h, T);
  ActIn delta = act_bf16(nullptr);
  const bf16* delta_bias = nullptr;
  for (int l = 0; l < c.num_layers; ++l) {
    LayerW& L = e->layers[l];
    bf16* kp = e->kv_pool + (size_t)(2 * l) * e->layer_kv_elems;
    bf16* vp = kp + e->layer_kv_elems;
    {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_add_layernorm(e->h, delta, delta_bias, L.ln1, L.ln1_b, e->x, T, H, c.rms_eps, e->stream));
    }
    if (l > 0) dbg_capture(e, l, e->h, T);
    ActIn qkv = linear(e, ln, B2K_GEMM_QKV, XB_X, e->x, L.wqkv, L.tm_qkv, e->qkv, T, e->qkv_size, H, &rc, KvPrefetch(), true);
    B2_TRY(rc);
    {
      // HF:...:151 "query_states = self.q_proj(hidden_states) * self.scaling", then attention with scaling 1.0
      KL k(e, B2K_ROPE_KV);
      if (!k.skip()) B2_TRY(launch_qknorm_rope_kv(qkv, nullptr, nullptr, e->cos_sin, e->d_positions, e->d_slots, e->qrot, kp, vp, T,
                                   e->nq, e->nkv, e->hd, c.block_size, c.rms_eps, e->stream, 0, L.bqkv, e->attn_scale));
    }
    if (ntiles > 0) {
      KL k(e, B2K_MISC);
      if (!k.skip()) B2_TRY(launch_attn_prefill(e->qrot, kp, vp, e->d_block_table, e->bt_stride, e->d_tiles, ntiles, e->attn,
                                 e->nq, e->nkv, e->hd, c.block_size, e->stream, 1.0f));
    } else {
      KL k(e, B2K_ATTN_DECODE);
      if (!k.skip())
        B2_TRY(launch_attn_decode(e->qrot, kp, vp, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, e->attn, T,
                                  e->nq, e->nkv, e->hd, c.block_size, e->stream, 1.0f));
    }
    ActIn o = linear(e, ln, B2K_GEMM_O, XB_ATTN, e->attn, L.wo, L.tm_o, e->proj, T, H, e->q_size, &rc, KvPrefetch(), true);
    B2_TRY(rc);
    {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_add_layernorm(e->h, o, L.bo, L.ln2, L.ln2_b, e->x, T, H, c.rms_eps, e->stream));
    }
    ActIn f1 = linear(e, ln, B2K_GEMM_GATEUP, XB_X, e->x, L.wgu, L.tm_gu, e->gu, T, I, H, &rc, KvPrefetch(), true);
    B2_TRY(rc);
    {
      KL k(e, B2K_ACT);
      if (!k.skip()) B2_TRY(launch_bias_relu(f1, L.b1, e->act, T, I, e->stream));
    }
    delta = linear(e, ln, B2K_GEMM_DOWN, XB_ACT, e->act, L.wd, L.tm_d, e->proj, T, H, I, &rc, KvPrefetch(), true);
    delta_bias = L.b2;
    B2_TRY(rc);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_add_layernorm(e->h, delta, delta_bias, e->final_norm, e->final_norm_b, e->x, T, H, c.rms_eps, e->stream));
  }
  dbg_capture(e, c.num_layers, e->h, T);
  dbg_capture(e, c.num_layers + 1, e->x, T);
  const bf16* xl = e->x;
  XBuf xb = XB_X;
  if (ntiles > 0) {
    KL k(e, B2K_MISC);
    if (!k.skip()) B2_TRY(launch_gather_rows(e->x, e->d_last_rows, e->xlast, nlast, H, e->stream));
    xl = e->xlast;
    xb = XB_LAST;
  }
  return lm_head_and_argmax(e, nlast, xl, xb);
}

// The decoder layers and the final norm over the lane's rows [row0, row0 + T): everything between the embedding and
// the lm_head.  Qwen3 / Phi-3 (HF:models/qwen3/modeling_qwen3.py:423-434).
int forward_layers(b2_engine* e, const Lane& ln, int T, int ntiles) {
  const b2_config& c = e->cfg;
  const int H = c.hidden, I = c.intermediate;
  const size_t r0 = (size_t)ln.row0;
  cudaStream_t st = ln.stream;
  const int tag = ln.row0 != 0 ? 1 : 0;  // lane marker in the step timeline
  bf16* h = e->h + r0 * H;
  bf16* x = e->x + r0 * H;
  bf16* qkvb = e->qkv + r0 * e->qkv_size;
  bf16* qrot = e->qrot + r0 * e->q_size;
  bf16* attn = e->attn + r0 * e->q_size;
  bf16* gub = e->gu + r0 * 2 * I;
  bf16* act = e->act + r0 * I;
  bf16* proj = e->proj + r0 * H;
  const int32_t* positions = e->d_positions + r0;
  const int32_t* slots = e->d_slots + r0;
  const int32_t* block_table = e->d_block_table + r0 * e->bt_stride;
  const int32_t* seq_lens = e->d_seq_lens + r0;
  int rc = 0;
  ActIn delta = act_bf16(nullptr);
  // decode only: the projections of layer l prefetch shares of the K/V pages the next attention pass
  // will read (QKV: this layer's own; O, gate-up, down: layer l+1's)
  auto prefetch_for = [&](int layer, int part) -> KvPrefetch {
    KvPrefetch pf;
    if (ntiles > 0 || e->kv_l2_budget <= 0 || layer >= c.num_layers) return pf;
    pf.k_pages = e->kv_pool + (size_t)(2 * layer) * e->layer_kv_elems;
    pf.v_pages = pf.k_pages + e->layer_kv_elems;
    pf.block_table = block_table;
    pf.seq_lens = seq_lens;
    pf.frac_q16 = e->d_pf_frac;
    pf.bt_stride = e->bt_stride;
    pf.B = T;
    pf.nkv = e->nkv;
    pf.part = part;
    pf.nparts = 4;
    return pf;
  };
  for (int l = 0; l < c.num_layers; ++l) {
    LayerW& L = e->layers[l];
    bf16* kp = e->kv_pool + (size_t)(2 * l) * e->layer_kv_elems;
    bf16* vp = kp + e->layer_kv_elems;
    // decode-sized forwards: the fused cluster-pair launches of gemm_pair.cu take the place of (projection, element-wise
    // kernel) pairs where the model's shapes allow it
    const bool pair_ok = ntiles == 0 && !ln.beside_attention && e->force_gemm_impl != 0 && T > e->simt_max_tokens && pair_shapes_ok(T, H) &&
                         !(e->debug_flags & 1) && e->kv_l2_budget <= 0;
    const bool qkv_pair = pair_ok && (e->use_pair & 2) && c.arch == B2_ARCH_QWEN3 && e->native_geom && e->rotary_dim == 128 && L.qnorm != nullptr &&
                          !((e->skip_mask >> B2K_ROPE_KV) & 1u);
    const bool gu_pair = pair_ok && (e->use_pair & 1) && I % 64 == 0 && !((e->skip_mask >> B2K_ACT) & 1u);
    // ... and with both in place the O / down projections add into the residual stream themselves (gemm_resid.cu) and the
    // pair kernels normalise h as they load it: no norm kernel inside the layer loop (skip-mask ablations take the old path)
    const bool resid = qkv_pair && gu_pair && (e->use_pair & 4) && e->ssq != nullptr && H / 16 <= 64 && resid_shapes_ok(T, H, e->q_size) &&
                       resid_shapes_ok(T, H, I) && !((e->skip_mask >> B2K_NORM) & 1u) && !((e->skip_mask >> B2K_GEMM_O) & 1u) &&
                       !((e->skip_mask >> B2K_GEMM_DOWN) & 1u) && !((e->skip_mask >> B2K_GEMM_QKV) & 1u) && !((e->skip_mask >> B2K_GEMM_GATEUP) & 1u);
    PairNorm pn1, pn2;
    if (resid) {
      pn1.ssq = pn2.ssq = e->ssq;
      pn1.gain = L.ln1; pn2.gain = L.ln2;
      pn1.pieces = pn2.pieces = H / 16;
      pn1.ld = pn2.ld = 64;
      pn1.eps = pn2.eps = c.rms_eps;
    }
    // resid path: each launch's idle lanes pull the NEXT launch's weights into L2 (the fat CTAs of these kernels cannot be
    // resident beside each other, so a launch can no longer start its own weight stream while its predecessor runs)
    L2Prefetch pf_gu, pf_d, pf_qkv_next;
    if (resid && e->l2_weight_prefetch) {
      pf_gu.ptr = L.wgu; pf_gu.bytes = (unsigned long long)2 * I * H * 2;
      pf_d.ptr = L.wd; pf_d.bytes = (unsigned long long)H * I * 2;
      if (l + 1 < c.num_layers) { pf_qkv_next.ptr = e->layers[l + 1].wqkv; pf_qkv_next.bytes = (unsigned long long)e->qkv_size * H * 2; }
      pn2.next_w = pf_d;
    }
    if (!(resid && l > 0)) {  // layer 0 (h comes from the embedding kernel) and every layer of the stand-alone path
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_add_rmsnorm(h, delta, L.ln1, x, T, H, c.rms_eps, st, tag));
    }
    if (l > 0) dbg_capture(e, l, e->h, T);
    const bool qkv_prefill_fused = ntiles > 0 && e->qkv_rope_prefill_fused && e->prefill_mc && e->force_gemm_impl != 0 && c.arch == B2_ARCH_QWEN3 &&
                                   e->native_geom && e->rotary_dim == 128 && L.qnorm != nullptr && linear_mc_shapes_ok(T, e->qkv_size, H) &&
                                   !((e->skip_mask >> B2K_ROPE_KV) & 1u) && !((e->skip_mask >> B2K_GEMM_QKV) & 1u);
    if (qkv_prefill_fused) {
      KL k(e, B2K_GEMM_QKV);  // prefill: QK-norm + RoPE + page write in the QKV projection's epilogue (gemm_mc.cu)
      B2_TRY(launch_qkv_rope_prefill(L.tm_qkv, e->tm_x[XB_X][bn_index(128)], L.qnorm, L.knorm, e->cos_sin, positions, slots, qrot, kp, vp, T, e->nq,
                                     e->nkv, H, c.block_size, c.rms_eps, ln.row0, st));
    } else if (qkv_pair) {
      KL k(e, B2K_GEMM_QKV);
      if (!k.skip())
        B2_TRY(launch_qkv_rope(L.tm_qkv, (resid && l > 0) ? h : x, L.qnorm, L.knorm, e->cos_sin, positions, slots, qrot, kp, vp, T, e->nq, e->nkv, H,
                               c.block_size, c.rms_eps, st, tag, (resid && l > 0) ? pn1 : PairNorm()));
    } else {
      ActIn qkv = linear(e, ln, B2K_GEMM_QKV, XB_X, x, L.wqkv, L.tm_qkv, qkvb, T, e->qkv_size, H, &rc, prefetch_for(l, 3));
      B2_TRY(rc);
      KL k(e, B2K_ROPE_KV);
      if (!k.skip()) B2_TRY(launch_qknorm_rope_kv(qkv, L.qnorm, L.knorm, e->cos_sin, positions, slots, qrot, kp, vp, T,
                                   e->nq, e->nkv, e->hd, c.block_size, c.rms_eps, st, e->rotary_dim, nullptr, 1.0f, tag));
    }
    if (ntiles > 0) {
      KL k(e, B2K_MISC);
      if (!k.skip()) {
        if (e->prefill_tc)
          B2_TRY(launch_attn_prefill_tc(qrot, kp, vp, e->num_blocks, block_table, e->bt_stride, e->d_tiles, ntiles, attn, e->nq, e->nkv, e->hd,
                                        c.block_size, st, e->attn_scale, c.sliding_window, prefill_tile_pairs(e) ? 1 : 0));
        else
          B2_TRY(launch_attn_prefill(qrot, kp, vp, block_table, e->bt_stride, e->d_tiles, ntiles, attn,
                                     e->nq, e->nkv, e->hd, c.block_size, st, e->attn_scale, c.sliding_window));
      }
    } else {
      KL k(e, B2K_ATTN_DECODE);
      if (!k.skip())
        B2_TRY(launch_attn_decode(qrot, kp, vp, block_table, e->bt_stride, seq_lens, ln.attn_scratch, attn, T,
                                  e->nq, e->nkv, e->hd, c.block_size, st, e->attn_scale, c.sliding_window, tag));
    }
    if (resid) {
      {
        KL k(e, B2K_GEMM_O);
        B2_TRY(launch_linear_resid(L.tm_o, attn, h, e->ssq, T, H, e->q_size, 64, st, tag, pf_gu));
      }
      {
        KL k(e, B2K_GEMM_GATEUP);
        B2_TRY(launch_gateup_swiglu(L.tm_gu64, h, act, T, I, H, st, tag, pn2));
      }
      KL k(e, B2K_GEMM_DOWN);
      B2_TRY(launch_linear_resid(L.tm_d, act, h, e->ssq, T, H, I, 64, st, tag, pf_qkv_next));
      delta = act_bf16(nullptr);  // h is up to date: the next norm (layer 0's successor never runs one; the final norm) adds nothing
      continue;
    }
    // prefill-sized forwards, opt-in (B2_RESID_FUSED=1): the O and down projections add their output to the residual stream in
    // their epilogue (gemm_tc.cu, `resid`), and the norm kernel behind them only normalises: half its traffic.  Measured at C2:
    // the projection grows by 3.8 us (32 two-byte loads per thread and chunk, behind the accumulator read), the norm kernel
    // shrinks by 1.7 us: 44.9 against 42.4 ms for the prefill on the same box.  Off.
    bf16* fuse_resid = (ntiles > 0 && e->prefill_resid_fused && !((e->skip_mask >> B2K_NORM) & 1u)) ? h : nullptr;
    bool o_added = false;
    ActIn o = linear(e, ln, B2K_GEMM_O, XB_ATTN, attn, L.wo, L.tm_o, proj, T, H, e->q_size, &rc, prefetch_for(l + 1, 0), false,
                     /*after_attention=*/ntiles == 0, fuse_resid, &o_added);
    B2_TRY(rc);
    {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_add_rmsnorm(h, o_added ? act_bf16(nullptr) : o, L.ln2, x, T, H, c.rms_eps, st, tag));
    }
    if (gu_pair) {
      KL k(e, B2K_GEMM_GATEUP);
      if (!k.skip()) B2_TRY(launch_gateup_swiglu(L.tm_gu64, x, act, T, I, H, st, tag));
    } else if (e->gu_prefill_fused && e->force_gemm_impl != 0 && gateup_prefill_shapes_ok(T, I, H) && !((e->skip_mask >> B2K_ACT) & 1u)) {
      KL k(e, B2K_GEMM_GATEUP);  // prefill-sized: SwiGLU in the projection's epilogue, no gu round trip through HBM
      if (!k.skip()) B2_TRY(launch_gateup_swiglu_prefill(L.tm_gu, e->tm_x[XB_X][bn_index(128)], act, T, I, H, ln.row0, st));
    } else {
      ActIn gu = linear(e, ln, B2K_GEMM_GATEUP, XB_X, x, L.wgu, L.tm_gu, gub, T, 2 * I, H, &rc, prefetch_for(l + 1, 1));
      B2_TRY(rc);
      KL k(e, B2K_ACT);
      if (!k.skip()) B2_TRY(launch_silu_mul(gu, act, T, I, st, tag));
    }
    bool d_added = false;
    delta = linear(e, ln, B2K_GEMM_DOWN, XB_ACT, act, L.wd, L.tm_d, proj, T, H, I, &rc, prefetch_for(l + 1, 2), false, false, fuse_resid, &d_added);
    B2_TRY(rc);
    if (d_added) delta = act_bf16(nullptr);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_add_rmsnorm(h, delta, e->final_norm, x, T, H, c.rms_eps, st, tag));
  }
  return 0;
}

// Layer-list families (Lerasun): h <- h + (mixer(n1(h)) + ff(n2(h))) on an fp32 residual stream.  The two norms of a
// layer share one statistic (one kernel).  Mixer = latent attention in absorbed form (attn_latent.cu); feed-forward =
// routed squared-ReLU experts as ragged groups of gemm_any.cu.  `rows` (device, nlast entries; null = every row) selects
// the positions that get logits.  Operands are bf16, or fp32 when the engine was created with compute_f32.
constexpr int LIST_TC_EXPERT_ROWS = 2048;

// C (fp32 [M][N]) = alpha * A (operand type [M][K]) . Wt^T for the layer-list families.  Prompt-sized bf16 products whose K the tcgen05
// projection kernel can tile (gemm_tc.cu: TMA needs 16-byte rows, its k-block is 64) take that kernel, fp32 sums written directly;
// everything else -- decode steps, fp32 mode, odd shapes -- takes gemm_any.cu.
bool list_use_tc() {
  static const bool use_tc = [] { const char* v = getenv("B2_LIST_TC"); return !(v && *v == '0'); }();
  return use_tc;
}
int list_dense(b2_engine* e, const void* A, const void* Wt, float* C, int M, int N, int K, float alpha, cudaStream_t stream = nullptr) {
  cudaStream_t ls = stream ? stream : e->stream;
  const int f = e->f32 ? 1 : 0;
  if (list_use_tc() && !f && alpha == 1.f && M > 64 && N >= 128 && K % 64 == 0) {
    TcGemmArgs a;
    a.bn = tc_pick_bn(M);
    B2_TRY(b2_make_tmap_bf16(&a.tmap_w, Wt, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128));
    B2_TRY(b2_make_tmap_bf16(&a.tmap_x, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)a.bn));
    a.T = M; a.N = N; a.K = K;
    a.nsplit = 1;
    a.out = C;
    a.x_raw = A;
    a.argmax_packed = nullptr;
    a.epilogue = TC_EPI_F32_PARTIAL;
    return launch_linear_tc(a, ls);
  }
  AnyGemm a;
  a.A = A; a.W = Wt; a.C = C; a.M = M; a.N = N; a.K = K; a.lda = K; a.ldw = K; a.ldc = N; a.alpha = alpha;
  return launch_gemm_any(a, f, f, 1, 1, 0, ls);
}   // (token, choice) pairs of a step from which the experts' products go expert by expert to the tcgen05 kernel

int forward_list(b2_engine* e, int T, int ntiles, int nlast) {
  const b2_config& c = e->cfg;
  const int W = c.hidden, f = e->f32 ? 1 : 0;
  cudaStream_t st = e->stream;
  auto dbg = [&](int slot) {
    if ((e->debug_flags & 1) && e->dbg_hidden_f32 != nullptr && T <= e->dbg_cap_tokens)
      cudaMemcpyAsync(e->dbg_hidden_f32 + (size_t)slot * e->dbg_cap_tokens * W, e->l_h, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st);
  };
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed_unit_norm(e->d_tokens, e->l_embed, f, e->l_embed_gain, e->l_h, T, W, c.vocab, c.rms_eps, st));
  }
  dbg(0);
  const PrefillTile* tiles = ntiles > 0 ? e->d_tiles : nullptr;
  const bool use_tc = list_use_tc();
  auto dense = [&](const void* A, const void* Wt, float* C, int M, int N, int K, float alpha) -> int { return list_dense(e, A, Wt, C, M, N, K, alpha); };
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    const b2_layer_spec& sp = L.sp;
    const bool has_ff = sp.ff == B2_FF_ROUTED_EXPERTS;
    const bool own = sp.kv_from < 0;
    LatentGeom g{sp.heads, sp.dim, sp.rot_dim, sp.vdim, sp.kv_rank, sp.rot_dims, sp.rot_base, sp.scale, c.rms_eps};
    char* cache_w = own ? e->regions[L.cache_region].base : nullptr;
    const char* cache_r = e->regions[L.cache_region].base;
    {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_unit_norm2(e->l_h, L.gain1, has_ff ? L.gain2 : nullptr, e->l_x1, has_ff ? e->l_x2 : nullptr, f, T, W, c.rms_eps, nullptr, st));
    }
    {
      KL k(e, B2K_GEMM_QKV);  // q of every head and, for a layer with its own latent, the latent and the shared key piece: one projection
      if (!k.skip()) B2_TRY(dense(e->l_x1, L.wqd, e->l_qd, T, L.nqd, W, 1.f));
    }
    {
      KL k(e, B2K_ROPE_KV);
      if (!k.skip()) B2_TRY(launch_latent_finish(e->l_qd, L.nqd, g, own ? 1 : 0, L.lat_gain, e->d_positions, e->d_slots, e->l_qnope, f, e->l_qrot, cache_w, f, T, st));
    }
    {
      KL k(e, B2K_GEMM_QKV);  // the query pulled through the key up-projection, all heads in one strided batch
      AnyGemm a;
      a.A = e->l_qnope; a.W = L.ukT; a.C = e->l_qabs; a.M = T; a.N = sp.kv_rank; a.K = sp.dim;
      a.lda = (long)sp.heads * sp.dim; a.ldw = sp.dim; a.ldc = (long)sp.heads * sp.kv_rank;
      a.a_bs = sp.dim; a.w_bs = (long)sp.kv_rank * sp.dim; a.c_bs = sp.kv_rank;
      if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, sp.heads, 0, st));
    }
    {
      KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
      if (!k.skip()) B2_TRY(launch_latent_attention(e->l_qabs, e->l_qrot, cache_r, f, g, e->d_block_table, e->bt_stride, c.block_size, tiles, ntiles,
                                                    e->d_positions, e->d_seq_lens, L.sink, e->l_olat, f, T, st, e->l_attn_scratch,
                                                    e->l_attn_scratch_floats, c.max_model_len));
    }
    {
      KL k(e, B2K_GEMM_O);  // values of every head from the weighted latent
      AnyGemm a;
      a.A = e->l_olat; a.W = L.uv; a.C = e->l_av; a.M = T; a.N = sp.vdim; a.K = sp.kv_rank;
      a.lda = (long)sp.heads * sp.kv_rank; a.ldw = sp.kv_rank; a.ldc = (long)sp.heads * sp.vdim;
      a.a_bs = sp.kv_rank; a.w_bs = (long)sp.vdim * sp.kv_rank; a.c_bs = sp.vdim;
      if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, f, sp.heads, 0, st));
    }
    {
      KL k(e, B2K_GEMM_O);
      if (!k.skip()) B2_TRY(dense(e->l_av, L.wo, e->l_mix, T, W, sp.heads * sp.vdim, 1.f));
    }
    if (has_ff) {
      RouteGeom rg{sp.experts, sp.top, sp.groups, sp.groups_keep};
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_route(e->l_x2, f, L.router, L.corr, rg, e->l_idx, e->l_rw, T, W, st));
      }
      {
        KL k(e, B2K_MISC);
        if (!k.skip()) B2_TRY(launch_route_permute(e->l_idx, T, sp.top, sp.experts, e->l_offsets, e->l_offsets_stride, e->l_slot_token, e->l_pair_slot, st));
      }
      // Prompt-sized bf16 steps: the rows are gathered into expert order, the experts' slot ranges are read back (one small
      // copy and a stream synchronisation per layer: nothing beside a pass that takes milliseconds), and every expert's two
      // products are plain dense projections on the tcgen05 kernel; the activation rounds the fp32 sums to the bf16 operand
      // of the second product.  Everything else (decode steps, short portions, fp32, odd sizes) runs as ragged groups.
      const bool tc_experts = use_tc && !f && ntiles > 0 && e->l_xperm != nullptr && T * sp.top >= LIST_TC_EXPERT_ROWS && W % 64 == 0 &&
                              sp.ff_dim % 64 == 0 && W >= 128 && sp.ff_dim >= 128 && e->skip_mask == 0;
      if (tc_experts) {
        B2_CUDA_OK(cudaMemcpyAsync(e->h_offsets, e->l_offsets, (size_t)(sp.experts + 1) * 4, cudaMemcpyDeviceToHost, st));
        {
          KL k(e, B2K_MISC);
          B2_TRY(launch_gather_rows((const bf16*)e->l_x2, e->l_slot_token, e->l_xperm, T * sp.top, W, st));
        }
        B2_CUDA_OK(cudaStreamSynchronize(st));
        const int32_t* off = e->h_offsets;
        B2_REQUIRE(off[0] == 0 && off[sp.experts] == T * sp.top, "layer %d: the experts' slot ranges do not cover the step's %d pairs", l, T * sp.top);
        {
          KL k(e, B2K_GEMM_GATEUP);
          for (int x = 0; x < sp.experts; ++x)
            if (off[x + 1] > off[x])
              B2_TRY(dense(e->l_xperm + (size_t)off[x] * W, (const bf16*)L.up + (size_t)x * sp.ff_dim * W, e->l_upf + (size_t)off[x] * sp.ff_dim,
                           off[x + 1] - off[x], sp.ff_dim, W, 1.f));
        }
        {
          KL k(e, B2K_ACT);
          B2_TRY(launch_relu2_round(e->l_upf, (bf16*)e->l_act, (size_t)T * sp.top * sp.ff_dim, st));
        }
        {
          KL k(e, B2K_GEMM_DOWN);
          for (int x = 0; x < sp.experts; ++x)
            if (off[x + 1] > off[x])
              B2_TRY(dense((const bf16*)e->l_act + (size_t)off[x] * sp.ff_dim, (const bf16*)L.down + (size_t)x * W * sp.ff_dim,
                           e->l_y + (size_t)off[x] * W, off[x + 1] - off[x], W, sp.ff_dim, 1.f));
        }
      } else {
        const int max_tiles = std::min(e->l_tiles_cap, (T * sp.top + any_gemm_tile_rows() - 1) / any_gemm_tile_rows() + sp.experts);
        if (T * sp.top > any_gemm_ragged_rows_limit() || W > 16384 || sp.ff_dim > 16384) {   // (a decode-sized step streams the experts' weights group by group instead)
          KL k(e, B2K_MISC);
          if (!k.skip()) B2_TRY(launch_ragged_tiles(e->l_offsets, sp.experts, e->l_tile_group, e->l_tile_row0, e->l_ntiles, max_tiles, st));
        }
        AnyGemm a;
        a.tile_group = e->l_tile_group; a.tile_row0 = e->l_tile_row0; a.n_tiles = e->l_ntiles; a.group_offsets = e->l_offsets;
        {
          KL k(e, B2K_GEMM_GATEUP);  // act[slot] = relu(U_e x[token(slot)])^2
          a.A = e->l_x2; a.a_rows = e->l_slot_token; a.W = L.up; a.C = e->l_act; a.N = sp.ff_dim; a.K = W; a.lda = W; a.ldw = W; a.ldc = sp.ff_dim;
          a.w_bs = (long)sp.ff_dim * W; a.epilogue = ANY_EPI_RELU2;
          if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, f, 1, max_tiles, st, T * sp.top, sp.experts));
        }
        {
          KL k(e, B2K_GEMM_DOWN);  // y[slot] = D_e act[slot]
          a.A = e->l_act; a.a_rows = nullptr; a.W = L.down; a.C = e->l_y; a.N = W; a.K = sp.ff_dim; a.lda = sp.ff_dim; a.ldw = sp.ff_dim; a.ldc = W;
          a.w_bs = (long)W * sp.ff_dim; a.epilogue = ANY_EPI_STORE;
          if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, 1, max_tiles, st, T * sp.top, sp.experts));
        }
      }
    }
    {
      KL k(e, B2K_NORM);  // h += mixer + sum_k w_k y_k
      if (!k.skip()) B2_TRY(launch_route_combine(e->l_h, e->l_mix, e->l_y, e->l_rw, e->l_pair_slot, T, W, has_ff ? sp.top : 0, st));
    }
    dbg(l + 1);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_unit_norm2(e->l_h, e->l_final_gain, nullptr, e->l_xl, nullptr, f, nlast, W, c.rms_eps, ntiles > 0 ? e->d_last_rows : nullptr, st));
  }
  {
    KL k(e, B2K_LMHEAD);
    if (!k.skip()) B2_TRY(dense(e->l_xl, e->l_head, e->l_logits, nlast, c.vocab, W, c.logit_scale != 0.f ? c.logit_scale : 1.f));
  }
  {
    KL k(e, B2K_MISC);
    bf16* lb = (e->debug_flags & 2) ? e->logits : nullptr;  // the sampler's rows: one per sequence, the leading rows
    if (!k.skip()) B2_TRY(launch_logits_finish(e->l_logits, e->d_out_tokens, lb, bucket_batch(std::max(c.max_seqs, 1)), nlast, c.vocab, e->v_pad, st));
  }
  return 0;
}

// Kedasun: h <- h + n1b(mixer(n1(h))), then h <- h + n2b(ff(n2(h))) on the same fp32 residual stream, every norm an RMS norm over
// equal pieces of the vector.  Mixers keep per-head keys and values (attn_heads.cu): q | k | v (| head gates) are ONE projection, the
// kernel behind it finishes the token (bias, convolution, rotary or unit norm, value mixing, cache rows), attention runs over the
// block table, and the norm behind the output projection adds into the stream.  Per-sequence state besides the cache (the
// convolution's last projected rows) lives in rings indexed by the sequence slot.
constexpr float KEDASUN_SLOPE_EXP = 8.0f;      // distance penalty of head a: 2^(-8 (a + 1) / heads) per position
constexpr float KEDASUN_GATE_SHARP = 1.702f;   // y = g * sigmoid(1.702 g) * (u + 1)

int forward_heads_list(b2_engine* e, int T, int ntiles, int nlast) {
  const b2_config& c = e->cfg;
  const int W = c.hidden, f = e->f32 ? 1 : 0, groups = c.norm_groups > 0 ? c.norm_groups : 1;
  cudaStream_t st = e->stream;
  auto dbg = [&](int slot) {
    if ((e->debug_flags & 1) && e->dbg_hidden_f32 != nullptr && T <= e->dbg_cap_tokens)
      cudaMemcpyAsync(e->dbg_hidden_f32 + (size_t)slot * e->dbg_cap_tokens * W, e->l_h, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st);
  };
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed_scaled(e->d_tokens, e->l_embed, f, c.embed_scale != 0.f ? c.embed_scale : 1.f, e->l_h, T, W, c.vocab, st));
  }
  dbg(0);
  const PrefillTile* tiles = ntiles > 0 ? e->d_tiles : nullptr;
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    const b2_layer_spec& sp = L.sp;
    const bool conv = sp.mixer == B2_MIXER_CONV_ATTENTION;
    HeadsGeom g{sp.heads, sp.kv_heads, sp.dim, sp.vdim, sp.rot_dims, sp.rot_base, sp.scale, c.rms_eps, conv ? sp.conv_taps : 0, conv ? 1 : 0,
                conv ? 1 : 0, KEDASUN_SLOPE_EXP, sp.window, sp.keep_first, conv ? 1 : 0, L.gqa_tc ? 1 : 0};
    char* kc = e->regions[L.cache_region].base;
    char* vc = e->regions[L.v_region].base;
    const bool has_ff = sp.ff == B2_FF_CLAMPED_GATED;
    const float* next_gain1 = l + 1 < c.num_layers && e->skip_mask == 0 ? e->ll[l + 1].gain1 : nullptr;  // the norm behind a sublayer also does the one in front of the next
    if (l == 0 || e->skip_mask != 0) {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_group_norm(e->l_h, L.gain1, e->l_x1, f, T, W, groups, c.rms_eps, nullptr, st));
    }
    {
      KL k(e, B2K_GEMM_QKV);  // q | k | v and, for the gated mixer, one gate logit per head: one projection
      if (!k.skip()) B2_TRY(list_dense(e, e->l_x1, L.wqd, e->l_qd, T, L.nqd, W, 1.f));
    }
    {
      KL k(e, B2K_ROPE_KV);
      if (!k.skip()) B2_TRY(launch_heads_finish(e->l_qd, L.nqd, g, L.qkv_bias, L.conv_w, L.conv_ring, e->d_row_seq, e->d_row_first, e->d_row_end,
                                                e->d_positions, e->d_slots, L.vmix_mode, L.vmix, e->l_vfirst, e->l_q, kc, vc, f, T, st,
                                                L.gqa_tc ? e->l_qb : nullptr));
    }
    if (L.gqa_tc) {   // the framework's GQA kernels: tcgen05 for prompt portions, the page-balanced stream for decode steps
      KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
      if (!k.skip()) {
        if (ntiles > 0)
          B2_TRY(launch_attn_prefill_tc(e->l_qb, (const bf16*)kc, (const bf16*)vc, e->num_blocks, e->d_block_table, e->bt_stride, e->d_tiles, ntiles,
                                        (bf16*)e->l_av, sp.heads, sp.kv_heads, 128, c.block_size, st, sp.scale, 0, 0));
        else
          B2_TRY(launch_attn_decode(e->l_qb, (const bf16*)kc, (const bf16*)vc, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, (bf16*)e->l_av, T,
                                    sp.heads, sp.kv_heads, 128, c.block_size, st, sp.scale, 0, 0));
      }
    } else {
      KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
      if (!k.skip()) B2_TRY(launch_heads_attention(e->l_q, kc, vc, f, g, e->d_block_table, e->bt_stride, c.block_size, tiles, ntiles, e->d_positions,
                                                   e->d_seq_lens, conv ? (void*)e->l_cross : e->l_av, conv ? 1 : f, T, st));
    }
    if (conv) {
      KL k(e, B2K_ACT);  // the heads' weights mixed (as sums over the per-head outputs) and the head gates
      if (!k.skip()) B2_TRY(launch_talk_gate(e->l_cross, L.talk, e->l_qd + (L.nq + L.nk + L.nv), L.nqd, e->l_av, f, sp.heads, sp.kv_heads, sp.vdim, T, st));
    }
    {
      KL k(e, B2K_GEMM_O);
      if (!k.skip()) B2_TRY(list_dense(e, e->l_av, L.wo, e->l_mix, T, W, sp.heads * sp.vdim, 1.f));
    }
    {
      KL k(e, B2K_NORM);  // h += n1b(mixer output + bias); x1 = the next sublayer's input norm
      const float* gn = e->skip_mask != 0 ? nullptr : has_ff ? L.gain2 : next_gain1;
      if (!k.skip()) B2_TRY(launch_group_norm_add(e->l_h, e->l_mix, L.o_bias, L.gain1b, T, W, groups, c.rms_eps, st, gn, gn ? e->l_x1 : nullptr, f));
    }
    if (has_ff) {
      if (e->skip_mask != 0) {
        KL k(e, B2K_NORM);
        if (!k.skip()) B2_TRY(launch_group_norm(e->l_h, L.gain2, e->l_x1, f, T, W, groups, c.rms_eps, nullptr, st));
      }
      {
        KL k(e, B2K_GEMM_GATEUP);  // gate | up: one projection
        if (!k.skip()) B2_TRY(list_dense(e, e->l_x1, L.up, e->l_y, T, 2 * sp.ff_dim, W, 1.f));
      }
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_clamped_gate(e->l_y, e->l_act, f, T, sp.ff_dim, sp.ff_limit, KEDASUN_GATE_SHARP, st));
      }
      {
        KL k(e, B2K_GEMM_DOWN);
        if (!k.skip()) B2_TRY(list_dense(e, e->l_act, L.down, e->l_mix, T, W, sp.ff_dim, 1.f));
      }
      {
        KL k(e, B2K_NORM);
        if (!k.skip()) B2_TRY(launch_group_norm_add(e->l_h, e->l_mix, nullptr, L.gain2b, T, W, groups, c.rms_eps, st, next_gain1, next_gain1 ? e->l_x1 : nullptr, f));
      }
    }
    dbg(l + 1);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_group_norm(e->l_h, e->l_final_gain, e->l_xl, f, nlast, W, groups, c.rms_eps, ntiles > 0 ? e->d_last_rows : nullptr, st));
  }
  {
    KL k(e, B2K_LMHEAD);
    if (!k.skip()) B2_TRY(list_dense(e, e->l_xl, e->l_head, e->l_logits, nlast, c.vocab, W, 1.f));
  }
  {
    KL k(e, B2K_MISC);
    bf16* lb = (e->debug_flags & 2) ? e->logits : nullptr;
    if (!k.skip()) B2_TRY(launch_logits_finish(e->l_logits, e->d_out_tokens, lb, bucket_batch(std::max(c.max_seqs, 1)), nlast, c.vocab, e->v_pad, st));
  }
  return 0;
}

// Bumalix: n = norm1(h); h <- h + (mixer(n) + ff(n)) on the same fp32 residual stream, one plain-gain RMS norm per layer feeding every
// branch.  The layers run in the order of e->runs: a looped run of layers appears once per pass, every pass with cache regions and state
// of its own, and the stream is re-mixed with the embedding output in front of every pass (x <- W_in [x; x0]).  Every projection that
// reads the norm output is ONE product (softmax q | k | v | state q | k | v | g | low-rank first stage); the softmax half runs on
// attn_heads.cu over the block table, the state half on attn_state.cu over the sequence slots; the last kernel of a layer adds every
// branch into the stream and forms the next layer's norm output.
constexpr float BUMALIX_UNIT_EPS = 1e-6f;   // q and k of the delta rule: x / sqrt(sum(x^2) + 1e-6)

int forward_state_list(b2_engine* e, int T, int ntiles, int nlast) {
  const b2_config& c = e->cfg;
  const int W = c.hidden, f = e->f32 ? 1 : 0;
  cudaStream_t st = e->stream;
  auto dbg = [&](int slot) {
    if ((e->debug_flags & 1) && e->dbg_hidden_f32 != nullptr && T <= e->dbg_cap_tokens && slot < e->dbg_slots)
      cudaMemcpyAsync(e->dbg_hidden_f32 + (size_t)slot * e->dbg_cap_tokens * W, e->l_h, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st);
  };
  // Short steps (a decode step, a few tokens of prompts) are chains of small launches: a layer's second mixer and its feed-forward then
  // run on streams of their own beside the first mixer and meet again at the kernel that adds the branches into the stream (inside a
  // captured step these become parallel branches of the graph).  Profiled and debugged steps stay on one stream.
  const bool multi = T <= 256 && !e->profiling && !(e->debug_flags & 1) && e->skip_mask == 0 && e->l_side[0] != nullptr;
  cudaStream_t sB = multi ? e->l_side[0] : st, sF = multi ? e->l_side[1] : st, sS = multi ? e->l_side[2] : st;
  auto fork = [&](cudaEvent_t ev, cudaStream_t to) -> int {     // `to` continues from this point of the main stream
    if (!multi) return 0;
    B2_CUDA_OK(cudaEventRecord(ev, st));
    B2_CUDA_OK(cudaStreamWaitEvent(to, ev, 0));
    return 0;
  };
  auto join = [&](cudaEvent_t ev, cudaStream_t from) -> int {   // the main stream waits for what `from` has been given
    if (!multi) return 0;
    B2_CUDA_OK(cudaEventRecord(ev, from));
    B2_CUDA_OK(cudaStreamWaitEvent(st, ev, 0));
    return 0;
  };
  auto first_on = [&](cudaStream_t) { if (multi) b2_pdl_skip_next(); };   // behind a cross-stream edge: an ordinary, full dependency
  auto dense = [&](const void* A, const void* Wt, float* C, int M, int N, int K, cudaStream_t s_) -> int { return list_dense(e, A, Wt, C, M, N, K, 1.f, s_); };
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed_scaled(e->d_tokens, e->l_embed, f, c.embed_scale != 0.f ? c.embed_scale : 1.f, e->l_h, T, W, c.vocab, st));
  }
  if (e->l_cat != nullptr) {
    KL k(e, B2K_MISC);   // x0, the half of W_in's input that every pass shares
    if (!k.skip()) B2_TRY(launch_store_rows(e->l_h, e->l_cat, f, 2 * W, W, T, W, st));
  }
  dbg(0);
  const PrefillTile* tiles = ntiles > 0 ? e->d_tiles : nullptr;
  const int portions = ntiles > 0 ? e->step_portions : T;
  const int32_t* last_rows = ntiles > 0 ? e->d_last_rows : nullptr;
  const bool use_tc = list_use_tc();
  bool have_norm = false;   // l_x1 already holds this layer's norm output (the layer before wrote it)
  for (size_t r = 0; r < e->runs.size(); ++r) {
    const ListRun& R = e->runs[r];
    ListLayer& L = e->ll[R.layer];
    const b2_layer_spec& sp = L.sp;
    if (R.pass_start) {
      {
        KL k(e, B2K_MISC);
        if (!k.skip()) B2_TRY(launch_store_rows(e->l_h, e->l_cat, f, 2 * W, 0, T, W, st));
      }
      KL k(e, B2K_GEMM_O);
      if (!k.skip()) B2_TRY(dense(e->l_cat, e->l_loop_in, e->l_h, T, W, 2 * W, st));
      have_norm = false;
    }
    if (!have_norm) {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_unit_norm2(e->l_h, L.gain1, nullptr, e->l_x1, nullptr, f, T, W, c.rms_eps, nullptr, st));   // (a CTA per row; the gain as it is)
    }
    const bool has_ff = sp.ff != B2_FF_NONE;
    if (has_ff) B2_TRY(fork(e->l_ev[0], sF));      // the feed-forward needs the norm output only
    const bool shared_beside = sp.ff == B2_FF_SCALED_GATED_EXPERTS && sp.shared_ff > 0;
    if (shared_beside) B2_TRY(fork(e->l_ev[4], sS));
    {
      KL k(e, B2K_GEMM_QKV);
      if (!k.skip()) B2_TRY(dense(e->l_x1, L.wqd, e->l_qd, T, L.nqd, W, st));
    }
    const bool two = sp.mixer == B2_MIXER_WINDOW_AND_STATE;
    if (two) B2_TRY(fork(e->l_ev[1], sB));         // the state mixer reads its part of the projection
    if (two) {
      HeadsGeom g{sp.heads, sp.kv_heads, sp.dim, sp.vdim, 0, 0.f, sp.scale, c.rms_eps, 0, 0, 0, 0.f, sp.window, 0, 0, L.gqa_tc ? 1 : 0};
      char* kc = e->regions[R.k_region].base;
      char* vc = e->regions[R.v_region].base;
      {
        KL k(e, B2K_ROPE_KV);
        if (!k.skip()) B2_TRY(launch_heads_finish_rownorm(e->l_qd, L.nqd, g, L.qkv_bias, L.qk_gain, e->d_slots, e->l_q, kc, vc, f, T, st, L.gqa_tc ? e->l_qb : nullptr));
      }
      if (L.gqa_tc) {   // the framework's GQA kernels: tcgen05 for prompt portions, the page-balanced stream for decode steps
        KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
        if (!k.skip()) {
          if (ntiles > 0)
            B2_TRY(launch_attn_prefill_tc(e->l_qb, (const bf16*)kc, (const bf16*)vc, e->num_blocks, e->d_block_table, e->bt_stride, e->d_tiles, ntiles,
                                          (bf16*)e->l_av, sp.heads, sp.kv_heads, 128, c.block_size, st, sp.scale, sp.window, 0));
          else
            B2_TRY(launch_attn_decode(e->l_qb, (const bf16*)kc, (const bf16*)vc, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, (bf16*)e->l_av, T,
                                      sp.heads, sp.kv_heads, 128, c.block_size, st, sp.scale, sp.window, 0));
        }
      } else {
        KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
        if (!k.skip()) B2_TRY(launch_heads_attention(e->l_q, kc, vc, f, g, e->d_block_table, e->bt_stride, c.block_size, tiles, ntiles, e->d_positions,
                                                     e->d_seq_lens, e->l_av, f, T, st));
      }
      {
        KL k(e, B2K_GEMM_O);
        if (!k.skip()) B2_TRY(dense(e->l_av, L.wo, e->l_mix, T, W, sp.heads * sp.vdim, st));
      }
      const StateGeom sg{sp.s_heads, sp.s_heads, sp.s_dim, sp.s_vdim, STATE_RULE_DECAY};
      first_on(sB);
      {
        KL k(e, B2K_ACT);   // decay per key channel: sigmoid(A2 (A1 n) + b)^(1 / tau)
        if (!k.skip()) B2_TRY(launch_lowrank_act(e->l_qd, L.nqd, L.n_fixed, L.rank_a, L.a2, L.a2_bias, LOWRANK_DECAY_SIGMOID_POW, 1.0f / sp.s_tau, nullptr, 0,
                                                 e->l_dec, T, sp.s_heads * sp.s_dim, sB));
      }
      {
        KL k(e, B2K_CHAIN);
        if (!k.skip()) B2_TRY(launch_state_scan(e->l_qd + L.off_sq, L.nqd, e->l_qd + L.off_sk, L.nqd, e->l_qd + L.off_sv, L.nqd, e->l_dec, nullptr, sg,
                                                1.0f / sqrtf((float)sp.s_dim), R.state, portions, last_rows, e->d_row_seq, e->d_row_first, e->d_row_end,
                                                e->d_positions, e->d_slots, e->l_so, sB));
      }
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_state_out_gate(e->l_so, L.head_gain, e->l_qd + L.off_sg, L.nqd, 1, e->l_av2, f, sp.s_heads, sp.s_vdim, c.rms_eps, T, sB));
      }
      {
        KL k(e, B2K_GEMM_O);
        if (!k.skip()) B2_TRY(dense(e->l_av2, L.wo2, e->l_mix2, T, W, sp.s_heads * sp.s_vdim, sB));
      }
    } else {
      const StateGeom sg{sp.heads, sp.kv_heads, sp.dim, sp.vdim, STATE_RULE_DELTA};
      const int nqk = sp.kv_heads * sp.dim, C = 2 * nqk + sp.heads * sp.vdim;
      B2_TRY(fork(e->l_ev[1], sB));
      first_on(sB);
      {
        KL k(e, B2K_ACT);   // decay exp(-exp(A_log) softplus(A2 (A1 n) + dt_bias)) and the output gate sigmoid(G2 (G1 n))
        if (!k.skip()) {
          B2_TRY(launch_lowrank_act(e->l_qd, L.nqd, L.n_fixed, L.rank_a, L.a2, L.a2_bias, LOWRANK_DECAY_SOFTPLUS, 0.f, L.a_log, sp.dim, e->l_dec, T,
                                    sp.heads * sp.dim, sB));
          B2_TRY(launch_lowrank_act(e->l_qd, L.nqd, L.n_fixed + L.rank_a, L.rank_g, L.g2, nullptr, LOWRANK_SIGMOID, 0.f, nullptr, 0, e->l_gate, T,
                                    sp.heads * sp.vdim, sB));
        }
      }
      if (multi) b2_pdl_skip_next();   // (the convolution's predecessor on the main stream is the projection, across the fork's record: keep it a full dependency)
      {
        KL k(e, B2K_ROPE_KV);
        if (!k.skip()) B2_TRY(launch_conv_unit_finish(e->l_qd, L.nqd, sg, sp.conv_taps, L.conv_w, R.ring, e->d_row_seq, e->d_row_first, e->d_row_end,
                                                      e->d_positions, e->d_slots, BUMALIX_UNIT_EPS, e->l_q, e->l_beta, T, st));
      }
      B2_TRY(join(e->l_ev[2], sB));   // (the low-rank stages ran beside the convolution)
      first_on(st);
      {
        KL k(e, B2K_CHAIN);
        if (!k.skip()) B2_TRY(launch_state_scan(e->l_q, C, e->l_q + nqk, C, e->l_q + 2 * nqk, C, e->l_dec, e->l_beta, sg, 1.0f, R.state, portions, last_rows,
                                                e->d_row_seq, e->d_row_first, e->d_row_end, e->d_positions, e->d_slots, e->l_so, st));
      }
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_state_out_gate(e->l_so, L.head_gain, e->l_gate, sp.heads * sp.vdim, 0, e->l_av, f, sp.heads, sp.vdim, c.rms_eps, T, st));
      }
      {
        KL k(e, B2K_GEMM_O);
        if (!k.skip()) B2_TRY(dense(e->l_av, L.wo, e->l_mix, T, W, sp.heads * sp.vdim, st));
      }
    }
    const float* d1 = nullptr;
    if (has_ff) first_on(sF);
    const float* yr = nullptr;
    if (sp.ff == B2_FF_POLYNORM) {
      {
        KL k(e, B2K_GEMM_GATEUP);
        if (!k.skip()) B2_TRY(dense(e->l_x1, L.up, e->l_upf, T, sp.ff_dim, W, sF));
      }
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_poly_norm(e->l_upf, L.poly, e->l_act, f, T, sp.ff_dim, c.rms_eps, sF));
      }
      {
        KL k(e, B2K_GEMM_DOWN);
        if (!k.skip()) B2_TRY(dense(e->l_act, L.down, e->l_ffd, T, W, sp.ff_dim, sF));
      }
      d1 = e->l_ffd;
    } else if (sp.ff == B2_FF_SCALED_GATED_EXPERTS) {
      const RouteGeom rg{sp.experts, sp.top, 1, 1, 1};
      const int F = sp.ff_dim, pairs = T * sp.top;
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_route(e->l_x1, f, L.router, nullptr, rg, e->l_idx, e->l_rw, T, W, sF));
      }
      {
        KL k(e, B2K_MISC);
        if (!k.skip()) {
          B2_TRY(launch_route_permute(e->l_idx, T, sp.top, sp.experts, e->l_offsets, e->l_offsets_stride, e->l_slot_token, e->l_pair_slot, sF));
          B2_TRY(launch_route_slot_weights(e->l_rw, e->l_pair_slot, e->l_slot_scale, pairs, sF));
        }
      }
      // The weight multiplies the expert's input: gate and up are linear in it, so it is applied to their fp32 sums inside the
      // activation.  Prompt-sized bf16 steps run expert by expert on the tcgen05 projection kernel (rows gathered into expert
      // order, slot ranges read back); everything else as ragged groups.
      const bool tc_experts = !multi && use_tc && !f && ntiles > 0 && e->l_xperm != nullptr && pairs >= LIST_TC_EXPERT_ROWS && W % 64 == 0 && F % 64 == 0 &&
                              W >= 128 && F >= 64 && e->skip_mask == 0;
      if (tc_experts) {
        B2_CUDA_OK(cudaMemcpyAsync(e->h_offsets, e->l_offsets, (size_t)(sp.experts + 1) * 4, cudaMemcpyDeviceToHost, st));
        {
          KL k(e, B2K_MISC);
          B2_TRY(launch_gather_rows((const bf16*)e->l_x1, e->l_slot_token, e->l_xperm, pairs, W, st));
        }
        B2_CUDA_OK(cudaStreamSynchronize(st));
        const int32_t* off = e->h_offsets;
        B2_REQUIRE(off[0] == 0 && off[sp.experts] == pairs, "layer %d: the experts' slot ranges do not cover the step's %d pairs", R.layer, pairs);
        {
          KL k(e, B2K_GEMM_GATEUP);
          for (int x = 0; x < sp.experts; ++x)
            if (off[x + 1] > off[x])
              B2_TRY(dense(e->l_xperm + (size_t)off[x] * W, (const bf16*)L.up + (size_t)x * 2 * F * W, e->l_upf + (size_t)off[x] * 2 * F, off[x + 1] - off[x],
                           2 * F, W, st));
        }
        {
          KL k(e, B2K_ACT);
          B2_TRY(launch_silu_gate(e->l_upf, e->l_slot_scale, nullptr, e->l_act, 0, pairs, F, st));
        }
        {
          KL k(e, B2K_GEMM_DOWN);
          for (int x = 0; x < sp.experts; ++x)
            if (off[x + 1] > off[x])
              B2_TRY(dense((const bf16*)e->l_act + (size_t)off[x] * F, (const bf16*)L.down + (size_t)x * W * F, e->l_y + (size_t)off[x] * W,
                           off[x + 1] - off[x], W, F, st));
        }
      } else {
        const int max_tiles = std::min(e->l_tiles_cap, (pairs + any_gemm_tile_rows() - 1) / any_gemm_tile_rows() + sp.experts);
        if (pairs > any_gemm_ragged_rows_limit() || W > 16384 || 2 * F > 16384) {
          KL k(e, B2K_MISC);
          if (!k.skip()) B2_TRY(launch_ragged_tiles(e->l_offsets, sp.experts, e->l_tile_group, e->l_tile_row0, e->l_ntiles, max_tiles, sF));
        }
        AnyGemm a;
        a.tile_group = e->l_tile_group; a.tile_row0 = e->l_tile_row0; a.n_tiles = e->l_ntiles; a.group_offsets = e->l_offsets;
        {
          KL k(e, B2K_GEMM_GATEUP);  // gate | up of every (token, choice) pair in expert order, fp32 sums
          a.A = e->l_x1; a.a_rows = e->l_slot_token; a.W = L.up; a.C = e->l_upf; a.N = 2 * F; a.K = W; a.lda = W; a.ldw = W; a.ldc = 2 * F;
          a.w_bs = (long)2 * F * W; a.epilogue = ANY_EPI_STORE;
          if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, 1, max_tiles, sF, pairs, sp.experts));
        }
        {
          KL k(e, B2K_ACT);
          if (!k.skip()) B2_TRY(launch_silu_gate(e->l_upf, e->l_slot_scale, nullptr, e->l_act, f, pairs, F, sF));
        }
        {
          KL k(e, B2K_GEMM_DOWN);
          a.A = e->l_act; a.a_rows = nullptr; a.W = L.down; a.C = e->l_y; a.N = W; a.K = F; a.lda = F; a.ldw = F; a.ldc = W;
          a.w_bs = (long)W * F; a.epilogue = ANY_EPI_STORE;
          if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, 1, max_tiles, sF, pairs, sp.experts));
        }
      }
      yr = e->l_y;
      if (sp.shared_ff > 0) {   // (buffers of its own: in short steps it runs beside the routed experts)
        first_on(sS);
        {
          KL k(e, B2K_GEMM_GATEUP);
          if (!k.skip()) B2_TRY(dense(e->l_x1, L.sh_up, e->l_upf2, T, 2 * sp.shared_ff, W, sS));
        }
        {
          KL k(e, B2K_ACT);
          if (!k.skip()) B2_TRY(launch_silu_gate(e->l_upf2, nullptr, nullptr, e->l_act2, f, T, sp.shared_ff, sS));
        }
        {
          KL k(e, B2K_GEMM_DOWN);
          if (!k.skip()) B2_TRY(dense(e->l_act2, L.sh_down, e->l_ffd, T, W, sp.shared_ff, sS));
        }
        d1 = e->l_ffd;
      }
    }
    if (two) B2_TRY(join(e->l_ev[2], sB));
    if (has_ff) B2_TRY(join(e->l_ev[3], sF));
    if (shared_beside) B2_TRY(join(e->l_ev[5], sS));
    if (multi) b2_pdl_skip_next();
    {
      KL k(e, B2K_NORM);  // h += (mixer + ff); the next layer's norm output, unless the loop's input mix comes first
      const bool next_plain = r + 1 < e->runs.size() && !e->runs[r + 1].pass_start && e->skip_mask == 0;
      const float* gn = next_plain ? e->ll[e->runs[r + 1].layer].gain1 : nullptr;
      if (!k.skip())
        B2_TRY(launch_branch_add(e->l_h, e->l_mix, two ? L.out_gain_l : nullptr, two ? e->l_mix2 : nullptr, two ? L.out_gain_r : nullptr, two ? 0.5f : 1.0f, d1,
                                 yr, e->l_pair_slot, sp.top, T, W, c.rms_eps, st, gn, gn ? e->l_x1 : nullptr, f));
      have_norm = gn != nullptr;
    }
    dbg((int)r + 1);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_unit_norm2(e->l_h, e->l_final_gain, nullptr, e->l_xl, nullptr, f, nlast, W, c.rms_eps, ntiles > 0 ? e->d_last_rows : nullptr, st));
  }
  {
    KL k(e, B2K_LMHEAD);
    if (!k.skip()) B2_TRY(dense(e->l_xl, e->l_head, e->l_logits, nlast, c.vocab, W, st));
  }
  {
    KL k(e, B2K_MISC);
    bf16* lb = (e->debug_flags & 2) ? e->logits : nullptr;
    if (!k.skip()) {
      if (c.logit_softcap > 0.f) B2_TRY(launch_softcap(e->l_logits, (size_t)nlast * c.vocab, c.logit_softcap, st));
      B2_TRY(launch_logits_finish(e->l_logits, e->d_out_tokens, lb, bucket_batch(std::max(c.max_seqs, 1)), nlast, c.vocab, e->v_pad, st));
    }
  }
  return 0;
}

// Tinevik: h <- h + ln1b(mixer(ln1(h))), then h <- h + ln2b(ff(ln2(h))) on the same fp32 residual stream, every norm a layer norm with gain
// and bias.  The layers run in the order of e->runs; a run names the layer whose tensors it uses (a layer may borrow another's) and owns
// its cache regions or its state.  Three mixers, each behind ONE fused projection of the norm output: a matrix-state mixer with a decay
// per key channel (attn_state.cu over the sequence slots), softmax attention whose scores are mixed over the heads before the softmax
// (attn_heads.cu over the block table, K and V regions), and attention over a cached latent with a window and an output gate
// (attn_latent.cu, absorbed form, one region).  Feed-forwards: a dense one, or experts named by a table row per token id.
constexpr float TINEVIK_GATE_SHARP = 1.702f;   // expert: y = g * sigmoid(1.702 g) * (u + 1)

int forward_mixed_list(b2_engine* e, int T, int ntiles, int nlast) {
  const b2_config& c = e->cfg;
  const int W = c.hidden, f = e->f32 ? 1 : 0;
  cudaStream_t st = e->stream;
  auto dbg = [&](int slot) {
    if ((e->debug_flags & 1) && e->dbg_hidden_f32 != nullptr && T <= e->dbg_cap_tokens && slot < e->dbg_slots)
      cudaMemcpyAsync(e->dbg_hidden_f32 + (size_t)slot * e->dbg_cap_tokens * W, e->l_h, (size_t)T * W * 4, cudaMemcpyDeviceToDevice, st);
  };
  auto dense = [&](const void* A, const void* Wt, float* C, int M, int N, int K) -> int { return list_dense(e, A, Wt, C, M, N, K, 1.f, st); };
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed_scaled(e->d_tokens, e->l_embed, f, c.embed_scale != 0.f ? c.embed_scale : 1.f, e->l_h, T, W, c.vocab, st));
  }
  dbg(0);
  const PrefillTile* tiles = ntiles > 0 ? e->d_tiles : nullptr;
  const int portions = ntiles > 0 ? e->step_portions : T;
  const int32_t* last_rows = ntiles > 0 ? e->d_last_rows : nullptr;
  const bool use_tc = list_use_tc();
  bool have_norm = false;   // l_x1 already holds this run's first norm output (the run before wrote it)
  for (size_t r = 0; r < e->runs.size(); ++r) {
    const ListRun& R = e->runs[r];
    ListLayer& L = e->ll[R.layer];
    const b2_layer_spec& sp = L.sp;
    if (!have_norm) {
      KL k(e, B2K_NORM);
      if (!k.skip()) B2_TRY(launch_layer_norm(e->l_h, L.gain1, L.bias1, e->l_x1, f, T, W, c.rms_eps, nullptr, st));
    }
    {
      KL k(e, B2K_GEMM_QKV);   // everything that reads the norm output: one projection
      if (!k.skip()) B2_TRY(dense(e->l_x1, L.wqd, e->l_qd, T, L.nqd, W));
    }
    const int HV = sp.heads * sp.vdim;
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      const StateGeom sg{sp.heads, sp.heads, sp.dim, sp.vdim, STATE_RULE_DECAY};
      {
        KL k(e, B2K_ACT);   // decay per key channel: sigmoid(A2 (A1 n) + b)^(1 / tau)
        if (!k.skip()) B2_TRY(launch_lowrank_act(e->l_qd, L.nqd, L.n_fixed, L.rank_a, L.a2, L.a2_bias, LOWRANK_DECAY_SIGMOID_POW, 1.0f / sp.s_tau, nullptr, 0,
                                                 e->l_dec, T, sp.heads * sp.dim, st));
      }
      {
        KL k(e, B2K_CHAIN);
        if (!k.skip()) B2_TRY(launch_state_scan(e->l_qd + L.off_sq, L.nqd, e->l_qd + L.off_sk, L.nqd, e->l_qd + L.off_sv, L.nqd, e->l_dec, nullptr, sg,
                                                1.0f / sqrtf((float)sp.dim), R.state, portions, last_rows, e->d_row_seq, e->d_row_first, e->d_row_end,
                                                e->d_positions, e->d_slots, e->l_so, st));
      }
      {
        KL k(e, B2K_ACT);   // per-head RMS norm of the read-out, times silu(g)
        if (!k.skip()) B2_TRY(launch_state_out_gate(e->l_so, L.head_gain, e->l_qd + L.off_sg, L.nqd, 1, e->l_av, f, sp.heads, sp.vdim, c.rms_eps, T, st));
      }
    } else if (sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
      HeadsGeom g{sp.heads, sp.kv_heads, sp.dim, sp.vdim, sp.rot_dims, sp.rot_base, sp.scale, c.rms_eps, 0, 0, 0, 0.f, sp.window, 0, 0, 0};
      g.rot_factor = sp.rot_factor;
      g.rot_values = sp.rot_values;
      g.softcap = sp.softcap;
      char* kc = e->regions[R.k_region].base;
      char* vc = e->regions[R.v_region].base;
      {
        KL k(e, B2K_ROPE_KV);
        if (!k.skip()) B2_TRY(launch_heads_finish_halves(e->l_qd, L.nqd, g, L.qk_gain, L.qk_gain + sp.dim, e->d_positions, e->d_slots, e->l_q, kc, vc, f, T, st));
      }
      {
        KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
        if (!k.skip()) B2_TRY(launch_heads_attention_premix(e->l_q, kc, vc, f, g, sp.score_mix ? L.talk : nullptr, e->d_block_table, e->bt_stride, c.block_size,
                                                            tiles, ntiles, e->d_positions, e->d_seq_lens, e->l_av, f, T, st, e->l_attn_scratch,
                                                            e->l_attn_scratch_floats, c.max_model_len));
      }
    } else {   // B2_MIXER_GATED_LATENT
      const LatentGeom g{sp.heads, sp.dim, 0, sp.vdim, sp.kv_rank, 0, 0.f, sp.scale, c.rms_eps, sp.window};
      char* cache = e->regions[R.k_region].base;
      {
        KL k(e, B2K_ROPE_KV);   // both latents normed: the query's becomes an operand, the other the token's cache row
        if (!k.skip()) B2_TRY(launch_latent_pair_finish(e->l_qd, L.nqd, L.off_sq, sp.q_rank, L.off_sk, sp.kv_rank, L.latq_gain, L.lat_gain, c.rms_eps,
                                                        e->d_slots, e->l_x2, cache, f, T, st));
      }
      {
        KL k(e, B2K_GEMM_QKV);   // q of every head from its latent
        if (!k.skip()) {
          B2_TRY(dense(e->l_x2, L.uq, e->l_q, T, sp.heads * sp.dim, sp.q_rank));
          B2_TRY(launch_store_rows(e->l_q, e->l_qnope, f, sp.heads * sp.dim, 0, T, sp.heads * sp.dim, st));
        }
      }
      {
        KL k(e, B2K_GEMM_QKV);   // the query pulled through the key up-projection, all heads in one strided batch
        AnyGemm a;
        a.A = e->l_qnope; a.W = L.ukT; a.C = e->l_qabs; a.M = T; a.N = sp.kv_rank; a.K = sp.dim;
        a.lda = (long)sp.heads * sp.dim; a.ldw = sp.dim; a.ldc = (long)sp.heads * sp.kv_rank;
        a.a_bs = sp.dim; a.w_bs = (long)sp.kv_rank * sp.dim; a.c_bs = sp.kv_rank;
        if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, sp.heads, 0, st));
      }
      {
        KL k(e, ntiles > 0 ? B2K_MISC : B2K_ATTN_DECODE);
        if (!k.skip()) B2_TRY(launch_latent_attention(e->l_qabs, e->l_q, cache, f, g, e->d_block_table, e->bt_stride, c.block_size, tiles, ntiles, e->d_positions,
                                                      e->d_seq_lens, nullptr, e->l_olat, f, T, st, e->l_attn_scratch, e->l_attn_scratch_floats, c.max_model_len));
      }
      {
        KL k(e, B2K_GEMM_O);   // values of every head from the weighted latent (fp32 sums: the gate follows)
        AnyGemm a;
        a.A = e->l_olat; a.W = L.uv; a.C = e->l_so; a.M = T; a.N = sp.vdim; a.K = sp.kv_rank;
        a.lda = (long)sp.heads * sp.kv_rank; a.ldw = sp.kv_rank; a.ldc = (long)HV;
        a.a_bs = sp.kv_rank; a.w_bs = (long)sp.vdim * sp.kv_rank; a.c_bs = sp.vdim;
        if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, sp.heads, 0, st));
      }
      {
        KL k(e, B2K_ACT);
        if (!k.skip()) B2_TRY(launch_sigmoid_gate(e->l_so, e->l_qd + L.off_sg, L.nqd, e->l_av, f, T, HV, st));
      }
    }
    {
      KL k(e, B2K_GEMM_O);
      if (!k.skip()) B2_TRY(dense(e->l_av, L.wo, e->l_mix, T, W, HV));
    }
    const bool has_ff = sp.ff != B2_FF_NONE;
    const ListLayer* NL = r + 1 < e->runs.size() ? &e->ll[e->runs[r + 1].layer] : nullptr;
    const bool fuse_next = NL != nullptr && e->skip_mask == 0;
    {
      KL k(e, B2K_NORM);   // h += ln1b(mixer); the norm in front of the next sublayer in the same pass
      const float* wn = has_ff ? L.gain2 : (fuse_next ? NL->gain1 : nullptr);
      const float* bn = has_ff ? L.bias2 : (fuse_next ? NL->bias1 : nullptr);
      if (!k.skip()) B2_TRY(launch_layer_norm_add(e->l_h, e->l_mix, nullptr, 0, 1.f, L.gain1b, L.bias1b, T, W, c.rms_eps, st, wn, bn, wn ? e->l_x1 : nullptr, f));
      have_norm = !has_ff && fuse_next;
    }
    if (has_ff) {
      const float* wn = fuse_next ? NL->gain1 : nullptr;
      const float* bn = fuse_next ? NL->bias1 : nullptr;
      if (sp.ff == B2_FF_XIELU) {
        {
          KL k(e, B2K_GEMM_GATEUP);
          if (!k.skip()) B2_TRY(dense(e->l_x1, L.up, e->l_upf, T, sp.ff_dim, W));
        }
        {
          KL k(e, B2K_ACT);
          if (!k.skip()) B2_TRY(launch_xielu(e->l_upf, L.poly, e->l_act, f, (size_t)T * sp.ff_dim, st));
        }
        {
          KL k(e, B2K_GEMM_DOWN);
          if (!k.skip()) B2_TRY(dense(e->l_act, L.down, e->l_mix, T, W, sp.ff_dim));
        }
        {
          KL k(e, B2K_NORM);
          if (!k.skip()) B2_TRY(launch_layer_norm_add(e->l_h, e->l_mix, nullptr, 0, 1.f, L.gain2b, L.bias2b, T, W, c.rms_eps, st, wn, bn, wn ? e->l_x1 : nullptr, f));
        }
      } else {   // B2_FF_TABLE_EXPERTS
        const int F = sp.ff_dim, pairs = T * sp.top;
        {
          KL k(e, B2K_ACT);
          if (!k.skip()) B2_TRY(launch_route_table(e->d_tokens, L.table, c.vocab, sp.experts, sp.top, e->l_idx, e->l_rw, T, st));
        }
        {
          KL k(e, B2K_MISC);
          if (!k.skip()) B2_TRY(launch_route_permute(e->l_idx, T, sp.top, sp.experts, e->l_offsets, e->l_offsets_stride, e->l_slot_token, e->l_pair_slot, st));
        }
        // Prompt-sized bf16 steps run expert by expert on the tcgen05 projection kernel (rows gathered into expert order, the experts' slot
        // ranges read back: one small copy and a stream synchronisation per layer); everything else as ragged groups.
        const bool tc_experts = use_tc && !f && ntiles > 0 && e->l_xperm != nullptr && pairs >= LIST_TC_EXPERT_ROWS && W % 64 == 0 && F % 64 == 0 && W >= 128 &&
                                F >= 64 && e->skip_mask == 0;
        if (tc_experts) {
          B2_CUDA_OK(cudaMemcpyAsync(e->h_offsets, e->l_offsets, (size_t)(sp.experts + 1) * 4, cudaMemcpyDeviceToHost, st));
          {
            KL k(e, B2K_MISC);
            B2_TRY(launch_gather_rows((const bf16*)e->l_x1, e->l_slot_token, e->l_xperm, pairs, W, st));
          }
          B2_CUDA_OK(cudaStreamSynchronize(st));
          const int32_t* off = e->h_offsets;
          B2_REQUIRE(off[0] == 0 && off[sp.experts] == pairs, "layer %d: the experts' slot ranges do not cover the step's %d pairs", R.layer, pairs);
          {
            KL k(e, B2K_GEMM_GATEUP);
            for (int x = 0; x < sp.experts; ++x)
              if (off[x + 1] > off[x])
                B2_TRY(dense(e->l_xperm + (size_t)off[x] * W, (const bf16*)L.up + (size_t)x * 2 * F * W, e->l_upf + (size_t)off[x] * 2 * F, off[x + 1] - off[x],
                             2 * F, W));
          }
          {
            KL k(e, B2K_ACT);
            B2_TRY(launch_clamped_gate(e->l_upf, e->l_act, 0, pairs, F, sp.ff_limit, TINEVIK_GATE_SHARP, st));
          }
          {
            KL k(e, B2K_GEMM_DOWN);
            for (int x = 0; x < sp.experts; ++x)
              if (off[x + 1] > off[x])
                B2_TRY(dense((const bf16*)e->l_act + (size_t)off[x] * F, (const bf16*)L.down + (size_t)x * W * F, e->l_y + (size_t)off[x] * W,
                             off[x + 1] - off[x], W, F));
          }
        } else {
          const int max_tiles = std::min(e->l_tiles_cap, (pairs + any_gemm_tile_rows() - 1) / any_gemm_tile_rows() + sp.experts);
          if (pairs > any_gemm_ragged_rows_limit() || W > 16384 || 2 * F > 16384) {
            KL k(e, B2K_MISC);
            if (!k.skip()) B2_TRY(launch_ragged_tiles(e->l_offsets, sp.experts, e->l_tile_group, e->l_tile_row0, e->l_ntiles, max_tiles, st));
          }
          AnyGemm a;
          a.tile_group = e->l_tile_group; a.tile_row0 = e->l_tile_row0; a.n_tiles = e->l_ntiles; a.group_offsets = e->l_offsets;
          {
            KL k(e, B2K_GEMM_GATEUP);  // gate | up of every (token, choice) pair in expert order, fp32 sums
            a.A = e->l_x1; a.a_rows = e->l_slot_token; a.W = L.up; a.C = e->l_upf; a.N = 2 * F; a.K = W; a.lda = W; a.ldw = W; a.ldc = 2 * F;
            a.w_bs = (long)2 * F * W; a.epilogue = ANY_EPI_STORE;
            if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, 1, max_tiles, st, pairs, sp.experts));
          }
          {
            KL k(e, B2K_ACT);
            if (!k.skip()) B2_TRY(launch_clamped_gate(e->l_upf, e->l_act, f, pairs, F, sp.ff_limit, TINEVIK_GATE_SHARP, st));
          }
          {
            KL k(e, B2K_GEMM_DOWN);
            a.A = e->l_act; a.a_rows = nullptr; a.W = L.down; a.C = e->l_y; a.N = W; a.K = F; a.lda = F; a.ldw = F; a.ldc = W;
            a.w_bs = (long)W * F; a.epilogue = ANY_EPI_STORE;
            if (!k.skip()) B2_TRY(launch_gemm_any(a, f, f, 1, 1, max_tiles, st, pairs, sp.experts));
          }
        }
        {
          KL k(e, B2K_NORM);   // h += ln2b(mean of the token's experts)
          if (!k.skip()) B2_TRY(launch_layer_norm_add(e->l_h, e->l_y, e->l_pair_slot, sp.top, 1.0f / (float)sp.top, L.gain2b, L.bias2b, T, W, c.rms_eps, st, wn, bn,
                                                      wn ? e->l_x1 : nullptr, f));
        }
      }
      have_norm = fuse_next;
    }
    dbg((int)r + 1);
  }
  {
    KL k(e, B2K_NORM);
    if (!k.skip()) B2_TRY(launch_layer_norm(e->l_h, e->l_final_gain, e->l_final_bias, e->l_xl, f, nlast, W, c.rms_eps, ntiles > 0 ? e->d_last_rows : nullptr, st));
  }
  {
    KL k(e, B2K_LMHEAD);
    if (!k.skip()) B2_TRY(list_dense(e, e->l_xl, e->l_head, e->l_logits, nlast, c.vocab, W, c.logit_scale != 0.f ? c.logit_scale : 1.f, st));
  }
  {
    KL k(e, B2K_MISC);
    bf16* lb = (e->debug_flags & 2) ? e->logits : nullptr;
    if (!k.skip()) B2_TRY(launch_logits_finish(e->l_logits, e->d_out_tokens, lb, bucket_batch(std::max(c.max_seqs, 1)), nlast, c.vocab, e->v_pad, st));
  }
  return 0;
}

// Two-lane decode.  At batch 64 a decode step is two things that do not overlap when they depend on each other: the
// attention pass of a layer (HBM-bound, about half the step) and the eight small kernels between two attention
// passes (a chain of dependent launches that moves 31 MB of weights in ~30 us: latency-bound, HBM nearly idle).
// Sequences are independent, so the batch is cut into two halves that run as two dependent chains on two streams of
// the same step (and the same captured graph): while one half is in its latency-bound chain the other half streams
// its K/V pages.  Both attention kernels want every SM (129 KB of shared memory per CTA), so they take turns by
// themselves and the halves fall into opposite phases; the projections of a lane use the short stage ring (<= 82 KB)
// so that their CTAs are resident NEXT to the other lane's attention CTAs instead of queueing behind them.  The price
// is that the weights are streamed once per lane (L2 keeps part of the second pass).
bool two_lane_decode(const b2_engine* e, int T, int ntiles) {
  return ntiles == 0 && e->mb_min_batch > 0 && T >= e->mb_min_batch && T <= 128 && T % 2 == 0 && e->stream2 != nullptr &&
         !e->profiling && !(e->debug_flags & 1) && e->force_gemm_impl != 0 && (T / 2) > e->simt_max_tokens;
}

int forward(b2_engine* e, int T, int ntiles, int nlast, int attn_split) {
  const b2_config& c = e->cfg;
  const int H = c.hidden;
  (void)attn_split;
  if (c.arch == B2_ARCH_LERASUN) return forward_list(e, T, ntiles, nlast);
  if (c.arch == B2_ARCH_KEDASUN) return forward_heads_list(e, T, ntiles, nlast);
  if (c.arch == B2_ARCH_BUMALIX) return forward_state_list(e, T, ntiles, nlast);
  if (c.arch == B2_ARCH_TINEVIK) return forward_mixed_list(e, T, ntiles, nlast);
  if (c.arch == B2_ARCH_OPT) return forward_opt(e, T, ntiles, nlast);
  if (ntiles == 0 && e->use_chain == 2 && e->fused_ok && c.arch == B2_ARCH_QWEN3 && !(e->debug_flags & 1) &&
      e->force_gemm_impl != 0 && T > e->simt_max_tokens && T <= 64 && e->skip_mask == 0)
    return forward_decode_fused(e, T);
  if (ntiles == 0 && e->use_chain == 1 && c.arch == B2_ARCH_QWEN3 && !(e->debug_flags & 1) && e->force_gemm_impl != 0 && T > e->simt_max_tokens)
    return forward_decode_chain(e, T);
  {
    KL k(e, B2K_EMBED);
    if (!k.skip()) B2_TRY(launch_embed(e->d_tokens, e->embed, e->h, T, H, c.vocab, e->d_argmax, nlast, e->stream));
  }
  dbg_capture(e, 0, e->h, T);
  if (two_lane_decode(e, T, ntiles)) {
    Lane a = whole_batch_lane(e), b;
    a.beside_attention = true;
    b.stream = e->stream2;
    b.row0 = T / 2;
    b.partial = e->partial2;
    b.partial_floats = e->partial2_floats;
    b.attn_scratch = e->attn_scratch2;
    b.beside_attention = true;
    // fork: lane b starts once the embedding is done (a full dependency: no programmatic edge across streams)
    B2_CUDA_OK(cudaEventRecord(e->ev_fork, e->stream));
    B2_CUDA_OK(cudaStreamWaitEvent(e->stream2, e->ev_fork, 0));
    b2_pdl_skip_next();
    int rc_b = forward_layers(e, b, T - T / 2, 0);
    int rc_a = forward_layers(e, a, T / 2, 0);
    // join (always, so that a capture in progress is left with both streams merged)
    cudaError_t j1 = cudaEventRecord(e->ev_join, e->stream2);
    cudaError_t j2 = cudaStreamWaitEvent(e->stream, e->ev_join, 0);
    B2_TRY(rc_a);
    B2_TRY(rc_b);
    B2_CUDA_OK(j1);
    B2_CUDA_OK(j2);
    b2_pdl_skip_next();  // the lm_head waits for both lanes in full
  } else {
    B2_TRY(forward_layers(e, whole_batch_lane(e), T, ntiles));
  }
  dbg_capture(e, c.num_layers, e->h, T);
  dbg_capture(e, c.num_layers + 1, e->x, T);

  // lm_head on the last position of every sequence + greedy argmax
  const bf16* xl = e->x;
  XBuf xb = XB_X;
  if (ntiles > 0) {
    KL k(e, B2K_MISC);
    if (!k.skip()) B2_TRY(launch_gather_rows(e->x, e->d_last_rows, e->xlast, nlast, H, e->stream));
    xl = e->xlast;
    xb = XB_LAST;
  }
  return lm_head_and_argmax(e, nlast, xl, xb);
}

int lm_head_and_argmax(b2_engine* e, int nlast, const bf16* xl, XBuf xb) {
  const b2_config& c = e->cfg;
  const int H = c.hidden;
  bf16* logits = (e->debug_flags & 2) ? e->logits : nullptr;
  int impl = e->force_gemm_impl >= 0 ? e->force_gemm_impl : (nlast <= e->simt_max_tokens ? 0 : 1);
  if (impl == 0) {
    if (e->logits == nullptr) {
      b2_set_error("SIMT lm_head path needs the logits buffer (b2_set_debug(e, 2))");
      return -22;
    }
    {
      KL k(e, B2K_LMHEAD);
      if (!k.skip()) B2_TRY(launch_linear_simt(xl, e->lm_head, e->logits, 0, nlast, c.vocab, H, e->stream));
    }
    KL k2(e, B2K_MISC);
    if (!k2.skip()) B2_TRY(launch_argmax_rows(e->logits, e->d_out_tokens, nlast, c.vocab, e->stream));
  } else {
    TcGemmArgs a;
    // operands trade places for the fused arg-max: tokens on MMA-M (128-row box of X), 128 vocabulary
    // rows per tile on MMA-N
    a.bn = 128;
    a.tmap_w = e->tm_x[xb][bn_index(128)];
    a.tmap_x = e->tm_lm_head;
    a.T = nlast; a.N = c.vocab; a.K = H;
    a.nsplit = 1;
    a.epilogue = TC_EPI_ARGMAX_ROWS;
    a.out = logits;
    a.argmax_packed = e->d_argmax;
    {
      KL k(e, B2K_LMHEAD);
      if (!k.skip()) B2_TRY(launch_linear_tc(a, e->stream));
    }
    KL k2(e, B2K_MISC);
    if (!k2.skip()) B2_TRY(launch_argmax_finalize(e->d_argmax, e->d_out_tokens, nlast, e->stream));
  }
  return 0;
}

__global__ void publish_tokens_kernel(const int32_t* __restrict__ out_tokens, int32_t* __restrict__ next_in,
                                      int32_t* __restrict__ log, int32_t* step, int B, int log_cap_steps, int stride) {
  pdl_wait();
  pdl_launch_dependents();
  const int st = *step;  // single CTA
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    next_in[b] = out_tokens[b];
    // the log has `stride` (= max_seqs) columns; B is the padded bucket and may be wider
    if (st < log_cap_steps && b < stride) log[(size_t)st * stride + b] = out_tokens[b];
  }
  __syncthreads();
  if (threadIdx.x == 0) *step = st < 0x7fffffff ? st + 1 : st;  // saturates: a server steps for weeks without b2_decode_run resetting it
}

// decode step body recorded into a graph (or run eagerly): bookkeeping, forward, token feedback
int decode_body(b2_engine* e, int B, int attn_split) {
  {
    KL k(e, B2K_MISC);
    if (!k.skip()) B2_TRY(launch_decode_advance(e->d_positions, e->d_seq_lens, e->d_slots, e->d_block_table, e->bt_stride,
                                 e->cfg.block_size, B, e->d_pf_frac, e->kv_l2_budget,
                                 (long long)e->nkv * e->cfg.block_size * e->hd * 2 * 2, e->stream));
  }
  B2_TRY(forward(e, B, 0, B, attn_split));
  {
    KL k(e, B2K_MISC);
    if (!k.skip()) B2_CUDA_OK(b2_launch(publish_tokens_kernel, dim3(1), dim3(256), 0, e->stream, (const int32_t*)e->d_out_tokens, e->d_tokens,
                         e->d_token_log, e->d_step, B, e->log_cap_steps, e->cfg.max_seqs));
  }
  return 0;
}

// Captures (once per (batch bucket, attention split)) the decode step as a CUDA graph.  Capture
// does not advance any state: the eager warm-up that precedes it runs on saved bookkeeping.
int ensure_graph(b2_engine* e, int B, int attn_split) {
  GraphKey key{B, attn_split};
  if (e->graphs.count(key)) return 0;
  // Warm every kernel once outside capture (function attributes, module load), then restore the
  // bookkeeping so the real state is not advanced twice.  (The warm-up writes K/V for position
  // pos+1 with the same values the real step will write.)
  std::vector<int32_t> save(3 * (size_t)B + 1);
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  B2_CUDA_OK(cudaMemcpy(save.data(), e->d_positions, B * 4, cudaMemcpyDeviceToHost));
  B2_CUDA_OK(cudaMemcpy(save.data() + B, e->d_seq_lens, B * 4, cudaMemcpyDeviceToHost));
  B2_CUDA_OK(cudaMemcpy(save.data() + 2 * B, e->d_tokens, B * 4, cudaMemcpyDeviceToHost));
  B2_CUDA_OK(cudaMemcpy(save.data() + 3 * B, e->d_step, 4, cudaMemcpyDeviceToHost));
  const int64_t l0 = e->launches;
  B2_TRY(decode_body(e, B, attn_split));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  const int64_t nodes = e->launches - l0;
  e->launches = l0;
  B2_CUDA_OK(cudaMemcpy(e->d_positions, save.data(), B * 4, cudaMemcpyHostToDevice));
  B2_CUDA_OK(cudaMemcpy(e->d_seq_lens, save.data() + B, B * 4, cudaMemcpyHostToDevice));
  B2_CUDA_OK(cudaMemcpy(e->d_tokens, save.data() + 2 * B, B * 4, cudaMemcpyHostToDevice));
  B2_CUDA_OK(cudaMemcpy(e->d_step, save.data() + 3 * B, 4, cudaMemcpyHostToDevice));
  cudaGraph_t g = nullptr;
  B2_CUDA_OK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
  int rc = decode_body(e, B, attn_split);
  cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
  e->launches = l0;
  if (rc != 0) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  B2_CUDA_OK(ce);
  cudaGraphExec_t ge = nullptr;
  B2_CUDA_OK(cudaGraphInstantiate(&ge, g, 0));
  cudaGraphDestroy(g);
  e->graphs[key] = ge;
  e->graph_nodes[key] = nodes;
  return 0;
}

// hidden-state capture needs eager launches; the logits buffer is just another kernel argument, so it
// only selects a different graph (attn_split slot of the key: 1 = argmax only, 2 = logits written too)
bool graphs_enabled(b2_engine* e) { return e->cfg.use_cuda_graphs && !e->profiling && !(e->debug_flags & 1); }

int run_decode_step(b2_engine* e, int B, int attn_split) {
  if (!graphs_enabled(e)) return decode_body(e, B, attn_split);
  B2_TRY(ensure_graph(e, B, attn_split));
  GraphKey key{B, attn_split};
  B2_CUDA_OK(cudaGraphLaunch(e->graphs[key], e->stream));
  e->launches += e->graph_nodes[key];
  return 0;
}

// Uploads the batch state of `seq_ids` (decode slow path).  Device positions hold len-1 so the
// advance kernel at the head of the step brings them to the position of the appended token.
int upload_decode_batch(b2_engine* e, int n, const int32_t* seq_ids, int B) {
  const int bs = e->cfg.block_size;
  size_t need = (size_t)6 * B + (size_t)B * e->bt_stride;
  if (need > e->h_stage_ints) {
    b2_set_error("decode batch of %d does not fit the staging buffer", B);
    return -12;
  }
  int32_t* pos = e->h_stage;
  int32_t* lens = pos + B;
  int32_t* slots = lens + B;
  int32_t* bt = slots + B;
  memset(e->h_stage, 0, need * sizeof(int32_t));
  for (int i = 0; i < B; ++i) {
    if (i < n) {
      Seq& s = e->seqs[seq_ids[i]];
      pos[i] = s.len - 1;
      lens[i] = s.len;
      slots[i] = -1;
      memcpy(bt + (size_t)i * e->bt_stride, s.blocks.data(), s.blocks.size() * sizeof(int32_t));
    } else {  // padding rows of the graph bucket: no KV write, empty attention
      pos[i] = -2;  // sentinel: decode_advance leaves padding rows inert
      lens[i] = 0;
      slots[i] = -1;
    }
  }
  (void)bs;
  B2_CUDA_OK(cudaMemcpyAsync(e->d_positions, pos, B * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_seq_lens, lens, B * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_slots, slots, B * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_block_table, bt, (size_t)B * e->bt_stride * 4, cudaMemcpyHostToDevice, e->stream));
  if (e->d_row_seq) {  // every row is a portion of one token of its own sequence slot
    int32_t* rs = bt + (size_t)B * e->bt_stride;
    for (int i = 0; i < B; ++i) {
      rs[i] = i < n ? seq_ids[i] : 0;
      rs[B + i] = i;
      rs[2 * B + i] = i + 1;
    }
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_seq, rs, B * 4, cudaMemcpyHostToDevice, e->stream));
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_first, rs + B, B * 4, cudaMemcpyHostToDevice, e->stream));
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_end, rs + 2 * B, B * 4, cudaMemcpyHostToDevice, e->stream));
  }
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));  // staging buffer is reused
  e->cur_batch.assign(seq_ids, seq_ids + n);
  e->cur_B = B;
  return 0;
}

int check_seq(b2_engine* e, int id) {
  if (id < 0 || id >= (int)e->seqs.size() || !e->seqs[id].active) {
    b2_set_error("invalid sequence id %d", id);
    return -22;
  }
  return 0;
}

// ---- page allocator with the prefix cache in it ----
int64_t pages_available(const b2_engine* e) { return (int64_t)e->free_blocks.size() + (int64_t)e->pc_lru.size(); }

void pc_unregister(b2_engine* e, int32_t b) {
  if (e->blk_hash[b] == 0) return;
  auto it = e->pc_map.find(e->blk_hash[b]);
  if (it != e->pc_map.end() && it->second == b) e->pc_map.erase(it);
  e->blk_hash[b] = 0;
}

// a page for exclusive use: a free one, else the registered page that has gone unused the longest
int32_t take_page(b2_engine* e) {
  if (!e->free_blocks.empty()) {
    const int32_t b = e->free_blocks.back();
    e->free_blocks.pop_back();
    e->blk_ref[b] = 1;
    return b;
  }
  const int32_t b = e->pc_lru.front();
  e->pc_lru.pop_front();
  e->pc_in_lru[b] = 0;
  pc_unregister(e, b);
  e->blk_ref[b] = 1;
  return b;
}

void release_page(b2_engine* e, int32_t b) {
  if (--e->blk_ref[b] > 0) return;
  e->blk_ref[b] = 0;
  if (e->prefix_cache && e->blk_hash[b] != 0) {  // still worth something to a later prompt
    e->pc_lru.push_back(b);
    e->pc_lru_pos[b] = std::prev(e->pc_lru.end());
    e->pc_in_lru[b] = 1;
  } else {
    pc_unregister(e, b);
    e->free_blocks.push_back(b);
  }
}

uint64_t pc_hash(uint64_t parent, const int32_t* tok) {
  uint64_t h = parent ^ 0x9e3779b97f4a7c15ull;
  for (int i = 0; i < 16; ++i) {
    h ^= (uint64_t)(uint32_t)tok[i] + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h *= 0xff51afd7ed558ccdull;
    h ^= h >> 33;
  }
  return h ? h : 1;  // 0 means "not registered"
}

// Leading pages of a fresh sequence's prompt that are already in the cache: the sequence drops its own pages for them
// and holds the cached ones.  At least one token is always left to compute (its logits are the call's result).
int pc_match(b2_engine* e, Seq& s, const int32_t* ids, int n) {
  const int bs = e->cfg.block_size;
  int matched = 0;
  uint64_t h = 0;
  int32_t parent = -1;
  const int max_pages = (n - 1) / bs;
  for (int j = 0; j < max_pages; ++j) {
    h = pc_hash(h, ids + (size_t)j * bs);
    auto it = e->pc_map.find(h);
    if (it == e->pc_map.end()) break;
    const int32_t b = it->second;
    if (e->blk_parent[b] != parent || memcmp(&e->blk_tokens[(size_t)b * bs], ids + (size_t)j * bs, bs * sizeof(int32_t)) != 0) break;
    if (e->blk_ref[b] == 0 && e->pc_in_lru[b]) {
      e->pc_lru.erase(e->pc_lru_pos[b]);
      e->pc_in_lru[b] = 0;
    }
    e->blk_ref[b] += 1;
    release_page(e, s.blocks[j]);  // the private page reserved for these positions is not needed
    s.blocks[j] = b;
    s.chain.push_back(h);
    parent = b;
    matched += bs;
  }
  return matched;
}

// After a prefill call: pages of this sequence that the call's tokens completed get registered.
void pc_register(b2_engine* e, Seq& s, const int32_t* ids, int n) {
  const int bs = e->cfg.block_size;
  if (!s.chain_open) return;
  for (int i = 0; i < n; ++i) {
    s.pending.push_back(ids[i]);
    if ((int)s.pending.size() < bs) continue;
    const int j = (int)s.chain.size();
    const uint64_t h = pc_hash(j > 0 ? s.chain[j - 1] : 0, s.pending.data());
    const int32_t b = s.blocks[j];
    if (e->blk_hash[b] == 0 && e->pc_map.find(h) == e->pc_map.end()) {
      e->blk_hash[b] = h;
      e->blk_parent[b] = j > 0 ? s.blocks[j - 1] : -1;
      // the parent must itself be the registered holder of its hash, or a later match could not verify the chain
      if (j > 0 && (e->blk_hash[s.blocks[j - 1]] != s.chain[j - 1])) e->blk_hash[b] = 0;
      if (e->blk_hash[b] != 0) {
        memcpy(&e->blk_tokens[(size_t)b * bs], s.pending.data(), bs * sizeof(int32_t));
        e->pc_map[h] = b;
      }
    }
    s.chain.push_back(h);
    s.pending.clear();
  }
}

int ensure_logits(b2_engine* e) {
  if (e->logits) return 0;
  // rows for the padded graph bucket: a captured step runs the lm_head over bucket_batch(n) rows, and max_seqs need
  // not be a bucket value (--max-num-seqs is free-form)
  return dalloc(&e->logits, (size_t)bucket_batch(std::max(e->cfg.max_seqs, 1)) * (e->v_pad > 0 ? e->v_pad : e->cfg.vocab));
}

// ---- layer-list families: tensors by name ----
// Uploads n bf16 values as operand elements (bf16 as they are, or widened to fp32 -- exact) at element offset `off` of dst.
int put_operand(b2_engine* e, void* dst, size_t off, const uint16_t* src, size_t n) {
  if (!e->f32) {
    B2_CUDA_OK(cudaMemcpy(reinterpret_cast<uint16_t*>(dst) + off, src, n * 2, cudaMemcpyHostToDevice));
    return 0;
  }
  std::vector<uint32_t> wide(n);
  for (size_t i = 0; i < n; ++i) wide[i] = (uint32_t)src[i] << 16;
  B2_CUDA_OK(cudaMemcpy(reinterpret_cast<uint32_t*>(dst) + off, wide.data(), n * 4, cudaMemcpyHostToDevice));
  return 0;
}
// fp32 copy of n bf16 values, plus `add` (a gain stored around zero becomes 1 + g)
int put_f32(float* dst, const uint16_t* src, size_t n, float add) {
  std::vector<float> v(n);
  for (size_t i = 0; i < n; ++i) {
    const uint32_t u = (uint32_t)src[i] << 16;
    float f;
    memcpy(&f, &u, 4);
    v[i] = f + add;
  }
  B2_CUDA_OK(cudaMemcpy(dst, v.data(), n * 4, cudaMemcpyHostToDevice));
  return 0;
}

int list_tensor(b2_engine* e, const std::string& name, const void* host, size_t nbytes) {
  const b2_config& c = e->cfg;
  const size_t W = c.hidden;
  const uint16_t* src = reinterpret_cast<const uint16_t*>(host);
  auto want = [&](size_t elems) -> int {
    if (nbytes != elems * 2) {
      b2_set_error("tensor %s: expected %zu bytes, got %zu", name.c_str(), elems * 2, nbytes);
      return -22;
    }
    return 0;
  };
  auto done = [&](int rc) {
    if (rc == 0) e->loaded[name] = 1;
    return rc;
  };
  if (name == "embed") { B2_TRY(want((size_t)c.vocab * W)); return done(put_operand(e, e->l_embed, 0, src, (size_t)c.vocab * W)); }
  if (name == "head" && e->l_head != e->l_embed) { B2_TRY(want((size_t)c.vocab * W)); return done(put_operand(e, e->l_head, 0, src, (size_t)c.vocab * W)); }
  if (name == "embed.norm") { B2_TRY(want(W)); return done(put_f32(e->l_embed_gain, src, W, 1.0f)); }
  if (name == "final.norm") { B2_TRY(want(W)); return done(put_f32(e->l_final_gain, src, W, c.arch == B2_ARCH_LERASUN ? 1.0f : 0.0f)); }
  if (name == "final.norm.b" && e->l_final_bias) { B2_TRY(want(W)); return done(put_f32(e->l_final_bias, src, W, 0.0f)); }
  if (c.arch == B2_ARCH_BUMALIX && name == "loop.in") {   // (a checkpoint may carry it although the config loops over nothing: nothing then uses it)
    B2_TRY(want(W * 2 * W));
    return done(e->l_loop_in ? put_operand(e, e->l_loop_in, 0, src, W * 2 * W) : 0);
  }
  size_t dot = name.find('.');
  if (name.size() < 3 || name[0] != 'l' || dot == std::string::npos || dot < 2) {
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  const int li = atoi(name.substr(1, dot - 1).c_str());
  if (li < 0 || li >= c.num_layers) {
    b2_set_error("tensor %s: layer out of range", name.c_str());
    return -22;
  }
  ListLayer& L = e->ll[li];
  const b2_layer_spec& sp = L.sp;
  const std::string rest = name.substr(dot + 1);
  const size_t H = sp.heads, dn = sp.dim, dr = sp.rot_dim, dv = sp.vdim, r = sp.kv_rank, ff = sp.ff_dim;
  if (c.arch == B2_ARCH_BUMALIX) {
    const bool two = sp.mixer == B2_MIXER_WINDOW_AND_STATE;
    // a tensor whose size the config does not give: the number of values decides (a fresh fp32 copy on the device)
    auto any_f32 = [&](float** dst, size_t* floats) -> int {
      B2_REQUIRE(nbytes >= 2 && nbytes % 2 == 0, "tensor %s: %zu bytes", name.c_str(), nbytes);
      if (*dst) cudaFree(*dst);
      *dst = nullptr;
      B2_TRY(dalloc(dst, nbytes / 2));
      *floats = nbytes / 2;
      e->weight_bytes += (int64_t)(nbytes * 2);
      return put_f32(*dst, src, nbytes / 2, 0.0f);
    };
    auto low_rank = [&](std::vector<uint16_t>* host, int* rank) -> int {   // [rank][W], rank from the size
      B2_REQUIRE(nbytes >= 2 * W && nbytes % (2 * W) == 0, "tensor %s: %zu bytes are not rows of %zu values", name.c_str(), nbytes, W);
      B2_REQUIRE(L.nqd == L.n_fixed, "tensor %s: the layer's projection is already joined", name.c_str());
      host->assign(src, src + nbytes / 2);
      *rank = (int)(nbytes / (2 * W));
      return 0;
    };
    if (rest == "norm1") { B2_TRY(want(W)); return done(put_f32(L.gain1, src, W, 0.0f)); }
    if (two) {
      const size_t nq = L.nq, nk = L.nk, nv = L.nv, sh = sp.s_heads, sd = sp.s_dim, sv = sp.s_vdim;
      if (rest == "mix.left.q") { B2_TRY(want(nq * W)); return done(put_operand(e, L.wqd, 0, src, nq * W)); }
      if (rest == "mix.left.k") { B2_TRY(want(nk * W)); return done(put_operand(e, L.wqd, nq * W, src, nk * W)); }
      if (rest == "mix.left.v") { B2_TRY(want(nv * W)); return done(put_operand(e, L.wqd, (nq + nk) * W, src, nv * W)); }
      if (rest == "mix.left.q.b") { B2_TRY(want(nq)); return done(put_f32(L.qkv_bias, src, nq, 0.0f)); }
      if (rest == "mix.left.k.b") { B2_TRY(want(nk)); return done(put_f32(L.qkv_bias + nq, src, nk, 0.0f)); }
      if (rest == "mix.left.v.b") { B2_TRY(want(nv)); return done(put_f32(L.qkv_bias + nq + nk, src, nv, 0.0f)); }
      if (rest == "mix.left.q.norm") { B2_TRY(want(nq)); return done(put_f32(L.qk_gain, src, nq, 0.0f)); }
      if (rest == "mix.left.k.norm") { B2_TRY(want(nk)); return done(put_f32(L.qk_gain + nq, src, nk, 0.0f)); }
      if (rest == "mix.left.o") { B2_TRY(want(W * H * dv)); return done(put_operand(e, L.wo, 0, src, W * H * dv)); }
      if (rest == "mix.left.out") { B2_TRY(want(W)); return done(put_f32(L.out_gain_l, src, W, 0.0f)); }
      if (rest == "mix.right.q") { B2_TRY(want(sh * sd * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sq * W, src, sh * sd * W)); }
      if (rest == "mix.right.k") { B2_TRY(want(sh * sd * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sk * W, src, sh * sd * W)); }
      if (rest == "mix.right.v") { B2_TRY(want(sh * sv * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sv * W, src, sh * sv * W)); }
      if (rest == "mix.right.g") { B2_TRY(want(sh * sv * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sg * W, src, sh * sv * W)); }
      if (rest == "mix.right.o") { B2_TRY(want(W * sh * sv)); return done(put_operand(e, L.wo2, 0, src, W * sh * sv)); }
      if (rest == "mix.right.norm") { B2_TRY(want(sv)); return done(put_f32(L.head_gain, src, sv, 0.0f)); }
      if (rest == "mix.right.a1") return done(low_rank(&L.a1_host, &L.rank_a));
      if (rest == "mix.right.a2") return done(any_f32(&L.a2, &L.a2_floats));
      if (rest == "mix.right.a2.b") { B2_TRY(want(sh * sd)); return done(put_f32(L.a2_bias, src, sh * sd, 0.0f)); }
      if (rest == "mix.right.out") { B2_TRY(want(W)); return done(put_f32(L.out_gain_r, src, W, 0.0f)); }
    } else {
      const size_t nqk = (size_t)sp.kv_heads * dn, nvv = H * dv, taps = sp.conv_taps;
      if (rest == "mix.q") { B2_TRY(want(nqk * W)); return done(put_operand(e, L.wqd, 0, src, nqk * W)); }
      if (rest == "mix.k") { B2_TRY(want(nqk * W)); return done(put_operand(e, L.wqd, nqk * W, src, nqk * W)); }
      if (rest == "mix.v") { B2_TRY(want(nvv * W)); return done(put_operand(e, L.wqd, 2 * nqk * W, src, nvv * W)); }
      if (rest == "mix.b") { B2_TRY(want(H * W)); return done(put_operand(e, L.wqd, (2 * nqk + nvv) * W, src, H * W)); }
      if (rest == "mix.q.conv") { B2_TRY(want(nqk * taps)); return done(put_f32(L.conv_w, src, nqk * taps, 0.0f)); }
      if (rest == "mix.k.conv") { B2_TRY(want(nqk * taps)); return done(put_f32(L.conv_w + nqk * taps, src, nqk * taps, 0.0f)); }
      if (rest == "mix.v.conv") { B2_TRY(want(nvv * taps)); return done(put_f32(L.conv_w + 2 * nqk * taps, src, nvv * taps, 0.0f)); }
      if (rest == "mix.A_log") { B2_TRY(want(H)); return done(put_f32(L.a_log, src, H, 0.0f)); }
      if (rest == "mix.norm") { B2_TRY(want(dv)); return done(put_f32(L.head_gain, src, dv, 0.0f)); }
      if (rest == "mix.a1") return done(low_rank(&L.a1_host, &L.rank_a));
      if (rest == "mix.a2") return done(any_f32(&L.a2, &L.a2_floats));
      if (rest == "mix.dt_bias") { B2_TRY(want(H * dn)); return done(put_f32(L.a2_bias, src, H * dn, 0.0f)); }
      if (rest == "mix.g1") return done(low_rank(&L.g1_host, &L.rank_g));
      if (rest == "mix.g2") return done(any_f32(&L.g2, &L.g2_floats));
      if (rest == "mix.o") { B2_TRY(want(W * nvv)); return done(put_operand(e, L.wo, 0, src, W * nvv)); }
    }
    if (sp.ff == B2_FF_POLYNORM) {
      if (rest == "mlp.up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, 0, src, ff * W)); }
      if (rest == "mlp.down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, 0, src, W * ff)); }
      if (rest == "mlp.act") { B2_TRY(want(4)); return done(put_f32(L.poly, src, 4, 0.0f)); }
    } else if (sp.ff == B2_FF_SCALED_GATED_EXPERTS) {
      const size_t sf = sp.shared_ff;
      if (rest == "mlp.router") { B2_TRY(want((size_t)sp.experts * W)); return done(put_f32(L.router, src, (size_t)sp.experts * W, 0.0f)); }
      if (sf > 0 && rest == "mlp.shared.gate") { B2_TRY(want(sf * W)); return done(put_operand(e, L.sh_up, 0, src, sf * W)); }
      if (sf > 0 && rest == "mlp.shared.up") { B2_TRY(want(sf * W)); return done(put_operand(e, L.sh_up, sf * W, src, sf * W)); }
      if (sf > 0 && rest == "mlp.shared.down") { B2_TRY(want(W * sf)); return done(put_operand(e, L.sh_down, 0, src, W * sf)); }
      if (rest.compare(0, 5, "mlp.e") == 0) {
        size_t d2 = rest.find('.', 5);
        if (d2 != std::string::npos) {
          const int ex = atoi(rest.substr(5, d2 - 5).c_str());
          const std::string which = rest.substr(d2 + 1);
          if (ex >= 0 && ex < sp.experts) {   // gate rows, then up rows, expert by expert: one product gives both
            if (which == "gate") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, (size_t)ex * 2 * ff * W, src, ff * W)); }
            if (which == "up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, ((size_t)ex * 2 + 1) * ff * W, src, ff * W)); }
            if (which == "down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, (size_t)ex * W * ff, src, W * ff)); }
          }
        }
      }
    }
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  if (c.arch == B2_ARCH_TINEVIK) {
    B2_REQUIRE(sp.weights_of < 0, "tensor %s: layer %d runs with layer %d's tensors and has none of its own", name.c_str(), li, sp.weights_of);
    const size_t HV = H * dv;
    if (rest == "norm1") { B2_TRY(want(W)); return done(put_f32(L.gain1, src, W, 0.0f)); }
    if (rest == "norm1.b") { B2_TRY(want(W)); return done(put_f32(L.bias1, src, W, 0.0f)); }
    if (rest == "norm1b") { B2_TRY(want(W)); return done(put_f32(L.gain1b, src, W, 0.0f)); }
    if (rest == "norm1b.b") { B2_TRY(want(W)); return done(put_f32(L.bias1b, src, W, 0.0f)); }
    if (sp.ff != B2_FF_NONE) {
      if (rest == "norm2") { B2_TRY(want(W)); return done(put_f32(L.gain2, src, W, 0.0f)); }
      if (rest == "norm2.b") { B2_TRY(want(W)); return done(put_f32(L.bias2, src, W, 0.0f)); }
      if (rest == "norm2b") { B2_TRY(want(W)); return done(put_f32(L.gain2b, src, W, 0.0f)); }
      if (rest == "norm2b.b") { B2_TRY(want(W)); return done(put_f32(L.bias2b, src, W, 0.0f)); }
    }
    if (rest == "mix.o") { B2_TRY(want(W * HV)); return done(put_operand(e, L.wo, 0, src, W * HV)); }
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      if (rest == "mix.q") { B2_TRY(want(H * dn * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sq * W, src, H * dn * W)); }
      if (rest == "mix.k") { B2_TRY(want(H * dn * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sk * W, src, H * dn * W)); }
      if (rest == "mix.v") { B2_TRY(want(HV * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sv * W, src, HV * W)); }
      if (rest == "mix.g") { B2_TRY(want(HV * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sg * W, src, HV * W)); }
      if (rest == "mix.norm") { B2_TRY(want(dv)); return done(put_f32(L.head_gain, src, dv, 0.0f)); }
      if (rest == "mix.a2.b") { B2_TRY(want(H * dn)); return done(put_f32(L.a2_bias, src, H * dn, 0.0f)); }
      if (rest == "mix.a1") {   // [rank][W], the rank from the size: it joins the fused projection when the weights are finalised
        B2_REQUIRE(nbytes >= 2 * W && nbytes % (2 * W) == 0, "tensor %s: %zu bytes are not rows of %zu values", name.c_str(), nbytes, W);
        B2_REQUIRE(L.nqd == L.n_fixed, "tensor %s: the layer's projection is already joined", name.c_str());
        L.a1_host.assign(src, src + nbytes / 2);
        L.rank_a = (int)(nbytes / (2 * W));
        return done(0);
      }
      if (rest == "mix.a2") {
        B2_REQUIRE(nbytes >= 2 && nbytes % 2 == 0, "tensor %s: %zu bytes", name.c_str(), nbytes);
        if (L.a2) cudaFree(L.a2);
        L.a2 = nullptr;
        B2_TRY(dalloc(&L.a2, nbytes / 2));
        L.a2_floats = nbytes / 2;
        e->weight_bytes += (int64_t)(nbytes * 2);
        return done(put_f32(L.a2, src, nbytes / 2, 0.0f));
      }
    } else if (sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
      const size_t nq = L.nq, nk = L.nk, nv = L.nv;
      if (rest == "mix.q") { B2_TRY(want(nq * W)); return done(put_operand(e, L.wqd, 0, src, nq * W)); }
      if (rest == "mix.k") { B2_TRY(want(nk * W)); return done(put_operand(e, L.wqd, nq * W, src, nk * W)); }
      if (rest == "mix.v") { B2_TRY(want(nv * W)); return done(put_operand(e, L.wqd, (nq + nk) * W, src, nv * W)); }
      if (rest == "mix.q.norm") { B2_TRY(want(dn)); return done(put_f32(L.qk_gain, src, dn, 0.0f)); }
      if (rest == "mix.k.norm") { B2_TRY(want(dn)); return done(put_f32(L.qk_gain + dn, src, dn, 0.0f)); }
      if (rest == "mix.talk") { B2_TRY(want(H * H)); return done(put_f32(L.talk, src, H * H, 0.0f)); }
    } else {
      const size_t qr = sp.q_rank;
      if (rest == "mix.dq") { B2_TRY(want(qr * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sq * W, src, qr * W)); }
      if (rest == "mix.dkv") { B2_TRY(want(r * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sk * W, src, r * W)); }
      if (rest == "mix.g") { B2_TRY(want(HV * W)); return done(put_operand(e, L.wqd, (size_t)L.off_sg * W, src, HV * W)); }
      if (rest == "mix.dq.norm") { B2_TRY(want(qr)); return done(put_f32(L.latq_gain, src, qr, 0.0f)); }
      if (rest == "mix.dkv.norm") { B2_TRY(want(r)); return done(put_f32(L.lat_gain, src, r, 0.0f)); }
      if (rest == "mix.uq") { B2_TRY(want(H * dn * qr)); return done(put_operand(e, L.uq, 0, src, H * dn * qr)); }
      if (rest == "mix.uk") {  // stored [heads * dim][kv_rank]; kept per head as [kv_rank][dim], the layout the absorbed-query product reads
        B2_TRY(want(H * dn * r));
        std::vector<uint16_t> tr(H * dn * r);
        for (size_t a = 0; a < H; ++a)
          for (size_t d = 0; d < dn; ++d)
            for (size_t j = 0; j < r; ++j) tr[(a * r + j) * dn + d] = src[(a * dn + d) * r + j];
        return done(put_operand(e, L.ukT, 0, tr.data(), tr.size()));
      }
      if (rest == "mix.uv") { B2_TRY(want(HV * r)); return done(put_operand(e, L.uv, 0, src, HV * r)); }
    }
    if (sp.ff == B2_FF_XIELU) {
      if (rest == "mlp.up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, 0, src, ff * W)); }
      if (rest == "mlp.down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, 0, src, W * ff)); }
      if (rest == "mlp.act") { B2_TRY(want(2)); return done(put_f32(L.poly, src, 2, 0.0f)); }
    } else if (sp.ff == B2_FF_TABLE_EXPERTS && rest.compare(0, 5, "mlp.e") == 0) {
      size_t d2 = rest.find('.', 5);
      if (d2 != std::string::npos) {
        const int ex = atoi(rest.substr(5, d2 - 5).c_str());
        const std::string which = rest.substr(d2 + 1);
        if (ex >= 0 && ex < sp.experts) {   // gate rows, then up rows, expert by expert: one product gives both
          if (which == "gate") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, (size_t)ex * 2 * ff * W, src, ff * W)); }
          if (which == "up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, ((size_t)ex * 2 + 1) * ff * W, src, ff * W)); }
          if (which == "down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, (size_t)ex * W * ff, src, W * ff)); }
        }
      }
    }
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  if (c.arch == B2_ARCH_KEDASUN) {
    const size_t nq = L.nq, nk = L.nk, nv = L.nv, taps = sp.conv_taps;
    const bool conv = sp.mixer == B2_MIXER_CONV_ATTENTION;
    if (rest == "norm1") { B2_TRY(want(W)); return done(put_f32(L.gain1, src, W, 0.0f)); }
    if (rest == "norm1b") { B2_TRY(want(W)); return done(put_f32(L.gain1b, src, W, 0.0f)); }
    if (rest == "norm2" && L.gain2) { B2_TRY(want(W)); return done(put_f32(L.gain2, src, W, 0.0f)); }
    if (rest == "norm2b" && L.gain2b) { B2_TRY(want(W)); return done(put_f32(L.gain2b, src, W, 0.0f)); }
    if (rest == "mix.q") { B2_TRY(want(nq * W)); return done(put_operand(e, L.wqd, 0, src, nq * W)); }
    if (rest == "mix.k") { B2_TRY(want(nk * W)); return done(put_operand(e, L.wqd, nq * W, src, nk * W)); }
    if (rest == "mix.v") { B2_TRY(want(nv * W)); return done(put_operand(e, L.wqd, (nq + nk) * W, src, nv * W)); }
    if (rest == "mix.o") { B2_TRY(want(W * H * dv)); return done(put_operand(e, L.wo, 0, src, W * H * dv)); }
    if (rest == "mix.vmix") { B2_TRY(want(1)); return done(put_f32(L.vmix, src, 1, 0.0f)); }
    if (conv) {
      if (rest == "mix.g") { B2_TRY(want(H * W)); return done(put_operand(e, L.wqd, (nq + nk + nv) * W, src, H * W)); }
      if (rest == "mix.q.b") { B2_TRY(want(nq)); return done(put_f32(L.qkv_bias, src, nq, 0.0f)); }
      if (rest == "mix.k.b") { B2_TRY(want(nk)); return done(put_f32(L.qkv_bias + nq, src, nk, 0.0f)); }
      if (rest == "mix.v.b") { B2_TRY(want(nv)); return done(put_f32(L.qkv_bias + nq + nk, src, nv, 0.0f)); }
      if (rest == "mix.o.b") { B2_TRY(want(W)); return done(put_f32(L.o_bias, src, W, 0.0f)); }
      if (rest == "mix.q.conv") { B2_TRY(want(nq * taps)); return done(put_f32(L.conv_w, src, nq * taps, 0.0f)); }
      if (rest == "mix.k.conv") { B2_TRY(want(nk * taps)); return done(put_f32(L.conv_w + nq * taps, src, nk * taps, 0.0f)); }
      if (rest == "mix.v.conv") { B2_TRY(want(nv * taps)); return done(put_f32(L.conv_w + (nq + nk) * taps, src, nv * taps, 0.0f)); }
      if (rest == "mix.talk") { B2_TRY(want(H * H)); return done(put_f32(L.talk, src, H * H, 0.0f)); }
    }
    if (sp.ff == B2_FF_CLAMPED_GATED) {
      if (rest == "mlp.gate") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, 0, src, ff * W)); }
      if (rest == "mlp.up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, ff * W, src, ff * W)); }
      if (rest == "mlp.down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, 0, src, W * ff)); }
    }
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  if (rest == "norm1") { B2_TRY(want(W)); return done(put_f32(L.gain1, src, W, 1.0f)); }
  if (rest == "norm2" && L.gain2) { B2_TRY(want(W)); return done(put_f32(L.gain2, src, W, 1.0f)); }
  if (rest == "mix.q") { B2_TRY(want((size_t)L.nq * W)); return done(put_operand(e, L.wqd, 0, src, (size_t)L.nq * W)); }
  if (rest == "mix.dkv" && sp.kv_from < 0) { B2_TRY(want((r + dr) * W)); return done(put_operand(e, L.wqd, (size_t)L.nq * W, src, (r + dr) * W)); }
  if (rest == "mix.dkv.norm" && sp.kv_from < 0) { B2_TRY(want(r)); return done(put_f32(L.lat_gain, src, r, 0.0f)); }
  if (rest == "mix.uk") {  // stored [heads * dim][kv_rank]; kept per head as [kv_rank][dim], the layout the absorbed-query product reads
    B2_TRY(want(H * dn * r));
    std::vector<uint16_t> tr(H * dn * r);
    for (size_t a = 0; a < H; ++a)
      for (size_t d = 0; d < dn; ++d)
        for (size_t j = 0; j < r; ++j) tr[(a * r + j) * dn + d] = src[(a * dn + d) * r + j];
    return done(put_operand(e, L.ukT, 0, tr.data(), tr.size()));
  }
  if (rest == "mix.uv") { B2_TRY(want(H * dv * r)); return done(put_operand(e, L.uv, 0, src, H * dv * r)); }
  if (rest == "mix.sink") { B2_TRY(want(H)); return done(put_f32(L.sink, src, H, 0.0f)); }
  if (rest == "mix.o") { B2_TRY(want(W * H * dv)); return done(put_operand(e, L.wo, 0, src, W * H * dv)); }
  if (sp.ff == B2_FF_ROUTED_EXPERTS) {
    if (rest == "mlp.router") { B2_TRY(want((size_t)sp.experts * W)); return done(put_f32(L.router, src, (size_t)sp.experts * W, 0.0f)); }
    if (rest == "mlp.correction") { B2_TRY(want((size_t)sp.experts)); return done(put_f32(L.corr, src, (size_t)sp.experts, 0.0f)); }
    if (rest.compare(0, 5, "mlp.e") == 0) {
      size_t d2 = rest.find('.', 5);
      if (d2 != std::string::npos) {
        const int ex = atoi(rest.substr(5, d2 - 5).c_str());
        const std::string which = rest.substr(d2 + 1);
        if (ex >= 0 && ex < sp.experts && which == "up") { B2_TRY(want(ff * W)); return done(put_operand(e, L.up, (size_t)ex * ff * W, src, ff * W)); }
        if (ex >= 0 && ex < sp.experts && which == "down") { B2_TRY(want(W * ff)); return done(put_operand(e, L.down, (size_t)ex * W * ff, src, W * ff)); }
      }
    }
  }
  b2_set_error("unknown tensor name %s", name.c_str());
  return -22;
}

int list_tensor_count(const b2_engine* e) {
  if (e->cfg.arch == B2_ARCH_KEDASUN) {
    int n = 3;  // embed, head, final.norm
    for (const ListLayer& L : e->ll) {
      n += 2 + 4;                                               // norm1, norm1b; q, k, v, o (vmix is counted apart: only a blending layer needs it)
      if (L.sp.mixer == B2_MIXER_CONV_ATTENTION) n += 4 + 3 + 2;  // biases of q, k, v, o; their convolutions; talk, g
      if (L.sp.ff == B2_FF_CLAMPED_GATED) n += 2 + 3;           // norm2, norm2b; gate, up, down
    }
    return n;
  }
  int n = 4;
  for (const ListLayer& L : e->ll) {
    n += 1 + 5 + (L.sp.kv_from < 0 ? 2 : 0);  // norm1; q, uk, uv, sink, o; dkv, dkv.norm
    if (L.sp.ff == B2_FF_ROUTED_EXPERTS) n += 1 + 2 + 2 * L.sp.experts;  // norm2; router, correction; experts
  }
  return n;
}

// The same for the family whose mixers keep per-head keys and values (Kedasun).
int heads_engine_alloc(b2_engine* e) {
  const b2_config& c = e->cfg;
  const size_t W = c.hidden, es = e->esz;
  B2_REQUIRE(!e->specs.empty() && (int)e->specs.size() == c.num_layers, "Kedasun: layer_specs missing");
  B2_REQUIRE(c.hidden >= 1 && c.vocab >= 1 && c.num_layers >= 1, "Kedasun: bad sizes");
  const int groups = c.norm_groups > 0 ? c.norm_groups : 1;
  B2_REQUIRE(c.hidden % groups == 0, "Kedasun: width %d is not %d equal norm pieces", c.hidden, groups);
  auto xalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, std::max<size_t>(elems, 1) * es));
    *p = q;
    e->weight_bytes += (int64_t)(elems * es);
    return 0;
  };
  auto falloc = [&](float** p, size_t n) -> int {
    B2_TRY(dalloc(p, std::max<size_t>(n, 1)));
    B2_CUDA_OK(cudaMemset(*p, 0, std::max<size_t>(n, 1) * 4));
    e->weight_bytes += (int64_t)(n * 4);
    return 0;
  };
  e->weight_bytes = 0;
  B2_TRY(xalloc(&e->l_embed, (size_t)c.vocab * W));
  B2_TRY(xalloc(&e->l_head, (size_t)c.vocab * W));
  B2_TRY(falloc(&e->l_final_gain, W));
  e->ll.resize(c.num_layers);
  size_t max_nqd = 1, max_nq = 1, max_nv = 1, max_hv = 1, max_cross = 0, max_ff = 1, gqa_scratch = 0;
  int first_vmix = -1;
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    L.sp = e->specs[l];
    const b2_layer_spec& sp = L.sp;
    const bool conv = sp.mixer == B2_MIXER_CONV_ATTENTION;
    B2_REQUIRE(sp.mixer == B2_MIXER_ATTENTION || conv, "layer %d: mixer kind %d not built for this family", l, sp.mixer);
    B2_REQUIRE(sp.heads >= 1 && sp.kv_heads >= 1 && sp.heads % sp.kv_heads == 0 && sp.dim >= 1 && sp.vdim >= 1,
               "layer %d: bad mixer sizes (heads %d, kv_heads %d, dim %d, vdim %d)", l, sp.heads, sp.kv_heads, sp.dim, sp.vdim);
    B2_REQUIRE(sp.rot_dims >= 0 && sp.rot_dims <= sp.dim && sp.rot_dims % 2 == 0, "layer %d: rot dims %d must be even and <= dim %d", l, sp.rot_dims, sp.dim);
    B2_REQUIRE(!conv || sp.conv_taps >= 1, "layer %d: the convolution needs at least one tap", l);
    B2_REQUIRE(sp.window >= 0 && sp.keep_first >= 0, "layer %d: bad window", l);
    B2_REQUIRE(sp.ff == B2_FF_NONE || (sp.ff == B2_FF_CLAMPED_GATED && sp.ff_dim >= 1), "layer %d: feed-forward kind %d not built for this family", l, sp.ff);
    L.nq = sp.heads * sp.dim;
    L.nk = sp.kv_heads * sp.dim;
    L.nv = sp.kv_heads * sp.vdim;
    L.nqd = L.nq + L.nk + L.nv + (conv ? sp.heads : 0);
    if (sp.v_mix) {
      if (first_vmix < 0) first_vmix = l;
      B2_REQUIRE(e->specs[first_vmix].kv_heads == sp.kv_heads && e->specs[first_vmix].vdim == sp.vdim, "layer %d: value mixing needs the value sizes of layer %d", l, first_vmix);
      L.vmix_mode = first_vmix == l ? 1 : 2;
    }
    B2_TRY(xalloc(&L.wqd, (size_t)L.nqd * W));
    B2_TRY(xalloc(&L.wo, W * sp.heads * sp.vdim));
    B2_TRY(falloc(&L.gain1, W));
    B2_TRY(falloc(&L.gain1b, W));
    B2_TRY(falloc(&L.vmix, 1));
    if (conv) {
      const size_t C = (size_t)L.nq + L.nk + L.nv;
      B2_TRY(falloc(&L.qkv_bias, C));
      B2_TRY(falloc(&L.o_bias, W));
      B2_TRY(falloc(&L.conv_w, C * sp.conv_taps));
      B2_TRY(falloc(&L.talk, (size_t)sp.heads * sp.heads));
      B2_TRY(dalloc(&L.conv_ring, (size_t)c.max_seqs * sp.conv_taps * C));
      e->l_has_state = e->l_has_state || sp.conv_taps > 1;
      max_cross = std::max(max_cross, (size_t)sp.heads * L.nv);
    }
    if (sp.ff == B2_FF_CLAMPED_GATED) {
      B2_TRY(falloc(&L.gain2, W));
      B2_TRY(falloc(&L.gain2b, W));
      B2_TRY(xalloc(&L.up, (size_t)2 * sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, W * sp.ff_dim));
      max_ff = std::max(max_ff, (size_t)sp.ff_dim);
    }
    static const bool use_gqa_tc = [] { const char* v = getenv("B2_HEADS_GQA_TC"); return !(v && *v == '0'); }();
    L.gqa_tc = use_gqa_tc && !e->f32 && !conv && sp.dim == 128 && sp.vdim == 128 && sp.heads == 2 * sp.kv_heads && sp.window == 0 &&
               c.block_size == 16 && (c.max_model_len + 15) / 16 <= 1024 && (long)bucket_batch(c.max_seqs) * sp.kv_heads <= 4096;
    if (L.gqa_tc) gqa_scratch = std::max(gqa_scratch, attn_decode_scratch_floats(bucket_batch(c.max_seqs), sp.heads, sp.kv_heads, 128));
    max_nqd = std::max(max_nqd, (size_t)L.nqd);
    max_nq = std::max(max_nq, (size_t)L.nq);
    max_nv = std::max(max_nv, (size_t)L.nv);
    max_hv = std::max(max_hv, (size_t)sp.heads * sp.vdim);
  }
  e->cap_tokens = ((std::max(c.max_batch_tokens, c.max_seqs) + 255) / 256) * 256;
  const size_t Tc = e->cap_tokens;
  e->l_rows_cap = (int)(Tc + bucket_batch(c.max_seqs));
  e->l_max_top = 1;
  e->v_pad = (c.vocab + 7) / 8 * 8;
  auto aalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, elems * es));
    *p = q;
    return 0;
  };
  B2_TRY(dalloc(&e->l_h, Tc * W));
  B2_TRY(dalloc(&e->l_qd, Tc * max_nqd));
  B2_TRY(dalloc(&e->l_q, Tc * max_nq));
  B2_TRY(dalloc(&e->l_vfirst, Tc * max_nv));
  if (max_cross > 0) B2_TRY(dalloc(&e->l_cross, Tc * max_cross));
  if (gqa_scratch > 0) {
    B2_TRY(dalloc(&e->l_qb, Tc * max_nq));
    e->attn_scratch_floats = gqa_scratch;
    B2_TRY(dalloc(&e->attn_scratch, gqa_scratch));
    B2_CUDA_OK(cudaMemset(e->attn_scratch, 0, gqa_scratch * sizeof(float)));   // arrival counters start at zero
  }
  B2_TRY(dalloc(&e->l_mix, Tc * W));
  B2_TRY(dalloc(&e->l_y, Tc * 2 * max_ff));
  B2_TRY(dalloc(&e->l_logits, (size_t)e->l_rows_cap * c.vocab));
  B2_TRY(aalloc(&e->l_x1, Tc * W));
  B2_TRY(aalloc(&e->l_av, Tc * max_hv));
  B2_TRY(aalloc(&e->l_act, Tc * max_ff));
  B2_TRY(aalloc(&e->l_xl, (size_t)e->l_rows_cap * W));
  B2_TRY(dalloc(&e->d_row_seq, Tc));
  B2_TRY(dalloc(&e->d_row_first, Tc));
  B2_TRY(dalloc(&e->d_row_end, Tc));
  B2_CUDA_OK(cudaMemset(e->d_row_seq, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_first, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_end, 0, Tc * 4));
  return 0;
}

// The same for the family with matrix-state mixers and a layer loop (Bumalix).  The fused projection of a layer and the buffer its
// output goes to are sized when the weights are finalised (state_finalize): the low-rank widths come with the tensors.
int state_engine_alloc(b2_engine* e) {
  const b2_config& c = e->cfg;
  const size_t W = c.hidden, es = e->esz;
  B2_REQUIRE(!e->specs.empty() && (int)e->specs.size() == c.num_layers, "Bumalix: layer_specs missing");
  B2_REQUIRE(c.hidden >= 1 && c.vocab >= 1 && c.num_layers >= 1, "Bumalix: bad sizes");
  B2_REQUIRE(c.loop_times >= 0 && (c.loop_times == 0 || (c.loop_start >= 0 && c.loop_start <= c.loop_stop && c.loop_stop <= c.num_layers)),
             "Bumalix: loop [%d, %d) x %d outside the %d layers", c.loop_start, c.loop_stop, c.loop_times, c.num_layers);
  auto xalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, std::max<size_t>(elems, 1) * es));
    *p = q;
    e->weight_bytes += (int64_t)(elems * es);
    return 0;
  };
  auto falloc = [&](float** p, size_t n) -> int {
    B2_TRY(dalloc(p, std::max<size_t>(n, 1)));
    B2_CUDA_OK(cudaMemset(*p, 0, std::max<size_t>(n, 1) * 4));
    e->weight_bytes += (int64_t)(n * 4);
    return 0;
  };
  e->weight_bytes = 0;
  B2_TRY(xalloc(&e->l_embed, (size_t)c.vocab * W));
  B2_TRY(xalloc(&e->l_head, (size_t)c.vocab * W));
  B2_TRY(falloc(&e->l_final_gain, W));
  const bool looped = c.loop_times > 0 && c.loop_stop > c.loop_start;
  if (looped) B2_TRY(xalloc(&e->l_loop_in, W * 2 * W));
  e->ll.resize(c.num_layers);
  size_t max_q = 1, max_dec = 1, max_hv = 1, max_hv2 = 1, max_heads = 1, max_up = 1, max_act = 1, max_sff = 0, gqa_scratch = 0;
  int max_top = 1, max_exp = 1;
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    L.sp = e->specs[l];
    const b2_layer_spec& sp = L.sp;
    const bool two = sp.mixer == B2_MIXER_WINDOW_AND_STATE;
    B2_REQUIRE(two || sp.mixer == B2_MIXER_DELTA_STATE, "layer %d: mixer kind %d not built for this family", l, sp.mixer);
    B2_REQUIRE(sp.heads >= 1 && sp.kv_heads >= 1 && sp.heads % sp.kv_heads == 0 && sp.dim >= 1 && sp.vdim >= 1,
               "layer %d: bad mixer sizes (heads %d, kv_heads %d, dim %d, vdim %d)", l, sp.heads, sp.kv_heads, sp.dim, sp.vdim);
    B2_TRY(falloc(&L.gain1, W));
    if (two) {
      B2_REQUIRE(sp.s_heads >= 1 && sp.s_dim >= 1 && sp.s_dim <= 256 && sp.s_vdim >= 1 && sp.s_tau > 0.f && sp.window >= 0,
                 "layer %d: bad state-mixer sizes (heads %d, dim %d (at most 256), vdim %d, tau %g)", l, sp.s_heads, sp.s_dim, sp.s_vdim, (double)sp.s_tau);
      L.nq = sp.heads * sp.dim;
      L.nk = sp.kv_heads * sp.dim;
      L.nv = sp.kv_heads * sp.vdim;
      L.off_sq = L.nq + L.nk + L.nv;
      L.off_sk = L.off_sq + sp.s_heads * sp.s_dim;
      L.off_sv = L.off_sk + sp.s_heads * sp.s_dim;
      L.off_sg = L.off_sv + sp.s_heads * sp.s_vdim;
      L.n_fixed = L.off_sg + sp.s_heads * sp.s_vdim;
      B2_TRY(falloc(&L.qkv_bias, (size_t)L.off_sq));
      B2_TRY(falloc(&L.qk_gain, (size_t)L.nq + L.nk));
      B2_TRY(xalloc(&L.wo, W * sp.heads * sp.vdim));
      B2_TRY(xalloc(&L.wo2, W * sp.s_heads * sp.s_vdim));
      B2_TRY(falloc(&L.head_gain, sp.s_vdim));
      B2_TRY(falloc(&L.a2_bias, (size_t)sp.s_heads * sp.s_dim));
      B2_TRY(falloc(&L.out_gain_l, W));
      B2_TRY(falloc(&L.out_gain_r, W));
      static const bool use_gqa_tc = [] { const char* v = getenv("B2_HEADS_GQA_TC"); return !(v && *v == '0'); }();
      // the geometry the engine's GQA attention kernels are built for (they take a sliding window as an argument): such a layer keeps its
      // caches in their page layout and runs on them
      L.gqa_tc = use_gqa_tc && !e->f32 && sp.dim == 128 && sp.vdim == 128 && sp.heads == 2 * sp.kv_heads && c.block_size == 16 &&
                 (c.max_model_len + 15) / 16 <= 1024 && (long)bucket_batch(c.max_seqs) * sp.kv_heads <= 4096;
      if (L.gqa_tc) gqa_scratch = std::max(gqa_scratch, attn_decode_scratch_floats(bucket_batch(c.max_seqs), sp.heads, sp.kv_heads, 128));
      max_q = std::max(max_q, (size_t)L.nq);
      max_dec = std::max(max_dec, (size_t)sp.s_heads * sp.s_dim);
      max_hv = std::max({max_hv, (size_t)sp.heads * sp.vdim, (size_t)sp.s_heads * sp.s_vdim});
      max_hv2 = std::max(max_hv2, (size_t)sp.s_heads * sp.s_vdim);
      max_heads = std::max(max_heads, (size_t)sp.s_heads);
    } else {
      B2_REQUIRE(sp.conv_taps >= 1 && sp.dim <= 256, "layer %d: the delta rule needs at least one convolution tap and a key width of at most 256", l);
      const size_t nqk = (size_t)sp.kv_heads * sp.dim, C = 2 * nqk + (size_t)sp.heads * sp.vdim;
      L.n_fixed = (int)(C + sp.heads);
      B2_TRY(falloc(&L.conv_w, C * sp.conv_taps));
      B2_TRY(falloc(&L.a_log, sp.heads));
      B2_TRY(falloc(&L.head_gain, sp.vdim));
      B2_TRY(falloc(&L.a2_bias, (size_t)sp.heads * sp.dim));
      B2_TRY(xalloc(&L.wo, W * sp.heads * sp.vdim));
      max_q = std::max(max_q, C);
      max_dec = std::max(max_dec, (size_t)sp.heads * sp.dim);
      max_hv = std::max(max_hv, (size_t)sp.heads * sp.vdim);
      max_heads = std::max(max_heads, (size_t)sp.heads);
    }
    L.nqd = L.n_fixed;
    B2_TRY(xalloc(&L.wqd, (size_t)L.n_fixed * W));
    if (sp.ff == B2_FF_POLYNORM) {
      B2_REQUIRE(sp.ff_dim >= 1, "layer %d: bad feed-forward width", l);
      B2_TRY(xalloc(&L.up, (size_t)sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, W * sp.ff_dim));
      B2_TRY(falloc(&L.poly, 4));
      max_up = std::max(max_up, (size_t)sp.ff_dim);
      max_act = std::max(max_act, (size_t)sp.ff_dim);
    } else if (sp.ff == B2_FF_SCALED_GATED_EXPERTS) {
      B2_REQUIRE(sp.experts >= 1 && sp.top >= 1 && sp.top <= sp.experts && sp.ff_dim >= 1 && sp.shared_ff >= 0,
                 "layer %d: bad router sizes (experts %d, top %d, ff %d)", l, sp.experts, sp.top, sp.ff_dim);
      B2_TRY(falloc(&L.router, (size_t)sp.experts * W));
      B2_TRY(xalloc(&L.up, (size_t)sp.experts * 2 * sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, (size_t)sp.experts * W * sp.ff_dim));
      if (sp.shared_ff > 0) {
        B2_TRY(xalloc(&L.sh_up, (size_t)2 * sp.shared_ff * W));
        B2_TRY(xalloc(&L.sh_down, W * sp.shared_ff));
      }
      max_top = std::max(max_top, sp.top);
      max_exp = std::max(max_exp, sp.experts);
      max_up = std::max(max_up, (size_t)sp.top * 2 * sp.ff_dim);
      max_act = std::max(max_act, (size_t)sp.top * sp.ff_dim);
      max_sff = std::max(max_sff, (size_t)sp.shared_ff);
    } else {
      B2_REQUIRE(sp.ff == B2_FF_NONE, "layer %d: feed-forward kind %d not built for this family", l, sp.ff);
    }
  }
  // ---- the order the layers run in, and the state of every run ----
  auto add_run = [&](int layer, bool pass_start) -> int {
    ListRun R;
    R.layer = layer;
    R.pass_start = pass_start;
    const b2_layer_spec& sp = e->ll[layer].sp;
    const bool two = sp.mixer == B2_MIXER_WINDOW_AND_STATE;
    const StateGeom sg{two ? sp.s_heads : sp.heads, two ? sp.s_heads : sp.kv_heads, two ? sp.s_dim : sp.dim, two ? sp.s_vdim : sp.vdim, 0};
    const size_t sf = (size_t)c.max_seqs * state_floats_per_slot(sg);
    B2_TRY(dalloc(&R.state, sf));
    B2_CUDA_OK(cudaMemset(R.state, 0, sf * 4));
    if (!two && sp.conv_taps > 1) {
      const size_t rf = (size_t)c.max_seqs * sp.conv_taps * (2 * (size_t)sp.kv_heads * sp.dim + (size_t)sp.heads * sp.vdim);
      B2_TRY(dalloc(&R.ring, rf));
      B2_CUDA_OK(cudaMemset(R.ring, 0, rf * 4));
    }
    e->runs.push_back(R);
    return 0;
  };
  if (!looped) {
    for (int l = 0; l < c.num_layers; ++l) B2_TRY(add_run(l, false));
  } else {
    for (int l = 0; l < c.loop_start; ++l) B2_TRY(add_run(l, false));
    for (int t = 0; t < c.loop_times; ++t)
      for (int l = c.loop_start; l < c.loop_stop; ++l) B2_TRY(add_run(l, l == c.loop_start));
    for (int l = c.loop_stop; l < c.num_layers; ++l) B2_TRY(add_run(l, false));
  }
  e->l_has_state = true;
  e->dbg_slots = (int)e->runs.size() + 1;
  for (auto& sd : e->l_side) B2_CUDA_OK(cudaStreamCreateWithFlags(&sd, cudaStreamNonBlocking));
  for (auto& ev : e->l_ev) B2_CUDA_OK(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  // ---- activations ----
  e->cap_tokens = ((std::max(c.max_batch_tokens, c.max_seqs) + 255) / 256) * 256;
  const size_t Tc = e->cap_tokens;
  e->l_rows_cap = (int)(Tc + bucket_batch(c.max_seqs));
  e->l_max_top = max_top;
  e->v_pad = (c.vocab + 7) / 8 * 8;
  auto aalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, elems * es));
    *p = q;
    return 0;
  };
  B2_TRY(dalloc(&e->l_h, Tc * W));
  B2_TRY(dalloc(&e->l_q, Tc * max_q));
  if (gqa_scratch > 0) {
    B2_TRY(dalloc(&e->l_qb, Tc * max_q));
    e->attn_scratch_floats = gqa_scratch;
    B2_TRY(dalloc(&e->attn_scratch, gqa_scratch));
    B2_CUDA_OK(cudaMemset(e->attn_scratch, 0, gqa_scratch * sizeof(float)));   // arrival counters start at zero
  }
  B2_TRY(dalloc(&e->l_dec, Tc * max_dec));
  B2_TRY(dalloc(&e->l_beta, Tc * max_heads));
  B2_TRY(dalloc(&e->l_gate, Tc * max_hv));
  B2_TRY(dalloc(&e->l_so, Tc * max_hv));
  B2_TRY(dalloc(&e->l_mix, Tc * W));
  B2_TRY(dalloc(&e->l_mix2, Tc * W));
  B2_TRY(dalloc(&e->l_ffd, Tc * W));
  B2_TRY(dalloc(&e->l_y, Tc * max_top * W));
  B2_TRY(dalloc(&e->l_upf, Tc * max_up));
  B2_TRY(dalloc(&e->l_rw, Tc * max_top));
  B2_TRY(dalloc(&e->l_slot_scale, Tc * max_top));
  B2_TRY(dalloc(&e->l_logits, (size_t)e->l_rows_cap * c.vocab));
  B2_TRY(aalloc(&e->l_x1, Tc * W));
  if (looped) B2_TRY(aalloc(&e->l_cat, Tc * 2 * W));
  B2_TRY(aalloc(&e->l_av, Tc * max_hv));
  B2_TRY(aalloc(&e->l_av2, Tc * max_hv2));
  B2_TRY(aalloc(&e->l_act, Tc * max_act));
  if (max_sff > 0) {
    B2_TRY(dalloc(&e->l_upf2, Tc * 2 * max_sff));
    B2_TRY(aalloc(&e->l_act2, Tc * max_sff));
  }
  B2_TRY(aalloc(&e->l_xl, (size_t)e->l_rows_cap * W));
  B2_TRY(dalloc(&e->l_idx, Tc * max_top));
  e->l_offsets_stride = max_exp + 1;
  B2_TRY(dalloc(&e->l_offsets, (size_t)3 * (max_exp + 1)));
  B2_CUDA_OK(cudaMemset(e->l_offsets, 0, (size_t)3 * (max_exp + 1) * 4));
  B2_TRY(dalloc(&e->l_slot_token, Tc * max_top));
  B2_TRY(dalloc(&e->l_pair_slot, Tc * max_top));
  e->l_tiles_cap = (int)(Tc * max_top / any_gemm_tile_rows() + max_exp + 1);
  B2_TRY(dalloc(&e->l_tile_group, (size_t)e->l_tiles_cap));
  B2_TRY(dalloc(&e->l_tile_row0, (size_t)e->l_tiles_cap));
  B2_TRY(dalloc(&e->l_ntiles, (size_t)1));
  if (!e->f32 && Tc * max_top >= (size_t)LIST_TC_EXPERT_ROWS && max_exp > 1) {   // prompt-sized expert products on the tcgen05 projection kernel
    B2_TRY(dalloc(&e->l_xperm, Tc * max_top * W));
    B2_CUDA_OK(cudaMallocHost(&e->h_offsets, (size_t)(max_exp + 1) * sizeof(int32_t)));
  }
  B2_CUDA_OK(cudaMemset(e->l_ntiles, 0, 4));
  B2_CUDA_OK(cudaMemset(e->l_pair_slot, 0, Tc * max_top * 4));
  B2_CUDA_OK(cudaMemset(e->l_slot_scale, 0, Tc * max_top * 4));
  B2_TRY(dalloc(&e->d_row_seq, Tc));
  B2_TRY(dalloc(&e->d_row_first, Tc));
  B2_TRY(dalloc(&e->d_row_end, Tc));
  B2_CUDA_OK(cudaMemset(e->d_row_seq, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_first, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_end, 0, Tc * 4));
  return 0;
}

// Names of the tensors a Bumalix checkpoint must hold.
std::vector<std::string> state_tensor_names(const b2_engine* e) {
  std::vector<std::string> n = {"embed", "head", "final.norm"};
  if (e->l_loop_in) n.push_back("loop.in");
  for (size_t l = 0; l < e->ll.size(); ++l) {
    const b2_layer_spec& sp = e->ll[l].sp;
    const std::string p = "l" + std::to_string(l) + ".";
    n.push_back(p + "norm1");
    if (sp.mixer == B2_MIXER_WINDOW_AND_STATE) {
      for (const char* t : {"q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "o", "out"}) n.push_back(p + "mix.left." + t);
      for (const char* t : {"q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b", "out"}) n.push_back(p + "mix.right." + t);
    } else {
      for (const char* t : {"q", "k", "v", "q.conv", "k.conv", "v.conv", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o"}) n.push_back(p + "mix." + t);
    }
    if (sp.ff == B2_FF_POLYNORM) {
      for (const char* t : {"up", "down", "act"}) n.push_back(p + "mlp." + t);
    } else if (sp.ff == B2_FF_SCALED_GATED_EXPERTS) {
      n.push_back(p + "mlp.router");
      for (int x = 0; x < sp.experts; ++x)
        for (const char* t : {"gate", "up", "down"}) n.push_back(p + "mlp.e" + std::to_string(x) + "." + t);
      if (sp.shared_ff > 0)
        for (const char* t : {"gate", "up", "down"}) n.push_back(p + "mlp.shared." + t);
    }
  }
  return n;
}

// Every tensor is in: the low-rank first stages join the fused projections, and the buffer the projections write is sized.
int join_low_rank(b2_engine* e, ListLayer& L);
int state_finalize(b2_engine* e) {
  for (const std::string& name : state_tensor_names(e)) B2_REQUIRE(e->loaded.count(name), "weights incomplete: %s missing", name.c_str());
  size_t max_nqd = 1;
  for (size_t l = 0; l < e->ll.size(); ++l) {
    ListLayer& L = e->ll[l];
    const b2_layer_spec& sp = L.sp;
    const bool two = sp.mixer == B2_MIXER_WINDOW_AND_STATE;
    const size_t dec = two ? (size_t)sp.s_heads * sp.s_dim : (size_t)sp.heads * sp.dim;
    B2_REQUIRE(L.rank_a >= 1 && L.a2_floats == dec * L.rank_a, "layer %zu: a1 has %d rows, a2 %zu numbers for %zu channels", l, L.rank_a, L.a2_floats, dec);
    B2_REQUIRE(two || (L.rank_g >= 1 && L.g2_floats == (size_t)sp.heads * sp.vdim * L.rank_g), "layer %zu: g1 has %d rows, g2 %zu numbers", l, L.rank_g,
               L.g2_floats);
    B2_TRY(join_low_rank(e, L));
    max_nqd = std::max(max_nqd, (size_t)L.nqd);
  }
  if (e->l_qd == nullptr || max_nqd > e->l_qd_cols) {
    if (e->l_qd) cudaFree(e->l_qd);
    e->l_qd = nullptr;
    B2_TRY(dalloc(&e->l_qd, (size_t)e->cap_tokens * max_nqd));
    e->l_qd_cols = max_nqd;
  }
  return 0;
}

// Integer tensors of a checkpoint (int32): the table that names every token id's experts.
int list_int_tensor(b2_engine* e, const std::string& name, const int32_t* host, size_t count) {
  const b2_config& c = e->cfg;
  size_t dot = name.find('.');
  B2_REQUIRE(c.arch == B2_ARCH_TINEVIK && name.size() >= 3 && name[0] == 'l' && dot != std::string::npos && dot >= 2, "integer tensor %s: no model of this family has it",
             name.c_str());
  const int li = atoi(name.substr(1, dot - 1).c_str());
  B2_REQUIRE(li >= 0 && li < c.num_layers, "tensor %s: layer out of range", name.c_str());
  ListLayer& L = e->ll[li];
  B2_REQUIRE(name.substr(dot + 1) == "mlp.table" && L.sp.ff == B2_FF_TABLE_EXPERTS && L.table != nullptr, "unknown integer tensor %s", name.c_str());
  B2_REQUIRE(count == (size_t)c.vocab * L.sp.top, "tensor %s: expected %zu entries, got %zu", name.c_str(), (size_t)c.vocab * L.sp.top, count);
  for (size_t i = 0; i < count; ++i)
    B2_REQUIRE(host[i] >= 0 && host[i] < L.sp.experts, "tensor %s: entry %zu names expert %d of %d", name.c_str(), i, host[i], L.sp.experts);
  B2_CUDA_OK(cudaMemcpy(L.table, host, count * 4, cudaMemcpyHostToDevice));
  e->loaded[name] = 1;
  return 0;
}

// The low-rank first stages of a layer (their widths came with the tensors) join its fused projection behind the n_fixed rows whose count
// the config gives.
int join_low_rank(b2_engine* e, ListLayer& L) {
  const size_t W = e->cfg.hidden;
  if (L.nqd != L.n_fixed) return 0;   // (already joined: finalize may be called again after more tensors)
  const size_t rows = (size_t)L.n_fixed + L.rank_a + L.rank_g;
  char* fused = nullptr;
  B2_TRY(dalloc(&fused, rows * W * e->esz));
  B2_CUDA_OK(cudaMemcpy(fused, L.wqd, (size_t)L.n_fixed * W * e->esz, cudaMemcpyDeviceToDevice));
  B2_TRY(put_operand(e, fused, (size_t)L.n_fixed * W, L.a1_host.data(), L.a1_host.size()));
  if (L.rank_g > 0) B2_TRY(put_operand(e, fused, ((size_t)L.n_fixed + L.rank_a) * W, L.g1_host.data(), L.g1_host.size()));
  cudaFree(L.wqd);
  L.wqd = fused;
  L.nqd = (int)rows;
  e->weight_bytes += (int64_t)((rows - L.n_fixed) * W * e->esz);
  L.a1_host.clear();
  L.a1_host.shrink_to_fit();
  L.g1_host.clear();
  L.g1_host.shrink_to_fit();
  return 0;
}

// The same for the family whose layers mix three kinds of mixers and two kinds of feed-forwards, with layer norms around every sublayer and
// layers that run with another layer's tensors (Tinevik).
int mixed_engine_alloc(b2_engine* e) {
  const b2_config& c = e->cfg;
  const size_t W = c.hidden, es = e->esz;
  B2_REQUIRE(!e->specs.empty() && (int)e->specs.size() == c.num_layers, "Tinevik: layer_specs missing");
  B2_REQUIRE(c.hidden >= 1 && c.vocab >= 1 && c.num_layers >= 1, "Tinevik: bad sizes");
  auto xalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, std::max<size_t>(elems, 1) * es));
    *p = q;
    e->weight_bytes += (int64_t)(elems * es);
    return 0;
  };
  auto falloc = [&](float** p, size_t n) -> int {
    B2_TRY(dalloc(p, std::max<size_t>(n, 1)));
    B2_CUDA_OK(cudaMemset(*p, 0, std::max<size_t>(n, 1) * 4));
    e->weight_bytes += (int64_t)(n * 4);
    return 0;
  };
  e->weight_bytes = 0;
  B2_TRY(xalloc(&e->l_embed, (size_t)c.vocab * W));
  if (c.tie_embeddings) e->l_head = e->l_embed;   // the embedding table itself is the head
  else B2_TRY(xalloc(&e->l_head, (size_t)c.vocab * W));
  B2_TRY(falloc(&e->l_final_gain, W));
  B2_TRY(falloc(&e->l_final_bias, W));
  e->ll.resize(c.num_layers);
  size_t max_q = 1, max_dec = 1, max_hv = 1, max_up = 1, max_act = 1, max_qr = 1, max_hr = 1, max_hd = 1;
  int max_top = 1, max_exp = 1, max_heads = 1, max_rank = 1;
  bool any_latent = false, any_experts = false;
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    L.sp = e->specs[l];
    const b2_layer_spec& sp = L.sp;
    B2_REQUIRE(sp.mixer == B2_MIXER_DECAY_STATE || sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION || sp.mixer == B2_MIXER_GATED_LATENT,
               "layer %d: mixer kind %d not built for this family", l, sp.mixer);
    B2_REQUIRE(sp.heads >= 1 && sp.dim >= 1 && sp.vdim >= 1, "layer %d: bad mixer sizes (heads %d, dim %d, vdim %d)", l, sp.heads, sp.dim, sp.vdim);
    B2_REQUIRE(sp.ff == B2_FF_NONE || (sp.ff == B2_FF_XIELU && sp.ff_dim >= 1) ||
                   (sp.ff == B2_FF_TABLE_EXPERTS && sp.ff_dim >= 1 && sp.experts >= 1 && sp.top >= 1 && sp.top <= sp.experts),
               "layer %d: feed-forward kind %d (ff %d, experts %d, top %d) not built for this family", l, sp.ff, sp.ff_dim, sp.experts, sp.top);
    const size_t HV = (size_t)sp.heads * sp.vdim;
    max_hv = std::max(max_hv, HV);
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      B2_REQUIRE(sp.dim <= 256 && sp.s_tau > 0.f, "layer %d: a state mixer needs a key width of at most 256 (%d) and tau > 0 (%g)", l, sp.dim, (double)sp.s_tau);
      max_dec = std::max(max_dec, (size_t)sp.heads * sp.dim);
    } else if (sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
      B2_REQUIRE(sp.kv_heads >= 1 && sp.heads % sp.kv_heads == 0, "layer %d: %d heads over %d key/value heads", l, sp.heads, sp.kv_heads);
      B2_REQUIRE(sp.rot_dims >= 0 && sp.rot_dims <= sp.dim && sp.rot_dims % 2 == 0, "layer %d: rot dims %d must be even and <= dim %d", l, sp.rot_dims, sp.dim);
      B2_REQUIRE(!sp.rot_values || sp.vdim % 2 == 0, "layer %d: rotated values need an even vdim (%d)", l, sp.vdim);
      max_q = std::max(max_q, (size_t)sp.heads * sp.dim);
    } else {
      B2_REQUIRE(sp.kv_rank >= 1 && sp.q_rank >= 1 && sp.window >= 0, "layer %d: bad latent sizes (kv_rank %d, q_rank %d)", l, sp.kv_rank, sp.q_rank);
      any_latent = true;
      max_q = std::max(max_q, (size_t)sp.heads * sp.dim);
      max_hd = std::max(max_hd, (size_t)sp.heads * sp.dim);
      max_qr = std::max(max_qr, (size_t)sp.q_rank);
      max_hr = std::max(max_hr, (size_t)sp.heads * sp.kv_rank);
      max_heads = std::max(max_heads, sp.heads);
      max_rank = std::max(max_rank, sp.kv_rank);
    }
    if (sp.ff == B2_FF_XIELU) {
      max_up = std::max(max_up, (size_t)sp.ff_dim);
      max_act = std::max(max_act, (size_t)sp.ff_dim);
    } else if (sp.ff == B2_FF_TABLE_EXPERTS) {
      any_experts = true;
      max_top = std::max(max_top, sp.top);
      max_exp = std::max(max_exp, sp.experts);
      max_up = std::max(max_up, (size_t)sp.top * 2 * sp.ff_dim);
      max_act = std::max(max_act, (size_t)sp.top * sp.ff_dim);
    }
    if (sp.weights_of >= 0) {   // the layer runs with another layer's tensors: the same kinds and sizes, nothing of its own to hold
      int root = sp.weights_of;   // a named layer may itself run with another's tensors: follow the chain to the layer that owns them
      for (int hops = 0; root >= 0 && root < c.num_layers && e->specs[root].weights_of >= 0 && hops <= c.num_layers; ++hops) root = e->specs[root].weights_of;
      B2_REQUIRE(root >= 0 && root < c.num_layers && root != l && e->specs[root].weights_of < 0, "layer %d: weights_of %d must lead to a layer with tensors of its own", l,
                 sp.weights_of);
      e->specs[l].weights_of = L.sp.weights_of = root;
      const b2_layer_spec& o = e->specs[sp.weights_of];
      B2_REQUIRE(o.mixer == sp.mixer && o.heads == sp.heads && o.kv_heads == sp.kv_heads && o.dim == sp.dim && o.vdim == sp.vdim && o.kv_rank == sp.kv_rank &&
                     o.q_rank == sp.q_rank && o.ff == sp.ff && o.ff_dim == sp.ff_dim && o.experts == sp.experts && o.top == sp.top,
                 "layer %d: its sizes differ from those of layer %d whose tensors it uses", l, sp.weights_of);
      continue;
    }
    B2_TRY(falloc(&L.gain1, W));
    B2_TRY(falloc(&L.bias1, W));
    B2_TRY(falloc(&L.gain1b, W));
    B2_TRY(falloc(&L.bias1b, W));
    B2_TRY(xalloc(&L.wo, W * HV));
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      L.off_sq = 0;
      L.off_sk = sp.heads * sp.dim;
      L.off_sv = 2 * sp.heads * sp.dim;
      L.off_sg = L.off_sv + (int)HV;
      L.n_fixed = L.off_sg + (int)HV;
      B2_TRY(falloc(&L.head_gain, sp.vdim));
      B2_TRY(falloc(&L.a2_bias, (size_t)sp.heads * sp.dim));
    } else if (sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
      L.nq = sp.heads * sp.dim;
      L.nk = sp.kv_heads * sp.dim;
      L.nv = sp.kv_heads * sp.vdim;
      L.n_fixed = L.nq + L.nk + L.nv;
      B2_TRY(falloc(&L.qk_gain, (size_t)2 * sp.dim));
      B2_TRY(falloc(&L.talk, (size_t)sp.heads * sp.heads));
    } else {
      L.off_sq = 0;
      L.off_sk = sp.q_rank;
      L.off_sg = sp.q_rank + sp.kv_rank;
      L.n_fixed = L.off_sg + (int)HV;
      B2_TRY(falloc(&L.latq_gain, sp.q_rank));
      B2_TRY(falloc(&L.lat_gain, sp.kv_rank));
      B2_TRY(xalloc(&L.uq, (size_t)sp.heads * sp.dim * sp.q_rank));
      B2_TRY(xalloc(&L.ukT, (size_t)sp.heads * sp.kv_rank * sp.dim));
      B2_TRY(xalloc(&L.uv, HV * sp.kv_rank));
    }
    L.nqd = L.n_fixed;
    B2_TRY(xalloc(&L.wqd, (size_t)L.n_fixed * W));
    if (sp.ff != B2_FF_NONE) {
      B2_TRY(falloc(&L.gain2, W));
      B2_TRY(falloc(&L.bias2, W));
      B2_TRY(falloc(&L.gain2b, W));
      B2_TRY(falloc(&L.bias2b, W));
    }
    if (sp.ff == B2_FF_XIELU) {
      B2_TRY(xalloc(&L.up, (size_t)sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, W * sp.ff_dim));
      B2_TRY(falloc(&L.poly, 2));
    } else if (sp.ff == B2_FF_TABLE_EXPERTS) {
      B2_TRY(xalloc(&L.up, (size_t)sp.experts * 2 * sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, (size_t)sp.experts * W * sp.ff_dim));
      B2_TRY(dalloc(&L.table, (size_t)c.vocab * sp.top));
      B2_CUDA_OK(cudaMemset(L.table, 0, (size_t)c.vocab * sp.top * 4));
      e->weight_bytes += (int64_t)c.vocab * sp.top * 4;
    }
  }
  // ---- the runs: one per listed layer, with the layer whose tensors it uses and a state of its own ----
  for (int l = 0; l < c.num_layers; ++l) {
    ListRun R;
    R.layer = e->specs[l].weights_of >= 0 ? e->specs[l].weights_of : l;
    const b2_layer_spec& sp = e->ll[R.layer].sp;
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      const StateGeom sg{sp.heads, sp.heads, sp.dim, sp.vdim, 0};
      const size_t sf = (size_t)c.max_seqs * state_floats_per_slot(sg);
      B2_TRY(dalloc(&R.state, sf));
      B2_CUDA_OK(cudaMemset(R.state, 0, sf * 4));
      e->l_has_state = true;
    }
    e->runs.push_back(R);
  }
  e->dbg_slots = (int)e->runs.size() + 1;
  // ---- activations ----
  e->cap_tokens = ((std::max(c.max_batch_tokens, c.max_seqs) + 255) / 256) * 256;
  const size_t Tc = e->cap_tokens;
  e->l_rows_cap = (int)(Tc + bucket_batch(c.max_seqs));
  e->l_max_top = max_top;
  e->v_pad = (c.vocab + 7) / 8 * 8;
  auto aalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, elems * es));
    *p = q;
    return 0;
  };
  B2_TRY(dalloc(&e->l_h, Tc * W));
  B2_TRY(dalloc(&e->l_q, Tc * max_q));
  B2_TRY(dalloc(&e->l_dec, Tc * max_dec));
  B2_TRY(dalloc(&e->l_so, Tc * max_hv));
  B2_TRY(dalloc(&e->l_mix, Tc * W));
  B2_TRY(dalloc(&e->l_upf, Tc * max_up));
  B2_TRY(dalloc(&e->l_logits, (size_t)e->l_rows_cap * c.vocab));
  B2_TRY(aalloc(&e->l_x1, Tc * W));
  B2_TRY(aalloc(&e->l_av, Tc * max_hv));
  B2_TRY(aalloc(&e->l_act, Tc * max_act));
  B2_TRY(aalloc(&e->l_xl, (size_t)e->l_rows_cap * W));
  size_t scratch = 0;   // the key splits of a decode step's attention (one buffer: the layers run one after the other)
  for (const ListLayer& L : e->ll)
    if (L.sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) scratch = std::max(scratch, heads_attention_premix_scratch_floats(bucket_batch(c.max_seqs), L.sp.heads, L.sp.vdim));
  if (any_latent) {
    B2_TRY(aalloc(&e->l_x2, Tc * max_qr));
    B2_TRY(aalloc(&e->l_qnope, Tc * max_hd));
    B2_TRY(dalloc(&e->l_qabs, Tc * max_hr));
    B2_TRY(aalloc(&e->l_olat, Tc * max_hr));
    if (!e->f32) scratch = std::max(scratch, latent_attention_scratch_floats(bucket_batch(c.max_seqs), max_heads, max_rank));
  }
  if (scratch > 0) {
    e->l_attn_scratch_floats = scratch;
    B2_TRY(dalloc(&e->l_attn_scratch, scratch));
  }
  if (any_experts) {
    B2_TRY(dalloc(&e->l_y, Tc * max_top * W));
    B2_TRY(dalloc(&e->l_rw, Tc * max_top));
    B2_TRY(dalloc(&e->l_idx, Tc * max_top));
    e->l_offsets_stride = max_exp + 1;
    B2_TRY(dalloc(&e->l_offsets, (size_t)3 * (max_exp + 1)));
    B2_CUDA_OK(cudaMemset(e->l_offsets, 0, (size_t)3 * (max_exp + 1) * 4));
    B2_TRY(dalloc(&e->l_slot_token, Tc * max_top));
    B2_TRY(dalloc(&e->l_pair_slot, Tc * max_top));
    e->l_tiles_cap = (int)(Tc * max_top / any_gemm_tile_rows() + max_exp + 1);
    B2_TRY(dalloc(&e->l_tile_group, (size_t)e->l_tiles_cap));
    B2_TRY(dalloc(&e->l_tile_row0, (size_t)e->l_tiles_cap));
    B2_TRY(dalloc(&e->l_ntiles, (size_t)1));
    if (!e->f32 && Tc * max_top >= (size_t)LIST_TC_EXPERT_ROWS && max_exp > 1) {   // prompt-sized expert products on the tcgen05 projection kernel
      B2_TRY(dalloc(&e->l_xperm, Tc * max_top * W));
      B2_CUDA_OK(cudaMallocHost(&e->h_offsets, (size_t)(max_exp + 1) * sizeof(int32_t)));
    }
    B2_CUDA_OK(cudaMemset(e->l_ntiles, 0, 4));
    B2_CUDA_OK(cudaMemset(e->l_pair_slot, 0, Tc * max_top * 4));
  }
  B2_TRY(dalloc(&e->d_row_seq, Tc));
  B2_TRY(dalloc(&e->d_row_first, Tc));
  B2_TRY(dalloc(&e->d_row_end, Tc));
  B2_CUDA_OK(cudaMemset(e->d_row_seq, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_first, 0, Tc * 4));
  B2_CUDA_OK(cudaMemset(e->d_row_end, 0, Tc * 4));
  return 0;
}

// Names of the tensors a Tinevik checkpoint must hold (layers that use another layer's tensors have none).
std::vector<std::string> mixed_tensor_names(const b2_engine* e) {
  std::vector<std::string> n = {"embed", "final.norm", "final.norm.b"};
  if (e->l_head != e->l_embed) n.push_back("head");
  for (size_t l = 0; l < e->ll.size(); ++l) {
    const b2_layer_spec& sp = e->ll[l].sp;
    if (sp.weights_of >= 0) continue;
    const std::string p = "l" + std::to_string(l) + ".";
    for (const char* t : {"norm1", "norm1.b", "norm1b", "norm1b.b"}) n.push_back(p + t);
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      for (const char* t : {"q", "k", "v", "g", "o", "norm", "a1", "a2", "a2.b"}) n.push_back(p + "mix." + t);
    } else if (sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
      for (const char* t : {"q", "k", "v", "o", "q.norm", "k.norm"}) n.push_back(p + "mix." + t);
      if (sp.score_mix) n.push_back(p + "mix.talk");
    } else {
      for (const char* t : {"dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "g", "o"}) n.push_back(p + "mix." + t);
    }
    if (sp.ff != B2_FF_NONE)
      for (const char* t : {"norm2", "norm2.b", "norm2b", "norm2b.b"}) n.push_back(p + t);
    if (sp.ff == B2_FF_XIELU) {
      for (const char* t : {"up", "down", "act"}) n.push_back(p + "mlp." + t);
    } else if (sp.ff == B2_FF_TABLE_EXPERTS) {
      n.push_back(p + "mlp.table");
      for (int x = 0; x < sp.experts; ++x)
        for (const char* t : {"gate", "up", "down"}) n.push_back(p + "mlp.e" + std::to_string(x) + "." + t);
    }
  }
  return n;
}

// Every tensor is in: the low-rank first stages join the fused projections, and the buffer the projections write is sized.
int mixed_finalize(b2_engine* e) {
  for (const std::string& name : mixed_tensor_names(e)) B2_REQUIRE(e->loaded.count(name), "weights incomplete: %s missing", name.c_str());
  size_t max_nqd = 1;
  for (size_t l = 0; l < e->ll.size(); ++l) {
    ListLayer& L = e->ll[l];
    const b2_layer_spec& sp = L.sp;
    if (sp.weights_of >= 0) continue;
    if (sp.mixer == B2_MIXER_DECAY_STATE) {
      const size_t dec = (size_t)sp.heads * sp.dim;
      B2_REQUIRE(L.rank_a >= 1 && L.a2_floats == dec * L.rank_a, "layer %zu: a1 has %d rows, a2 %zu numbers for %zu channels", l, L.rank_a, L.a2_floats, dec);
      B2_TRY(join_low_rank(e, L));
    }
    max_nqd = std::max(max_nqd, (size_t)L.nqd);
  }
  if (e->l_qd == nullptr || max_nqd > e->l_qd_cols) {
    if (e->l_qd) cudaFree(e->l_qd);
    e->l_qd = nullptr;
    B2_TRY(dalloc(&e->l_qd, (size_t)e->cap_tokens * max_nqd));
    e->l_qd_cols = max_nqd;
  }
  return 0;
}

// Validates the layer list and allocates weights, activations and scratch of a layer-list engine.
int list_engine_alloc(b2_engine* e) {
  if (e->cfg.arch == B2_ARCH_TINEVIK) return mixed_engine_alloc(e);
  if (e->cfg.arch == B2_ARCH_BUMALIX) return state_engine_alloc(e);
  if (e->cfg.arch == B2_ARCH_KEDASUN) return heads_engine_alloc(e);
  const b2_config& c = e->cfg;
  const size_t W = c.hidden, es = e->esz;
  B2_REQUIRE(!e->specs.empty() && (int)e->specs.size() == c.num_layers, "Lerasun: layer_specs missing");
  B2_REQUIRE(c.hidden >= 1 && c.vocab >= 1 && c.num_layers >= 1, "Lerasun: bad sizes");
  auto xalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, std::max<size_t>(elems, 1) * es));
    *p = q;
    e->weight_bytes += (int64_t)(elems * es);
    return 0;
  };
  auto falloc = [&](float** p, size_t n) -> int {
    B2_TRY(dalloc(p, std::max<size_t>(n, 1)));
    e->weight_bytes += (int64_t)(n * 4);
    return 0;
  };
  e->weight_bytes = 0;
  B2_TRY(xalloc(&e->l_embed, (size_t)c.vocab * W));
  B2_TRY(xalloc(&e->l_head, (size_t)c.vocab * W));
  B2_TRY(falloc(&e->l_embed_gain, W));
  B2_TRY(falloc(&e->l_final_gain, W));
  e->ll.resize(c.num_layers);
  size_t max_nqd = 1, max_hn = 1, max_hr = 1, max_hrot = 1, max_hv = 1, max_ff = 1;
  int max_top = 1, max_exp = 1;
  for (int l = 0; l < c.num_layers; ++l) {
    ListLayer& L = e->ll[l];
    L.sp = e->specs[l];
    const b2_layer_spec& sp = L.sp;
    B2_REQUIRE(sp.mixer == B2_MIXER_LATENT_ATTENTION, "layer %d: mixer kind %d not built", l, sp.mixer);
    B2_REQUIRE(sp.heads >= 1 && sp.dim >= 1 && sp.rot_dim >= 0 && sp.vdim >= 1 && sp.kv_rank >= 1, "layer %d: bad mixer sizes", l);
    B2_REQUIRE(sp.rot_dims >= 0 && sp.rot_dims <= sp.rot_dim && sp.rot_dims % 2 == 0, "layer %d: rot dims %d must be even and <= rot_dim %d", l, sp.rot_dims, sp.rot_dim);
    if (sp.kv_from >= 0) {
      B2_REQUIRE(sp.kv_from < l && e->specs[sp.kv_from].kv_from < 0, "layer %d: kv_from %d must name an earlier layer with its own latent", l, sp.kv_from);
      const b2_layer_spec& o = e->specs[sp.kv_from];
      B2_REQUIRE(o.kv_rank == sp.kv_rank && o.rot_dim == sp.rot_dim, "layer %d: latent sizes differ from layer %d's", l, sp.kv_from);
    }
    B2_REQUIRE(sp.ff == B2_FF_NONE || sp.ff == B2_FF_ROUTED_EXPERTS, "layer %d: feed-forward kind %d not built", l, sp.ff);
    L.nq = sp.heads * (sp.dim + sp.rot_dim);
    L.nqd = L.nq + (sp.kv_from < 0 ? sp.kv_rank + sp.rot_dim : 0);
    B2_TRY(xalloc(&L.wqd, (size_t)L.nqd * W));
    B2_TRY(xalloc(&L.ukT, (size_t)sp.heads * sp.kv_rank * sp.dim));
    B2_TRY(xalloc(&L.uv, (size_t)sp.heads * sp.vdim * sp.kv_rank));
    B2_TRY(xalloc(&L.wo, W * sp.heads * sp.vdim));
    B2_TRY(falloc(&L.gain1, W));
    B2_TRY(falloc(&L.sink, sp.heads));
    if (sp.kv_from < 0) B2_TRY(falloc(&L.lat_gain, sp.kv_rank));
    if (sp.ff == B2_FF_ROUTED_EXPERTS) {
      B2_REQUIRE(sp.experts >= 1 && sp.top >= 1 && sp.ff_dim >= 1 && sp.groups >= 1 && sp.experts % sp.groups == 0 && sp.groups_keep >= 1 &&
                     sp.groups_keep <= sp.groups && sp.top <= sp.groups_keep * (sp.experts / sp.groups),
                 "layer %d: bad router sizes (experts %d, top %d, groups %d, keep %d)", l, sp.experts, sp.top, sp.groups, sp.groups_keep);
      B2_TRY(falloc(&L.gain2, W));
      B2_TRY(falloc(&L.router, (size_t)sp.experts * W));
      B2_TRY(falloc(&L.corr, sp.experts));
      B2_TRY(xalloc(&L.up, (size_t)sp.experts * sp.ff_dim * W));
      B2_TRY(xalloc(&L.down, (size_t)sp.experts * W * sp.ff_dim));
      max_top = std::max(max_top, sp.top);
      max_exp = std::max(max_exp, sp.experts);
      max_ff = std::max(max_ff, (size_t)sp.ff_dim);
    }
    max_nqd = std::max(max_nqd, (size_t)L.nqd);
    max_hn = std::max(max_hn, (size_t)sp.heads * sp.dim);
    max_hr = std::max(max_hr, (size_t)sp.heads * sp.kv_rank);
    max_hrot = std::max(max_hrot, (size_t)sp.heads * std::max(sp.rot_dim, 1));
    max_hv = std::max(max_hv, (size_t)sp.heads * sp.vdim);
  }
  // ---- activations ----
  e->cap_tokens = ((std::max(c.max_batch_tokens, c.max_seqs) + 255) / 256) * 256;
  const size_t Tc = e->cap_tokens;
  e->l_rows_cap = (int)(Tc + bucket_batch(c.max_seqs));
  e->l_max_top = max_top;
  e->v_pad = (c.vocab + 7) / 8 * 8;
  auto aalloc = [&](void** p, size_t elems) -> int {
    char* q = nullptr;
    B2_TRY(dalloc(&q, elems * es));
    *p = q;
    return 0;
  };
  B2_TRY(dalloc(&e->l_h, Tc * W));
  B2_TRY(dalloc(&e->l_qd, Tc * max_nqd));
  B2_TRY(dalloc(&e->l_qrot, Tc * max_hrot));
  B2_TRY(dalloc(&e->l_qabs, Tc * max_hr));
  B2_TRY(dalloc(&e->l_mix, Tc * W));
  B2_TRY(dalloc(&e->l_y, Tc * max_top * W));
  B2_TRY(dalloc(&e->l_rw, Tc * max_top));
  B2_TRY(dalloc(&e->l_logits, (size_t)e->l_rows_cap * c.vocab));
  B2_TRY(aalloc(&e->l_x1, Tc * W));
  B2_TRY(aalloc(&e->l_x2, Tc * W));
  B2_TRY(aalloc(&e->l_qnope, Tc * max_hn));
  B2_TRY(aalloc(&e->l_olat, Tc * max_hr));
  B2_TRY(aalloc(&e->l_av, Tc * max_hv));
  B2_TRY(aalloc(&e->l_act, Tc * max_top * max_ff));
  B2_TRY(aalloc(&e->l_xl, (size_t)e->l_rows_cap * W));
  B2_TRY(dalloc(&e->l_idx, Tc * max_top));
  e->l_offsets_stride = max_exp + 1;
  B2_TRY(dalloc(&e->l_offsets, (size_t)3 * (max_exp + 1)));
  B2_CUDA_OK(cudaMemset(e->l_offsets, 0, (size_t)3 * (max_exp + 1) * 4));
  B2_TRY(dalloc(&e->l_slot_token, Tc * max_top));
  B2_TRY(dalloc(&e->l_pair_slot, Tc * max_top));
  e->l_tiles_cap = (int)(Tc * max_top / any_gemm_tile_rows() + max_exp + 1);
  B2_TRY(dalloc(&e->l_tile_group, (size_t)e->l_tiles_cap));
  B2_TRY(dalloc(&e->l_tile_row0, (size_t)e->l_tiles_cap));
  B2_TRY(dalloc(&e->l_ntiles, (size_t)1));
  if (!e->f32) {
    int max_heads = 1, max_rank = 1;
    for (const ListLayer& L : e->ll) {
      max_heads = std::max(max_heads, L.sp.heads);
      max_rank = std::max(max_rank, L.sp.kv_rank);
    }
    e->l_attn_scratch_floats = latent_attention_scratch_floats(bucket_batch(c.max_seqs), max_heads, max_rank);
    B2_TRY(dalloc(&e->l_attn_scratch, e->l_attn_scratch_floats));
    if (max_top > 0 && Tc * max_top >= (size_t)LIST_TC_EXPERT_ROWS) {   // prompt-sized expert products on the tcgen05 projection kernel
      B2_TRY(dalloc(&e->l_xperm, Tc * max_top * W));
      B2_TRY(dalloc(&e->l_upf, Tc * max_top * max_ff));
      B2_CUDA_OK(cudaMallocHost(&e->h_offsets, (size_t)(max_exp + 1) * sizeof(int32_t)));
    }
  }
  B2_CUDA_OK(cudaMemset(e->l_ntiles, 0, 4));
  B2_CUDA_OK(cudaMemset(e->l_pair_slot, 0, Tc * max_top * 4));
  return 0;
}

int layer_tensor(b2_engine* e, const std::string& name, const void* host, size_t nbytes) {
  const b2_config& c = e->cfg;
  if (list_arch(c.arch)) return list_tensor(e, name, host, nbytes);
  const int H = c.hidden, I = c.intermediate;
  auto put = [&](bf16* dst, size_t elems) -> int {
    if (nbytes != elems * 2) {
      b2_set_error("tensor %s: expected %zu bytes, got %zu", name.c_str(), elems * 2, nbytes);
      return -22;
    }
    B2_CUDA_OK(cudaMemcpy(dst, host, nbytes, cudaMemcpyHostToDevice));
    e->loaded[name] = 1;
    return 0;
  };
  // Per-head blocks of the attention projections go through the internal geometry (see b2_engine):
  // head h of the checkpoint lands at internal head h * step, its head_dim rows (or columns, for the
  // output projection) at the start of a 128-wide slot; everything else in the slot stays zero.
  const int hd_r = c.head_dim;
  auto put_head_rows = [&](bf16* dst, const uint16_t* src, int heads, int step, int slots) -> int {
    std::vector<uint16_t> stage((size_t)slots * 128 * H, 0);
    for (int h = 0; h < heads; ++h)
      memcpy(&stage[(size_t)h * step * 128 * H], src + (size_t)h * hd_r * H, (size_t)hd_r * H * 2);
    B2_CUDA_OK(cudaMemcpy(dst, stage.data(), stage.size() * 2, cudaMemcpyHostToDevice));
    return 0;
  };
  auto put_head_cols = [&](bf16* dst, const uint16_t* src, int heads, int step, int slots) -> int {
    const size_t in_cols = (size_t)heads * hd_r, out_cols = (size_t)slots * 128;
    std::vector<uint16_t> stage((size_t)H * out_cols, 0);
    for (int r = 0; r < H; ++r)
      for (int h = 0; h < heads; ++h)
        memcpy(&stage[(size_t)r * out_cols + (size_t)h * step * 128], src + (size_t)r * in_cols + (size_t)h * hd_r, (size_t)hd_r * 2);
    B2_CUDA_OK(cudaMemcpy(dst, stage.data(), stage.size() * 2, cudaMemcpyHostToDevice));
    return 0;
  };
  auto expect = [&](size_t elems) -> int {
    if (nbytes != elems * 2) {
      b2_set_error("tensor %s: expected %zu bytes, got %zu", name.c_str(), elems * 2, nbytes);
      return -22;
    }
    return 0;
  };
  const size_t q_r = (size_t)c.num_q_heads * hd_r, kv_r = (size_t)c.num_kv_heads * hd_r;  // checkpoint widths
  const uint16_t* src16 = reinterpret_cast<const uint16_t*>(host);
  if (c.arch == B2_ARCH_OPT) {
    // HF:models/opt/modeling_opt.py state dict: model.decoder.{embed_tokens,embed_positions,final_layer_norm,layers.N.*}
    auto put_head_vec = [&](bf16* dst, int heads, int step) -> int {  // bias of a per-head projection, zero in the padding
      std::vector<uint16_t> stage((size_t)heads * step * 128, 0);
      for (int h = 0; h < heads; ++h) memcpy(&stage[(size_t)h * step * 128], src16 + (size_t)h * hd_r, (size_t)hd_r * 2);
      B2_CUDA_OK(cudaMemcpy(dst, stage.data(), stage.size() * 2, cudaMemcpyHostToDevice));
      return 0;
    };
    auto mark = [&](int rc) {
      if (rc == 0) e->loaded[name] = 1;
      return rc;
    };
    const std::string dec = "model.decoder.";
    if (name == "lm_head.weight") {
      e->loaded[name] = 1;  // tied to embed_tokens
      return 0;
    }
    if (name.compare(0, dec.size(), dec) != 0) {
      b2_set_error("unknown tensor name %s", name.c_str());
      return -22;
    }
    const std::string r0 = name.substr(dec.size());
    if (r0 == "embed_tokens.weight") return put(e->embed, (size_t)c.vocab * H);
    if (r0 == "embed_positions.weight") return put(e->pos_embed, (size_t)e->pos_rows * H);
    if (r0 == "final_layer_norm.weight") return put(e->final_norm, H);
    if (r0 == "final_layer_norm.bias") return put(e->final_norm_b, H);
    const std::string lp = "layers.";
    size_t d2 = r0.find('.', lp.size());
    if (r0.compare(0, lp.size(), lp) != 0 || d2 == std::string::npos) {
      b2_set_error("unknown tensor name %s", name.c_str());
      return -22;
    }
    const int li = atoi(r0.substr(lp.size(), d2 - lp.size()).c_str());
    if (li < 0 || li >= c.num_layers) {
      b2_set_error("tensor %s: layer out of range", name.c_str());
      return -22;
    }
    LayerW& L = e->layers[li];
    const std::string rest = r0.substr(d2 + 1);
    bf16* wq = L.wqkv;
    bf16* wk = L.wqkv + (size_t)e->q_size * H;
    bf16* wv = L.wqkv + (size_t)(e->q_size + e->kv_size) * H;
    if (rest == "self_attn_layer_norm.weight") return put(L.ln1, H);
    if (rest == "self_attn_layer_norm.bias") return put(L.ln1_b, H);
    if (rest == "final_layer_norm.weight") return put(L.ln2, H);
    if (rest == "final_layer_norm.bias") return put(L.ln2_b, H);
    if (rest == "self_attn.q_proj.weight") { B2_TRY(expect(q_r * H)); return mark(put_head_rows(wq, src16, c.num_q_heads, e->qhead_step, e->nq)); }
    if (rest == "self_attn.k_proj.weight") { B2_TRY(expect(kv_r * H)); return mark(put_head_rows(wk, src16, c.num_kv_heads, 1, e->nkv)); }
    if (rest == "self_attn.v_proj.weight") { B2_TRY(expect(kv_r * H)); return mark(put_head_rows(wv, src16, c.num_kv_heads, 1, e->nkv)); }
    if (rest == "self_attn.out_proj.weight") { B2_TRY(expect((size_t)H * q_r)); return mark(put_head_cols(L.wo, src16, c.num_q_heads, e->qhead_step, e->nq)); }
    if (rest == "self_attn.q_proj.bias") { B2_TRY(expect(q_r)); return mark(put_head_vec(L.bqkv, c.num_q_heads, e->qhead_step)); }
    if (rest == "self_attn.k_proj.bias") { B2_TRY(expect(kv_r)); return mark(put_head_vec(L.bqkv + e->q_size, c.num_kv_heads, 1)); }
    if (rest == "self_attn.v_proj.bias") { B2_TRY(expect(kv_r)); return mark(put_head_vec(L.bqkv + e->q_size + e->kv_size, c.num_kv_heads, 1)); }
    if (rest == "self_attn.out_proj.bias") return put(L.bo, H);
    if (rest == "fc1.weight") return put(L.wgu, (size_t)I * H);
    if (rest == "fc1.bias") return put(L.b1, I);
    if (rest == "fc2.weight") return put(L.wd, (size_t)H * I);
    if (rest == "fc2.bias") return put(L.b2, H);
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  if (name == "model.embed_tokens.weight") return put(e->embed, (size_t)c.vocab * H);
  if (name == "model.norm.weight") return put(e->final_norm, H);
  if (name == "lm_head.weight") {
    if (c.tie_embeddings) {
      e->loaded[name] = 1;  // tied: ignore the duplicate
      return 0;
    }
    return put(e->lm_head, (size_t)c.vocab * H);
  }
  const std::string pre = "model.layers.";
  if (name.compare(0, pre.size(), pre) != 0) {
    b2_set_error("unknown tensor name %s", name.c_str());
    return -22;
  }
  size_t dot = name.find('.', pre.size());
  if (dot == std::string::npos) {
    b2_set_error("bad tensor name %s", name.c_str());
    return -22;
  }
  int l = atoi(name.substr(pre.size(), dot - pre.size()).c_str());
  if (l < 0 || l >= c.num_layers) {
    b2_set_error("tensor %s: layer out of range", name.c_str());
    return -22;
  }
  LayerW& L = e->layers[l];
  std::string rest = name.substr(dot + 1);
  if (rest == "input_layernorm.weight") return put(L.ln1, H);
  if (rest == "post_attention_layernorm.weight") return put(L.ln2, H);
  bf16* wq = L.wqkv;
  bf16* wk = L.wqkv + (size_t)e->q_size * H;
  bf16* wv = L.wqkv + (size_t)(e->q_size + e->kv_size) * H;
  auto done = [&](int rc) {
    if (rc == 0) e->loaded[name] = 1;
    return rc;
  };
  if (c.arch == B2_ARCH_QWEN3) {
    if (rest == "self_attn.q_norm.weight") return put(L.qnorm, c.head_dim);
    if (rest == "self_attn.k_norm.weight") return put(L.knorm, c.head_dim);
    if (rest == "mlp.gate_proj.weight") return put(L.wgu, (size_t)I * H);
    if (rest == "mlp.up_proj.weight") return put(L.wgu + (size_t)I * H, (size_t)I * H);
    if (e->native_geom) {
      if (rest == "self_attn.q_proj.weight") return put(wq, (size_t)e->q_size * H);
      if (rest == "self_attn.k_proj.weight") return put(wk, (size_t)e->kv_size * H);
      if (rest == "self_attn.v_proj.weight") return put(wv, (size_t)e->kv_size * H);
      if (rest == "self_attn.o_proj.weight") return put(L.wo, (size_t)H * e->q_size);
    } else {
      if (rest == "self_attn.q_proj.weight") { B2_TRY(expect(q_r * H)); return done(put_head_rows(wq, src16, c.num_q_heads, e->qhead_step, e->nq)); }
      if (rest == "self_attn.k_proj.weight") { B2_TRY(expect(kv_r * H)); return done(put_head_rows(wk, src16, c.num_kv_heads, 1, e->nkv)); }
      if (rest == "self_attn.v_proj.weight") { B2_TRY(expect(kv_r * H)); return done(put_head_rows(wv, src16, c.num_kv_heads, 1, e->nkv)); }
      if (rest == "self_attn.o_proj.weight") { B2_TRY(expect((size_t)H * q_r)); return done(put_head_cols(L.wo, src16, c.num_q_heads, e->qhead_step, e->nq)); }
    }
  } else {  // Phi-3: fused projections in the checkpoint, HF:models/phi3/modeling_phi3.py:53-54,224,237-241
    if (rest == "self_attn.qkv_proj.weight") {
      B2_TRY(expect((q_r + 2 * kv_r) * H));
      B2_TRY(put_head_rows(wq, src16, c.num_q_heads, e->qhead_step, e->nq));
      B2_TRY(put_head_rows(wk, src16 + q_r * H, c.num_kv_heads, 1, e->nkv));
      return done(put_head_rows(wv, src16 + (q_r + kv_r) * H, c.num_kv_heads, 1, e->nkv));
    }
    if (rest == "self_attn.o_proj.weight") { B2_TRY(expect((size_t)H * q_r)); return done(put_head_cols(L.wo, src16, c.num_q_heads, e->qhead_step, e->nq)); }
    if (rest == "mlp.gate_up_proj.weight") return put(L.wgu, (size_t)2 * I * H);  // [gate; up], the order chunk(2) splits
  }
  if (rest == "mlp.down_proj.weight") return put(L.wd, (size_t)H * I);
  b2_set_error("unknown tensor name %s", name.c_str());
  return -22;
}

int load_safetensors(b2_engine* e, const char* path) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) {
    b2_set_error("cannot open %s: %s", path, strerror(errno));
    return -2;
  }
  struct stat st;
  fstat(fd, &st);
  void* map = mmap(nullptr, st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (map == MAP_FAILED) {
    b2_set_error("mmap %s failed", path);
    return -5;
  }
  int rc = 0;
  try {
    const uint8_t* p = reinterpret_cast<const uint8_t*>(map);
    uint64_t hlen = 0;
    memcpy(&hlen, p, 8);
    if (hlen + 8 > (uint64_t)st.st_size) throw std::runtime_error("header length exceeds file");
    b2json::Value hdr = b2json::parse(reinterpret_cast<const char*>(p + 8), (size_t)hlen);
    const uint8_t* data = p + 8 + hlen;
    std::vector<uint16_t> conv;
    for (auto& kv : *hdr.obj) {
      if (kv.first == "__metadata__") continue;
      const b2json::Value* dt = kv.second.find("dtype");
      const b2json::Value* off = kv.second.find("data_offsets");
      if (!dt || !off || off->size() != 2) throw std::runtime_error("malformed entry " + kv.first);
      uint64_t a = (uint64_t)off->at(0).as_int(), b = (uint64_t)off->at(1).as_int();
      if (b < a || 8 + hlen + b > (uint64_t)st.st_size) throw std::runtime_error("offsets out of range for " + kv.first);
      const void* src = data + a;
      size_t nbytes = b - a;
      if (dt->as_string() == "F32") {  // convert to bf16 (round to nearest even)
        size_t n = nbytes / 4;
        conv.resize(n);
        const uint32_t* f = reinterpret_cast<const uint32_t*>(src);
        for (size_t i = 0; i < n; ++i) {
          uint32_t u = f[i];
          conv[i] = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
        }
        src = conv.data();
        nbytes = n * 2;
      } else if (dt->as_string() == "F16") {  // fp16 -> fp32 (exact) -> bf16 (round to nearest even)
        size_t n = nbytes / 2;
        conv.resize(n);
        const uint16_t* hsrc = reinterpret_cast<const uint16_t*>(src);
        for (size_t i = 0; i < n; ++i) {
          const uint32_t hbits = hsrc[i], sign = (hbits & 0x8000u) << 16, ex = (hbits >> 10) & 0x1fu, man = hbits & 0x3ffu;
          uint32_t u;
          if (ex == 0) {
            if (man == 0) u = sign;
            else {  // subnormal half: normalise
              int sh = 0;
              uint32_t m = man;
              while (!(m & 0x400u)) { m <<= 1; ++sh; }
              u = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | ((m & 0x3ffu) << 13);
            }
          } else if (ex == 31) u = sign | 0x7f800000u | (man << 13);
          else u = sign | ((ex + 112u) << 23) | (man << 13);
          conv[i] = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
        }
        src = conv.data();
        nbytes = n * 2;
      } else if (dt->as_string() == "I32") {   // integer tables (the layer-list families that have one)
        rc = list_arch(e->cfg.arch) ? list_int_tensor(e, kv.first, reinterpret_cast<const int32_t*>(src), nbytes / 4)
                                    : (b2_set_error("tensor %s: this family has no integer tensors", kv.first.c_str()), -22);
        if (rc != 0) break;
        continue;
      } else if (dt->as_string() != "BF16") {
        throw std::runtime_error("tensor " + kv.first + ": dtype " + dt->as_string() + " not supported (BF16/F16/F32/I32)");
      }
      if (kv.first.find("rotary_emb.inv_freq") != std::string::npos) continue;
      rc = layer_tensor(e, kv.first, src, nbytes);
      if (rc != 0) break;
    }
  } catch (const std::exception& ex) {
    b2_set_error("safetensors %s: %s", path, ex.what());
    rc = -22;
  }
  munmap(map, st.st_size);
  return rc;
}

}  // namespace

// =======================================================================================
// C ABI
// =======================================================================================
extern "C" int b2_engine_create(const b2_config* cfg, const char* safetensors_path, int device, b2_engine** out) {
  B2_REQUIRE(cfg != nullptr && out != nullptr, "b2_engine_create: null argument");
  B2_REQUIRE(cfg->abi_version == B2_ABI_VERSION, "b2_engine_create: abi_version %d != %d", cfg->abi_version, B2_ABI_VERSION);
  B2_REQUIRE(cfg->arch == B2_ARCH_QWEN3 || cfg->arch == B2_ARCH_PHI3 || cfg->arch == B2_ARCH_OPT || list_arch(cfg->arch),
             "arch %d not built (0 = Qwen3, 1 = Phi-3, 2 = OPT, 3 = Lerasun, 4 = Kedasun, 5 = Bumalix, 6 = Tinevik)", cfg->arch);
  const bool ls = list_arch(cfg->arch);  // a layer-list family: its sizes live in layer_specs and are checked in list_engine_alloc
  B2_REQUIRE(ls || !cfg->compute_f32, "compute_f32: only the layer-list families have an fp32 path");
  B2_REQUIRE(!ls || cfg->layer_specs != nullptr, "layer-list family: layer_specs is NULL");
  B2_REQUIRE(cfg->arch != B2_ARCH_OPT || cfg->tie_embeddings, "OPT: the lm_head is tied to embed_tokens");
  B2_REQUIRE(cfg->sliding_window >= 0 && (cfg->sliding_window == 0 || cfg->arch == B2_ARCH_PHI3),
             "sliding_window %d: only the Phi-3 family has one", cfg->sliding_window);
  B2_REQUIRE(ls || (cfg->head_dim >= 8 && cfg->head_dim <= 128 && cfg->head_dim % 8 == 0), "head_dim %d not supported (multiple of 8, <= 128)",
             cfg->head_dim);
  B2_REQUIRE(ls || (cfg->num_kv_heads >= 1 && (cfg->num_q_heads == 2 * cfg->num_kv_heads || cfg->num_q_heads == cfg->num_kv_heads)),
             "query heads per kv head must be 1 or 2 (nq=%d nkv=%d)", cfg->num_q_heads, cfg->num_kv_heads);
  if (!ls) {
    const int rd = cfg->arch == B2_ARCH_OPT ? 0 : (cfg->rotary_dim > 0 ? cfg->rotary_dim : cfg->head_dim);
    B2_REQUIRE(rd % 8 == 0 && rd <= cfg->head_dim, "rotary_dim %d must be a multiple of 8 and <= head_dim", rd);
    B2_REQUIRE(cfg->arch != B2_ARCH_QWEN3 || (rd == cfg->head_dim && cfg->head_dim == 128),
               "Qwen3: QK-norm is built for 128-wide, fully rotated heads (head_dim %d, rotary_dim %d)", cfg->head_dim, rd);
  }
  B2_REQUIRE(cfg->block_size == 16, "block_size %d not built (16 only)", cfg->block_size);
  B2_REQUIRE(ls || (cfg->hidden % 256 == 0 && cfg->intermediate % 256 == 0), "hidden/intermediate must be multiples of 256");
  B2_REQUIRE(cfg->max_seqs >= 1 && cfg->max_batch_tokens >= 1 && cfg->max_model_len >= 1, "bad sizing");
  int ndev = 0;
  cudaError_t ce = cudaGetDeviceCount(&ndev);
  if (ce != cudaSuccess || ndev <= device) {
    b2_set_error("no CUDA device %d available (%s); this engine has no CPU path", device,
                 ce == cudaSuccess ? "device count too small" : cudaGetErrorString(ce));
    return -19;
  }
  B2_CUDA_OK(cudaSetDevice(device));
  cudaDeviceProp prop;
  B2_CUDA_OK(cudaGetDeviceProperties(&prop, device));
  B2_REQUIRE(prop.major == 10, "device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);

  b2_engine* e = new b2_engine();
  e->cfg = *cfg;
  e->cfg.rope_inv_freq = nullptr;
  e->cfg.layer_specs = nullptr;
  if (ls) {
    e->specs.assign(cfg->layer_specs, cfg->layer_specs + cfg->num_layers);
    e->f32 = cfg->compute_f32 != 0;
    e->esz = e->f32 ? 4 : 2;
    e->cfg.num_kv_heads = e->cfg.num_q_heads = 1;  // unused by this family; keeps the derived GQA geometry below finite
    e->cfg.head_dim = 128;
  }
  e->device = device;
  e->num_sms = prop.multiProcessorCount;
  const b2_config& c = e->cfg;
  e->hd = 128;
  e->nkv = c.num_kv_heads;
  e->nq = 2 * c.num_kv_heads;
  e->qhead_step = (c.num_q_heads == c.num_kv_heads) ? 2 : 1;
  e->native_geom = (c.head_dim == 128 && e->qhead_step == 1);
  e->attn_scale = (float)(1.0 / sqrt((double)c.head_dim));  // HF passes head_dim**-0.5 as a double
  e->rotary_dim = c.arch == B2_ARCH_OPT ? 0 : (c.rotary_dim > 0 ? c.rotary_dim : c.head_dim);
  e->gu_rows = c.arch == B2_ARCH_OPT ? c.intermediate : 2 * c.intermediate;
  e->pos_rows = c.arch == B2_ARCH_OPT ? (c.max_positions > 0 ? c.max_positions : c.max_model_len) + 2 : 0;
  e->q_size = e->nq * e->hd;
  e->kv_size = e->nkv * e->hd;
  e->qkv_size = e->q_size + 2 * e->kv_size;
  e->simt_max_tokens = env_int("B2_SIMT_MAX_TOKENS", 0);
  e->attn_split_override = env_int("B2_ATTN_SPLITS", 0);
  e->force_gemm_impl = env_int("B2_GEMM_IMPL", -1);
  e->skip_mask = (unsigned)env_int("B2_SKIP_MASK", 0);
  // 0 separate kernels (default: fastest measured), 1 eight-step chain kernel (chain.cu), 2 fused four-step cluster
  // chain (chain_cluster.cu); 1 and 2 are kept as measured experiments with parity tests
  e->use_chain = env_int("B2_CHAIN", 0);
  e->use_pair = env_int("B2_PAIR", 7);  // bit 2: O / down projections update the residual stream themselves (gemm_resid.cu)
  e->prefill_tc = env_int("B2_PREFILL_TC", 1);
  e->gu_prefill_fused = env_int("B2_GU_FUSED", 1);
  e->prefill_mc = env_int("B2_MC", 1);
  e->prefill_pairs = env_int("B2_PREFILL_PAIRS", 1);
  e->qkv_rope_prefill_fused = env_int("B2_QKV_ROPE_FUSED", 1);
  e->prefill_resid_fused = env_int("B2_RESID_FUSED", 0);
  e->l2_weight_prefetch = env_int("B2_WPF", 0);
  e->o_small_smem = env_int("B2_O_SMALL", 0);
  // Off by default: measured on B200 at C2 (ms/step) 0 MB 2.22, 40 MB 2.24, 72 MB 2.33, 100 MB 2.38 --
  // un-paced prefetch bursts queue ahead of the projections' own latency-critical weight loads.
  e->kv_l2_budget = (long long)env_int("B2_KV_L2_MB", 0) << 20;
  const int H = c.hidden, I = c.intermediate;
  int rc = 0;
#define E_TRY(expr)        \
  do {                     \
    rc = (expr);           \
    if (rc != 0) goto fail; \
  } while (0)
#define E_CUDA(expr)                                                                           \
  do {                                                                                         \
    cudaError_t _e = (expr);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      b2_set_error("%s:%d: %s failed: %s", __FILE__, __LINE__, #expr, cudaGetErrorString(_e)); \
      rc = -5;                                                                                 \
      goto fail;                                                                               \
    }                                                                                          \
  } while (0)
  {
    E_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    if (ls) E_TRY(list_engine_alloc(e));
    if (!ls) {
    // ---- weights ----
    E_TRY(dalloc(&e->embed, (size_t)c.vocab * H));
    if (c.tie_embeddings) e->lm_head = e->embed;
    else E_TRY(dalloc(&e->lm_head, (size_t)c.vocab * H));
    E_TRY(dalloc(&e->final_norm, (size_t)H));
    e->layers.resize(c.num_layers);
    for (auto& L : e->layers) {
      E_TRY(dalloc(&L.ln1, (size_t)H));
      E_TRY(dalloc(&L.ln2, (size_t)H));
      if (c.arch == B2_ARCH_QWEN3) {  // Phi-3 has no QK-norm: the null gains switch it off in the kernel
        E_TRY(dalloc(&L.qnorm, (size_t)c.head_dim));
        E_TRY(dalloc(&L.knorm, (size_t)c.head_dim));
      }
      E_TRY(dalloc(&L.wqkv, (size_t)e->qkv_size * H));
      E_TRY(dalloc(&L.wo, (size_t)H * e->q_size));
      E_TRY(dalloc(&L.wgu, (size_t)e->gu_rows * H));
      E_TRY(dalloc(&L.wd, (size_t)H * I));
      if (c.arch == B2_ARCH_OPT) {
        E_TRY(dalloc(&L.bqkv, (size_t)e->qkv_size));
        E_CUDA(cudaMemset(L.bqkv, 0, (size_t)e->qkv_size * 2));  // padded slots keep a zero bias
        E_TRY(dalloc(&L.bo, (size_t)H));
        E_TRY(dalloc(&L.ln1_b, (size_t)H));
        E_TRY(dalloc(&L.ln2_b, (size_t)H));
        E_TRY(dalloc(&L.b1, (size_t)I));
        E_TRY(dalloc(&L.b2, (size_t)H));
      }
    }
    if (c.arch == B2_ARCH_OPT) {
      E_TRY(dalloc(&e->final_norm_b, (size_t)H));
      E_TRY(dalloc(&e->pos_embed, (size_t)e->pos_rows * H));
    }
    e->weight_bytes = 2ll * ((int64_t)c.vocab * H * (c.tie_embeddings ? 1 : 2) + H +
                             (int64_t)c.num_layers * (2 * H + (c.arch == B2_ARCH_QWEN3 ? 2 * c.head_dim : 0) + (int64_t)e->qkv_size * H +
                                                      (int64_t)H * e->q_size + ((int64_t)e->gu_rows + I) * H) +
                             (c.arch == B2_ARCH_OPT ? (int64_t)e->pos_rows * H + H +
                                                          (int64_t)c.num_layers * (e->qkv_size + 4ll * H + I) : 0));
    // ---- RoPE table: cos/sin in fp32 from fp32 inv_freq * position, rounded to bf16
    //      (HF:models/qwen3/modeling_qwen3.py:132-148) ----
    {
      // table row = [cos 64 | sin 64]; a rotary width below 128 (Phi-3: 96) fills the first rotary_dim/2
      // entries of each half, HF:models/phi3/modeling_phi3.py:199-205
      const int rd = e->rotary_dim, half = rd / 2, row = 128;
      std::vector<float> inv(half);
      for (int i = 0; i < half; ++i) {
        if (cfg->rope_inv_freq) inv[i] = cfg->rope_inv_freq[i];
        else inv[i] = (float)(1.0 / pow((double)c.rope_theta, (double)(2 * i) / (double)rd));
      }
      std::vector<uint16_t> tab((size_t)c.max_model_len * row);
      auto to_bf16 = [](float f) -> uint16_t {
        uint32_t u;
        memcpy(&u, &f, 4);
        return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
      };
      for (int p = 0; p < c.max_model_len; ++p) {
        for (int i = 0; i < 64; ++i) {
          tab[(size_t)p * row + i] = to_bf16(1.0f);
          tab[(size_t)p * row + 64 + i] = to_bf16(0.0f);
        }
        for (int i = 0; i < half; ++i) {
          float fr = (float)p * inv[i];  // fp32 product, as the fp32 matmul in HF
          tab[(size_t)p * row + i] = to_bf16((float)cos((double)fr));
          tab[(size_t)p * row + 64 + i] = to_bf16((float)sin((double)fr));
        }
      }
      E_TRY(dalloc(&e->cos_sin, tab.size()));
      E_CUDA(cudaMemcpy(e->cos_sin, tab.data(), tab.size() * 2, cudaMemcpyHostToDevice));
    }
    // ---- activations ----
    e->cap_tokens = ((std::max(c.max_batch_tokens, c.max_seqs) + 255) / 256) * 256;
    const size_t Tc = e->cap_tokens;
    E_TRY(dalloc(&e->h, Tc * H));
    E_TRY(dalloc(&e->x, Tc * H));
    E_TRY(dalloc(&e->qkv, Tc * e->qkv_size));
    E_TRY(dalloc(&e->qrot, Tc * e->q_size));
    E_TRY(dalloc(&e->attn, Tc * e->q_size));
    E_TRY(dalloc(&e->gu, Tc * 2 * I));
    E_TRY(dalloc(&e->act, Tc * I));
    E_TRY(dalloc(&e->proj, Tc * H));
    const size_t last_rows = ((size_t)(c.max_seqs + 255) / 256) * 256;
    E_TRY(dalloc(&e->xlast, last_rows * H));
    E_CUDA(cudaMemset(e->x, 0, Tc * H * 2));
    E_CUDA(cudaMemset(e->attn, 0, Tc * e->q_size * 2));
    E_CUDA(cudaMemset(e->act, 0, Tc * I * 2));
    E_CUDA(cudaMemset(e->xlast, 0, last_rows * H * 2));
    e->partial_floats = (size_t)16 << 20;  // 64 MB of fp32 split-K partials
    if (c.arch == B2_ARCH_OPT)  // every projection hands over fp32 sums (the bias goes in before the rounding), even unsplit
      e->partial_floats = std::max(e->partial_floats, Tc * (size_t)std::max(std::max(e->qkv_size, I), H));
    E_TRY(dalloc(&e->partial, e->partial_floats));
    e->attn_scratch_floats = attn_decode_scratch_floats(bucket_batch(c.max_seqs), e->nq, e->nkv, e->hd);
    E_TRY(dalloc(&e->attn_scratch, e->attn_scratch_floats));
    E_CUDA(cudaMemset(e->attn_scratch, 0, e->attn_scratch_floats * sizeof(float)));  // arrival counters start at zero
    // two-lane decode: B2_MB = smallest padded decode batch that is cut into two half-batch lanes (0 = off)
    // Off by default: measured slower (C2: 2.03 against 1.90 ms/step) -- DESIGN.md section 4 has the timeline.
    e->mb_min_batch = c.arch == B2_ARCH_OPT ? 0 : env_int("B2_MB", 0);
    if (c.arch != B2_ARCH_OPT && c.max_seqs >= 2) {
      E_CUDA(cudaStreamCreateWithFlags(&e->stream2, cudaStreamNonBlocking));
      E_CUDA(cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming));
      E_CUDA(cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming));
      // a lane has at most 64 rows: 8 splits x 64 x the widest projection
      e->partial2_floats = (size_t)8 * 64 * (size_t)std::max(std::max(e->qkv_size, 2 * I), H);
      E_TRY(dalloc(&e->partial2, e->partial2_floats));
      E_TRY(dalloc(&e->attn_scratch2, e->attn_scratch_floats));
      E_CUDA(cudaMemset(e->attn_scratch2, 0, e->attn_scratch_floats * sizeof(float)));
    }
    E_TRY(dalloc(&e->ssq, (size_t)(H / 16) * 64));
    for (int bi = 0; bi < 5; ++bi) {
      E_TRY(b2_make_tmap_bf16(&e->tm_x[XB_X][bi], e->x, Tc, H, H, kBnList[bi]));
      E_TRY(b2_make_tmap_bf16(&e->tm_x[XB_ATTN][bi], e->attn, Tc, e->q_size, e->q_size, kBnList[bi]));
      E_TRY(b2_make_tmap_bf16(&e->tm_x[XB_ACT][bi], e->act, Tc, I, I, kBnList[bi]));
      E_TRY(b2_make_tmap_bf16(&e->tm_x[XB_LAST][bi], e->xlast, last_rows, H, H, kBnList[bi]));
    }
    for (auto& L : e->layers) {
      E_TRY(b2_make_tmap_bf16(&L.tm_qkv, L.wqkv, e->qkv_size, H, H, 128));
      E_TRY(b2_make_tmap_bf16(&L.tm_o, L.wo, H, e->q_size, e->q_size, 128));
      E_TRY(b2_make_tmap_bf16(&L.tm_gu, L.wgu, e->gu_rows, H, H, 128));
      E_TRY(b2_make_tmap_bf16(&L.tm_o32, L.wo, H, e->q_size, e->q_size, 32));
      E_TRY(b2_make_tmap_bf16(&L.tm_gu96, L.wgu, e->gu_rows, H, H, 96));
      E_TRY(b2_make_tmap_bf16(&L.tm_gu64, L.wgu, e->gu_rows, H, H, 64));
      E_TRY(b2_make_tmap_bf16(&L.tm_d32, L.wd, H, I, I, 32));
      E_TRY(b2_make_tmap_bf16(&L.tm_d, L.wd, H, I, I, 128));
    }
    E_TRY(b2_make_tmap_bf16(&e->tm_lm_head, e->lm_head, c.vocab, H, H, 128));
    }  // !ls
    const size_t Tc = e->cap_tokens;
    // ---- batch state ----
    e->bt_stride = (c.max_model_len + c.block_size - 1) / c.block_size;
    const size_t Bcap = bucket_batch(c.max_seqs);
    E_TRY(dalloc(&e->d_tokens, Tc));
    E_TRY(dalloc(&e->d_positions, Tc));
    E_TRY(dalloc(&e->d_slots, Tc));
    E_TRY(dalloc(&e->d_seq_lens, Bcap));
    E_TRY(dalloc(&e->d_block_table, Bcap * e->bt_stride));
    E_TRY(dalloc(&e->d_last_rows, Bcap + (ls ? Tc : 0)));  // layer-list families: logits at any of a call's rows
    E_TRY(dalloc(&e->d_out_tokens, Bcap + (ls ? Tc : 0)));
    E_TRY(dalloc(&e->d_argmax, Bcap));
    E_TRY(dalloc(&e->d_step, (size_t)1));
    E_TRY(dalloc(&e->d_pf_frac, (size_t)1));
    E_TRY(dalloc(&e->d_sample_out, Bcap));
    E_TRY(dalloc(&e->d_sample_rows, Bcap));
    E_TRY(dalloc(&e->d_gbar, (size_t)1));
    E_CUDA(cudaMemset(e->d_gbar, 0, 8));
    E_TRY(dalloc(&e->d_gbar2, (size_t)1));
    E_CUDA(cudaMemset(e->d_gbar2, 0, 8));
    // the fused chain spins on a grid-wide barrier: all of its 32 clusters must be resident at once
    e->fused_ok = !ls && e->native_geom && c.arch == B2_ARCH_QWEN3 &&
                  fused_chain_supported(H, I, e->nq, e->nkv, e->hd, 1, c.block_size) && fused_chain_max_clusters() >= 32;
    E_TRY(dalloc(&e->d_ss, (size_t)2 * 32 * 64));
    E_CUDA(cudaMemset(e->d_ss, 0, 2 * 32 * 64 * 4));
    E_CUDA(cudaMemset(e->d_pf_frac, 0, 4));
    e->log_cap_steps = 4096;
    E_TRY(dalloc(&e->d_token_log, (size_t)e->log_cap_steps * c.max_seqs));
    E_CUDA(cudaMemset(e->d_step, 0, 4));
    E_CUDA(cudaMemset(e->d_block_table, 0, Bcap * e->bt_stride * 4));
    e->tiles_cap = (int)(Tc / 64 + 2 * Bcap + 16);
    E_TRY(dalloc(&e->d_tiles, (size_t)e->tiles_cap));
    e->h_stage_ints = std::max((size_t)7 * Tc + Bcap * (size_t)e->bt_stride + 8 * Bcap, (size_t)1 << 16);
    E_CUDA(cudaMallocHost(&e->h_stage, e->h_stage_ints * sizeof(int32_t)));
    E_CUDA(cudaMallocHost(&e->h_tiles, (size_t)e->tiles_cap * sizeof(PrefillTile)));
    E_CUDA(cudaMallocHost(&e->h_out, (size_t)e->log_cap_steps * c.max_seqs * sizeof(int32_t)));
    E_CUDA(cudaMallocHost(&e->h_tok, Bcap * sizeof(int32_t)));
    E_CUDA(cudaEventCreateWithFlags(&e->ev_tok, cudaEventDisableTiming));
    e->seqs.resize(c.max_seqs);
    // ---- KV pool ----
    {
      const size_t blk_elems = (size_t)e->nkv * c.block_size * e->hd;
      // bytes one page takes in all regions together
      size_t page_bytes_all = blk_elems * 2 * 2 * c.num_layers;
      const bool heads_cache = c.arch == B2_ARCH_KEDASUN;  // a K region and a V region per layer, rows of kv_heads * dim / kv_heads * vdim
      const bool state_arch = c.arch == B2_ARCH_BUMALIX;   // a K and a V region per RUN of a layer that has a softmax mixer
      const bool mixed_arch = c.arch == B2_ARCH_TINEVIK;   // per RUN: a K and a V region for a softmax mixer, one region of latents for a latent mixer
      if (state_arch) {
        page_bytes_all = 0;
        for (const ListRun& R : e->runs)
          if (e->ll[R.layer].sp.mixer == B2_MIXER_WINDOW_AND_STATE) page_bytes_all += (size_t)c.block_size * (e->ll[R.layer].nk + e->ll[R.layer].nv) * e->esz;
        page_bytes_all = std::max<size_t>(page_bytes_all, 16);
      } else if (mixed_arch) {
        page_bytes_all = 0;
        for (const ListRun& R : e->runs) {
          const ListLayer& L = e->ll[R.layer];
          if (L.sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) page_bytes_all += (size_t)c.block_size * (L.nk + L.nv) * e->esz;
          else if (L.sp.mixer == B2_MIXER_GATED_LATENT) page_bytes_all += (size_t)c.block_size * L.sp.kv_rank * e->esz;
        }
        page_bytes_all = std::max<size_t>(page_bytes_all, 16);
      } else if (ls) {
        page_bytes_all = 0;
        for (const ListLayer& L : e->ll) {
          if (heads_cache) page_bytes_all += (size_t)c.block_size * (L.nk + L.nv) * e->esz;
          else if (L.sp.kv_from < 0) page_bytes_all += (size_t)c.block_size * (L.sp.kv_rank + L.sp.rot_dim) * e->esz;
        }
      }
      int64_t nb = c.num_blocks;
      if (nb <= 0) {
        size_t free_b = 0, total_b = 0;
        E_CUDA(cudaMemGetInfo(&free_b, &total_b));
        const double frac = c.gpu_mem_fraction > 0 ? c.gpu_mem_fraction : 0.9;
        const double usable = (double)free_b - (1.0 - frac) * (double)total_b - (512.0 * 1024 * 1024);
        nb = (int64_t)(usable / (double)page_bytes_all);
        if (nb < 16) {
          b2_set_error("not enough free device memory for a KV pool (free %zu MiB)", free_b >> 20);
          rc = -12;
          goto fail;
        }
      }
      e->num_blocks = nb;
      e->layer_kv_elems = (size_t)nb * blk_elems;
      if (ls) {
        E_TRY(dalloc(&e->l_pool, (size_t)nb * page_bytes_all));
        E_CUDA(cudaMemset(e->l_pool, 0, (size_t)nb * page_bytes_all));
        size_t off = 0;
        if (state_arch) {
          for (ListRun& R : e->runs) {
            const ListLayer& L = e->ll[R.layer];
            if (L.sp.mixer != B2_MIXER_WINDOW_AND_STATE) continue;
            const size_t kb = (size_t)c.block_size * L.nk * e->esz, vb = (size_t)c.block_size * L.nv * e->esz;
            R.k_region = (int)e->regions.size();
            e->regions.push_back({e->l_pool + off, kb});
            off += (size_t)nb * kb;
            R.v_region = (int)e->regions.size();
            e->regions.push_back({e->l_pool + off, vb});
            off += (size_t)nb * vb;
          }
        }
        if (mixed_arch) {
          for (ListRun& R : e->runs) {
            const ListLayer& L = e->ll[R.layer];
            if (L.sp.mixer == B2_MIXER_MIXED_SCORE_ATTENTION) {
              const size_t kb = (size_t)c.block_size * L.nk * e->esz, vb = (size_t)c.block_size * L.nv * e->esz;
              R.k_region = (int)e->regions.size();
              e->regions.push_back({e->l_pool + off, kb});
              off += (size_t)nb * kb;
              R.v_region = (int)e->regions.size();
              e->regions.push_back({e->l_pool + off, vb});
              off += (size_t)nb * vb;
            } else if (L.sp.mixer == B2_MIXER_GATED_LATENT) {
              const size_t pb = (size_t)c.block_size * L.sp.kv_rank * e->esz;
              R.k_region = (int)e->regions.size();
              e->regions.push_back({e->l_pool + off, pb});
              off += (size_t)nb * pb;
            }
          }
        }
        for (ListLayer& L : e->ll) {
          if (state_arch || mixed_arch) break;
          if (heads_cache) {
            const size_t kb = (size_t)c.block_size * L.nk * e->esz, vb = (size_t)c.block_size * L.nv * e->esz;
            L.cache_region = (int)e->regions.size();
            e->regions.push_back({e->l_pool + off, kb});
            off += (size_t)nb * kb;
            L.v_region = (int)e->regions.size();
            e->regions.push_back({e->l_pool + off, vb});
            off += (size_t)nb * vb;
            continue;
          }
          if (L.sp.kv_from >= 0) continue;
          const size_t pb = (size_t)c.block_size * (L.sp.kv_rank + L.sp.rot_dim) * e->esz;
          L.cache_region = (int)e->regions.size();
          e->regions.push_back({e->l_pool + off, pb});
          off += (size_t)nb * pb;
        }
        for (ListLayer& L : e->ll)
          if (!state_arch && !mixed_arch && !heads_cache && L.sp.kv_from >= 0) L.cache_region = e->ll[L.sp.kv_from].cache_region;
      } else {
        E_TRY(dalloc(&e->kv_pool, (size_t)2 * c.num_layers * e->layer_kv_elems));
        E_CUDA(cudaMemset(e->kv_pool, 0, (size_t)2 * c.num_layers * e->layer_kv_elems * 2));
        for (int r = 0; r < 2 * c.num_layers; ++r)
          e->regions.push_back({reinterpret_cast<char*>(e->kv_pool + (size_t)r * e->layer_kv_elems), blk_elems * 2});
      }
      e->free_blocks.reserve(nb);
      for (int64_t b = nb - 1; b >= 1; --b) e->free_blocks.push_back((int32_t)b);  // page 0 = null page
      e->blk_ref.assign(nb, 0);
      e->blk_hash.assign(nb, 0);
      e->blk_parent.assign(nb, -1);
      e->blk_tokens.assign((size_t)nb * c.block_size, 0);
      e->pc_lru_pos.assign(nb, e->pc_lru.end());
      e->pc_in_lru.assign(nb, 0);
      e->prefix_cache = env_int("B2_PREFIX_CACHE", 0) != 0;
    }
    if (e->force_gemm_impl == 0 || e->simt_max_tokens > 0) E_TRY(ensure_logits(e));  // SIMT lm_head writes logits
    e->ev_pool.resize(2 * 400);
    for (auto& ev : e->ev_pool) E_CUDA(cudaEventCreate(&ev));
    if (safetensors_path) {
      E_TRY(load_safetensors(e, safetensors_path));
      E_TRY(b2_engine_finalize(e));
    }
  }
  *out = e;
  return 0;
fail:
  b2_engine_free(e);
  return rc;
#undef E_TRY
#undef E_CUDA
}

extern "C" int b2_engine_load_tensor(b2_engine* e, const char* hf_name, const void* host_bf16, size_t nbytes) {
  B2_REQUIRE(e && hf_name && host_bf16, "b2_engine_load_tensor: null argument");
  B2_CUDA_OK(cudaSetDevice(e->device));
  return layer_tensor(e, hf_name, host_bf16, nbytes);
}

extern "C" int b2_engine_load_int_tensor(b2_engine* e, const char* name, const int32_t* host_i32, size_t count) {
  B2_REQUIRE(e && name && host_i32, "b2_engine_load_int_tensor: null argument");
  B2_REQUIRE(list_arch(e->cfg.arch), "b2_engine_load_int_tensor: this family has no integer tensors");
  B2_CUDA_OK(cudaSetDevice(e->device));
  return list_int_tensor(e, name, host_i32, count);
}

extern "C" int b2_engine_load_safetensors(b2_engine* e, const char* path) {
  B2_REQUIRE(e && path, "b2_engine_load_safetensors: null argument");
  B2_CUDA_OK(cudaSetDevice(e->device));
  return load_safetensors(e, path);
}

extern "C" int b2_engine_finalize(b2_engine* e) {
  B2_REQUIRE(e, "b2_engine_finalize: null engine");
  const int arch = e->cfg.arch;
  if (arch == B2_ARCH_BUMALIX || arch == B2_ARCH_TINEVIK) {
    B2_CUDA_OK(cudaSetDevice(e->device));
    B2_TRY(arch == B2_ARCH_BUMALIX ? state_finalize(e) : mixed_finalize(e));
    e->finalized = true;
    return 0;
  }
  if (list_arch(arch)) {
    const int want = list_tensor_count(e);
    int have = 0;
    for (auto& kv : e->loaded)
      if (kv.first.size() < 9 || kv.first.compare(kv.first.size() - 9, 9, ".mix.vmix") != 0) ++have;
    for (size_t l = 0; l < e->ll.size(); ++l)   // the blend weight: needed by the layers that blend, harmless elsewhere
      B2_REQUIRE(e->ll[l].vmix_mode != 2 || e->loaded.count("l" + std::to_string(l) + ".mix.vmix"), "weights incomplete: l%zu.mix.vmix missing", l);
    B2_REQUIRE(have == want, "weights incomplete: %d of %d tensors loaded", have, want);
    e->finalized = true;
    return 0;
  }
  const int per_layer = arch == B2_ARCH_QWEN3 ? 11 : arch == B2_ARCH_PHI3 ? 6 : 16;
  const int want = (arch == B2_ARCH_OPT ? 4 : 2) + e->cfg.num_layers * per_layer;
  int have = 0;
  for (auto& kv : e->loaded)
    if (kv.first != "lm_head.weight") ++have;
  if (!e->cfg.tie_embeddings) {
    B2_REQUIRE(e->loaded.count("lm_head.weight"), "weights incomplete: lm_head.weight missing (untied head)");
  }
  B2_REQUIRE(have == want, "weights incomplete: %d of %d tensors loaded", have, want);
  e->finalized = true;
  return 0;
}

extern "C" void b2_engine_free(b2_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  for (auto& kv : e->graphs) cudaGraphExecDestroy(kv.second);
  for (auto& ev : e->ev_pool)
    if (ev) cudaEventDestroy(ev);
  auto F = [](void* p) {
    if (p) cudaFree(p);
  };
  if (e->lm_head != e->embed) F(e->lm_head);
  F(e->embed); F(e->final_norm); F(e->cos_sin); F(e->final_norm_b); F(e->pos_embed);
  for (auto& L : e->layers) {
    F(L.ln1); F(L.ln2); F(L.qnorm); F(L.knorm); F(L.wqkv); F(L.wo); F(L.wgu); F(L.wd);
    F(L.bqkv); F(L.bo); F(L.ln1_b); F(L.ln2_b); F(L.b1); F(L.b2);
  }
  F(e->kv_pool); F(e->h); F(e->x); F(e->qkv); F(e->qrot); F(e->attn); F(e->gu); F(e->act); F(e->proj); F(e->xlast);
  F(e->partial); F(e->attn_scratch); F(e->d_tokens); F(e->d_positions); F(e->d_seq_lens); F(e->d_slots);
  F(e->d_block_table); F(e->d_last_rows); F(e->d_out_tokens); F(e->d_token_log); F(e->d_step); F(e->d_argmax); F(e->d_pf_frac); F(e->d_sample_out); F(e->d_sample_rows); F(e->d_gbar); F(e->d_gbar2); F(e->d_ss);
  F(e->d_tiles); F(e->dbg_hidden); F(e->logits);
  if (e->h_stage) cudaFreeHost(e->h_stage);
  if (e->h_tiles) cudaFreeHost(e->h_tiles);
  if (e->h_out) cudaFreeHost(e->h_out);
  if (e->h_tok) cudaFreeHost(e->h_tok);
  if (e->ev_tok) cudaEventDestroy(e->ev_tok);
  F(e->partial2); F(e->attn_scratch2); F(e->ssq);
  if (e->l_head == e->l_embed) e->l_head = nullptr;   // (a tied head is the embedding table)
  F(e->l_final_bias);
  F(e->l_embed); F(e->l_head); F(e->l_embed_gain); F(e->l_final_gain); F(e->l_pool); F(e->l_h); F(e->l_qd); F(e->l_qrot); F(e->l_qabs);
  F(e->l_xperm); F(e->l_upf); if (e->h_offsets) cudaFreeHost(e->h_offsets);
  F(e->l_q); F(e->l_vfirst); F(e->l_cross); F(e->l_qb); F(e->d_row_seq); F(e->d_row_first); F(e->d_row_end);
  F(e->l_mix); F(e->l_y); F(e->l_rw); F(e->l_logits); F(e->l_x1); F(e->l_x2); F(e->l_qnope); F(e->l_olat); F(e->l_av); F(e->l_act); F(e->l_xl);
  F(e->l_attn_scratch); F(e->l_idx); F(e->l_offsets); F(e->l_slot_token); F(e->l_pair_slot); F(e->l_tile_group); F(e->l_tile_row0); F(e->l_ntiles); F(e->dbg_hidden_f32);
  for (auto& L : e->ll) {
    F(L.wqd); F(L.ukT); F(L.uv); F(L.wo); F(L.up); F(L.down); F(L.gain1); F(L.gain2); F(L.lat_gain); F(L.sink); F(L.router); F(L.corr);
    F(L.gain1b); F(L.gain2b); F(L.qkv_bias); F(L.o_bias); F(L.conv_w); F(L.talk); F(L.vmix); F(L.conv_ring);
    F(L.wo2); F(L.sh_up); F(L.sh_down); F(L.qk_gain); F(L.head_gain); F(L.a2); F(L.a2_bias); F(L.g2); F(L.a_log); F(L.out_gain_l); F(L.out_gain_r); F(L.poly);
    F(L.bias1); F(L.bias1b); F(L.bias2); F(L.bias2b); F(L.latq_gain); F(L.uq); F(L.table);
  }
  for (auto& R : e->runs) {
    F(R.state); F(R.ring);
  }
  for (auto& ev : e->l_ev)
    if (ev) cudaEventDestroy(ev);
  for (auto& sd : e->l_side)
    if (sd) cudaStreamDestroy(sd);
  F(e->l_upf2); F(e->l_act2); F(e->l_loop_in); F(e->l_cat); F(e->l_av2); F(e->l_dec); F(e->l_beta); F(e->l_gate); F(e->l_so); F(e->l_mix2); F(e->l_ffd); F(e->l_slot_scale);
  if (e->ev_fork) cudaEventDestroy(e->ev_fork);
  if (e->ev_join) cudaEventDestroy(e->ev_join);
  if (e->stream2) cudaStreamDestroy(e->stream2);
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
}

extern "C" int b2_engine_info(b2_engine* e, int64_t* num_blocks, int64_t* free_blocks, int64_t* weight_bytes) {
  B2_REQUIRE(e, "b2_engine_info: null engine");
  if (num_blocks) *num_blocks = e->num_blocks;
  if (free_blocks) *free_blocks = pages_available(e);  // cached pages nobody holds are reusable at once
  if (weight_bytes) *weight_bytes = e->weight_bytes;
  return 0;
}

extern "C" int b2_seq_create(b2_engine* e, int32_t reserve_tokens, int32_t* seq_id) {
  B2_REQUIRE(e && seq_id, "b2_seq_create: null argument");
  B2_REQUIRE(reserve_tokens >= 1 && reserve_tokens <= e->cfg.max_model_len, "reserve_tokens %d outside [1, max_model_len=%d]",
             reserve_tokens, e->cfg.max_model_len);
  const int bs = e->cfg.block_size;
  const int need = (reserve_tokens + bs - 1) / bs;
  if (pages_available(e) < need) {
    b2_set_error("KV pool exhausted: need %d pages, %lld free", need, (long long)pages_available(e));
    return -12;
  }
  int id = -1;
  for (int i = 0; i < (int)e->seqs.size(); ++i)
    if (!e->seqs[i].active) {
      id = i;
      break;
    }
  if (id < 0) {
    b2_set_error("all %d sequence slots in use", e->cfg.max_seqs);
    return -11;
  }
  Seq& s = e->seqs[id];
  s.active = true;
  s.len = 0;
  s.reserved = need * bs;
  s.blocks.clear();
  for (int i = 0; i < need; ++i) s.blocks.push_back(take_page(e));
  s.chain.clear();
  s.pending.clear();
  s.chain_open = e->prefix_cache;
  *seq_id = id;
  return 0;
}

extern "C" int b2_seq_reserve(b2_engine* e, int32_t seq_id, int32_t total_tokens) {
  B2_REQUIRE(e, "b2_seq_reserve: null engine");
  B2_TRY(check_seq(e, seq_id));
  Seq& s = e->seqs[seq_id];
  B2_REQUIRE(total_tokens >= 1 && total_tokens <= e->cfg.max_model_len, "total_tokens %d outside [1, max_model_len=%d]", total_tokens,
             e->cfg.max_model_len);
  const int bs = e->cfg.block_size;
  const int need = (total_tokens + bs - 1) / bs - (int)s.blocks.size();
  if (need <= 0) return 0;
  if (pages_available(e) < need) {
    b2_set_error("KV pool exhausted: need %d more pages, %lld free", need, (long long)pages_available(e));
    return -12;
  }
  for (int i = 0; i < need; ++i) s.blocks.push_back(take_page(e));
  s.reserved = (int)s.blocks.size() * bs;
  e->cur_batch.clear();  // the device copy of this sequence's block-table row is stale
  return 0;
}

extern "C" int b2_seq_free(b2_engine* e, int32_t seq_id) {
  B2_REQUIRE(e, "b2_seq_free: null engine");
  B2_TRY(check_seq(e, seq_id));
  Seq& s = e->seqs[seq_id];
  // leading pages first, so that on the LRU list a prefix outlives its continuations
  for (auto it = s.blocks.rbegin(); it != s.blocks.rend(); ++it) release_page(e, *it);
  s.blocks.clear();
  s.chain.clear();
  s.pending.clear();
  s.chain_open = false;
  s.active = false;
  s.len = 0;
  e->cur_batch.clear();
  return 0;
}

extern "C" int b2_seq_len(b2_engine* e, int32_t seq_id) {
  if (!e || check_seq(e, seq_id) != 0) return -22;
  return e->seqs[seq_id].len;
}

extern "C" int b2_seq_truncate(b2_engine* e, int32_t seq_id, int32_t new_len) {
  B2_REQUIRE(e, "b2_seq_truncate: null engine");
  B2_TRY(check_seq(e, seq_id));
  Seq& s = e->seqs[seq_id];
  B2_REQUIRE(new_len >= 0 && new_len <= s.len, "b2_seq_truncate: new_len %d outside [0, %d]", new_len, s.len);
  // State besides the cache (the convolutions' last projected rows) exists for the sequence's end only: it cannot be cut back
  // to an earlier position, only kept (new_len == len) or started over (new_len == 0).
  B2_REQUIRE(!e->l_has_state || new_len == s.len || new_len == 0, "b2_seq_truncate: this model keeps per-sequence state; a sequence can only be cut back to 0");
  // Positions >= new_len will be written again.  Pages from there on that are registered in the prefix cache or held by
  // other sequences too must not be: the sequence swaps them for private pages (copying the kept part of the page
  // new_len falls into), and its own chain ends at the cut.
  const int bs = e->cfg.block_size;
  const int first = new_len / bs;
  int need = 0;
  for (int j = first; j < (int)s.blocks.size(); ++j)
    if (e->blk_hash[s.blocks[j]] != 0 || e->blk_ref[s.blocks[j]] > 1) ++need;
  if (need > 0) {
    B2_REQUIRE(pages_available(e) >= need, "b2_seq_truncate: no free pages to un-share %d cached pages", need);
    B2_CUDA_OK(cudaSetDevice(e->device));
    B2_CUDA_OK(cudaStreamSynchronize(e->stream));
    for (int j = first; j < (int)s.blocks.size(); ++j) {
      const int32_t old_b = s.blocks[j];
      if (e->blk_hash[old_b] == 0 && e->blk_ref[old_b] <= 1) continue;
      const int32_t nb = take_page(e);
      if (j == first && new_len % bs != 0) {
        for (const auto& rg : e->regions)
          B2_CUDA_OK(cudaMemcpyAsync(rg.base + (size_t)nb * rg.page_bytes, rg.base + (size_t)old_b * rg.page_bytes, rg.page_bytes,
                                     cudaMemcpyDeviceToDevice, e->stream));
      }
      s.blocks[j] = nb;
      release_page(e, old_b);
    }
    B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  }
  if ((int)s.chain.size() > first) s.chain.resize(first);
  s.pending.clear();
  s.chain_open = false;
  s.len = new_len;
  e->cur_batch.clear();
  return 0;
}

namespace {
int prefill_impl(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq, const int32_t* seq_ids, const int32_t* rows,
                 int32_t nrows, float* out_logits, int32_t* out_tokens);
}
extern "C" int b2_prefill(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq, const int32_t* seq_ids,
                          int32_t* out_tokens) {
  return prefill_impl(e, ids, seq_offsets, nseq, seq_ids, nullptr, 0, nullptr, out_tokens);
}
extern "C" int b2_prefill_logits(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq, const int32_t* seq_ids,
                                 const int32_t* rows, int32_t nrows, float* out_logits, int32_t* out_tokens) {
  B2_REQUIRE(e && nrows >= 0 && (nrows == 0 || (rows && out_logits)), "b2_prefill_logits: bad arguments");
  B2_REQUIRE(list_arch(e->cfg.arch), "b2_prefill_logits: built for the families whose lm_head writes fp32 rows (the layer-list families)");
  return prefill_impl(e, ids, seq_offsets, nseq, seq_ids, rows, nrows, out_logits, out_tokens);
}
namespace {
int prefill_impl(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq, const int32_t* seq_ids, const int32_t* rows,
                 int32_t nrows, float* out_logits, int32_t* out_tokens) {
  B2_REQUIRE(e && ids && seq_offsets && seq_ids && nseq >= 1, "b2_prefill: bad arguments");
  B2_REQUIRE(e->finalized, "b2_prefill: weights not finalized");
  B2_REQUIRE(nseq <= e->cfg.max_seqs, "b2_prefill: %d sequences > max_seqs %d", nseq, e->cfg.max_seqs);
  B2_CUDA_OK(cudaSetDevice(e->device));
  const int T_in = seq_offsets[nseq] - seq_offsets[0];
  B2_REQUIRE(T_in >= 1 && T_in <= e->cap_tokens && T_in <= e->cfg.max_batch_tokens, "b2_prefill: %d tokens exceed max_batch_tokens %d", T_in,
             e->cfg.max_batch_tokens);
  const int bs = e->cfg.block_size;
  // ---- validate, then let fresh sequences take what the prefix cache already holds of their prompt ----
  std::vector<int> skip(nseq, 0);
  for (int i = 0; i < nseq; ++i) {
    B2_TRY(check_seq(e, seq_ids[i]));
    Seq& s = e->seqs[seq_ids[i]];
    const int n = seq_offsets[i + 1] - seq_offsets[i];
    B2_REQUIRE(n >= 1, "b2_prefill: sequence %d has no tokens", i);
    B2_REQUIRE(s.len + n <= s.reserved, "b2_prefill: sequence %d would exceed its reservation (%d + %d > %d)", seq_ids[i], s.len, n,
               s.reserved);
  }
  for (int i = 0; i < nseq; ++i) {
    Seq& s = e->seqs[seq_ids[i]];
    const int n = seq_offsets[i + 1] - seq_offsets[i];
    if (e->prefix_cache && !e->l_has_state && nrows == 0 && s.len == 0 && s.chain_open && s.chain.empty()) {   // (state besides the cache cannot be skipped into)
      skip[i] = pc_match(e, s, ids + seq_offsets[i], n);
      s.len = skip[i];  // K/V of those positions are in the pages just taken
      e->pc_queries += n;
      e->pc_hits += skip[i];
    }
  }
  int T = 0;
  for (int i = 0; i < nseq; ++i) T += seq_offsets[i + 1] - seq_offsets[i] - skip[i];
  int32_t* tok = e->h_stage;
  int32_t* pos = tok + T;
  int32_t* slots = pos + T;
  int32_t* last = slots + T;
  int32_t* bt = last + nseq + nrows;
  B2_REQUIRE(nrows == 0 || (nseq + nrows <= e->l_rows_cap && (size_t)(bt - e->h_stage) + (size_t)nseq * e->bt_stride <= e->h_stage_ints),
             "b2_prefill_logits: %d rows exceed the engine's capacity", nrows);
  for (int i = 0; i < nrows; ++i) {
    B2_REQUIRE(rows[i] >= 0 && rows[i] < T_in, "b2_prefill_logits: row %d outside the call's %d tokens", rows[i], T_in);
    last[nseq + i] = rows[i];  // (no prefix-cache skip in this form: rows index the tokens as given)
  }
  // families with per-sequence state besides the cache: every token row's sequence slot and the row range of its portion
  int32_t* rowinfo = e->d_row_seq ? bt + (size_t)nseq * e->bt_stride : nullptr;
  B2_REQUIRE(!rowinfo || (size_t)(rowinfo - e->h_stage) + (size_t)3 * T <= e->h_stage_ints, "b2_prefill: %d tokens exceed the staging buffer", T);
  int ntiles = 0, row0 = 0;
  for (int i = 0; i < nseq; ++i) {
    Seq& s = e->seqs[seq_ids[i]];
    const int n = seq_offsets[i + 1] - seq_offsets[i] - skip[i];
    const int32_t* src = ids + seq_offsets[i] + skip[i];
    for (int j = 0; j < n; ++j) {
      const int p = s.len + j;
      tok[row0 + j] = src[j];
      pos[row0 + j] = p;
      slots[row0 + j] = s.blocks[p / bs] * bs + p % bs;
    }
    if (rowinfo)
      for (int j = 0; j < n; ++j) {
        rowinfo[row0 + j] = seq_ids[i];
        rowinfo[T + row0 + j] = row0;
        rowinfo[2 * T + row0 + j] = row0 + n;
      }
    last[i] = row0 + n - 1;
    memset(bt + (size_t)i * e->bt_stride, 0, (size_t)e->bt_stride * 4);
    memcpy(bt + (size_t)i * e->bt_stride, s.blocks.data(), s.blocks.size() * 4);
    const int first_tile = ntiles;
    for (int j = 0; j < n; j += 64) {
      B2_REQUIRE(ntiles < e->tiles_cap, "b2_prefill: too many attention tiles");
      e->h_tiles[ntiles++] = PrefillTile{row0 + j, s.len + j, std::min(64, n - j), i};
    }
    if (prefill_tile_pairs(e) && ((ntiles - first_tile) & 1)) {  // attn_prefill_tc.cu, pair mode: tiles 2i and 2i + 1 belong together
      B2_REQUIRE(ntiles < e->tiles_cap, "b2_prefill: too many attention tiles");
      e->h_tiles[ntiles++] = PrefillTile{row0, s.len + n, 0, i};
    }
    row0 += n;
  }
  B2_CUDA_OK(cudaMemcpyAsync(e->d_tokens, tok, T * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_positions, pos, T * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_slots, slots, T * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_last_rows, last, (nseq + nrows) * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_block_table, bt, (size_t)nseq * e->bt_stride * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaMemcpyAsync(e->d_tiles, e->h_tiles, ntiles * sizeof(PrefillTile), cudaMemcpyHostToDevice, e->stream));
  if (rowinfo) {
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_seq, rowinfo, T * 4, cudaMemcpyHostToDevice, e->stream));
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_first, rowinfo + T, T * 4, cudaMemcpyHostToDevice, e->stream));
    B2_CUDA_OK(cudaMemcpyAsync(e->d_row_end, rowinfo + 2 * T, T * 4, cudaMemcpyHostToDevice, e->stream));
  }
  if (e->debug_flags & 2) B2_TRY(ensure_logits(e));
  e->cur_batch.clear();
  e->step_portions = nseq;
  B2_TRY(forward(e, T, ntiles, nseq + nrows, 1));
  // the produced tokens become the device-resident "next input" of these sequences
  B2_CUDA_OK(cudaMemcpyAsync(e->h_out, e->d_out_tokens, nseq * 4, cudaMemcpyDeviceToHost, e->stream));
  if (nrows > 0)
    B2_CUDA_OK(cudaMemcpyAsync(out_logits, e->l_logits + (size_t)nseq * e->cfg.vocab, (size_t)nrows * e->cfg.vocab * 4, cudaMemcpyDeviceToHost,
                               e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  for (int i = 0; i < nseq; ++i) {
    Seq& s = e->seqs[seq_ids[i]];
    const int n = seq_offsets[i + 1] - seq_offsets[i] - skip[i];
    s.len += n;
    s.next_token = e->h_out[i];
    s.next_valid = true;
    if (e->prefix_cache) pc_register(e, s, ids + seq_offsets[i] + skip[i], n);  // the forward that filled the pages is complete
  }
  if (out_tokens) memcpy(out_tokens, e->h_out, nseq * 4);
  // remember them host-side too so the first decode step can seed d_tokens
  e->last_n = nseq;
  e->last_tokens = T;
  return 0;
}
}  // namespace

namespace {
// Prepares device state for a decode step over seq_ids; returns padded batch B.
int prepare_decode(b2_engine* e, int n, const int32_t* seq_ids, const int32_t* in_tokens, int* B_out, int* split_out) {
  B2_REQUIRE(e->finalized, "decode: weights not finalized");
  B2_REQUIRE(n >= 1 && n <= e->cfg.max_seqs, "decode: batch %d outside [1, max_seqs=%d]", n, e->cfg.max_seqs);
  int max_len = 0;
  for (int i = 0; i < n; ++i) {
    B2_TRY(check_seq(e, seq_ids[i]));
    Seq& s = e->seqs[seq_ids[i]];
    B2_REQUIRE(s.len >= 1, "decode: sequence %d has no prefilled tokens", seq_ids[i]);
    B2_REQUIRE(s.len + 1 <= s.reserved, "decode: sequence %d would exceed its reservation (%d tokens)", seq_ids[i], s.reserved);
    s.chain_open = false;  // generated tokens are not registered in the prefix cache
    max_len = std::max(max_len, s.len + 1);
  }
  const int B = e->cfg.use_cuda_graphs ? bucket_batch(n) : n;
  const bool same = (int)e->cur_batch.size() == n && e->cur_B == B && std::equal(seq_ids, seq_ids + n, e->cur_batch.begin());
  if (!same) {
    // The batch composition changed: the device-resident "next tokens" belong to another batch
    // order, so seed this batch from the host copies kept per sequence (or from in_tokens).
    if (in_tokens == nullptr) {
      for (int i = 0; i < n; ++i) {
        Seq& s = e->seqs[seq_ids[i]];
        B2_REQUIRE(s.next_valid, "decode: batch changed and sequence %d has no host copy of its next token; pass in_tokens",
                   seq_ids[i]);
        e->h_stage[i] = s.next_token;
      }
      for (int i = n; i < B; ++i) e->h_stage[i] = 0;
      B2_CUDA_OK(cudaMemcpyAsync(e->d_tokens, e->h_stage, B * 4, cudaMemcpyHostToDevice, e->stream));
      B2_CUDA_OK(cudaStreamSynchronize(e->stream));
    }
    B2_TRY(upload_decode_batch(e, n, seq_ids, B));
  }
  if (in_tokens != nullptr) {
    // dedicated pinned slot for the per-step token upload; the event keeps a later call from
    // overwriting it while the copy is still in flight (callers may skip the D2H sync)
    B2_CUDA_OK(cudaEventSynchronize(e->ev_tok));
    memcpy(e->h_tok, in_tokens, n * 4);
    for (int i = n; i < B; ++i) e->h_tok[i] = 0;
    B2_CUDA_OK(cudaMemcpyAsync(e->d_tokens, e->h_tok, B * 4, cudaMemcpyHostToDevice, e->stream));
    B2_CUDA_OK(cudaEventRecord(e->ev_tok, e->stream));
  }
  *B_out = B;
  *split_out = pick_attn_split(e, B, max_len);
  return 0;
}
}  // namespace

namespace {
int fetch_next_tokens(b2_engine* e, int nseq, const int32_t* seq_ids) {
  int32_t* tmp = e->h_stage;
  B2_CUDA_OK(cudaMemcpyAsync(tmp, e->d_out_tokens, nseq * 4, cudaMemcpyDeviceToHost, e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  for (int i = 0; i < nseq; ++i) {
    e->seqs[seq_ids[i]].next_token = tmp[i];
    e->seqs[seq_ids[i]].next_valid = true;
  }
  return 0;
}
}  // namespace

extern "C" int b2_decode_step(b2_engine* e, int32_t nseq, const int32_t* seq_ids, const int32_t* in_tokens, int32_t* out_tokens) {
  B2_REQUIRE(e && seq_ids, "b2_decode_step: null argument");
  B2_CUDA_OK(cudaSetDevice(e->device));
  int B = 0, split = 1;
  B2_TRY(prepare_decode(e, nseq, seq_ids, in_tokens, &B, &split));
  if (e->debug_flags & 2) B2_TRY(ensure_logits(e));
  B2_TRY(run_decode_step(e, B, split));
  for (int i = 0; i < nseq; ++i) e->seqs[seq_ids[i]].len += 1;
  e->last_n = nseq;
  e->last_tokens = nseq;
  if (out_tokens) {
    B2_CUDA_OK(cudaMemcpyAsync(e->h_out, e->d_out_tokens, nseq * 4, cudaMemcpyDeviceToHost, e->stream));
    B2_CUDA_OK(cudaStreamSynchronize(e->stream));
    memcpy(out_tokens, e->h_out, nseq * 4);
    for (int i = 0; i < nseq; ++i) {
      e->seqs[seq_ids[i]].next_token = e->h_out[i];
      e->seqs[seq_ids[i]].next_valid = true;
    }
  } else {
    for (int i = 0; i < nseq; ++i) e->seqs[seq_ids[i]].next_valid = false;
  }
  return 0;
}

extern "C" int b2_decode_run(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t steps, int32_t* out_tokens,
                             float* elapsed_ms) {
  B2_REQUIRE(e && seq_ids && steps >= 1, "b2_decode_run: bad arguments");
  B2_REQUIRE(steps <= e->log_cap_steps, "b2_decode_run: steps %d > %d", steps, e->log_cap_steps);
  B2_CUDA_OK(cudaSetDevice(e->device));
  for (int i = 0; i < nseq; ++i) {
    B2_TRY(check_seq(e, seq_ids[i]));
    Seq& s = e->seqs[seq_ids[i]];
    B2_REQUIRE(s.len + steps <= s.reserved, "b2_decode_run: sequence %d reservation too small for %d steps", seq_ids[i], steps);
  }
  int B = 0, split = 1;
  B2_TRY(prepare_decode(e, nseq, seq_ids, nullptr, &B, &split));
  B2_CUDA_OK(cudaMemsetAsync(e->d_step, 0, 4, e->stream));
  // the graph is captured before the timed region; the event pair brackets exactly `steps` steps
  cudaEvent_t ev0 = e->ev_pool[e->ev_pool.size() - 2], ev1 = e->ev_pool[e->ev_pool.size() - 1];
  int done = 0;
  {
    int max_len = 0;
    for (int i = 0; i < nseq; ++i) max_len = std::max(max_len, e->seqs[seq_ids[i]].len + steps);
    split = pick_attn_split(e, B, max_len);  // one graph for the whole run
  }
  if (graphs_enabled(e)) B2_TRY(ensure_graph(e, B, split));
  B2_CUDA_OK(cudaEventRecord(ev0, e->stream));
  for (; done < steps; ++done) B2_TRY(run_decode_step(e, B, split));
  B2_CUDA_OK(cudaEventRecord(ev1, e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  if (elapsed_ms) B2_CUDA_OK(cudaEventElapsedTime(elapsed_ms, ev0, ev1));
  for (int i = 0; i < nseq; ++i) e->seqs[seq_ids[i]].len += steps;
  e->last_n = nseq;
  e->last_tokens = nseq;
  B2_TRY(fetch_next_tokens(e, nseq, seq_ids));
  if (out_tokens) {
    B2_CUDA_OK(cudaMemcpy(e->h_out, e->d_token_log, (size_t)steps * e->cfg.max_seqs * 4, cudaMemcpyDeviceToHost));
    for (int st = 0; st < steps; ++st)
      memcpy(out_tokens + (size_t)st * nseq, e->h_out + (size_t)st * e->cfg.max_seqs, nseq * 4);
  }
  return 0;
}

extern "C" int b2_decode_profile(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t steps, float* ms_by_class,
                                 int64_t* launches_by_class) {
  B2_REQUIRE(e && seq_ids && steps >= 1 && ms_by_class && launches_by_class, "b2_decode_profile: bad arguments");
  B2_CUDA_OK(cudaSetDevice(e->device));
  for (int k = 0; k < B2_NUM_KERNEL_CLASSES; ++k) {
    ms_by_class[k] = 0.f;
    launches_by_class[k] = 0;
  }
  for (int st = 0; st < steps; ++st) {
    int B = 0, split = 1;
    B2_TRY(prepare_decode(e, nseq, seq_ids, nullptr, &B, &split));
    e->profiling = true;
    e->ev_next = 0;
    e->ev_used.clear();
    int rc = run_decode_step(e, B, split);
    e->profiling = false;
    B2_TRY(rc);
    B2_CUDA_OK(cudaStreamSynchronize(e->stream));
    for (auto& u : e->ev_used) {
      float ms = 0.f;
      B2_CUDA_OK(cudaEventElapsedTime(&ms, e->ev_pool[u.second], e->ev_pool[u.second + 1]));
      ms_by_class[u.first] += ms;
      launches_by_class[u.first] += 1;
    }
    for (int i = 0; i < nseq; ++i) e->seqs[seq_ids[i]].len += 1;
  }
  e->last_n = nseq;
  e->last_tokens = nseq;
  B2_TRY(fetch_next_tokens(e, nseq, seq_ids));
  return 0;
}

extern "C" int b2_attn_profile(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t reps, float* ms_per_launch,
                               int64_t* kv_bytes_per_launch) {
  B2_REQUIRE(e && seq_ids && reps >= 1 && ms_per_launch && kv_bytes_per_launch, "b2_attn_profile: bad arguments");
  B2_CUDA_OK(cudaSetDevice(e->device));
  B2_REQUIRE(!list_arch(e->cfg.arch), "b2_attn_profile: times the GQA decode-attention kernel; this family has none");
  B2_REQUIRE((int)e->cur_batch.size() == nseq && std::equal(seq_ids, seq_ids + nseq, e->cur_batch.begin()),
             "b2_attn_profile: run a decode step on exactly this batch first (the pass reuses its device-side page tables)");
  const b2_config& c = e->cfg;
  int64_t bytes = 0;
  for (int i = 0; i < nseq; ++i) bytes += (int64_t)(e->seqs[seq_ids[i]].len + 1) * e->nkv * e->hd * 2 * 2;
  const int B = e->cur_B;
  auto pass = [&]() -> int {
    for (int l = 0; l < c.num_layers; ++l) {
      bf16* kp = e->kv_pool + (size_t)(2 * l) * e->layer_kv_elems;
      bf16* vp = kp + e->layer_kv_elems;
      B2_TRY(launch_attn_decode(e->qrot, kp, vp, e->d_block_table, e->bt_stride, e->d_seq_lens, e->attn_scratch, e->attn, B,
                                e->nq, e->nkv, e->hd, c.block_size, e->stream, e->attn_scale));
    }
    return 0;
  };
  cudaEvent_t a, b;
  B2_CUDA_OK(cudaEventCreate(&a));
  B2_CUDA_OK(cudaEventCreate(&b));
  int rc = pass();  // warm-up; each layer's K/V (B x S x 4 KB) is a different region, so no pass finds its pages in L2
  if (rc == 0) rc = cudaEventRecord(a, e->stream) == cudaSuccess ? 0 : -5;
  for (int r = 0; r < reps && rc == 0; ++r) rc = pass();
  if (rc == 0) rc = cudaEventRecord(b, e->stream) == cudaSuccess ? 0 : -5;
  if (rc == 0) rc = cudaEventSynchronize(b) == cudaSuccess ? 0 : -5;
  float ms = 0.f;
  if (rc == 0) rc = cudaEventElapsedTime(&ms, a, b) == cudaSuccess ? 0 : -5;
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  if (rc != 0) {
    if (rc == -5) b2_set_error("b2_attn_profile: CUDA error: %s", cudaGetErrorString(cudaGetLastError()));
    return rc;
  }
  *ms_per_launch = ms / (float)(reps * c.num_layers);
  *kv_bytes_per_launch = bytes;
  return 0;
}

extern "C" int64_t b2_launch_count(b2_engine* e) { return e ? e->launches : 0; }

extern "C" int b2_prefix_cache_stats(b2_engine* e, int64_t* queried_tokens, int64_t* hit_tokens, int64_t* cached_pages) {
  B2_REQUIRE(e, "b2_prefix_cache_stats: null engine");
  if (queried_tokens) *queried_tokens = e->pc_queries;
  if (hit_tokens) *hit_tokens = e->pc_hits;
  if (cached_pages) *cached_pages = (int64_t)e->pc_map.size();
  return 0;
}

extern "C" int b2_set_tuning(b2_engine* e, int32_t key, int64_t value) {
  B2_REQUIRE(e, "b2_set_tuning: null engine");
  B2_CUDA_OK(cudaSetDevice(e->device));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  switch (key) {
    case B2_TUNE_SKIP_MASK: e->skip_mask = (unsigned)value; break;
    case B2_TUNE_PREFIX_CACHE:
      e->prefix_cache = value != 0;
      if (!e->prefix_cache) {  // forget everything: registered pages nobody holds go back to the free list
        for (int32_t b : e->pc_lru) {
          e->pc_in_lru[b] = 0;
          e->free_blocks.push_back(b);
        }
        e->pc_lru.clear();
        e->pc_map.clear();
        std::fill(e->blk_hash.begin(), e->blk_hash.end(), 0);
      }
      break;
    case B2_TUNE_TWO_LANE:
      B2_REQUIRE(value == 0 || e->stream2 != nullptr, "b2_set_tuning: this engine was created without a second lane (B2_MB=0 or OPT)");
      e->mb_min_batch = (int)value;
      break;
    default: b2_set_error("b2_set_tuning: unknown key %d", key); return -22;
  }
  for (auto& kv : e->graphs) cudaGraphExecDestroy(kv.second);  // captured with the old setting
  e->graphs.clear();
  e->graph_nodes.clear();
  return 0;
}

extern "C" int b2_set_debug(b2_engine* e, int32_t flags) {
  B2_REQUIRE(e, "b2_set_debug: null engine");
  B2_CUDA_OK(cudaSetDevice(e->device));
  e->debug_flags = flags;
  if ((flags & 1) && list_arch(e->cfg.arch)) {
    if (e->dbg_hidden_f32 == nullptr) {
      e->dbg_cap_tokens = std::min(e->cap_tokens, 1024);
      if (e->dbg_slots <= 0) e->dbg_slots = e->cfg.num_layers + 1;
      B2_TRY(dalloc(&e->dbg_hidden_f32, (size_t)e->dbg_slots * e->dbg_cap_tokens * e->cfg.hidden));
    }
  } else if ((flags & 1) && e->dbg_hidden == nullptr) {
    e->dbg_cap_tokens = std::min(e->cap_tokens, 1024);
    B2_TRY(dalloc(&e->dbg_hidden, (size_t)(e->cfg.num_layers + 2) * e->dbg_cap_tokens * e->cfg.hidden));
  }
  if (flags & 2) B2_TRY(ensure_logits(e));
  return 0;
}

extern "C" int b2_get_hidden(b2_engine* e, int32_t layer, int32_t ntokens, uint16_t* out_bf16) {
  B2_REQUIRE(e && out_bf16, "b2_get_hidden: null argument");
  B2_REQUIRE(!list_arch(e->cfg.arch), "b2_get_hidden: this family's residual stream is fp32 (b2_get_hidden_f32)");
  B2_REQUIRE((e->debug_flags & 1) && e->dbg_hidden, "b2_get_hidden: hidden capture not enabled (b2_set_debug(e, 1))");
  B2_REQUIRE(layer >= -1 && layer <= e->cfg.num_layers, "b2_get_hidden: layer %d out of range", layer);
  B2_REQUIRE(ntokens >= 1 && ntokens <= e->dbg_cap_tokens && ntokens <= e->last_tokens, "b2_get_hidden: ntokens %d out of range", ntokens);
  B2_CUDA_OK(cudaSetDevice(e->device));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  const int slot = layer + 1;  // -1 -> embeddings, l -> residual after layer l, L -> final norm output
  B2_CUDA_OK(cudaMemcpy(out_bf16, e->dbg_hidden + (size_t)slot * e->dbg_cap_tokens * e->cfg.hidden,
                        (size_t)ntokens * e->cfg.hidden * 2, cudaMemcpyDeviceToHost));
  return 0;
}

extern "C" int b2_get_hidden_f32(b2_engine* e, int32_t layer, int32_t ntokens, float* out_f32) {
  B2_REQUIRE(e && out_f32, "b2_get_hidden_f32: null argument");
  B2_REQUIRE((e->debug_flags & 1) && e->dbg_hidden_f32, "b2_get_hidden_f32: hidden capture not enabled, or the family's residual stream is bf16");
  B2_REQUIRE(layer >= -1 && layer + 1 < e->dbg_slots, "b2_get_hidden_f32: layer %d out of range (a looped layer counts once per pass)", layer);
  B2_REQUIRE(ntokens >= 1 && ntokens <= e->dbg_cap_tokens && ntokens <= e->last_tokens, "b2_get_hidden_f32: ntokens %d out of range", ntokens);
  B2_CUDA_OK(cudaSetDevice(e->device));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  B2_CUDA_OK(cudaMemcpy(out_f32, e->dbg_hidden_f32 + (size_t)(layer + 1) * e->dbg_cap_tokens * e->cfg.hidden, (size_t)ntokens * e->cfg.hidden * 4,
                        cudaMemcpyDeviceToHost));
  return 0;
}

extern "C" int b2_get_logits(b2_engine* e, int32_t nseq, float* out_logits) {
  B2_REQUIRE(e && out_logits, "b2_get_logits: null argument");
  B2_REQUIRE(list_arch(e->cfg.arch) || ((e->debug_flags & 2) && e->logits), "b2_get_logits: logits capture not enabled (b2_set_debug(e, 2))");
  B2_REQUIRE(nseq >= 1 && nseq <= e->last_n, "b2_get_logits: nseq %d > sequences of the last forward (%d)", nseq, e->last_n);
  B2_CUDA_OK(cudaSetDevice(e->device));
  const size_t n = (size_t)nseq * e->cfg.vocab;
  if (list_arch(e->cfg.arch)) {  // these families' lm_head writes fp32 rows; the leading rows are the sequences' last positions
    B2_CUDA_OK(cudaMemcpyAsync(out_logits, e->l_logits, n * 4, cudaMemcpyDeviceToHost, e->stream));
    B2_CUDA_OK(cudaStreamSynchronize(e->stream));
    return 0;
  }
  float* tmp = nullptr;
  B2_TRY(dalloc(&tmp, n));
  int rc = launch_logits_to_f32(e->logits, tmp, n, e->stream);
  if (rc == 0) {
    cudaError_t ce = cudaMemcpyAsync(out_logits, tmp, n * 4, cudaMemcpyDeviceToHost, e->stream);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
    if (ce != cudaSuccess) {
      b2_set_error("b2_get_logits: copy failed: %s", cudaGetErrorString(ce));
      rc = -5;
    }
  }
  cudaFree(tmp);
  return rc;
}

extern "C" int b2_set_next_tokens(b2_engine* e, int32_t nseq, const int32_t* seq_ids, const int32_t* tokens) {
  B2_REQUIRE(e && seq_ids && tokens, "b2_set_next_tokens: null argument");
  B2_REQUIRE((int)e->cur_batch.size() == nseq && std::equal(seq_ids, seq_ids + nseq, e->cur_batch.begin()),
             "b2_set_next_tokens: sequences must be the resident decode batch, in order");
  B2_CUDA_OK(cudaSetDevice(e->device));
  memcpy(e->h_stage, tokens, nseq * 4);
  B2_CUDA_OK(cudaMemcpyAsync(e->d_tokens, e->h_stage, nseq * 4, cudaMemcpyHostToDevice, e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  return 0;
}

extern "C" int b2_sample(b2_engine* e, int32_t nseq, const b2_sampling* params, int32_t* out_tokens) {
  B2_REQUIRE(e && params && out_tokens, "b2_sample: null argument");
  B2_REQUIRE((e->debug_flags & 2) && e->logits, "b2_sample: logits capture not enabled (b2_set_debug(e, 2))");
  B2_REQUIRE(nseq >= 1 && nseq <= e->last_n, "b2_sample: nseq %d > sequences of the last forward (%d)", nseq, e->last_n);
  B2_CUDA_OK(cudaSetDevice(e->device));
  e->h_sample_rows.resize(nseq);
  for (int i = 0; i < nseq; ++i) {
    // one seed for the whole batch: row i draws from its own stream derived from (seed, i)
    unsigned long long sd = params->seed == 0 ? 0ull : (params->seed * 0x9E3779B97F4A7C15ull + (unsigned long long)i);
    if (params->seed != 0 && sd == 0) sd = 1;
    e->h_sample_rows[i] = SampleRow{i, params->temperature, params->top_k, params->top_p, sd};
  }
  B2_TRY(launch_sample_rows(e->logits, e->h_sample_rows.data(), e->d_sample_rows, e->d_out_tokens, nseq, e->v_pad > 0 ? e->v_pad : e->cfg.vocab, (uint64_t)e->launches,
                            e->stream));
  e->launches++;
  B2_CUDA_OK(cudaMemcpyAsync(e->h_out, e->d_out_tokens, nseq * 4, cudaMemcpyDeviceToHost, e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  memcpy(out_tokens, e->h_out, nseq * 4);
  return 0;
}

extern "C" int b2_sample_rows(b2_engine* e, int32_t nrows, const int32_t* rows, const b2_sampling* params, int32_t* out_tokens) {
  B2_REQUIRE(e && rows && params && out_tokens && nrows >= 1, "b2_sample_rows: bad arguments");
  B2_REQUIRE((e->debug_flags & 2) && e->logits, "b2_sample_rows: logits capture not enabled (b2_set_debug(e, 2))");
  B2_REQUIRE(nrows <= e->cfg.max_seqs, "b2_sample_rows: too many rows");
  B2_CUDA_OK(cudaSetDevice(e->device));
  e->h_sample_rows.resize(nrows);
  for (int i = 0; i < nrows; ++i) {
    B2_REQUIRE(rows[i] >= 0 && rows[i] < e->last_n, "b2_sample_rows: row %d outside the last forward (%d rows)", rows[i], e->last_n);
    e->h_sample_rows[i] = SampleRow{rows[i], params[i].temperature, params[i].top_k, params[i].top_p, params[i].seed};
  }
  // one launch for all rows (the host vector outlives the copy: the call synchronises below)
  B2_TRY(launch_sample_rows(e->logits, e->h_sample_rows.data(), e->d_sample_rows, e->d_sample_out, nrows, e->v_pad > 0 ? e->v_pad : e->cfg.vocab, (uint64_t)e->launches,
                            e->stream));
  e->launches++;
  B2_CUDA_OK(cudaMemcpyAsync(e->h_out, e->d_sample_out, nrows * 4, cudaMemcpyDeviceToHost, e->stream));
  B2_CUDA_OK(cudaStreamSynchronize(e->stream));
  memcpy(out_tokens, e->h_out, nrows * 4);
  return 0;
}
