/*
 * b2_engine.h -- C ABI of the B200-native model-server engine (libb2engine.so).
 *
 * The reference (redhat-et/aws-k8s-ansible-provisioner) has no FFI or plugin interface for
 * its hot path: the path is the forward pass of the model-server container that
 * llm-d-deploy.yaml:176-184 launches for the model named at llm-d-deploy.yaml:118, reached
 * over HTTP by llm-d-test.yaml:32-43,61-73.  The arithmetic contract is HF transformers'
 * Qwen3 forward (models/qwen3/modeling_qwen3.py, cited per entry point below as "HF:").
 * This header is the in-process boundary the C++ server (b2serve) and the Python host mirror
 * (aws-k8s-ansible-provisioner_b200/engine.py) both bind; INTEGRATION.md shows the ctypes stub.
 *
 * Conventions: plain pointers and sizes only.  Every function returns 0 on success or a
 * negative errno-style code; b2_last_error() returns the message for the calling thread.
 * "host" pointers are caller-owned CPU memory; "dev" pointers are CUDA device memory.
 * One engine per device; an engine is NOT thread-safe (the server serialises onto one GPU
 * thread).  There is no CPU fallback anywhere behind this ABI.
 */
#ifndef B2_ENGINE_H
#define B2_ENGINE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_ABI_VERSION 6

typedef struct b2_engine b2_engine;

/* One entry of a model whose layers are listed one by one (b2_config.layer_specs): which mixer the layer has, the
 * mixer's sizes and constants, and its feed-forward.  Families whose layers are all alike (Qwen3, Phi-3, OPT) leave
 * the list NULL and describe the layer through the scalar fields of b2_config. */
enum b2_mixer_kind {
  B2_MIXER_LATENT_ATTENTION = 1, /* one shared low-rank latent per token (Lerasun) */
  B2_MIXER_ATTENTION = 2,        /* per-head keys and values, grouped queries, rotary positions on interleaved pairs (Kedasun "attention") */
  B2_MIXER_CONV_ATTENTION = 3    /* biased projections, a short causal convolution on q / k / v, unit-RMS q and k, a linear distance penalty,
                                    a window that keeps the first tokens, mixing of the heads' softmax weights, an output gate (Kedasun
                                    "attention_2") */
  ,
  B2_MIXER_WINDOW_AND_STATE = 4, /* two mixers side by side on the same input, each output RMS-normed over the model width, half their sum
                                    (Bumalix "parallel"): grouped-query softmax attention with biased projections, whole-row RMS norms of q
                                    and k, no positions, a sliding window; and gated linear attention, a matrix state per head with a decay
                                    per key channel (s_heads, s_dim, s_vdim, s_tau) */
  B2_MIXER_DELTA_STATE = 5,      /* gated delta rule: a matrix state per head, short causal convolutions on q / k / v, unit-vector q and k,
                                    a decay per head and key channel, a step size per head, a low-rank output gate (Bumalix "channel_delta") */
  B2_MIXER_DECAY_STATE = 6,      /* gated linear attention alone: a matrix state per head with a decay per key channel sigmoid(.)^(1 / s_tau)
                                    (heads, dim, vdim, s_tau), per-head RMS norm of the read-out, a silu gate (Tinevik "gla") */
  B2_MIXER_MIXED_SCORE_ATTENTION = 7, /* grouped-query softmax attention whose scores pass a cap and a heads x heads mixing BEFORE the softmax;
                                    q and k heads RMS-normed with one gain per entry of a head; rotary positions on half-split pairs
                                    (i, i + rot_dims/2) with the angles divided by rot_factor; values rotated by their own position over
                                    all of vdim and the weighted sum turned back by the query's (Tinevik "attention") */
  B2_MIXER_GATED_LATENT = 8      /* attention over a per-token latent with no rotated piece: the query itself goes through a normed latent of
                                    q_rank entries, a sliding window, a sigmoid gate on the concatenated heads (Tinevik "latent_attention") */
};
enum b2_ff_kind {
  B2_FF_NONE = 0,
  B2_FF_ROUTED_EXPERTS = 1,
  B2_FF_CLAMPED_GATED = 2,       /* y = g sigmoid(1.702 g) (u + 1), g = min(W_g x, limit), u = clamp(W_u x, -limit, limit); out = W_d y */
  B2_FF_POLYNORM = 3,            /* W_d p(W_u x), p(z) = a N(z) + b N(z^2) + c N(z^3) + e, N = division by the root mean square over the ff values */
  B2_FF_SCALED_GATED_EXPERTS = 4,/* sigmoid router, the `top` largest scores; expert = W_d (silu(W_g y) * (W_u y)) on y = score * x (scores not
                                    renormalised); a shared expert of the same form (shared_ff) on x itself is added */
  B2_FF_XIELU = 5,               /* W_d a(W_u x), a(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise */
  B2_FF_TABLE_EXPERTS = 6        /* experts of the B2_FF_CLAMPED_GATED form; an integer table row per token id names the token's `top` experts,
                                    each weighted 1 / top (no router) */
};
typedef struct b2_layer_spec {
  int32_t mixer;        /* b2_mixer_kind */
  int32_t heads;        /* query heads */
  int32_t dim;          /* per head: query/key dims that are NOT rotated */
  int32_t rot_dim;      /* per head: rotated query dims; the rotated key piece (one per token, shared by the heads) is as wide */
  int32_t vdim;         /* per head: value dims */
  int32_t kv_rank;      /* width of the per-token latent the keys and values are rebuilt from */
  int32_t kv_from;      /* -1: the layer projects and stores its own latent; j >= 0: it reads what layer j stored */
  int32_t rot_dims;     /* rotary positions turn the first rot_dims entries of the rotated piece, pairs (2i, 2i+1) */
  float   rot_base;     /* angle of pair i at position p: p * rot_base^(-2i/rot_dims) */
  float   scale;        /* softmax scale of the scores */
  int32_t ff;           /* b2_ff_kind */
  int32_t ff_dim;       /* inner width of one expert */
  int32_t experts;      /* experts per layer */
  int32_t top;          /* experts used per token */
  int32_t groups;       /* experts form `groups` equal groups of neighbours ... */
  int32_t groups_keep;  /* ... of which the best groups_keep may supply experts */
  /* ABI 4: mixers with per-head keys and values (B2_MIXER_ATTENTION, B2_MIXER_CONV_ATTENTION; `dim` is then the whole per-head
   * query / key width, rot_dim and kv_rank are unused) and the dense feed-forward */
  int32_t kv_heads;     /* key/value heads; query head a reads key/value head a / (heads / kv_heads) */
  int32_t conv_taps;    /* taps of the causal convolution over time on every q / k / v channel (0 = none) */
  int32_t window;       /* > 0: query i sees key j only when i - j < window or j < keep_first (0 = every earlier key) */
  int32_t keep_first;   /* the first keep_first tokens stay visible whatever the window */
  int32_t v_mix;        /* 1: the layer takes part in value mixing (the first such layer supplies, the others blend) */
  float   ff_limit;     /* B2_FF_CLAMPED_GATED: the clamp */
  /* ABI 5: mixers with a matrix state.  B2_MIXER_WINDOW_AND_STATE: heads / kv_heads / dim / vdim / scale / window describe the softmax half,
   * s_* the state half.  B2_MIXER_DELTA_STATE: heads (value heads) / kv_heads (query/key heads) / dim / vdim / conv_taps. */
  int32_t s_heads;      /* state heads of the second mixer */
  int32_t s_dim;        /* its query/key width per head */
  int32_t s_vdim;       /* its value width per head */
  float   s_tau;        /* its decay is sigmoid(.)^(1 / s_tau) */
  int32_t shared_ff;    /* B2_FF_SCALED_GATED_EXPERTS: inner width of the shared expert (0 = none) */
  /* ABI 6 */
  int32_t weights_of;   /* -1: the layer has tensors of its own; j >= 0: it runs with layer j's tensors and a cache / state of its own */
  int32_t q_rank;       /* B2_MIXER_GATED_LATENT: width of the normed latent the queries are rebuilt from */
  float   rot_factor;   /* rotary angles of q and k are divided by this (0 = 1) */
  float   softcap;      /* scores <- softcap * tanh(scores / softcap) before the softmax (0 = none) */
  int32_t score_mix;    /* 1: the heads' capped scores are mixed by a heads x heads matrix before the softmax */
  int32_t rot_values;   /* 1: values are rotated by their position over all of vdim and the output turned back */
} b2_layer_spec;

/* Architecture + runtime sizing.  Field meanings follow HF Qwen3Config
 * (HF:models/qwen3/configuration_qwen3.py) and `vllm serve` flags the llm-d chart passes
 * (--max-model-len, --block-size, --max-num-seqs, --gpu-memory-utilization). */
typedef struct b2_config {
  int32_t abi_version;       /* must be B2_ABI_VERSION */
  int32_t num_layers;        /* 28 */
  int32_t hidden;            /* 1024 */
  int32_t num_q_heads;       /* 16 */
  int32_t num_kv_heads;      /* 8 */
  int32_t head_dim;          /* 128; narrower heads (Phi-3: 96) run zero-padded to 128 */
  int32_t intermediate;      /* 3072 */
  int32_t vocab;             /* 151936 */
  int32_t tie_embeddings;    /* 1: lm_head shares embed_tokens (HF:...modeling_qwen3.py:443) */
  float   rms_eps;           /* 1e-6 */
  float   rope_theta;        /* 1e6 */
  int32_t max_model_len;     /* longest prompt+output per sequence */
  int32_t block_size;        /* KV page size in tokens; 16 */
  int32_t num_blocks;        /* KV pool size in pages; 0 = derive from gpu_mem_fraction */
  float   gpu_mem_fraction;  /* used when num_blocks == 0 */
  int32_t max_seqs;          /* max concurrently resident sequences (decode batch ceiling) */
  int32_t max_batch_tokens;  /* max tokens in one prefill forward */
  int32_t use_cuda_graphs;   /* 1: decode steps replay a captured graph per batch bucket */
  const float* rope_inv_freq;/* optional host [rotary_dim/2] fp32 table (HF:...:129-131); NULL =
                                computed as theta^(-2i/d) in double, rounded to fp32 */
  int32_t arch;              /* B2_ARCH_*: which HF model family the tensors and the layer follow */
  int32_t rotary_dim;        /* width of the rotated prefix of each head; 0 = head_dim */
  int32_t max_positions;     /* OPT: rows of the learned position table minus 2; 0 = max_model_len */
  int32_t sliding_window;    /* Phi-3: every query attends to its last `sliding_window` keys only; 0 = all */
  /* ABI 3 */
  const b2_layer_spec* layer_specs; /* [num_layers] for families with a layer list (Lerasun), else NULL; copied by b2_engine_create */
  int32_t compute_f32;       /* 1: activations, weights and cache in fp32, every product in true fp32 (families that have such a
                                path: Lerasun); 0: bf16 operands with fp32 accumulation */
  float   logit_scale;       /* the lm_head's output is multiplied by this (0 = 1) */
  /* ABI 4 */
  float   embed_scale;       /* the embedding row is multiplied by this (0 = 1; Kedasun) */
  int32_t norm_groups;       /* Kedasun: every norm splits its vector into this many equal pieces with a statistic each (0 = 1) */
  /* ABI 5 */
  int32_t loop_start;        /* layers [loop_start, loop_stop) run loop_times times in a row with the same weights, each pass with a cache and */
  int32_t loop_stop;         /* state of its own; in front of every pass the stream becomes W_in [x; x0], x0 the embedding output */
  int32_t loop_times;        /* 0 = no loop (and no W_in) */
  float   logit_softcap;     /* logits <- cap * tanh(logits / cap) (0 = none) */
  /* ABI 6 */
  int32_t norm_kind;         /* layer-list families: 0 = RMS norms as the family defines them; 1 = layer norms with gain and bias
                                ((x - mean) / sqrt(variance + eps) * w + b), in front of and behind every sublayer and at the end */
} b2_config;

/* Model families.  QWEN3: HF:models/qwen3/modeling_qwen3.py (QK-norm, separate q/k/v and gate/up
 * tensors, GQA).  PHI3: HF:models/phi3/modeling_phi3.py:49-64,208-272 (fused qkv_proj and
 * gate_up_proj tensors, no QK-norm, one query head per kv head or two, rotary over rotary_dim,
 * usually an untied lm_head, sliding-window attention when config.sliding_window is set).
 * OPT: HF:models/opt/modeling_opt.py:45-70,97-181,184-254,273-397 (learned positions with the +2
 * offset, LayerNorm with bias before attention and before the feed-forward, biased q/k/v/out and
 * fc1/fc2 projections, query pre-scaled by head_dim^-0.5, ReLU, tied lm_head; rms_eps carries the
 * LayerNorm eps; the do_layer_norm_before=False (350m) and word_embed_proj_dim != hidden variants are
 * not built). */
/* LERASUN: a layer list (b2_config.layer_specs).  Every layer adds a mixer branch and a feed-forward branch, both computed
 * from the same residual stream through two unit-offset RMS norms, back onto an fp32 residual stream; mixers are
 * latent attention (one shared low-rank latent + one rotated key piece per token, a per-head softmax sink, optional reuse of
 * an earlier layer's cache), feed-forwards are routed squared-ReLU experts.  Tensor names: embed, embed.norm,
 * l<i>.norm1|norm2, l<i>.mix.{q,dkv,dkv.norm,uk,uv,sink,o}, l<i>.mlp.{e<k>.up,e<k>.down,router,correction}, final.norm, head.
 * hidden = width; num_q_heads, head_dim, intermediate are unused. */
/* KEDASUN: a layer list as well.  h <- h + n1b(mixer(n1(h))), then h <- h + n2b(ff(n2(h))) on an fp32 residual stream; every norm
 * is an RMS norm over norm_groups pieces with a plain gain; the embedding is scaled by embed_scale.  Mixers: B2_MIXER_ATTENTION and
 * B2_MIXER_CONV_ATTENTION; feed-forward: B2_FF_CLAMPED_GATED or none.  Tensor names: embed, l<i>.norm1|norm1b|norm2|norm2b,
 * l<i>.mix.{q,k,v,o,vmix} (+ .b biases, {q,k,v}.conv, talk, g for the convolution mixer), l<i>.mlp.{gate,up,down}, final.norm, head. */
/* BUMALIX: a layer list as well.  n = norm1(h); h <- h + (mixer(n) + ff(n)) on an fp32 residual stream, ONE plain-gain RMS norm per layer;
 * the embedding is scaled by embed_scale; an optional loop over a run of layers (loop_*); logits capped by logit_softcap.  Mixers:
 * B2_MIXER_WINDOW_AND_STATE and B2_MIXER_DELTA_STATE; feed-forwards: B2_FF_POLYNORM, B2_FF_SCALED_GATED_EXPERTS or none.  Tensor names: embed,
 * loop.in, l<i>.norm1, l<i>.mix.left.{q,k,v (+ .b), q.norm, k.norm, o, out}, l<i>.mix.right.{q,k,v,g,o,norm,a1,a2,a2.b,out},
 * l<i>.mix.{q,k,v (+ .conv), b, A_log, a1, a2, dt_bias, g1, g2, norm, o}, l<i>.mlp.{up,down,act} or l<i>.mlp.{router, e<k>.{gate,up,down},
 * shared.{gate,up,down}}, final.norm, head.  The low-rank widths (a1, g1) are taken from the tensors. */
/* TINEVIK: a layer list as well.  h <- h + n1b(mixer(n1(h))), then h <- h + n2b(ff(n2(h))) on an fp32 residual stream, every norm a layer norm
 * with gain and bias (norm_kind 1); the embedding is scaled by embed_scale and is the head as well (tie_embeddings), logits times logit_scale.  A
 * layer may run with another layer's tensors (weights_of).  Mixers: B2_MIXER_DECAY_STATE, B2_MIXER_MIXED_SCORE_ATTENTION, B2_MIXER_GATED_LATENT;
 * feed-forwards: B2_FF_XIELU, B2_FF_TABLE_EXPERTS or none.  Tensor names: embed, l<i>.norm1|norm1b|norm2|norm2b (+ .b), l<i>.mix.{q,k,v,g,o,norm,a1,a2,
 * a2.b} (gla), l<i>.mix.{q,k,v,o,q.norm,k.norm,talk} (attention), l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o} (latent_attention),
 * l<i>.mlp.{up,down,act} or l<i>.mlp.{table (int32), e<k>.{gate,up,down}}, final.norm (+ .b).  The low-rank width (a1) is taken from the tensors. */
enum b2_arch { B2_ARCH_QWEN3 = 0, B2_ARCH_PHI3 = 1, B2_ARCH_OPT = 2, B2_ARCH_LERASUN = 3, B2_ARCH_KEDASUN = 4, B2_ARCH_BUMALIX = 5, B2_ARCH_TINEVIK = 6 };

/* Model registry: reads MODEL_DIR/config.json and fills the architecture fields of *cfg (the runtime sizing fields --
 * max_model_len, block_size, num_blocks, max_seqs, max_batch_tokens, use_cuda_graphs, compute_f32 -- are left as the caller
 * set them).  HF configs are told apart by "model_type" (qwen3, phi3, opt); a config with "architecture": "Lerasun", "Kedasun", "Bumalix" or "Tinevik" fills
 * specs[0 .. num_layers) as well and points cfg->layer_specs at it (max_specs = capacity of specs; may be 0 / NULL for the
 * HF families).  Returns 0, or a negative code with b2_last_error(). */
int  b2_config_from_dir(const char* model_dir, b2_config* cfg, b2_layer_spec* specs, int32_t max_specs);

const char* b2_last_error(void);
int  b2_abi_version(void);

/* ---- engine lifetime ------------------------------------------------------------------- */
/* Creates the engine on CUDA device `device`.  If safetensors_path is non-NULL, every
 * HF-named tensor is read from that file (bf16) and the weights are finalised; otherwise
 * the caller uploads tensors with b2_engine_load_tensor and calls b2_engine_finalize.
 * Replaces: the model-server container start at llm-d-deploy.yaml:176-193. */
int  b2_engine_create(const b2_config* cfg, const char* safetensors_path, int device, b2_engine** out);
int  b2_engine_load_tensor(b2_engine* e, const char* hf_name, const void* host_bf16, size_t nbytes);
/* Integer tensors (int32), for the families whose checkpoints hold one (Tinevik: l<i>.mlp.table [vocab][top]). */
int  b2_engine_load_int_tensor(b2_engine* e, const char* name, const int32_t* host_i32, size_t count);
/* Reads every tensor of one safetensors file (BF16, F16 or F32, converted to bf16; I32 for integer tables) into an engine created without
 * a path: call it once per shard of a sharded checkpoint (model-0000i-of-0000N.safetensors), then finalize. */
int  b2_engine_load_safetensors(b2_engine* e, const char* path);
int  b2_engine_finalize(b2_engine* e);
void b2_engine_free(b2_engine* e);
/* Info: KV pages total / free, bytes of weights resident. */
int  b2_engine_info(b2_engine* e, int64_t* num_blocks, int64_t* free_blocks, int64_t* weight_bytes);

/* ---- sequences (paged KV allocator; HF:...modeling_qwen3.py:270-271 cache update) ------- */
/* Reserves pages for up to reserve_tokens tokens (prompt + output) and returns a slot id. */
int  b2_seq_create(b2_engine* e, int32_t reserve_tokens, int32_t* seq_id);
/* Grows the reservation of a live sequence to total_tokens (no-op when it already holds that many): a scheduler that does
 * not know a request's final length takes pages as the tokens arrive.  Fails with -12 when the pool has no pages left. */
int  b2_seq_reserve(b2_engine* e, int32_t seq_id, int32_t total_tokens);
int  b2_seq_free(b2_engine* e, int32_t seq_id);
int  b2_seq_len(b2_engine* e, int32_t seq_id);
/* Drops the tail of a sequence (new_len <= current length); its pages stay reserved.  Used to
 * re-run a measurement over the same context and by stop-string handling in the server. */
int  b2_seq_truncate(b2_engine* e, int32_t seq_id, int32_t new_len);

/* ---- forward passes --------------------------------------------------------------------- */
/* Prefill: appends ids[seq_offsets[i] .. seq_offsets[i+1]) to sequence seq_ids[i], runs the
 * forward over all appended tokens (HF:...modeling_qwen3.py:378-438), and returns the greedy
 * next token of every sequence (HF:...:504-505 lm_head on the last position + argmax, lowest
 * index on ties) in out_tokens (host, may be NULL).  The next token is NOT appended. */
int  b2_prefill(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq,
                const int32_t* seq_ids, int32_t* out_tokens);

/* One decode step: appends in_tokens[i] to sequence seq_ids[i] (in_tokens == NULL: append the
 * token the previous forward produced for that sequence, kept on the device), runs one
 * forward, returns the greedy next tokens in out_tokens (host, may be NULL = no D2H copy). */
int  b2_decode_step(b2_engine* e, int32_t nseq, const int32_t* seq_ids, const int32_t* in_tokens,
                    int32_t* out_tokens);

/* `steps` decode steps back to back, token feedback on the device, no host round trip
 * between steps.  elapsed_ms (may be NULL) receives the CUDA-event time of the region on
 * the engine stream.  out_tokens (host, [steps][nseq], may be NULL) is copied at the end. */
int  b2_decode_run(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t steps,
                   int32_t* out_tokens, float* elapsed_ms);

/* Like b2_prefill, for callers that want logits at chosen places instead of a next token per sequence: rows[0 .. nrows)
 * index the call's tokens in the order given (0 = first token of the first sequence), out_logits (host) receives
 * [nrows][vocab] fp32.  nrows may be 0.  A sequence may bring a single token (a decode step run beside other sequences'
 * prompt portions).  Greedy next tokens are still produced for every sequence's last position. */
int  b2_prefill_logits(b2_engine* e, const int32_t* ids, const int32_t* seq_offsets, int32_t nseq, const int32_t* seq_ids,
                       const int32_t* rows, int32_t nrows, float* out_logits, int32_t* out_tokens);

/* Logits of the last forward's last positions, [nseq][vocab] fp32 on the host. */
int  b2_get_logits(b2_engine* e, int32_t nseq, float* out_logits);
/* Residual stream after layer `layer` (0-based; -1 = embeddings, num_layers = final norm
 * output) for the tokens of the last forward, [ntokens][hidden] as bf16 bits on the host.
 * Only filled when debug capture was enabled with b2_set_debug(e, 1). */
int  b2_set_debug(b2_engine* e, int32_t capture_hidden);
int  b2_get_hidden(b2_engine* e, int32_t layer, int32_t ntokens, uint16_t* out_bf16);
/* The same for families whose residual stream is fp32 (the layer-list families): [ntokens][hidden] floats.  In a model with a looped run of
 * layers, `layer` counts layer RUNS (a looped layer once per pass, in the order they run); -1 is the embedding output. */
int  b2_get_hidden_f32(b2_engine* e, int32_t layer, int32_t ntokens, float* out_f32);

/* Measurement knobs that can change while the engine lives (bench.py's ablation leg, the two-lane tests); every
 * call drops the captured decode graphs, so the next step re-captures with the new setting.
 *   B2_TUNE_SKIP_MASK   bit k set = kernel class k (b2_kernel_class order) is left out of the step: timing only,
 *                       the outputs are then meaningless
 *   B2_TUNE_PREFIX_CACHE  1 = full pages of prompt tokens are kept under the hash of the token prefix they end, and
 *                       b2_prefill lets a fresh sequence whose prompt starts with the same tokens take those pages
 *                       instead of recomputing them (vLLM's --enable-prefix-caching; environment B2_PREFIX_CACHE).
 *                       Results are unchanged: the cached K/V are the bits the same prefill would write.  0 = off and
 *                       forget what was cached (the default)
 *   B2_TUNE_TWO_LANE    smallest padded decode batch that runs as two half-batch lanes (0 = never, the default;
 *                       environment B2_MB) */
enum b2_tuning_key { B2_TUNE_SKIP_MASK = 0, B2_TUNE_TWO_LANE = 1, B2_TUNE_PREFIX_CACHE = 2 };
int  b2_set_tuning(b2_engine* e, int32_t key, int64_t value);
/* Prefix cache counters since the engine was created: prompt tokens looked up, prompt tokens served from cached pages,
 * pages currently registered (any pointer may be NULL). */
int  b2_prefix_cache_stats(b2_engine* e, int64_t* queried_tokens, int64_t* hit_tokens, int64_t* cached_pages);

/* Sampling for the API surface (temperature / top-k / top-p over the last logits). */
typedef struct b2_sampling {
  float    temperature;  /* 0 = greedy */
  int32_t  top_k;        /* <=0 = off */
  float    top_p;        /* >=1 = off; taken over what top_k leaves (top-k first, then top-p, as vLLM) */
  uint64_t seed;         /* != 0: the draw depends on (seed, row parameters, logits) only -- a caller that wants a
                          * different draw per generated token advances the seed itself (b2serve adds the number of
                          * tokens generated so far); 0: no seed given, draws also mix in a launch counter */
} b2_sampling;
int  b2_sample(b2_engine* e, int32_t nseq, const b2_sampling* params, int32_t* out_tokens);
/* Per-row variant for a batch whose requests carry different sampling parameters: rows[i] indexes
 * the last forward's batch, params[i] applies to it (temperature 0 = greedy). */
int  b2_sample_rows(b2_engine* e, int32_t nrows, const int32_t* rows, const b2_sampling* params,
                    int32_t* out_tokens);
/* Overrides the device-resident "next token" of each listed sequence (after sampling on host
 * or with b2_sample) so the following b2_decode_step(in_tokens=NULL) consumes it. */
int  b2_set_next_tokens(b2_engine* e, int32_t nseq, const int32_t* seq_ids, const int32_t* tokens);

/* ---- measurement ------------------------------------------------------------------------ */
#define B2_NUM_KERNEL_CLASSES 12
/* Runs `steps` decode steps eagerly (no graph) with a CUDA event pair around every kernel
 * launch on the engine stream; ms_by_class / launches_by_class receive totals per class
 * (index = enum below).  Used by bench.py for the live roofline figure. */
enum b2_kernel_class {
  B2K_EMBED = 0, B2K_NORM = 1, B2K_GEMM_QKV = 2, B2K_ROPE_KV = 3, B2K_ATTN_DECODE = 4,
  B2K_CHAIN = 5, B2K_GEMM_O = 6, B2K_GEMM_GATEUP = 7, B2K_ACT = 8, B2K_GEMM_DOWN = 9,
  B2K_LMHEAD = 10, B2K_MISC = 11
};
int  b2_decode_profile(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t steps,
                       float* ms_by_class, int64_t* launches_by_class);
/* Times the dominant kernel on its own: the decode-attention pass of every layer, launched back to
 * back on the engine stream over the batch's real K/V pages (the batch of the last decode call),
 * `reps` times, between ONE pair of CUDA events.  ms_per_launch = elapsed / (reps * layers);
 * kv_bytes_per_launch = the K and V bytes one launch has to read (sum over sequences of
 * (len + 1) * kv_heads * head_dim * 2 tensors * 2 bytes).  Results of the pass are discarded.
 * bench.py's roofline figure comes from here: an event pair around every single launch (as
 * b2_decode_profile does) adds several microseconds of launch latency to a ~30 us kernel. */
int  b2_attn_profile(b2_engine* e, int32_t nseq, const int32_t* seq_ids, int32_t reps,
                     float* ms_per_launch, int64_t* kv_bytes_per_launch);
/* Number of kernel launches (graph nodes included) issued by this engine so far. */
int64_t b2_launch_count(b2_engine* e);

/* ---- kernel-level entry points (tests call each kernel on device buffers) --------------- */
/* All take a cudaStream_t as void*; NULL = default stream.  Shapes are row-major. */

/* HF:...modeling_qwen3.py:59-64 (+ residual add :327,333).  h [T][H] bf16 in/out; delta may be
 * NULL, bf16 [T][H] (delta_is_f32 = 0) or fp32 split partials [nsplit][T][H] (= 1) that are
 * summed in split order and rounded to bf16 before the add.  x = RMSNorm(h) * w. */
int b2k_add_rmsnorm(void* h_bf16, const void* delta, int delta_is_f32, int nsplit,
                    const void* w_bf16, void* x_bf16, int T, int H, float eps, void* stream);

/* HF:...:248-249,263-264 (QK-norm), :151-181 (RoPE), :270-271 (cache write).
 * qkv [T][(nq+2nkv)*hd] bf16 (or fp32 partials), positions/slots [T] int32,
 * cos_sin [max_pos][hd] bf16 = cos[hd/2] | sin[hd/2].  Writes q_out [T][nq*hd] and the K/V
 * pages (layout: see "KV page layout" below). */
int b2k_qknorm_rope_kv(const void* qkv, int qkv_is_f32, int nsplit, const void* qnorm_w,
                       const void* knorm_w, const void* cos_sin, const int32_t* positions,
                       const int32_t* slots, void* q_out, void* k_pages, void* v_pages, int T,
                       int nq, int nkv, int hd, int block_size, float eps, void* stream);

/* HF:...:81-83: act = silu(gate) * up, gu [T][2*I] (gate | up) bf16 or fp32 partials. */
int b2k_silu_mul(const void* gu, int gu_is_f32, int nsplit, void* act_bf16, int T, int I, void* stream);

/* y[T][N] = x[T][K] . W[N][K]^T, bf16 in, fp32 accumulate (HF nn.Linear, :236-247).
 * impl: 0 = SIMT GEMV path, 1 = tcgen05/TMEM path.  nsplit > 1: out is fp32 partials
 * [nsplit][T][N]; nsplit == 1 && out_is_f32 == 0: bf16 [T][N]. */
int b2k_linear(const void* x_bf16, const void* w_bf16, void* out, int out_is_f32, int nsplit,
               int T, int N, int K, int impl, void* stream);

/* The two fused projections of a decode step (csrc/gemm_pair.cu), T <= 64 tokens, K <= 1024 in steps of 128:
 *   b2k_gateup_swiglu: act[T][I] = bf16(bf16(silu(g)) * u) with g | u = bf16(x . Wgu^T), Wgu [2I][K] = gate rows then up
 *                      rows (HF:...:81-83); the [T][2I] intermediate is never written
 *   b2k_qkv_rope:      b2k_linear with Wqkv [(nq + 2 nkv) * 128][K] followed by b2k_qknorm_rope_kv, in one launch
 * Same rounding points as the separate kernels; the fp32 sum of a dot product is formed from two K halves. */
int b2k_gateup_swiglu(const void* x_bf16, const void* w_gu_bf16, void* act_bf16, int T, int I, int K, void* stream);
int b2k_qkv_rope(const void* x_bf16, const void* w_qkv_bf16, const void* qnorm_w, const void* knorm_w, const void* cos_sin,
                 const int32_t* positions, const int32_t* slots, void* q_out, void* k_pages, void* v_pages, int T, int nq,
                 int nkv, int K, int block_size, float eps, void* stream);

/* The decode step's norm-free layer chain: the two projections that feed the residual stream update it
 * themselves, and the two projections that read it normalise it as they load it, so that no RMSNorm kernel runs between
 * them (HF:models/qwen3/modeling_qwen3.py:339-351 for the adds, :50-62 for the norm).
 * b2k_linear_resid: h[T][N] (bf16, in place) = bf16(h + bf16(x[T][K] . W[N][K]^T)), T <= 64, N % 128 == 0, K % 512 == 0,
 *   K <= 3072; ssq[N/16][ssq_ld] (fp32) receives per token column the sum of squares of each 16-feature piece of the new h.
 * b2k_gateup_swiglu_norm / b2k_qkv_rope_norm: b2k_gateup_swiglu / b2k_qkv_rope with x = bf16(norm_w * bf16(h * rstd)) formed
 *   on the fly, rstd = rsqrt(sum of the `pieces` pieces of ssq / K + eps). */
/* Prefill-sized y[T][N] (bf16) = x[T][K] . W[N][K]^T by pairs of CTAs that share the token tile through TMA multicast (both
 * operands in this GPU's memory); T >= 512, N % 256 == 0, K % 64 == 0.  Bit-identical to b2k_linear's bf16 output. */
int b2k_linear_multicast(const void* x_bf16, const void* w_bf16, void* out_bf16, int T, int N, int K, void* stream);
/* Prefill-sized residual add in the projection's epilogue: h[T][N] (bf16, in place) = bf16(h + bf16(x[T][K] . W[N][K]^T)), T > 16. */
int b2k_linear_add(const void* x_bf16, const void* w_bf16, void* h_bf16, int T, int N, int K, void* stream);
int b2k_linear_resid(const void* x_bf16, const void* w_bf16, void* h_bf16, float* ssq, int T, int N, int K, int ssq_ld, void* stream);
int b2k_gateup_swiglu_norm(const void* h_bf16, const void* w_gu_bf16, const void* norm_w, const float* ssq, int pieces, int ssq_ld,
                           float eps, void* act_bf16, int T, int I, int K, void* stream);
int b2k_qkv_rope_norm(const void* h_bf16, const void* w_qkv_bf16, const void* norm_w, const float* ssq, int pieces, int ssq_ld,
                      float norm_eps, const void* qnorm_w, const void* knorm_w, const void* cos_sin, const int32_t* positions,
                      const int32_t* slots, void* q_out, void* k_pages, void* v_pages, int T, int nq, int nkv, int K, int block_size,
                      float eps, void* stream);

/* Diagnostics (tools/step_timeline.py): register a device buffer of uint64 in which thread 0 of every CTA of every
 * kernel on the decode path appends one 4-word record {class | blockIdx << 8 | smid << 32 | aux << 40, CTA start,
 * dependency wait returned, CTA end} in %globaltimer ns.  The caller sets buf[0] = 0 (record counter) and
 * buf[1] = capacity in records; records start at buf[4].  NULL switches the trace off.  class 100 = a projection
 * (aux = N/64 | (K/64) << 12 | second lane << 23); for the other kernels aux = 1 on the second lane of a two-lane step. */
int b2k_debug_step_trace(void* dev_u64_buf);
/* Diagnostics: register a device buffer of (148 * 8) uint64 in which every CTA of the tcgen05
 * projection kernel stamps %globaltimer at its phase boundaries (NULL switches the trace off). */
int b2k_debug_gemm_trace(void* dev_u64_buf);
/* Same for the decode chain kernel: (148 * 32) uint64; slots 0..7 = entry into step i, 16..23 = the
 * CTA finished step i's work (before the grid barrier), 8 = CTA start, 9 = dependency satisfied,
 * 10 = CTA done. */
int b2k_debug_chain_trace(void* dev_u64_buf);
int b2k_debug_fused_trace(void* dev_u64_buf);  /* same, for the fused four-step chain: 128 CTAs x 32 slots */

/* lm_head + greedy argmax fused (HF:...:504-505 + generate(do_sample=False)).
 * logits_bf16 may be NULL.  out_tokens [T] int32 (device). scratch: [T] uint64 (device). */
int b2k_lmhead_argmax(const void* x_bf16, const void* w_bf16, void* logits_bf16,
                      int32_t* out_tokens, void* scratch_u64, int T, int V, int K, int impl,
                      void* stream);

/* KV page layout shared by every kernel below: one allocation per layer and per K/V,
 * [page][kv_head][block_size = 16 tokens][head_dim = 128] bf16, i.e. a 4 KB slice per (page, kv head),
 * in which the 16-byte chunk c (8 dims) of token row r sits at chunk position c ^ (r & 7).
 * b2k_qknorm_rope_kv writes that layout; the two attention entry points read it. */

/* HF:integrations/sdpa_attention.py:40-104 at T == 1: paged GQA decode attention.
 * q [B][nq*hd]; pages as above; block_table [B][bt_stride]; seq_lens [B] (including the current
 * token; 0 = empty row, output zeros).  scratch_f32: b2k_attn_decode_scratch_floats(...) floats of
 * device memory for the partial records of the page-balanced attention pass.  out [B][nq*hd] bf16. */
int b2k_attn_decode(const void* q, const void* k_pages, const void* v_pages,
                    const int32_t* block_table, int bt_stride, const int32_t* seq_lens,
                    void* scratch_f32, void* out, int B, int nq, int nkv, int hd, int block_size,
                    void* stream);
size_t b2k_attn_decode_scratch_floats(int B, int nq, int nkv, int hd);

/* No counterpart in the reference (it has no kernels at all).  Same computation and arguments as
 * b2k_attn_decode, minus scratch_f32: for callers that cannot allocate device memory -- a server
 * whose KV pool already owns the free HBM, request-path code that cannot afford the device-wide
 * synchronisation of cudaMalloc/cudaFree, a plugin that is only handed input/output pointers.  The
 * partial records go to an array compiled into the library (B2K_ATTN_NOALLOC_MAX_FLOATS floats =
 * 8 MiB, resident on every GPU that loads the library until the process exits).  The call allocates
 * and frees nothing.  It fails with a message if b2k_attn_decode_scratch_floats(B, nq, nkv, hd)
 * exceeds that size: 5120 + (B * nkv + 2560) * 260 floats must fit, i.e. B * nkv <= 5486 (sequence, kv
 * head) units; the kernel itself handles at most 4096 units per launch, so that is the limit reached
 * first, and it is reported the same way.
 * The first call on each device looks up the array's device address (that device must be current)
 * and caches it; make that first call before starting any stream capture.
 * All calls share the one array and it keeps whatever the last call wrote.  The only words that must
 * start at zero are 16 KB of arrival counters, and every call clears them itself (a memset on the
 * caller's stream ahead of the kernel); everything else is written before it is read.  Two calls
 * whose kernels overlap on the GPU (different streams, or different host threads) race on the array
 * -- serialise them. */
#define B2K_ATTN_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)
int b2k_attn_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                            const int32_t* block_table, int bt_stride, const int32_t* seq_lens,
                            void* out, int B, int nq, int nkv, int hd, int block_size, void* stream);

/* Same contract at T > 1 (causal): ragged prefill over the paged cache.  q [T][nq*hd];
 * q_seq[T] / q_pos[T] int32 give the sequence row in block_table and the position of each
 * query token (tokens of one sequence contiguous and ascending).  Host arrays.
 * A test hook, not a serving call: it cudaMallocs a tile list, synchronises `stream` before it returns and frees
 * the list again (the engine's own prefill keeps its tile list in engine-owned buffers and does none of that). */
int b2k_attn_prefill(const void* q, const void* k_pages, const void* v_pages,
                     const int32_t* block_table_dev, int bt_stride, const int32_t* host_seq_first_tok,
                     const int32_t* host_seq_pos0, const int32_t* host_seq_ntok,
                     const int32_t* host_seq_row, int nseq, void* out, int nq, int nkv, int hd,
                     int block_size, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B2_ENGINE_H */
