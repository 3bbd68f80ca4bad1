"""Host-side mirror of the engine's C ABI (include/b2_engine.h) for tests, bench.py and the
Python tooling.  Every method is one C call; there is no arithmetic here and no fallback.

The names follow the serving domain of the reference deployment (sequences, pages, prefill,
decode step; llm-d-deploy.yaml:118, llm-d-test.yaml:61-73), not a training framework's.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import capi
from .capi import B2Error, b2_config, b2_layer_spec, b2_sampling, check, load_library

KERNEL_CLASSES = ["embed", "norm", "gemm_qkv", "rope_kv", "attn_decode", "chain", "gemm_o", "gemm_gateup", "act",
                  "gemm_down", "lmhead", "misc"]


@dataclass
class EngineConfig:
    num_layers: int = 28
    hidden: int = 1024
    num_q_heads: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 3072
    vocab: int = 151936
    tie_embeddings: bool = True
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    max_model_len: int = 4096
    block_size: int = 16
    num_blocks: int = 0
    gpu_mem_fraction: float = 0.9
    max_seqs: int = 64
    max_batch_tokens: int = 8192
    use_cuda_graphs: bool = True
    arch: str = "qwen3"          # "qwen3" | "phi3" | "opt" | "lerasun" | "kedasun" | "bumalix" | "tinevik" (include/b2_engine.h, enum b2_arch)
    rotary_dim: int = 0          # 0 = head_dim
    max_positions: int = 0       # OPT: learned position table rows - 2 (0 = max_model_len)
    sliding_window: int = 0      # Phi-3: attend to the last N keys only (0 = all)
    layers: list | None = None   # layer-list families (arch "lerasun", "kedasun", "bumalix"): the "layers" entries of the model's config.json
    compute_f32: bool = False    # families with an fp32 path: operands, weights and cache in fp32
    logit_scale: float = 0.0     # lm_head output multiplier (0 = 1)
    embed_scale: float = 0.0     # embedding multiplier (0 = 1)
    norm_groups: int = 0         # Kedasun: pieces of every norm (0 = 1)
    loop: tuple = (0, 0, 0)      # Bumalix: layers [start, stop) run `times` times in a row (times 0 = no loop)
    logit_softcap: float = 0.0   # logits <- cap * tanh(logits / cap) (0 = none)
    norm_kind: int = 0           # 1: layer norms with gain and bias around every sublayer (Tinevik)

    @staticmethod
    def lerasun(model_cfg: dict, **runtime) -> "EngineConfig":
        """From the dict a Lerasun config.json holds (width, vocab, norm.eps, logit_scale, layers) plus runtime sizing."""
        return EngineConfig(num_layers=len(model_cfg["layers"]), hidden=model_cfg["width"], vocab=model_cfg["vocab"],
                            rms_eps=model_cfg["norm"]["eps"], logit_scale=model_cfg.get("logit_scale", 1.0), arch="lerasun",
                            layers=model_cfg["layers"], tie_embeddings=False, num_q_heads=0, num_kv_heads=0, head_dim=0,
                            intermediate=0, **runtime)

    @staticmethod
    def kedasun(model_cfg: dict, **runtime) -> "EngineConfig":
        """From the dict a Kedasun config.json holds (width, vocab, embedding.scale, norm.eps, norm.groups, layers) plus runtime sizing."""
        return EngineConfig(num_layers=len(model_cfg["layers"]), hidden=model_cfg["width"], vocab=model_cfg["vocab"],
                            rms_eps=model_cfg["norm"]["eps"], norm_groups=model_cfg["norm"].get("groups", 1),
                            embed_scale=model_cfg.get("embedding", {}).get("scale", 1.0), logit_scale=1.0, arch="kedasun",
                            layers=model_cfg["layers"], tie_embeddings=False, num_q_heads=0, num_kv_heads=0, head_dim=0,
                            intermediate=0, **runtime)

    @staticmethod
    def bumalix(model_cfg: dict, **runtime) -> "EngineConfig":
        """From the dict a Bumalix config.json holds (width, vocab, embedding.scale, norm.eps, loop, logit_softcap, layers) plus runtime sizing."""
        lp = model_cfg.get("loop") or {}
        return EngineConfig(num_layers=len(model_cfg["layers"]), hidden=model_cfg["width"], vocab=model_cfg["vocab"],
                            rms_eps=model_cfg["norm"]["eps"], embed_scale=model_cfg.get("embedding", {}).get("scale", 1.0), logit_scale=1.0,
                            arch="bumalix", layers=model_cfg["layers"], tie_embeddings=False, num_q_heads=0, num_kv_heads=0, head_dim=0,
                            intermediate=0, loop=(int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 0))),
                            logit_softcap=float(model_cfg.get("logit_softcap") or 0.0), **runtime)

    @staticmethod
    def tinevik(model_cfg: dict, **runtime) -> "EngineConfig":
        """From the dict a Tinevik config.json holds (width, vocab, embedding.scale, logit_scale, norm.eps, layers) plus runtime sizing."""
        return EngineConfig(num_layers=len(model_cfg["layers"]), hidden=model_cfg["width"], vocab=model_cfg["vocab"],
                            rms_eps=model_cfg["norm"]["eps"], embed_scale=(model_cfg.get("embedding") or {}).get("scale", 1.0),
                            logit_scale=model_cfg.get("logit_scale", 1.0), arch="tinevik", layers=model_cfg["layers"], tie_embeddings=True,
                            num_q_heads=0, num_kv_heads=0, head_dim=0, intermediate=0, norm_kind=1, **runtime)

    def kv_bytes_per_token(self) -> int:
        return 2 * self.num_layers * self.num_kv_heads * self.head_dim * 2

    def weight_bytes(self) -> int:
        q, kv = self.num_q_heads * self.head_dim, self.num_kv_heads * self.head_dim
        per_layer = (q + 2 * kv) * self.hidden + self.hidden * q + 3 * self.intermediate * self.hidden + 2 * self.hidden + 2 * self.head_dim
        total = self.num_layers * per_layer + self.vocab * self.hidden * (1 if self.tie_embeddings else 2) + self.hidden
        return 2 * total


QWEN3_0_6B = EngineConfig()


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


def _p32(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_int32))


class Engine:
    """One engine per GPU (request-level data parallelism: one replica per device, no collective)."""

    def __init__(self, cfg: EngineConfig, device: int = 0, safetensors_path: str | None = None, rope_inv_freq=None):
        self.lib = load_library()
        self.cfg = cfg
        c = b2_config()
        c.abi_version = capi.ABI_VERSION
        for f in ("num_layers", "hidden", "num_q_heads", "num_kv_heads", "head_dim", "intermediate", "vocab", "max_model_len",
                  "block_size", "num_blocks", "max_seqs", "max_batch_tokens"):
            setattr(c, f, int(getattr(cfg, f)))
        c.tie_embeddings = int(cfg.tie_embeddings)
        c.use_cuda_graphs = int(cfg.use_cuda_graphs)
        c.rms_eps = cfg.rms_eps
        c.rope_theta = cfg.rope_theta
        c.gpu_mem_fraction = cfg.gpu_mem_fraction
        c.arch = {"qwen3": capi.ARCH_QWEN3, "phi3": capi.ARCH_PHI3, "opt": capi.ARCH_OPT, "lerasun": capi.ARCH_LERASUN,
                  "kedasun": capi.ARCH_KEDASUN, "bumalix": capi.ARCH_BUMALIX, "tinevik": capi.ARCH_TINEVIK}[cfg.arch]
        c.norm_kind = int(cfg.norm_kind)
        c.loop_start, c.loop_stop, c.loop_times = (int(v) for v in cfg.loop)
        c.logit_softcap = float(cfg.logit_softcap)
        c.compute_f32 = int(cfg.compute_f32)
        c.logit_scale = float(cfg.logit_scale)
        c.embed_scale = float(cfg.embed_scale)
        c.norm_groups = int(cfg.norm_groups)
        self._specs = None
        if cfg.layers is not None:
            self._specs = (b2_layer_spec * len(cfg.layers))()
            for sp, layer in zip(self._specs, cfg.layers):
                _fill_layer_spec(sp, dict(layer, _tinevik=True) if cfg.arch == "tinevik" else layer)
            c.layer_specs = self._specs
        c.rotary_dim = int(cfg.rotary_dim)
        c.max_positions = int(cfg.max_positions)
        c.sliding_window = int(cfg.sliding_window)
        self._inv = None
        if rope_inv_freq is not None:
            self._inv = np.ascontiguousarray(np.asarray(rope_inv_freq, dtype=np.float32))
            assert self._inv.shape == ((cfg.rotary_dim or cfg.head_dim) // 2,)
            c.rope_inv_freq = self._inv.ctypes.data_as(C.POINTER(C.c_float))
        h = C.c_void_p()
        path = safetensors_path.encode() if safetensors_path else None
        check(self.lib.b2_engine_create(C.byref(c), path, device, C.byref(h)), self.lib)
        self.h = h
        self.device = device

    @classmethod
    def from_model_dir(cls, model_dir: str, device: int = 0, dtype: str = "bfloat16", **runtime) -> "Engine":
        """The engine for the model a directory holds: the library's registry reads config.json and picks the family,
        model.safetensors supplies the weights.  runtime: max_model_len, num_blocks, max_seqs, max_batch_tokens, ..."""
        import os

        lib = load_library()
        c = b2_config()
        specs = (b2_layer_spec * 1024)()
        check(lib.b2_config_from_dir(model_dir.encode(), C.byref(c), specs, 1024), lib)
        arch = {capi.ARCH_QWEN3: "qwen3", capi.ARCH_PHI3: "phi3", capi.ARCH_OPT: "opt", capi.ARCH_LERASUN: "lerasun",
                capi.ARCH_KEDASUN: "kedasun", capi.ARCH_BUMALIX: "bumalix", capi.ARCH_TINEVIK: "tinevik"}[c.arch]
        layers = None
        if arch in ("lerasun", "kedasun", "bumalix", "tinevik"):
            layers = [_layer_dict(specs[i]) for i in range(c.num_layers)]
        cfg = EngineConfig(num_layers=c.num_layers, hidden=c.hidden, num_q_heads=c.num_q_heads, num_kv_heads=c.num_kv_heads,
                           head_dim=c.head_dim, intermediate=c.intermediate, vocab=c.vocab, tie_embeddings=bool(c.tie_embeddings),
                           rms_eps=c.rms_eps, rope_theta=c.rope_theta, arch=arch, rotary_dim=c.rotary_dim,
                           max_positions=c.max_positions, sliding_window=c.sliding_window, layers=layers,
                           compute_f32=(dtype == "float32"), logit_scale=c.logit_scale, embed_scale=c.embed_scale,
                           norm_groups=c.norm_groups, loop=(c.loop_start, c.loop_stop, c.loop_times), logit_softcap=c.logit_softcap,
                           norm_kind=c.norm_kind, **runtime)
        return cls(cfg, device=device, safetensors_path=os.path.join(model_dir, "model.safetensors"))

    # ---- weights -----------------------------------------------------------------------
    def load_safetensors(self, paths) -> None:
        """Loads one or more safetensors files (the shards of a checkpoint) and finalises the weights."""
        for p in ([paths] if isinstance(paths, str) else list(paths)):
            check(self.lib.b2_engine_load_safetensors(self.h, p.encode()), self.lib)
        check(self.lib.b2_engine_finalize(self.h), self.lib)

    def load_state_dict(self, sd) -> None:
        """Uploads an HF-named state dict of torch bf16 CPU tensors (no file round trip)."""
        import torch

        for name, t in sd.items():
            if "rotary_emb" in name:
                continue
            if t.dtype in (torch.int32, torch.int64):   # integer tables
                t = t.detach().to(torch.int32).contiguous().cpu()
                check(self.lib.b2_engine_load_int_tensor(self.h, name.encode(), C.cast(C.c_void_p(t.data_ptr()), C.POINTER(C.c_int32)), t.numel()),
                      self.lib)
                continue
            t = t.detach().to(torch.bfloat16).contiguous().cpu()
            check(self.lib.b2_engine_load_tensor(self.h, name.encode(), C.c_void_p(t.data_ptr()), t.numel() * 2), self.lib)
        check(self.lib.b2_engine_finalize(self.h), self.lib)

    # ---- sequences ----------------------------------------------------------------------
    def seq_create(self, reserve_tokens: int) -> int:
        sid = C.c_int32(-1)
        check(self.lib.b2_seq_create(self.h, int(reserve_tokens), C.byref(sid)), self.lib)
        return sid.value

    def seq_reserve(self, seq_id: int, total_tokens: int) -> None:
        """Grows a live sequence's page reservation to total_tokens."""
        check(self.lib.b2_seq_reserve(self.h, int(seq_id), int(total_tokens)), self.lib)

    def seq_free(self, seq_id: int) -> None:
        check(self.lib.b2_seq_free(self.h, int(seq_id)), self.lib)

    def seq_len(self, seq_id: int) -> int:
        return self.lib.b2_seq_len(self.h, int(seq_id))

    def seq_truncate(self, seq_id: int, new_len: int) -> None:
        check(self.lib.b2_seq_truncate(self.h, int(seq_id), int(new_len)), self.lib)

    def info(self) -> dict:
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        check(self.lib.b2_engine_info(self.h, C.byref(a), C.byref(b), C.byref(c)), self.lib)
        return {"num_blocks": a.value, "free_blocks": b.value, "weight_bytes": c.value}

    # ---- forward passes ------------------------------------------------------------------
    def prefill(self, seq_ids, prompts) -> np.ndarray:
        """prompts: list of int sequences (ragged).  Returns the greedy next token per sequence."""
        ids = _i32(np.concatenate([np.asarray(p, dtype=np.int32) for p in prompts]))
        offs = _i32(np.cumsum([0] + [len(p) for p in prompts]))
        sids = _i32(seq_ids)
        out = np.zeros(len(prompts), dtype=np.int32)
        check(self.lib.b2_prefill(self.h, _p32(ids), _p32(offs), len(prompts), _p32(sids), _p32(out)), self.lib)
        return out

    def prefill_logits(self, seq_ids, chunks, rows):
        """Appends chunks[i] to sequence seq_ids[i] (a prompt portion, or one decoded token) in ONE forward and returns
        (fp32 logits [len(rows)][vocab] at the given rows of the packed tokens, greedy next token per sequence)."""
        ids = _i32(np.concatenate([np.asarray(p, dtype=np.int32) for p in chunks]))
        offs = _i32(np.cumsum([0] + [len(p) for p in chunks]))
        sids, r = _i32(seq_ids), _i32(rows)
        out = np.zeros(len(chunks), dtype=np.int32)
        logits = np.zeros((len(r), self.cfg.vocab), dtype=np.float32)
        check(self.lib.b2_prefill_logits(self.h, _p32(ids), _p32(offs), len(chunks), _p32(sids), _p32(r), len(r),
                                         logits.ctypes.data_as(C.POINTER(C.c_float)), _p32(out)), self.lib)
        return logits, out

    def decode_step(self, seq_ids, in_tokens=None, want_output: bool = True):
        sids = _i32(seq_ids)
        n = len(sids)
        tin = _i32(in_tokens) if in_tokens is not None else None
        out = np.zeros(n, dtype=np.int32) if want_output else None
        check(self.lib.b2_decode_step(self.h, n, _p32(sids), _p32(tin) if tin is not None else None,
                                      _p32(out) if out is not None else None), self.lib)
        return out

    def decode_run(self, seq_ids, steps: int, want_tokens: bool = True):
        """`steps` decode steps with token feedback on the device.  Returns (tokens[steps][n], ms)."""
        sids = _i32(seq_ids)
        n = len(sids)
        out = np.zeros((steps, n), dtype=np.int32) if want_tokens else None
        ms = C.c_float(0)
        check(self.lib.b2_decode_run(self.h, n, _p32(sids), int(steps), _p32(out) if out is not None else None, C.byref(ms)),
              self.lib)
        return out, ms.value

    def decode_profile(self, seq_ids, steps: int) -> dict:
        sids = _i32(seq_ids)
        ms = (C.c_float * capi.NUM_KERNEL_CLASSES)()
        cnt = (C.c_int64 * capi.NUM_KERNEL_CLASSES)()
        check(self.lib.b2_decode_profile(self.h, len(sids), _p32(sids), int(steps), ms, cnt), self.lib)
        return {KERNEL_CLASSES[i]: {"ms": float(ms[i]), "launches": int(cnt[i])} for i in range(capi.NUM_KERNEL_CLASSES)}

    def attn_profile(self, seq_ids, reps: int = 8):
        """Decode-attention pass of every layer back to back, `reps` times, between one event pair.
        Returns (ms per launch, K/V bytes one launch must read)."""
        sids = _i32(seq_ids)
        ms = C.c_float(0)
        nbytes = C.c_int64(0)
        check(self.lib.b2_attn_profile(self.h, len(sids), _p32(sids), int(reps), C.byref(ms), C.byref(nbytes)), self.lib)
        return ms.value, int(nbytes.value)

    def prefix_cache_stats(self) -> dict:
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        check(self.lib.b2_prefix_cache_stats(self.h, C.byref(a), C.byref(b), C.byref(c)), self.lib)
        return {"queried_tokens": a.value, "hit_tokens": b.value, "cached_pages": c.value}

    def set_tuning(self, skip_mask: int | None = None, two_lane_min_batch: int | None = None, prefix_cache: bool | None = None) -> None:
        """Run-time measurement knobs (include/b2_engine.h, b2_set_tuning); drops the captured decode graphs."""
        if skip_mask is not None:
            check(self.lib.b2_set_tuning(self.h, 0, int(skip_mask)), self.lib)
        if two_lane_min_batch is not None:
            check(self.lib.b2_set_tuning(self.h, 1, int(two_lane_min_batch)), self.lib)
        if prefix_cache is not None:
            check(self.lib.b2_set_tuning(self.h, 2, 1 if prefix_cache else 0), self.lib)

    def launch_count(self) -> int:
        return int(self.lib.b2_launch_count(self.h))

    # ---- inspection ----------------------------------------------------------------------
    def set_debug(self, hidden: bool = False, logits: bool = False) -> None:
        check(self.lib.b2_set_debug(self.h, (1 if hidden else 0) | (2 if logits else 0)), self.lib)

    def get_logits(self, nseq: int) -> np.ndarray:
        out = np.zeros((nseq, self.cfg.vocab), dtype=np.float32)
        check(self.lib.b2_get_logits(self.h, nseq, out.ctypes.data_as(C.POINTER(C.c_float))), self.lib)
        return out

    def get_hidden(self, layer: int, ntokens: int) -> np.ndarray:
        """bf16 bit patterns [ntokens][hidden] as uint16."""
        out = np.zeros((ntokens, self.cfg.hidden), dtype=np.uint16)
        check(self.lib.b2_get_hidden(self.h, layer, ntokens, out.ctypes.data_as(C.POINTER(C.c_uint16))), self.lib)
        return out

    def get_hidden_f32(self, layer: int, ntokens: int) -> np.ndarray:
        """Residual stream after `layer` (-1 = the embedding output) of the last forward, families with an fp32 stream; with a looped run of
        layers `layer` counts layer runs (a looped layer once per pass)."""
        out = np.zeros((ntokens, self.cfg.hidden), dtype=np.float32)
        check(self.lib.b2_get_hidden_f32(self.h, layer, ntokens, out.ctypes.data_as(C.POINTER(C.c_float))), self.lib)
        return out

    def sample(self, nseq: int, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> np.ndarray:
        p = b2_sampling(temperature, top_k, top_p, seed)
        out = np.zeros(nseq, dtype=np.int32)
        check(self.lib.b2_sample(self.h, nseq, C.byref(p), _p32(out)), self.lib)
        return out

    def set_next_tokens(self, seq_ids, tokens) -> None:
        sids, toks = _i32(seq_ids), _i32(tokens)
        check(self.lib.b2_set_next_tokens(self.h, len(sids), _p32(sids), _p32(toks)), self.lib)

    # ---- lifetime ------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.b2_engine_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def _fill_layer_spec(sp, layer: dict) -> None:
    """One "layers" entry of a layer-list config.json -> b2_layer_spec (the C registry does the same for a directory)."""
    if layer["type"] == "gla" or layer["mixer"].get("q_rank") is not None or (layer["type"] == "attention" and layer.get("_tinevik")):
        return _fill_mixed_spec(sp, layer)
    if layer["type"] in ("attention", "attention_2"):
        return _fill_heads_spec(sp, layer)
    if layer["type"] in ("parallel", "channel_delta"):
        return _fill_state_spec(sp, layer)
    if layer["type"] != "latent_attention":
        raise B2Error("mixer type %r not built" % layer["type"])
    m = layer["mixer"]
    sp.mixer = capi.MIXER_LATENT_ATTENTION
    for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
        setattr(sp, k, int(m[k]))
    sp.kv_from = int(m["kv_from"]) if m.get("kv_from") is not None else -1
    sp.rot_dims, sp.rot_base, sp.scale = int(m["rot"]["dims"]), float(m["rot"]["base"]), float(m["scale"])
    mlp = layer.get("mlp")
    sp.ff = capi.FF_NONE
    if mlp is not None:
        if mlp["kind"] != "moe":
            raise B2Error("feed-forward kind %r not built" % mlp["kind"])
        r = mlp["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        sp.ff, sp.ff_dim, sp.experts, sp.top = capi.FF_ROUTED_EXPERTS, int(mlp["expert"]["ff"]), int(r["experts"]), int(r["top"])
        sp.groups, sp.groups_keep = int(g["count"]), int(g["keep"])


def _fill_mixed_spec(sp, layer: dict) -> None:
    """Tinevik: "gla", "attention" (scores mixed over the heads before the softmax, rotated values) and "latent_attention" (query latent,
    window, output gate).  An "attention" entry of this family is marked with "_tinevik": True (Engine.__init__ does it for arch "tinevik")."""
    m = layer["mixer"]
    sp.kv_from = -1
    sp.weights_of = int(layer["weights_of"]) if layer.get("weights_of") is not None else -1
    sp.heads, sp.dim, sp.vdim = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    sp.kv_heads = sp.heads
    if layer["type"] == "gla":
        sp.mixer, sp.s_tau = capi.MIXER_DECAY_STATE, float(m["tau"])
        sp.s_heads, sp.s_dim, sp.s_vdim = sp.heads, sp.dim, sp.vdim
    elif layer["type"] == "attention":
        sp.mixer = capi.MIXER_MIXED_SCORE_ATTENTION
        sp.kv_heads = int(m.get("kv_heads", m["heads"]))
        sp.scale, sp.softcap, sp.score_mix, sp.rot_factor = float(m["scale"]), float(m.get("softcap") or 0.0), 1, 1.0
        rot = m.get("rot")
        if rot:
            sp.rot_base, sp.rot_dims, sp.rot_values = float(rot["base"]), int(rot["dims"]), 1
            if rot.get("scaling"):
                sp.rot_factor = float(rot["scaling"]["factor"])
    else:
        sp.mixer = capi.MIXER_GATED_LATENT
        sp.kv_rank, sp.q_rank, sp.scale = int(m["kv_rank"]), int(m["q_rank"]), float(m["scale"])
        sp.window = int(m["mask"]["size"]) if m.get("mask") else 0
    mlp = layer.get("mlp")
    sp.ff = capi.FF_NONE
    if mlp is not None:
        if mlp["kind"] == "dense":
            sp.ff, sp.ff_dim = capi.FF_XIELU, int(mlp["ff"])
        elif mlp["kind"] == "moe":
            sp.ff, sp.ff_dim, sp.ff_limit = capi.FF_TABLE_EXPERTS, int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
            sp.experts, sp.top, sp.groups, sp.groups_keep = int(mlp["router"]["experts"]), int(mlp["router"]["top"]), 1, 1
        else:
            raise B2Error("feed-forward kind %r not built" % mlp["kind"])


def _mixed_layer_dict(sp) -> dict:
    if sp.mixer == capi.MIXER_DECAY_STATE:
        ty, m = "gla", {"heads": sp.heads, "dim": sp.dim, "vdim": sp.vdim, "tau": sp.s_tau}
    elif sp.mixer == capi.MIXER_MIXED_SCORE_ATTENTION:
        ty, m = "attention", {"heads": sp.heads, "kv_heads": sp.kv_heads, "dim": sp.dim, "vdim": sp.vdim, "scale": sp.scale}
        if sp.softcap > 0:
            m["softcap"] = sp.softcap
        if sp.rot_values:
            m["rot"] = {"base": sp.rot_base, "dims": sp.rot_dims, "scaling": {"factor": sp.rot_factor}}
    else:
        ty, m = "latent_attention", {"heads": sp.heads, "dim": sp.dim, "vdim": sp.vdim, "kv_rank": sp.kv_rank, "q_rank": sp.q_rank, "scale": sp.scale}
        if sp.window > 0:
            m["mask"] = {"size": sp.window}
    mlp = None
    if sp.ff == capi.FF_XIELU:
        mlp = {"kind": "dense", "ff": sp.ff_dim}
    elif sp.ff == capi.FF_TABLE_EXPERTS:
        mlp = {"kind": "moe", "expert": {"ff": sp.ff_dim, "limit": sp.ff_limit}, "router": {"experts": sp.experts, "top": sp.top}}
    d = {"type": ty, "mixer": m, "mlp": mlp, "_tinevik": True}
    if sp.weights_of >= 0:
        d["weights_of"] = sp.weights_of
    return d


def _fill_state_spec(sp, layer: dict) -> None:
    """Bumalix: "parallel" (windowed softmax attention beside gated linear attention) and "channel_delta" (gated delta rule)."""
    m = layer["mixer"]
    sp.kv_from = -1
    if layer["type"] == "parallel":
        a, b = m["left"], m["right"]
        sp.mixer = capi.MIXER_WINDOW_AND_STATE
        sp.heads, sp.kv_heads, sp.dim, sp.vdim = int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"])
        sp.scale = float(a["scale"])
        sp.window = int(a["mask"]["size"]) if a.get("mask") else 0
        sp.s_heads, sp.s_dim, sp.s_vdim, sp.s_tau = int(b["heads"]), int(b["dim"]), int(b["vdim"]), float(b["tau"])
    else:
        sp.mixer = capi.MIXER_DELTA_STATE
        sp.heads, sp.kv_heads, sp.dim, sp.vdim = int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"])
        sp.conv_taps = int(m["conv"])
    mlp = layer.get("mlp")
    sp.ff = capi.FF_NONE
    if mlp is not None:
        if mlp["kind"] == "dense":
            sp.ff, sp.ff_dim = capi.FF_POLYNORM, int(mlp["ff"])
        elif mlp["kind"] == "moe":
            sp.ff, sp.ff_dim = capi.FF_SCALED_GATED_EXPERTS, int(mlp["expert"]["ff"])
            sp.experts, sp.top, sp.groups, sp.groups_keep = int(mlp["router"]["experts"]), int(mlp["router"]["top"]), 1, 1
            sp.shared_ff = int(mlp["shared"]["ff"]) if mlp.get("shared") else 0
        else:
            raise B2Error("feed-forward kind %r not built" % mlp["kind"])


def _fill_heads_spec(sp, layer: dict) -> None:
    """Kedasun: "attention" (rotary grouped-query attention) and "attention_2" (convolution, window, weight mixing, gate)."""
    m = layer["mixer"]
    conv = layer["type"] == "attention_2"
    sp.mixer = capi.MIXER_CONV_ATTENTION if conv else capi.MIXER_ATTENTION
    for k in ("heads", "dim", "vdim"):
        setattr(sp, k, int(m[k]))
    sp.kv_heads = int(m.get("kv_heads", m["heads"]))
    sp.scale, sp.kv_from, sp.v_mix = float(m["scale"]), -1, int(bool(m.get("v_mix")))
    if conv:
        sp.conv_taps = int(m["conv"])
        mask = m.get("mask")
        if mask:
            sp.window, sp.keep_first = int(mask["size"]), int(mask.get("keep_first", 0))
    elif m.get("rot"):
        sp.rot_dims, sp.rot_base = int(m["rot"]["dims"]), float(m["rot"]["base"])
    mlp = layer.get("mlp")
    sp.ff = capi.FF_NONE
    if mlp is not None:
        if mlp["kind"] != "dense":
            raise B2Error("feed-forward kind %r not built" % mlp["kind"])
        sp.ff, sp.ff_dim, sp.ff_limit = capi.FF_CLAMPED_GATED, int(mlp["ff"]), float(mlp["limit"])


def _layer_dict(sp) -> dict:
    if sp.mixer in (capi.MIXER_DECAY_STATE, capi.MIXER_MIXED_SCORE_ATTENTION, capi.MIXER_GATED_LATENT):
        return _mixed_layer_dict(sp)
    if sp.mixer in (capi.MIXER_WINDOW_AND_STATE, capi.MIXER_DELTA_STATE):
        if sp.mixer == capi.MIXER_WINDOW_AND_STATE:
            left = {"heads": sp.heads, "kv_heads": sp.kv_heads, "dim": sp.dim, "vdim": sp.vdim, "scale": sp.scale}
            if sp.window > 0:
                left["mask"] = {"size": sp.window}
            m = {"left": left, "right": {"heads": sp.s_heads, "dim": sp.s_dim, "vdim": sp.s_vdim, "tau": sp.s_tau}}
        else:
            m = {"heads": sp.heads, "kv_heads": sp.kv_heads, "dim": sp.dim, "vdim": sp.vdim, "conv": sp.conv_taps}
        mlp = None
        if sp.ff == capi.FF_POLYNORM:
            mlp = {"kind": "dense", "ff": sp.ff_dim}
        elif sp.ff == capi.FF_SCALED_GATED_EXPERTS:
            mlp = {"kind": "moe", "expert": {"ff": sp.ff_dim}, "router": {"experts": sp.experts, "top": sp.top}}
            if sp.shared_ff > 0:
                mlp["shared"] = {"ff": sp.shared_ff}
        return {"type": "parallel" if sp.mixer == capi.MIXER_WINDOW_AND_STATE else "channel_delta", "mixer": m, "mlp": mlp}
    if sp.mixer in (capi.MIXER_ATTENTION, capi.MIXER_CONV_ATTENTION):
        m = {"heads": sp.heads, "kv_heads": sp.kv_heads, "dim": sp.dim, "vdim": sp.vdim, "scale": sp.scale, "v_mix": bool(sp.v_mix)}
        if sp.mixer == capi.MIXER_CONV_ATTENTION:
            m["conv"] = sp.conv_taps
            if sp.window > 0:
                m["mask"] = {"size": sp.window, "keep_first": sp.keep_first}
        elif sp.rot_dims > 0:
            m["rot"] = {"base": sp.rot_base, "dims": sp.rot_dims}
        mlp = {"kind": "dense", "ff": sp.ff_dim, "limit": sp.ff_limit} if sp.ff == capi.FF_CLAMPED_GATED else None
        return {"type": "attention_2" if sp.mixer == capi.MIXER_CONV_ATTENTION else "attention", "mixer": m, "mlp": mlp}
    m = {"heads": sp.heads, "dim": sp.dim, "rot_dim": sp.rot_dim, "vdim": sp.vdim, "kv_rank": sp.kv_rank, "scale": sp.scale,
         "rot": {"base": sp.rot_base, "dims": sp.rot_dims}}
    if sp.kv_from >= 0:
        m["kv_from"] = sp.kv_from
    mlp = None
    if sp.ff == capi.FF_ROUTED_EXPERTS:
        mlp = {"kind": "moe", "expert": {"ff": sp.ff_dim},
               "router": {"experts": sp.experts, "top": sp.top, "groups": {"count": sp.groups, "keep": sp.groups_keep}}}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)
