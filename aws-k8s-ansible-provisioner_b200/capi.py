"""ctypes binding of include/b2_engine.h (the same stub INTEGRATION.md shows a maintainer)."""
from __future__ import annotations

import ctypes as C
import os

# B2_LIB_PATH: an alternative build of the same library (A/B measurements of one source change); never a fallback
LIB_PATH = os.environ.get("B2_LIB_PATH") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libb2engine.so")
ABI_VERSION = 6
ARCH_QWEN3, ARCH_PHI3, ARCH_OPT, ARCH_LERASUN, ARCH_KEDASUN, ARCH_BUMALIX, ARCH_TINEVIK = 0, 1, 2, 3, 4, 5, 6
MIXER_LATENT_ATTENTION, MIXER_ATTENTION, MIXER_CONV_ATTENTION, MIXER_WINDOW_AND_STATE, MIXER_DELTA_STATE = 1, 2, 3, 4, 5
MIXER_DECAY_STATE, MIXER_MIXED_SCORE_ATTENTION, MIXER_GATED_LATENT = 6, 7, 8
FF_NONE, FF_ROUTED_EXPERTS, FF_CLAMPED_GATED, FF_POLYNORM, FF_SCALED_GATED_EXPERTS, FF_XIELU, FF_TABLE_EXPERTS = 0, 1, 2, 3, 4, 5, 6
NUM_KERNEL_CLASSES = 12


class B2Error(RuntimeError):
    pass


class b2_layer_spec(C.Structure):
    _fields_ = [
        ("mixer", C.c_int32), ("heads", C.c_int32), ("dim", C.c_int32), ("rot_dim", C.c_int32), ("vdim", C.c_int32),
        ("kv_rank", C.c_int32), ("kv_from", C.c_int32), ("rot_dims", C.c_int32), ("rot_base", C.c_float), ("scale", C.c_float),
        ("ff", C.c_int32), ("ff_dim", C.c_int32), ("experts", C.c_int32), ("top", C.c_int32), ("groups", C.c_int32),
        ("groups_keep", C.c_int32), ("kv_heads", C.c_int32), ("conv_taps", C.c_int32), ("window", C.c_int32),
        ("keep_first", C.c_int32), ("v_mix", C.c_int32), ("ff_limit", C.c_float),
        ("s_heads", C.c_int32), ("s_dim", C.c_int32), ("s_vdim", C.c_int32), ("s_tau", C.c_float), ("shared_ff", C.c_int32),
        ("weights_of", C.c_int32), ("q_rank", C.c_int32), ("rot_factor", C.c_float), ("softcap", C.c_float), ("score_mix", C.c_int32),
        ("rot_values", C.c_int32),
    ]


class b2_config(C.Structure):
    _fields_ = [
        ("abi_version", C.c_int32), ("num_layers", C.c_int32), ("hidden", C.c_int32), ("num_q_heads", C.c_int32),
        ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("intermediate", C.c_int32), ("vocab", C.c_int32),
        ("tie_embeddings", C.c_int32), ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("max_model_len", C.c_int32),
        ("block_size", C.c_int32), ("num_blocks", C.c_int32), ("gpu_mem_fraction", C.c_float), ("max_seqs", C.c_int32),
        ("max_batch_tokens", C.c_int32), ("use_cuda_graphs", C.c_int32), ("rope_inv_freq", C.POINTER(C.c_float)),
        ("arch", C.c_int32), ("rotary_dim", C.c_int32), ("max_positions", C.c_int32), ("sliding_window", C.c_int32),
        ("layer_specs", C.POINTER(b2_layer_spec)), ("compute_f32", C.c_int32), ("logit_scale", C.c_float),
        ("embed_scale", C.c_float), ("norm_groups", C.c_int32),
        ("loop_start", C.c_int32), ("loop_stop", C.c_int32), ("loop_times", C.c_int32), ("logit_softcap", C.c_float),
        ("norm_kind", C.c_int32),
    ]


class b2_sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("seed", C.c_uint64)]


_P = C.c_void_p
_I = C.c_int
_I32P = C.POINTER(C.c_int32)

# name -> (restype, argtypes); every symbol include/b2_engine.h declares
SIGNATURES = {
    "b2_last_error": (C.c_char_p, []),
    "b2_abi_version": (_I, []),
    "b2_engine_create": (_I, [C.POINTER(b2_config), C.c_char_p, _I, C.POINTER(_P)]),
    "b2_engine_load_tensor": (_I, [_P, C.c_char_p, _P, C.c_size_t]),
    "b2_engine_load_int_tensor": (_I, [_P, C.c_char_p, _I32P, C.c_size_t]),
    "b2_engine_load_safetensors": (_I, [_P, C.c_char_p]),
    "b2_engine_finalize": (_I, [_P]),
    "b2_engine_free": (None, [_P]),
    "b2_engine_info": (_I, [_P, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "b2_seq_create": (_I, [_P, C.c_int32, _I32P]),
    "b2_seq_reserve": (_I, [_P, C.c_int32, C.c_int32]),
    "b2_seq_free": (_I, [_P, C.c_int32]),
    "b2_seq_len": (_I, [_P, C.c_int32]),
    "b2_seq_truncate": (_I, [_P, C.c_int32, C.c_int32]),
    "b2_prefill": (_I, [_P, _I32P, _I32P, C.c_int32, _I32P, _I32P]),
    "b2_decode_step": (_I, [_P, C.c_int32, _I32P, _I32P, _I32P]),
    "b2_decode_run": (_I, [_P, C.c_int32, _I32P, C.c_int32, _I32P, C.POINTER(C.c_float)]),
    "b2_get_logits": (_I, [_P, C.c_int32, C.POINTER(C.c_float)]),
    "b2_config_from_dir": (_I, [C.c_char_p, C.POINTER(b2_config), C.POINTER(b2_layer_spec), C.c_int32]),
    "b2_prefill_logits": (_I, [_P, _I32P, _I32P, C.c_int32, _I32P, _I32P, C.c_int32, C.POINTER(C.c_float), _I32P]),
    "b2_get_hidden_f32": (_I, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_float)]),
    "b2_set_debug": (_I, [_P, C.c_int32]),
    "b2_get_hidden": (_I, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_uint16)]),
    "b2_sample": (_I, [_P, C.c_int32, C.POINTER(b2_sampling), _I32P]),
    "b2_sample_rows": (_I, [_P, C.c_int32, _I32P, C.POINTER(b2_sampling), _I32P]),
    "b2_set_next_tokens": (_I, [_P, C.c_int32, _I32P, _I32P]),
    "b2_decode_profile": (_I, [_P, C.c_int32, _I32P, C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
    "b2_attn_profile": (_I, [_P, C.c_int32, _I32P, C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
    "b2_launch_count": (C.c_int64, [_P]),
    "b2_set_tuning": (_I, [_P, C.c_int32, C.c_int64]),
    "b2_prefix_cache_stats": (_I, [_P, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "b2k_add_rmsnorm": (_I, [_P, _P, _I, _I, _P, _P, _I, _I, C.c_float, _P]),
    "b2k_qknorm_rope_kv": (_I, [_P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, C.c_float, _P]),
    "b2k_silu_mul": (_I, [_P, _I, _I, _P, _I, _I, _P]),
    "b2k_linear": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P]),
    "b2k_gateup_swiglu": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "b2k_qkv_rope": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, C.c_float, _P]),
    "b2k_linear_resid": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "b2k_linear_add": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "b2k_linear_multicast": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "b2k_gateup_swiglu_norm": (_I, [_P, _P, _P, _P, _I, _I, C.c_float, _P, _I, _I, _I, _P]),
    "b2k_qkv_rope_norm": (_I, [_P, _P, _P, _P, _I, _I, C.c_float, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, C.c_float, _P]),
    "b2k_debug_step_trace": (_I, [_P]),
    "b2k_debug_gemm_trace": (_I, [_P]),
    "b2k_debug_chain_trace": (_I, [_P]),
    "b2k_debug_fused_trace": (_I, [_P]),
    "b2k_lmhead_argmax": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "b2k_attn_decode": (_I, [_P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "b2k_attn_decode_scratch_floats": (C.c_size_t, [_I, _I, _I, _I]),
    "b2k_attn_decode_noalloc": (_I, [_P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P]),
    "b2k_attn_prefill": (_I, [_P, _P, _P, _P, _I, _I32P, _I32P, _I32P, _I32P, _I, _P, _I, _I, _I, _I, _P]),
}

_lib = None


def load_library(path: str | None = None):
    """Loads libb2engine.so and types every entry point.  Fails loudly when it is not built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise B2Error(
            "%s is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`. "
            "There is no CPU fallback for this engine." % p)
    lib = C.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    if lib.b2_abi_version() != ABI_VERSION:
        raise B2Error("ABI mismatch: library %d, binding %d" % (lib.b2_abi_version(), ABI_VERSION))
    if path is None:
        _lib = lib
    return lib


def check(rc: int, lib=None) -> None:
    if rc != 0:
        lib = lib or load_library()
        raise B2Error("b2 error %d: %s" % (rc, (lib.b2_last_error() or b"").decode("utf-8", "replace")))
