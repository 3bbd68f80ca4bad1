// model_config.cu -- the model registry: MODEL_DIR/config.json -> b2_config (+ the layer list of the families that have
// one).  b2serve, the Python mirror and bin/trace_run all choose the model class through this one function, so a family
// is added to the framework here, in b2_engine_create and nowhere else.  Host code only.
//
// The fourth layer-list family, Tinevik, is described above its reader (tinevik_config).
// HF families are told apart by "model_type" (the keys follow HF's Qwen3Config / Phi3Config / OPTConfig); Lerasun by
// "architecture": "Lerasun", whose config lists its layers one by one:
//   {"architecture": "Lerasun", "vocab": V, "width": W, "logit_scale": s, "norm": {"eps": e},
//    "layers": [{"type": "latent_attention",
//                "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"}, "kv_from"?},
//                "mlp": null | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}}}}, ...]}
// Kedasun by "architecture": "Kedasun":
//   {"architecture": "Kedasun", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e, "groups": n},
//    "layers": [{"type": "attention",   "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"base", "dims"}, "v_mix"?}, "mlp": ...},
//               {"type": "attention_2", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "conv", "mask": {"size", "keep_first"}?, "v_mix"?},
//                "mlp": null | {"kind": "dense", "ff", "limit"}}, ...]}
// Bumalix by "architecture": "Bumalix":
//   {"architecture": "Bumalix", "vocab": V, "width": W, "embedding": {"scale": s}, "norm": {"eps": e}, "logit_softcap": c?,
//    "loop": {"start", "stop", "times"}?,
//    "layers": [{"type": "parallel", "mixer": {"left": {"heads", "kv_heads"?, "dim", "vdim", "scale", "mask": {"size"}?},
//                                              "right": {"heads", "dim", "vdim", "tau"}}, "mlp": ...},
//               {"type": "channel_delta", "mixer": {"heads", "kv_heads"?, "dim", "vdim", "conv"},
//                "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared": {"ff"}?}}, ...]}
#include <fstream>
#include <sstream>
#include <string>

#include "../../include/b2_engine.h"
#include "common.cuh"
#include "json.hpp"

using b2json::Value;

namespace {

int need_int(const Value& o, const char* key, const char* where, int* out) {
  const Value* v = o.find(key);
  if (!v || !v->is_number()) {
    b2_set_error("config.json: %s.%s missing or not a number", where, key);
    return -22;
  }
  *out = (int)v->as_int();
  return 0;
}
int need_float(const Value& o, const char* key, const char* where, float* out) {
  const Value* v = o.find(key);
  if (!v || !v->is_number()) {
    b2_set_error("config.json: %s.%s missing or not a number", where, key);
    return -22;
  }
  *out = (float)v->as_double();
  return 0;
}
#define CFG_TRY(expr)       \
  do {                      \
    int _r = (expr);        \
    if (_r != 0) return _r; \
  } while (0)

int lerasun_config(const Value& j, b2_config* c, b2_layer_spec* specs, int max_specs) {
  c->arch = B2_ARCH_LERASUN;
  CFG_TRY(need_int(j, "vocab", "config", &c->vocab));
  CFG_TRY(need_int(j, "width", "config", &c->hidden));
  const Value* norm = j.find("norm");
  if (!norm || !norm->is_object()) {
    b2_set_error("config.json: norm missing");
    return -22;
  }
  CFG_TRY(need_float(*norm, "eps", "norm", &c->rms_eps));
  c->logit_scale = 1.0f;
  if (const Value* ls = j.find("logit_scale"))
    if (ls->is_number()) c->logit_scale = (float)ls->as_double();
  const Value* layers = j.find("layers");
  if (!layers || !layers->is_array() || layers->size() == 0) {
    b2_set_error("config.json: layers missing or empty");
    return -22;
  }
  c->num_layers = (int)layers->size();
  if (c->num_layers > max_specs || specs == nullptr) {
    b2_set_error("config.json: %d layers, room for %d layer specs", c->num_layers, max_specs);
    return -22;
  }
  for (int i = 0; i < c->num_layers; ++i) {
    const Value& L = layers->at(i);
    b2_layer_spec& s = specs[i];
    memset(&s, 0, sizeof s);
    char where[48];
    snprintf(where, sizeof where, "layers[%d].mixer", i);
    const Value* type = L.find("type");
    const Value* m = L.find("mixer");
    if (!type || !type->is_string() || !m || !m->is_object()) {
      b2_set_error("config.json: layers[%d] needs type and mixer", i);
      return -22;
    }
    if (type->as_string() != "latent_attention") {
      b2_set_error("config.json: layers[%d]: mixer type '%s' not built (latent_attention)", i, type->as_string().c_str());
      return -22;
    }
    s.mixer = B2_MIXER_LATENT_ATTENTION;
    CFG_TRY(need_int(*m, "heads", where, &s.heads));
    CFG_TRY(need_int(*m, "dim", where, &s.dim));
    CFG_TRY(need_int(*m, "rot_dim", where, &s.rot_dim));
    CFG_TRY(need_int(*m, "vdim", where, &s.vdim));
    CFG_TRY(need_int(*m, "kv_rank", where, &s.kv_rank));
    CFG_TRY(need_float(*m, "scale", where, &s.scale));
    const Value* rot = m->find("rot");
    if (!rot || !rot->is_object()) {
      b2_set_error("config.json: %s.rot missing", where);
      return -22;
    }
    CFG_TRY(need_float(*rot, "base", where, &s.rot_base));
    CFG_TRY(need_int(*rot, "dims", where, &s.rot_dims));
    s.kv_from = -1;
    if (const Value* kf = m->find("kv_from"))
      if (kf->is_number()) s.kv_from = (int)kf->as_int();
    const Value* mlp = L.find("mlp");
    s.ff = B2_FF_NONE;
    if (mlp && mlp->is_object()) {
      snprintf(where, sizeof where, "layers[%d].mlp", i);
      const Value* kind = mlp->find("kind");
      if (!kind || !kind->is_string() || kind->as_string() != "moe") {
        b2_set_error("config.json: %s.kind '%s' not built (moe)", where, kind && kind->is_string() ? kind->as_string().c_str() : "?");
        return -22;
      }
      s.ff = B2_FF_ROUTED_EXPERTS;
      const Value* ex = mlp->find("expert");
      const Value* ro = mlp->find("router");
      if (!ex || !ex->is_object() || !ro || !ro->is_object()) {
        b2_set_error("config.json: %s needs expert and router", where);
        return -22;
      }
      CFG_TRY(need_int(*ex, "ff", where, &s.ff_dim));
      CFG_TRY(need_int(*ro, "experts", where, &s.experts));
      CFG_TRY(need_int(*ro, "top", where, &s.top));
      s.groups = 1;
      s.groups_keep = 1;
      if (const Value* gr = ro->find("groups"))
        if (gr->is_object()) {
          CFG_TRY(need_int(*gr, "count", where, &s.groups));
          CFG_TRY(need_int(*gr, "keep", where, &s.groups_keep));
        }
    }
  }
  c->layer_specs = specs;
  c->tie_embeddings = 0;
  // the GQA fields describe nothing in this family
  c->num_q_heads = c->num_kv_heads = 0;
  c->head_dim = c->intermediate = 0;
  return 0;
}

int kedasun_config(const Value& j, b2_config* c, b2_layer_spec* specs, int max_specs) {
  c->arch = B2_ARCH_KEDASUN;
  CFG_TRY(need_int(j, "vocab", "config", &c->vocab));
  CFG_TRY(need_int(j, "width", "config", &c->hidden));
  const Value* norm = j.find("norm");
  if (!norm || !norm->is_object()) {
    b2_set_error("config.json: norm missing");
    return -22;
  }
  CFG_TRY(need_float(*norm, "eps", "norm", &c->rms_eps));
  c->norm_groups = 1;
  if (const Value* g = norm->find("groups"))
    if (g->is_number()) c->norm_groups = (int)g->as_int();
  c->embed_scale = 1.0f;
  if (const Value* em = j.find("embedding"))
    if (em->is_object())
      if (const Value* sc = em->find("scale"))
        if (sc->is_number()) c->embed_scale = (float)sc->as_double();
  c->logit_scale = 1.0f;
  const Value* layers = j.find("layers");
  if (!layers || !layers->is_array() || layers->size() == 0) {
    b2_set_error("config.json: layers missing or empty");
    return -22;
  }
  c->num_layers = (int)layers->size();
  if (c->num_layers > max_specs || specs == nullptr) {
    b2_set_error("config.json: %d layers, room for %d layer specs", c->num_layers, max_specs);
    return -22;
  }
  for (int i = 0; i < c->num_layers; ++i) {
    const Value& L = layers->at(i);
    b2_layer_spec& s = specs[i];
    memset(&s, 0, sizeof s);
    s.kv_from = -1;
    char where[48];
    snprintf(where, sizeof where, "layers[%d].mixer", i);
    const Value* type = L.find("type");
    const Value* m = L.find("mixer");
    if (!type || !type->is_string() || !m || !m->is_object()) {
      b2_set_error("config.json: layers[%d] needs type and mixer", i);
      return -22;
    }
    if (type->as_string() == "attention") s.mixer = B2_MIXER_ATTENTION;
    else if (type->as_string() == "attention_2") s.mixer = B2_MIXER_CONV_ATTENTION;
    else {
      b2_set_error("config.json: layers[%d]: mixer type '%s' not built (attention, attention_2)", i, type->as_string().c_str());
      return -22;
    }
    CFG_TRY(need_int(*m, "heads", where, &s.heads));
    s.kv_heads = s.heads;   // no "kv_heads": every query head has its own keys and values
    if (const Value* kh = m->find("kv_heads"))
      if (kh->is_number()) s.kv_heads = (int)kh->as_int();
    CFG_TRY(need_int(*m, "dim", where, &s.dim));
    CFG_TRY(need_int(*m, "vdim", where, &s.vdim));
    CFG_TRY(need_float(*m, "scale", where, &s.scale));
    if (const Value* vm = m->find("v_mix")) s.v_mix = vm->is_bool() ? (vm->b ? 1 : 0) : (vm->is_number() && vm->as_int() != 0 ? 1 : 0);
    if (s.mixer == B2_MIXER_ATTENTION) {
      const Value* rot = m->find("rot");
      if (rot && rot->is_object()) {  // no "rot": nothing is rotated
        CFG_TRY(need_float(*rot, "base", where, &s.rot_base));
        CFG_TRY(need_int(*rot, "dims", where, &s.rot_dims));
      }
    } else {
      CFG_TRY(need_int(*m, "conv", where, &s.conv_taps));
      const Value* mask = m->find("mask");
      if (mask && mask->is_object()) {  // no "mask": every earlier key is seen
        CFG_TRY(need_int(*mask, "size", where, &s.window));
        if (const Value* kf = mask->find("keep_first"))
          if (kf->is_number()) s.keep_first = (int)kf->as_int();
      }
    }
    const Value* mlp = L.find("mlp");
    s.ff = B2_FF_NONE;
    if (mlp && mlp->is_object()) {
      snprintf(where, sizeof where, "layers[%d].mlp", i);
      const Value* kind = mlp->find("kind");
      if (!kind || !kind->is_string() || kind->as_string() != "dense") {
        b2_set_error("config.json: %s.kind '%s' not built (dense)", where, kind && kind->is_string() ? kind->as_string().c_str() : "?");
        return -22;
      }
      s.ff = B2_FF_CLAMPED_GATED;
      CFG_TRY(need_int(*mlp, "ff", where, &s.ff_dim));
      CFG_TRY(need_float(*mlp, "limit", where, &s.ff_limit));
    }
  }
  c->layer_specs = specs;
  c->tie_embeddings = 0;
  c->num_q_heads = c->num_kv_heads = 0;
  c->head_dim = c->intermediate = 0;
  return 0;
}

int bumalix_config(const Value& j, b2_config* c, b2_layer_spec* specs, int max_specs) {
  c->arch = B2_ARCH_BUMALIX;
  CFG_TRY(need_int(j, "vocab", "config", &c->vocab));
  CFG_TRY(need_int(j, "width", "config", &c->hidden));
  const Value* norm = j.find("norm");
  if (!norm || !norm->is_object()) {
    b2_set_error("config.json: norm missing");
    return -22;
  }
  CFG_TRY(need_float(*norm, "eps", "norm", &c->rms_eps));
  c->norm_groups = 1;
  c->embed_scale = 1.0f;
  if (const Value* em = j.find("embedding"))
    if (em->is_object())
      if (const Value* sc = em->find("scale"))
        if (sc->is_number()) c->embed_scale = (float)sc->as_double();
  c->logit_scale = 1.0f;
  c->logit_softcap = 0.f;
  if (const Value* cap = j.find("logit_softcap"))
    if (cap->is_number()) c->logit_softcap = (float)cap->as_double();
  c->loop_start = c->loop_stop = c->loop_times = 0;
  if (const Value* loop = j.find("loop"))
    if (loop->is_object()) {
      CFG_TRY(need_int(*loop, "start", "loop", &c->loop_start));
      CFG_TRY(need_int(*loop, "stop", "loop", &c->loop_stop));
      CFG_TRY(need_int(*loop, "times", "loop", &c->loop_times));
    }
  const Value* layers = j.find("layers");
  if (!layers || !layers->is_array() || layers->size() == 0) {
    b2_set_error("config.json: layers missing or empty");
    return -22;
  }
  c->num_layers = (int)layers->size();
  if (c->num_layers > max_specs || specs == nullptr) {
    b2_set_error("config.json: %d layers, room for %d layer specs", c->num_layers, max_specs);
    return -22;
  }
  if (c->loop_times > 0 && !(c->loop_start >= 0 && c->loop_start <= c->loop_stop && c->loop_stop <= c->num_layers)) {
    b2_set_error("config.json: loop [%d, %d) outside the %d layers", c->loop_start, c->loop_stop, c->num_layers);
    return -22;
  }
  for (int i = 0; i < c->num_layers; ++i) {
    const Value& L = layers->at(i);
    b2_layer_spec& s = specs[i];
    memset(&s, 0, sizeof s);
    s.kv_from = -1;
    char where[64];
    snprintf(where, sizeof where, "layers[%d].mixer", i);
    const Value* type = L.find("type");
    const Value* m = L.find("mixer");
    if (!type || !type->is_string() || !m || !m->is_object()) {
      b2_set_error("config.json: layers[%d] needs type and mixer", i);
      return -22;
    }
    if (type->as_string() == "parallel") {
      s.mixer = B2_MIXER_WINDOW_AND_STATE;
      const Value* a = m->find("left");
      const Value* b = m->find("right");
      if (!a || !a->is_object() || !b || !b->is_object()) {
        b2_set_error("config.json: %s needs left and right", where);
        return -22;
      }
      snprintf(where, sizeof where, "layers[%d].mixer.left", i);
      CFG_TRY(need_int(*a, "heads", where, &s.heads));
      s.kv_heads = s.heads;
      if (const Value* kh = a->find("kv_heads"))
        if (kh->is_number()) s.kv_heads = (int)kh->as_int();
      CFG_TRY(need_int(*a, "dim", where, &s.dim));
      CFG_TRY(need_int(*a, "vdim", where, &s.vdim));
      CFG_TRY(need_float(*a, "scale", where, &s.scale));
      const Value* mask = a->find("mask");
      if (mask && mask->is_object()) CFG_TRY(need_int(*mask, "size", where, &s.window));  // no "mask": every earlier key is seen
      snprintf(where, sizeof where, "layers[%d].mixer.right", i);
      CFG_TRY(need_int(*b, "heads", where, &s.s_heads));
      CFG_TRY(need_int(*b, "dim", where, &s.s_dim));
      CFG_TRY(need_int(*b, "vdim", where, &s.s_vdim));
      CFG_TRY(need_float(*b, "tau", where, &s.s_tau));
    } else if (type->as_string() == "channel_delta") {
      s.mixer = B2_MIXER_DELTA_STATE;
      CFG_TRY(need_int(*m, "heads", where, &s.heads));
      s.kv_heads = s.heads;
      if (const Value* kh = m->find("kv_heads"))
        if (kh->is_number()) s.kv_heads = (int)kh->as_int();
      CFG_TRY(need_int(*m, "dim", where, &s.dim));
      CFG_TRY(need_int(*m, "vdim", where, &s.vdim));
      CFG_TRY(need_int(*m, "conv", where, &s.conv_taps));
    } else {
      b2_set_error("config.json: layers[%d]: mixer type '%s' not built (parallel, channel_delta)", i, type->as_string().c_str());
      return -22;
    }
    const Value* mlp = L.find("mlp");
    s.ff = B2_FF_NONE;
    if (mlp && mlp->is_object()) {
      snprintf(where, sizeof where, "layers[%d].mlp", i);
      const Value* kind = mlp->find("kind");
      const std::string kd = kind && kind->is_string() ? kind->as_string() : "?";
      if (kd == "dense") {
        s.ff = B2_FF_POLYNORM;
        CFG_TRY(need_int(*mlp, "ff", where, &s.ff_dim));
      } else if (kd == "moe") {
        s.ff = B2_FF_SCALED_GATED_EXPERTS;
        const Value* ex = mlp->find("expert");
        const Value* ro = mlp->find("router");
        if (!ex || !ex->is_object() || !ro || !ro->is_object()) {
          b2_set_error("config.json: %s needs expert and router", where);
          return -22;
        }
        CFG_TRY(need_int(*ex, "ff", where, &s.ff_dim));
        CFG_TRY(need_int(*ro, "experts", where, &s.experts));
        CFG_TRY(need_int(*ro, "top", where, &s.top));
        s.groups = s.groups_keep = 1;
        if (const Value* sh = mlp->find("shared"))
          if (sh->is_object()) CFG_TRY(need_int(*sh, "ff", where, &s.shared_ff));
      } else {
        b2_set_error("config.json: %s.kind '%s' not built (dense, moe)", where, kd.c_str());
        return -22;
      }
    }
  }
  c->layer_specs = specs;
  c->tie_embeddings = 0;
  c->num_q_heads = c->num_kv_heads = 0;
  c->head_dim = c->intermediate = 0;
  return 0;
}

// Tinevik: {"architecture": "Tinevik", "vocab": V, "width": W, "embedding": {"scale": s}?, "logit_scale": s?, "norm": {"eps": e},
//   "layers": [{"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ..., "weights_of": j?},
//              {"type": "attention", "mixer": {"heads", "kv_heads"?, "dim", "vdim", "scale", "softcap"?,
//                                              "rot": {"base", "dims", "scaling": {"factor"}?}?}, "mlp": ...},
//              {"type": "latent_attention", "mixer": {"heads", "dim", "vdim", "kv_rank", "q_rank", "scale", "mask": {"size"}?},
//               "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}}, ...]}
int tinevik_config(const Value& j, b2_config* c, b2_layer_spec* specs, int max_specs) {
  c->arch = B2_ARCH_TINEVIK;
  CFG_TRY(need_int(j, "vocab", "config", &c->vocab));
  CFG_TRY(need_int(j, "width", "config", &c->hidden));
  const Value* norm = j.find("norm");
  if (!norm || !norm->is_object()) {
    b2_set_error("config.json: norm missing");
    return -22;
  }
  CFG_TRY(need_float(*norm, "eps", "norm", &c->rms_eps));
  c->norm_groups = 1;
  c->norm_kind = 1;
  c->embed_scale = 1.0f;
  if (const Value* em = j.find("embedding"))
    if (em->is_object())
      if (const Value* sc = em->find("scale"))
        if (sc->is_number()) c->embed_scale = (float)sc->as_double();
  c->logit_scale = 1.0f;
  if (const Value* ls = j.find("logit_scale"))
    if (ls->is_number()) c->logit_scale = (float)ls->as_double();
  const Value* layers = j.find("layers");
  if (!layers || !layers->is_array() || layers->size() == 0) {
    b2_set_error("config.json: layers missing or empty");
    return -22;
  }
  c->num_layers = (int)layers->size();
  if (c->num_layers > max_specs || specs == nullptr) {
    b2_set_error("config.json: %d layers, room for %d layer specs", c->num_layers, max_specs);
    return -22;
  }
  for (int i = 0; i < c->num_layers; ++i) {
    const Value& L = layers->at(i);
    b2_layer_spec& s = specs[i];
    memset(&s, 0, sizeof s);
    s.kv_from = -1;
    s.weights_of = -1;
    char where[64];
    snprintf(where, sizeof where, "layers[%d].mixer", i);
    const Value* type = L.find("type");
    const Value* m = L.find("mixer");
    if (!type || !type->is_string() || !m || !m->is_object()) {
      b2_set_error("config.json: layers[%d] needs type and mixer", i);
      return -22;
    }
    if (const Value* wo = L.find("weights_of"))
      if (wo->is_number()) {
        s.weights_of = (int)wo->as_int();
        if (s.weights_of < 0 || s.weights_of >= c->num_layers || s.weights_of == i) {
          b2_set_error("config.json: layers[%d].weights_of %d names no other layer", i, s.weights_of);
          return -22;
        }
      }
    const std::string ty = type->as_string();
    CFG_TRY(need_int(*m, "heads", where, &s.heads));
    s.kv_heads = s.heads;
    CFG_TRY(need_int(*m, "dim", where, &s.dim));
    CFG_TRY(need_int(*m, "vdim", where, &s.vdim));
    if (ty == "gla") {
      s.mixer = B2_MIXER_DECAY_STATE;
      CFG_TRY(need_float(*m, "tau", where, &s.s_tau));
      s.s_heads = s.heads;
      s.s_dim = s.dim;
      s.s_vdim = s.vdim;
    } else if (ty == "attention") {
      s.mixer = B2_MIXER_MIXED_SCORE_ATTENTION;
      if (const Value* kh = m->find("kv_heads"))
        if (kh->is_number()) s.kv_heads = (int)kh->as_int();
      CFG_TRY(need_float(*m, "scale", where, &s.scale));
      if (const Value* cap = m->find("softcap"))
        if (cap->is_number()) s.softcap = (float)cap->as_double();
      s.score_mix = 1;
      s.rot_factor = 1.0f;
      const Value* rot = m->find("rot");
      if (rot && rot->is_object()) {  // no "rot": nothing is rotated, values included
        CFG_TRY(need_float(*rot, "base", where, &s.rot_base));
        CFG_TRY(need_int(*rot, "dims", where, &s.rot_dims));
        s.rot_values = 1;
        if (const Value* sc = rot->find("scaling"))
          if (sc->is_object()) CFG_TRY(need_float(*sc, "factor", where, &s.rot_factor));
      }
    } else if (ty == "latent_attention") {
      s.mixer = B2_MIXER_GATED_LATENT;
      CFG_TRY(need_int(*m, "kv_rank", where, &s.kv_rank));
      CFG_TRY(need_int(*m, "q_rank", where, &s.q_rank));
      CFG_TRY(need_float(*m, "scale", where, &s.scale));
      const Value* mask = m->find("mask");
      if (mask && mask->is_object()) CFG_TRY(need_int(*mask, "size", where, &s.window));  // no "mask": every earlier key is seen
    } else {
      b2_set_error("config.json: layers[%d]: mixer type '%s' not built (gla, attention, latent_attention)", i, ty.c_str());
      return -22;
    }
    const Value* mlp = L.find("mlp");
    s.ff = B2_FF_NONE;
    if (mlp && mlp->is_object()) {
      snprintf(where, sizeof where, "layers[%d].mlp", i);
      const Value* kind = mlp->find("kind");
      const std::string kd = kind && kind->is_string() ? kind->as_string() : "?";
      if (kd == "dense") {
        s.ff = B2_FF_XIELU;
        CFG_TRY(need_int(*mlp, "ff", where, &s.ff_dim));
      } else if (kd == "moe") {
        s.ff = B2_FF_TABLE_EXPERTS;
        const Value* ex = mlp->find("expert");
        const Value* ro = mlp->find("router");
        if (!ex || !ex->is_object() || !ro || !ro->is_object()) {
          b2_set_error("config.json: %s needs expert and router", where);
          return -22;
        }
        CFG_TRY(need_int(*ex, "ff", where, &s.ff_dim));
        CFG_TRY(need_float(*ex, "limit", where, &s.ff_limit));
        CFG_TRY(need_int(*ro, "experts", where, &s.experts));
        CFG_TRY(need_int(*ro, "top", where, &s.top));
        s.groups = s.groups_keep = 1;
      } else {
        b2_set_error("config.json: %s.kind '%s' not built (dense, moe)", where, kd.c_str());
        return -22;
      }
    }
  }
  c->layer_specs = specs;
  c->tie_embeddings = 1;
  c->num_q_heads = c->num_kv_heads = 0;
  c->head_dim = c->intermediate = 0;
  return 0;
}

}  // namespace

extern "C" int b2_config_from_dir(const char* model_dir, b2_config* c, b2_layer_spec* specs, int32_t max_specs) {
  B2_REQUIRE(model_dir && c, "b2_config_from_dir: null argument");
  const std::string path = std::string(model_dir) + "/config.json";
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    b2_set_error("cannot open %s", path.c_str());
    return -2;
  }
  std::stringstream ss;
  ss << f.rdbuf();
  Value j;
  try {
    j = b2json::parse(ss.str());
  } catch (const std::exception& ex) {
    b2_set_error("%s: %s", path.c_str(), ex.what());
    return -22;
  }
  c->abi_version = B2_ABI_VERSION;
  c->layer_specs = nullptr;
  c->logit_scale = 0.f;
  c->embed_scale = 0.f;
  c->norm_groups = 0;
  c->loop_start = c->loop_stop = c->loop_times = 0;
  c->logit_softcap = 0.f;
  c->norm_kind = 0;
  const Value* archv = j.find("architecture");
  if (archv && archv->is_string()) {
    if (archv->as_string() == "Lerasun") return lerasun_config(j, c, specs, max_specs);
    if (archv->as_string() == "Kedasun") return kedasun_config(j, c, specs, max_specs);
    if (archv->as_string() == "Bumalix") return bumalix_config(j, c, specs, max_specs);
    if (archv->as_string() == "Tinevik") return tinevik_config(j, c, specs, max_specs);
    b2_set_error("%s: architecture '%s' not built", path.c_str(), archv->as_string().c_str());
    return -22;
  }
  // ---- HF families ----
  auto geti = [&](const char* k, int d) { const Value* v = j.find(k); return v && v->is_number() ? (int)v->as_int() : d; };
  auto getf = [&](const char* k, double d) { const Value* v = j.find(k); return v && v->is_number() ? v->as_double() : d; };
  c->arch = B2_ARCH_QWEN3;
  c->num_layers = geti("num_hidden_layers", c->num_layers);
  c->hidden = geti("hidden_size", c->hidden);
  c->num_q_heads = geti("num_attention_heads", c->num_q_heads);
  c->num_kv_heads = geti("num_key_value_heads", c->num_kv_heads);
  c->head_dim = geti("head_dim", c->hidden / (c->num_q_heads > 0 ? c->num_q_heads : 1));
  c->intermediate = geti("intermediate_size", c->intermediate);
  c->vocab = geti("vocab_size", c->vocab);
  const Value* tie = j.find("tie_word_embeddings");
  if (tie && tie->is_bool()) c->tie_embeddings = tie->b ? 1 : 0;
  c->rms_eps = (float)getf("rms_norm_eps", c->rms_eps);
  double theta = getf("rope_theta", c->rope_theta);
  const Value* rp = j.find("rope_parameters");
  if (rp && rp->find("rope_theta")) theta = rp->find("rope_theta")->as_double(theta);
  c->rope_theta = (float)theta;
  const Value* mt = j.find("model_type");
  if (mt && mt->is_string() && mt->as_string() == "phi3") {
    c->arch = B2_ARCH_PHI3;
    c->rotary_dim = (int)(getf("partial_rotary_factor", 1.0) * c->head_dim + 0.5);
    c->sliding_window = geti("sliding_window", 0);  // null in the config parses as "not a number" -> 0
  } else if (mt && mt->is_string() && mt->as_string() == "opt") {
    // HF OPTConfig names: ffn_dim, no kv-head count (MHA), LayerNorm eps is torch's default
    c->arch = B2_ARCH_OPT;
    c->num_kv_heads = c->num_q_heads;
    c->head_dim = c->hidden / (c->num_q_heads > 0 ? c->num_q_heads : 1);
    c->intermediate = geti("ffn_dim", c->intermediate);
    c->max_positions = geti("max_position_embeddings", 2048);
    c->rms_eps = 1e-5f;
    c->tie_embeddings = 1;
  }
  return 0;
}
