"""Host-side checks for the Bumalix family: the registry reads a model directory's config.json into the C structs, and the
plain restatement the GPU tests lean on is itself checked mechanism by mechanism on hand-made cases (no GPU)."""
import ctypes as C
import json
import math

import torch

from oracle import bumalix_oracle as O


def small_cfg():
    left = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "mask": {"size": 5}}
    right = {"heads": 3, "dim": 4, "vdim": 7, "tau": 8.0}
    d = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "conv": 3}
    return {"architecture": "Bumalix", "vocab": 31, "width": 12, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "logit_softcap": 7.5,
            "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
                {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": 14}},
                {"type": "channel_delta", "mixer": d, "mlp": {"kind": "moe", "expert": {"ff": 9}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 11}}},
                {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None}]}


def test_registry_reads_the_layer_list(pkg, lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    eng = import_module("aws-k8s-ansible-provisioner_b200.engine")
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (c.arch, c.num_layers, c.hidden, c.vocab) == (capi.ARCH_BUMALIX, 3, 12, 31)
    assert (c.loop_start, c.loop_stop, c.loop_times) == (1, 3, 2)
    assert abs(c.embed_scale - 3.0) < 1e-6 and abs(c.rms_eps - 1e-5) < 1e-11 and abs(c.logit_softcap - 7.5) < 1e-6
    s0, s1, s2 = specs[0], specs[1], specs[2]
    assert (s0.mixer, s0.heads, s0.kv_heads, s0.dim, s0.vdim, s0.window) == (capi.MIXER_WINDOW_AND_STATE, 4, 2, 6, 5, 5)
    assert (s0.s_heads, s0.s_dim, s0.s_vdim) == (3, 4, 7) and abs(s0.s_tau - 8.0) < 1e-6 and abs(s0.scale - 0.4) < 1e-6
    assert (s0.ff, s0.ff_dim) == (capi.FF_POLYNORM, 14)
    assert (s1.mixer, s1.heads, s1.kv_heads, s1.dim, s1.vdim, s1.conv_taps) == (capi.MIXER_DELTA_STATE, 4, 2, 6, 5, 3)
    assert (s1.ff, s1.ff_dim, s1.experts, s1.top, s1.shared_ff) == (capi.FF_SCALED_GATED_EXPERTS, 9, 5, 2, 11)
    assert s2.ff == capi.FF_NONE
    for i, layer in enumerate(cfg["layers"]):   # the Python mirror fills the same bytes, and reads them back
        sp = capi.b2_layer_spec()
        eng._fill_layer_spec(sp, layer)
        assert bytes(sp) == bytes(specs[i])
        back = eng._layer_dict(sp)
        assert back["type"] == layer["type"] and back["mlp"] == layer["mlp"]
    ec = eng.EngineConfig.bumalix(cfg, max_model_len=64)
    assert ec.loop == (1, 3, 2) and ec.logit_softcap == 7.5 and ec.arch == "bumalix"
    plain = small_cfg()     # no "kv_heads": as many as query heads; no "mask": no window; no loop, no cap, no shared expert
    del plain["layers"][1]["mixer"]["kv_heads"], plain["loop"], plain["logit_softcap"], plain["layers"][1]["mlp"]["shared"]
    plain["layers"][0]["mixer"]["left"] = {"heads": 4, "dim": 6, "vdim": 5, "scale": 0.4}
    (tmp_path / "config.json").write_text(json.dumps(plain))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (specs[0].kv_heads, specs[0].window, specs[1].kv_heads, specs[1].shared_ff) == (4, 0, 4, 0)
    assert (c.loop_times, c.logit_softcap) == (0, 0.0)
    sp = capi.b2_layer_spec()
    eng._fill_layer_spec(sp, plain["layers"][0])
    assert bytes(sp) == bytes(specs[0])
    bad = small_cfg()
    bad["layers"][1]["mlp"] = {"kind": "gated"}
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"gated" in lib.b2_last_error()
    bad = small_cfg()
    bad["layers"][0]["type"] = "attention"
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0
    bad = small_cfg()
    bad["loop"]["stop"] = 4
    (tmp_path / "config.json").write_text(json.dumps(bad))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"loop" in lib.b2_last_error()


def test_layer_runs_follow_the_loop():
    cfg = small_cfg()
    assert O.layer_runs(cfg) == [(0, False), (1, True), (2, False), (1, True), (2, False)]
    del cfg["loop"]
    assert O.layer_runs(cfg) == [(0, False), (1, False), (2, False)]
    cfg["loop"] = {"start": 0, "stop": 1, "times": 3}
    assert O.layer_runs(cfg) == [(0, True), (0, True), (0, True), (1, False), (2, False)]


def test_poly_norm_by_hand():
    z = torch.tensor([1.0, -2.0, 3.0, 0.5], dtype=torch.float64)
    coef = torch.tensor([0.5, -1.0, 2.0, 0.25], dtype=torch.float64)
    want = []
    for i in range(4):
        t = 0.25
        for p, c in ((1, 0.5), (2, -1.0), (3, 2.0)):
            rms = math.sqrt(sum(float(v) ** (2 * p) for v in z) / 4 + 1e-6)
            t += c * float(z[i]) ** p / rms
        want.append(t)
    assert torch.allclose(O.poly_norm(z, coef, 1e-6), torch.tensor(want, dtype=torch.float64), atol=1e-12)


def test_window_attention_sees_exactly_the_window():
    torch.manual_seed(0)
    keys, vals = torch.randn(9, 4, dtype=torch.float64), torch.randn(9, 3, dtype=torch.float64)
    q = torch.randn(8, dtype=torch.float64)     # two query heads over one key/value head
    full = O.window_attention_step(q, keys, vals, 2, 1, 4, 3, 0.7, None)
    win4 = O.window_attention_step(q, keys, vals, 2, 1, 4, 3, 0.7, 4)
    only = O.window_attention_step(q, keys[5:], vals[5:], 2, 1, 4, 3, 0.7, None)
    assert torch.allclose(win4, only, atol=1e-12) and (full - win4).abs().max() > 1e-3
    one = O.window_attention_step(q, keys, vals, 2, 1, 4, 3, 0.7, 1)     # itself only: the value row, for both heads
    assert torch.allclose(one, torch.cat([vals[8], vals[8]]), atol=1e-12)


def test_state_rules_by_hand():
    S = torch.tensor([[1.0, 2.0], [3.0, 4.0], [0.0, -1.0]], dtype=torch.float64)      # dim 3, vdim 2
    q = torch.tensor([1.0, 0.0, 2.0], dtype=torch.float64)
    k = torch.tensor([0.5, -1.0, 0.0], dtype=torch.float64)
    v = torch.tensor([2.0, 1.0], dtype=torch.float64)
    a = torch.tensor([0.5, 1.0, 0.0], dtype=torch.float64)
    S1, o = O.gla_step(S, q, k, v, a)
    assert torch.allclose(S1, torch.tensor([[1.5, 1.5], [1.0, 3.0], [0.0, 0.0]], dtype=torch.float64))
    assert torch.allclose(o, torch.tensor([1.5, 1.5], dtype=torch.float64))
    # delta rule: decay, then the write moves S^T k toward v by beta; with beta 1 and a unit key the read-out along k is v itself
    kk = torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64)
    S2, o2 = O.delta_step(S, kk, kk, v, a, torch.tensor(1.0, dtype=torch.float64))
    assert torch.allclose(o2, v) and torch.allclose(S2[0], a[0] * S[0]) and torch.allclose(S2[2], a[2] * S[2])
    S3, _ = O.delta_step(S, q, kk, v, a, torch.tensor(0.0, dtype=torch.float64))       # beta 0: only the decay acts
    assert torch.allclose(S3, a[:, None] * S)


def test_router_takes_the_largest_scores_unnormalised():
    router = torch.tensor([[1.0, 0.0], [0.0, 1.0], [1.0, 1.0], [-1.0, 0.0]], dtype=torch.float64)
    idx, sc = O.route(torch.tensor([2.0, 1.0], dtype=torch.float64), router, 2)
    assert idx == [2, 0] and abs(float(sc[0]) - 1 / (1 + math.exp(-3.0))) < 1e-12 and abs(float(sc[1]) - 1 / (1 + math.exp(-2.0))) < 1e-12
    idx, _ = O.route(torch.zeros(2, dtype=torch.float64), router, 3)     # ties: lowest index first
    assert idx == [0, 1, 2]


def test_whole_sequence_equals_token_by_token_state():
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=5)
    toks = [3, 30, 7, 7, 1, 12, 25, 0, 9, 18, 4]
    logits, streams = O.forward(cfg, w, toks)
    assert streams.shape == (5, len(toks), 12) and torch.isfinite(logits).all()
    assert float(logits.abs().max()) < 7.5          # the cap
    s = O.Stepper(cfg, w)
    for i, t in enumerate(toks):
        assert torch.allclose(s.step(t), logits[i], atol=1e-12)
    # the loop's passes keep states of their own: the same layer's two runs differ
    assert (streams[1] - streams[3]).abs().max() > 1e-3
    names = set(O.tensor_shapes(cfg))
    assert {"loop.in", "l0.mix.left.q.b", "l0.mix.right.a2.b", "l1.mix.dt_bias", "l1.mlp.e4.gate", "l1.mlp.shared.down", "l0.mlp.act"} <= names
    assert not any(n.startswith("l2.mlp") for n in names)
