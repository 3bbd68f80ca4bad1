"""Host-side checks for the Tinevik family: the registry reads a model directory's config.json into the C structs (and the Python
mirror fills the same bytes), and the plain restatement the GPU tests lean on is itself checked mechanism by mechanism on
hand-made cases (no GPU)."""
import ctypes as C
import json
import math

import torch

from oracle import tinevik_oracle as O

D = torch.float64


def small_cfg():
    g = {"heads": 3, "dim": 4, "vdim": 6, "tau": 8.0}
    a = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 4, "scale": 0.4, "softcap": 9.0, "rot": {"base": 500.0, "dims": 4, "scaling": {"factor": 2.0}}}
    l = {"heads": 2, "dim": 5, "vdim": 3, "kv_rank": 7, "q_rank": 6, "scale": 0.3, "mask": {"size": 5}}
    moe = {"kind": "moe", "expert": {"ff": 9, "limit": 1.25}, "router": {"experts": 5, "top": 2}}
    return {"architecture": "Tinevik", "vocab": 31, "width": 12, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5}, "logit_scale": 0.5, "layers": [
        {"type": "gla", "mixer": g, "mlp": {"kind": "dense", "ff": 14}},
        {"type": "attention", "mixer": a, "mlp": moe},
        {"type": "latent_attention", "mixer": l, "mlp": None},
        {"type": "attention", "mixer": a, "mlp": moe, "weights_of": 1}]}


def test_registry_reads_the_layer_list(pkg, lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    eng = import_module("aws-k8s-ansible-provisioner_b200.engine")
    cfg = small_cfg()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert (c.arch, c.num_layers, c.hidden, c.vocab, c.norm_kind, c.tie_embeddings) == (capi.ARCH_TINEVIK, 4, 12, 31, 1, 1)
    assert abs(c.embed_scale - 3.0) < 1e-6 and abs(c.rms_eps - 1e-5) < 1e-11 and abs(c.logit_scale - 0.5) < 1e-6
    s0, s1, s2, s3 = specs[0], specs[1], specs[2], specs[3]
    assert (s0.mixer, s0.heads, s0.dim, s0.vdim, s0.weights_of) == (capi.MIXER_DECAY_STATE, 3, 4, 6, -1) and abs(s0.s_tau - 8.0) < 1e-6
    assert (s0.ff, s0.ff_dim) == (capi.FF_XIELU, 14)
    assert (s1.mixer, s1.heads, s1.kv_heads, s1.dim, s1.vdim, s1.rot_dims, s1.rot_values, s1.score_mix) == (capi.MIXER_MIXED_SCORE_ATTENTION, 4, 2, 6, 4, 4, 1, 1)
    assert abs(s1.rot_base - 500.0) < 1e-3 and abs(s1.rot_factor - 2.0) < 1e-6 and abs(s1.softcap - 9.0) < 1e-6 and abs(s1.scale - 0.4) < 1e-6
    assert (s1.ff, s1.ff_dim, s1.experts, s1.top) == (capi.FF_TABLE_EXPERTS, 9, 5, 2) and abs(s1.ff_limit - 1.25) < 1e-6
    assert (s2.mixer, s2.heads, s2.dim, s2.vdim, s2.kv_rank, s2.q_rank, s2.window, s2.ff) == (capi.MIXER_GATED_LATENT, 2, 5, 3, 7, 6, 5, capi.FF_NONE)
    assert (s3.mixer, s3.weights_of) == (capi.MIXER_MIXED_SCORE_ATTENTION, 1)
    # the Python mirror fills the same bytes from the same dict, and reads them back into an equal layer list
    mine = (capi.b2_layer_spec * 4)()
    for sp, layer in zip(mine, cfg["layers"]):
        eng._fill_layer_spec(sp, dict(layer, _tinevik=True))
    assert bytes(mine) == bytes(specs)[:C.sizeof(mine)]
    back = [eng._layer_dict(specs[i]) for i in range(4)]
    again = (capi.b2_layer_spec * 4)()
    for sp, layer in zip(again, back):
        eng._fill_layer_spec(sp, layer)
    assert bytes(again) == bytes(mine)


def test_registry_optional_keys_and_refusals(pkg, lib, tmp_path):
    from importlib import import_module
    capi = import_module("aws-k8s-ansible-provisioner_b200.capi")
    c = capi.b2_config()
    specs = (capi.b2_layer_spec * 8)()
    cfg = small_cfg()
    del cfg["embedding"], cfg["logit_scale"]
    a = cfg["layers"][1]["mixer"]
    del a["kv_heads"], a["softcap"], a["rot"]["scaling"]
    del cfg["layers"][2]["mixer"]["mask"]
    cfg["layers"][3]["mixer"] = a
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert abs(c.embed_scale - 1.0) < 1e-6 and abs(c.logit_scale - 1.0) < 1e-6
    assert specs[1].kv_heads == 4 and specs[1].softcap == 0.0 and abs(specs[1].rot_factor - 1.0) < 1e-6 and specs[2].window == 0
    del a["rot"]      # nothing is rotated, values included
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) == 0, lib.b2_last_error()
    assert specs[1].rot_dims == 0 and specs[1].rot_values == 0
    cfg["layers"][0]["type"] = "gated"
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"gated" in lib.b2_last_error()
    cfg = small_cfg()
    cfg["layers"][3]["weights_of"] = 3
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 8) != 0 and b"weights_of" in lib.b2_last_error()
    assert lib.b2_config_from_dir(str(tmp_path).encode(), C.byref(c), specs, 2) != 0


def test_norms_and_activation_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=D)
    y = O.layer_norm(x, torch.tensor([1.0, 1.0, 2.0, 1.0], dtype=D), torch.tensor([0.0, 0.5, 0.0, 0.0], dtype=D), 0.0)
    sd = math.sqrt((4 + 1 + 0 + 9) / 4)
    assert torch.allclose(y, torch.tensor([[-2 / sd, -1 / sd + 0.5, 0.0, 3 / sd]], dtype=D))
    r = O.rms_norm(torch.tensor([3.0, 4.0], dtype=D), torch.tensor([2.0, 1.0], dtype=D), 0.0)
    assert torch.allclose(r, torch.tensor([6.0, 4.0], dtype=D) / math.sqrt(12.5))
    p, q = torch.tensor(0.3, dtype=D), torch.tensor(-0.7, dtype=D)
    z = torch.tensor([2.0, 0.0, -1.0], dtype=D)
    sp = lambda v: math.log1p(math.exp(v))
    want = [sp(0.3) * 4 + 1.0, 0.0, (0.5 + sp(-0.7)) * (math.exp(-1.0) - 1 + 1) - 0.5]
    assert torch.allclose(O.xielu(z, p, q), torch.tensor(want, dtype=D))


def test_clamped_expert_and_table_by_hand():
    w = {"e0.gate": torch.tensor([[1.0, 0.0]], dtype=D), "e0.up": torch.tensor([[0.0, 1.0]], dtype=D), "e0.down": torch.tensor([[2.0], [1.0]], dtype=D),
         "e1.gate": torch.tensor([[0.0, 1.0]], dtype=D), "e1.up": torch.tensor([[1.0, 0.0]], dtype=D), "e1.down": torch.tensor([[1.0], [0.0]], dtype=D),
         "table": torch.tensor([[0, 1], [1, 0], [0, 0]])}
    n = torch.tensor([3.0, -5.0], dtype=D)
    y0 = O.clamped_expert(n, w, "e0.", 2.0)      # g = min(3, 2) = 2, u = clamp(-5) = -2: 2 sigmoid(3.404) (-1)
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(y0, torch.tensor([-2 * g, -g], dtype=D))
    y1 = O.clamped_expert(n, w, "e1.", 2.0)      # g = -5 (no lower clamp), u = 2
    g1 = -5.0 / (1.0 + math.exp(1.702 * 5.0))
    assert torch.allclose(y1, torch.tensor([3 * g1, 0.0], dtype=D))
    mlp = {"expert": {"ff": 1, "limit": 2.0}, "router": {"experts": 2, "top": 2}}
    out = O.table_moe_ff(torch.stack([n, n]), [0, 1], w, "", mlp)     # both tokens name both experts: the mean, whatever the order
    assert torch.allclose(out[0], (y0 + y1) / 2) and torch.allclose(out[1], out[0])


def test_rotation_pairs_halves_and_turns_back():
    x = torch.arange(1.0, 9.0, dtype=D)[None, :]      # one position, 8 entries, the first 4 rotated: pairs (0, 2) and (1, 3)
    pos = torch.tensor([3])
    y = O.rotate_halves(x, pos, 4, 100.0, 2.0)
    a0, a1 = 3 * 1.0 / 2.0, 3 * 100.0 ** (-2.0 / 4) / 2.0
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0),
            4 * math.cos(a1) + 2 * math.sin(a1), 5, 6, 7, 8]
    assert torch.allclose(y, torch.tensor([want], dtype=D))
    assert torch.allclose(O.rotate_halves(y, -pos, 4, 100.0, 2.0), x)


def one_layer(layer, width=10, vocab=23):
    return {"architecture": "Tinevik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": [layer]}


def test_gla_is_its_recurrence_and_forgets_with_the_decay():
    torch.manual_seed(0)
    m = {"heads": 2, "dim": 3, "vdim": 4, "tau": 2.0}
    cfg = one_layer({"type": "gla", "mixer": m, "mlp": None})
    w = {k: v.to(D) for k, v in O.random_weights(cfg, seed=1).items()}
    h = torch.randn(6, 10, dtype=D)
    got = O.gla_mixer(h, w, "l0.mix.", m, 1e-6)
    # by hand for the last token: o = sum_j (prod_{j < t <= last} a_t) * (q . k_j) v_j
    q = (h @ w["l0.mix.q"].T).view(6, 2, 3) * 3 ** -0.5
    k = (h @ w["l0.mix.k"].T).view(6, 2, 3)
    v = (h @ w["l0.mix.v"].T).view(6, 2, 4)
    a = (torch.sigmoid((h @ w["l0.mix.a1"].T) @ w["l0.mix.a2"].T + w["l0.mix.a2.b"]) ** 0.5).view(6, 2, 3)
    o = torch.zeros(2, 4, dtype=D)
    for j in range(6):
        decay = torch.ones(2, 3, dtype=D)
        for t in range(j + 1, 6):
            decay = decay * a[t]
        o += ((q[5] * decay * k[j]).sum(-1))[:, None] * v[j]
    o = O.rms_norm(o, w["l0.mix.norm"], 1e-6).reshape(8)
    g = h[5] @ w["l0.mix.g"].T
    assert torch.allclose(got[5], (o * g * torch.sigmoid(g)) @ w["l0.mix.o"].T, atol=1e-10)


def test_attention_mixes_scores_before_the_softmax_and_is_causal():
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.5, "softcap": 3.0, "rot": {"base": 10.0, "dims": 2}}
    cfg = one_layer({"type": "attention", "mixer": m, "mlp": None})
    w = {k: v.to(D) for k, v in O.random_weights(cfg, seed=2).items()}
    torch.manual_seed(1)
    h = torch.randn(7, 10, dtype=D)
    full = O.attention_mixer(h, w, "l0.mix.", m, 1e-6)
    assert torch.allclose(O.attention_mixer(h[:4], w, "l0.mix.", m, 1e-6), full[:4], atol=1e-12)     # later tokens change nothing earlier
    # swapping the two rows of the mixing matrix swaps the heads' weights, hence (one key/value head) the heads' outputs
    w2 = dict(w)
    w2["l0.mix.talk"] = w["l0.mix.talk"].flip(0)
    w2["l0.mix.o"] = torch.cat([w["l0.mix.o"][:, 4:], w["l0.mix.o"][:, :4]], dim=1)
    assert torch.allclose(O.attention_mixer(h, w2, "l0.mix.", m, 1e-6), full, atol=1e-12)
    # a mixing matrix that is not the identity matters
    w3 = dict(w)
    w3["l0.mix.talk"] = torch.eye(2, dtype=D)
    assert (O.attention_mixer(h, w3, "l0.mix.", m, 1e-6) - full).abs().max() > 1e-4
    # relative positions only: the same tokens later in a sequence of copies give the same output for values AND keys
    m0 = dict(m)
    del m0["rot"]
    assert (O.attention_mixer(h, w, "l0.mix.", m0, 1e-6) - full).abs().max() > 1e-4


def test_latent_attention_sees_exactly_the_window():
    m = {"heads": 2, "dim": 3, "vdim": 2, "kv_rank": 5, "q_rank": 4, "scale": 0.6, "mask": {"size": 3}}
    cfg = one_layer({"type": "latent_attention", "mixer": m, "mlp": None})
    w = {k: v.to(D) for k, v in O.random_weights(cfg, seed=3).items()}
    torch.manual_seed(2)
    h = torch.randn(8, 10, dtype=D)
    full = O.latent_mixer(h, w, "l0.mix.", m, 1e-6)
    h2 = h.clone()
    h2[:5] = torch.randn(5, 10, dtype=D)          # tokens 0..4 lie outside the window of token 7 (it sees 5, 6, 7)
    assert torch.allclose(O.latent_mixer(h2, w, "l0.mix.", m, 1e-6)[7], full[7], atol=1e-12)
    h2 = h.clone()
    h2[5] = torch.randn(10, dtype=D)              # token 5 lies just inside
    assert (O.latent_mixer(h2, w, "l0.mix.", m, 1e-6)[7] - full[7]).abs().max() > 1e-5
    m1 = dict(m, mask={"size": 1})                # itself only: the value of its own latent, gated
    one = O.latent_mixer(h, w, "l0.mix.", m1, 1e-6)
    c = O.rms_norm(h @ w["l0.mix.dkv"].T, w["l0.mix.dkv.norm"], 1e-6)
    want = ((c @ w["l0.mix.uv"].T) * torch.sigmoid(h @ w["l0.mix.g"].T)) @ w["l0.mix.o"].T
    assert torch.allclose(one, want, atol=1e-12)


def test_whole_model_shapes_and_borrowed_tensors():
    cfg = small_cfg()
    w = O.random_weights(cfg, seed=5)
    toks = [3, 30, 7, 7, 1, 12, 25, 0, 9, 18, 4]
    logits, streams = O.forward(cfg, w, toks)
    assert streams.shape == (4, len(toks), 12) and logits.shape == (len(toks), 31) and torch.isfinite(logits).all()
    names = set(O.tensor_shapes(cfg))
    assert {"l0.mix.a2.b", "l0.mlp.act", "l1.mix.talk", "l1.mlp.table", "l1.mlp.e4.gate", "l2.mix.dq.norm", "final.norm.b"} <= names
    assert not any(n.startswith(("l3.", "l2.mlp", "head")) for n in names)
    short, _ = O.forward(cfg, w, toks[:6])
    assert torch.allclose(short, logits[:6], atol=1e-5)          # causal throughout
    assert O.greedy(cfg, w, toks[:4], 3)[0] == int(torch.argmax(O.forward(cfg, w, toks[:4])[0][-1]))
