"""Synthetic checkpoints for the benchmark and the server: there is no network for HF downloads
(the reference pulls Qwen/Qwen3-0.6B with an HF token, llm-d-deploy.yaml:121-132,184), so weights
are random-init bf16 with HF's default init statistics (N(0, 0.02) for Linear/Embedding, ones for
norms), under HF's tensor names."""
from __future__ import annotations

import json
import struct

import torch

from .engine import EngineConfig


def tensor_shapes(cfg: EngineConfig) -> dict[str, tuple[int, ...]]:
    q, kv = cfg.num_q_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    s: dict[str, tuple[int, ...]] = {"model.embed_tokens.weight": (cfg.vocab, cfg.hidden)}
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (cfg.hidden,)
        s[p + "self_attn.q_proj.weight"] = (q, cfg.hidden)
        s[p + "self_attn.k_proj.weight"] = (kv, cfg.hidden)
        s[p + "self_attn.v_proj.weight"] = (kv, cfg.hidden)
        s[p + "self_attn.o_proj.weight"] = (cfg.hidden, q)
        s[p + "self_attn.q_norm.weight"] = (cfg.head_dim,)
        s[p + "self_attn.k_norm.weight"] = (cfg.head_dim,)
        s[p + "post_attention_layernorm.weight"] = (cfg.hidden,)
        s[p + "mlp.gate_proj.weight"] = (cfg.intermediate, cfg.hidden)
        s[p + "mlp.up_proj.weight"] = (cfg.intermediate, cfg.hidden)
        s[p + "mlp.down_proj.weight"] = (cfg.hidden, cfg.intermediate)
    s["model.norm.weight"] = (cfg.hidden,)
    if not cfg.tie_embeddings:
        s["lm_head.weight"] = (cfg.vocab, cfg.hidden)
    return s


def random_state_dict(cfg: EngineConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(cfg).items():
        if "norm" in name:
            sd[name] = torch.ones(shape, dtype=torch.bfloat16)
        else:
            sd[name] = (torch.randn(shape, generator=g, dtype=torch.float32) * std).to(torch.bfloat16)
    return sd


def write_safetensors(sd: dict[str, torch.Tensor], path: str) -> None:
    """Minimal safetensors writer so the C++ server can mmap a synthetic checkpoint: every tensor is stored in its
    own dtype (bf16, fp16, fp32 or int32 -- the ones the engine's loader reads)."""
    names = {torch.bfloat16: "BF16", torch.float16: "F16", torch.float32: "F32", torch.int32: "I32"}
    header = {}
    off = 0
    for name, t in sd.items():
        n = t.numel() * t.element_size()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in sd.values():
            t = t.contiguous()
            f.write(t.view(torch.int16 if t.element_size() == 2 else torch.int32).numpy().tobytes())


def lerasun_tensor_shapes(model_cfg: dict) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a Lerasun checkpoint for the dict its config.json holds."""
    W, V = model_cfg["width"], model_cfg["vocab"]
    s: dict[str, tuple[int, ...]] = {"embed": (V, W), "embed.norm": (W,)}
    for i, layer in enumerate(model_cfg["layers"]):
        m, mlp, p = layer["mixer"], layer.get("mlp"), f"l{i}."
        H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        s[p + "norm1"] = (W,)
        s[p + "mix.q"] = (H * (dn + dr), W)
        if m.get("kv_from") is None:
            s[p + "mix.dkv"] = (r + dr, W)
            s[p + "mix.dkv.norm"] = (r,)
        s[p + "mix.uk"] = (H * dn, r)
        s[p + "mix.uv"] = (H * dv, r)
        s[p + "mix.sink"] = (H,)
        s[p + "mix.o"] = (W, H * dv)
        if mlp is not None:
            s[p + "norm2"] = (W,)
            for e in range(mlp["router"]["experts"]):
                s[p + f"mlp.e{e}.up"] = (mlp["expert"]["ff"], W)
                s[p + f"mlp.e{e}.down"] = (W, mlp["expert"]["ff"])
            s[p + "mlp.router"] = (mlp["router"]["experts"], W)
            s[p + "mlp.correction"] = (mlp["router"]["experts"],)
    s["final.norm"] = (W,)
    s["head"] = (V, W)
    return s


def lerasun_random_state_dict(model_cfg: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    """Random bf16 weights scaled by 1/sqrt(fan-in) (gains and offsets small), so activations stay O(1) at any depth."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in lerasun_tensor_shapes(model_cfg).items():
        if name.endswith("dkv.norm"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif "norm" in name or name.endswith(("sink", "correction")):
            t = 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (shape[-1] ** -0.5)
        sd[name] = t.to(torch.bfloat16)
    return sd


def kedasun_tensor_shapes(model_cfg: dict) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a Kedasun checkpoint for the dict its config.json holds."""
    W, V = model_cfg["width"], model_cfg["vocab"]
    s: dict[str, tuple[int, ...]] = {"embed": (V, W)}
    for i, layer in enumerate(model_cfg["layers"]):
        m, mlp, p = layer["mixer"], layer.get("mlp"), f"l{i}."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"], s[p + "norm1b"] = (W,), (W,)
        s[p + "mix.q"], s[p + "mix.k"], s[p + "mix.v"] = (H * D, W), (G * D, W), (G * Dv, W)
        s[p + "mix.vmix"], s[p + "mix.o"] = (), (W, H * Dv)
        if layer["type"] == "attention_2":
            for n, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                s[p + f"mix.{n}.b"], s[p + f"mix.{n}.conv"] = (c,), (c, m["conv"])
            s[p + "mix.talk"], s[p + "mix.g"], s[p + "mix.o.b"] = (H, H), (H, W), (W,)
        if mlp is not None:
            s[p + "norm2"], s[p + "norm2b"] = (W,), (W,)
            s[p + "mlp.gate"], s[p + "mlp.up"], s[p + "mlp.down"] = (mlp["ff"], W), (mlp["ff"], W), (W, mlp["ff"])
    s["final.norm"] = (W,)
    s["head"] = (V, W)
    return s


def kedasun_random_state_dict(model_cfg: dict, seed: int = 0) -> dict[str, torch.Tensor]:
    """Random bf16 weights scaled by 1/sqrt(fan-in), gains around one, a near-identity weight-mixing matrix."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in kedasun_tensor_shapes(model_cfg).items():
        if "norm" in name:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("vmix"):
            t = torch.rand(shape, generator=g)
        elif name.endswith("talk"):
            t = torch.eye(shape[0]) + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (shape[-1] ** -0.5)
        sd[name] = t.to(torch.bfloat16)
    return sd


def bumalix_tensor_shapes(model_cfg: dict, rank_a: int = 32, rank_g: int = 32) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a Bumalix checkpoint for the dict its config.json holds.  The widths of the low-rank first stages
    (a1, g1) are not in the config -- a checkpoint's tensors carry them -- so they are arguments here."""
    W, V = model_cfg["width"], model_cfg["vocab"]
    s: dict[str, tuple[int, ...]] = {"embed": (V, W)}
    if model_cfg.get("loop"):
        s["loop.in"] = (W, 2 * W)
    for i, layer in enumerate(model_cfg["layers"]):
        m, mlp, p = layer["mixer"], layer.get("mlp"), f"l{i}."
        s[p + "norm1"] = (W,)
        if layer["type"] == "parallel":
            a, b, q = m["left"], m["right"], p + "mix.left."
            H, G, D, Dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"]
            for n, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                s[q + n], s[q + n + ".b"] = (c, W), (c,)
            s[q + "q.norm"], s[q + "k.norm"], s[q + "o"], s[q + "out"] = (H * D,), (G * D,), (W, H * Dv), (W,)
            H, D, Dv, q = b["heads"], b["dim"], b["vdim"], p + "mix.right."
            s[q + "q"], s[q + "k"], s[q + "v"], s[q + "g"], s[q + "o"] = (H * D, W), (H * D, W), (H * Dv, W), (H * Dv, W), (W, H * Dv)
            s[q + "norm"], s[q + "a1"], s[q + "a2"], s[q + "a2.b"], s[q + "out"] = (Dv,), (rank_a, W), (H * D, rank_a), (H * D,), (W,)
        else:
            H, G, D, Dv, q = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], p + "mix."
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                s[q + n], s[q + n + ".conv"] = (c, W), (c, m["conv"])
            s[q + "b"], s[q + "A_log"], s[q + "norm"], s[q + "o"] = (H, W), (H,), (Dv,), (W, H * Dv)
            s[q + "a1"], s[q + "a2"], s[q + "dt_bias"], s[q + "g1"], s[q + "g2"] = (rank_a, W), (H * D, rank_a), (H * D,), (rank_g, W), (H * Dv, rank_g)
        if mlp is not None and mlp["kind"] == "dense":
            s[p + "mlp.up"], s[p + "mlp.down"], s[p + "mlp.act"] = (mlp["ff"], W), (W, mlp["ff"]), (4,)
        elif mlp is not None:
            F = mlp["expert"]["ff"]
            s[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                s[p + f"mlp.e{e}.gate"], s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (F, W), (F, W), (W, F)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                s[p + "mlp.shared.gate"], s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (Fs, W), (Fs, W), (W, Fs)
    s["final.norm"] = (W,)
    s["head"] = (V, W)
    return s


def bumalix_random_state_dict(model_cfg: dict, seed: int = 0, rank_a: int = 32, rank_g: int = 32) -> dict[str, torch.Tensor]:
    """Random bf16 weights scaled by 1/sqrt(fan-in), gains around one, decays that forget over tens to hundreds of tokens."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in bumalix_tensor_shapes(model_cfg, rank_a, rank_g).items():
        last = name.rsplit(".", 1)[-1]
        if "norm" in name or last == "out":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.tensor([0.6, 0.3, 0.2, 0.0])
        elif last == "A_log":
            t = torch.log(0.5 + 2.0 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = torch.randn(shape, generator=g) - 3.0
        elif name.endswith("a2.b"):
            t = torch.randn(shape, generator=g) + 3.0
        elif last == "b" and len(shape) == 1:
            t = 0.1 * torch.randn(shape, generator=g)
        elif last == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = 0.5 * torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * (shape[-1] ** -0.5)
        sd[name] = t.to(torch.bfloat16)
    return sd


def tinevik_tensor_shapes(model_cfg: dict, rank_a: int = 16) -> dict[str, tuple[int, ...]]:
    """Tensor names and shapes of a Tinevik checkpoint for the dict its config.json holds.  A layer with "weights_of" has no tensors.  The
    width of the decay's low-rank first stage (a1) is not in the config -- a checkpoint's tensors carry it -- so it is an argument here."""
    W, V = model_cfg["width"], model_cfg["vocab"]
    s: dict[str, tuple[int, ...]] = {"embed": (V, W)}
    for i, layer in enumerate(model_cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, mlp, p = layer["mixer"], layer.get("mlp"), f"l{i}."
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if mlp is not None else ()):
            s[p + n], s[p + n + ".b"] = (W,), (W,)
        q = p + "mix."
        if layer["type"] == "gla":
            s[q + "q"], s[q + "k"], s[q + "v"], s[q + "g"], s[q + "o"] = (H * D, W), (H * D, W), (H * Dv, W), (H * Dv, W), (W, H * Dv)
            s[q + "norm"], s[q + "a1"], s[q + "a2"], s[q + "a2.b"] = (Dv,), (rank_a, W), (H * D, rank_a), (H * D,)
        elif layer["type"] == "attention":
            G = m.get("kv_heads", H)
            s[q + "q"], s[q + "k"], s[q + "v"], s[q + "o"] = (H * D, W), (G * D, W), (G * Dv, W), (W, H * Dv)
            s[q + "q.norm"], s[q + "k.norm"], s[q + "talk"] = (D,), (D,), (H, H)
        else:
            R, Q = m["kv_rank"], m["q_rank"]
            s[q + "dq"], s[q + "dq.norm"], s[q + "uq"] = (Q, W), (Q,), (H * D, Q)
            s[q + "dkv"], s[q + "dkv.norm"], s[q + "uk"], s[q + "uv"] = (R, W), (R,), (H * D, R), (H * Dv, R)
            s[q + "g"], s[q + "o"] = (H * Dv, W), (W, H * Dv)
        if mlp is not None and mlp["kind"] == "dense":
            s[p + "mlp.up"], s[p + "mlp.down"], s[p + "mlp.act"] = (mlp["ff"], W), (W, mlp["ff"]), (2,)
        elif mlp is not None:
            F = mlp["expert"]["ff"]
            s[p + "mlp.table"] = (V, mlp["router"]["top"])
            for e in range(mlp["router"]["experts"]):
                s[p + f"mlp.e{e}.gate"], s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (F, W), (F, W), (W, F)
    s["final.norm"], s["final.norm.b"] = (W,), (W,)
    return s


def tinevik_random_state_dict(model_cfg: dict, seed: int = 0, rank_a: int = 16) -> dict[str, torch.Tensor]:
    """Random bf16 weights scaled by 1/sqrt(fan-in), gains around one, small biases, decays that forget over tens to hundreds of tokens, a
    near-identity score-mixing matrix; the experts' table (int32) gives every token id `top` different experts."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tinevik_tensor_shapes(model_cfg, rank_a).items():
        last = name.rsplit(".", 1)[-1]
        if last == "table":
            i = int(name[1:name.index(".")])
            n_exp = model_cfg["layers"][i]["mlp"]["router"]["experts"]
            sd[name] = torch.stack([torch.randperm(n_exp, generator=g)[:shape[1]] for _ in range(shape[0])]).to(torch.int32)
            continue
        if name.endswith("a2.b"):
            t = torch.randn(shape, generator=g) + 3.0
        elif last == "b":
            t = 0.1 * torch.randn(shape, generator=g)
        elif "norm" in name:
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.tensor([0.3, -0.2])
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.2 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) * (shape[-1] ** -0.5)
        else:
            t = torch.randn(shape, generator=g) * (shape[-1] ** -0.5)
        sd[name] = t.to(torch.bfloat16)
    return sd


def write_model_dir(model_cfg: dict, sd: dict[str, torch.Tensor], path: str) -> str:
    """config.json + model.safetensors of a layer-list model, as the registry and the loader read them."""
    import os

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(model_cfg, f)
    write_safetensors(sd, os.path.join(path, "model.safetensors"))
    return path
