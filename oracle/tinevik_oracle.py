"""Plain, slow restatement of the Tinevik decoder, one function per mechanism, for the tests.

Tinevik is a decoder-only model given as a list of layers.  The embedding row is multiplied by a constant.  Every
norm of the stream is a layer norm with gain and bias, one in front of and one behind each sublayer:

    x <- x + ln1b(mixer(ln1(x)));   x <- x + ln2b(ff(ln2(x)))      (the second line only when the layer has a feed-forward)

A layer may name another layer whose tensors it uses (`weights_of`); its cache / state are its own.  The logits are
`embed . ln_final(x) * logit_scale` with the embedding table itself (unscaled) as the head.

Mixers (h is the mixer's input):

* "gla": gated linear attention.  Per head a matrix state S [dim, vdim], zero at the start of a sequence:
      S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
  a_t = sigmoid(A2 (A1 h_t) + b)^(1 / tau) per key channel, q scaled by dim^(-1/2).  o is RMS-normed per head with a gain
  shared by the heads, multiplied by silu(G h_t) and projected.
* "attention": grouped-query softmax attention.  q and k heads are RMS-normed with one gain of `dim` entries each,
  then the first `rot.dims` entries of every q and k head are rotated by the position, entry i paired with entry
  i + dims/2, angle p * base^(-2i/dims) / factor.  The VALUE of position j is rotated by j over all of vdim (entry m with
  m + vdim/2, angle j * base^(-2m/vdim), no factor) and cached so; the weighted sum of a query at position i is turned
  back by -i.  Scores: (q . k) * scale, then cap * tanh(score / cap), then mixed over the heads, s'_a = sum_b T[a, b] s_b,
  then the causal softmax.
* "latent_attention": q = U_q rms(D_q h), a latent c = rms(D_kv h) per token (the only thing a cache needs), k = U_k c and
  v = U_v c per head, no positions, scores (q . k) * scale, a sliding window (query i sees key j when 0 <= i - j < size),
  softmax, the concatenated heads multiplied by sigmoid(G h), projected.

Feed-forwards:

* "dense": W_down xielu(W_up n), xielu(z) = softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
  otherwise, (p, q) the layer's two activation numbers.
* "moe": a table row per token id names the token's `top` experts, each weighted 1 / top.  An expert is
  W_down (g sigmoid(1.702 g) (u + 1)) with g = min(W_gate n, limit), u = clamp(W_up n, -limit, limit).

Nothing here shares code with the engine.  Tensors go in as a dict of torch tensors under the checkpoint's names
(fp32 or fp64; the integer tables as int64).  `forward` runs one whole sequence and returns the logits of every position
and the stream behind every layer.
"""
from __future__ import annotations

import math

import torch

GATE_SHARP = 1.702


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def xielu(z, p, q):
    sp = torch.nn.functional.softplus
    pos = sp(p) * z * z + z / 2
    neg = (0.5 + sp(q)) * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + z / 2
    return torch.where(z > 0, pos, neg)


def dense_ff(n, w, pre):
    a = w[pre + "act"]
    return xielu(n @ w[pre + "up"].T, a[0], a[1]) @ w[pre + "down"].T


def clamped_expert(n, w, pre, limit):
    g = torch.clamp(n @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(n @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(GATE_SHARP * g) * (u + 1)) @ w[pre + "down"].T


def table_moe_ff(n, tokens, w, pre, mlp):
    """n [T, W], tokens [T] -> the mean of the outputs of the experts the table names for each token id."""
    top = mlp["router"]["top"]
    limit = float(mlp["expert"]["limit"])
    out = torch.zeros_like(n)
    for t in range(n.shape[0]):
        row = w[pre + "table"][int(tokens[t])]
        for j in range(top):
            out[t] += clamped_expert(n[t], w, pre + "e%d." % int(row[j]), limit) / top
    return out


def rotate_halves(x, pos, n, base, factor=1.0):
    """x [..., T, d]: the first n entries turned by the position, entry i paired with entry i + n/2."""
    if n == 0:
        return x
    half = n // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (float(base) ** (-2.0 * i / n)) / factor
    ang = pos.to(torch.float64)[:, None] * freq[None, :]
    c, s = torch.cos(ang).to(x.dtype), torch.sin(ang).to(x.dtype)
    u, v = x[..., :half], x[..., half:n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., n:]], dim=-1)


def gla_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    a = (torch.sigmoid(z) ** (1.0 / tau)).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w[pre + "norm"], eps).reshape(T, H * dv)
    g = h @ w[pre + "g"].T
    return (o * g * torch.sigmoid(g)) @ w[pre + "o"].T


def attention_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    rot = m.get("rot")
    pos = torch.arange(T)
    q = rms_norm((h @ w[pre + "q"].T).view(T, H, d), w[pre + "q.norm"], eps).transpose(0, 1)   # [H, T, d]
    k = rms_norm((h @ w[pre + "k"].T).view(T, G, d), w[pre + "k.norm"], eps).transpose(0, 1)
    v = (h @ w[pre + "v"].T).view(T, G, dv).transpose(0, 1)
    if rot is not None:
        factor = float(rot.get("scaling", {}).get("factor", 1.0)) if rot.get("scaling") else 1.0
        q = rotate_halves(q, pos, rot["dims"], rot["base"], factor)
        k = rotate_halves(k, pos, rot["dims"], rot["base"], factor)
        v = rotate_halves(v, pos, dv, rot["base"])
    rep = H // G
    s = torch.stack([q[a] @ k[a // rep].T for a in range(H)]) * float(m["scale"])             # [H, T, T]
    cap = m.get("softcap")
    if cap:
        s = float(cap) * torch.tanh(s / float(cap))
    if pre + "talk" in w:
        s = torch.einsum("ab,bij->aij", w[pre + "talk"], s)
    vis = pos[:, None] >= pos[None, :]
    s = s.masked_fill(~vis, float("-inf"))
    p = torch.softmax(s, dim=-1)
    o = torch.stack([p[a] @ v[a // rep] for a in range(H)])                                   # [H, T, dv]
    if rot is not None:
        o = rotate_halves(o, -pos, dv, rot["base"])
    return o.transpose(0, 1).reshape(T, H * dv) @ w[pre + "o"].T


def latent_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ w[pre + "dq"].T, w[pre + "dq.norm"], eps)
    q = (cq @ w[pre + "uq"].T).view(T, H, d).transpose(0, 1)
    c = rms_norm(h @ w[pre + "dkv"].T, w[pre + "dkv.norm"], eps)
    k = (c @ w[pre + "uk"].T).view(T, H, d).transpose(0, 1)
    v = (c @ w[pre + "uv"].T).view(T, H, dv).transpose(0, 1)
    s = q @ k.transpose(1, 2) * float(m["scale"])
    pos = torch.arange(T)
    dist = pos[:, None] - pos[None, :]
    vis = dist >= 0
    if m.get("mask"):
        vis = vis & (dist < int(m["mask"]["size"]))
    p = torch.softmax(s.masked_fill(~vis, float("-inf")), dim=-1)
    o = (p @ v).transpose(0, 1).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ w[pre + "g"].T)) @ w[pre + "o"].T


MIXERS = {"gla": gla_mixer, "attention": attention_mixer, "latent_attention": latent_mixer}


def forward(cfg, w, tokens):
    """tokens: list of ints -> (logits [T, vocab], stream behind every layer [layers, T, W])."""
    eps = float(cfg["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x = w["embed"][tok] * float(cfg.get("embedding", {}).get("scale", 1.0))
    streams = []
    for i, L in enumerate(cfg["layers"]):
        j = i
        while cfg["layers"][j].get("weights_of") is not None:    # a named layer may itself name another: the tensors are the last one's
            j = int(cfg["layers"][j]["weights_of"])
        p = "l%d." % j
        ln = lambda name, y: layer_norm(y, w[p + name], w[p + name + ".b"], eps)
        x = x + ln("norm1b", MIXERS[L["type"]](ln("norm1", x), w, p + "mix.", L["mixer"], eps))
        mlp = L.get("mlp")
        if mlp:
            n = ln("norm2", x)
            y = dense_ff(n, w, p + "mlp.") if mlp["kind"] == "dense" else table_moe_ff(n, tok, w, p + "mlp.", mlp)
            x = x + ln("norm2b", y)
        streams.append(x)
    n = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return n @ w["embed"].T * float(cfg.get("logit_scale", 1.0)), torch.stack(streams)


def tensor_shapes(cfg):
    """Names and shapes of the tensors a model of this design holds; the low-rank width of a gla mixer is the test-only key "rank" (4)."""
    W, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        m, mlp, p = L["mixer"], L.get("mlp"), "l%d." % i
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        for n in ["norm1", "norm1b"] + (["norm2", "norm2b"] if mlp else []):
            s[p + n] = s[p + n + ".b"] = (W,)
        q = p + "mix."
        if L["type"] == "gla":
            r = m.get("rank", 4)
            s.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * dv, W), q + "g": (H * dv, W), q + "o": (W, H * dv),
                      q + "norm": (dv,), q + "a1": (r, W), q + "a2": (H * d, r), q + "a2.b": (H * d,)})
        elif L["type"] == "attention":
            G = m.get("kv_heads", H)
            s.update({q + "q": (H * d, W), q + "k": (G * d, W), q + "v": (G * dv, W), q + "o": (W, H * dv), q + "q.norm": (d,),
                      q + "k.norm": (d,), q + "talk": (H, H)})
        else:
            R, Q = m["kv_rank"], m["q_rank"]
            s.update({q + "dq": (Q, W), q + "dq.norm": (Q,), q + "uq": (H * d, Q), q + "dkv": (R, W), q + "dkv.norm": (R,),
                      q + "uk": (H * d, R), q + "uv": (H * dv, R), q + "g": (H * dv, W), q + "o": (W, H * dv)})
        if mlp and mlp["kind"] == "dense":
            s.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"]), p + "mlp.act": (2,)})
        elif mlp:
            F = mlp["expert"]["ff"]
            s[p + "mlp.table"] = (V, mlp["router"]["top"])
            for e in range(mlp["router"]["experts"]):
                s.update({p + "mlp.e%d.gate" % e: (F, W), p + "mlp.e%d.up" % e: (F, W), p + "mlp.e%d.down" % e: (W, F)})
    return s


def random_weights(cfg, seed=0):
    """Random weights, already rounded to bf16 (held as fp32) so that the engine's bf16 checkpoint holds exactly the same numbers; the
    experts' tables as int64."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "table":
            n_exp = cfg["layers"][int(name[1:name.index(".")])]["mlp"]["router"]["experts"]
            w[name] = torch.stack([torch.randperm(n_exp, generator=g)[:shape[1]] for _ in range(shape[0])]).long()
            continue
        if name.endswith("a2.b"):
            t = torch.randn(shape, generator=g) + 2.0
        elif last == "b":
            t = 0.2 * torch.randn(shape, generator=g)
        elif "norm" in name:
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "act":
            t = torch.randn(shape, generator=g)
        elif last == "talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) * shape[-1] ** -0.5
        else:
            t = torch.randn(shape, generator=g) * shape[-1] ** -0.5
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


def greedy(cfg, w, prompt, n):
    """n tokens generated greedily (lowest index on ties) behind the prompt, recomputing the whole sequence every time."""
    toks = list(prompt)
    out = []
    for _ in range(n):
        logits, _ = forward(cfg, w, toks)
        out.append(int(torch.argmax(logits[-1])))
        toks.append(out[-1])
    return out
