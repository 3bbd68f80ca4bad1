"""Plain, slow restatement of the Bumalix decoder, one function per mechanism, for the tests.

Bumalix is a decoder-only model given as a list of layers.  Every layer is *parallel* with ONE norm:

    n = rms_norm(x) * gain;   x <- x + (mixer(n) + ff(n))

The embedding row is multiplied by a constant.  A run of layers [start, stop) may be *looped*: it runs `times` times
in a row with the same weights, every pass with a cache and state of its own, and in front of every pass the stream is
re-mixed with the embedding output x0:  x <- W_in [x; x0].  The logits are cap * tanh(head . norm(x) / cap).

Mixers:

* "parallel": two mixers read the same input and the result is half the sum of their outputs, each RMS-normed over
  the model width with its own gain first.
    - left: grouped-query softmax attention with biased q / k / v projections, an RMS norm with a gain over the WHOLE
      q row (all heads at once) and over the whole k row, no positions in the scores, a configured scale and a sliding
      window (query i sees key j when 0 <= i - j < size).
    - right: gated linear attention.  Per head a matrix state S [dim, vdim]:
          S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t,
      alpha_t = sigmoid(A2 (A1 n_t) + b)^(1 / tau) per key channel, q scaled by dim^(-1/2).  o is RMS-normed per head
      with a gain shared by the heads, multiplied by silu(G n_t) and projected.
* "channel_delta": the gated delta rule.  q, k (kv_heads x dim) and v (heads x vdim) each pass a short causal
  convolution over time and silu; q and k heads become unit vectors (x / sqrt(sum x^2 + 1e-6)), q is scaled by
  dim^(-1/2).  beta_t = sigmoid(B n_t) per head, g_t = exp(-exp(A_log) softplus(A2 (A1 n_t) + dt_bias)) per head and key
  channel.  Per head:
          S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t.
  o is divided by its root mean square per head, multiplied by a gain and by sigmoid(G2 (G1 n_t)), and projected.

Feed-forwards:

* "dense": W_down poly(W_up n) with poly(z) = a N(z) + b N(z^2) + c N(z^3) + e, N(y) = y / sqrt(mean(y^2) + eps) over a
  token's ff values, powers element by element.
* "moe": a sigmoid router picks the `top` experts with the largest scores; an expert is
  W_down (silu(W_gate y) * (W_up y)) and it sees y = score * n (the weight multiplies the expert's INPUT, scores are not
  renormalised); a shared expert of the same form sees n itself and is added.

Nothing here shares code with the engine.  Tensors go in as a dict of torch tensors under the checkpoint's names.
`Stepper` runs token by token from explicit state (cached keys and values, matrix states, the last inputs of the
convolutions); `forward` feeds a whole sequence through it.
"""
from __future__ import annotations

import math

import torch

UNIT_EPS = 1e-6          # q and k of the delta rule: x / sqrt(sum(x^2) + UNIT_EPS)


def rms_norm(x: torch.Tensor, gain: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms_norm(z, None, eps) + b * rms_norm(z * z, None, eps) + c * rms_norm(z * z * z, None, eps) + e


def dense_ff(n: torch.Tensor, w: dict, pre: str, eps: float) -> torch.Tensor:
    return poly_norm(n @ w[pre + "up"].T, w[pre + "act"], eps) @ w[pre + "down"].T


def gated_expert(y: torch.Tensor, w: dict, pre: str) -> torch.Tensor:
    return (silu(y @ w[pre + "gate"].T) * (y @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(n: torch.Tensor, router: torch.Tensor, top: int):
    """n [W] -> (expert indices, their scores): the `top` largest sigmoid scores, lowest index first on ties."""
    s = torch.sigmoid(router @ n)
    order = sorted(range(s.numel()), key=lambda i: (-float(s[i]), i))[:top]
    return order, [s[i] for i in order]


def moe_ff(n: torch.Tensor, w: dict, pre: str, mlp: dict) -> torch.Tensor:
    """n [T, W]."""
    out = torch.zeros_like(n)
    for t in range(n.shape[0]):
        idx, sc = route(n[t], w[pre + "router"], mlp["router"]["top"])
        for i, s in zip(idx, sc):
            out[t] = out[t] + gated_expert(s * n[t], w, "%se%d." % (pre, i))
    if mlp.get("shared"):
        out = out + gated_expert(n, w, pre + "shared.")
    return out


def window_attention_step(q, keys, values, heads, kv_heads, dim, vdim, scale, window):
    """One query token q [heads*dim] at the END of keys [n, kv_heads*dim] / values [n, kv_heads*vdim] (its own row is the
    last one).  window None = every earlier key."""
    n = keys.shape[0]
    lo = 0 if window is None else max(0, n - window)
    out = []
    for a in range(heads):
        c = a // (heads // kv_heads)
        qa = q[a * dim:(a + 1) * dim]
        s = (keys[lo:, c * dim:(c + 1) * dim] @ qa) * scale
        p = torch.softmax(s, 0)
        out.append(p @ values[lo:, c * vdim:(c + 1) * vdim])
    return torch.cat(out)


def gla_step(S, q, k, v, alpha):
    """S [dim, vdim]; returns (S', o)."""
    S = alpha[:, None] * S + k[:, None] * v[None, :]
    return S, S.T @ q


def delta_step(S, q, k, v, g, beta):
    S = g[:, None] * S
    u = beta * (v - S.T @ k)
    S = S + k[:, None] * u[None, :]
    return S, S.T @ q


def unit_vector(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + UNIT_EPS)


def layer_runs(cfg: dict):
    """The order the layers run in: (layer index, first of a pass?) -- a looped layer appears once per pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    runs += [(i, False) for i in range(b, n)]
    return runs


class Stepper:
    """Token-by-token evaluation from explicit state; one state per layer RUN."""

    def __init__(self, cfg: dict, w: dict, dtype=torch.float64):
        self.cfg = cfg
        self.w = {k: v.to(dtype) for k, v in w.items()}
        self.dtype = dtype
        self.runs = layer_runs(cfg)
        self.state = [dict() for _ in self.runs]
        self.trace = []          # residual stream after every layer run of the last token

    def left(self, st, n, m, pre, eps):
        w = self.w
        q = w[pre + "q"] @ n + w[pre + "q.b"]
        k = w[pre + "k"] @ n + w[pre + "k.b"]
        v = w[pre + "v"] @ n + w[pre + "v.b"]
        q = rms_norm(q, w[pre + "q.norm"], eps)
        k = rms_norm(k, w[pre + "k.norm"], eps)
        st["k"] = k[None] if "k" not in st else torch.cat([st["k"], k[None]], 0)
        st["v"] = v[None] if "v" not in st else torch.cat([st["v"], v[None]], 0)
        window = m["mask"]["size"] if m.get("mask") else None
        o = window_attention_step(q, st["k"], st["v"], m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["scale"], window)
        return w[pre + "o"] @ o

    def right(self, st, n, m, pre, eps):
        w = self.w
        H, D, V = m["heads"], m["dim"], m["vdim"]
        q = (w[pre + "q"] @ n) * D ** -0.5
        k = w[pre + "k"] @ n
        v = w[pre + "v"] @ n
        alpha = torch.sigmoid(w[pre + "a2"] @ (w[pre + "a1"] @ n) + w[pre + "a2.b"]) ** (1.0 / m["tau"])
        if "S" not in st:
            st["S"] = [torch.zeros(D, V, dtype=self.dtype) for _ in range(H)]
        outs = []
        for a in range(H):
            st["S"][a], o = gla_step(st["S"][a], q[a * D:(a + 1) * D], k[a * D:(a + 1) * D], v[a * V:(a + 1) * V], alpha[a * D:(a + 1) * D])
            outs.append(rms_norm(o, w[pre + "norm"], eps))
        return w[pre + "o"] @ (torch.cat(outs) * silu(w[pre + "g"] @ n))

    def conv(self, st, key, x, taps_w):
        """x [C]: the newest input of the convolution; st[key] keeps the last taps - 1 inputs."""
        taps = taps_w.shape[1]
        hist = st.get(key)
        if hist is None:
            hist = torch.zeros(taps - 1, x.numel(), dtype=self.dtype)
        ext = torch.cat([hist, x[None]], 0)
        st[key] = ext[1:]
        return (taps_w.T * ext).sum(0)

    def delta(self, st, n, m, pre, eps):
        w = self.w
        H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
        q = silu(self.conv(st, "cq", w[pre + "q"] @ n, w[pre + "q.conv"]))
        k = silu(self.conv(st, "ck", w[pre + "k"] @ n, w[pre + "k.conv"]))
        v = silu(self.conv(st, "cv", w[pre + "v"] @ n, w[pre + "v.conv"]))
        q = unit_vector(q.reshape(G, D)) * D ** -0.5
        k = unit_vector(k.reshape(G, D))
        beta = torch.sigmoid(w[pre + "b"] @ n)
        dt = torch.nn.functional.softplus(w[pre + "a2"] @ (w[pre + "a1"] @ n) + w[pre + "dt_bias"]).reshape(H, D)
        g = torch.exp(-torch.exp(w[pre + "A_log"])[:, None] * dt)
        gate = torch.sigmoid(w[pre + "g2"] @ (w[pre + "g1"] @ n)).reshape(H, V)
        if "S" not in st:
            st["S"] = [torch.zeros(D, V, dtype=self.dtype) for _ in range(H)]
        outs = []
        for a in range(H):
            c = a // (H // G)
            st["S"][a], o = delta_step(st["S"][a], q[c], k[c], v[a * V:(a + 1) * V], g[a], beta[a])
            outs.append(rms_norm(o, w[pre + "norm"], eps) * gate[a])
        return w[pre + "o"] @ torch.cat(outs)

    def step(self, token: int) -> torch.Tensor:
        """Appends one token; returns its logits."""
        cfg, w = self.cfg, self.w
        eps = cfg["norm"]["eps"]
        x0 = w["embed"][token] * cfg.get("embedding", {}).get("scale", 1.0)
        x = x0
        self.trace = []
        for r, (li, pass_start) in enumerate(self.runs):
            L = cfg["layers"][li]
            st = self.state[r]
            pre = "l%d." % li
            if pass_start:
                x = w["loop.in"] @ torch.cat([x, x0])
            n = rms_norm(x, w[pre + "norm1"], eps)
            m = L["mixer"]
            if L["type"] == "parallel":
                lo = self.left(st.setdefault("left", {}), n, m["left"], pre + "mix.left.", eps)
                ro = self.right(st.setdefault("right", {}), n, m["right"], pre + "mix.right.", eps)
                mix = 0.5 * (rms_norm(lo, w[pre + "mix.left.out"], eps) + rms_norm(ro, w[pre + "mix.right.out"], eps))
            elif L["type"] == "channel_delta":
                mix = self.delta(st, n, m, pre + "mix.", eps)
            else:
                raise ValueError("mixer type %r" % L["type"])
            mlp = L.get("mlp")
            if not mlp:
                ff = torch.zeros_like(x)
            elif mlp["kind"] == "dense":
                ff = dense_ff(n[None], w, pre + "mlp.", eps)[0]
            elif mlp["kind"] == "moe":
                ff = moe_ff(n[None], w, pre + "mlp.", mlp)[0]
            else:
                raise ValueError("mlp kind %r" % mlp["kind"])
            x = x + (mix + ff)
            self.trace.append(x)
        y = w["head"] @ rms_norm(x, w["final.norm"], eps)
        cap = cfg.get("logit_softcap")
        return cap * torch.tanh(y / cap) if cap else y


    def greedy(self, prompt, n: int):
        """Feeds the prompt, then n times the most likely token (lowest index on ties); returns the n tokens."""
        for t in prompt:
            y = self.step(int(t))
        out = []
        for _ in range(n):
            out.append(int(torch.argmax(y)))
            y = self.step(out[-1])
        return out


def forward(cfg: dict, w: dict, tokens, dtype=torch.float64):
    """-> (logits [T, vocab], residual stream after every layer run [runs, T, W])."""
    s = Stepper(cfg, w, dtype)
    logits, traces = [], []
    for t in tokens:
        logits.append(s.step(int(t)))
        traces.append(torch.stack(s.trace))
    return torch.stack(logits), torch.stack(traces, 1)


def tensor_shapes(cfg: dict) -> dict:
    """name -> shape of every tensor a checkpoint of this config holds."""
    W, V = cfg["width"], cfg["vocab"]
    sh = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    if cfg.get("loop"):
        sh["loop.in"] = (W, 2 * W)
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        sh[p + "norm1"] = (W,)
        m = L["mixer"]
        if L["type"] == "parallel":
            a, b = m["left"], m["right"]
            H, G, D, Dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a["vdim"]
            q = p + "mix.left."
            sh.update({q + "q": (H * D, W), q + "q.b": (H * D,), q + "k": (G * D, W), q + "k.b": (G * D,), q + "v": (G * Dv, W),
                       q + "v.b": (G * Dv,), q + "q.norm": (H * D,), q + "k.norm": (G * D,), q + "o": (W, H * Dv), q + "out": (W,)})
            H, D, Dv, R = b["heads"], b["dim"], b["vdim"], b.get("rank", 4)
            q = p + "mix.right."
            sh.update({q + "q": (H * D, W), q + "k": (H * D, W), q + "v": (H * Dv, W), q + "g": (H * Dv, W), q + "o": (W, H * Dv),
                       q + "norm": (Dv,), q + "a1": (R, W), q + "a2": (H * D, R), q + "a2.b": (H * D,), q + "out": (W,)})
        else:
            H, G, D, Dv, taps, R = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"], m["conv"], m.get("rank", 8)
            q = p + "mix."
            sh.update({q + "q": (G * D, W), q + "k": (G * D, W), q + "v": (H * Dv, W), q + "q.conv": (G * D, taps), q + "k.conv": (G * D, taps),
                       q + "v.conv": (H * Dv, taps), q + "b": (H, W), q + "A_log": (H,), q + "norm": (Dv,), q + "a1": (R, W),
                       q + "a2": (H * D, R), q + "dt_bias": (H * D,), q + "g1": (R, W), q + "g2": (H * Dv, R), q + "o": (W, H * Dv)})
        mlp = L.get("mlp")
        if mlp and mlp["kind"] == "dense":
            sh.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"]), p + "mlp.act": (4,)})
        elif mlp:
            F = mlp["expert"]["ff"]
            sh[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for x in range(mlp["router"]["experts"]):
                sh.update({"%smlp.e%d.gate" % (p, x): (F, W), "%smlp.e%d.up" % (p, x): (F, W), "%smlp.e%d.down" % (p, x): (W, F)})
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                sh.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs)})
    return sh


def random_weights(cfg: dict, seed: int, spread: float = 1.0) -> dict:
    """bf16-representable random weights (the low-rank widths are not in the config: a checkpoint's shapes give them;
    here they come from an optional "rank" entry of the mixer, which the engine ignores)."""
    gen = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm", "out") or name.endswith(".q.norm") or name.endswith(".k.norm") or name == "final.norm":
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif last == "act":
            t = torch.tensor([0.6, 0.3, 0.2, 0.05]) + 0.05 * torch.randn(4, generator=gen)
        elif last == "A_log":
            t = torch.log(0.5 + 3.0 * torch.rand(shape, generator=gen))
        elif last == "dt_bias":
            t = torch.randn(shape, generator=gen) - 2.0
        elif last == "conv":
            t = 0.5 * torch.randn(shape, generator=gen)
        elif last == "b" and len(shape) == 1:
            t = (torch.randn(shape, generator=gen) + 2.0) if name.endswith("a2.b") else 0.3 * torch.randn(shape, generator=gen)
        elif name == "embed":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1]) * 2.0
        else:
            t = spread * torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w
