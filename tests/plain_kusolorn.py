"""Kusolorn, written down plainly: one slow function per mechanism, in the precision of the tensors it is given
(the tests pass float64), token by token where the design has a recurrence.  Shares no code with the package.

Notation: W width, T tokens of ONE sequence (positions 0..T-1 unless ``start`` says otherwise).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


# ---- rotary angles ---------------------------------------------------------------------------------------------------
def rotary_frequencies(base: float, dims: int, scaling: Optional[dict]) -> List[float]:
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_pairs(x, positions, freqs):
    """x [T, heads, d]; the first 2*len(freqs) dimensions are rotated in neighbouring pairs."""
    out = x.clone()
    for i, f in enumerate(freqs):
        a = positions.to(x.dtype) * f
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


# ---- attention with a window that keeps the first tokens ---------------------------------------------------------------
def visible(i: int, j: int, window: Optional[int], keep_first: int) -> bool:
    if j > i:
        return False
    if window is None:
        return True
    return i - j < window or j < keep_first


def attention_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float, v_first=None, mix_index: int = -1):
    """h [T, W] -> (output [T, W], the layer's own unmixed values [T, G, vdim])."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = (h @ w["v"].T).view(T, G, dv)
    v_own = v
    if m.get("v_mix") and mix_index > 0:
        lam = w["vmix"]
        v = (1.0 - lam) * v + lam * v_first
    rot = m.get("rot")
    pos = torch.arange(T)
    if rot and rot.get("dims", 0):
        freqs = rotary_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q, k = rotate_pairs(q, pos, freqs), rotate_pairs(k, pos, freqs)
    q, k = rms(q, eps), rms(k, eps)
    mask = m.get("mask")
    window = int(mask["size"]) if mask else None
    keep = int(mask.get("keep_first", 0)) if mask else 0
    cap = m.get("softcap")
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) if window is None else (j <= i) & ((i - j < window) | (j < keep))     # visible(i, j, ...) as a table
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = float(cap) * torch.tanh(s / float(cap))
        s = s.masked_fill(~seen, -math.inf)
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * dv) @ w["o"].T, v_own


# ---- matrix memory with exponential gates ---------------------------------------------------------------------------------
def mlstm_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        n = torch.zeros(d, dtype=h.dtype)
        mx = torch.zeros((), dtype=h.dtype)
        for t in range(T):
            m_new = torch.maximum(fg[t, hh] + mx, ig[t, hh])
            a, b = torch.exp(fg[t, hh] + mx - m_new), torch.exp(ig[t, hh] - m_new)
            S = a * S + b * torch.outer(k[t, hh], v[t, hh])
            n = a * n + b * k[t, hh]
            mx = m_new
            den = torch.maximum((n @ q[t, hh]).abs(), torch.exp(-mx)) + 1e-6
            out[t, hh] = (S.T @ q[t, hh]) / den
    o = rms(out, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ---- gated delta rule -------------------------------------------------------------------------------------------------------
def causal_conv_silu(x, taps):
    """x [T, C], taps [C, K]: y_t = silu(sum_j taps[:, K-1-j] * x_{t-j}), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        if j < T:
            y[j:] += taps[:, K - 1 - j] * x[:T - j]
    return torch.nn.functional.silu(y)


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_mixer(h, w: Dict[str, torch.Tensor], m: dict, eps: float):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ w["q"].T, w["q.conv"]).view(T, G, d)
    k = causal_conv_silu(h @ w["k"].T, w["k.conv"]).view(T, G, d)
    v = causal_conv_silu(h @ w["v"].T, w["v.conv"]).view(T, H, dv)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(h @ w["b"].T)
    decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    gate = torch.nn.functional.silu(h @ w["g"].T).view(T, H, dv)
    o = rms(out, eps) * w["norm"] * gate
    return o.reshape(T, H * dv) @ w["o"].T


# ---- feed-forwards ----------------------------------------------------------------------------------------------------------
def dense_ff(h, w):
    return gelu_tanh(h @ w["up"].T) @ w["down"].T


def expert_ff(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def moe_ff(h, w, f: dict, routers=None):
    E, top, limit = int(f["router"]["experts"]), int(f["router"]["top"]), float(f["expert"]["limit"])
    z = h @ w["router"].T
    if routers is not None:
        routers.append((top, z))
    vals, idx = torch.topk(z, top, dim=-1)
    p = torch.softmax(vals, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += p[t, c] * expert_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], limit)[0]
    return out


def token_side(x, tokens, layer: int, dim: int, w: Dict[str, torch.Tensor], side_embed, eps):
    e = side_embed[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w["gate"].T) * e
    y = g @ w["proj"].T
    return x + rms(y, eps) * w["norm"]


# ---- the model ------------------------------------------------------------------------------------------------------------------
def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, tap=None, routers=None):
    """Logits [T, vocab] of one sequence; ``tap(i, x)`` sees the stream after every layer; ``routers``, a list, collects
    ``(top, logits)`` of every routed feed-forward."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = weights["embed"][tokens]
    side = config.get("token_side")
    v_first, n_mix = None, 0
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mw = _sub(weights, p + "mix.")
        h = rms_norm(x, weights[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            mixes = bool(m.get("v_mix"))
            y, v_own = attention_mixer(h, mw, m, eps, v_first, n_mix if mixes else -1)
            if mixes:
                if n_mix == 0:
                    v_first = v_own
                n_mix += 1
        elif kind == "mlstm":
            y = mlstm_mixer(h, mw, m, eps)
        elif kind == "delta":
            y = delta_mixer(h, mw, m, eps)
        else:
            raise ValueError(kind)
        x = x + y
        f = layer.get("mlp")
        if f:
            h = rms_norm(x, weights[p + "norm2"], eps)
            fw = _sub(weights, p + "mlp.")
            x = x + (dense_ff(h, fw) if f["kind"] == "dense" else moe_ff(h, fw, f, routers))
        if side:
            x = token_side(x, tokens, i, int(side["dim"]), _sub(weights, p + "side."), weights["side.embed"], eps)
        if tap is not None:
            tap(i, x)
    return rms_norm(x, weights["final.norm"], eps) @ weights["head"].T


def greedy(config: dict, weights: Dict[str, torch.Tensor], prompt, steps: int) -> List[int]:
    """Greedy continuation, recomputing the whole sequence every step (the lower id wins a tie)."""
    toks = list(prompt)
    out = []
    for _ in range(steps):
        nxt = int(torch.argmax(forward(config, weights, toks)[-1]))
        out.append(nxt)
        toks.append(nxt)
    return out


# ---- random weights for the tests -------------------------------------------------------------------------------------------------
def random_model(config: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights whose values are bfloat16 numbers.  The routers are made robust against rounding, so that a bfloat16
    engine and this implementation choose the same experts: the first E columns of the embedding carry, per token id, a
    ranking of the experts in steps of 1.5; every tensor that writes into the stream is small in those columns; a router's
    row e reads column e (plus a little of everything else, so that the weights still depend on the context)."""
    g = torch.Generator().manual_seed(seed)
    W, V = config["width"], config["vocab"]
    E_max = max([L["mlp"]["router"]["experts"] for L in config["layers"] if L.get("mlp") and L["mlp"]["kind"] == "moe"] + [0])

    def mat(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).bfloat16().to(dtype)

    def vec(n, around=0.0, spread=0.1):
        return (around + spread * torch.randn(n, generator=g)).bfloat16().to(dtype)

    def writer(i, gain=1.0):                         # [W, i]: output rows of the router's columns are small
        m = torch.randn(W, i, generator=g) * gain / math.sqrt(i)
        m[:E_max] *= 0.05
        return m.bfloat16().to(dtype)

    embed = torch.randn(V, W, generator=g)
    for tok in range(V):
        ranks = torch.randperm(E_max, generator=g) if E_max else []
        for e in range(E_max):
            embed[tok, e] = 7.5 - 1.5 * float(ranks[e])
    t: Dict[str, torch.Tensor] = {"embed": embed.bfloat16().to(dtype), "head": mat(V, W, 2.0), "final.norm": vec(W, 1.0)}
    side = config.get("token_side")
    if side:
        t["side.embed"] = (torch.randn(V, len(config["layers"]) * side["dim"], generator=g)).bfloat16().to(dtype)
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        t[p + "norm1"] = vec(W, 1.0)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"] = mat(H * d, W), mat(G * d, W), mat(G * dv, W)
            t[p + "mix.o"] = writer(H * dv)
            if m.get("v_mix"):
                t[p + "mix.vmix"] = (0.2 + 0.5 * torch.rand((), generator=g)).bfloat16().to(dtype)
        elif L["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * dv, W), mat(H * dv, W)
            t[p + "mix.i"], t[p + "mix.f"] = mat(H, W, 3.0), mat(H, W, 3.0)
            t[p + "mix.i.b"], t[p + "mix.f.b"] = vec(H, 0.0, 1.0), vec(H, 2.0, 1.0)
            t[p + "mix.norm"] = vec(H * dv, 1.0)
            t[p + "mix.o"] = writer(H * dv)
        else:
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"] = mat(G * d, W, 2.0), mat(G * d, W, 2.0), mat(H * dv, W, 2.0), mat(H * dv, W)
            for n, size in (("q", G * d), ("k", G * d), ("v", H * dv)):
                t[p + f"mix.{n}.conv"] = (torch.randn(size, K, generator=g) * 0.6).bfloat16().to(dtype)
            t[p + "mix.b"], t[p + "mix.a"] = mat(H, W, 2.0), mat(H, W, 2.0)
            t[p + "mix.A_log"], t[p + "mix.dt_bias"] = vec(H, -1.0, 0.7), vec(H, 0.0, 1.0)
            t[p + "mix.norm"] = vec(dv, 1.0)
            t[p + "mix.o"] = writer(H * dv)
        f = L.get("mlp")
        if f:
            t[p + "norm2"] = vec(W, 1.0)
            if f["kind"] == "dense":
                t[p + "mlp.up"], t[p + "mlp.down"] = mat(f["ff"], W), writer(f["ff"])
            else:
                E, ff = f["router"]["experts"], f["expert"]["ff"]
                for e in range(E):
                    t[f"{p}mlp.e{e}.gate"], t[f"{p}mlp.e{e}.up"], t[f"{p}mlp.e{e}.down"] = mat(ff, W, 2.0), mat(ff, W, 2.0), writer(ff)
                router = torch.randn(E, W, generator=g) * 0.05 / math.sqrt(W)
                router[:, :E_max] = 0.0
                for e in range(E):
                    router[e, e] = 2.0
                t[p + "mlp.router"] = router.bfloat16().to(dtype)
                t[p + "norm2"][:E_max] = 1.0
        if side:
            t[p + "side.gate"], t[p + "side.proj"] = mat(side["dim"], W), mat(W, side["dim"])
            gain = 0.5 + 0.1 * torch.randn(W, generator=g)
            gain[:E_max] = 0.02
            t[p + "side.norm"] = gain.bfloat16().to(dtype)
    return t


def router_margin(config: dict, weights: Dict[str, torch.Tensor], tokens) -> float:
    """The smallest gap between the last chosen and the first rejected router logit over the sequence's tokens and
    layers, as a fraction of the spread of the logits (tests assert that their weights leave a safe margin)."""
    logits: List[torch.Tensor] = []
    forward(config, weights, tokens, routers=logits)
    worst = math.inf
    for top, z in logits:
        if top < z.shape[1]:
            s = torch.sort(z, dim=-1, descending=True).values
            worst = min(worst, float(((s[:, top - 1] - s[:, top]) / (s[:, 0] - s[:, -1]).clamp_min(1e-9)).min()))
    return worst
