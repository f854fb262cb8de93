"""A plain, slow Bilolorn decoder on the CPU: one function per mechanism, written from the design's equations.

It shares no code with the package: it reads a config dictionary and a dictionary of tensors by name, keeps no cache
(every call recomputes the whole sequence) and uses torch only for arithmetic, in whatever floating type the tensors
have (the tests use float64).  Notation: ``W`` width of the residual stream, ``H`` heads, ``dn`` unrotated and ``dr``
rotated query/key dimensions per head, ``dv`` value size per head, ``rk`` latent size of keys and values.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Sequence

import torch

Tensors = Mapping[str, torch.Tensor]


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [..., T, d]: element 2i pairs with 2i+1 for i < dims/2; the rest of d passes unchanged.  Frequencies and
    angles are 32-bit numbers, as the design has them; sine and cosine are taken in x's type."""
    out = x.clone()
    for i in range(dims // 2):
        f = torch.tensor(base ** (-2.0 * i / dims), dtype=torch.float32)
        a = (positions.to(torch.float32) * f).to(x.dtype)
        c, s = torch.cos(a), torch.sin(a)
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_with_sink(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, T, S] (masked entries -inf), sink [H]: weights whose denominator also holds exp(sink)."""
    m = torch.maximum(scores.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def latent_attention(h: torch.Tensor, t: Tensors, p: str, m: Mapping, eps: float) -> torch.Tensor:
    """h [T, W] of one sequence starting at position 0 → [T, W]."""
    T = h.shape[0]
    H, dn, dr, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(h @ t[p + "dq"].T, t[p + "dq.norm"], eps)
    q = (cq @ t[p + "uq"].T).view(T, H, dn + dr).transpose(0, 1)                 # [H, T, dn + dr]
    q_plain, q_rot = q[..., :dn], rotate_interleaved(q[..., dn:], pos[None, :], m["rot"]["base"], m["rot"]["dims"])
    down = h @ t[p + "dkv"].T                                                      # [T, rk + dr]
    c = rms_norm(down[:, :rk], t[p + "dkv.norm"], eps)
    k_rot = rotate_interleaved(down[:, rk:], pos, m["rot"]["base"], m["rot"]["dims"])      # shared by all heads
    k_plain = (c @ t[p + "uk"].T).view(T, H, dn).transpose(0, 1)
    v = (c @ t[p + "uv"].T).view(T, H, dv).transpose(0, 1)
    scores = (q_plain @ k_plain.transpose(1, 2) + q_rot @ k_rot.T[None]) * m["scale"]
    causal = pos[None, :] <= pos[:, None]
    scores = scores.masked_fill(~causal[None], -math.inf)
    w = softmax_with_sink(scores, t[p + "sink"].to(h.dtype))
    heads = (w @ v).transpose(0, 1).reshape(T, H * dv)
    gate = torch.sigmoid(h @ t[p + "g"].T)
    return (heads * gate) @ t[p + "o"].T


def dense_ff(h: torch.Tensor, t: Tensors, p: str) -> torch.Tensor:
    return (torch.relu(h @ t[p + "up"].T) ** 2) @ t[p + "down"].T


def gated_expert(h: torch.Tensor, t: Tensors, p: str) -> torch.Tensor:
    g = h @ t[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def table_moe(h: torch.Tensor, tokens: Sequence[int], t: Tensors, p: str, mlp: Mapping) -> torch.Tensor:
    top = mlp["router"]["top"]
    out = torch.zeros_like(h)
    table = t[p + "table"]
    for i, tok in enumerate(tokens):
        for e in table[tok].tolist():
            out[i] += gated_expert(h[i:i + 1], t, f"{p}e{e}.")[0] / top
    if mlp.get("shared"):
        out = out + gated_expert(h, t, p + "shared.")
    return out


def run_order(cfg: Mapping) -> List[tuple]:
    """(layer, adds the embedding output first?) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, False) for i in range(a)]
    for k in range(times):
        runs += [(i, k > 0 and i == a) for i in range(a, b)]
    runs += [(i, False) for i in range(b, n)]
    return runs


def forward(cfg: Mapping, t: Tensors, tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    idx = torch.tensor(list(tokens), dtype=torch.long)
    x0 = t["embed"][idx] * cfg["embedding"]["scale"]
    x = x0
    after = []
    for layer, add_embedding in run_order(cfg):
        L = cfg["layers"][layer]
        p = f"l{layer}."
        if add_embedding:
            x = x + x0
        assert L["type"] == "latent_attention"
        h = layer_norm(x, t[p + "norm1"], t[p + "norm1.b"], eps)
        y = latent_attention(h, t, p + "mix.", L["mixer"], eps)
        x = x + layer_norm(y, t[p + "norm1b"], t[p + "norm1b.b"], eps)
        mlp = L.get("mlp")
        if mlp:
            h = layer_norm(x, t[p + "norm2"], t[p + "norm2.b"], eps)
            y = dense_ff(h, t, p + "mlp.") if mlp["kind"] == "dense" else table_moe(h, tokens, t, p + "mlp.", mlp)
            x = x + layer_norm(y, t[p + "norm2b"], t[p + "norm2b.b"], eps)
        after.append(x)
    logits = layer_norm(x, t["final.norm"], t["final.norm.b"], eps) @ t["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(cfg: Mapping, t: Tensors, prompt: Sequence[int], n: int) -> List[int]:
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, t, seq)[-1].argmax()))
    return seq[len(prompt):]


# ---- small random models for the tests ---------------------------------------------------------------------------------
def random_model(cfg: Mapping, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    """Tensors by name for ``cfg``: matrices N(0, 1/fan_in) rounded to bfloat16 values, gains near one, small biases,
    sinks of either sign, a table whose rows name ``top`` different experts."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).bfloat16().to(dtype)

    def vec(n, around=0.0, spread=0.1):
        return (around + spread * torch.randn(n, generator=g)).bfloat16().to(dtype)

    t: Dict[str, torch.Tensor] = {"embed": mat(V, W, math.sqrt(W)), "head": mat(V, W), "final.norm": vec(W, 1.0),
                                  "final.norm.b": vec(W)}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if L.get("mlp") else [])
        for n in names:
            t[p + n] = vec(W, 1.0)
            t[p + n + ".b"] = vec(W)
        m = L["mixer"]
        H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        t[p + "mix.dq"] = mat(rq, W)
        t[p + "mix.dq.norm"] = vec(rq, 1.0)
        t[p + "mix.uq"] = mat(H * (dn + dr), rq, 2.0)
        t[p + "mix.dkv"] = mat(rk + dr, W)
        t[p + "mix.dkv.norm"] = vec(rk, 1.0)
        t[p + "mix.uk"] = mat(H * dn, rk, 2.0)
        t[p + "mix.uv"] = mat(H * dv, rk)
        t[p + "mix.sink"] = vec(H, 0.0, 1.0)
        t[p + "mix.g"] = mat(H * dv, W)
        t[p + "mix.o"] = mat(W, H * dv)
        mlp = L.get("mlp")
        if not mlp:
            continue
        if mlp["kind"] == "dense":
            t[p + "mlp.up"] = mat(mlp["ff"], W)
            t[p + "mlp.down"] = mat(W, mlp["ff"])
        else:
            E, top, ff = mlp["router"]["experts"], mlp["router"]["top"], mlp["expert"]["ff"]
            for e in range(E):
                t[f"{p}mlp.e{e}.gate"] = mat(ff, W)
                t[f"{p}mlp.e{e}.up"] = mat(ff, W)
                t[f"{p}mlp.e{e}.down"] = mat(W, ff)
            t[p + "mlp.table"] = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(V)]).to(torch.int32)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                t[p + "mlp.shared.gate"] = mat(sf, W)
                t[p + "mlp.shared.up"] = mat(sf, W)
                t[p + "mlp.shared.down"] = mat(W, sf)
    return t
