"""Bilolorn as data: a decoder whose layers norm every sub-layer on both sides, attend through latents, and take
their feed-forward from a per-layer menu; a span of layers may run several times.

``config.json`` (every size and every constant that can differ between models of the design is read from it):

* ``architecture``: "Bilolorn"; ``vocab``, ``width``; ``embedding.scale``; ``norm.eps``;
* ``layers``: a list; entry i has ``type`` (the mixer), ``mixer`` (its sizes) and ``mlp`` (its feed-forward, or null);
  its tensors start with ``l<i>.``;
* ``loop``: ``{start, stop, times}`` — layers start..stop-1 run ``times`` times in a row with the same weights and
  a cache of their own per pass; before every pass but the first the embedding output is added to the stream.

The network: ``x = embed[token] * scale``; per layer ``x += norm1b(mixer(norm1(x)))`` and, when it has a feed-forward,
``x += norm2b(ff(norm2(x)))`` with layer norms (gain ``<name>``, bias ``<name>.b``); ``logits = head(final.norm(x))``.

Mixer ``latent_attention`` (``heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims}``): see
``parts/latent_attention.py``; here with a sink per head, an output gate, interleaved rotary pairs and no window.
Feed-forward ``dense`` (``ff``): ``down(relu(up h) ** 2)``.  ``moe`` (``router: {experts, top}``, ``expert.ff``,
optional ``shared.ff``): experts by a table from token id, weight ``1 / top`` each, plus a shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

ARCHITECTURE = "Bilolorn"
# The design has no table of positions and hence no largest position of its own; this bounds what one request may hold.
MAX_POSITIONS = 1 << 17


def _obj(raw: Mapping[str, Any], key: str, where: str, optional: bool = False) -> Optional[Mapping[str, Any]]:
    value = raw.get(key)
    if value is None:
        if optional:
            return None
        raise ConfigError(f"invalid model config: {where}'{key}' is missing")
    if not isinstance(value, dict):
        raise ConfigError(f"invalid model config: {where}'{key}' must be an object")
    return value


def _positive(raw: Mapping[str, Any], key: str, where: str) -> int:
    try:
        v = take(raw, key, int)
    except ConfigError as exc:
        raise ConfigError(f"{exc} (in {where})") from None
    if v <= 0:
        raise ConfigError(f"invalid model config: {where}'{key}' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "LatentMixerConfig":
        rot = _obj(raw, "rot", where)
        out = cls(heads=_positive(raw, "heads", where), dim=_positive(raw, "dim", where), rot_dim=_positive(raw, "rot_dim", where),
                  vdim=_positive(raw, "vdim", where), q_rank=_positive(raw, "q_rank", where), kv_rank=_positive(raw, "kv_rank", where),
                  scale=take(raw, "scale", float), rot_base=take(rot, "base", float), rot_dims=take(rot, "dims", int))
        if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.rot_dim:
            raise ConfigError(f"invalid model config: {where}rot.dims={out.rot_dims} must be even and at most rot_dim={out.rot_dim}")
        if not out.rot_base > 0:
            raise ConfigError(f"invalid model config: {where}rot.base must be positive")
        return out

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int                     # dense: its size; moe: an expert's size
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = take(raw, "kind", str)
        if kind == "dense":
            return cls("dense", _positive(raw, "ff", where))
        if kind == "moe":
            router, expert = _obj(raw, "router", where), _obj(raw, "expert", where)
            shared = _obj(raw, "shared", where, optional=True)
            out = cls("moe", _positive(expert, "ff", where + "expert."), _positive(router, "experts", where + "router."),
                      _positive(router, "top", where + "router."), _positive(shared, "ff", where + "shared.") if shared else 0)
            if out.top > out.experts:
                raise ConfigError(f"invalid model config: {where}router.top={out.top} exceeds router.experts={out.experts}")
            return out
        raise ConfigError(f"unsupported option: {where}kind={kind!r} (dense or moe)")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class BilolornLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class BilolornConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[BilolornLayerConfig, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def max_model_len(self) -> int:
        return MAX_POSITIONS

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BilolornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("invalid model config: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"invalid model config: layers[{i}] must be an object")
            kind = take(entry, "type", str)
            if kind != "latent_attention":
                raise ConfigError(f"unsupported option: {where}type={kind!r} (this design's mixer is latent_attention)")
            mlp = _obj(entry, "mlp", where, optional=True)
            layers.append(BilolornLayerConfig(kind, LatentMixerConfig.from_dict(_obj(entry, "mixer", where), where + "mixer."),
                                              FeedForwardConfig.from_dict(mlp, where + "mlp.") if mlp else None))
        loop = _obj(raw, "loop", "", optional=True)
        start, stop, times = (take(loop, "start", int), take(loop, "stop", int), take(loop, "times", int)) if loop else (0, 0, 1)
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ConfigError(f"invalid model config: loop start={start} stop={stop} times={times} does not fit {len(layers)} layers")
        eps = take(_obj(raw, "norm", ""), "eps", float)
        if not eps > 0:
            raise ConfigError("invalid model config: norm.eps must be positive")
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""),
                   embedding_scale=take(_obj(raw, "embedding", ""), "scale", float), norm_eps=eps, layers=tuple(layers),
                   loop_start=start, loop_stop=stop, loop_times=times, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "architectures": [ARCHITECTURE], "vocab": self.vocab, "width": self.width,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None} for l in self.layers],
               "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def run_order(cfg: BilolornConfig) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """(layer of every run, runs before which the embedding output is added again)."""
    order = list(range(cfg.loop_start))
    again = []
    for k in range(cfg.loop_times):
        if k > 0 and cfg.loop_stop > cfg.loop_start:
            again.append(len(order))
        order += list(range(cfg.loop_start, cfg.loop_stop))
    order += list(range(cfg.loop_stop, len(cfg.layers)))
    return tuple(order), tuple(again)


def bilolorn_spec(cfg: BilolornConfig) -> ModelSpec:
    norm = PartSpec("layernorm", eps=cfg.norm_eps, weight_suffix="", bias_suffix=".b")
    block = PartSpec("sandwich", norm_names=("norm1", "norm1b", "norm2", "norm2b"))
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        mixer = PartSpec("latent_attention", name="mix", num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                         q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, eps=cfg.norm_eps, sink=True, gate=True, window=None,
                         position=PartSpec("rope_interleaved", theta=m.rot_base, rotary_dim=m.rot_dims))
        f = layer.mlp
        if f is None:
            ffn = PartSpec("none", name="mlp")
        elif f.kind == "dense":
            ffn = PartSpec("relu2", name="mlp", intermediate_size=f.ff, names=("up", "down"))
        else:
            ffn = PartSpec("moe_table", name="mlp", experts=f.experts, top=f.top, intermediate_size=f.ff, vocab_size=cfg.vocab,
                           shared_size=f.shared_ff, expert_names=("e{}.gate", "e{}.up", "e{}.down"), table_name="table",
                           shared_names=("shared.gate", "shared.up", "shared.down"))
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    order, again = run_order(cfg)
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, layers=tuple(layers),
                     final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm", lm_head_name="head",
                     order=order, eos_token_ids=tuple(cfg.eos_token_ids), embedding_scale=cfg.embedding_scale,
                     reinject_embedding_before=again)


register_architecture(ARCHITECTURE, BilolornConfig.from_dict, bilolorn_spec, replace=True)
