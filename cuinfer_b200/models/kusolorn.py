"""Kusolorn as data: a pre-norm decoder whose layers choose their mixer — windowed attention with kept first tokens,
a matrix memory with exponential gates, or the gated delta rule — and their feed-forward per layer, and add a
per-layer input from the token's id at the end of every layer.

``config.json`` (every size, and every constant that can differ between models of the design, is read from it):

* ``architecture``: "Kusolorn"; ``vocab``, ``width``; ``norm.eps``; ``token_side.dim`` (absent: no per-layer input);
* ``layers``: a list; entry i has ``type`` (``attention``, ``mlstm`` or ``delta``), ``mixer`` (its sizes) and ``mlp``
  (``{kind: dense, ff}``, ``{kind: moe, router: {experts, top}, expert: {ff, limit}}``, or null); its tensors start
  with ``l<i>.``.

The network: ``x = embed[token]``; per layer ``x += mixer(rms(x) * norm1)``, ``x += ff(rms(x) * norm2)``, then
``x += rms(proj(gelu(gate x) * side_embed[token, layer's columns])) * side.norm``; ``logits = head(rms(x) * final.norm)``.
Mixers: ``parts/window_attention.py`` (``heads, kv_heads, dim, vdim, scale, softcap, mask: {size, keep_first},
rot: {base, dims, scaling: {factor, low, high, original}}, v_mix``), ``parts/recurrent.py`` (``mlstm``: ``heads, dim, vdim,
gate_cap``; ``delta``: ``heads, kv_heads, dim, vdim, conv``).  Of the attention layers that say ``v_mix``, the first one
in the model publishes its values and the later ones mix them into their own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, take
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec

ARCHITECTURE = "Kusolorn"
# The design has no table of positions and hence no largest position of its own; this bounds what one request may hold.
MAX_POSITIONS = 1 << 17
MIXER_TYPES = ("attention", "mlstm", "delta")


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


def _number(raw: Mapping[str, Any], key: str, where: str) -> float:
    try:
        return float(take(raw, key, float))
    except ConfigError as exc:
        raise ConfigError(f"{exc} (in {where})") from None


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    keep_first: int
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[Tuple[float, float, float, float]]     # factor, low, high, original
    v_mix: bool

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "AttentionConfig":
        mask = _obj(raw, "mask", where, optional=True)
        rot = _obj(raw, "rot", where, optional=True)
        scaling = _obj(rot, "scaling", where + "rot.", optional=True) if rot else None
        cap = raw.get("softcap")
        out = cls(heads=_positive(raw, "heads", where), kv_heads=_positive(raw, "kv_heads", where), dim=_positive(raw, "dim", where),
                  vdim=_positive(raw, "vdim", where), scale=_number(raw, "scale", where),
                  softcap=float(cap) if cap else None,
                  window=_positive(mask, "size", where + "mask.") if mask else None,
                  keep_first=int(mask.get("keep_first", 0) or 0) if mask else 0,
                  rot_base=_number(rot, "base", where + "rot.") if rot else 1.0,
                  rot_dims=take(rot, "dims", int) if rot else 0,
                  rot_scaling=tuple(_number(scaling, k, where + "rot.scaling.") for k in ("factor", "low", "high", "original")) if scaling else None,
                  v_mix=bool(raw.get("v_mix", False)))
        if out.heads % out.kv_heads:
            raise ConfigError(f"invalid model config: {where}heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        if out.rot_dims < 0 or out.rot_dims % 2 or out.rot_dims > out.dim:
            raise ConfigError(f"invalid model config: {where}rot.dims={out.rot_dims} must be even and at most dim={out.dim}")
        if rot and not out.rot_base > 0:
            raise ConfigError(f"invalid model config: {where}rot.base must be positive")
        if out.keep_first < 0:
            raise ConfigError(f"invalid model config: {where}mask.keep_first must not be negative")
        return out

    def to_dict(self) -> dict:
        out: dict = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale,
                     "softcap": self.softcap, "v_mix": self.v_mix}
        if self.window is not None:
            out["mask"] = {"size": self.window, "keep_first": self.keep_first}
        if self.rot_dims:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling:
                out["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), self.rot_scaling))
        return out


@dataclass(frozen=True)
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "MatrixMemoryConfig":
        out = cls(_positive(raw, "heads", where), _positive(raw, "dim", where), _positive(raw, "vdim", where),
                  _number(raw, "gate_cap", where))
        if not out.gate_cap > 0:
            raise ConfigError(f"invalid model config: {where}gate_cap must be positive")
        return out

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "DeltaConfig":
        out = cls(_positive(raw, "heads", where), _positive(raw, "kv_heads", where), _positive(raw, "dim", where),
                  _positive(raw, "vdim", where), _positive(raw, "conv", where))
        if out.heads % out.kv_heads:
            raise ConfigError(f"invalid model config: {where}heads={out.heads} is not a multiple of kv_heads={out.kv_heads}")
        return out

    def to_dict(self) -> dict:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}


_MIXER_CONFIGS = {"attention": AttentionConfig, "mlstm": MatrixMemoryConfig, "delta": DeltaConfig}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                   # "dense" or "moe"
    ff: int                     # dense: its size; moe: an expert's size
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any], where: str) -> "FeedForwardConfig":
        kind = take(raw, "kind", str)
        if kind == "dense":
            return cls("dense", _positive(raw, "ff", where))
        if kind == "moe":
            router, expert = _obj(raw, "router", where), _obj(raw, "expert", where)
            out = cls("moe", _positive(expert, "ff", where + "expert."), _positive(router, "experts", where + "router."),
                      _positive(router, "top", where + "router."), _number(expert, "limit", where + "expert."))
            if out.top > out.experts:
                raise ConfigError(f"invalid model config: {where}router.top={out.top} exceeds router.experts={out.experts}")
            if not out.limit > 0:
                raise ConfigError(f"invalid model config: {where}expert.limit must be positive")
            return out
        raise ConfigError(f"unsupported option: {where}kind={kind!r} (dense or moe)")

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class KusolornLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class KusolornConfig:
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                 # 0: no per-layer input from the token's id
    layers: Tuple[KusolornLayerConfig, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @property
    def max_model_len(self) -> int:
        return MAX_POSITIONS

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "KusolornConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("invalid model config: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"invalid model config: layers[{i}] must be an object")
            kind = take(entry, "type", str)
            if kind not in _MIXER_CONFIGS:
                raise ConfigError(f"unsupported option: {where}type={kind!r} (one of {', '.join(MIXER_TYPES)})")
            mlp = _obj(entry, "mlp", where, optional=True)
            layers.append(KusolornLayerConfig(kind, _MIXER_CONFIGS[kind].from_dict(_obj(entry, "mixer", where), where + "mixer."),
                                              FeedForwardConfig.from_dict(mlp, where + "mlp.") if mlp else None))
        eps = _number(_obj(raw, "norm", ""), "eps", "norm.")
        if not eps > 0:
            raise ConfigError("invalid model config: norm.eps must be positive")
        side = _obj(raw, "token_side", "", optional=True)
        eos = raw.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        mixes = [l.mixer for l in layers if l.type == "attention" and l.mixer.v_mix]
        if len({(m.kv_heads, m.vdim) for m in mixes}) > 1:
            raise ConfigError("invalid model config: attention layers that mix values must agree in kv_heads and vdim")
        return cls(vocab=_positive(raw, "vocab", ""), width=_positive(raw, "width", ""), norm_eps=eps,
                   side_dim=_positive(side, "dim", "token_side.") if side else 0, layers=tuple(layers), eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": l.mlp.to_dict() if l.mlp else None} for l in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out


def _mixer_spec(layer: KusolornLayerConfig, eps: float, mixes_before: int) -> PartSpec:
    m = layer.mixer
    if layer.type == "attention":
        role = None if not m.v_mix else "source" if mixes_before == 0 else "mixed"
        position = PartSpec("rope_interleaved", theta=m.rot_base, rotary_dim=m.rot_dims, scaling=m.rot_scaling) if m.rot_dims else PartSpec("none")
        return PartSpec("window_attention", name="mix", num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                        scale=m.scale, softcap=m.softcap, window=m.window, keep_first=m.keep_first, qk_unit_norm=True, eps=eps,
                        value_mix=role, position=position, names=("q", "k", "v", "o", "vmix"))
    if layer.type == "mlstm":
        return PartSpec("mlstm", name="mix", num_heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap, eps=eps)
    return PartSpec("gated_delta", name="mix", num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, taps=m.conv, eps=eps)


def kusolorn_spec(cfg: KusolornConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", eps=cfg.norm_eps, weight_suffix="")
    layers = []
    mixes = 0
    for i, layer in enumerate(cfg.layers):
        mixer = _mixer_spec(layer, cfg.norm_eps, mixes)
        if layer.type == "attention" and layer.mixer.v_mix:
            mixes += 1
        f = layer.mlp
        if f is None:
            ffn = PartSpec("none", name="mlp")
        elif f.kind == "dense":
            ffn = PartSpec("gelu_tanh", name="mlp", intermediate_size=f.ff, names=("up", "down"))
        else:
            ffn = PartSpec("moe_routed", name="mlp", experts=f.experts, top=f.top, intermediate_size=f.ff, activation="clamped",
                           limit=f.limit, router_name="router", expert_names=("e{}.gate", "e{}.up", "e{}.down"))
        after = None
        if cfg.side_dim:
            after = PartSpec("token_side", name="side", dim=cfg.side_dim, index=i, layers=len(cfg.layers), vocab_size=cfg.vocab,
                             eps=cfg.norm_eps, table_name="side.embed", names=("gate", "proj", "norm"))
        block = PartSpec("prenorm", norm_names=("norm1", "norm2"), after=after)
        layers.append(LayerSpec(prefix=f"l{i}", block=block, mixer=mixer, feed_forward=ffn, norm=norm))
    return ModelSpec(hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, layers=tuple(layers),
                     final_norm=norm, embedding_name="embed", final_norm_prefix="final.norm", lm_head_name="head",
                     eos_token_ids=tuple(cfg.eos_token_ids))


register_architecture(ARCHITECTURE, KusolornConfig.from_dict, kusolorn_spec, replace=True)
