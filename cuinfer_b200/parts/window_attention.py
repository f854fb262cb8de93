"""Grouped-query attention with sizes of its own for keys and values, a capped score, and a sliding window that keeps
the first tokens of a sequence visible.

For the mixer's input h, H query heads and G key/value heads (query head i uses key/value head ``i // (H / G)``), query
and key size ``dim``, value size ``vdim``:

* ``q = Wq h``, ``k = Wk h``, ``v = Wv h``, no biases;
* the position encoding (rotary, on the first ``rotary_dim`` values of each head) on q and k, then each head of q and
  k divided by its root mean square over ``dim`` (``eps`` inside the root, no gain) when ``qk_unit_norm``;
* value mixing (``value_mix``): the ``"source"`` layer publishes its values of the step's tokens; a ``"mixed"`` layer
  caches ``(1 - m) v + m v_source`` with its own learned number ``m``;
* ``score = scale * q . k``, then ``softcap * tanh(score / softcap)`` when a cap is given;
* the query at position i sees key j when ``j <= i`` and (no window, or ``i - j < window``, or ``j < keep_first``);
  kept tokens keep their own positions; ordinary softmax; output projection ``Wo`` on the concatenated heads.

The cache holds a token's key and (mixed) value side by side: ``PagedCacheNeed(G, dim + vdim, window, planes=1,
keep_first)``; pages behind the window are given back, except those of the kept tokens.

Spec: ``PartSpec("window_attention", num_heads, num_kv_heads, dim, vdim, scale, softcap, window, keep_first,
qk_unit_norm, eps, value_mix, position=PartSpec(...), names=(q, k, v, o, mix))``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from . import attention_dispatch
from .base import Mixer
from .context import StepContext
from .linear import Linear
from .registry import MIXERS, POSITION_ENCODINGS
from .spec import PagedCacheNeed, PartSpec, TensorSpec

VALUE_MIX_KEY = "window_attention.values"


@MIXERS.register("window_attention")
class WindowAttention(Mixer):
    accepts_lazy_norm = True       # the q/k/v projection can compute the norm of its input itself

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads = int(spec.num_heads)
        self.num_kv_heads = int(spec.num_kv_heads)
        self.dim = int(spec.dim)
        self.vdim = int(spec.vdim)
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError("window_attention: num_heads must be a positive multiple of num_kv_heads")
        if not (0 < self.dim <= 512 and 0 < self.vdim <= 512):
            raise ValueError(f"window_attention: key size {self.dim} / value size {self.vdim} are beyond what the kernels take (512)")
        self.scale = float(spec.scale)
        self.softcap = float(spec.get("softcap") or 0.0)
        self.window = int(spec.get("window") or 0)
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.eps = float(spec.get("eps", 1e-6))
        if not spec.get("qk_unit_norm", True):
            raise ValueError("window_attention: queries and keys without the unit norm are not built")
        self.value_mix = spec.get("value_mix")
        if self.value_mix not in (None, "source", "mixed"):
            raise ValueError(f"window_attention: value_mix must be None, 'source' or 'mixed', got {self.value_mix!r}")
        pos_spec: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        if self.position.rotary_dim > self.dim:
            raise ValueError("window_attention: rotary_dim exceeds dim")
        if self.position.rotary_dim and not hasattr(self.position, "frequencies"):
            raise ValueError("window_attention: the position encoding must hand out frequencies (rope_interleaved)")
        q, k, v, o, mix = spec.get("names", ("q", "k", "v", "o", "vmix"))
        p = prefix
        self.q_size, self.k_size, self.v_size = self.num_heads * self.dim, self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim
        self.qkv = Linear([f"{p}.{q}", f"{p}.{k}", f"{p}.{v}"], [self.q_size, self.k_size, self.v_size], hidden_size, dtype)
        self.o = Linear([f"{p}.{o}"], [hidden_size], self.num_heads * self.vdim, dtype)
        self._mix_spec = TensorSpec(f"{p}.{mix}", (), init="zeros") if self.value_mix else None
        self.mix: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorSpec]:
        return self.qkv.tensors() + self.o.tensors() + ([self._mix_spec] if self._mix_spec else []) + self.position.tensors()

    def load(self, store) -> None:
        self.qkv.load(store)
        self.o.load(store)
        if self._mix_spec is not None:
            self.mix = store.get(self._mix_spec).reshape(1).contiguous()
        self.position.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.qkv.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    def cache_need(self) -> Optional[PagedCacheNeed]:
        return PagedCacheNeed(self.num_kv_heads, self.dim + self.vdim, self.window or None, planes=1,
                              keep_first=self.keep_first)

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        return self.qkv.workspace_bytes(tokens) + tokens * self.num_heads * self.vdim * width + self.o.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        kv = ctx.paged_kv(run)
        qkv = self.qkv.forward(x)
        v_first = None
        if self.value_mix == "source":
            ctx.shared[VALUE_MIX_KEY] = qkv[:, self.q_size + self.k_size:]        # stays unmixed: only the cache gets values
        elif self.value_mix == "mixed":
            v_first = ctx.shared.get(VALUE_MIX_KEY)
            if v_first is None or v_first.shape != (qkv.shape[0], self.v_size):
                raise RuntimeError("window_attention: no earlier layer of this step published values of this shape to mix in")
        freq = self.position.frequencies() if self.position.rotary_dim else None
        kernels.window_attention_prep(qkv, ctx.positions, kv.group.slot_mapping if kv.writes else None, freq,
                                      self.position.rotary_dim, self.eps, self.num_heads, self.num_kv_heads, self.dim, self.vdim,
                                      v_first, self.mix if v_first is not None else None, kv.cache if kv.writes else None)
        out = torch.empty((qkv.shape[0], self.num_heads * self.vdim), dtype=qkv.dtype, device=qkv.device)
        attention_dispatch.window_attention(qkv, out, kv, ctx, self.num_heads, self.num_kv_heads, self.dim, self.vdim,
                                            self.scale, self.softcap, self.window, self.keep_first)
        return self.o.forward(out)
