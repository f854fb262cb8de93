"""A per-layer input from the token's id, added to the stream at the end of a layer.

With x the residual stream after the layer's sub-layers, ``e`` this layer's ``dim`` columns of a table row chosen by the
token's id, and three small tensors of the layer::

    g = gelu_tanh(gate x) * e          gate [dim, W]
    y = proj g                         proj [W, dim]
    x <- x + y / sqrt(mean(y^2) + eps) * gain

The table ``[vocab, layers * dim]`` is one tensor for the whole model; a layer keeps its own column range.  The stream
itself (not a normed copy) feeds the gate: the part folds whatever is outstanding into the 32-bit residual and reads
it rounded to the engine's dtype in the same kernel.  Its output stays pending together with its RMS norm, so the next
layer's input norm (or the model's last norm) adds it in its own pass.

Spec: ``PartSpec("token_side", dim, index, vocab_size, eps, table_name, names=(gate, proj, norm))``; ``table_name`` is
absolute, the other names are relative to the part's prefix.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from .base import Part, ResidualStream
from .context import StepContext
from .linear import Linear
from .norm import RMSNorm
from .registry import TAILS
from .spec import PartSpec, TensorSpec


@TAILS.register("token_side")
class TokenSideInput(Part):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.dim = int(spec.dim)
        self.index = int(spec.index)
        self.layers = int(spec.layers)
        self.vocab_size = int(spec.vocab_size)
        if self.dim <= 0 or not 0 <= self.index < self.layers:
            raise ValueError(f"token_side: dim={self.dim}, layer {self.index} of {self.layers}")
        gate, proj, norm = spec.get("names", ("gate", "proj", "norm"))
        self.gate = Linear([f"{prefix}.{gate}"], [self.dim], hidden_size, dtype)
        self.proj = Linear([f"{prefix}.{proj}"], [hidden_size], self.dim, dtype)
        self.norm = RMSNorm(PartSpec("rmsnorm", eps=float(spec.eps), weight_suffix=""), hidden_size=hidden_size,
                            prefix=f"{prefix}.{norm}", dtype=dtype)
        self._table_spec = TensorSpec(spec.table_name, (self.vocab_size, self.layers * self.dim))
        self.table: Optional[torch.Tensor] = None

    def parts(self) -> List[Part]:
        return [self, self.norm]

    def tensors(self) -> List[TensorSpec]:
        return self.gate.tensors() + self.proj.tensors() + [self._table_spec]

    def load(self, store) -> None:
        self.gate.load(store)
        self.proj.load(store)
        whole = store.get(self._table_spec)
        self.table = whole[:, self.index * self.dim:(self.index + 1) * self.dim].to(self.dtype).contiguous()

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        return tokens * (2 * self.hidden_size + 2 * self.dim) * width

    def forward(self, stream: ResidualStream, ctx: StepContext) -> None:
        if stream.extra is not None or (stream.pending_norm is not None and not isinstance(stream.pending_norm, RMSNorm)):
            stream.settle()
        x = torch.empty(stream.residual.shape, dtype=self.dtype, device=stream.residual.device)
        post = stream.pending_norm
        kernels.rms_stream(stream.residual, stream.pending, (post.weight, post.eps) if post is not None else None, None, None, raw=x)
        stream.pending = stream.pending_norm = None
        z = self.gate.forward(x)
        g = torch.empty_like(z)
        kernels.gelu_tanh(z, g, self.table, ctx.token_ids)
        stream.pending = self.proj.forward(g)
        stream.pending_norm = self.norm
