"""Mixers that carry a matrix per head from token to token instead of a cache of keys.

Both keep their state in 32 bits in the request's state slot (zero when the request is admitted), read it at the start
of a step and write it back at the end, so a prompt may be cut anywhere.  What enters the recurrence besides the
projections — gates, decays, their logarithms and exponentials, unit norms, the read-out, the norm after it — is 32-bit.

``mlstm`` — a matrix memory with exponential gates.  For the input h, H heads, key size d, value size dv:
``q = Wq h / sqrt(d)``, ``k = Wk h``, ``v = Wv h``; per head a log input gate ``i = c tanh((Wi h + bi) / c)`` and a log
forget gate ``f = logsigmoid(c tanh((Wf h + bf) / c))`` (c = ``gate_cap``); with a running maximum m that starts at 0::

    m' = max(f + m, i);  S' = exp(f + m - m') S + exp(i - m') k v^T;  n' = exp(f + m - m') n + exp(i - m') k
    o  = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)

then each head's o divided by its root mean square, times a gain over all heads, times ``sigmoid(Wg h)``, then ``Wo``.
Spec: ``PartSpec("mlstm", num_heads, dim, vdim, gate_cap, eps, names={...})``.

``gated_delta`` — the gated delta rule.  G query/key heads of size d, H value heads of size dv (head i uses q/k head
``i // (H / G)``): q, k, v go through a short causal convolution per channel (``taps`` columns, the last one the current
token's; the last ``taps - 1`` inputs are state too) and SiLU; q and k become unit vectors (``x / sqrt(sum x^2 + 1e-6)``),
q also times ``1 / sqrt(d)``; ``beta = sigmoid(Wb h)`` and ``g = exp(-exp(A_log) * softplus(Wa h + dt_bias))`` per head::

    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q

then each head's o divided by its root mean square over dv, times a gain of dv values shared by the heads, times
``silu(Wg h)``, then ``Wo``.  Spec: ``PartSpec("gated_delta", num_heads, num_kv_heads, dim, vdim, taps, eps, names={...})``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from .base import Mixer
from .context import StepContext
from .linear import Linear
from .registry import MIXERS
from .spec import PartSpec, StateNeed, TensorSpec

MLSTM_FLOOR = 1e-6          # added to the read-out's denominator
DELTA_UNIT_EPS = 1e-6       # inside the root of the unit norm of queries and keys


def _names(spec: PartSpec, defaults: Dict[str, str]) -> Dict[str, str]:
    names = dict(defaults)
    names.update(spec.get("names") or {})
    return names


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads, self.dim, self.vdim = int(spec.num_heads), int(spec.dim), int(spec.vdim)
        self.gate_cap = float(spec.gate_cap)
        self.eps = float(spec.get("eps", 1e-6))
        if min(self.num_heads, self.dim, self.vdim) <= 0 or not self.gate_cap > 0:
            raise ValueError("mlstm: sizes and gate_cap must be positive")
        if self.dim > 256:
            raise ValueError(f"mlstm: key size {self.dim} is beyond what the scan kernel keeps in registers (256)")
        n = _names(spec, {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "f": "f",
                          "i_bias": "i.b", "f_bias": "f.b"})
        p, H, d, dv = prefix, self.num_heads, self.dim, self.vdim
        self.main = Linear([f"{p}.{n['q']}", f"{p}.{n['k']}", f"{p}.{n['v']}", f"{p}.{n['g']}"], [H * d, H * d, H * dv, H * dv],
                           hidden_size, dtype)
        self.gates = Linear([f"{p}.{n['i']}", f"{p}.{n['f']}"], [H, H], hidden_size, dtype)
        self.o = Linear([f"{p}.{n['o']}"], [hidden_size], H * dv, dtype)
        self._vec_specs = [TensorSpec(f"{p}.{n['norm']}", (H * dv,), keep_stored_precision=True, init="ones"),
                           TensorSpec(f"{p}.{n['i_bias']}", (H,), keep_stored_precision=True, init="zeros"),
                           TensorSpec(f"{p}.{n['f_bias']}", (H,), keep_stored_precision=True, init="zeros")]
        self.gain = self.i_bias = self.f_bias = None

    def tensors(self) -> List[TensorSpec]:
        return self.main.tensors() + self.gates.tensors() + self.o.tensors() + self._vec_specs

    def load(self, store) -> None:
        for lin in (self.main, self.gates, self.o):
            lin.load(store)
        self.gain, self.i_bias, self.f_bias = (store.get(s) for s in self._vec_specs)
        if self.i_bias.dtype != self.f_bias.dtype:
            self.i_bias, self.f_bias = self.i_bias.float(), self.f_bias.float()

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.main.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    def state_need(self):
        return StateNeed((self.num_heads, self.dim * self.vdim + self.dim + 1), "float32")

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        return (self.main.workspace_bytes(tokens) + tokens * 2 * self.num_heads * 4 + tokens * self.num_heads * self.vdim * (4 + width)
                + self.o.workspace_bytes(tokens))

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        H, d, dv = self.num_heads, self.dim, self.vdim
        rows = self.main.forward(x)
        gates = self.gates.forward(x, out_dtype=torch.float32)
        q, k, v, g = rows[:, :H * d], rows[:, H * d:2 * H * d], rows[:, 2 * H * d:2 * H * d + H * dv], rows[:, 2 * H * d + H * dv:]
        o = torch.empty((rows.shape[0], H * dv), dtype=torch.float32, device=rows.device)
        kernels.mlstm_scan(q, k, v, gates, self.i_bias, self.f_bias, self.gate_cap, d ** -0.5, ctx.run_state(run),
                           ctx.query_start_loc, ctx.state_slots, o, H, d, dv, floor=MLSTM_FLOOR)
        out = torch.empty((rows.shape[0], H * dv), dtype=rows.dtype, device=rows.device)
        kernels.head_rms_gate(o, g, self.gain, self.eps, False, out, H, dv)
        return self.o.forward(out)


@MIXERS.register("gated_delta")
class GatedDelta(Mixer):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads, self.num_kv_heads = int(spec.num_heads), int(spec.num_kv_heads)
        self.dim, self.vdim, self.taps = int(spec.dim), int(spec.vdim), int(spec.taps)
        self.eps = float(spec.get("eps", 1e-6))
        if min(self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.taps) <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError("gated_delta: sizes must be positive and num_heads a multiple of num_kv_heads")
        if self.dim > 256:
            raise ValueError(f"gated_delta: key size {self.dim} is beyond what the scan kernel keeps in registers (256)")
        n = _names(spec, {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "b": "b", "a": "a",
                          "A_log": "A_log", "dt_bias": "dt_bias", "conv": "{}.conv"})
        p, H, G, d, dv = prefix, self.num_heads, self.num_kv_heads, self.dim, self.vdim
        self.channels = 2 * G * d + H * dv
        self.main = Linear([f"{p}.{n['q']}", f"{p}.{n['k']}", f"{p}.{n['v']}", f"{p}.{n['g']}"], [G * d, G * d, H * dv, H * dv],
                           hidden_size, dtype)
        self.gates = Linear([f"{p}.{n['b']}", f"{p}.{n['a']}"], [H, H], hidden_size, dtype)
        self.o = Linear([f"{p}.{n['o']}"], [hidden_size], H * dv, dtype)
        self._tap_specs = [TensorSpec(f"{p}.{n['conv'].format(n[role])}", (size, self.taps))
                           for role, size in (("q", G * d), ("k", G * d), ("v", H * dv))]
        self._vec_specs = [TensorSpec(f"{p}.{n['norm']}", (dv,), keep_stored_precision=True, init="ones"),
                           TensorSpec(f"{p}.{n['A_log']}", (H,), keep_stored_precision=True, init="zeros"),
                           TensorSpec(f"{p}.{n['dt_bias']}", (H,), keep_stored_precision=True, init="zeros")]
        self.conv_taps = self.gain = self.a_log = self.dt_bias = None

    def tensors(self) -> List[TensorSpec]:
        return self.main.tensors() + self.gates.tensors() + self.o.tensors() + self._tap_specs + self._vec_specs

    def load(self, store) -> None:
        for lin in (self.main, self.gates, self.o):
            lin.load(store)
        self.conv_taps = store.get_stacked(self._tap_specs).to(self.dtype).contiguous()
        self.gain, self.a_log, self.dt_bias = (store.get(s) for s in self._vec_specs)
        if self.a_log.dtype != self.dt_bias.dtype:
            self.a_log, self.dt_bias = self.a_log.float(), self.dt_bias.float()

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.main.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    def state_need(self):
        return (StateNeed((self.num_heads, self.dim * self.vdim), "float32", name="memory"),
                StateNeed((max(self.taps - 1, 1), self.channels), "float32", name="conv"))

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        return (self.main.workspace_bytes(tokens) + tokens * (2 * self.num_heads + self.channels) * 4
                + tokens * self.num_heads * self.vdim * (4 + width) + self.o.workspace_bytes(tokens))

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        H, G, d, dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        state = ctx.run_state(run)
        rows = self.main.forward(x)
        gates = self.gates.forward(x, out_dtype=torch.float32)
        qkv = torch.empty((rows.shape[0], self.channels), dtype=torch.float32, device=rows.device)
        kernels.delta_prep(rows, self.conv_taps, state["conv"], ctx.query_start_loc, ctx.token_request, ctx.state_slots, G, H, d, dv,
                           DELTA_UNIT_EPS, d ** -0.5, qkv)
        o = torch.empty((rows.shape[0], H * dv), dtype=torch.float32, device=rows.device)
        kernels.delta_scan(qkv, gates, self.a_log, self.dt_bias, state["memory"], ctx.query_start_loc, ctx.state_slots, o, G, H, d, dv)
        out = torch.empty((rows.shape[0], H * dv), dtype=rows.dtype, device=rows.device)
        kernels.head_rms_gate(o, rows[:, self.channels:], self.gain, self.eps, True, out, H, dv)
        return self.o.forward(out)
