"""Recurrent mixers with a matrix state per head: a matrix memory with exponential gates, and linear attention with
a fixed decay per head. Both are ``S_t = a_t S_(t-1) + b_t k_t v_t^T``, ``o_t = S_t^T q_t`` (``csrc/linear_recurrence.cu``)
and differ in where a_t and b_t come from, in a normaliser and in the output's norm."""
from __future__ import annotations

from typing import Sequence

import torch

from .. import ops
from .base import Mixer, Runtime
from .linear import Linear
from .registry import register
from .spec import StateNeed, WeightSpec


class _MatrixStateMixer(Mixer):
    """What the two mixers share: the q|k|v|g product, the output projection, names, the state's shape."""
    ROLES: Sequence[str] = ()
    STATE = "recurrent.state"

    def __init__(self, hidden_size: int, n_heads: int, dim: int, vdim: int, norm_eps: float, names=None,
                 prefix: str = ""):
        if dim > 256:
            raise ValueError(f"heads of {dim} key channels: the recurrence kernel takes at most 256")
        self.hidden_size, self.n_heads, self.dim, self.vdim = hidden_size, n_heads, dim, vdim
        self.norm_eps, self.prefix = float(norm_eps), prefix
        self.names = {role: role for role in self.ROLES}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.k_width, self.v_width = n_heads * dim, n_heads * vdim

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def _common_specs(self):
        H, nm = self.hidden_size, self._name
        return [WeightSpec(nm("q"), (self.k_width, H)), WeightSpec(nm("k"), (self.k_width, H)),
                WeightSpec(nm("v"), (self.v_width, H)), WeightSpec(nm("g"), (self.v_width, H)),
                WeightSpec(nm("o"), (H, self.v_width)), WeightSpec(nm("norm"), (self.v_width,), role="norm")]

    def _bind_common(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in ("q", "k", "v", "g")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        self.norm_w = tensors[nm("norm")].to(torch.float32).contiguous()

    def _split(self, proj):
        K, V = self.k_width, self.v_width
        return proj[:, :K], proj[:, K:2 * K], proj[:, 2 * K:2 * K + V], proj[:, 2 * K + V:2 * K + 2 * V]


@register("mixer", "mlstm")
class MatrixMemory(_MatrixStateMixer):
    """Matrix memory with exponential gates (mLSTM). Per head, with q = W_q x * q_scale (default dim^-1/2), k, v, a log
    input gate ``i = cap * tanh((W_i x + b_i) / cap)`` and a log forget gate
    ``f = logsigmoid(cap * tanh((W_f x + b_f) / cap))``:

        m_t = max(f + m_(t-1), i)                      (m starts at ``m_start``, 0 by default, not at -inf)
        S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T,     n_t likewise with k alone
        o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + den_eps)

    then each head's o is divided by its root mean square (``norm_eps``), the heads are concatenated, multiplied by a
    weight and by sigmoid(W_g x), and projected. The gates' pre-activations are a float32 product; gates, m, S and n
    are float32, kept per request slot. ``names`` maps the roles q, k, v, g, o, norm, i, i_bias, f, f_bias to tensor
    names after the prefix."""
    ROLES = ("q", "k", "v", "g", "o", "norm", "i", "i_bias", "f", "f_bias")
    NORMALISER, MAXIMUM = "recurrent.normaliser", "recurrent.maximum"

    def __init__(self, hidden_size: int, n_heads: int, dim: int, vdim: int, gate_cap: float, norm_eps: float = 1e-6,
                 den_eps: float = 1e-6, q_scale=None, names=None, prefix: str = ""):
        super().__init__(hidden_size, n_heads, dim, vdim, norm_eps, names, prefix)
        self.gate_cap, self.den_eps = float(gate_cap), float(den_eps)
        self.q_scale = float(q_scale) if q_scale is not None else dim ** -0.5

    def weight_specs(self):
        H, nm, nh = self.hidden_size, self._name, self.n_heads
        return self._common_specs() + [
            WeightSpec(nm("i"), (nh, H)), WeightSpec(nm("i_bias"), (nh,), role="bias"),
            WeightSpec(nm("f"), (nh, H)), WeightSpec(nm("f_bias"), (nh,), role="bias")]

    def bind(self, tensors, runtime: Runtime):
        self._bind_common(tensors, runtime)
        nm = self._name
        f32 = lambda role: tensors[nm(role)].to(torch.float32)
        # The gates' product is float32 whatever the activation type: what enters the recurrence is not rounded.
        self.gate_w = torch.cat([f32("i"), f32("f")], dim=0).contiguous()
        self.gate_b = torch.cat([f32("i_bias"), f32("f_bias")], dim=0).contiguous()
        stored = [tensors[nm("i")], tensors[nm("f")]]       # as the folder stores them (see ``ops.product_f32``)
        self.gate_w_stored = torch.cat(stored, dim=0).contiguous() if stored[0].dtype == stored[1].dtype else self.gate_w

    def state_need(self):
        return StateNeed({self.STATE: (self.n_heads, self.dim, self.vdim), self.NORMALISER: (self.n_heads, self.dim),
                          self.MAXIMUM: (self.n_heads,)})

    def forward(self, x, ctx, cache):
        q, k, v, g = self._split(self.in_proj.forward(x))
        gates = ops.product_f32(x, self.gate_w_stored, self.gate_w, self.gate_b)
        decay, gain, floor = ops.gate_scan(gates, self.gate_cap, cache.state[self.MAXIMUM], ctx, self.n_heads)
        out = ops.linear_recurrence(q, k, v, g, self.norm_w, cache.state[self.STATE], ctx, self.n_heads, self.dim,
                                    self.vdim, self.norm_eps, q_scale=self.q_scale, decay=decay, gain=gain,
                                    normaliser=cache.state[self.NORMALISER], floor=floor, den_eps=self.den_eps,
                                    per_head_norm=True)
        return self.o_proj.forward(out)


@register("mixer", "lightning")
class LightningAttention(_MatrixStateMixer):
    """Linear attention with one fixed decay per head: q, k, v = act(W x) (``activation`` "silu" or "none"),
    ``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with no other scale; the concatenated heads are divided
    by their common root mean square (``norm_eps``), multiplied by a weight and by sigmoid(W_g x), and projected.
    The state is float32, kept per request slot. ``names`` maps the roles q, k, v, g, o, norm."""
    ROLES = ("q", "k", "v", "g", "o", "norm")

    def __init__(self, hidden_size: int, n_heads: int, dim: int, vdim: int, decay: Sequence[float],
                 norm_eps: float = 1e-6, activation: str = "silu", names=None, prefix: str = ""):
        super().__init__(hidden_size, n_heads, dim, vdim, norm_eps, names, prefix)
        if len(decay) != n_heads:
            raise ValueError(f"{len(decay)} decays for {n_heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"unknown activation {activation!r}; known: 'silu', 'none'")
        self.decay, self.activation = [float(d) for d in decay], activation

    def weight_specs(self):
        return self._common_specs()

    def bind(self, tensors, runtime: Runtime):
        self._bind_common(tensors, runtime)
        self.head_decay = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def state_need(self):
        return StateNeed({self.STATE: (self.n_heads, self.dim, self.vdim)})

    def forward(self, x, ctx, cache):
        q, k, v, g = self._split(self.in_proj.forward(x))
        out = ops.linear_recurrence(q, k, v, g, self.norm_w, cache.state[self.STATE], ctx, self.n_heads, self.dim,
                                    self.vdim, self.norm_eps, act_silu=self.activation == "silu",
                                    head_decay=self.head_decay, per_head_norm=False)
        return self.o_proj.forward(out)
