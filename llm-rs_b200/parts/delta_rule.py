"""The generalized delta rule, a recurrent mixer with a matrix state per head."""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import Mixer, Runtime
from .linear import Linear
from .registry import register
from .spec import StateNeed, WeightSpec


@register("mixer", "general_delta")
class GeneralDelta(Mixer):
    """Per head a state S [key channel, value channel] (float32, zero at a sequence's start, kept per request):

        S_t = diag(w_t) S_{t-1} - (a_t * u_t) (u_t^T S_{t-1}) + k_t v_t^T,      o_t = S_t^T r_t

    with r, k, v projections of the input (``n_heads`` x ``dim``), the unit key ``u = k / sqrt(sum(k^2) + key_eps)``,
    the decay ``w = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 x) + w0))`` and the removal rate
    ``a = sigmoid(W_a x + a_bias)``, both per head and key channel. Each head's o is divided by its root mean square
    (``norm_eps``), the heads are concatenated, multiplied by a plain weight and by ``sigmoid(W_g x)``, then the
    output projection. Decay, removal rate, unit key, state and the norm are float32; the projections run in the
    activation type. ``decay_scale`` defaults to exp(-1/2).

    r, k, v, g, a and the first decay projection read the same input and are one product. No pages: the mixer asks for
    fixed-size state only, so its cost per token does not grow with the sequence.

    ``names`` maps the roles r, k, v, g, a, a_bias, w1, w2, w0, norm, o to tensor names after the prefix.
    """
    ROLES = ("r", "k", "v", "g", "a", "a_bias", "w1", "w2", "w0", "norm", "o")
    STATE = "delta.state"

    def __init__(self, hidden_size: int, n_heads: int, dim: int, decay_rank: int, norm_eps: float = 1e-6,
                 key_eps: float = 1e-6, decay_scale: float = math.exp(-0.5), names=None, prefix: str = ""):
        if dim > 256:
            raise ValueError(f"heads of {dim} channels: the recurrence kernel takes at most 256")
        self.hidden_size, self.n_heads, self.dim, self.decay_rank = hidden_size, n_heads, dim, decay_rank
        self.norm_eps, self.key_eps, self.decay_scale = float(norm_eps), float(key_eps), float(decay_scale)
        self.prefix = prefix
        self.names = {"r": "r", "k": "k", "v": "v", "g": "g", "a": "a", "a_bias": "a.b", "w1": "w1", "w2": "w2",
                      "w0": "w0", "norm": "norm", "o": "o"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.width = n_heads * dim

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, W, nm = self.hidden_size, self.width, self._name
        return [WeightSpec(nm(r), (W, H)) for r in ("r", "k", "v", "g", "a")] + [
            WeightSpec(nm("a_bias"), (W,), role="bias"), WeightSpec(nm("w1"), (self.decay_rank, H)),
            WeightSpec(nm("w2"), (W, self.decay_rank)), WeightSpec(nm("w0"), (W,), role="bias"),
            WeightSpec(nm("norm"), (W,), role="norm"), WeightSpec(nm("o"), (H, W))]

    def bind(self, tensors, runtime: Runtime):
        nm = self._name
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm(r)] for r in ("r", "k", "v", "g", "a", "w1")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.decay_proj = Linear(tensors[nm("w2")], None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        f32 = lambda role: tensors[nm(role)].to(torch.float32).contiguous()
        self.a_bias, self.decay_bias, self.norm_w = f32("a_bias"), f32("w0"), f32("norm")

    def state_need(self):
        return StateNeed({self.STATE: (self.n_heads, self.dim, self.dim)})

    def forward(self, x, ctx, cache):
        W = self.width
        proj = self.in_proj.forward(x)
        r, k, v, g, a = (proj[:, i * W:(i + 1) * W] for i in range(5))
        hidden = ops.tanh_slice(proj[:, 5 * W: 5 * W + self.decay_rank], self.act_dtype)
        decay_raw = self.decay_proj.forward(hidden, out_dtype=torch.float32)
        out = ops.delta_rule(r, k, v, g, a, decay_raw, self.decay_bias, self.a_bias, self.norm_w,
                             cache.state[self.STATE], ctx, self.n_heads, self.dim, self.decay_scale, self.key_eps,
                             self.norm_eps)
        return self.o_proj.forward(out)
