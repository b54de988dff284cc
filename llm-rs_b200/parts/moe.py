"""Mixtures of experts."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, Runtime
from .registry import register
from .spec import WeightSpec


@register("feed_forward", "moe")
class MixtureOfExperts(FeedForward):
    """``experts`` small gated feed-forward layers of which every token uses ``top``; the output is the weighted sum
    of the chosen experts' outputs.

    Expert (no biases): ``g = min(W_gate x, limit)``, ``u = clamp(W_up x, -limit, limit)``,
    ``y = g * sigmoid(alpha * g) * (u + up_shift)``, output ``W_down y``; ``limit``, ``alpha`` and ``up_shift`` are
    parameters.

    Router ``"table"``: no learned router; an integer table [vocab, top] names each token id's experts (the entries
    of a row differ), each weighted 1/top. The router only fills (expert, weight) per assignment on the device; the
    grouping of rows by expert, the two grouped products and the weighted sum do not depend on which router ran.

    The rows are sorted by expert so that a tile of rows shares one expert's weights; the first product has the gated
    unit as its epilogue; bfloat16 products run on the tensor cores (``csrc/gemm_grouped.cu``). ``forward`` takes the
    float32 residual stream itself (``reads_residual``) and rounds its rows to the activation type. Tensor names: ``<prefix>e<i>.gate|up|down`` and
    ``<prefix>table`` unless ``names`` renames the roles."""

    reads_residual = True
    ROLES = ("expert", "gate", "up", "down", "table")

    def __init__(self, hidden_size: int, expert_size: int, n_experts: int, top: int, vocab_size: int = 0,
                 router: str = "table", limit: float = 1.0, alpha: float = 1.702, up_shift: float = 1.0,
                 names=None, prefix: str = ""):
        if router != "table":
            raise ValueError(f"unknown router {router!r}; known: 'table'")
        if not 1 <= top <= n_experts:
            raise ValueError(f"top {top} of {n_experts} experts")
        if router == "table" and vocab_size < 1:
            raise ValueError("the table router needs the vocabulary's size")
        self.hidden_size, self.expert_size, self.n_experts, self.top = hidden_size, expert_size, n_experts, top
        self.vocab_size, self.router = vocab_size, router
        self.limit, self.alpha, self.up_shift = float(limit), float(alpha), float(up_shift)
        self.prefix = prefix
        self.names = {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")

    def _name(self, e: int, role: str) -> str:
        return f"{self.prefix}{self.names['expert'].format(e)}{self.names[role]}"

    def weight_specs(self):
        H, F = self.hidden_size, self.expert_size
        specs = []
        for e in range(self.n_experts):
            specs += [WeightSpec(self._name(e, "gate"), (F, H)), WeightSpec(self._name(e, "up"), (F, H)),
                      WeightSpec(self._name(e, "down"), (H, F))]
        specs.append(WeightSpec(self.prefix + self.names["table"], (self.vocab_size, self.top), role="expert_table",
                                limit=self.n_experts))
        return specs

    def bind(self, tensors, runtime: Runtime):
        self.act_dtype = runtime.act_dtype
        stack = lambda role: torch.stack([tensors[self._name(e, role)] for e in range(self.n_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        if len({self.w_gate.dtype, self.w_up.dtype, self.w_down.dtype}) != 1:
            self.w_gate, self.w_up, self.w_down = (w.to(torch.float32) for w in (self.w_gate, self.w_up, self.w_down))
        self.table = tensors[self.prefix + self.names["table"]].contiguous()
        bad = (self.table < 0) | (self.table >= self.n_experts)
        if bool(bad.any()):
            raise ValueError(f"{self.prefix}{self.names['table']} names experts outside 0..{self.n_experts - 1}")

    def forward(self, x, ctx):
        """x: the step's rows, float32 (the residual stream) or the activation type. Returns float32 [tokens, hidden]."""
        expert_of, weight_of = ops.moe_route_table(ctx.token_ids, self.table, self.n_experts)
        n_rows = expert_of.numel()
        tile_rows = ops.grouped_tile_rows(n_rows, self.n_experts)
        row_of, src_token, tiles, n_tiles = ops.moe_sort(expert_of, self.top, self.n_experts, tile_rows)
        if self.act_dtype == torch.bfloat16 and x.dtype == torch.float32:
            x = ops.token_shift(x, None, None, None, torch.bfloat16)     # the rows as activations: the tensor cores' type
        act = torch.empty((n_rows, self.expert_size), dtype=self.act_dtype, device=x.device)
        ops.gemm_grouped(x, self.w_gate, act, tiles, n_tiles, src_token, w2=self.w_up, limit=self.limit,
                         alpha=self.alpha, shift=self.up_shift, tile_rows=tile_rows)
        rows = torch.empty((n_rows, self.hidden_size), dtype=torch.float32, device=x.device)
        ops.gemm_grouped(act, self.w_down, rows, tiles, n_tiles, None, tile_rows=tile_rows)
        return ops.moe_combine(rows, row_of, weight_of, self.top)
