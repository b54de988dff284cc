"""Latent attention: all heads share one cached row per token."""
from __future__ import annotations

import os
from typing import Optional

import numpy as np
import torch

from .. import ops
from .base import Mixer, Plan, Runtime, StepInfo
from .linear import Linear
from .registry import register
from .spec import CacheNeed, WeightSpec


# Prompt portions in bfloat16 take the tensor-core kernel from this many tokens a step on; LLMRS_LATENT_MMA=0 keeps the
# CUDA-core kernel for everything.
_LATENT_MMA = os.environ.get("LLMRS_LATENT_MMA", "1") != "0"
PREFILL_MIN_TOKENS = 32


def portion_tiles(q_start, n_new, tile_tokens: int) -> np.ndarray:
    """int32 [n, 2]: (first token of the step, tokens) of tiles of at most ``tile_tokens`` consecutive tokens that do
    not cross a request."""
    firsts, counts = [], []
    for qs, n in zip(np.asarray(q_start).tolist(), np.asarray(n_new).tolist()):
        a = np.arange(0, n, tile_tokens, dtype=np.int32)
        firsts.append(qs + a)
        counts.append(np.minimum(tile_tokens, n - a))
    if not firsts:
        return np.zeros((0, 2), np.int32)
    return np.stack([np.concatenate(firsts), np.concatenate(counts)], axis=1).astype(np.int32)


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Attention whose keys and values are up-projections of a small cached latent.

    Per token the down-projection gives ``rank + rot_dim`` numbers: the first ``rank``, RMS-normed with a plain
    weight, are the latent c; the last ``rot_dim`` (rotated by position, not normed) are a key part shared by all
    heads. Only these are cached. A query head is [``dim`` unrotated | ``rot_dim`` rotated]; head h's unrotated key
    is ``W_uk,h c`` and its value ``W_uv,h c``. The score is ``(q_n . k_n + q_r . k_r) * scale`` over the causal keys
    (the last ``window`` of them when ``window`` > 0), ordinary softmax; head h's output is multiplied by
    ``sigmoid(W_g x)_h`` when ``gated``; then the output projection.

    Computed in the folded form: ``qa_h = W_uk,h^T q_n,h`` (a batched product), attention over the cached rows with
    values c, then ``W_uv,h`` on the result (a batched product): the cache is read once for all heads and no key or
    value is ever materialised. The rotation pairs entry i of the rotated part with entry i + rot_dims/2 for the first
    ``rot_dims`` entries, angle ``position * rot_base^(-2i/rot_dims)``.

    A layer with ``shares_cache`` has no down-projection: its run-order entry reads another entry's pages
    (``RunStep.cache_of``) with its own up-projections, queries and window. ``cache_window`` is the window the pages
    are kept for (the widest window of the layers that read them; default: this layer's).

    ``names`` maps the roles q, dkv, dkv_norm, uk, uv, g, o to tensor names after the prefix.
    """
    ROLES = ("q", "dkv", "dkv_norm", "uk", "uv", "g", "o")

    def __init__(self, hidden_size: int, n_heads: int, dim: int, rot_dim: int, vdim: int, rank: int, scale: float,
                 rot_base: float, rot_dims: Optional[int] = None, window: int = 0, cache_window: Optional[int] = None,
                 norm_eps: float = 1e-6, gated: bool = True, shares_cache: bool = False, names=None,
                 prefix: str = ""):
        self.hidden_size, self.n_heads, self.dim, self.rot_dim, self.vdim = hidden_size, n_heads, dim, rot_dim, vdim
        self.rank, self.scale, self.rot_base = rank, float(scale), float(rot_base)
        self.rot_dims = rot_dim if rot_dims is None else int(rot_dims)
        if self.rot_dims % 2 or not 0 <= self.rot_dims <= rot_dim:
            raise ValueError(f"{self.rot_dims} rotated dimensions of a rotated part of {rot_dim}")
        if rank > 512:
            raise ValueError(f"a latent of {rank}: the attention kernel takes at most 512")
        self.window = int(window)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window and (self.window == 0 or self.window > self.cache_window):
            raise ValueError(f"pages kept for the last {self.cache_window} keys cannot serve a window of "
                             f"{self.window or 'all'} keys")
        self.norm_eps, self.gated, self.shares_cache = float(norm_eps), bool(gated), bool(shares_cache)
        self.prefix = prefix
        self.names = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "g": "g", "o": "o"}
        self.names.update(names or {})
        if set(self.names) != set(self.ROLES):
            raise ValueError(f"names may rename {self.ROLES}, got {sorted(set(self.names) - set(self.ROLES))}")
        self.q_width = n_heads * (dim + rot_dim)
        self._tile = None

    def _name(self, role: str) -> str:
        return self.prefix + self.names[role]

    def weight_specs(self):
        H, nh, nm = self.hidden_size, self.n_heads, self._name
        specs = [WeightSpec(nm("q"), (self.q_width, H)), WeightSpec(nm("uk"), (nh * self.dim, self.rank)),
                 WeightSpec(nm("uv"), (nh * self.vdim, self.rank)), WeightSpec(nm("o"), (H, nh * self.vdim))]
        if self.gated:
            specs.append(WeightSpec(nm("g"), (nh, H)))
        if not self.shares_cache:
            specs += [WeightSpec(nm("dkv"), (self.rank + self.rot_dim, H)),
                      WeightSpec(nm("dkv_norm"), (self.rank,), role="norm")]
        return specs

    def bind(self, tensors, runtime: Runtime):
        nm, nh = self._name, self.n_heads
        self.act_dtype = runtime.act_dtype
        ws = [tensors[nm("q")]]
        if self.gated:
            ws.append(tensors[nm("g")])
        if not self.shares_cache:
            ws.append(tensors[nm("dkv")])
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        # One product for the queries, the gates and the down-projection: they read the same input.
        self.in_proj = Linear(torch.cat([w.to(dt) for w in ws], dim=0).contiguous(), None, runtime.act_dtype)
        self.o_proj = Linear(tensors[nm("o")], None, runtime.act_dtype)
        # W_uk,h transposed to [rank, dim]: the folded query is an ordinary product with it.
        self.w_uk_t = tensors[nm("uk")].view(nh, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[nm("uv")].view(nh, self.vdim, self.rank).contiguous()
        self.latent_norm_w = None if self.shares_cache else tensors[nm("dkv_norm")].to(torch.float32).contiguous()
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.inv_freq = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).to(runtime.device)

    def cache_need(self):
        if self.shares_cache:
            return None
        return CacheNeed("window" if self.cache_window > 0 else "full", 1, self.rank, self.cache_window,
                         planes=(self.rank, self.rot_dim))

    # -- the step's plan: tiles of a prompt's tokens for the tensor-core kernel -------------------------------------
    def _tile_tokens(self) -> int:
        if self._tile is None:      # asked of the kernel library at first use: constructing a part needs no library
            self._tile = ops.latent_prefill_tile_tokens(self.n_heads)
        return self._tile

    def plan_key(self):
        return ("latent_attention_tiles", self._tile_tokens())

    def plan(self, step: StepInfo) -> Plan:
        """Steps that bring a prompt's portion are cut into tiles of tokens (none for steps of single tokens, which
        the CUDA-core kernel takes with its keys cut over blocks, and which may be replayed from a graph)."""
        if step.for_graph or step.n_tokens < PREFILL_MIN_TOKENS or int(np.max(step.n_new, initial=0)) <= 1:
            return Plan(arrays={"tiles": np.zeros((0, 2), np.int32)}, values={"n_tiles": 0})
        tiles = portion_tiles(step.q_start, step.n_new, self._tile_tokens())
        return Plan(arrays={"tiles": tiles}, values={"n_tiles": int(tiles.shape[0])})

    def _tiles(self, ctx):
        """(device tiles, how many) for this step; None when the step has no plan of them."""
        if hasattr(ctx, "plan"):
            view = ctx.plan(self.plan_key())
            return (view.arrays["tiles"], view.values["n_tiles"]) if view.values["n_tiles"] else None
        # Called outside the step function (a part alone): plan here, from the device's arrays.
        n_new = ctx.n_new.cpu().numpy()
        if ctx.n_tokens < PREFILL_MIN_TOKENS or int(n_new.max(initial=0)) <= 1:
            return None
        tiles = portion_tiles(ctx.q_start.cpu().numpy(), n_new, self._tile_tokens())
        return torch.from_numpy(tiles).to(ctx.n_new.device), int(tiles.shape[0])

    def forward(self, x, ctx, cache):
        nh, dn, dr, rank = self.n_heads, self.dim, self.rot_dim, self.rank
        if cache.owns == self.shares_cache:
            raise RuntimeError("a latent attention layer that shares a cache must run as an entry with cache_of "
                               "(and one that owns its cache must not)")
        T = ctx.n_tokens
        proj = self.in_proj.forward(x)
        q = proj[:, : self.q_width]
        at = self.q_width
        if self.gated:
            gate = proj[:, at: at + nh]
            at += nh
        else:       # sigmoid(+large) = 1
            gate = torch.full((T, nh), 30.0, dtype=proj.dtype, device=proj.device)
        dkv = None if self.shares_cache else proj[:, at: at + rank + dr]
        pages = self._pages(cache)
        ops.latent_prepare(q, dkv, self.latent_norm_w, self.inv_freq, ctx, cache.block_table,
                           None if self.shares_cache else pages, cache.page_size, nh, dn, dr, self.rot_dims, rank,
                           self.norm_eps)
        q3 = q.unflatten(1, (nh, dn + dr))
        qa = torch.empty((T, nh, rank), dtype=proj.dtype, device=proj.device)
        ops.gemm_batched(q3[:, :, :dn], self.w_uk_t, qa)
        lat = torch.empty((T, nh, rank), dtype=proj.dtype, device=proj.device)
        tiles = self._tiles(ctx) if _LATENT_MMA and proj.dtype == torch.bfloat16 else None
        if tiles is not None and ops.latent_attention_prefill(
                qa, q, gate, pages, cache.block_table, ctx, tiles[0], tiles[1], lat, nh, dn, dr, rank, cache.page_size,
                self.window, self.scale):
            out = torch.empty((T, nh, self.vdim), dtype=proj.dtype, device=proj.device)
            ops.gemm_batched(lat, self.w_uv, out)
            return self.o_proj.forward(out.view(T, nh * self.vdim))
        # Steps of few tokens cut the visible keys over several blocks. The span is what the step's shape implies (the
        # window, else what the block table can hold), not the requests' lengths: a captured step replays it.
        span = self.window if self.window > 0 else cache.block_table.size(1) * cache.page_size
        splits, split_keys = ops.latent_attention_splits(T, nh, span, ops.sm_count(proj.device))
        ops.latent_attention(qa, q, gate, pages, cache.block_table, ctx, lat, nh, dn, dr, rank, cache.page_size,
                             self.window, self.scale, splits=splits, split_keys=split_keys)
        out = torch.empty((T, nh, self.vdim), dtype=proj.dtype, device=proj.device)
        ops.gemm_batched(lat, self.w_uv, out)
        return self.o_proj.forward(out.view(T, nh * self.vdim))

    @staticmethod
    def _pages(cache):
        """The entry's pages as one tensor [pages, page_size * (rank + rot_dim)]: plane 0 (the latents) and plane 1
        (the rotated key parts) of a page follow one another."""
        p0 = cache.planes[0]
        return p0.as_strided((p0.size(0), p0.stride(0)), (p0.stride(0), 1), p0.storage_offset())
