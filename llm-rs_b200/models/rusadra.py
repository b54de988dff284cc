"""The Rusadra design as a ``ModelSpec``.

Every layer is an ``outnorm`` block (the branches read the residual stream, the norms sit on their outputs, a token
shift precedes the mixer) around one of two mixers, ``latent_attention`` or ``general_delta``, and an optional
mixture of experts routed by a table over token ids; the norms' weights are stored around zero; the logits are
soft-capped. A latent-attention layer with ``kv_from`` runs as a run-order entry that reads the named layer's pages,
which are then kept for the widest window among their readers.

The constants the design fixes are given to the parts here: the decay's scale exp(-1/2), the unit key's 1e-6, the
experts' sigmoid slope 1.702 and the 1 added to their up branch.
"""
from __future__ import annotations

import math

from ..config import ArchitectureEntry, register_architecture
from ..config.rusadra import LatentMixer, RusadraConfig
from ..parts import LayerSpec, ModelSpec, PartSpec, RunStep

EMBEDDING, FINAL_NORM, HEAD = "embed", "final.norm", "head"
MIXER_SCOPE, FEED_FORWARD_SCOPE, TOKEN_SHIFT = "mix.", "mlp.", "shift"
DECAY_SCALE, KEY_EPS, EXPERT_SLOPE, EXPERT_UP_SHIFT = math.exp(-0.5), 1e-6, 1.702, 1.0
# No key of the configuration bounds a sequence: windows and fixed-size state let it run on.
MAX_POSITIONS = 1 << 30


def build_spec(cfg: RusadraConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": name, "offset": 1.0})
    # The pages of a layer are kept for the widest window among the layers that read them.
    kept = {}
    for i, layer in enumerate(cfg.layers):
        if isinstance(layer.mixer, LatentMixer):
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            w = layer.mixer.window
            kept[owner] = w if owner not in kept else (0 if 0 in (w, kept[owner]) else max(w, kept[owner]))
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        cache_of = None
        if isinstance(m, LatentMixer):
            owner = i if m.kv_from is None else m.kv_from
            cache_of = m.kv_from
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "n_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "rank": m.kv_rank, "scale": m.scale, "rot_base": m.rot_base, "rot_dims": m.rot_dims,
                "window": m.window, "cache_window": kept[owner], "norm_eps": cfg.norm_eps, "gated": True,
                "shares_cache": m.kv_from is not None})
        else:
            mixer = PartSpec("general_delta", {
                "hidden_size": D, "n_heads": m.heads, "dim": m.dim, "decay_rank": m.decay_rank,
                "norm_eps": cfg.norm_eps, "key_eps": KEY_EPS, "decay_scale": DECAY_SCALE})
        ffn = None
        if layer.mlp is not None:
            f = layer.mlp
            ffn = PartSpec("moe", {"hidden_size": D, "expert_size": f.ff, "n_experts": f.experts, "top": f.top,
                                   "vocab_size": cfg.vocab, "router": "table", "limit": f.limit,
                                   "alpha": EXPERT_SLOPE, "up_shift": EXPERT_UP_SHIFT})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block=PartSpec("outnorm", {"token_shift": TOKEN_SHIFT}), mixer=mixer, feed_forward=ffn,
            mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2") if ffn is not None else None,
            mixer_scope=MIXER_SCOPE, feed_forward_scope=FEED_FORWARD_SCOPE))
        order.append(RunStep(i, cache_of=cache_of))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, layers=tuple(layers), run_order=tuple(order),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": EMBEDDING}),
        final_norm=PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": FINAL_NORM, "offset": 1.0}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": D, "name": HEAD,
                                         "softcap": cfg.logit_softcap}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(ArchitectureEntry(
    name=RusadraConfig.architecture, model_type=RusadraConfig.model_type,
    config_cls=RusadraConfig, build_spec=build_spec), replace=True)
