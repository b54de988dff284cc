"""The Pusazen design as a ``ModelSpec``.

Every layer is a ``postnorm`` block (``h = norm(alpha * h + ls * branch(h))``, the branches read the stream itself)
around one of three mixers: ``mlstm`` (a matrix memory with exponential gates), ``lightning`` (linear attention with
a fixed decay per head) or ``scored_attention`` (grouped heads, norms over the whole q and k rows, partial rotation,
capped scores, a chunked mask, a sink); the feed-forward is dense with a squared relu, a mixture of experts with a
learned router, softmax over the chosen logits and a gated shared expert, or absent. The logits are scaled.

The constants the design fixes are given to the parts here: the matrix memory's query scale dim^-1/2 and the 1e-6 in
its denominator, the experts' plain SiLU unit, the squared relu.
"""
from __future__ import annotations

from ..config import ArchitectureEntry, register_architecture
from ..config.pusazen import AttentionMixer, DenseMLP, LightningMixer, MatrixMemoryMixer, PusazenConfig
from ..parts import LayerSpec, ModelSpec, PartSpec, RunStep

EMBEDDING, FINAL_NORM, HEAD = "embed", "final.norm", "head"
MIXER_SCOPE, FEED_FORWARD_SCOPE = "mix.", "mlp."
LAYER_SCALES = ("ls1", "ls2")
MEMORY_DEN_EPS = 1e-6
GATE_NAMES = {"i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b"}
# No key of the configuration bounds a sequence; a layer that keeps every key bounds it by the pool.
MAX_POSITIONS = 1 << 30


def build_spec(cfg: PusazenConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": name})
    layers, order = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, MatrixMemoryMixer):
            mixer = PartSpec("mlstm", {"hidden_size": D, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                       "gate_cap": m.gate_cap, "norm_eps": cfg.norm_eps, "den_eps": MEMORY_DEN_EPS,
                                       "q_scale": m.dim ** -0.5, "names": GATE_NAMES})
        elif isinstance(m, LightningMixer):
            mixer = PartSpec("lightning", {"hidden_size": D, "n_heads": m.heads, "dim": m.dim, "vdim": m.vdim,
                                           "decay": m.decay, "norm_eps": cfg.norm_eps, "activation": "silu"})
        else:
            assert isinstance(m, AttentionMixer)
            mixer = PartSpec("scored_attention", {
                "hidden_size": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                "scale": m.scale, "softcap": m.softcap, "sink": m.sink, "mask": "chunk" if m.chunk else "causal",
                "mask_size": m.chunk, "qk_norm": "whole", "norm_eps": cfg.norm_eps, "rot_dims": m.rot_dims,
                "rot_base": m.rot_base})
        f, ffn = layer.mlp, None
        if isinstance(f, DenseMLP):
            ffn = PartSpec("dense", {"hidden_size": D, "intermediate_size": f.ff, "activation": "relu_sq"})
        elif f is not None:
            ffn = PartSpec("moe", {"hidden_size": D, "expert_size": f.ff, "n_experts": f.experts, "top": f.top,
                                   "router": "linear", "limit": None, "alpha": 1.0, "up_shift": 0.0,
                                   "shared_size": f.shared_ff, "shared_gated": True})
        second = ffn is not None or layer.lone_norm
        layers.append(LayerSpec(
            prefix=f"l{i}.",
            block=PartSpec("postnorm", {"alpha": cfg.alpha, "layer_scale": LAYER_SCALES if layer.layer_scale else (),
                                        "lone_norm": layer.lone_norm}),
            mixer=mixer, feed_forward=ffn, mixer_norm=norm("norm1"),
            feed_forward_norm=norm("norm2") if second else None,
            mixer_scope=MIXER_SCOPE, feed_forward_scope=FEED_FORWARD_SCOPE))
        order.append(RunStep(i))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, layers=tuple(layers), run_order=tuple(order),
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "name": EMBEDDING}),
        final_norm=PartSpec("rmsnorm", {"dim": D, "eps": cfg.norm_eps, "name": FINAL_NORM}),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": D, "name": HEAD,
                                         "scale": cfg.logit_scale}),
        max_positions=MAX_POSITIONS, eos_token_ids=())


register_architecture(ArchitectureEntry(
    name=PusazenConfig.architecture, model_type=PusazenConfig.model_type,
    config_cls=PusazenConfig, build_spec=build_spec), replace=True)
