"""Typed configuration of the Rusadra design, read from its own config.json keys.

A Rusadra model is a list of layers, each with one of two mixers and an optional mixture-of-experts feed-forward:

    {"architecture": "Rusadra", "vocab": V, "width": D, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "latent_attention" | "general_delta", "mixer": {...}, "mlp": {...} | null}, ...]}

    latent_attention mixer: heads, dim, rot_dim, vdim, kv_rank, scale, mask.size, rot.base, rot.dims,
                            kv_from (optional: the layer whose cached rows this layer reads)
    general_delta mixer:    heads, dim          (the rank of the decay projection is the shape of its tensor)
    mlp:                    kind "moe", expert.ff, expert.limit, router.experts, router.top

Every size and constant that may differ between models comes from here or from a tensor's shape; constants that the
design fixes live with the parts (``models/rusadra.py`` passes them as parameters).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError

MIXERS = ("latent_attention", "general_delta")


def _get(raw: Mapping, path: str, kind, where: str, minimum=None, optional=False):
    node: Any = raw
    for key in path.split("."):
        if not isinstance(node, Mapping) or key not in node:
            if optional:
                return None
            raise ConfigError(f"{where}: {path} missing from config")
        node = node[key]
    if isinstance(node, bool) or not isinstance(node, (int, float) if kind is float else kind):
        raise ConfigError(f"{where}: {path} must be {'a number' if kind is float else 'an integer'}, got {node!r}")
    if minimum is not None and node < minimum:
        raise ConfigError(f"{where}: {path} must be >= {minimum}, got {node}")
    return kind(node)


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int          # mask.size: a token sees itself and the window - 1 before it; 0 (no mask key): all before it
    rot_base: float
    rot_dims: int
    kv_from: Optional[int] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
             "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class DeltaMixer:
    heads: int
    dim: int
    decay_rank: int      # rows of the first decay projection; read from the tensor when config.json has no such key

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "decay_rank": self.decay_rank}


@dataclass(frozen=True)
class MoE:
    ff: int
    limit: float
    experts: int
    top: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class RusadraLayer:
    type: str
    mixer: Any
    mlp: Optional[MoE]


@dataclass(frozen=True)
class RusadraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RusadraLayer, ...]
    logit_softcap: float = 0.0
    torch_dtype: str = "bfloat16"

    architecture = "Rusadra"
    model_type = "rusadra"
    wants_tensor_shapes = True      # ``load_config`` passes the folder's tensor shapes to ``from_dict``

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], tensor_shapes: Optional[Mapping[str, Tuple[int, ...]]] = None):
        vocab = _get(raw, "vocab", int, "config", 1)
        width = _get(raw, "width", int, "config", 1)
        eps = _get(raw, "norm.eps", float, "config", 0.0)
        cap = _get(raw, "logit_softcap", float, "config", 0.0, optional=True) or 0.0
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config: layers must be a non-empty list")
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in MIXERS:
                raise ConfigError(f"{where}: type must be one of {MIXERS}, got {lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            m = lr.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}: mixer missing from config")
            if lr["type"] == "latent_attention":
                kv_from = _get(m, "kv_from", int, where, 0, optional=True)
                mixer = LatentMixer(
                    heads=_get(m, "heads", int, where, 1), dim=_get(m, "dim", int, where, 1),
                    rot_dim=_get(m, "rot_dim", int, where, 2), vdim=_get(m, "vdim", int, where, 1),
                    kv_rank=_get(m, "kv_rank", int, where, 1), scale=_get(m, "scale", float, where),
                    window=_get(m, "mask.size", int, where, 1, optional=True) or 0, rot_base=_get(m, "rot.base", float, where),
                    rot_dims=_get(m, "rot.dims", int, where, 0), kv_from=kv_from)
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"{where}: rot.dims {mixer.rot_dims} must be even and at most rot_dim {mixer.rot_dim}")
                if kv_from is not None:
                    if kv_from >= i or not isinstance(layers[kv_from].mixer, LatentMixer) \
                            or layers[kv_from].mixer.kv_from is not None:
                        raise ConfigError(f"{where}: kv_from {kv_from} must name an earlier latent_attention layer "
                                          f"that has a down-projection of its own")
                    src = layers[kv_from].mixer
                    if (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != (
                            mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                        raise ConfigError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {kv_from}")
            else:
                rank = _get(m, "decay_rank", int, where, 1, optional=True)
                if rank is None:
                    shape = (tensor_shapes or {}).get(f"l{i}.mix.w1")
                    if shape is None or len(shape) != 2:
                        raise ConfigError(f"{where}: the decay projection's rank is neither in the config "
                                          f"(mixer.decay_rank) nor given by the shape of l{i}.mix.w1")
                    rank = int(shape[0])
                mixer = DeltaMixer(heads=_get(m, "heads", int, where, 1), dim=_get(m, "dim", int, where, 1),
                                   decay_rank=rank)
            mlp_raw = lr.get("mlp")
            mlp = None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, Mapping) or mlp_raw.get("kind") != "moe":
                    raise ConfigError(f"{where}: mlp.kind must be 'moe' (or mlp null)")
                mlp = MoE(ff=_get(mlp_raw, "expert.ff", int, where, 1), limit=_get(mlp_raw, "expert.limit", float, where),
                          experts=_get(mlp_raw, "router.experts", int, where, 1),
                          top=_get(mlp_raw, "router.top", int, where, 1))
                if mlp.top > mlp.experts:
                    raise ConfigError(f"{where}: router.top {mlp.top} exceeds router.experts {mlp.experts}")
            layers.append(RusadraLayer(lr["type"], mixer, mlp))
        return cls(vocab=vocab, width=width, norm_eps=eps, layers=tuple(layers), logit_softcap=cap,
                   torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": l.mixer.to_dict(), "mlp": None if l.mlp is None else l.mlp.to_dict()}
                       for l in self.layers]}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out
