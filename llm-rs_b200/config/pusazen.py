"""Typed configuration of the Pusazen design, read from its own config.json keys.

A Pusazen model is a list of layers, each with one of three mixers and a dense or mixture-of-experts feed-forward
(or none); the norm of a layer comes after the residual sum:

    {"architecture": "Pusazen", "vocab": V, "width": D, "norm": {"eps": e}, "postln_alpha": a, "logit_scale": s,
     "layers": [{"type": "mlstm" | "lightning" | "attention", "mixer": {...}, "mlp": {...} | null}, ...]}

    mlstm mixer:      heads, dim, vdim, gate_cap
    lightning mixer:  heads, dim, vdim, decay (one number per head)
    attention mixer:  heads, kv_heads, dim, vdim, scale, softcap (optional), mask.size (optional: chunks of that many
                      positions), rot.base, rot.dims (optional)
    mlp:              kind "dense": ff
                      kind "moe":   expert.ff, router.experts, router.top, shared.ff (optional)

Every size and constant that may differ between models comes from here; whether a layer has layer-scale vectors, a
sink, or a second norm without a feed-forward is read from which tensors the folder holds. Constants the design fixes
live with the parts (``models/pusazen.py`` passes them as parameters).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .rusadra import _get

MIXERS = ("mlstm", "lightning", "attention")


@dataclass(frozen=True)
class MatrixMemoryMixer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "gate_cap": self.gate_cap}


@dataclass(frozen=True)
class LightningMixer:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float       # 0: scores are not capped
    chunk: int           # mask.size; 0 (no mask key): every earlier token is seen
    rot_base: float
    rot_dims: int        # 0: no rotation
    sink: bool = True

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.softcap:
            d["softcap"] = self.softcap
        if self.chunk:
            d["mask"] = {"size": self.chunk}
        if self.rot_dims:
            d["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
        return d


@dataclass(frozen=True)
class DenseMLP:
    ff: int

    def to_dict(self) -> Dict[str, Any]:
        return {"kind": "dense", "ff": self.ff}


@dataclass(frozen=True)
class MoEMLP:
    ff: int
    experts: int
    top: int
    shared_ff: int = 0       # 0: no shared expert

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff},
                             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class PusazenLayer:
    type: str
    mixer: Any
    mlp: Any                      # DenseMLP, MoEMLP or None
    layer_scale: bool = True      # the folder holds the layer's scale vectors
    lone_norm: bool = False       # no feed-forward, yet the folder holds a second norm


@dataclass(frozen=True)
class PusazenConfig:
    vocab: int
    width: int
    norm_eps: float
    alpha: float
    logit_scale: float
    layers: Tuple[PusazenLayer, ...]
    torch_dtype: str = "bfloat16"

    architecture = "Pusazen"
    model_type = "pusazen"
    wants_tensor_shapes = True      # ``load_config`` passes the folder's tensor shapes to ``from_dict``

    @classmethod
    def from_dict(cls, raw: Dict[str, Any], tensor_shapes: Optional[Mapping[str, Tuple[int, ...]]] = None):
        vocab = _get(raw, "vocab", int, "config", 1)
        width = _get(raw, "width", int, "config", 1)
        eps = _get(raw, "norm.eps", float, "config", 0.0)
        alpha = _get(raw, "postln_alpha", float, "config", optional=True)
        logit_scale = _get(raw, "logit_scale", float, "config", optional=True)
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config: layers must be a non-empty list")
        has = (lambda name: name in tensor_shapes) if tensor_shapes is not None else None
        layers = []
        for i, lr in enumerate(layers_raw):
            where = f"layers[{i}]"
            if not isinstance(lr, Mapping) or lr.get("type") not in MIXERS:
                raise ConfigError(f"{where}: type must be one of {MIXERS}, got "
                                  f"{lr.get('type') if isinstance(lr, Mapping) else lr!r}")
            m = lr.get("mixer")
            if not isinstance(m, Mapping):
                raise ConfigError(f"{where}: mixer missing from config")
            heads, dim = _get(m, "heads", int, where, 1), _get(m, "dim", int, where, 1)
            vdim = _get(m, "vdim", int, where, 1, optional=True) or dim
            if lr["type"] == "mlstm":
                mixer = MatrixMemoryMixer(heads, dim, vdim, _get(m, "gate_cap", float, where))
                if mixer.gate_cap <= 0:
                    raise ConfigError(f"{where}: gate_cap must be positive, got {mixer.gate_cap}")
            elif lr["type"] == "lightning":
                decay = m.get("decay")
                if not isinstance(decay, list) or len(decay) != heads or \
                        any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                    raise ConfigError(f"{where}: decay must list one number per head ({heads})")
                mixer = LightningMixer(heads, dim, vdim, tuple(float(d) for d in decay))
            else:
                kv_heads = _get(m, "kv_heads", int, where, 1, optional=True) or heads
                if heads % kv_heads:
                    raise ConfigError(f"{where}: {heads} heads are no multiple of {kv_heads} kv_heads")
                rot_dims = _get(m, "rot.dims", int, where, 0, optional=True) or 0
                if rot_dims % 2 or rot_dims > dim:
                    raise ConfigError(f"{where}: rot.dims {rot_dims} must be even and at most dim {dim}")
                mixer = AttentionMixer(
                    heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=_get(m, "scale", float, where),
                    softcap=_get(m, "softcap", float, where, 0.0, optional=True) or 0.0,
                    chunk=_get(m, "mask.size", int, where, 1, optional=True) or 0,
                    rot_base=(_get(m, "rot.base", float, where) if rot_dims else 1.0), rot_dims=rot_dims,
                    sink=has(f"l{i}.mix.sink") if has else bool(m.get("sink", True)))
            mlp_raw, mlp = lr.get("mlp"), None
            if mlp_raw is not None:
                if not isinstance(mlp_raw, Mapping) or mlp_raw.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"{where}: mlp.kind must be 'dense' or 'moe' (or mlp null)")
                if mlp_raw["kind"] == "dense":
                    mlp = DenseMLP(_get(mlp_raw, "ff", int, where, 1))
                else:
                    mlp = MoEMLP(ff=_get(mlp_raw, "expert.ff", int, where, 1),
                                 experts=_get(mlp_raw, "router.experts", int, where, 1),
                                 top=_get(mlp_raw, "router.top", int, where, 1),
                                 shared_ff=_get(mlp_raw, "shared.ff", int, where, 1, optional=True) or 0)
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"{where}: router.top {mlp.top} exceeds router.experts {mlp.experts}")
            layers.append(PusazenLayer(
                lr["type"], mixer, mlp,
                layer_scale=has(f"l{i}.ls1") if has else bool(lr.get("layer_scale", True)),
                lone_norm=bool(mlp is None and has and has(f"l{i}.norm2"))))
        return cls(vocab=vocab, width=width, norm_eps=eps, alpha=1.0 if alpha is None else alpha,
                   logit_scale=1.0 if logit_scale is None else logit_scale, layers=tuple(layers),
                   torch_dtype=str(raw.get("torch_dtype", "bfloat16")))

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "postln_alpha": self.alpha, "logit_scale": self.logit_scale,
                "layers": [{"type": l.type, "mixer": l.mixer.to_dict(),
                            "mlp": None if l.mlp is None else l.mlp.to_dict()} for l in self.layers]}
