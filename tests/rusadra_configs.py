"""Small Rusadra configurations for the tests: they differ in every size and option (layer order, a layer that reads
another's cached rows through a window of its own, a layer without feed-forward, one or several experts per token,
partial rotation, a window that is never reached, soft cap or none, sizes that are multiples of nothing useful)."""
import os

import torch


def _latent(heads, dim, rot_dim, vdim, rank, window, base=10000.0, dims=None, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": rot_dim if dims is None else dims}}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def _delta(heads, dim, decay_rank):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": decay_rank}}


def _moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _layers(*pairs):
    return [{**mixer, "mlp": mlp} for mixer, mlp in pairs]


# Delta first; a window of 20; a reader of layer 1's rows with a wider window (33); two experts per token; a layer
# without feed-forward; a delta head of 48 channels (no power of two).
RUSADRA_A = {
    "architecture": "Rusadra", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "logit_softcap": 12.0,
    "layers": _layers(
        (_delta(2, 16, 8), _moe(40, 0.7, 4, 2)),
        (_latent(3, 16, 8, 24, 40, 20), _moe(40, 0.7, 4, 2)),
        (_delta(1, 48, 5), None),
        (_latent(3, 16, 8, 24, 40, 33, kv_from=1), _moe(24, 1.5, 3, 3)))}

# Attention first; partial rotation (8 of 16); a window that no request reaches; one head; one expert per token out
# of five; no soft cap; a reader with a NARROWER window (7) than its source; an odd width.
RUSADRA_B = {
    "architecture": "Rusadra", "vocab": 157, "width": 72, "norm": {"eps": 1e-6},
    "layers": _layers(
        (_latent(1, 24, 16, 40, 50, 1000, base=500000.0, dims=8), _moe(56, 1.0, 5, 1)),
        (_latent(5, 8, 16, 8, 50, 7, base=500000.0, dims=8, kv_from=0, scale=0.3), _moe(56, 1.0, 5, 1)),
        (_delta(3, 32, 12), _moe(30, 2.0, 2, 1)),
        (_latent(2, 32, 32, 32, 96, 64, base=1000.0), None))}

# Sizes at which the bfloat16 engine's products take its tcgen05 kernel in small steps (multiples of 8), heads of 64
# channels in the recurrent layer, a latent of 128, eight experts.
RUSADRA_C = {
    "architecture": "Rusadra", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
    "layers": _layers(
        (_latent(4, 64, 32, 64, 128, 48, base=1e6), _moe(128, 1.0, 8, 1)),
        (_delta(4, 64, 16), _moe(128, 1.0, 8, 2)),
        (_latent(8, 32, 32, 32, 128, 130, base=1e6, kv_from=0), _moe(64, 1.0, 8, 2)))}

# Recurrent layers only: the model asks for no pages at all, only state. One head of 16 channels, one expert out of
# one, a layer without feed-forward.
RUSADRA_D = {
    "architecture": "Rusadra", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "logit_softcap": 8.0,
    "layers": _layers(
        (_delta(1, 16, 3), _moe(32, 1.0, 1, 1)),
        (_delta(3, 24, 6), None),
        (_delta(2, 64, 9), _moe(16, 0.5, 6, 2)))}

# Attention layers only, no feed-forward anywhere: one layer that owns its rows, two that read them through other
# windows, a second owner with a window of one key (a token sees only itself).
RUSADRA_E = {
    "architecture": "Rusadra", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
    "layers": _layers(
        (_latent(4, 16, 16, 16, 64, 40, base=1e5), None),
        (_latent(2, 32, 16, 8, 64, 17, base=1e5, kv_from=0), None),
        (_latent(4, 8, 8, 24, 32, 1, base=50.0), None),
        (_latent(6, 16, 16, 16, 64, 64, base=1e5, kv_from=0), None))}

# Two attention layers that own rows of the same shape and window (one page group with two entries, one block table
# for both), a reader of the SECOND, a recurrent layer between them; pages of 32 keys.
RUSADRA_F = {
    "architecture": "Rusadra", "vocab": 150, "width": 64, "norm": {"eps": 1e-6}, "logit_softcap": 20.0,
    "layers": _layers(
        (_latent(4, 16, 16, 16, 64, 24, base=1e4), _moe(32, 1.0, 4, 2)),
        (_delta(2, 32, 8), None),
        (_latent(2, 32, 16, 32, 64, 24, base=1e4), _moe(32, 1.0, 4, 1)),
        (_latent(4, 16, 16, 16, 64, 24, base=1e4, kv_from=2), None))}

# name -> (config.json, seed, sigma of matrices, page size)
RUSADRA = {"A": (RUSADRA_A, 3, 0.08, 16), "B": (RUSADRA_B, 4, 0.1, 8), "C": (RUSADRA_C, 5, 0.05, 16),
           "D": (RUSADRA_D, 6, 0.1, 16), "E": (RUSADRA_E, 7, 0.1, 16), "F": (RUSADRA_F, 8, 0.1, 32)}


def write_rusadra_model(name: str, folder: str, dtype=torch.bfloat16) -> str:
    """Write a small Rusadra folder with random weights; returns its path."""
    from llm_rs_b200.config import RusadraConfig
    from llm_rs_b200.weights import write_random_model
    raw, seed, sigma, _ = RUSADRA[name]
    path = os.path.join(folder, f"rusadra_{name}")
    return write_random_model(path, RusadraConfig.from_dict(raw), seed=seed, sigma=sigma, norm_jitter=0.2, dtype=dtype)
