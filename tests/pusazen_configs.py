"""Small Pusazen configurations for the tests: they differ in every size and option (layer order, key and value widths
that differ, grouped and single key heads, chunks shorter and longer than a page and none at all, partial, full and
no rotation, with and without a soft cap, dense / routed / no feed-forward, with and without a shared expert, one or
several experts per token, sizes that are multiples of nothing useful)."""
import os

import torch


def _memory(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _attention(heads, kv_heads, dim, vdim, scale, chunk=0, softcap=0.0, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if softcap:
        m["softcap"] = softcap
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, shared=0):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layers(*pairs):
    return [{**mixer, "mlp": mlp} for mixer, mlp in pairs]


# Memory first; values wider than keys; grouped key heads (4 over 2); a chunk of 20 (longer than a page of 16, no
# multiple of it); rotation of 8 of 16 channels; a layer without feed-forward; two experts of four plus a shared one.
PUSAZEN_A = {
    "architecture": "Pusazen", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 1.8, "logit_scale": 0.7,
    "layers": _layers(
        (_memory(2, 16, 24, 8.0), _dense(80)),
        (_attention(4, 2, 16, 32, 0.4, chunk=20, softcap=6.0, rot=(10000.0, 8)), _moe(40, 4, 2, shared=24)),
        (_lightning(3, 8, 16, (0.5, 0.9, 0.99)), None),
        (_memory(1, 48, 16, 15.0), _moe(24, 3, 3)))}

# Attention first; one key head for five query heads; a chunk of 7 (shorter than a page of 8); full rotation; no soft
# cap; one expert of five, no shared expert; an odd width; alpha 1; keys wider than values; a chunk of ONE position.
PUSAZEN_B = {
    "architecture": "Pusazen", "vocab": 157, "width": 72, "norm": {"eps": 1e-6}, "postln_alpha": 1.0, "logit_scale": 1.5,
    "layers": _layers(
        (_attention(5, 1, 24, 8, 0.25, chunk=7, rot=(500.0, 24)), _moe(56, 5, 1)),
        (_lightning(2, 24, 8, (0.8, 1.0)), _dense(50)),
        (_attention(2, 2, 8, 40, 0.5, chunk=1, softcap=2.0), None),
        (_memory(3, 20, 12, 3.0), _moe(30, 2, 1, shared=16)))}

# Sizes at which the bfloat16 engine's products take its tensor-core kernels (multiples of 8 and 16): heads of 64, a
# chunk of 48, eight experts, a shared expert of 128.
PUSAZEN_C = {
    "architecture": "Pusazen", "vocab": 512, "width": 256, "norm": {"eps": 1e-6}, "postln_alpha": 2.0, "logit_scale": 0.5,
    "layers": _layers(
        (_attention(4, 2, 64, 64, 0.125, chunk=48, softcap=30.0, rot=(1e6, 32)), _moe(128, 8, 2, shared=128)),
        (_memory(4, 64, 64, 15.0), _moe(128, 8, 1)),
        (_lightning(4, 64, 32, (0.6, 0.9, 0.97, 0.999)), _dense(256)),
        (_attention(8, 8, 32, 64, 0.2, chunk=130, rot=(1e4, 16)), _moe(64, 8, 2, shared=64)))}

# Recurrent layers only: no pages at all, only state. Key sizes that are no multiple of four, one head, one expert of one.
PUSAZEN_D = {
    "architecture": "Pusazen", "vocab": 97, "width": 48, "norm": {"eps": 1e-6}, "postln_alpha": 3.0, "logit_scale": 1.0,
    "layers": _layers(
        (_lightning(1, 18, 10, (0.95,)), _moe(32, 1, 1)),
        (_memory(3, 10, 7, 4.0), None),
        (_memory(2, 64, 40, 20.0), _dense(30)),
        (_lightning(5, 4, 4, (0.1, 0.5, 0.9, 0.99, 0.999)), _moe(16, 6, 2, shared=8)))}

# Attention without a mask (every earlier key is seen: its pages stay) beside a chunked one; no rotation in one, no
# soft cap in the other; pages of 32.
PUSAZEN_E = {
    "architecture": "Pusazen", "vocab": 130, "width": 64, "norm": {"eps": 1e-5}, "postln_alpha": 2.5, "logit_scale": 0.9,
    "layers": _layers(
        (_attention(4, 4, 16, 16, 0.3, softcap=4.0), _dense(64)),
        (_attention(6, 3, 16, 16, 0.3, chunk=33, rot=(1e5, 16)), None),
        (_memory(2, 32, 32, 10.0), _moe(32, 4, 2, shared=32)))}

# Sizes that are multiples of nothing: a width of 100, heads of 12 x 20 and 80 x 48 (no tensor-core kernel is built for
# the first), a chunk of 5, rotation of 2 channels and of all 80, every expert chosen (5 of 5), two experts with one
# chosen, a vocabulary of 61, alpha below 1.
PUSAZEN_F = {
    "architecture": "Pusazen", "vocab": 61, "width": 100, "norm": {"eps": 1e-6}, "postln_alpha": 0.7, "logit_scale": 2.0,
    "layers": _layers(
        (_attention(3, 3, 12, 20, 0.33, chunk=5, softcap=50.0, rot=(77.0, 2)), _moe(28, 5, 5, shared=12)),
        (_memory(5, 12, 20, 2.5), _dense(36)),
        (_lightning(2, 36, 52, (0.7, 0.98)), None),
        (_attention(8, 2, 80, 48, 0.1, chunk=64, rot=(1e4, 80)), _moe(20, 2, 1)))}

# name -> (config.json, seed, sigma of matrices, page size)
PUSAZEN = {"A": (PUSAZEN_A, 3, 0.15, 16), "B": (PUSAZEN_B, 4, 0.15, 8), "C": (PUSAZEN_C, 5, 0.06, 16),
           "D": (PUSAZEN_D, 6, 0.2, 16), "E": (PUSAZEN_E, 7, 0.15, 32), "F": (PUSAZEN_F, 8, 0.12, 16)}


def write_pusazen_model(name: str, folder: str, dtype=torch.bfloat16) -> str:
    """Write a small Pusazen folder with random weights; returns its path."""
    from llm_rs_b200.config import PusazenConfig
    from llm_rs_b200.weights import write_random_model
    raw, seed, sigma, _ = PUSAZEN[name]
    path = os.path.join(folder, f"pusazen_{name}")
    return write_random_model(path, PusazenConfig.from_dict(raw), seed=seed, sigma=sigma, norm_jitter=0.2, dtype=dtype)
