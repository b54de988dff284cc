"""A plain, slow implementation of the Rusadra design: one function per mechanism, PyTorch on the
CPU, no cache, whole sequences at once (the recurrent layer walks token by token). It shares no
code with the package; tests compare the engine with it.

Notation: T tokens, D the model width, H heads. A linear weight is stored [out, in] and applied as
``W @ x``. ``cfg`` is the parsed config.json, ``w`` maps tensor names to tensors of ``dtype``
(float64 unless a test asks otherwise; integer tables stay integers).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# ---- files -------------------------------------------------------------------------------------
def read_safetensors(path):
    """name -> torch tensor (bfloat16 widened to float32, integers kept), read by hand."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = np.frombuffer(data[lo:hi], dtype=np.uint8)
        kind = meta["dtype"]
        if kind == "BF16":
            bits = raw.view(np.uint16).astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif kind == "F32":
            t = torch.from_numpy(raw.view(np.float32).copy())
        elif kind == "I32":
            t = torch.from_numpy(raw.view(np.int32).copy())
        elif kind == "I64":
            t = torch.from_numpy(raw.view(np.int64).copy())
        else:
            raise ValueError(f"{name}: type {kind}")
        out[name] = t.reshape(meta["shape"])
    return out


def load_model_dir(path, dtype=torch.float64):
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(path, "model.safetensors"))
    return cfg, {k: (v.to(dtype) if v.is_floating_point() else v.long()) for k, v in w.items()}


# ---- small functions ---------------------------------------------------------------------------
def rms(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """RMS norm whose stored weight lies around zero: the factor is 1 + weight."""
    return rms(x, eps) * (1.0 + weight)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def token_shift(h, mu):
    """h_t + (h_{t-1} - h_t) * mu, with h_{-1} = 0; h: [T, D] of one sequence."""
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (prev - h) * mu


def rotate_half(x, positions, base, dims):
    """Rotary positions on the first ``dims`` entries of the last axis; entry i is paired with
    entry i + dims/2. x: [T, ..., n]; positions: [T]."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cos, sin = ang.cos(), ang.sin()
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., dims:]], -1)


# ---- mixers ------------------------------------------------------------------------------------
def latent_kv(h, w, pre, m, eps):
    """The cached part of latent attention for one sequence: the normed latent c [T, kv_rank] and
    the rotated shared key part [T, rot_dim]."""
    T = h.shape[0]
    dkv = h @ w[pre + "dkv"].T
    c = rms(dkv[:, : m["kv_rank"]], eps) * w[pre + "dkv.norm"]
    kr = rotate_half(dkv[:, m["kv_rank"]:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, pre, m, eps, kv=None):
    """Latent attention over one sequence h [T, D]. ``kv`` is (c, kr) of the layer whose cache this
    layer reads, or None when it makes its own. Returns (output [T, D], (c, kr))."""
    T = h.shape[0]
    H, dn, dr, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    if kv is None:
        kv = latent_kv(h, w, pre, m, eps)
    c, kr = kv
    q = (h @ w[pre + "q"].T).view(T, H, dn + dr)
    qn = q[..., :dn]
    qr = rotate_half(q[..., dn:], torch.arange(T), m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ w[pre + "uk"].T).view(T, H, dn)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (i - j >= 0) & (i - j < m["mask"]["size"])
    s = s.masked_fill(~seen, float("-inf"))
    p = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", p, v)
    gate = torch.sigmoid(h @ w[pre + "g"].T)                 # [T, H]
    o = (o * gate[:, :, None]).reshape(T, H * dv)
    return o @ w[pre + "o"].T, kv


def general_delta(h, w, pre, m, eps, state=None):
    """Generalized delta rule over one sequence h [T, D], token by token. ``state`` [H, d, d]
    (key channel, value channel) continues an earlier part. Returns (output [T, D], state)."""
    T = h.shape[0]
    H, d = m["heads"], m["dim"]
    r = (h @ w[pre + "r"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, H, d)
    v = (h @ w[pre + "v"].T).view(T, H, d)
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(
        torch.tanh(h @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, d)
    a = torch.sigmoid(h @ w[pre + "a"].T + w[pre + "a.b"]).view(T, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=h.dtype) if state is None else state.clone()
    out = torch.empty(T, H, d, dtype=h.dtype)
    for t in range(T):
        uS = torch.einsum("hi,hij->hj", u[t], S)                       # u^T S, old state
        S = decay[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hij,hi->hj", S, r[t])                  # S^T r
    o = rms(out, eps).reshape(T, H * d) * w[pre + "norm"]
    o = o * torch.sigmoid(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, S


# ---- feed-forward ------------------------------------------------------------------------------
def expert(h, w, pre, limit):
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def table_moe(h, tokens, w, pre, f):
    """Every token id has a row of the table: its experts, each weighted 1/top."""
    top = f["router"]["top"]
    table = w[pre + "table"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[tokens[t]].tolist():
            out[t] += expert(h[t:t + 1], w, f"{pre}e{e}.", f["expert"]["limit"])[0] / top
    return out


# ---- the model ---------------------------------------------------------------------------------
def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][tokens]
    kvs, layers = {}, []
    for i, layer in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        h = token_shift(x, w[pre + "shift"])
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, kvs[i] = latent_attention(h, w, pre + "mix.", m, eps, None if src is None else kvs[src])
        elif layer["type"] == "general_delta":
            y, _ = general_delta(h, w, pre + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + offset_norm(y, w[pre + "norm1"], eps)
        if layer.get("mlp") is not None:
            x = x + offset_norm(table_moe(x, tokens, w, pre + "mlp.", layer["mlp"]), w[pre + "norm2"], eps)
        layers.append(x)
    logits = offset_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(layers)) if return_layers else logits


def greedy_generate(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
