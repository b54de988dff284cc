"""A plain, slow implementation of the Pusazen design: float64 PyTorch on the CPU, no cache, no batching, one function
per mechanism, every token of a sequence recomputed from the start. It shares no code with the package; the tests
compare the engine with it.

A model is (config dict, {tensor name: float64 tensor}). Linear weights are [out, in] and applied as W x.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softcap(z, cap: float):
    return cap * torch.tanh(z / cap)


# -- mixers ----------------------------------------------------------------------------------------------
def mlstm(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Matrix memory with exponential gates and a running maximum that starts at 0. h: [T, width]."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    T = h.size(0)
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                                     # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        a = torch.exp(gf[t] + mx - m_new)
        b = torch.exp(gi[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = rms(out, eps).reshape(T, H * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def lightning(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Linear attention with one fixed decay per head; no other scale."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    decay = torch.tensor([float(x) for x in m["decay"]], dtype=F64)
    T = h.size(0)
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(out.reshape(T, H * dv), eps) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def rotate_half(x: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, dim]; the first ``dims`` dimensions of each head turn, i paired with i + dims/2."""
    if dims == 0:
        return x
    T = x.size(0)
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    a = torch.arange(T, dtype=F64)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """Grouped heads, norms over the whole q and k projections, partial rotation, capped scores, a mask of chunks
    counted from position 0 (none without ``mask``), a sink in the softmax's denominator."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.size(0)
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_half(q.view(T, H, d), int(rot["dims"]), float(rot["base"]))
    k = rotate_half(k.view(T, G, d), int(rot["dims"]), float(rot["base"]))
    size = int(m["mask"]["size"]) if m.get("mask") else 0
    cap = float(m.get("softcap") or 0.0)
    pos = torch.arange(T)
    seen = pos[None, :] <= pos[:, None]
    if size:
        seen = seen & ((pos[None, :] // size) == (pos[:, None] // size))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = softcap(s, cap)
        s = s.masked_fill(~seen, -math.inf)
        sink = w[p + "sink"][hd]
        mx = torch.maximum(s.max(dim=-1).values, sink)
        e = torch.exp(s - mx[:, None])
        out[:, hd] = (e @ v[:, g]) / (e.sum(-1) + torch.exp(sink - mx))[:, None]
    return out.reshape(T, H * dv) @ w[p + "o"].T


# -- feed-forward ------------------------------------------------------------------------------------------
def dense_ff(h, w, p: str) -> torch.Tensor:
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def gated_expert(h, w, p: str) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe_ff(h, w, p: str, f: dict) -> torch.Tensor:
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.size(0)):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        wt = torch.softmax(z[t, order], dim=0)
        for j, e in enumerate(order):
            out[t] += wt[j] * gated_expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + gated_expert(h, w, p + "shared.") * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


# -- the model ---------------------------------------------------------------------------------------------
MIXERS = {"mlstm": mlstm, "lightning": lightning, "attention": attention}


def forward(config: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: list = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its start. ``layers_out`` collects the stream after every layer."""
    eps, alpha = float(config["norm"]["eps"]), float(config["postln_alpha"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        y = MIXERS[layer["type"]](x, w, p + "mix.", layer["mixer"], eps)
        if p + "ls1" in w:
            y = y * w[p + "ls1"]
        x = rms(alpha * x + y, eps) * w[p + "norm1"]
        f = layer.get("mlp")
        if f is not None:
            y = dense_ff(x, w, p + "mlp.") if f["kind"] == "dense" else moe_ff(x, w, p + "mlp.", f)
            if p + "ls2" in w:
                y = y * w[p + "ls2"]
            x = rms(alpha * x + y, eps) * w[p + "norm2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * w["final.norm"]
    return (x @ w["head"].T) * float(config["logit_scale"])


# -- folders and generation -----------------------------------------------------------------------------
def load_model_dir(path: str):
    """(config dict, {name: float64 tensor}) of a model folder."""
    import json
    import os

    from plain_rusadra import read_safetensors
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    w = read_safetensors(os.path.join(path, "model.safetensors"))
    return cfg, {k: v.to(F64) for k, v in w.items()}


def greedy_generate(config: dict, w, prompt: List[int], n_new: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward(config, w, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
