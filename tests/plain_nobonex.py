"""Plain, slow implementation of the Nobonex decoder, used only as the tests' oracle.

Whole sequences on the CPU, no cache: attention sees the prefix through an explicit mask, the
state-space layer walks the sequence token by token from a zero state, every token visits its
experts one by one.  One function per mechanism; nothing is shared with the product package
(config.json is parsed here, weights are read with the `safetensors` package).  The default
element type is float64, which bounds how much of a difference between the engine and this file
is rounding.

The model, in this file's notation (T: the elementwise norm tanh(a v) * w + b; m: one number):

    x = E[token] * s_e
    per layer:   x <- x + m * T1b(mixer(T1(x))),   then   x <- x + m * T2b(ff(T2(x)))   (ff may be absent)
    logits = W_head T_f(x)

Three mixers: "attention" (queries and keys through a short convolution over time, values = the
convolved keys, an RMS norm over the whole projection, rotation of neighbouring pairs), "attention_2"
(biases, RMS norm per head, rotate-half rotation with stretched frequencies, soft-capped scores, a
mask of chunks, a sigmoid gate on the heads' outputs, optionally the keys and values of an earlier
layer) and "mamba2" (a matrix state per head with one decay per head and token).  Two feed-forwards:
dense GEGLU, and a mixture of clamped gated experts whose routing weight multiplies their input.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch
import torch.nn.functional as F


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------- norms and activations

def tanh_norm(v: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    """tanh(a v) * w + b, entry by entry: no mean, no variance."""
    return torch.tanh(w[name + ".alpha"] * v) * w[name] + w[name + ".b"]


def rms_norm(v: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * gain


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def short_conv(u: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """u [T, C], taps [C, K]: y_t = sum_j taps[:, j] * u_(t - K + 1 + j), zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([u.new_zeros(K - 1, C), u], dim=0)
    y = u.new_zeros(T, C)
    for j in range(K):
        y = y + padded[j:j + T] * taps[:, j]
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- rotations

def frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(f_i for i < dims/2, the factor on cos and sin)."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(turns(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turns(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(v: torch.Tensor, positions: torch.Tensor, rot: dict, neighbours: bool) -> torch.Tensor:
    """v [T, heads, size]; the first rot.dims entries of each head are rotated, pair by pair: neighbours (2i, 2i+1), or
    halves (i, i + dims/2)."""
    dims = int(rot["dims"])
    if dims == 0:
        return v
    f, mult = frequencies(dims, float(rot["base"]), rot.get("scaling"))
    ang = positions.to(v.dtype)[:, None] * torch.tensor(f, dtype=v.dtype)[None, :]          # [T, dims/2]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    out = v.clone()
    if neighbours:
        a, b = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = v[..., :dims // 2], v[..., dims // 2:dims]
        out[..., :dims // 2] = a * c - b * s
        out[..., dims // 2:dims] = b * c + a * s
    return out


# --------------------------------------------------------------------------- attention

def visible(T: int, chunk: Optional[int]) -> torch.Tensor:
    """[T, T] True where row i may read column j: j <= i, and with chunks only inside i's chunk."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_attention(q, k, v, scale, mask, softcap=None, probs_out: Optional[list] = None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key/value head h // (H/G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = q.new_zeros(T, H, v.shape[2])
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, -math.inf)
        p = torch.softmax(s, dim=-1)
        if probs_out is not None:
            probs_out.append(p)
        out[:, h] = p @ v[:, g]
    return out


def conv_attention(h, w, p, m, eps, positions, kept: dict, probs_out=None):
    """Mixer "attention": no value matrix, the values are the keys as they leave the convolution."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T, w[p + "q.conv"])
    k = short_conv(h @ w[p + "k"].T, w[p + "k.conv"])
    v = k.reshape(T, G, dv)
    q = rms_norm(q, w[p + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, w[p + "k.norm"], eps).reshape(T, G, d)
    q = rotate(q, positions, m["rot"], neighbours=True)
    k = rotate(k, positions, m["rot"], neighbours=True)
    o = softmax_attention(q, k, v, m["scale"], visible(T, None), probs_out=probs_out)
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_attention(h, w, p, m, eps, positions, kept: dict, index: int, probs_out=None):
    """Mixer "attention_2".  `kept[j]` holds layer j's keys and values for a later layer that names it in kv_from."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).reshape(T, H, d)
    q = rotate(rms_norm(q, w[p + "q.norm"], eps), positions, m["rot"], neighbours=False)
    if m.get("kv_from") is not None:
        k, v = kept[int(m["kv_from"])]
    else:
        k = (h @ w[p + "k"].T + w[p + "k.b"]).reshape(T, G, d)
        v = (h @ w[p + "v"].T + w[p + "v.b"]).reshape(T, G, dv)
        k = rotate(rms_norm(k, w[p + "k.norm"], eps), positions, m["rot"], neighbours=False)
        kept[index] = (k, v)
    chunk = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, k, v, m["scale"], visible(T, chunk), softcap=m.get("softcap"), probs_out=probs_out)
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# --------------------------------------------------------------------------- state space

def mamba2(h, w, p, m, eps, state_out: Optional[list] = None):
    """Per head a state S [N, dv]: S <- exp(-exp(A_log) dt) S + dt B xᵀ; y = Sᵀ C + D x."""
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = F.softplus(dt + w[p + "dt_bias"])                                 # [T, H]
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = h.new_zeros(T, H, dv)
    S = h.new_zeros(H, N, dv)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    if state_out is not None:
        state_out.append(S.clone())
    y = y.reshape(T, inner) * silu(z)
    parts = int(m.get("norm_groups") or 1)
    y = y.reshape(T, parts, inner // parts)
    y = y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)
    return (y.reshape(T, inner) * w[p + "norm"]) @ w[p + "o"].T


# --------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router: dict):
    """(ids [T, top], weights [T, top]): the experts with the largest sigmoid scores, and those scores as they are."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    weights, ids = torch.topk(s, int(router["top"]), dim=-1)
    return ids, weights


def expert(v, w, p, limit: float):
    g = torch.clamp(v @ w[p + "gate"].T, max=limit)
    u = torch.clamp(v @ w[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def moe_ff(h, w, p, mlp):
    ids, weights = route(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            out[t] = out[t] + expert(weights[t, j] * h[t], w, f"{p}e{int(ids[t, j])}.", float(mlp["expert"]["limit"]))
    return out


# --------------------------------------------------------------------------- the model

def mixer(h, w, i, spec, cfg, positions, kept):
    p, m, eps = f"l{i}.mix.", spec["mixer"], float(cfg["norm"]["eps"])
    if spec["type"] == "attention":
        return conv_attention(h, w, p, m, eps, positions, kept)
    if spec["type"] == "attention_2":
        return gated_attention(h, w, p, m, eps, positions, kept, i)
    if spec["type"] == "mamba2":
        return mamba2(h, w, p, m, eps)
    raise ValueError(spec["type"])


def layer(x, w, i, spec, cfg, positions, kept):
    mult = float(cfg.get("residual_mult", 1.0))
    n = f"l{i}."
    x = x + mult * tanh_norm(mixer(tanh_norm(x, w, n + "norm1"), w, i, spec, cfg, positions, kept), w, n + "norm1b")
    mlp = spec.get("mlp")
    if mlp is not None:
        h = tanh_norm(x, w, n + "norm2")
        f = dense_ff(h, w, n + "mlp.") if mlp.get("kind", "dense") == "dense" else moe_ff(h, w, n + "mlp.", mlp)
        x = x + mult * tanh_norm(f, w, n + "norm2b")
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, stream_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token; `stream_out` collects the stream behind every layer."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    kept: dict = {}
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg, positions, kept)
        if stream_out is not None:
            stream_out.append(x.clone())
    return tanh_norm(x, w, "final.norm") @ w["head"].T
