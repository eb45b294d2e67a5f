"""Plain, slow implementation of the Lonulix decoder, used only as the tests' oracle.

Whole sequences on the CPU, no cache: attention sees the prefix through an explicit mask, the
recurrence walks the sequence token by token from a zero state, every token visits its experts
one by one.  One function per mechanism; nothing is shared with the product package (config.json
is parsed here, weights are read with the `safetensors` package).  The default element type is
float64, which bounds how much of a difference between the engine and this file is rounding.

The model, in this file's notation (N: RMS norm in groups; g: a gate per entry; a: one number):

    x = E[token] * s_e
    per layer:   x <- N1(a x + g1 * mixer(x)),   then   x <- N2(a x + g2 * ff(x))   (ff may be absent)
                 g = sigmoid(W_g x + b_g), from the same x that the branch reads
    logits = W_head N_f(x)

Two mixers: "latent_attention" (queries through a normed latent; keys and values expanded from a
normed low-rank latent, plus one rotated key part shared by the heads; rotation of neighbouring
pairs; a sliding window) and "hgrn2" (a matrix memory per head whose rows decay by a forget gate
bounded from below and take in the value scaled by the gate's complement).  Two feed-forwards:
dense SwiGLU, and a mixture of ungated GELU experts routed by softmax scores with a correction on
the choice, groups of experts of which the best are kept, and identity experts.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, Optional

import torch


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def read_weights(folder: str, dtype=torch.float64) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file
    return {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


# --------------------------------------------------------------------------- norms and activations

def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x²) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The row in `groups` equal consecutive parts, each divided by its own root mean square; one gain over the row."""
    T, d = x.shape
    parts = x.reshape(T, groups, d // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, d) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# --------------------------------------------------------------------------- rotation

def rotate_neighbours(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: of each head's first `dims` entries, entry 2i turns with entry 2i + 1 by the angle
    position * base^(-2i/dims); the rest pass.  The angle is the float32 product of position and float32 frequency."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = float(base) ** (-2.0 * i / dims)
    angle = (positions.to(torch.float32)[:, None] * f.to(torch.float32)[None, :]).to(x.dtype)
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------- latent attention

def window_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i sees key j when 0 <= i - j < size (no size: every j <= i)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size is not None:
        m = m & (i - j < int(size))
    return m


def latent_attention(h, w, p, m, eps, positions, probs_out: Optional[list] = None):
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    c_q = rms_norm(h @ w[p + "dq"].t(), w[p + "dq.norm"], eps)
    q = (c_q @ w[p + "uq"].t()).view(T, H, d + r)
    down = h @ w[p + "dkv"].t()
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_shared = down[:, None, rank:]                                       # one head, not normed
    if r:
        q_turn = rotate_neighbours(q[..., d:], positions, int(rot["dims"]), rot["base"])
        k_turn = rotate_neighbours(k_shared, positions, int(rot["dims"]), rot["base"])[:, 0]
    k = (c @ w[p + "uk"].t()).view(T, H, d)
    v = (c @ w[p + "uv"].t()).view(T, H, dv)
    mask = window_mask(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        s = q[:, head, :d] @ k[:, head].t()
        if r:
            s = s + q_turn[:, head] @ k_turn.t()
        s = (s * float(m["scale"])).masked_fill(~mask, float("-inf"))
        pr = torch.softmax(s, dim=-1)
        if probs_out is not None:
            probs_out.append(pr)
        out[:, head] = pr @ v[:, head]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


# --------------------------------------------------------------------------- forget-gate linear attention

def forget_gates(h, w, p, m):
    """[T, heads, dim]: lower + (1 - lower) * sigmoid(W_f h + b)."""
    lower = w[p + "lower"]
    f = lower + (1.0 - lower) * torch.sigmoid(h @ w[p + "f"].t() + w[p + "f.b"])
    return f.view(h.shape[0], m["heads"], m["dim"])


def hgrn2(h, w, p, m, eps, state_out: Optional[list] = None):
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].t()).view(T, H, d)
    v = (h @ w[p + "v"].t()).view(T, H, dv)
    f = forget_gates(h, w, p, m)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    if state_out is not None:
        state_out.append(S)
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return o @ w[p + "o"].t()


# --------------------------------------------------------------------------- feed-forwards

def dense_ff(h, w, p):
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


def route(h, w, p, router: dict):
    """Chosen router outputs [T, top] (numbers >= experts are identity experts) and their weights."""
    E, extra, top = int(router["experts"]), int(router.get("identity") or 0), int(router["top"])
    n_out = E + extra
    s = torch.softmax(h @ w[p + "router"].t(), dim=-1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    groups = router.get("groups")
    if groups and int(groups["count"]) > 1:
        G, keep = int(groups["count"]), int(groups["keep"])
        best = choice.view(-1, G, n_out // G).max(dim=-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, torch.topk(best, keep, dim=-1).indices, True)
        open_ = kept[:, :, None].expand(-1, -1, n_out // G).reshape(-1, n_out)
        choice = choice.masked_fill(~open_, float("-inf"))
    idx = torch.topk(choice, top, dim=-1).indices
    wt = s.gather(1, idx)
    wt = wt / (wt.sum(dim=-1, keepdim=True) + 1e-20) * float(router.get("scale", 1.0))
    return idx, wt


def expert(h, w, p):
    return gelu_erf(h @ w[p + "up"].t()) @ w[p + "down"].t()


def moe_ff(h, w, p, mlp):
    router = mlp["router"]
    E = int(router["experts"])
    idx, wt = route(h, w, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            e = int(idx[t, j])
            out[t] += wt[t, j] * (h[t] if e >= E else expert(h[t], w, p + f"e{e}."))
    return out


# --------------------------------------------------------------------------- the model

def gate(x, w, name):
    return torch.sigmoid(x @ w[name].t() + w[name + ".b"])


def layer(x, w, i, spec, cfg, positions):
    p = f"l{i}."
    eps, groups, a = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups") or 1), float(cfg.get("postln_alpha", 1.0))
    if spec["type"] == "latent_attention":
        y = latent_attention(x, w, p + "mix.", spec["mixer"], eps, positions)
    elif spec["type"] == "hgrn2":
        y = hgrn2(x, w, p + "mix.", spec["mixer"], eps)
    else:
        raise ValueError(spec["type"])
    x = group_norm(a * x + gate(x, w, p + "rg1") * y, w[p + "norm1"], groups, eps)
    mlp = spec.get("mlp")
    if mlp is not None:
        y = dense_ff(x, w, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, p + "mlp.", mlp)
        x = group_norm(a * x + gate(x, w, p + "rg2") * y, w[p + "norm2"], groups, eps)
    return x


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, stream_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from its first token."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["embed"][tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, w, i, spec, cfg, positions)
        if stream_out is not None:
            stream_out.append(x.clone())
    x = group_norm(x, w["final.norm"], int(cfg["norm"].get("groups") or 1), float(cfg["norm"]["eps"]))
    return x @ w["head"].t()
