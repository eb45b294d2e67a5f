"""Shared by the Nobonex tests: small configurations of their own (sizes chosen so that nothing that could be equal is equal:
key and value head sizes, heads and key/value heads, rotated and unrotated entries, state and value sizes, groups of one and
of several; chunks that are no multiple of a page, exactly a page, one token; a reader of another layer's keys with the
owner's mask and with another; `top` of one, of several and of all; factors of one and other than one), model folders with
random weights in which some tensors are set by hand so that what they do shows, and the comparison with the plain
implementation."""
from __future__ import annotations

import functools
import os
from typing import Dict, Sequence

import torch

import helpers
import mini_llama_cpp_release_b200 as ml
import plain_nobonex as pn
from kebesun_helpers import check  # noqa: F401  (the same bounds on rows of logits)
from mini_llama_cpp_release_b200.config import ModelConfig


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def conv_attention(heads, kv_heads, dim, conv, scale, rotation):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": conv, "scale": scale, "rot": rotation}


def gated_attention(heads, kv_heads, dim, vdim, scale, rotation, softcap=None, chunk=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation}
    if softcap is not None:
        m["softcap"] = softcap
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba2(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def model(vocab, width, eps, mult, scale, layers):
    return {"architecture": "Nobonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": scale}, "layers": layers}


YARN = (3.0, 64, 16.0, 2.0)

# all three mixers and all three feed-forwards; a reader of layer 0's keys under the same mask of 50
MIXED = model(300, 96, 1e-5, 0.6, 3.0, [
    {"type": "attention_2", "mlp": moe(48, 5, 2, 1.5), "mixer": gated_attention(4, 2, 24, 20, 0.2, rot(8, 3000.0, YARN), 8.0, 50)},
    {"type": "mamba2", "mlp": dense(112), "mixer": mamba2(3, 16, 24, 1, 3, 3)},
    {"type": "attention", "mlp": None, "mixer": conv_attention(6, 3, 16, 4, 0.3, rot(6, 500.0))},
    {"type": "attention_2", "mlp": dense(64), "mixer": gated_attention(4, 2, 24, 20, 0.15, rot(8, 3000.0, YARN), 5.0, 50, kv_from=0)},
    {"type": "mamba2", "mlp": moe(32, 4, 4, 0.8), "mixer": mamba2(4, 8, 40, 2, 2, 1)},
])

# head sizes of 64 and 128 (the tensor-core attention kernels), chunks of exactly a page and of 130 (over two pages), a
# state of 128, factors of one
WIDE = model(257, 128, 2e-6, 1.0, 1.0, [
    {"type": "attention_2", "mlp": moe(64, 6, 3, 2.5), "mixer": gated_attention(4, 2, 64, 64, 0.1, rot(32, 40000.0, (4.0, 128, 32.0, 1.0)), 15.0, 130)},
    {"type": "mamba2", "mlp": None, "mixer": mamba2(4, 64, 128, 2, 4, 2)},
    {"type": "attention", "mlp": dense(144), "mixer": conv_attention(2, 1, 128, 2, 0.09, rot(64, 1e6))},
    {"type": "attention_2", "mlp": dense(80), "mixer": gated_attention(2, 2, 128, 96, 0.11, rot(128, 1e4), None, 64)},
])

# sizes the fast paths do not take: a width that is no multiple of 8, a chunk of one token, a layer without a mask and one
# without a soft cap, no rotation at all, a reader whose mask differs from its owner's, one tap, 33 experts with one chosen,
# all of three experts chosen
ODD = model(77, 100, 1e-5, 1.3, 0.3, [
    {"type": "attention_2", "mlp": moe(20, 33, 1, 3.0), "mixer": gated_attention(5, 5, 12, 10, 0.3, rot(6, 50.0), 3.0, 7)},
    {"type": "mamba2", "mlp": None, "mixer": mamba2(5, 12, 10, 5, 1, 5)},
    {"type": "attention_2", "mlp": dense(36), "mixer": gated_attention(5, 5, 12, 10, 0.4, rot(6, 50.0), None, 1, kv_from=0)},
    {"type": "attention", "mlp": moe(12, 3, 3, 1.0), "mixer": conv_attention(3, 1, 20, 1, 0.2, rot(0, 1.0))},
    {"type": "attention_2", "mlp": None, "mixer": gated_attention(2, 1, 8, 24, 0.5, rot(8, 2.0, (2.0, 16, 4.0, 1.0)))},
    {"type": "attention_2", "mlp": None, "mixer": gated_attention(5, 5, 12, 10, 0.25, rot(6, 50.0), 2.0, None, kv_from=0)},
])

TINY_MIXER = gated_attention(1, 1, 8, 8, 0.3, rot(4, 100.0))
ONLY_GATED = model(200, 64, 1e-5, 0.8, 2.0, [{"type": "attention_2", "mlp": None,
                                              "mixer": gated_attention(6, 2, 20, 28, 0.21, rot(12, 700.0, YARN), 30.0, 33)}])
ONLY_CONV = model(200, 64, 1e-5, 1.0, 1.5, [{"type": "attention", "mlp": None,
                                             "mixer": conv_attention(4, 2, 24, 3, 0.2, rot(10, 300.0))}])
ONLY_MAMBA = model(200, 64, 1e-5, 0.7, 1.0, [{"type": "mamba2", "mlp": None, "mixer": mamba2(6, 12, 20, 3, 4, 2)}])
ONLY_MOE = model(200, 64, 1e-5, 2.0, 1.0, [{"type": "attention_2", "mixer": TINY_MIXER, "mlp": moe(40, 7, 3, 1.2)}])
ONLY_DENSE = model(200, 64, 1e-5, 0.9, 1.0, [{"type": "attention_2", "mixer": TINY_MIXER, "mlp": dense(72)}])
# a layer that reads the layer before it under the same mask, both without a feed-forward
SHARED = model(150, 64, 1e-5, 1.0, 1.0, [
    {"type": "attention_2", "mlp": None, "mixer": gated_attention(4, 1, 16, 16, 0.25, rot(16, 1000.0), 10.0, 70)},
    {"type": "attention_2", "mlp": None, "mixer": gated_attention(4, 1, 16, 16, 0.3, rot(16, 1000.0), 4.0, 70, kv_from=0)}])

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "gated": ONLY_GATED, "conv": ONLY_CONV, "mamba": ONLY_MAMBA, "moe": ONLY_MOE,
           "dense": ONLY_DENSE, "shared": SHARED}


def shape_weights(weights: Dict[str, torch.Tensor], seed: int, peaked: float = 1.0) -> None:
    """Random weights hide some faults.  The state-space layers get slow decays and step sizes around one (tokens hundreds of
    places back still count), their skip factors and the norms' biases and slopes are spread out, routers are made decisive
    (so that the chosen experts do not hang on the last bit), the projections' biases are as large as the projections, and
    with `peaked` the gains of the attention's query norms are scaled so that single keys decide rows."""
    g = torch.Generator().manual_seed(seed)
    for name, t in weights.items():
        if name.endswith(".A_log"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5 - 5.5)
        elif name.endswith(".dt_bias"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)
        elif name.endswith(".D"):
            t.copy_(torch.randn(t.shape, generator=g))
        elif name.endswith(".alpha"):
            t.copy_(torch.rand(t.shape, generator=g) * 1.5 + 0.5)
        elif ".norm" in name and name.endswith(".b") and ".mix." not in name:
            t.copy_(torch.randn(t.shape, generator=g) * 0.3)
        elif name.endswith(".router"):
            t.mul_(6.0)
        elif name.endswith((".q.b", ".k.b", ".v.b", ".conv.b")):
            t.copy_(torch.randn(t.shape, generator=g) * 0.5)
        elif name.endswith("mix.q.norm") and peaked != 1.0:
            t.mul_(peaked)                   # the queries are normed: their gain, not their matrix, sets how sharp the scores are


@functools.lru_cache(maxsize=None)
def folder_of(name: str, seed: int = 1, std: float = 0.08, peaked: float = 1.0) -> str:
    from safetensors.torch import load_file, save_file
    folder = os.path.join(helpers.tmp_root(), f"nobonex_{name}_{seed}_{std}_{peaked}")
    ml.write_random_model(ModelConfig.from_dict(CONFIGS[name]), folder, seed, torch.bfloat16, std=std)
    path = os.path.join(folder, "model.safetensors")
    weights = {k: v.float() for k, v in load_file(path).items()}
    shape_weights(weights, seed, peaked)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, path)
    return folder


@functools.lru_cache(maxsize=None)
def oracle(folder: str):
    return pn.read_config(folder), pn.read_weights(folder, torch.float64)


def oracle_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    cfg, w = oracle(folder)
    return pn.forward(cfg, w, tokens).float()
