"""Shared by the Lonulix tests: small configurations of their own (sizes chosen so that nothing that could be equal is
equal: plain, rotated and value head sizes, the two latents' ranks, heads of the two mixers; windows that are no multiple
of a page, exactly a page, one token; norm groups of one and of several; factors of one and other than one; router
outputs that are no power of two, identity experts none and several, `top` of one and of all, one group and several),
model folders with random weights in which some tensors are set by hand so that what they do shows, and the comparison
with the plain implementation."""
from __future__ import annotations

import functools
import os
from typing import Dict, Sequence

import torch

import helpers
import mini_llama_cpp_release_b200 as ml
import plain_lonulix as pl
from kebesun_helpers import check  # noqa: F401  (the same bounds on rows of logits)
from mini_llama_cpp_release_b200.config import ModelConfig


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, window=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def hgrn2(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, identity=0, groups=None, scale=1.0):
    router = {"experts": experts, "top": top, "identity": identity, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def model(vocab, width, eps, groups, alpha, scale, layers):
    return {"architecture": "Lonulix", "vocab": vocab, "width": width, "norm": {"eps": eps, "groups": groups},
            "postln_alpha": alpha, "embedding": {"scale": scale}, "layers": layers}


# both mixers and all three feed-forwards; norm in three groups; a window of 40 and one of 70; six router outputs in three
# groups of which two are kept, one of them an identity expert
MIXED = model(300, 96, 1e-5, 3, 1.5, 2.5, [
    {"type": "latent_attention", "mlp": moe(48, 5, 2, identity=1, groups=(3, 2), scale=1.5),
     "mixer": latent(3, 24, 8, 20, 40, 28, 0.17, 3000.0, window=40)},
    {"type": "hgrn2", "mlp": dense(112), "mixer": hgrn2(3, 24, 40)},
    {"type": "hgrn2", "mlp": None, "mixer": hgrn2(2, 16, 24)},
    {"type": "latent_attention", "mlp": dense(64), "mixer": latent(4, 16, 16, 16, 32, 48, 0.25, 100.0, window=70)},
    {"type": "hgrn2", "mlp": moe(32, 4, 4, identity=4, groups=(2, 2), scale=0.7), "mixer": hgrn2(1, 40, 16)},
])

# cached rows of 64 and of 128 (the tensor-core attention kernels) under windows of 130 (over two pages) and of exactly a
# page; one norm group, both factors one; keys of 128 in the linear attention; eight router outputs in four pairs
WIDE = model(257, 128, 2e-6, 1, 1.0, 1.0, [
    {"type": "latent_attention", "mlp": moe(64, 6, 3, identity=2, groups=(4, 2), scale=0.5),
     "mixer": latent(2, 64, 16, 40, 48, 80, 0.1, 40000.0, window=130)},
    {"type": "hgrn2", "mlp": None, "mixer": hgrn2(2, 128, 64)},
    {"type": "latent_attention", "mlp": dense(144), "mixer": latent(4, 32, 32, 64, 96, 64, 0.11, 1e6, window=64)},
])

# sizes the fast paths do not take: a width that is no multiple of 8 in five groups, keys of 200, value heads of 36, a
# window of one token, a layer without a window, 33 experts in one group with one chosen and no identity expert, all of six
# router outputs chosen (three of them identity experts)
ODD = model(77, 100, 1e-5, 5, 0.5, 0.3, [
    {"type": "hgrn2", "mlp": moe(20, 33, 1), "mixer": hgrn2(2, 200, 36)},
    {"type": "latent_attention", "mlp": None, "mixer": latent(5, 12, 6, 10, 30, 18, 0.3, 50.0, window=1)},
    {"type": "latent_attention", "mlp": dense(36), "mixer": latent(1, 8, 4, 24, 12, 10, 0.4, 500.0, window=5)},
    {"type": "hgrn2", "mlp": moe(12, 3, 6, identity=3, groups=(2, 2), scale=3.0), "mixer": hgrn2(5, 8, 8)},
    {"type": "latent_attention", "mlp": None, "mixer": latent(2, 20, 2, 16, 24, 40, 0.2, 2.0)},
])

ONLY_LATENT = model(200, 64, 1e-5, 2, 2.0, 1.0, [{"type": "latent_attention", "mlp": None,
                                                  "mixer": latent(6, 20, 12, 28, 50, 36, 0.21, 700.0, window=33)}])
ONLY_HGRN2 = model(200, 64, 1e-5, 4, 1.0, 3.0, [{"type": "hgrn2", "mlp": None, "mixer": hgrn2(5, 40, 24)}])
ONLY_MOE = model(200, 64, 1e-5, 1, 2.0, 1.0, [{"type": "hgrn2", "mixer": hgrn2(1, 8, 8),
                                               "mlp": moe(40, 7, 3, identity=2, groups=(3, 2), scale=2.5)}])
ONLY_DENSE = model(200, 64, 1e-5, 2, 0.8, 1.0, [{"type": "hgrn2", "mixer": hgrn2(1, 8, 8), "mlp": dense(72)}])

# a latent of 280 with 24 rotated entries: cached rows of 304, above what the tensor-core attention kernels take
BIG_LATENT = model(120, 64, 1e-5, 2, 1.0, 1.0, [{"type": "latent_attention", "mlp": None,
                                                 "mixer": latent(2, 24, 24, 16, 280, 30, 0.2, 900.0, window=77)}])

CONFIGS = {"mixed": MIXED, "wide": WIDE, "odd": ODD, "latent": ONLY_LATENT, "hgrn2": ONLY_HGRN2, "moe": ONLY_MOE,
           "dense": ONLY_DENSE, "big_latent": BIG_LATENT}


def shape_weights(weights: Dict[str, torch.Tensor], seed: int, peaked: float = 1.0) -> None:
    """Random weights hide some faults.  The forget gates' biases are moved up (slow decays: tokens hundreds of places back
    still count), routers are made decisive (so that the chosen experts do not hang on the last bit) and their corrections
    as large as the scores (so that a choice by the scores alone, or weights that include the correction, are wrong), the
    branch gates' biases are spread out, and with `peaked` the attention's queries are scaled so that single keys decide
    rows."""
    g = torch.Generator().manual_seed(seed)
    for name, t in weights.items():
        if name.endswith(".f.b"):
            t.copy_(torch.randn(t.shape, generator=g) * 1.0 + 3.0)
        elif name.endswith(".router"):
            t.mul_(5.0)
        elif name.endswith(".correction"):
            t.copy_(torch.randn(t.shape, generator=g) * 0.2)
        elif name.endswith((".rg1.b", ".rg2.b")):
            t.copy_(torch.randn(t.shape, generator=g) * 1.5)
        elif name.endswith("mix.uq") and peaked != 1.0:
            t.mul_(peaked)


@functools.lru_cache(maxsize=None)
def folder_of(name: str, seed: int = 1, std: float = 0.08, peaked: float = 1.0) -> str:
    from safetensors.torch import load_file, save_file
    folder = os.path.join(helpers.tmp_root(), f"lonulix_{name}_{seed}_{std}_{peaked}")
    ml.write_random_model(ModelConfig.from_dict(CONFIGS[name]), folder, seed, torch.bfloat16, std=std)
    path = os.path.join(folder, "model.safetensors")
    weights = {k: v.float() for k, v in load_file(path).items()}
    shape_weights(weights, seed, peaked)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, path)
    return folder


@functools.lru_cache(maxsize=None)
def oracle(folder: str):
    return pl.read_config(folder), pl.read_weights(folder, torch.float64)


def oracle_logits(folder: str, tokens: Sequence[int]) -> torch.Tensor:
    cfg, w = oracle(folder)
    return pl.forward(cfg, w, tokens).float()
