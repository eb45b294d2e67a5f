"""Lonulix: a decoder whose config.json lists its layers, with the norm behind each residual sum and a gate on each branch.

    x = E[token] · s_e
    per layer:  x <- N1(alpha · x + g1 * mixer(x));   x <- N2(alpha · x + g2 * ff(x))        (the second only with a feed-forward)
                g = sigmoid(W_g x + b_g), a gate of each branch's own on the branch's input
                N: RMS norm in `norm.groups` equal parts of the row, each by its own root mean square, times one gain
    logits = W_head N_f(x)

Mixers: "latent_attention" (queries through a normed latent, keys and values expanded from a cached normed latent, one
rotated key part shared by the heads with the rotation pairing neighbouring entries, a sliding window:
`parts/attention.py: LatentAttention`) and "hgrn2" (linear attention whose forget gate, bounded from below, also scales
what is written: `parts/recurrent.py: ForgetGateAttention`).
Feed-forwards: dense SwiGLU, or a mixture of ungated GELU experts routed by scores (softmax over all router outputs, a
correction on the choice, groups of experts of which the best are kept, identity experts, scaled weights:
`parts/feed_forward.py: MixtureOfExperts`), or none.

config.json (every size and constant comes from it):
    architecture, vocab, width, postln_alpha, embedding {scale}, norm {eps, groups},
    layers[i]: type, mixer {...}, mlp {kind: "dense", ff} | {kind: "moe", expert {ff}, router {experts, top, identity, scale,
               groups {count, keep}}} | null
      latent_attention:  heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, rot {base, dims}, mask {size}
      hgrn2:             heads, dim, vdim
Tensors: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.rg1, l<i>.rg1.b, l<i>.rg2, l<i>.rg2.b, l<i>.mix.<...>,
l<i>.mlp.<...>.  The model names no largest position; sequences are bounded by the cache alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from ..config.model_config import ConfigError, ModelConfig, as_int
from ..config.registry import register_architecture
from ..config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mepolix import NO_POSITION_LIMIT, _count, _need, _number

MIXERS = ("latent_attention", "hgrn2")


@dataclass(frozen=True, kw_only=True)
class LonulixConfig(ModelConfig):
    hidden_size: int
    norm_eps: float
    norm_groups: int
    alpha: float
    embedding_scale: float
    layers: Tuple[Dict[str, Any], ...]

    KEYS = ("vocab", "width", "norm", "layers", "postln_alpha", "embedding")

    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "LonulixConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config key layers must be a list with at least one layer")
        shared = dict(cls.shared_fields({**raw, "vocab_size": raw["vocab"],
                                         "max_position_embeddings": raw.get("max_position_embeddings", NO_POSITION_LIMIT)}))
        norm = raw["norm"]
        emb = raw.get("embedding") or {}
        cfg = cls(**shared, hidden_size=as_int(raw, "width"), norm_eps=_number(norm, "eps", "norm"),
                  norm_groups=int(norm.get("groups") or 1),
                  alpha=_number(raw, "postln_alpha", "config") if raw.get("postln_alpha") is not None else 1.0,
                  embedding_scale=_number(emb, "scale", "embedding") if emb.get("scale") is not None else 1.0,
                  layers=tuple(raw["layers"]),
                  extra={k: v for k, v in raw.items() if k not in cls.SHARED_KEYS and k not in cls.KEYS})
        cfg.validate()
        return cfg

    def validate(self) -> None:
        super().validate()
        if self.hidden_size <= 0:
            raise ConfigError(f"width must be positive, got {self.hidden_size}")
        if not self.norm_eps > 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.norm_groups < 1 or self.hidden_size % self.norm_groups:
            raise ConfigError(f"norm.groups must divide width ({self.hidden_size}), got {self.norm_groups}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}.type must be one of {', '.join(MIXERS)}; got {kind!r}")
            _need(layer, "mixer", where)
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") not in ("dense", "moe"):
                raise ConfigError(f"{where}.mlp.kind must be \"dense\" or \"moe\", got {mlp.get('kind')!r}")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "postln_alpha": self.alpha, "embedding": {"scale": self.embedding_scale},
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": [dict(l) for l in self.layers]}
        if self.max_position_embeddings != NO_POSITION_LIMIT:
            d["max_position_embeddings"] = self.max_position_embeddings
        d["torch_dtype"] = self.torch_dtype
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None:
                d[key] = list(v) if isinstance(v, tuple) and len(v) > 1 else (v[0] if isinstance(v, tuple) else v)
        d.update(self.extra)
        return d


def _latent(c: LonulixConfig, m: Dict[str, Any], where: str) -> PartSpec:
    rot_dim = int(_need(m, "rot_dim", where))
    rot = dict(m.get("rot") or {})
    if rot_dim and int(rot.get("dims", rot_dim)) != rot_dim:
        raise ConfigError(f"{where}.rot.dims must equal rot_dim ({rot_dim}), got {rot.get('dims')}")
    if rot_dim:
        position = PartSpec("position", "rope_partial", dict(dims=rot_dim, base=_number(rot, "base", where + ".rot"),
                                                             scaling=None, pairing="interleaved"))
    else:
        position = PartSpec("position", "rope_partial", dict(dims=0, base=1.0, scaling=None))
    mask = m.get("mask") or {}
    return PartSpec("mixer", "latent_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), head_dim=int(_need(m, "dim", where)), rot_dim=rot_dim,
        v_head_dim=_count(m, "vdim", where), kv_rank=_count(m, "kv_rank", where), q_rank=_count(m, "q_rank", where),
        scale=_number(m, "scale", where), norm_eps=c.norm_eps, position=position,
        window=_count(mask, "size", where + ".mask") if mask.get("size") is not None else None))


def _hgrn2(c: LonulixConfig, m: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("mixer", "forget_gate_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), head_dim=_count(m, "dim", where),
        v_head_dim=_count(m, "vdim", where), norm_eps=c.norm_eps))


def _feed_forward(c: LonulixConfig, mlp: Dict[str, Any], where: str) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=_count(mlp, "ff", where),
                                                       names={"gate": "gate", "up": "up", "down": "down"}))
    router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
    groups = router.get("groups") or {}
    count = _count(groups, "count", where + ".router.groups") if groups else 1
    return PartSpec("feed_forward", "mixture", dict(
        hidden_size=c.hidden_size, intermediate_size=_count(expert, "ff", where + ".expert"),
        num_experts=_count(router, "experts", where + ".router"), top=_count(router, "top", where + ".router"),
        gated=False, activation="gelu", routing="scores", correction=True, router_bias=False,
        group_count=count, group_keep=_count(groups, "keep", where + ".router.groups") if groups else 1,
        identity=int(router.get("identity") or 0),
        weight_scale=_number(router, "scale", where + ".router") if router.get("scale") is not None else 1.0))


@register_architecture("Lonulix", config_class=LonulixConfig)
def lonulix(config: LonulixConfig) -> ModelSpec:
    c = config
    norm = lambda tensor: PartSpec("norm", "rmsnorm_grouped", dict(size=c.hidden_size, eps=c.norm_eps, groups=c.norm_groups,
                                                                    tensor=tensor))
    builders = {"latent_attention": _latent, "hgrn2": _hgrn2}
    layers: List[LayerSpec] = []
    for i, layer in enumerate(c.layers):
        params: Dict[str, Any] = dict(
            mixer=builders[layer["type"]](c, layer["mixer"], f"layers[{i}].mixer"), mixer_norm=norm("norm1"),
            alpha=c.alpha, gated=True,
            names={"mixer": "mix.", "mixer_norm": "", "feed_forward": "mlp.", "feed_forward_norm": "",
                   "mixer_gate": "rg1", "mixer_gate_bias": "rg1.b", "feed_forward_gate": "rg2", "feed_forward_gate_bias": "rg2.b"})
        if layer.get("mlp") is not None:
            params["feed_forward"] = _feed_forward(c, layer["mlp"], f"layers[{i}].mlp")
            params["feed_forward_norm"] = norm("norm2")
        layers.append(LayerSpec(f"l{i}.", PartSpec("block", "post_norm", params)))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="embed",
                                                                scale=c.embedding_scale)),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
        final_norm=norm("norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="head")),
        names={"embedding": "", "final_norm": "final.", "head": ""},
    )
