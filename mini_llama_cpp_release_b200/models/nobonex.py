"""Nobonex: a decoder whose config.json lists its layers, with an elementwise tanh norm before and behind every branch.

    x = E[token] · s_e
    per layer:  x <- x + m · T1b(mixer(T1(x)));   x <- x + m · T2b(ff(T2(x)))        (the second only with a feed-forward)
                T(v) = tanh(a · v) · w + b, entry by entry (no mean, no variance); m = residual_mult
    logits = W_head T_f(x)

Mixers: "attention" (queries and keys through a short convolution over time, values = the convolved keys, RMS norm over the
whole projection, rotation of neighbouring pairs: `parts/attention.py: ConvKeyAttention`), "attention_2" (biases, RMS norm per
head, rotate-half rotation with stretched frequencies, soft-capped scores, a mask of chunks, a sigmoid gate on the heads'
outputs, optionally the keys and values of an earlier layer: `parts/attention.py: SinkAttention` with those options) and
"mamba2" (`parts/recurrent.py: StateSpaceMixer`).
Feed-forwards: dense GEGLU (`parts/feed_forward.py: SwiGLU` with the tanh form of GELU), a mixture of clamped gated experts
routed by sigmoid scores whose weights multiply the experts' inputs (`parts/feed_forward.py: MixtureOfExperts`), or none.

config.json (every size and constant comes from it):
    architecture, vocab, width, residual_mult, embedding {scale}, norm {eps},
    layers[i]: type, mixer {...}, mlp {kind: "dense", ff} | {kind: "moe", expert {ff, limit}, router {experts, top}} | null
      attention:    heads, kv_heads, dim, vdim, conv, scale, rot {base, dims}
      attention_2:  heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims, scaling {factor, original, fast, slow}},
                    mask {size}, kv_from
      mamba2:       heads, vdim, state, groups, conv, norm_groups
Tensors: embed, head, final.norm{,.b,.alpha}, l<i>.norm1 / norm1b / norm2 / norm2b (each with .b and .alpha), l<i>.mix.<...>,
l<i>.mlp.<...>.  The model names no largest position; sequences are bounded by the cache alone.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from ..config.model_config import ConfigError, ModelConfig, as_int
from ..config.registry import register_architecture
from ..config.specs import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .mepolix import NO_POSITION_LIMIT, _count, _need, _number

MIXERS = ("attention", "attention_2", "mamba2")
EXPERT_SIGMOID_FACTOR = 1.702           # the experts' gate is g · sigmoid(1.702 g): fixed by the design


@dataclass(frozen=True, kw_only=True)
class NobonexConfig(ModelConfig):
    hidden_size: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    layers: Tuple[Dict[str, Any], ...]

    KEYS = ("vocab", "width", "norm", "layers", "residual_mult", "embedding")

    @classmethod
    def parse(cls, raw: Dict[str, Any]) -> "NobonexConfig":
        for key in ("vocab", "width", "layers", "norm"):
            if key not in raw:
                raise ConfigError(f"missing config key: {key}")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config key layers must be a list with at least one layer")
        shared = dict(cls.shared_fields({**raw, "vocab_size": raw["vocab"],
                                         "max_position_embeddings": raw.get("max_position_embeddings", NO_POSITION_LIMIT)}))
        emb = raw.get("embedding") or {}
        cfg = cls(**shared, hidden_size=as_int(raw, "width"), norm_eps=_number(raw["norm"], "eps", "norm"),
                  residual_mult=_number(raw, "residual_mult", "config") if raw.get("residual_mult") is not None else 1.0,
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
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in MIXERS:
                raise ConfigError(f"{where}.type must be one of {', '.join(MIXERS)}; got {kind!r}")
            m = _need(layer, "mixer", where)
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind", "dense") not in ("dense", "moe"):
                raise ConfigError(f"{where}.mlp.kind must be \"dense\" or \"moe\", got {mlp.get('kind')!r}")
            src = m.get("kv_from")
            if src is not None:
                if kind != "attention_2":
                    raise ConfigError(f"{where}.mixer.kv_from belongs to attention_2 layers")
                if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                    raise ConfigError(f"{where}.mixer.kv_from must name an earlier layer, got {src!r}")
                owner = self.layers[src]
                if owner.get("type") != "attention_2" or (owner.get("mixer") or {}).get("kv_from") is not None:
                    raise ConfigError(f"{where}.mixer.kv_from names layer {src}, which is no attention_2 layer with keys of its own")
                om = owner["mixer"]
                for key in ("kv_heads", "dim", "vdim"):
                    if om.get(key) != m.get(key):
                        raise ConfigError(f"{where}.mixer.{key} differs from layer {src}'s, whose keys and values it reads")

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "residual_mult": self.residual_mult, "embedding": {"scale": self.embedding_scale},
             "norm": {"eps": self.norm_eps}, "layers": [dict(l) for l in self.layers]}
        if self.max_position_embeddings != NO_POSITION_LIMIT:
            d["max_position_embeddings"] = self.max_position_embeddings
        d["torch_dtype"] = self.torch_dtype
        for key in ("bos_token_id", "eos_token_id"):
            v = getattr(self, key)
            if v is not None:
                d[key] = list(v) if isinstance(v, tuple) and len(v) > 1 else (v[0] if isinstance(v, tuple) else v)
        d.update(self.extra)
        return d


def _rotation(m: Dict[str, Any], where: str, pairing: str) -> PartSpec:
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    if not dims:
        return PartSpec("position", "rope_partial", dict(dims=0, base=1.0, scaling=None))
    if dims % 2 or dims > int(m["dim"]):
        raise ConfigError(f"{where}.rot.dims must be even and at most dim, got {dims}")
    return PartSpec("position", "rope_partial", dict(dims=dims, base=_number(rot, "base", where + ".rot"),
                                                     scaling=dict(rot["scaling"]) if rot.get("scaling") else None, pairing=pairing))


def _conv_attention(c: NobonexConfig, m: Dict[str, Any], where: str) -> PartSpec:
    dim = _count(m, "dim", where)
    if m.get("vdim") is not None and int(m["vdim"]) != dim:
        raise ConfigError(f"{where}.vdim must equal dim ({dim}): the values are the keys")
    return PartSpec("mixer", "conv_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), num_kv_heads=_count(m, "kv_heads", where), head_dim=dim,
        scale=_number(m, "scale", where), norm_eps=c.norm_eps, conv=_count(m, "conv", where),
        position=_rotation(m, where, "interleaved")))


def _mask_size(m: Dict[str, Any]) -> Optional[int]:
    size = (m.get("mask") or {}).get("size")
    return int(size) if size is not None else None


def _gated_attention(c: NobonexConfig, m: Dict[str, Any], where: str, keep_all_keys: bool = False) -> PartSpec:
    mask = m.get("mask") or {}
    return PartSpec("mixer", "sink_attention", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), num_kv_heads=_count(m, "kv_heads", where),
        head_dim=_count(m, "dim", where), v_head_dim=_count(m, "vdim", where), scale=_number(m, "scale", where),
        norm_eps=c.norm_eps, position=_rotation(m, where, "half"), qk_norm=True, sink=False, bias=True,
        softcap=_number(m, "softcap", where) if m.get("softcap") is not None else None,
        chunk=_count(mask, "size", where + ".mask") if mask.get("size") is not None else None,
        out_gate=True, own_kv=m.get("kv_from") is None, keep_all_keys=keep_all_keys))


def _state_space(c: NobonexConfig, m: Dict[str, Any], where: str) -> PartSpec:
    return PartSpec("mixer", "state_space", dict(
        hidden_size=c.hidden_size, num_heads=_count(m, "heads", where), v_head_dim=_count(m, "vdim", where),
        state=_count(m, "state", where), groups=_count(m, "groups", where), conv=_count(m, "conv", where),
        norm_eps=c.norm_eps, norm_groups=int(m.get("norm_groups") or 1)))


def _feed_forward(c: NobonexConfig, mlp: Dict[str, Any], where: str) -> PartSpec:
    if mlp.get("kind", "dense") == "dense":
        return PartSpec("feed_forward", "swiglu", dict(hidden_size=c.hidden_size, intermediate_size=_count(mlp, "ff", where),
                                                       activation="gelu_tanh", names={"gate": "gate", "up": "up", "down": "down"}))
    router, expert = _need(mlp, "router", where), _need(mlp, "expert", where)
    return PartSpec("feed_forward", "mixture", dict(
        hidden_size=c.hidden_size, intermediate_size=_count(expert, "ff", where + ".expert"),
        num_experts=_count(router, "experts", where + ".router"), top=_count(router, "top", where + ".router"),
        gated=True, activation="clamped", limit=_number(expert, "limit", where + ".expert"), act_alpha=EXPERT_SIGMOID_FACTOR,
        routing="sigmoid", router_bias=False, weight_on="input"))


@register_architecture("Nobonex", config_class=NobonexConfig)
def nobonex(config: NobonexConfig) -> ModelSpec:
    c = config
    norm = lambda tensor: PartSpec("norm", "dynamic_tanh", dict(size=c.hidden_size, tensor=tensor))
    builders = {"attention": _conv_attention, "attention_2": _gated_attention, "mamba2": _state_space}
    layers: List[LayerSpec] = []
    schedule: List[ScheduleEntry] = []
    # a layer whose keys another layer reads under another mask keeps all of them: its own mask's chunks may end elsewhere
    other_mask = {int(l["mixer"]["kv_from"]) for l in c.layers if l["mixer"].get("kv_from") is not None
                  and _mask_size(l["mixer"]) != _mask_size(c.layers[int(l["mixer"]["kv_from"])]["mixer"])}
    for i, layer in enumerate(c.layers):
        where = f"layers[{i}].mixer"
        mixer = (_gated_attention(c, layer["mixer"], where, keep_all_keys=i in other_mask) if layer["type"] == "attention_2"
                 else builders[layer["type"]](c, layer["mixer"], where))
        params: Dict[str, Any] = dict(
            mixer=mixer, mixer_norm=norm("norm1"),
            mixer_out_norm=norm("norm1b"), residual_mult=c.residual_mult,
            names={"mixer": "mix.", "mixer_norm": "", "mixer_out_norm": "", "feed_forward": "mlp.", "feed_forward_norm": "",
                   "feed_forward_out_norm": ""})
        if layer.get("mlp") is not None:
            params["feed_forward"] = _feed_forward(c, layer["mlp"], f"layers[{i}].mlp")
            params["feed_forward_norm"] = norm("norm2")
            params["feed_forward_out_norm"] = norm("norm2b")
        layers.append(LayerSpec(f"l{i}.", PartSpec("block", "sandwich", params)))
        # one run per layer, in order: a layer that names kv_from reads that layer's cache entry instead of keeping one
        schedule.append(ScheduleEntry(layer=i, reads_cache_of=layer["mixer"].get("kv_from")))
    return ModelSpec(
        config=c,
        embedding=PartSpec("embedding", "token_embedding", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="embed",
                                                                scale=c.embedding_scale)),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=c.vocab_size, hidden_size=c.hidden_size, tensor="head")),
        names={"embedding": "", "final_norm": "final.", "head": ""},
    )
