"""SwiGLU feed-forward: down( gate·sigmoid(gate)·up ), no biases
(src/forward.cpp:672-702; src/ops.cpp:94-107).  Gate and up are one matrix product over
[Wgate; Wup]; the activation and the product are one kernel.  With `activation="gelu_tanh"` the
gate passes the tanh form of GELU instead (GEGLU)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec
from .linear import Linear




@register_part("feed_forward", "swiglu")
class SwiGLU(Part):
    graph_safe = True

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 names: Optional[dict] = None):
        """`names`: the three matrices' names below the part's prefix, by role ("gate", "up", "down")."""
        super().__init__(name, hidden_size=hidden_size, intermediate_size=intermediate_size, activation=activation, names=names)
        names = names or {}
        self.t_gate = name + names.get("gate", "gate_proj.weight")
        self.t_up = name + names.get("up", "up_proj.weight")
        self.t_down = name + names.get("down", "down_proj.weight")
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"feed-forward: the gate's activation is silu (src/ops.cpp:94-107) or gelu_tanh, got {activation!r}")
        self.activation = activation
        self.hidden, self.inter = int(hidden_size), int(intermediate_size)

    def tensors(self):
        return [
            TensorSpec(self.t_gate, (self.inter, self.hidden)),
            TensorSpec(self.t_up, (self.inter, self.hidden)),
            TensorSpec(self.t_down, (self.hidden, self.inter)),
        ]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        gate, up = get(self.t_gate), get(self.t_up)
        # The fused product (SiLU·mul inside the tcgen05 kernel's epilogue) wants gate_j and up_j on
        # neighbouring rows: g0, u0, g1, u1, ...  Otherwise the rows are [gate; up].
        self.fused = runtime.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16 \
            and self.hidden % 8 == 0
        if self.fused:
            w = torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden)
        else:
            w = torch.cat([gate, up], dim=0)
        self.gate_up = Linear(w, runtime)
        self.down = Linear(get(self.t_down), runtime)

    def weight_bytes(self) -> int:
        return self.gate_up.nbytes() + self.down.nbytes()

    accumulates = True        # forward(..., residual=x) may add the branch into the float32 stream and return None

    def forward(self, h: torch.Tensor, step=None, residual=None):
        rt = self.runtime
        a = rt.empty(h.shape[0], self.inter)
        if self.fused and kernels.gemm_rows_takes(h.shape[0], 2 * self.inter, self.hidden):
            kernels.gemm_prompt(h, self.gate_up.weight, a, kernels.bindings.EPI_SILU_MUL, n_sms=rt.n_sms, glu=self.activation)    # prompts
        elif self.fused:
            kernels.gemm_tcgen05(h, self.gate_up.weight, a, kernels.bindings.EPI_SILU_MUL, n_sms=rt.n_sms, glu=self.activation)
        elif self.activation != "silu":
            kernels.glu(self.gate_up(h, rt.dtype), a, self.activation, interleaved=self.fused)
        else:
            kernels.silu_mul(self.gate_up(h, rt.dtype), a, interleaved=self.fused)
        if residual is not None and self.down.can_add_into_stream(h.shape[0]):
            self.down.add_into(a, residual)
            return None
        return self.down(a, torch.float32, partial_ok=True)


@register_part("feed_forward", "mixture")
class MixtureOfExperts(Part):
    """A mixture of experts.  The output is the weighted sum of the chosen experts' outputs; experts have no biases.

    Experts: `gated=True`: SwiGLU, W_down (act(W_gate h) * W_up h); `gated=False`: W_down act(W_up h).  `activation`:
    "silu", "gelu" (with erf) or "gelu_tanh" (the gated form takes silu only).

    Routing, `routing="top_logits"`: router logits z = W_r h + b_r in float32; each token uses the `top` experts with the
    largest logits, weighted by the softmax over those chosen logits only.  `routing="scores"`: s = softmax(z) over all
    router outputs; chosen are the `top` largest s + correction (a stored per-expert term, `correction=True`) among the
    experts of the `group_keep` best of `group_count` equal groups of neighbours (a group's score is its largest choice
    score; one group: no grouping); the weights are s of the chosen (without the correction), divided by their sum
    + 1e-20, times `weight_scale`.  `identity`: that many further router outputs, behind the experts', belong to identity
    experts, which have no tensors and return their input; they take part in scores, groups and choice like the others.
    `routing="sigmoid"`: s = sigmoid(z); chosen are the `top` largest; the weights are the chosen scores as they are.

    `weight_on="input"`: a chosen expert's weight multiplies its input, not its output: the output is the plain sum of
    expert(w · h) over the chosen (for experts that are not linear in their input this is another function).

    Gated experts with `activation="clamped"` (`limit`, `act_alpha`): g = min(W_gate h, limit), u = clamp(W_up h, -limit,
    limit), W_down (g · sigmoid(act_alpha · g) · (u + 1)).

    On the device and without a word to the host: the step's (token, expert) pairs are sorted by expert into runs that
    start on tile borders (`kernels.moe_plan`), every run's rows are multiplied by that expert's matrices, and each
    token adds up its rows with its weights, in the order of its choices.

    `names`: the tensors' names below the part's prefix, by role: router, router_bias, correction, and the pattern of an
    expert's prefix (`expert`, with {e} for its number) before gate / up / down."""
    graph_safe = True

    NAMES = dict(router="router", router_bias="router.b", correction="correction", expert="e{e}.", gate="gate", up="up",
                 down="down")
    TILE = 64                        # rows per block of the grouped product; an expert's run is padded to it

    def __init__(self, name: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 router_bias: bool = True, names: Optional[dict] = None, gated: bool = True, activation: str = "silu",
                 routing: str = "top_logits", correction: bool = False, group_count: int = 1, group_keep: int = 1,
                 identity: int = 0, weight_scale: float = 1.0, weight_on: str = "output", limit: Optional[float] = None,
                 act_alpha: float = 1.0):
        super().__init__(name, hidden_size=hidden_size, intermediate_size=intermediate_size, num_experts=num_experts, top=top,
                         router_bias=router_bias, gated=gated, activation=activation, routing=routing, correction=correction,
                         group_count=group_count, group_keep=group_keep, identity=identity, weight_scale=weight_scale,
                         weight_on=weight_on, limit=limit, act_alpha=act_alpha)
        self.hidden, self.inter, self.E, self.top = int(hidden_size), int(intermediate_size), int(num_experts), int(top)
        self.identity = int(identity)
        self.outputs = self.E + self.identity                     # what the router puts out
        if self.E < 1 or self.identity < 0 or not 1 <= self.top <= self.outputs or self.top > 32 or self.outputs > 256:
            raise ValueError(f"mixture of experts: top {top} of {num_experts} experts (+ {identity} identity experts) is not "
                             f"supported (top <= 32, router outputs <= 256)")
        if routing not in ("top_logits", "scores", "sigmoid"):
            raise ValueError(f"mixture of experts: routing must be \"top_logits\", \"scores\" or \"sigmoid\", got {routing!r}")
        if gated and activation not in ("silu", "clamped"):
            raise ValueError(f"mixture of experts: activation {activation!r} is not supported by gated experts")
        if not gated and activation not in kernels.bindings.ACTIVATIONS:
            raise ValueError(f"mixture of experts: activation {activation!r} is not supported")
        if weight_on not in ("output", "input"):
            raise ValueError(f"mixture of experts: weight_on must be \"output\" or \"input\", got {weight_on!r}")
        self.limit, self.act_alpha = (float(limit) if limit is not None else 0.0), float(act_alpha)
        if activation == "clamped" and not self.limit > 0:
            raise ValueError(f"mixture of experts: clamped experts need a positive limit, got {limit}")
        self.weight_on_input = weight_on == "input"
        if self.weight_on_input and identity:
            raise ValueError("mixture of experts: identity experts with weights on the input are not supported")
        self.gated, self.activation, self.routing = bool(gated), activation, routing
        self.has_bias = bool(router_bias) and routing in ("top_logits", "sigmoid")
        self.has_correction = bool(correction)
        self.group_count, self.group_keep = max(1, int(group_count)), int(group_keep)
        self.weight_scale = float(weight_scale)
        if routing != "scores" and (self.identity or self.has_correction or self.group_count > 1 or self.weight_scale != 1.0):
            raise ValueError("mixture of experts: identity experts, a correction, groups and a weight scale belong to routing=\"scores\"")
        if self.group_count > 1:
            if self.outputs % self.group_count or not 1 <= self.group_keep <= self.group_count:
                raise ValueError(f"mixture of experts: {self.outputs} router outputs do not form {group_count} equal groups of "
                                 f"which {group_keep} are kept")
            if self.group_keep * (self.outputs // self.group_count) < self.top:
                raise ValueError(f"mixture of experts: {group_keep} groups of {self.outputs // self.group_count} hold fewer than top = {top} experts")
        self.t = {**self.NAMES, **(names or {})}

    def _expert(self, e: int, role: str) -> str:
        return self.name + self.t["expert"].format(e=e) + self.t[role]

    def tensors(self):
        specs = [TensorSpec(self.name + self.t["router"], (self.outputs, self.hidden))]
        if self.has_bias:
            specs.append(TensorSpec(self.name + self.t["router_bias"], (self.E,), role="bias"))
        if self.has_correction:
            specs.append(TensorSpec(self.name + self.t["correction"], (self.outputs,), role="bias"))
        for e in range(self.E):
            if self.gated:
                specs.append(TensorSpec(self._expert(e, "gate"), (self.inter, self.hidden)))
            specs += [TensorSpec(self._expert(e, "up"), (self.inter, self.hidden)),
                      TensorSpec(self._expert(e, "down"), (self.hidden, self.inter))]
        return specs

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.router = get(self.name + self.t["router"]).to(torch.float32).contiguous()        # the router is float32 in both modes
        self.router_bias = get(self.name + self.t["router_bias"]).to(torch.float32).contiguous() if self.has_bias else None
        self.correction = get(self.name + self.t["correction"]).to(torch.float32).contiguous() if self.has_correction else None
        # [E, 2*inter, hidden]: an expert's gate rows, then its up rows (ungated: [E, inter, hidden]); [E, hidden, inter]
        ups = [get(self._expert(e, "up")) for e in range(self.E)]
        self.down = torch.stack([get(self._expert(e, "down")) for e in range(self.E)]).contiguous()
        # The tensor-core form (bfloat16 engine, sizes the tcgen05 product takes): an expert's gate and up rows alternate,
        # g0, u0, g1, u1, ..., so that SiLU(gate)·up is the product's epilogue, and runs are padded to its tiles of 128
        # rows.  Otherwise float32 multiply-adds on [gate; up] with tiles of 64 rows.
        self.fused = (runtime.dtype == torch.bfloat16 and self.down.dtype == torch.bfloat16 and ups[0].dtype == torch.bfloat16
                      and self.hidden % 16 == 0 and self.inter % (8 if self.gated else 16) == 0)
        # the gated unit the grouped product's epilogue forms
        self.glu = ("clamped", self.limit, self.act_alpha) if self.activation == "clamped" else self.activation
        if not self.gated:
            self.gate_up = torch.stack(ups).contiguous()
        elif self.fused:
            gates = [get(self._expert(e, "gate")) for e in range(self.E)]
            self.gate_up = torch.stack([torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden)
                                        for g, u in zip(gates, ups)]).contiguous()
        else:
            gates = [get(self._expert(e, "gate")) for e in range(self.E)]
            self.gate_up = torch.stack([torch.cat([g, u], dim=0) for g, u in zip(gates, ups)]).contiguous()

    def weight_bytes(self) -> int:
        """Bytes a step of many tokens reads; a step of few tokens reads `top` experts per token at most."""
        return (self.gate_up.numel() * self.gate_up.element_size() + self.down.numel() * self.down.element_size()
                + self.router.numel() * 4)

    def flops_per_token(self) -> float:
        """Multiply-adds x 2 a token costs: the router and `top` experts."""
        return 2.0 * (self.outputs * self.hidden + self.top * (3 if self.gated else 2) * self.inter * self.hidden)

    def route(self, h: torch.Tensor):
        """(ids int32 [n, top], weights float32 [n, top]); an id of `num_experts` or more names an identity expert."""
        rt = self.runtime
        n = h.shape[0]
        ids = rt.empty(n, self.top, dtype=torch.int32)
        weights = rt.empty(n, self.top, dtype=torch.float32)
        if self.routing == "scores":
            kernels.moe_route_scored(h, self.router, self.correction, self.top, self.group_count, self.group_keep,
                                     self.weight_scale, ids, weights)
        else:
            # logits, choice and weights in one kernel
            kernels.moe_route(h, self.router_bias, self.top, ids, weights, router=self.router,
                              weighting="sigmoid" if self.routing == "sigmoid" else "softmax")
        return ids, weights

    defers_sum = True         # forward(..., deferred=True) may leave the weighted sum of a token's rows to the caller

    @property
    def sum_is_plain(self) -> bool:
        """Whether the deferred sum is the plain sum of a token's rows (the weights already acted on the experts' inputs)."""
        return self.weight_on_input

    def forward(self, h: torch.Tensor, step=None, residual=None, deferred: bool = False):
        """The mixture's output float32 [n, hidden]; with `deferred`, instead the pieces of its last step, (rows float32
        [sorted rows, hidden], row_of int32 [n, top], weights float32 [n, top]), for a caller whose own kernel adds
        sum_j weights[t, j] · rows[row_of[t, j]] into the stream (`kernels.scaled_add_experts`, `kernels.group_norm`); a
        negative row_of stands for the token's own input h (an identity expert)."""
        rt = self.runtime
        n = h.shape[0]
        ids, weights = self.route(h)
        tile = kernels.GROUPED_TILE if self.fused else self.TILE
        rows = kernels.moe_plan_rows(n * self.top, self.E, tile)
        row_of = rt.empty(n, self.top, dtype=torch.int32)
        src_tok = rt.empty(rows, dtype=torch.int32)
        tile_expert = rt.empty(rows // tile, dtype=torch.int32)
        kernels.moe_plan(ids, self.E, tile, row_of, src_tok, tile_expert)
        y = rt.empty(rows, self.hidden, dtype=torch.float32)
        act = rt.empty(rows, self.inter)
        on_input = (weights, row_of) if self.weight_on_input else (None, None)
        if self.fused:
            hs = rt.empty(rows, self.hidden)
            kernels.moe_gather(h, src_tok, hs, *on_input)            # the sorted rows, dense, as the product's TMA loads want them
            if self.gated:
                kernels.gemm_tcgen05_grouped(hs, self.gate_up, tile_expert, act, kernels.bindings.EPI_SILU_MUL, n_sms=rt.n_sms,
                                             glu=self.glu)
            else:
                kernels.gemm_tcgen05_grouped(hs, self.gate_up, tile_expert, act, kernels.bindings.EPI_ACT[self.activation], n_sms=rt.n_sms)
            kernels.gemm_tcgen05_grouped(act, self.down, tile_expert, y, kernels.bindings.EPI_STORE, n_sms=rt.n_sms)
        else:
            gu = rt.empty(rows, (2 if self.gated else 1) * self.inter)
            if self.weight_on_input:
                hs = rt.empty(rows, self.hidden)
                kernels.moe_gather(h, src_tok, hs, *on_input)
                kernels.grouped_linear(hs, None, self.gate_up, tile_expert, tile, gu)
            else:
                kernels.grouped_linear(h, src_tok, self.gate_up, tile_expert, tile, gu)
            if self.gated and self.activation != "silu":
                kernels.glu(gu, act, self.activation, limit=self.limit, alpha=self.act_alpha)
            elif self.gated:
                kernels.silu_mul(gu, act)
            else:
                kernels.activation(gu, self.activation, act)
            kernels.grouped_linear(act, None, self.down, tile_expert, tile, y)
        if deferred:
            return y, row_of, weights
        out = rt.empty(n, self.hidden, dtype=torch.float32)
        kernels.moe_combine(y, row_of, None if self.weight_on_input else weights, out, ident=h if self.identity else None)
        return out
