"""Mixers that keep a fixed-size state per sequence: the gated delta rule, the gated diagonal
linear recurrence, and the arrangement that runs two mixers side by side on one input.

What they share: every matrix that reads the mixer's input is a row range of one product
(`fused_rows`), whose float32 output the kernels of csrc/recurrent.cu read by column; whatever
enters a recurrence stays float32 in both engine modes (convolution inputs and outputs, unit
norms, decays, gates, the state); the state of a sequence is one row of float32 per slot, cut
into the pieces a mixer needs, zero when the slot is taken and carried from step to step.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..config.registry import build_part, register_part
from ..config.specs import PartSpec
from .attention import fused_rows
from .base import MixerMemory, Part, StateSpec, TensorSpec
from .linear import Linear


def _f32(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float32).contiguous()


@register_part("mixer", "gated_delta")
class GatedDeltaMixer(Part):
    """The gated delta rule (Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule").

        q, k = W_q h, W_k h (kv_heads x dim);  v = W_v h (heads x vdim);  head n reads q/k head n // (heads/kv_heads)
        each of q, k, v: causal convolution over time per channel (`conv` taps, no bias), then silu
        q, k: unit vectors per head, x / sqrt(sum x² + 1e-6);  q also times dim^-1/2
        beta = sigmoid(W_b h),  g = exp(-exp(A_log) · softplus(W_a h + dt_bias))           (one per head)
        per head:  S ← g S;  u = beta (v - Sᵀk);  S ← S + k uᵀ;  o = Sᵀq
        out = W_o ( o / rms(o) · w_norm · silu(W_g h) )                                      (rms over vdim, per head)

    State per sequence: S [heads, dim, vdim] and the last conv-1 inputs of the convolutions, all float32.
    `names`: the tensors' names below the part's prefix, by role."""
    graph_safe = True

    NAMES = dict(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", b="b", a="a", g="g", o="o",
                 A_log="A_log", dt_bias="dt_bias", norm="norm")

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 conv: int, norm_eps: float, names: Optional[dict] = None):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                         v_head_dim=v_head_dim, conv=conv, norm_eps=norm_eps)
        if num_heads % num_kv_heads:
            raise ValueError(f"gated delta rule: {num_heads} heads are not a multiple of {num_kv_heads} q/k heads")
        if not 1 <= head_dim <= 256:
            raise ValueError(f"gated delta rule: q/k head sizes up to 256 are supported, got {head_dim}")
        if conv < 1:
            raise ValueError("gated delta rule: the convolution needs at least one tap")
        self.hidden, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim, self.taps, self.eps = int(head_dim), int(v_head_dim), int(conv), float(norm_eps)
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}
        self.n_qk, self.n_v = self.G * self.dim, self.H * self.vdim
        self.n_conv = 2 * self.n_qk + self.n_v                       # channels that pass the convolution: q | k | v
        self.n_S = self.H * self.dim * self.vdim

    def tensors(self):
        t, hid = self.t, self.hidden
        return [TensorSpec(t["q"], (self.n_qk, hid)), TensorSpec(t["k"], (self.n_qk, hid)), TensorSpec(t["v"], (self.n_v, hid)),
                TensorSpec(t["q_conv"], (self.n_qk, self.taps)), TensorSpec(t["k_conv"], (self.n_qk, self.taps)),
                TensorSpec(t["v_conv"], (self.n_v, self.taps)),
                TensorSpec(t["b"], (self.H, hid)), TensorSpec(t["a"], (self.H, hid)), TensorSpec(t["g"], (self.n_v, hid)),
                TensorSpec(t["A_log"], (self.H,), role="bias"), TensorSpec(t["dt_bias"], (self.H,), role="bias"),
                TensorSpec(t["norm"], (self.vdim,), role="gain", init="one_plus_normal"),
                TensorSpec(t["o"], (hid, self.n_v))]

    def cache_need(self):
        return None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.n_S + (self.taps - 1) * self.n_conv,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        t = self.t
        # columns of the input product: q | k | v | g | b | a
        self.in_proj = fused_rows([get(t[r]) for r in ("q", "k", "v", "g", "b", "a")], runtime)
        self.g_col = self.n_conv
        self.b_col = self.g_col + self.n_v
        self.a_col = self.b_col + self.H
        self.conv_w = _f32(torch.cat([get(t["q_conv"]), get(t["k_conv"]), get(t["v_conv"])], dim=0))
        self.A_log, self.dt_bias, self.gain = _f32(get(t["A_log"])), _f32(get(t["dt_bias"])), _f32(get(t["norm"]))
        self.o = Linear(get(t["o"]), runtime)

    def weight_bytes(self) -> int:
        return self.in_proj.nbytes() + self.o.nbytes() + self.conv_w.numel() * 4

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        rt = self.runtime
        n = h.shape[0]
        proj = self.in_proj(h, torch.float32)
        S, conv_state = memory.state[:, :self.n_S], memory.state[:, self.n_S:]
        qkv = rt.empty(n, self.n_conv, dtype=torch.float32)
        kernels.causal_conv(proj, 0, self.conv_w, None, True, conv_state, step, qkv)
        o = rt.empty(n, self.n_v, dtype=torch.float32)
        kernels.gated_delta_rule(qkv, 0, self.n_qk, 2 * self.n_qk, proj, self.b_col, self.a_col, self.A_log, self.dt_bias,
                                 S, step, self.H, self.G, self.dim, self.vdim, o)
        act = rt.empty(n, self.n_v)
        kernels.gated_rmsnorm(o, proj, self.g_col, self.gain, self.eps, self.H, self.vdim, act)
        return self.o(act, torch.float32, partial_ok=True)


@register_part("mixer", "gated_linear_attention")
class GatedLinearAttention(Part):
    """Gated linear attention (Yang, Wang, Shen, Panda, Kim, "Gated Linear Attention Transformers with Hardware-Efficient
    Training"): per head a matrix memory S [dim, vdim] whose rows decay at rates of their own.

        q = W_q h · dim^-1/2,  k = W_k h  (heads x dim);   v = W_v h  (heads x vdim)
        a = sigmoid(W_a2 (W_a1 h) + b_a2)^(1/tau)          (heads x dim, a low-rank product; the rank is the tensors' own)
        S_t = diag(a_t) S_{t-1} + k_t v_tᵀ;   o_t = S_tᵀ q_t
        out = W_o ( o / rms(o) · w_norm · silu(W_g h) )     (rms over vdim per head, w_norm shared by the heads)

    State per sequence: S for every head, float32, zero at the start.  Decays, their logarithms and the whole
    recurrence are float32 in both engine modes.  `names`: the tensors' names below the part's prefix, by role."""
    graph_safe = True

    NAMES = dict(q="q", k="k", v="v", g="g", o="o", norm="norm", a1="a1", a2="a2", a2_bias="a2.b")
    DEFAULT_DECAY_RANK = 16          # what the random-weights mode writes when no tensor says

    def __init__(self, name: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float, norm_eps: float,
                 decay_rank: Optional[int] = None, names: Optional[dict] = None):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, head_dim=head_dim, v_head_dim=v_head_dim, tau=tau,
                         norm_eps=norm_eps, decay_rank=decay_rank)
        if not 1 <= head_dim <= 256:
            raise ValueError(f"gated linear attention: key sizes up to 256 are supported, got {head_dim}")
        if not tau > 0:
            raise ValueError(f"gated linear attention: tau must be positive, got {tau}")
        self.hidden, self.H, self.dim, self.vdim = int(hidden_size), int(num_heads), int(head_dim), int(v_head_dim)
        self.tau, self.eps = float(tau), float(norm_eps)
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}
        self.n_qk, self.n_v = self.H * self.dim, self.H * self.vdim

    def tensors(self):
        t, hid = self.t, self.hidden
        r = self.decay_rank if self.decay_rank else -1
        dr = self.decay_rank or self.DEFAULT_DECAY_RANK
        return [TensorSpec(t["q"], (self.n_qk, hid)), TensorSpec(t["k"], (self.n_qk, hid)), TensorSpec(t["v"], (self.n_v, hid)),
                TensorSpec(t["g"], (self.n_v, hid)), TensorSpec(t["o"], (hid, self.n_v)),
                TensorSpec(t["norm"], (self.vdim,), role="gain", init="one_plus_normal"),
                TensorSpec(t["a1"], (r, hid), default_shape=(dr, hid)),
                TensorSpec(t["a2"], (self.n_qk, r), default_shape=(self.n_qk, dr)),
                TensorSpec(t["a2_bias"], (self.n_qk,), role="bias")]

    def cache_need(self):
        return None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.H * self.vdim * self.dim,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        t = self.t
        a1, a2 = get(t["a1"]), get(t["a2"])
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"gated linear attention: {t['a1']} has {a1.shape[0]} rows but {t['a2']} has {a2.shape[1]} columns")
        self.rank = int(a1.shape[0])
        # columns of the input product: q | k | v | g | a1
        self.in_proj = fused_rows([get(t[r]) for r in ("q", "k", "v", "g")] + [a1], runtime)
        self.k_col, self.v_col = self.n_qk, 2 * self.n_qk
        self.g_col = self.v_col + self.n_v
        self.a_col = self.g_col + self.n_v
        self.a2 = a2.contiguous()
        self.a2_bias, self.gain = _f32(get(t["a2_bias"])), _f32(get(t["norm"]))
        self.o = Linear(get(t["o"]), runtime)

    def weight_bytes(self) -> int:
        return self.in_proj.nbytes() + self.o.nbytes() + self.a2.numel() * self.a2.element_size()

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        rt = self.runtime
        n = h.shape[0]
        proj = self.in_proj(h, torch.float32)
        z = rt.empty(n, self.n_qk, dtype=torch.float32)
        kernels.linear_simt(proj[:, self.a_col:self.a_col + self.rank].contiguous(), self.a2, z)
        # partial outputs, one slice per slab of the state's rows; the head norm adds them up as it reads them
        o = rt.empty(kernels.gla_slices(step.n_seqs, self.H, self.dim, self.vdim, rt.device), n, self.n_v, dtype=torch.float32)
        kernels.gla(proj, 0, self.k_col, self.v_col, z, self.a2_bias, self.tau, memory.state, step, self.H, self.dim, self.vdim, o)
        act = rt.empty(n, self.n_v)
        kernels.gated_rmsnorm(o, proj, self.g_col, self.gain, self.eps, self.H, self.vdim, act)
        return self.o(act, torch.float32, partial_ok=True)


@register_part("mixer", "forget_gate_attention")
class ForgetGateAttention(Part):
    """The forget-gate form of gated linear attention (the HGRN2 design): per head a matrix memory S [dim, vdim] whose rows
    decay by a forget gate with a lower bound, and what a row takes in is scaled by the gate's complement; there is no key.

        q = silu(W_q h)  (heads x dim);   v = W_v h  (heads x vdim)
        f = l + (1 - l) · sigmoid(W_f h + b_f)           (heads x dim; l the stored lower bound per channel)
        S_t = diag(f_t) S_{t-1} + (1 - f_t) v_tᵀ;   o_t = S_tᵀ q_t                (no further scale)
        out = W_o ( o / rms(o) · w_norm )                 (rms over vdim per head, w_norm shared by the heads)

    State per sequence: S for every head, float32, zero at the start.  Gates, their complements, silu(q) and the whole
    recurrence are float32 in both engine modes.  The walk over tokens is the one of `GatedLinearAttention`, with decay f,
    key 1 - f and query silu(z_q).  Without a lower-bound tensor (`lower_bound=False`) l = 0; `gate_bias=False`: no b_f.
    Offers `in_weights()`, `in_width()`, `mix()` and `o` to an arrangement that computes other matrices on the same input
    in the mixer's input product.  `names`: the tensors' names below the part's prefix, by role."""
    graph_safe = True

    NAMES = dict(q="q", f="f", f_bias="f.b", lower="lower", v="v", o="o", norm="norm")

    def __init__(self, name: str, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, norm_eps: float,
                 lower_bound: bool = True, gate_bias: bool = True, names: Optional[dict] = None):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, head_dim=head_dim, v_head_dim=v_head_dim,
                         norm_eps=norm_eps, lower_bound=lower_bound, gate_bias=gate_bias)
        if not 1 <= head_dim <= 256:
            raise ValueError(f"forget-gate linear attention: key sizes up to 256 are supported, got {head_dim}")
        self.hidden, self.H, self.dim, self.vdim = int(hidden_size), int(num_heads), int(head_dim), int(v_head_dim)
        self.eps = float(norm_eps)
        self.has_lower, self.has_bias = bool(lower_bound), bool(gate_bias)
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}
        self.n_qk, self.n_v = self.H * self.dim, self.H * self.vdim

    def tensors(self):
        t, hid = self.t, self.hidden
        specs = [TensorSpec(t["q"], (self.n_qk, hid)), TensorSpec(t["f"], (self.n_qk, hid)), TensorSpec(t["v"], (self.n_v, hid)),
                 TensorSpec(t["o"], (hid, self.n_v)), TensorSpec(t["norm"], (self.vdim,), role="gain", init="one_plus_normal")]
        if self.has_bias:
            specs.append(TensorSpec(t["f_bias"], (self.n_qk,), role="bias"))
        if self.has_lower:
            specs.append(TensorSpec(t["lower"], (self.n_qk,), role="bias", init="unit_interval"))
        return specs

    def cache_need(self):
        return None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.H * self.vdim * self.dim,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        t = self.t
        self._in = [get(t[r]) for r in ("q", "f", "v")]          # columns of the input product: q | f | v
        self.in_proj: Optional[Linear] = None
        self.f_bias = _f32(get(t["f_bias"])) if self.has_bias else None
        self.lower = _f32(get(t["lower"])) if self.has_lower else None
        self.gain = _f32(get(t["norm"]))
        self.o = Linear(get(t["o"]), runtime)

    def in_weights(self):
        return list(self._in)

    def in_width(self) -> int:
        return 2 * self.n_qk + self.n_v

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in self._in) + self.o.nbytes()

    def mix(self, proj: torch.Tensor, col: int, step, memory: MixerMemory) -> torch.Tensor:
        """From the float32 projection rows `proj`, whose columns from `col` on are [q | f | v]: the normed heads
        [n, heads·vdim] in the engine's type, the input of `self.o`."""
        rt = self.runtime
        n = proj.shape[0]
        # partial outputs, one slice per slab of the state's rows; the head norm adds them up as it reads them
        o = rt.empty(kernels.gla_slices(step.n_seqs, self.H, self.dim, self.vdim, rt.device), n, self.n_v, dtype=torch.float32)
        kernels.forget_gate_attention(proj, col, col + self.n_qk, col + 2 * self.n_qk, self.f_bias, self.lower, memory.state,
                                      step, self.H, self.dim, self.vdim, o)
        act = rt.empty(n, self.n_v)
        kernels.gated_rmsnorm(o, None, 0, self.gain, self.eps, self.H, self.vdim, act)
        return act

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        if self.in_proj is None:
            self.in_proj = fused_rows(self._in, self.runtime)
        return self.o(self.mix(self.in_proj(h, torch.float32), 0, step, memory), torch.float32, partial_ok=True)


@register_part("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Part):
    """The recurrent block of Griffin (De et al., "Griffin: Mixing Gated Linear Recurrences with Local Attention for
    Efficient Language Models") with its real-gated linear recurrent unit.  Two branches of `width` channels:

        y = gelu_tanh(W_y h + b_y);   u = conv(W_x h + b_x)        (causal, per channel, `conv` taps, with a bias)
        in each of `blocks` equal parts of the channels:  r = sigmoid(R u + b_r),  i = sigmoid(I u + b_i)
        a = exp(-c · r · softplus(lam)),  c = 8;   S_t = a S_{t-1} + sqrt(1 - a²) · i · u;   out = W_o (S · y)

    State per sequence: S [width] and the convolution's last conv-1 inputs, float32.  `out_scale` multiplies S·y in
    float32 before it is rounded for the output product.  Offers `in_weights()` and `mix()` like the attention."""
    graph_safe = True

    DECAY_CONSTANT = 8.0

    NAMES = dict(y="y", y_bias="y.b", x="x", x_bias="x.b", conv="conv", conv_bias="conv.b", r="ra", r_bias="ra.b", i="ri",
                 i_bias="ri.b", lam="lam", o="o")

    def __init__(self, name: str, hidden_size: int, width: int, blocks: int, conv: int, out_scale: float = 1.0,
                 names: Optional[dict] = None):
        super().__init__(name, hidden_size=hidden_size, width=width, blocks=blocks, conv=conv, out_scale=out_scale)
        if blocks < 1 or width % blocks:
            raise ValueError(f"linear recurrence: {width} channels do not divide into {blocks} equal parts")
        if conv < 1:
            raise ValueError("linear recurrence: the convolution needs at least one tap")
        self.hidden, self.W, self.B, self.taps = int(hidden_size), int(width), int(blocks), int(conv)
        self.out_scale = float(out_scale)
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}

    def tensors(self):
        t, W, bw = self.t, self.W, self.W // self.B
        return [TensorSpec(t["y"], (W, self.hidden)), TensorSpec(t["y_bias"], (W,), role="bias"),
                TensorSpec(t["x"], (W, self.hidden)), TensorSpec(t["x_bias"], (W,), role="bias"),
                TensorSpec(t["conv"], (W, self.taps)), TensorSpec(t["conv_bias"], (W,), role="bias"),
                TensorSpec(t["r"], (self.B, bw, bw)), TensorSpec(t["r_bias"], (self.B, bw), role="bias"),
                TensorSpec(t["i"], (self.B, bw, bw)), TensorSpec(t["i_bias"], (self.B, bw), role="bias"),
                TensorSpec(t["lam"], (W,), role="bias"), TensorSpec(t["o"], (self.hidden, W))]

    def cache_need(self):
        return None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.W * self.taps,), torch.float32)          # S, then taps-1 rows of inputs

    def bind(self, get, runtime):
        super().bind(get, runtime)
        t = self.t
        self._in = [get(t["y"]), get(t["x"])]
        self.in_proj: Optional[Linear] = None
        self.y_bias, self.x_bias = _f32(get(t["y_bias"])), _f32(get(t["x_bias"]))
        self.conv_w, self.conv_bias = _f32(get(t["conv"])), _f32(get(t["conv_bias"]))
        self.w_r, self.w_i = _f32(get(t["r"])), _f32(get(t["i"]))
        # for steps of one token per sequence: [block][in][out], so that neighbouring outputs lie side by side
        self.w_r_t, self.w_i_t = self.w_r.transpose(1, 2).contiguous(), self.w_i.transpose(1, 2).contiguous()
        self.one_token_form = kernels.gates_scan_step_takes(self.W, self.B)
        self.b_r, self.b_i = _f32(get(t["r_bias"])).view(-1), _f32(get(t["i_bias"])).view(-1)
        self.lam = _f32(get(t["lam"]))
        self.o = Linear(get(t["o"]), runtime)

    def in_weights(self):
        return list(self._in)

    def in_width(self) -> int:
        return 2 * self.W

    def weight_bytes(self) -> int:
        return (sum(w.numel() * w.element_size() for w in self._in) + self.o.nbytes()
                + 4 * (self.w_r.numel() + self.w_i.numel() + self.conv_w.numel()))

    def mix(self, proj: torch.Tensor, col: int, step, memory: MixerMemory) -> torch.Tensor:
        """From the float32 projection rows `proj`, whose columns from `col` on are [y | x]: S·y [n, width] in the engine's
        type, the input of `self.o`."""
        rt = self.runtime
        n, W = proj.shape[0], self.W
        S, conv_state = memory.state[:, :W], memory.state[:, W:]
        u = rt.empty(n, W, dtype=torch.float32)
        kernels.causal_conv(proj, col + W, self.conv_w, self.conv_bias, False, conv_state, step, u, in_bias=self.x_bias)
        act = rt.empty(n, W)
        if step.max_q_len == 1 and n == step.n_seqs and self.one_token_form:
            kernels.gates_scan_step(u, self.w_r_t, self.w_i_t, self.b_r, self.b_i, self.lam, self.DECAY_CONSTANT, proj, col,
                                    self.y_bias, S, step, self.out_scale, act)
            return act
        a, drive = rt.empty(n, W, dtype=torch.float32), rt.empty(n, W, dtype=torch.float32)
        kernels.block_gates(u, self.w_r, self.w_i, self.b_r, self.b_i, self.lam, self.DECAY_CONSTANT, a, drive)
        kernels.linear_scan(a, drive, proj, col, self.y_bias, S, step, self.out_scale, act)
        return act

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        if self.in_proj is None:
            self.in_proj = fused_rows(self._in, self.runtime)
        act = self.mix(self.in_proj(h, torch.float32), 0, step, memory)
        return self.o(act, torch.float32, partial_ok=True)


@register_part("mixer", "parallel")
class ParallelMixer(Part):
    """Two mixers side by side on the same input: out = left_scale · left(h) + right_scale · right(h).

    Both children offer `in_weights()` (the matrices that read h), `mix(proj, col, step, memory)` (everything between
    the input product and the output product) and `o` (the output product): the pair's input matrices are one
    product, and the two output products add up into one float32 result.  The factors reach the children as
    `value_scale` / `out_scale` parameters (the builder passes them), so they act in float32 inside the children's
    kernels.  The left child may keep keys and values, the right one a state: the pair asks the cache for both."""
    graph_safe = True

    def __init__(self, name: str, left: PartSpec, right: PartSpec, names: Optional[dict] = None):
        super().__init__(name)
        names = names or {}
        self.left = build_part(left, name + names.get("left", "left."))
        self.right = build_part(right, name + names.get("right", "right."))
        for side, part in (("left", self.left), ("right", self.right)):
            if not all(hasattr(part, a) for a in ("in_weights", "in_width", "mix")):
                raise ValueError(f"parallel mixer: the {side} mixer does not offer in_weights / in_width / mix")
        needs = [p.cache_need() for p in (self.left, self.right) if hasattr(p, "cache_need") and p.cache_need() is not None]
        states = [p.state_spec() for p in (self.left, self.right) if hasattr(p, "state_spec") and p.state_spec() is not None]
        if len(needs) > 1 or len(states) > 1:
            raise ValueError("parallel mixer: at most one child may keep keys and values, and at most one a state")

    def children(self):
        return (self.left, self.right)

    def cache_need(self):
        return next((n for n in (p.cache_need() for p in (self.left, self.right)) if n is not None), None)

    def state_spec(self):
        return next((s for s in (p.state_spec() for p in (self.left, self.right)) if s is not None), None)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.in_proj = fused_rows(self.left.in_weights() + self.right.in_weights(), runtime)
        self.right_col = self.left.in_width()

    def weight_bytes(self) -> int:
        return self.left.weight_bytes() + self.right.weight_bytes()

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        n = h.shape[0]
        proj = self.in_proj(h, torch.float32)
        a_left = self.left.mix(proj, 0, step, memory)
        a_right = self.right.mix(proj, self.right_col, step, memory)
        lo, ro = self.left.o, self.right.o
        if ro.can_add_into_stream(n) and a_right.dtype == torch.bfloat16:
            out = lo(a_left, torch.float32)
            ro.add_into(a_right, out)
            return out
        out = self.runtime.empty(2, n, lo.out_features, dtype=torch.float32)      # two slices; whoever reads them adds them up
        if a_left.dtype == torch.float32:
            kernels.linear_simt(a_left, lo.weight, out[0])
            kernels.linear_simt(a_right, ro.weight, out[1])
        else:
            out[0].copy_(lo(a_left, torch.float32))
            out[1].copy_(ro(a_right, torch.float32))
        return out


@register_part("mixer", "state_space")
class StateSpaceMixer(Part):
    """The state-space layer of Mamba-2 (Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms
    Through Structured State Space Duality").  With inner = heads x vdim, N = `state` and G = `groups`:

        [z | x | B | C | dt] = W_in h          (inner | inner | G·N | G·N | heads)
        [x | B | C] <- silu(conv([x | B | C]) + b_conv)     (causal, per channel, `conv` taps, the last one on the current token)
        dt <- softplus(dt + dt_bias)           (no clamp)
        per head n (group n // (heads / G)):  S_t = exp(-exp(A_log_n) dt) S_{t-1} + dt · B_t x_tᵀ;   y_t = S_tᵀ C_t + D_n x_t
        out = W_o ( rms_parts(y · silu(z)) · w_norm )      (the gate first; then `norm_groups` equal parts of the row, each
                                                            divided by its own root mean square)

    State per sequence: S [heads, vdim, N] and the convolution's last conv-1 inputs, float32, zero at the start.  Step sizes,
    decays, the convolution's outputs and the whole recurrence are float32 in both engine modes.  The walk over tokens is the
    one of `GatedLinearAttention` (one decay per head instead of one per key channel; keys and queries shared by a group's
    heads).  `names`: the tensors' names below the part's prefix, by role."""
    graph_safe = True

    NAMES = dict(w_in="in", conv="conv", conv_bias="conv.b", dt_bias="dt_bias", A_log="A_log", D="D", norm="norm", o="o")

    def __init__(self, name: str, hidden_size: int, num_heads: int, v_head_dim: int, state: int, groups: int, conv: int,
                 norm_eps: float, norm_groups: int = 1, names: Optional[dict] = None):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, v_head_dim=v_head_dim, state=state, groups=groups,
                         conv=conv, norm_eps=norm_eps, norm_groups=norm_groups)
        self.hidden, self.H, self.vdim, self.N, self.G = int(hidden_size), int(num_heads), int(v_head_dim), int(state), int(groups)
        self.taps, self.eps, self.norm_groups = int(conv), float(norm_eps), int(norm_groups)
        if self.G < 1 or self.H % self.G:
            raise ValueError(f"state-space layer: {num_heads} heads do not divide into {groups} groups")
        if not 1 <= self.N <= 256:
            raise ValueError(f"state-space layer: state sizes up to 256 are supported, got {state}")
        if self.taps < 1:
            raise ValueError("state-space layer: the convolution needs at least one tap")
        self.inner = self.H * self.vdim
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError(f"state-space layer: {self.inner} channels do not split into {norm_groups} equal parts")
        if self.inner * 4 > 48 * 1024:
            raise ValueError(f"state-space layer: up to 12288 inner channels are supported, got {self.inner}")
        self.n_conv = self.inner + 2 * self.G * self.N                # channels that pass the convolution: x | B | C
        self.n_S = self.inner * self.N
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}

    def tensors(self):
        t = self.t
        return [TensorSpec(t["w_in"], (2 * self.inner + 2 * self.G * self.N + self.H, self.hidden)),
                TensorSpec(t["conv"], (self.n_conv, self.taps)), TensorSpec(t["conv_bias"], (self.n_conv,), role="bias"),
                TensorSpec(t["dt_bias"], (self.H,), role="bias"), TensorSpec(t["A_log"], (self.H,), role="bias"),
                TensorSpec(t["D"], (self.H,), role="gain", init="one_plus_normal"),
                TensorSpec(t["norm"], (self.inner,), role="gain", init="one_plus_normal"),
                TensorSpec(t["o"], (self.hidden, self.inner))]

    def cache_need(self):
        return None

    def state_spec(self) -> StateSpec:
        return StateSpec((self.n_S + (self.taps - 1) * self.n_conv,), torch.float32)

    def bind(self, get, runtime):
        super().bind(get, runtime)
        t = self.t
        self.in_proj = fused_rows([get(t["w_in"])], runtime)                  # columns: z | x | B | C | dt
        self.conv_col = self.inner
        self.dt_col = self.inner + self.n_conv
        self.conv_w, self.conv_bias = _f32(get(t["conv"])), _f32(get(t["conv_bias"]))
        self.dt_bias, self.A_log, self.D, self.gain = (_f32(get(t[r])) for r in ("dt_bias", "A_log", "D", "norm"))
        self.o = Linear(get(t["o"]), runtime)

    def weight_bytes(self) -> int:
        return self.in_proj.nbytes() + self.o.nbytes() + self.conv_w.numel() * 4

    def forward(self, h: torch.Tensor, step, memory: MixerMemory) -> torch.Tensor:
        rt = self.runtime
        n = h.shape[0]
        proj = self.in_proj(h, torch.float32)
        S, conv_state = memory.state[:, :self.n_S], memory.state[:, self.n_S:]
        xbc = rt.empty(n, self.n_conv, dtype=torch.float32)
        kernels.causal_conv(proj, self.conv_col, self.conv_w, self.conv_bias, True, conv_state, step, xbc)
        act = rt.empty(n, self.inner)
        kernels.state_space(proj, 0, self.dt_col, xbc, self.inner, self.inner + self.G * self.N, self.dt_bias, self.A_log, self.D,
                            self.gain, self.eps, self.norm_groups, S, step, self.H, self.G, self.N, self.vdim, act)
        return self.o(act, torch.float32, partial_ok=True)
