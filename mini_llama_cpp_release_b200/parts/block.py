"""The arrangement of a layer's parts around the residual stream.

Pre-norm: x ← x + mixer(norm(x)); x ← x + feed_forward(norm(x)) (src/forward.cpp:726-780).
The additions are deferred: a branch's output travels as `pending` and is added, in
float32, by the next norm's kernel — the block's own second norm, the next block's first
norm, or the model's final norm.  On the tensor-core path of small steps the addition moves into
the preceding product's epilogue (atomic adds into the stream) and nothing is pending at all."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import kernels
from ..config.registry import register_part, build_part
from ..config.specs import PartSpec
from .base import MixerMemory, Part, TensorSpec


@register_part("block", "prenorm")
class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, name: str, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec, names: Optional[dict] = None):
        super().__init__(name)
        names = names or {}
        self.mixer_norm = build_part(mixer_norm, name + names.get("mixer_norm", "mixer_norm."))
        self.mixer = build_part(mixer, name + names.get("mixer", "mixer."))
        self.feed_forward_norm = build_part(feed_forward_norm, name + names.get("feed_forward_norm", "feed_forward_norm."))
        self.feed_forward = build_part(feed_forward, name + names.get("feed_forward", "feed_forward."))

    def children(self):
        return (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """A part either adds its output into the stream x itself (`accumulates`, asked through `residual=x`;
        it then returns None) or returns its output, which waits in `pending` for the next norm to add it."""
        mixer, ffn = self.mixer, self.feed_forward
        h = self.mixer_norm.forward(x, pending)
        a = mixer.forward(h, step, memory, residual=x) if getattr(mixer, "accumulates", False) else mixer.forward(h, step, memory)
        h2 = self.feed_forward_norm.forward(x, a)
        f = ffn.forward(h2, step, residual=x) if getattr(ffn, "accumulates", False) else ffn.forward(h2, step)
        return x, f


@register_part("block", "branch_norm")
class BranchNormBlock(Part):
    """Norm on each branch's output only: x ← x + norm(mixer(x)); x ← x + norm(feed_forward(x)).  The branches read
    the stream itself.  The feed-forward (with its norm) may be absent.

    The stream is float32.  An engine that computes in 16 bits gives the branches a 16-bit copy of it: the kernel
    that adds a normalised branch writes the copy of the new stream as well, and leaves it in the step's
    `handover` for whoever reads the stream next (the block's own feed-forward, or the next block of this kind);
    only a block that finds no copy there makes one."""
    graph_safe = True

    COPY = "stream_copy"

    def __init__(self, name: str, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 feed_forward_norm: Optional[PartSpec] = None, names: Optional[dict] = None):
        super().__init__(name)
        names = names or {}
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("branch_norm block: a feed-forward and its norm come together or not at all")
        self.mixer = build_part(mixer, name + names.get("mixer", "mixer."))
        self.mixer_norm = build_part(mixer_norm, name + names.get("mixer_norm", "mixer_norm."))
        self.feed_forward = build_part(feed_forward, name + names.get("feed_forward", "feed_forward.")) if feed_forward else None
        self.feed_forward_norm = (build_part(feed_forward_norm, name + names.get("feed_forward_norm", "feed_forward_norm."))
                                  if feed_forward_norm else None)

    def children(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm) if p is not None)

    def _input(self, x: torch.Tensor, step) -> torch.Tensor:
        """What a branch reads: the stream itself in a float32 engine, else its copy in the engine's type."""
        rt = self.runtime
        if rt.dtype == torch.float32:
            return x
        left = step.handover.pop(self.COPY, None)
        if left is not None and left[0] is x:
            return left[1]
        h = rt.empty(*x.shape)
        kernels.convert(x, h)
        return h

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        rt = self.runtime
        if pending is not None:                     # a block of another kind left a branch output to be added
            x.add_(pending.sum(dim=0) if pending.dim() == 3 else pending)
        copy_dtype = None if rt.dtype == torch.float32 else rt.dtype
        y = self.mixer.forward(self._input(x, step), step, memory)
        h = self.mixer_norm.add_normed(x, y, copy_dtype)
        if h is not None:
            step.handover[self.COPY] = (x, h)
        if self.feed_forward is not None:
            f = self.feed_forward.forward(self._input(x, step), step)
            h = self.feed_forward_norm.add_normed(x, f, copy_dtype)
            if h is not None:
                step.handover[self.COPY] = (x, h)
        return x, None


@register_part("block", "post_norm")
class PostNormBlock(Part):
    """Norm behind the sum: x <- N1(alpha · x + g1 * mixer(x)); x <- N2(alpha · x + g2 * feed_forward(x)).  The branches
    read the stream itself (the stream is what the norm before left).  alpha weighs the stream against the branch.  With
    `gated`, each branch's output is multiplied entry by entry by g = sigmoid(W_g x + b_g), a gate of the branch's own
    computed from the branch's input (tensors `mixer_gate`, `mixer_gate_bias`, `feed_forward_gate`,
    `feed_forward_gate_bias`); without, g = 1.  The feed-forward (with its norm and gate) may be absent.

    The stream is float32 and so are the gate, the sum and the norm: one kernel (`kernels.group_norm`) forms
    alpha · x + sigmoid(z + b) * branch, norms it, writes the stream back and, for an engine that computes in 16 bits, the
    16-bit copy that the next branch reads (handed on in the step's `handover`, as the branch-norm block does).  The gate's
    matrix rides in the mixer's input product when the mixer offers `in_weights / mix / o` (one product over
    [W_g ; the mixer's own matrices]).  A mixture of experts that defers its weighted sum has it made by the same kernel."""
    graph_safe = True

    COPY = BranchNormBlock.COPY

    def __init__(self, name: str, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 feed_forward_norm: Optional[PartSpec] = None, alpha: float = 1.0, gated: bool = False,
                 names: Optional[dict] = None):
        super().__init__(name, alpha=alpha, gated=gated)
        names = names or {}
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("post_norm block: a feed-forward and its norm come together or not at all")
        self.alpha, self.gated = float(alpha), bool(gated)
        self.mixer = build_part(mixer, name + names.get("mixer", "mixer."))
        self.mixer_norm = build_part(mixer_norm, name + names.get("mixer_norm", "mixer_norm."))
        self.feed_forward = build_part(feed_forward, name + names.get("feed_forward", "feed_forward.")) if feed_forward else None
        self.feed_forward_norm = (build_part(feed_forward_norm, name + names.get("feed_forward_norm", "feed_forward_norm."))
                                  if feed_forward_norm else None)
        for norm in (self.mixer_norm, self.feed_forward_norm):
            if norm is not None and not hasattr(norm, "renorm"):
                raise ValueError("post_norm block: its norms must offer `renorm` (the norm of a gated residual sum)")
        self.size = self.mixer_norm.size
        self.t = {k: name + names.get(k, k) for k in ("mixer_gate", "mixer_gate_bias", "feed_forward_gate", "feed_forward_gate_bias")}

    def children(self):
        return tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.feed_forward_norm) if p is not None)

    def tensors(self):
        if not self.gated:
            return []
        d, t = self.size, self.t
        specs = [TensorSpec(t["mixer_gate"], (d, d)), TensorSpec(t["mixer_gate_bias"], (d,), role="bias")]
        if self.feed_forward is not None:
            specs += [TensorSpec(t["feed_forward_gate"], (d, d)), TensorSpec(t["feed_forward_gate_bias"], (d,), role="bias")]
        return specs

    def bind(self, get, runtime):
        super().bind(get, runtime)
        from .attention import fused_rows
        from .linear import Linear
        self.gate1 = self.gate2 = self.b1 = self.b2 = self.joint = None
        self.side_by_side = all(hasattr(self.mixer, a) for a in ("in_weights", "mix", "o"))
        if self.gated:
            w1 = get(self.t["mixer_gate"])
            self.b1 = get(self.t["mixer_gate_bias"]).to(torch.float32).contiguous()
            if self.side_by_side:
                self.joint = fused_rows([w1] + list(self.mixer.in_weights()), runtime)       # [gate | the mixer's columns]
            else:
                self.gate1 = Linear(w1, runtime)
            if self.feed_forward is not None:
                self.gate2 = Linear(get(self.t["feed_forward_gate"]), runtime)
                self.b2 = get(self.t["feed_forward_gate_bias"]).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        own = sum(l.nbytes() for l in (self.gate1, self.gate2) if l is not None)
        if self.joint is not None:
            own += self.size * self.size * self.joint.weight.element_size()
        return super().weight_bytes() + own + sum(b.numel() * 4 for b in (self.b1, self.b2) if b is not None)

    def _input(self, x: torch.Tensor, step) -> torch.Tensor:
        """What a branch reads: the stream itself in a float32 engine, else its copy in the engine's type."""
        rt = self.runtime
        if rt.dtype == torch.float32:
            return x
        left = step.handover.pop(self.COPY, None)
        if left is not None and left[0] is x:
            return left[1]
        h = rt.empty(*x.shape)
        kernels.convert(x, h)
        return h

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        rt = self.runtime
        if pending is not None:                     # a block of another kind left a branch output to be added
            x.add_(pending.sum(dim=0) if pending.dim() == 3 else pending)
        copy_dtype = None if rt.dtype == torch.float32 else rt.dtype
        h = self._input(x, step)
        gate, gate_col = None, 0
        if self.joint is not None:
            proj = self.joint(h, torch.float32)
            y = self.mixer.o(self.mixer.mix(proj, self.size, step, memory), torch.float32, partial_ok=True)
            gate = proj
        else:
            if self.gate1 is not None:
                gate = self.gate1(h, torch.float32)
            y = self.mixer.forward(h, step, memory)
        h = self.mixer_norm.renorm(x, self.alpha, y=y, gate=gate, gate_col=gate_col, gate_bias=self.b1, copy_dtype=copy_dtype)
        if h is not None:
            step.handover[self.COPY] = (x, h)
        ff = self.feed_forward
        if ff is not None:
            h = self._input(x, step)
            gate = self.gate2(h, torch.float32) if self.gate2 is not None else None
            if getattr(ff, "defers_sum", False):
                # a mixture of experts: the weighted sum of a token's expert rows is made by the kernel that norms
                rows, row_of, weights = ff.forward(h, step, deferred=True)
                h = self.feed_forward_norm.renorm(x, self.alpha, expert_rows=(rows, row_of, weights, h if getattr(ff, "identity", 0) else None),
                                                  gate=gate, gate_bias=self.b2, copy_dtype=copy_dtype)
            else:
                h = self.feed_forward_norm.renorm(x, self.alpha, y=ff.forward(h, step), gate=gate, gate_bias=self.b2,
                                                  copy_dtype=copy_dtype)
            if h is not None:
                step.handover[self.COPY] = (x, h)
        return x, None


@register_part("block", "parallel")
class ParallelBlock(Part):
    """One norm, two branches that both read it: h = norm(x); x <- x + s1 * mixer(h) + s2 * feed_forward(h).
    s1 and s2 are per-channel factors ("layer scale") stored as tensors; without them the factors are one.  The
    feed-forward may be absent.  The sum is float32: the branches return float32 (or partial sums), and one kernel
    multiplies, adds them up and adds them into the stream."""
    graph_safe = True

    def __init__(self, name: str, mixer: PartSpec, norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 layer_scale: bool = False, names: Optional[dict] = None):
        super().__init__(name, layer_scale=layer_scale)
        names = names or {}
        self.norm = build_part(norm, name + names.get("norm", "norm."))
        self.mixer = build_part(mixer, name + names.get("mixer", "mixer."))
        self.feed_forward = build_part(feed_forward, name + names.get("feed_forward", "feed_forward.")) if feed_forward else None
        self.layer_scale = bool(layer_scale)
        self.t_s1 = name + names.get("mixer_scale", "mixer_scale")
        self.t_s2 = name + names.get("feed_forward_scale", "feed_forward_scale")
        self.s1 = self.s2 = None

    def children(self):
        return tuple(p for p in (self.norm, self.mixer, self.feed_forward) if p is not None)

    def tensors(self):
        if not self.layer_scale:
            return []
        size = self.norm.size
        specs = [TensorSpec(self.t_s1, (size,), role="gain", init="one_plus_normal")]
        if self.feed_forward is not None:
            specs.append(TensorSpec(self.t_s2, (size,), role="gain", init="one_plus_normal"))
        return specs

    def bind(self, get, runtime):
        super().bind(get, runtime)
        if self.layer_scale:
            self.s1 = get(self.t_s1).to(torch.float32).contiguous()
            self.s2 = get(self.t_s2).to(torch.float32).contiguous() if self.feed_forward is not None else None

    def weight_bytes(self) -> int:
        return super().weight_bytes() + sum(s.numel() * 4 for s in (self.s1, self.s2) if s is not None)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        h = self.norm.forward(x, pending)
        y = self.mixer.forward(h, step, memory)
        ff = self.feed_forward
        if ff is not None and getattr(ff, "defers_sum", False):
            # a mixture of experts: the weighted sum of a token's expert rows is made by the kernel that adds the branches
            rows, row_of, weights = ff.forward(h, step, deferred=True)
            kernels.scaled_add_experts(x, y, self.s1, rows, row_of, weights, self.s2)
            return x, None
        f = ff.forward(h, step) if ff is not None else None
        kernels.scaled_add(x, y, self.s1, f, self.s2)
        return x, None


@register_part("block", "stream_mix")
class StreamMix(Part):
    """Not a layer but a step between layers: x <- W [x ; e], with e the embedding's output of the step's tokens and W
    [size, 2 size] (the stream's columns first).  A model that walks a run of its layers several times places one
    before each walk.  It keeps nothing per sequence.  The model's step function leaves e in the step's `handover`
    under `EMBEDDING` when a block asks for it (`reads_embedding`)."""
    graph_safe = True
    reads_embedding = True
    EMBEDDING = "embedding_output"

    def __init__(self, name: str, size: int, tensor: str = "weight"):
        super().__init__(name, size=size, tensor=tensor)
        self.size = int(size)
        self.tensor = name + tensor

    def tensors(self):
        return [TensorSpec(self.tensor, (self.size, 2 * self.size))]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        from .linear import Linear
        self.w = Linear(get(self.tensor), runtime)

    def weight_bytes(self) -> int:
        return self.w.nbytes()

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        if pending is not None:
            x.add_(pending.sum(dim=0) if pending.dim() == 3 else pending)
        e = step.handover[self.EMBEDDING]
        both = self.runtime.empty(x.shape[0], 2 * self.size)
        both[:, :self.size].copy_(x)
        both[:, self.size:].copy_(e)
        return self.w(both, torch.float32), None


class DeferredBranch:
    """A branch output that a block left for whoever reads the stream next: x += mult · norm(branch) is still to be done.
    The next block of the same kind does it inside its own first norm's kernel; anybody else calls `finish()`."""

    def __init__(self, x: torch.Tensor, norm, mult: float, y: Optional[torch.Tensor] = None, expert_rows=None):
        self.x, self.norm, self.mult, self.y, self.expert_rows = x, norm, mult, y, expert_rows

    def finish(self) -> None:
        self.norm.add_normed(self.x, y=self.y, expert_rows=self.expert_rows, mult=self.mult)


DEFERRED = "deferred_update"          # the key under which a `DeferredBranch` waits in a step's `handover`


def finish_deferred(step) -> None:
    """Carry out the stream update a block may have left in the step's `handover`."""
    left = step.handover.pop(DEFERRED, None)
    if left is not None:
        left.finish()


@register_part("block", "sandwich")
class SandwichBlock(Part):
    """A norm before and a norm behind each branch: x <- x + m · Nb(mixer(Na(x))); x <- x + m · Nd(feed_forward(Nc(x))), with
    m one number (`residual_mult`).  The feed-forward (with its two norms) may be absent.

    The norms are of a kind that offers `add_normed(x, branch, mult, then)` and `triple()` (the elementwise tanh norm): the
    addition of a normed branch and the norm that the next branch reads are one kernel.  The layer's last addition is left
    in the step's `handover` as a `DeferredBranch` for the next block of this kind, whose first norm's kernel carries it
    out; the model's step function finishes it where no such block follows (`takes_deferred_update`).  A mixture of experts
    that defers its sum has its rows added up by the same kernel."""
    graph_safe = True
    takes_deferred_update = True

    def __init__(self, name: str, mixer: PartSpec, mixer_norm: PartSpec, mixer_out_norm: PartSpec,
                 feed_forward: Optional[PartSpec] = None, feed_forward_norm: Optional[PartSpec] = None,
                 feed_forward_out_norm: Optional[PartSpec] = None, residual_mult: float = 1.0, names: Optional[dict] = None):
        super().__init__(name, residual_mult=residual_mult)
        names = names or {}
        if not ((feed_forward is None) == (feed_forward_norm is None) == (feed_forward_out_norm is None)):
            raise ValueError("sandwich block: a feed-forward and its two norms come together or not at all")
        self.mult = float(residual_mult)

        def make(spec, role):
            return build_part(spec, name + names.get(role, role + ".")) if spec is not None else None
        self.mixer_norm, self.mixer, self.mixer_out_norm = make(mixer_norm, "mixer_norm"), make(mixer, "mixer"), make(mixer_out_norm, "mixer_out_norm")
        self.feed_forward_norm, self.feed_forward = make(feed_forward_norm, "feed_forward_norm"), make(feed_forward, "feed_forward")
        self.feed_forward_out_norm = make(feed_forward_out_norm, "feed_forward_out_norm")
        for norm in (self.mixer_norm, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward_out_norm):
            if norm is not None and not (hasattr(norm, "add_normed") and hasattr(norm, "triple")):
                raise ValueError("sandwich block: its norms must offer `add_normed` and `triple`")

    def children(self):
        return tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.feed_forward_norm, self.feed_forward,
                                 self.feed_forward_out_norm) if p is not None)

    def forward(self, x: torch.Tensor, pending: Optional[torch.Tensor], step, memory: MixerMemory
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        left = step.handover.pop(DEFERRED, None)
        if left is not None and left.x is x and pending is None:
            # the block before left its last addition: it and this block's first norm are one kernel
            h = left.norm.add_normed(x, y=left.y, expert_rows=left.expert_rows, mult=left.mult, then=self.mixer_norm)
        else:
            if left is not None:
                left.finish()
            h = self.mixer_norm.forward(x, pending)
        y = self.mixer.forward(h, step, memory)
        ff = self.feed_forward
        if ff is None:
            step.handover[DEFERRED] = DeferredBranch(x, self.mixer_out_norm, self.mult, y=y)
            return x, None
        h = self.mixer_out_norm.add_normed(x, y=y, mult=self.mult, then=self.feed_forward_norm)
        if getattr(ff, "defers_sum", False) and getattr(ff, "sum_is_plain", False):
            rows, row_of, _ = ff.forward(h, step, deferred=True)
            step.handover[DEFERRED] = DeferredBranch(x, self.feed_forward_out_norm, self.mult, expert_rows=(rows, row_of))
        else:
            step.handover[DEFERRED] = DeferredBranch(x, self.feed_forward_out_norm, self.mult, y=ff.forward(h, step))
        return x, None
