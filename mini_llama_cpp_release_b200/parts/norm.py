"""RMSNorm, fused with the residual addition that precedes it.

y_i = x_i · 1/sqrt(mean(x²) + eps) · w_i: eps inside the square root, multiply order
x·scale·w, statistics in float32 (src/ops.cpp:19-41).  The reference adds a branch's
output to the residual stream with a separate pass (src/forward.cpp:772, 779); here that
addition rides in the next norm's kernel, in float32, and the stream itself stays float32.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part
from .base import Part, TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Part):
    graph_safe = True

    def __init__(self, name: str, size: int, eps: float, tensor: str = "weight", offset: float = 0.0):
        """`tensor`: the gain's name below the part's prefix.  `offset` is added to the stored values: a gain that is
        stored around zero and applied as 1 + w has offset 1."""
        super().__init__(name, size=size, eps=eps, tensor=tensor, offset=offset)
        self.size = int(size)
        self.eps = float(eps)
        self.offset = float(offset)
        self.tensor = self.name + tensor

    def tensors(self):
        return [TensorSpec(self.tensor, (self.size,), role="gain", init="normal" if self.offset else "one_plus_normal")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.gain = (get(self.tensor).to(torch.float32) + self.offset).contiguous()

    def weight_bytes(self) -> int:
        return self.gain.numel() * 4

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x: float32 [n, size], updated in place to x + delta when delta is given."""
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype)
        kernels.add_rmsnorm(x, delta, self.gain, self.eps, out)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Part):
    """Layer norm with a gain and no bias: (v - mean) / sqrt(var + eps) · w, var the mean of the squared deviations,
    statistics in float32.  Two uses: `forward`, the norm of the stream (as `RMSNorm.forward`: adds `delta` first),
    and `add_normed`, for arrangements that normalise a branch's output before it joins the stream.  `tensor` is the
    gain's name below the part's prefix."""
    graph_safe = True

    def __init__(self, name: str, size: int, eps: float, tensor: str = "weight"):
        super().__init__(name, size=size, eps=eps, tensor=tensor)
        self.size = int(size)
        self.eps = float(eps)
        self.tensor = self.name + tensor

    def tensors(self):
        return [TensorSpec(self.tensor, (self.size,), role="gain", init="one_plus_normal")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.gain = get(self.tensor).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.gain.numel() * 4

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x: float32 [n, size], updated in place to x + delta when delta is given; returns LN(x)."""
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype)
        kernels.layernorm(x, delta, self.gain, self.eps, out, of_branch=False)
        return out

    def add_normed(self, x: torch.Tensor, y: torch.Tensor, copy_dtype: Optional[torch.dtype] = None
                   ) -> Optional[torch.Tensor]:
        """x (float32 [n, size], in place) += LN(y), y float32 [n, size] or slices [s, n, size] that are added up first.
        With `copy_dtype`, also returns the new x in that type (the next part's input)."""
        out = self.runtime.empty(*x.shape, dtype=copy_dtype) if copy_dtype is not None else None
        kernels.layernorm(x, y, self.gain, self.eps, out, of_branch=True)
        return out


@register_part("norm", "rmsnorm_grouped")
class GroupRMSNorm(Part):
    """RMS norm in groups: the row is cut into `groups` equal consecutive parts, each divided by its own
    sqrt(mean(part²) + eps), and the whole row is multiplied by the gain.  One group is the ordinary RMS norm.  Two
    uses, as `LayerNorm` has: `forward`, the norm of the stream (adds `delta` first), and `renorm`, for arrangements
    that put the norm behind the residual sum.  `tensor` is the gain's name below the part's prefix."""
    graph_safe = True

    def __init__(self, name: str, size: int, eps: float, groups: int = 1, tensor: str = "weight"):
        super().__init__(name, size=size, eps=eps, groups=groups, tensor=tensor)
        self.size, self.eps, self.groups = int(size), float(eps), int(groups)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"norm in groups: {size} entries do not split into {groups} equal groups")
        self.tensor = self.name + tensor

    def tensors(self):
        return [TensorSpec(self.tensor, (self.size,), role="gain", init="one_plus_normal")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.gain = get(self.tensor).to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.gain.numel() * 4

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x: float32 [n, size], updated in place to x + delta when delta is given; returns the normed copy."""
        if delta is not None:
            x.add_(delta.sum(dim=0) if delta.dim() == 3 else delta)
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype)
        kernels.group_norm(x, self.groups, self.gain, self.eps, out=out)
        return out

    def renorm(self, x: torch.Tensor, alpha: float, y: Optional[torch.Tensor] = None, expert_rows=None,
               gate: Optional[torch.Tensor] = None, gate_col: int = 0, gate_bias: Optional[torch.Tensor] = None,
               copy_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """x (float32 [n, size], in place) <- norm(alpha · x + s * branch): the branch is `y` (float32 [n, size] or slices
        that are added up) or `expert_rows` (see `kernels.group_norm`); s = sigmoid(gate columns + gate_bias) if a gate
        is given, else one.  With `copy_dtype`, also returns the new x in that type (the next part's input)."""
        out = self.runtime.empty(*x.shape, dtype=copy_dtype) if copy_dtype is not None else None
        kernels.group_norm(x, self.groups, self.gain, self.eps, out=out, write_x=True, alpha=alpha, y=y, expert_rows=expert_rows,
                           gate=gate, gate_col=gate_col, gate_bias=gate_bias)
        return out


@register_part("norm", "dynamic_tanh")
class TanhNorm(Part):
    """The elementwise norm T(v) = tanh(a · v) · w + b ("Dynamic Tanh"; Zhu, Chen, He, LeCun, Liu, "Transformers without
    Normalization"): one stored number a, a gain w and a bias b per entry; no mean and no variance are taken.  Three uses:
    `forward`, the norm of the stream (as `RMSNorm.forward`: adds `delta` first, as it is); `add_normed`, for arrangements
    that norm a branch's output before it joins the stream, x += m · T(branch), optionally followed in the same kernel by
    another norm of this kind on the new stream (the next part's input); `triple`, the norm as data for such a kernel.
    `tensor` is the gain's name below the part's prefix; a and b are stored beside it as `<tensor>.alpha` and `<tensor>.b`."""
    graph_safe = True

    def __init__(self, name: str, size: int, tensor: str = "weight", alpha: str = ".alpha", bias: str = ".b"):
        super().__init__(name, size=size, tensor=tensor, alpha=alpha, bias=bias)
        self.size = int(size)
        self.tensor = self.name + tensor
        self.t_alpha, self.t_bias = self.tensor + alpha, self.tensor + bias

    def tensors(self):
        return [TensorSpec(self.tensor, (self.size,), role="gain", init="one_plus_normal"),
                TensorSpec(self.t_bias, (self.size,), role="bias"),
                TensorSpec(self.t_alpha, (), role="gain", init="one_plus_normal")]

    def bind(self, get, runtime):
        super().bind(get, runtime)
        self.gain = get(self.tensor).to(torch.float32).contiguous()
        self.bias = get(self.t_bias).to(torch.float32).contiguous()
        self.alpha = float(get(self.t_alpha).to(torch.float32).reshape(-1)[0].item())     # read once, at load

    def weight_bytes(self) -> int:
        return (self.gain.numel() + self.bias.numel() + 1) * 4

    def triple(self):
        return (self.alpha, self.gain, self.bias)

    def forward(self, x: torch.Tensor, delta: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """x: float32 [n, size], updated in place to x + delta when delta is given; returns T(x)."""
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype)
        kernels.tanh_norm(x, y=delta, next_norm=self.triple(), out=out)
        return out

    def add_normed(self, x: torch.Tensor, y: Optional[torch.Tensor] = None, expert_rows=None, mult: float = 1.0,
                   then: Optional["TanhNorm"] = None, out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """x (float32 [n, size], in place) += mult · T(branch); the branch is y (float32 [n, size], or slices that are added
        up first) or expert_rows = (rows, row_of), the plain sum of each token's expert rows.  With `then`, also returns
        then(x) of the new x in `out_dtype` (the engine's type by default)."""
        out = self.runtime.empty(*x.shape, dtype=out_dtype or self.runtime.dtype) if then is not None else None
        kernels.tanh_norm(x, y=y, expert_rows=expert_rows, branch_norm=self.triple(), mult=mult,
                          next_norm=then.triple() if then is not None else None, out=out)
        return out
