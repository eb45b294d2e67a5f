"""Grouped-query attention over the paged cache.

q = Wq·h + bq, k = Wk·h + bk, v = Wv·h + bv (bias only if the checkpoint has it); heads are
contiguous slices of the projection; q and k are rotated after the bias and before the
cache write; query head h reads kv head h // (H/KV); score = (q·k)·1/sqrt(hd) over keys
0..p (or the last `window` of them); softmax; weighted sum of values; output projection
without bias (src/forward.cpp:293-335, 524-526, 553, 585-611, 742-772).

Differences of form, not of arithmetic: the three projections are one matrix product over
[Wq; Wk; Wv]; bias, rotation and the cache write are one kernel; all tokens of a step, of
all sequences, run at once against the cache.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import kernels
from ..config.registry import register_part, build_part
from ..config.specs import PartSpec
from .base import CacheNeed, MixerMemory, Part, TensorSpec
from .linear import Linear


@register_part("mixer", "gqa_attention")
class GQAttention(Part):
    graph_safe = True

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, window: Optional[int] = None, scale: Optional[float] = None,
                 out_bias: bool = False):
        super().__init__(name, hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads,
                         head_dim=head_dim, qkv_bias=qkv_bias, window=window, scale=scale)
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        if head_dim > 256:
            raise ValueError(f"attention: head sizes up to 256 are supported, got {head_dim}")
        if out_bias:
            raise ValueError("attention: an output-projection bias is not supported")
        self.hidden, self.H, self.KV, self.hd = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.qkv_bias = bool(qkv_bias)
        self.window = int(window) if window else None
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))   # src/forward.cpp:585
        self.position = build_part(position, name)

    def children(self):
        return (self.position,)

    # ---- what it asks of the checkpoint and of the cache
    def tensors(self):
        n = self.name
        specs = [
            TensorSpec(n + "q_proj.weight", (self.H * self.hd, self.hidden)),
            TensorSpec(n + "k_proj.weight", (self.KV * self.hd, self.hidden)),
            TensorSpec(n + "v_proj.weight", (self.KV * self.hd, self.hidden)),
            TensorSpec(n + "o_proj.weight", (self.hidden, self.H * self.hd)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(n + "q_proj.bias", (self.H * self.hd,), role="bias"),
                TensorSpec(n + "k_proj.bias", (self.KV * self.hd,), role="bias"),
                TensorSpec(n + "v_proj.bias", (self.KV * self.hd,), role="bias"),
            ]
        return specs

    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window else "all", self.KV, self.hd, self.window)

    def state_spec(self):
        return None

    def bind(self, get, runtime):
        super().bind(get, runtime)
        n = self.name
        wq, wk, wv = get(n + "q_proj.weight"), get(n + "k_proj.weight"), get(n + "v_proj.weight")
        w = torch.cat([wq, wk, wv], dim=0)
        if self.qkv_bias:
            bias = torch.cat([get(n + "q_proj.bias"), get(n + "k_proj.bias"), get(n + "v_proj.bias")]).to(torch.float32)
        else:
            bias = None
        # The fused projection (bias, rotation and cache write inside the tcgen05 kernel's epilogue)
        # wants each head's rows in the order (0, hd/2, 1, hd/2+1, ...): rotation partners then sit
        # on neighbouring accumulator lanes.
        self.fused = (runtime.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and self.hidden % 8 == 0
                      and getattr(self.position, "fusable", False))
        if self.fused:
            half = self.hd // 2
            within = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1)
            order = (torch.arange(self.H + 2 * self.KV)[:, None] * self.hd + within[None, :]).reshape(-1).to(w.device)
            w = w[order]
            bias = bias[order] if bias is not None else None
        self.qkv = Linear(w, runtime)
        self.bias = bias.contiguous() if bias is not None else None
        self.q_only: Optional[Linear] = None                    # made when a run reads another run's cache
        self.o = Linear(get(n + "o_proj.weight"), runtime)
        self.use_tensor_cores = runtime.dtype == torch.bfloat16 and self.hd % 16 == 0
        if self.use_tensor_cores:
            kernels.attention_library(self.hd)          # compiled now, for this model's head size, not at the first step

    def weight_bytes(self) -> int:
        b = self.qkv.nbytes() + self.o.nbytes()
        return b + (self.bias.numel() * 4 if self.bias is not None else 0)

    # ---- the step
    accumulates = True        # forward(..., residual=x) may add the branch into the float32 stream and return None

    def forward(self, h: torch.Tensor, step, memory: MixerMemory, residual: Optional[torch.Tensor] = None):
        rt = self.runtime
        n = h.shape[0]
        if hasattr(self.position, "prepare"):
            self.position.prepare(step.max_kv_len)
        table = getattr(self.position, "table", None)
        q = rt.empty(n, self.H * self.hd)
        kv_heads = self.KV if memory.writes_cache else 0
        if memory.writes_cache:
            proj, bias = self.qkv, self.bias
        else:
            if self.q_only is None:
                self.q_only = Linear(self.qkv.weight[: self.H * self.hd], rt)   # a view of the fused rows
            proj = self.q_only
            bias = self.bias[: self.H * self.hd] if self.bias is not None else None
        if self.fused and kernels.gemm_rows_takes(n, proj.weight.shape[0], self.hidden) and self.hd % 16 == 0:
            # prompts: tokens as the M operand, a thread of the epilogue holds a token's rotation pairs
            kernels.gemm_tcgen05_rows(h, proj.weight, q, kernels.bindings.EPI_QKV, bias=bias, positions=step.positions,
                                      tok_seq=step.tok_seq, rope=table, q_heads=self.H, kv_heads=kv_heads, head_dim=self.hd,
                                      kv=memory.kv if memory.writes_cache else None, n_sms=rt.n_sms)
        elif self.fused:
            # short epilogues in more blocks beat one long one; the few tiles' K range shared out over clusters of blocks
            splits = kernels.gemm_qkv_cluster_splits(n, proj.weight.shape[0], self.hidden) if n <= 64 else 1
            kernels.gemm_tcgen05(h, proj.weight, q, kernels.bindings.EPI_QKV, splits, bias=bias, positions=step.positions,
                                 tok_seq=step.tok_seq, rope=table, q_heads=self.H, kv_heads=kv_heads, head_dim=self.hd,
                                 kv=memory.kv if memory.writes_cache else None, n_sms=rt.n_sms,
                                 block_tokens=16 if n <= 64 else None)
        elif getattr(self.position, "fusable", False):
            kernels.qkv_post(proj(h, torch.float32), bias, step.positions, step.tok_seq, table, self.H, kv_heads,
                             self.hd, q, memory.kv if memory.writes_cache else None)
        else:
            # an encoding that is not a table of rotate-half angles: the part rotates the float32 queries and keys
            # itself, after the bias and before the cache write, as the fused forms do
            qkv = proj(h, torch.float32)
            if bias is not None:
                qkv += bias
            nq, nk = self.H * self.hd, kv_heads * self.hd
            qkv[:, :nq] = self.position.rotate(qkv[:, :nq].reshape(n, self.H, self.hd), step.positions,
                                               out_dtype=torch.float32).reshape(n, nq)
            if nk:
                qkv[:, nq:nq + nk] = self.position.rotate(qkv[:, nq:nq + nk].reshape(n, kv_heads, self.hd), step.positions,
                                                          out_dtype=torch.float32).reshape(n, nk)
            kernels.qkv_post(qkv, None, step.positions, step.tok_seq, None, self.H, kv_heads, self.hd, q,
                             memory.kv if memory.writes_cache else None)
        o = rt.empty(n, self.H * self.hd)
        self.attend(q, o, step, memory.kv)
        if residual is not None and self.o.can_add_into_stream(n):
            self.o.add_into(o, residual)
            return None
        return self.o(o, torch.float32, partial_ok=True)

    def attend(self, q: torch.Tensor, o: torch.Tensor, step, kv) -> None:
        """Attention of the step's tokens over the cache entry `kv` (which already holds their keys)."""
        rt = self.runtime
        window = self.window or 0
        keep = getattr(self, "keep_first", 0) if window else 0     # first keys that stay visible beside the window
        sinks = getattr(self, "sinks", None)          # float32 [heads] or None: a logit per head that joins every softmax
        chunk = getattr(self, "chunk", None) or 0     # a mask of chunks instead of a window
        softcap = getattr(self, "softcap", None) or 0.0
        if self.use_tensor_cores:
            row_tiles, n_splits = kernels.attention_mma_plan(step.max_q_len, step.n_seqs, step.max_kv_len, self.H,
                                                             self.KV, rt.n_sms)
            if (step.max_q_len >= 16 and n_splits == 1
                    and kernels.attention_tcgen05_takes(self.hd, kv.page_size, self.H, self.KV)):
                # prompts whose rows fill the GPU without sharing out the keys: the tcgen05 kernel
                kernels.attention_tcgen05(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                                          self.scale, window, sinks=sinks, keep_first=keep, chunk=chunk, softcap=softcap)
                return
            part_ml = part_o = None
            if step.max_q_len == 1 and row_tiles == 1:
                # single tokens: the blocks that share out a head's keys form a cluster and merge among themselves
                blocks = step.n_seqs * self.KV * max(1, (self.H // self.KV + 15) // 16)
                n_splits = kernels.attention_decode_splits(self.hd, blocks, step.max_kv_len)
            elif n_splits > 1:
                part_ml = rt.empty(q.shape[0] * self.H * n_splits * 2, dtype=torch.float32)
                part_o = rt.empty(q.shape[0] * self.H * n_splits * self.hd, dtype=torch.float32)
            kernels.attention_mma(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                                  self.scale, window, row_tiles, n_splits, part_ml, part_o, sinks=sinks, keep_first=keep,
                                  chunk=chunk, softcap=softcap)
            return
        n_splits = choose_splits(step, self.H, self.KV, rt.n_sms, tokens_per_block=max(1, 16 // min(16, self.H // self.KV)))
        part_ml = part_o = None
        if n_splits > 1:
            part_ml = rt.empty(q.shape[0] * self.H * n_splits * 2, dtype=torch.float32)
            part_o = rt.empty(q.shape[0] * self.H * n_splits * self.hd, dtype=torch.float32)
        kernels.attention_simt(q, o, step.cu_seqlens, step.start_pos, step.n_seqs, step.max_q_len, self.H, kv,
                               self.scale, window, n_splits, part_ml, part_o, sinks=sinks, keep_first=keep, chunk=chunk,
                               softcap=softcap)


def choose_splits(step, q_heads: int, kv_heads: int, n_sms: int, tokens_per_block: int, keys_per_split: int = 256,
                  max_splits: int = 32) -> int:
    """How many blocks share one row's key range: enough to fill the GPU when the step
    has few rows and long sequences (decoding), one when the rows alone fill it."""
    q_tiles = (step.max_q_len + tokens_per_block - 1) // tokens_per_block
    blocks = q_tiles * kv_heads * max(1, (q_heads // kv_heads + 15) // 16) * step.n_seqs
    if blocks >= 2 * n_sms:
        return 1
    by_fill = (2 * n_sms + blocks - 1) // blocks
    by_len = max(1, step.max_kv_len // keys_per_split)
    return max(1, min(by_fill, by_len, max_splits))


def fused_rows(weights, runtime) -> Linear:
    """One `Linear` over several matrices that read the same input, their rows stacked in order; rows of zeros bring
    the count to a multiple of 16, which the tensor-core products of prompts want."""
    w = torch.cat(list(weights), dim=0)
    pad = (-w.shape[0]) % 16
    if pad:
        w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype, device=w.device)], dim=0)
    return Linear(w, runtime)


@register_part("mixer", "sink_attention")
class SinkAttention(GQAttention):
    """Grouped-query attention whose softmax has a sink: per head a learned logit that joins the denominator once, with
    no key and no value, outside the scale.  Queries and keys are normalised per head (RMS over the head, a gain shared
    by the heads) before they are rotated; keys and queries have `head_dim` entries, values `v_head_dim`; the score's
    scale is a parameter.  No biases.

        q = rot(rms(W_q h)·g_q), k = rot(rms(W_k h)·g_k), v = W_v h
        p_ij = exp(scale·q_i·k_j) / (exp(sink) + sum_{j' <= i} exp(scale·q_i·k_j')),   out = W_o (p v)

    In the cache and in the kernels a head has D = max(head_dim, v_head_dim) entries, rounded up to 16; what lies
    beyond a head's own size is zero (and the output projection has zero columns there).  `value_scale` multiplies
    the values as they are stored, which multiplies the attention's output (an arrangement that adds this mixer to
    another with a factor passes the factor here, so that it acts in float32 before anything is rounded).

    Options.  `bias`: q, k and v have biases (the tensor's name with `.b`), added in the projection, before the norm.
    `softcap` c: score <- c · tanh(score / c) behind the scale.  `chunk` s: position i sees j <= i only if i // s == j // s,
    chunks counted from the sequence's first position (instead of a window; the cache gives a chunk's pages back once the
    sequence has left it).  `out_gate`: the heads' outputs are multiplied entry by entry by sigmoid(W_g h) before the output
    product; W_g (`g`) reads the mixer's input and rides in the input product.  `own_kv=False`: the mixer has no key and value
    tensors (projections, biases, key norm) and only ever reads another run's cache entry, with queries, mask and everything
    else of its own.  `keep_all_keys`: the cache keeps every position whatever this mixer's own mask (for an entry that
    another run reads under another mask).  The position part's `interleaved` says which entries form a rotation pair.

    `names`: the tensors' names below the part's prefix, by role (q, k, v, o, q_norm, k_norm, sink, g; a bias is its matrix's
    name with `.b`).  Offers `in_weights()` and `mix()` to an arrangement that computes several mixers' input projections in
    one product."""
    graph_safe = True
    accumulates = False

    NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm", sink="sink", g="g")

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int,
                 scale: float, norm_eps: float, position: PartSpec, qk_norm: bool = True, sink: bool = True,
                 window: Optional[int] = None, value_scale: float = 1.0, names: Optional[dict] = None, keep_first: int = 0,
                 bias: bool = False, softcap: Optional[float] = None, chunk: Optional[int] = None, out_gate: bool = False,
                 own_kv: bool = True, keep_all_keys: bool = False):
        """`window`, `keep_first`: position i sees j <= i with i - j < window or j < keep_first (no window: every j <= i)."""
        Part.__init__(self, name, hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim,
                      v_head_dim=v_head_dim, scale=scale, norm_eps=norm_eps, qk_norm=qk_norm, sink=sink, window=window,
                      value_scale=value_scale, keep_first=keep_first, bias=bias, softcap=softcap, chunk=chunk, out_gate=out_gate,
                      own_kv=own_kv, keep_all_keys=keep_all_keys)
        if num_heads % num_kv_heads:
            raise ValueError(f"attention: {num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden, self.H, self.KV = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.dim, self.vdim = int(head_dim), int(v_head_dim)
        self.hd = (max(self.dim, self.vdim) + 15) // 16 * 16          # a head's size in the cache and the kernels
        if self.hd > 256:
            raise ValueError(f"attention: head sizes up to 256 are supported, got {max(self.dim, self.vdim)}")
        if not scale > 0:
            raise ValueError(f"attention: the score's scale must be positive, got {scale}")
        self.scale, self.eps = float(scale), float(norm_eps)
        self.qk_norm, self.has_sink = bool(qk_norm), bool(sink)
        self.window = int(window) if window else None
        self.keep_first = max(0, int(keep_first)) if self.window else 0
        self.value_scale = float(value_scale)
        self.has_bias, self.out_gate, self.own_kv = bool(bias), bool(out_gate), bool(own_kv)
        self.keep_all_keys = bool(keep_all_keys)
        self.softcap = float(softcap) if softcap else None
        self.chunk = int(chunk) if chunk else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"attention: the soft cap must be positive, got {softcap}")
        if self.chunk is not None and (self.chunk < 1 or self.window):
            raise ValueError("attention: a mask of chunks needs a positive size and excludes a window")
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}
        self.position = build_part(position, name)
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        self.sinks: Optional[torch.Tensor] = None

    def tensors(self):
        t = self.t
        specs = [TensorSpec(t["q"], (self.H * self.dim, self.hidden)), TensorSpec(t["o"], (self.hidden, self.H * self.vdim))]
        if self.own_kv:
            specs += [TensorSpec(t["k"], (self.KV * self.dim, self.hidden)), TensorSpec(t["v"], (self.KV * self.vdim, self.hidden))]
        if self.has_bias:
            specs.append(TensorSpec(t["q"] + ".b", (self.H * self.dim,), role="bias"))
            if self.own_kv:
                specs += [TensorSpec(t["k"] + ".b", (self.KV * self.dim,), role="bias"),
                          TensorSpec(t["v"] + ".b", (self.KV * self.vdim,), role="bias")]
        if self.qk_norm:
            specs.append(TensorSpec(t["q_norm"], (self.dim,), role="gain", init="one_plus_normal"))
            if self.own_kv:
                specs.append(TensorSpec(t["k_norm"], (self.dim,), role="gain", init="one_plus_normal"))
        if self.has_sink:
            specs.append(TensorSpec(t["sink"], (self.H,), role="bias"))
        if self.out_gate:
            specs.append(TensorSpec(t["g"], (self.H * self.vdim, self.hidden)))
        return specs

    def cache_need(self) -> CacheNeed:
        if self.keep_all_keys:              # another run reads this entry under a mask of its own
            return CacheNeed("all", self.KV, self.hd)
        if self.chunk:
            return CacheNeed("chunk", self.KV, self.hd, self.chunk)
        return CacheNeed("window" if self.window else "all", self.KV, self.hd, self.window, self.keep_first)

    def bind(self, get, runtime):
        Part.bind(self, get, runtime)
        t = self.t
        f32 = lambda name: get(name).to(torch.float32).contiguous()
        # columns of the input product: q | k | v | g (without the parts the mixer does not have)
        self._in = [get(t["q"])] + ([get(t["k"]), get(t["v"])] if self.own_kv else []) + ([get(t["g"])] if self.out_gate else [])
        self.in_proj: Optional[Linear] = None
        self.q_gain = f32(t["q_norm"]) if self.qk_norm else None
        self.k_gain = f32(t["k_norm"]) if self.qk_norm and self.own_kv else None
        self.q_bias = f32(t["q"] + ".b") if self.has_bias else None
        self.k_bias = f32(t["k"] + ".b") if self.has_bias and self.own_kv else None
        self.v_bias = f32(t["v"] + ".b") if self.has_bias and self.own_kv else None
        self.sinks = f32(t["sink"]) if self.has_sink else None
        wo = get(t["o"])
        if self.hd != self.vdim:            # the kernels' heads are wider than the values: columns of zeros
            padded = torch.zeros(self.hidden, self.H, self.hd, dtype=wo.dtype, device=wo.device)
            padded[:, :, :self.vdim] = wo.view(self.hidden, self.H, self.vdim)
            wo = padded.view(self.hidden, self.H * self.hd)
        self.o = Linear(wo, runtime)
        self.use_tensor_cores = runtime.dtype == torch.bfloat16
        if self.use_tensor_cores:
            kernels.attention_library(self.hd)

    def in_weights(self):
        """The matrices that read the mixer's input, in the order of the columns `mix` expects."""
        return list(self._in)

    def in_width(self) -> int:
        return sum(w.shape[0] for w in self._in)

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in self._in) + self.o.nbytes()

    def mix(self, proj: torch.Tensor, col: int, step, memory: MixerMemory) -> torch.Tensor:
        """Attention from the float32 projection rows `proj`, whose columns from `col` on are [q | k | v | g]; returns the
        heads' outputs [n, heads·D] in the engine's type, the input of `self.o`."""
        rt = self.runtime
        n = proj.shape[0]
        if memory.writes_cache != self.own_kv:
            raise ValueError("attention: a mixer without keys and values of its own reads another run's cache entry, and only "
                             "such a mixer does")
        table = self.position.table_for(step.max_kv_len) if hasattr(self.position, "table_for") else None
        rot = getattr(self.position, "dims", 0) if table is not None else 0
        kv_heads = self.KV if memory.writes_cache else 0
        q = rt.empty(n, self.H * self.hd)
        q_col = col
        k_col = q_col + self.H * self.dim
        v_col = k_col + self.KV * self.dim
        g_col = v_col + self.KV * self.vdim if self.own_kv else k_col
        kernels.qk_norm_rope_cache(proj, q_col, k_col, v_col, self.q_gain, self.k_gain, self.eps if self.qk_norm else -1.0,
                                   step.positions, step.tok_seq, table, rot, self.H, kv_heads, self.dim, self.vdim,
                                   self.value_scale, q, memory.kv if memory.writes_cache else None, q_bias=self.q_bias,
                                   k_bias=self.k_bias, v_bias=self.v_bias, interleaved=self.interleaved)
        o = rt.empty(n, self.H * self.hd)
        self.attend(q, o, step, memory.kv)
        if self.out_gate:
            kernels.sigmoid_gate(o, proj, g_col, self.H, self.vdim)
        return o

    def forward(self, h: torch.Tensor, step, memory: MixerMemory, residual: Optional[torch.Tensor] = None):
        if self.in_proj is None:
            self.in_proj = fused_rows(self._in, self.runtime)
        o = self.mix(self.in_proj(h, torch.float32), 0, step, memory)
        return self.o(o, torch.float32, partial_ok=True)


@register_part("mixer", "latent_attention")
class LatentAttention(GQAttention):
    """Attention whose keys and values are expansions of a low-rank latent (the "multi-head latent attention" of
    DeepSeek-V2).  Per token, with H heads, `dim` unrotated and `rot_dim` rotated query/key entries per head, values of
    `v_head_dim`, a latent of `kv_rank`:

        q = W_q h, head by head [dim | rot_dim];      [c_raw | k_rot] = W_dkv h  (kv_rank + rot_dim rows)
        c = c_raw / rms(c_raw) · g  (eps inside the root),   k_rot and the rot_dim part of every q head are rotated
        k_h = [W_uk,h c | k_rot],  v_h = W_uv,h c,  score = scale · q_h · k_h,  causal softmax,  out = W_o [heads' sums]

    Only [c | k_rot] is cached: one row of D = ceil16(kv_rank + rot_dim) entries per token, one "key/value head" that all
    query heads read, the values being the row's first kv_rank entries (`CacheNeed.shared_kv`).  The two expansions
    move to the query side: q'_h = [W_uk,hᵀ q_h,plain | q_h,rot] meets the cached rows directly, and W_uv,h is applied
    to the head's weighted sum of latents, so a step never expands the keys and values of the tokens before it.  The
    attention kernels are the ones every other attention uses.

    Options.  `q_rank`: the queries go through a latent of their own, c_q = rms(W_dq h) · g_q (eps inside the root),
    q = W_uq c_q (tensors dq, dq_norm, uq instead of q).  `window`: position i sees the keys j with 0 <= i - j < window
    (no window: every j <= i); the cache then keeps a window of rows.  The position part's `interleaved` says which
    entries of the rotated part form a pair.

    Offers `in_weights()`, `in_width()`, `mix()` and `o` to an arrangement that computes other matrices on the same input
    in the mixer's input product.

    `names`: the tensors' names below the part's prefix, by role (q, dq, dq_norm, uq, dkv, dkv_norm, uk, uv, o)."""
    graph_safe = True
    accumulates = False

    NAMES = dict(q="q", dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o")

    def __init__(self, name: str, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int,
                 scale: float, norm_eps: float, position: PartSpec, names: Optional[dict] = None, q_rank: Optional[int] = None,
                 window: Optional[int] = None):
        Part.__init__(self, name, hidden_size=hidden_size, num_heads=num_heads, head_dim=head_dim, rot_dim=rot_dim,
                      v_head_dim=v_head_dim, kv_rank=kv_rank, scale=scale, norm_eps=norm_eps, q_rank=q_rank, window=window)
        self.hidden, self.H, self.KV = int(hidden_size), int(num_heads), 1
        self.dim, self.rot, self.vdim, self.rank = int(head_dim), int(rot_dim), int(v_head_dim), int(kv_rank)
        self.q_rank = int(q_rank) if q_rank else None
        if self.rot % 2 or self.rot < 0 or self.dim < 0 or self.dim + self.rot <= 0:
            raise ValueError(f"latent attention: a head has {head_dim} plain and {rot_dim} rotated entries; the rotated size must be even")
        self.hd = (self.rank + self.rot + 15) // 16 * 16              # a cached row, and a query row, in the kernels
        if self.hd > 512:
            raise ValueError(f"latent attention: kv_rank + rot_dim up to 512 is supported, got {self.rank + self.rot}")
        if not scale > 0:
            raise ValueError(f"latent attention: the score's scale must be positive, got {scale}")
        self.scale, self.eps = float(scale), float(norm_eps)
        self.window = int(window) if window else None
        self.t = {role: name + n for role, n in {**self.NAMES, **(names or {})}.items()}
        self.position = build_part(position, name)
        self.interleaved = bool(getattr(self.position, "interleaved", False))

    def tensors(self):
        t, H = self.t, self.H
        nq = H * (self.dim + self.rot)
        if self.q_rank:
            q = [TensorSpec(t["dq"], (self.q_rank, self.hidden)),
                 TensorSpec(t["dq_norm"], (self.q_rank,), role="gain", init="one_plus_normal"),
                 TensorSpec(t["uq"], (nq, self.q_rank))]
        else:
            q = [TensorSpec(t["q"], (nq, self.hidden))]
        return q + [TensorSpec(t["dkv"], (self.rank + self.rot, self.hidden)),
                    TensorSpec(t["dkv_norm"], (self.rank,), role="gain", init="one_plus_normal"),
                    TensorSpec(t["uk"], (H * self.dim, self.rank)), TensorSpec(t["uv"], (H * self.vdim, self.rank)),
                    TensorSpec(t["o"], (self.hidden, H * self.vdim))]

    def cache_need(self) -> CacheNeed:
        return CacheNeed("window" if self.window else "all", 1, self.hd, self.window, 0, True)

    def bind(self, get, runtime):
        Part.bind(self, get, runtime)
        t = self.t
        # columns of the input product: [q heads | latent | shared rotated key part], or with a query latent
        # [query latent | latent | shared rotated key part]
        self._in = [get(t["dq"]) if self.q_rank else get(t["q"]), get(t["dkv"])]
        self.in_proj: Optional[Linear] = None
        self.kv_col = self._in[0].shape[0]
        if self.q_rank:
            self.q_gain = get(t["dq_norm"]).to(torch.float32).contiguous()
            self.uq = Linear(get(t["uq"]), runtime)
        self.gain = get(t["dkv_norm"]).to(torch.float32).contiguous()
        self.w_uk, self.w_uv = get(t["uk"]).contiguous(), get(t["uv"]).contiguous()
        self.o = Linear(get(t["o"]), runtime)
        # rows of more than 256 entries run on the float32-arithmetic kernel in both engine types (the tensor-core
        # attention kernels are compiled for head sizes up to 256)
        self.use_tensor_cores = runtime.dtype == torch.bfloat16 and self.hd <= 256
        if self.use_tensor_cores:
            kernels.attention_library(self.hd)

    def in_weights(self):
        """The matrices that read the mixer's input, in the order of the columns `mix` expects."""
        return list(self._in)

    def in_width(self) -> int:
        return self.kv_col + self.rank + self.rot

    def weight_bytes(self) -> int:
        b = sum(w.numel() * w.element_size() for w in self._in) + self.o.nbytes()
        b += sum(w.numel() * w.element_size() for w in (self.w_uk, self.w_uv))
        return b + (self.uq.nbytes() if self.q_rank else 0)

    def flops_per_token(self) -> float:
        """Multiply-adds x 2 of the two per-head expansions (and of the queries' expansion from their latent)."""
        f = 2.0 * self.H * self.rank * (self.dim + self.vdim)
        return f + (2.0 * self.q_rank * self.H * (self.dim + self.rot) if self.q_rank else 0.0)

    def mix(self, proj: torch.Tensor, col: int, step, memory: MixerMemory) -> torch.Tensor:
        """Attention from the float32 projection rows `proj`, whose columns from `col` on are this mixer's input product;
        returns the heads' values [n, heads·vdim] in the engine's type, the input of `self.o`."""
        rt = self.runtime
        n, H, D = proj.shape[0], self.H, self.hd
        q_rows, q_col = None, col
        if self.q_rank:
            cq = rt.empty(n, self.q_rank)
            kernels.group_norm(proj[:, col:col + self.q_rank], 1, self.q_gain, self.eps, out=cq)
            q_rows, q_col = self.uq(cq, torch.float32), 0
        qsrc = proj if q_rows is None else q_rows
        table = self.position.table_for(step.max_kv_len) if self.rot and hasattr(self.position, "table_for") else None
        q = rt.empty(n, H * D)
        kernels.latent_prepare(proj, q_col, col + self.kv_col, self.gain, self.eps, step.positions, step.tok_seq, table, H,
                               self.dim, self.rot, self.rank, q, memory.kv if memory.writes_cache else None, q_rows=q_rows,
                               interleaved=self.interleaved)
        if self.dim:
            # the key expansion on the query's side: q'[t, h, :rank] = W_uk,hᵀ q_plain[t, h]
            kernels.head_project(qsrc, (qsrc.stride(0), self.dim + self.rot), self.w_uk, (self.dim * self.rank, self.rank, 1),
                                 q, (H * D, D), n, H, self.dim, self.rank, src_offset=q_col)
        else:
            q.view(n, H, D)[:, :, :self.rank].zero_()
        o = rt.empty(n, H * D)
        self.attend(q, o, step, memory.kv)
        # the value expansion behind the sum: val[t, h] = W_uv,h (sum_j p c_j)
        val = rt.empty(n, H * self.vdim)
        kernels.head_project(o, (H * D, D), self.w_uv, (self.vdim * self.rank, 1, self.rank), val, (H * self.vdim, self.vdim),
                             n, H, self.rank, self.vdim)
        return val

    def forward(self, h: torch.Tensor, step, memory: MixerMemory, residual: Optional[torch.Tensor] = None):
        if self.in_proj is None:
            self.in_proj = fused_rows(self._in, self.runtime)
        val = self.mix(self.in_proj(h, torch.float32), 0, step, memory)
        return self.o(val, torch.float32, partial_ok=True)


@register_part("mixer", "conv_attention")
class ConvKeyAttention(SinkAttention):
    """Grouped-query attention whose queries and keys pass a short causal convolution over time, and whose values are the
    convolved keys: there is no value matrix.

        q = conv_q(W_q h),  k = conv_k(W_k h)        (per channel, `conv` taps, no bias; zeros before the sequence's start)
        v = k, head by head, as it leaves the convolution
        q <- rot(rms(q) · g_q),  k <- rot(rms(k) · g_k)   (rms over the whole projection, all heads at once; gains of that size)
        out = W_o softmax(scale · q kᵀ, causal) v

    Keys and values have the same head size.  State per sequence: the last conv-1 projected rows [q | k], float32; the
    convolution's inputs and outputs are float32 in both engine modes.  No biases, no sink.  The position part's
    `interleaved` says which entries form a rotation pair.  `names`: the tensors' names below the part's prefix, by role
    (q, k, o, q_norm, k_norm, q_conv, k_conv)."""
    graph_safe = True
    accumulates = False

    NAMES = dict(q="q", k="k", o="o", q_norm="q.norm", k_norm="k.norm", q_conv="q.conv", k_conv="k.conv")

    def __init__(self, name: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 norm_eps: float, conv: int, position: PartSpec, names: Optional[dict] = None):
        SinkAttention.__init__(self, name, hidden_size=hidden_size, num_heads=num_heads, num_kv_heads=num_kv_heads,
                               head_dim=head_dim, v_head_dim=head_dim, scale=scale, norm_eps=norm_eps, position=position,
                               qk_norm=True, sink=False, names=names)
        if conv < 1:
            raise ValueError("attention: the convolution needs at least one tap")
        self.taps = int(conv)
        self.params["conv"] = self.taps
        self.n_q, self.n_k = self.H * self.dim, self.KV * self.dim

    def tensors(self):
        t = self.t
        return [TensorSpec(t["q"], (self.n_q, self.hidden)), TensorSpec(t["k"], (self.n_k, self.hidden)),
                TensorSpec(t["o"], (self.hidden, self.n_q)),
                TensorSpec(t["q_norm"], (self.n_q,), role="gain", init="one_plus_normal"),
                TensorSpec(t["k_norm"], (self.n_k,), role="gain", init="one_plus_normal"),
                TensorSpec(t["q_conv"], (self.n_q, self.taps)), TensorSpec(t["k_conv"], (self.n_k, self.taps))]

    def state_spec(self):
        from .base import StateSpec
        return StateSpec(((self.taps - 1) * (self.n_q + self.n_k),), torch.float32) if self.taps > 1 else None

    def bind(self, get, runtime):
        Part.bind(self, get, runtime)
        t = self.t
        f32 = lambda name: get(name).to(torch.float32).contiguous()
        self._in = [get(t["q"]), get(t["k"])]                     # columns of the input product: q | k
        self.in_proj: Optional[Linear] = None
        self.conv_w = torch.cat([f32(t["q_conv"]), f32(t["k_conv"])], dim=0).contiguous()
        self.q_gain, self.k_gain = f32(t["q_norm"]), f32(t["k_norm"])
        self.sinks = None
        wo = get(t["o"])
        if self.hd != self.dim:             # the kernels' heads are wider than the values: columns of zeros
            padded = torch.zeros(self.hidden, self.H, self.hd, dtype=wo.dtype, device=wo.device)
            padded[:, :, :self.dim] = wo.view(self.hidden, self.H, self.dim)
            wo = padded.view(self.hidden, self.H * self.hd)
        self.o = Linear(wo, runtime)
        self.use_tensor_cores = runtime.dtype == torch.bfloat16
        if self.use_tensor_cores:
            kernels.attention_library(self.hd)
        self._no_state: Optional[torch.Tensor] = None

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in self._in) + self.o.nbytes() + self.conv_w.numel() * 4

    def mix(self, proj: torch.Tensor, col: int, step, memory: MixerMemory) -> torch.Tensor:
        """Attention from the float32 projection rows `proj`, whose columns from `col` on are [q | k]; returns the heads'
        outputs [n, heads·D] in the engine's type, the input of `self.o`."""
        rt = self.runtime
        n = proj.shape[0]
        if not memory.writes_cache:
            raise ValueError("attention: this mixer keeps its own keys")
        qk = rt.empty(n, self.n_q + self.n_k, dtype=torch.float32)
        state = memory.state
        if state is None:                  # one tap: nothing is remembered
            if self._no_state is None:
                self._no_state = torch.zeros(1, 0, dtype=torch.float32, device=rt.device)
            state = self._no_state
        kernels.causal_conv(proj, col, self.conv_w, None, False, state, step, qk)
        table = self.position.table_for(step.max_kv_len) if hasattr(self.position, "table_for") else None
        rot = getattr(self.position, "dims", 0) if table is not None else 0
        q = rt.empty(n, self.H * self.hd)
        # the values are the key columns themselves, before norm and rotation
        kernels.qk_norm_rope_cache(qk, 0, self.n_q, self.n_q, self.q_gain, self.k_gain, self.eps, step.positions, step.tok_seq,
                                   table, rot, self.H, self.KV, self.dim, self.dim, 1.0, q, memory.kv, whole_row=True,
                                   interleaved=self.interleaved)
        o = rt.empty(n, self.H * self.hd)
        self.attend(q, o, step, memory.kv)
        return o
