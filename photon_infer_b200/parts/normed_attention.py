"""Grouped-query attention with normed queries and keys over the paged cache.

Per head, queries and keys are divided by their root mean square (``x / sqrt(mean(x^2) + eps)``), with or without
a weight ``[head_dim]`` that all heads share; then, optionally, the first ``rot_dims`` numbers of every head are
rotated by the token's position (number ``j`` paired with ``j + rot_dims / 2``, angle ``p * rot_base^(-2j / rot_dims)``),
the rest pass unchanged.  ``score = (q . k) * scale``, optionally bounded by ``softcap * tanh(score / softcap)``.  A
token at position ``i`` sees key ``j <= i`` when ``i - j < window`` or ``j < keep_first`` (no window: every earlier
key).  The softmax may have a sink: one more key with score 0 and no value, ``p_j = exp(s_j) / (1 + sum_i exp(s_i))``.
The heads' outputs may be multiplied by ``sigmoid(W_g h)`` (``h`` the mixer's input) before the output projection.
A value may have another width than a key.

Kernels of a step: ONE product for q, k, v (and the gate); one pass that norms and rotates in 32-bit (angles in
64-bit) and writes queries, keys and values (``qk_norm.cu``); attention, with the gate in its epilogue; the output product.  Prompt portions, decoded tokens and mixed batches take the same path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .attention import attend_tensor_cores
from .base import LayerCache, Mixer, PagedCacheSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer

DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "q_norm": "q.norm", "k_norm": "k.norm"}


class NormedAttention(Mixer):
    kernel_modules = ("qk_norm", "attention", "elementwise")

    def __init__(self, hidden_size: int, n_q_heads: int, n_kv_heads: int, head_dim: int, eps: float,
                 value_dim: Optional[int] = None, scale: Optional[float] = None, norm_weight: bool = False,
                 rot_dims: int = 0, rot_base: float = 10000.0, softcap: Optional[float] = None,
                 window: Optional[int] = None, keep_first: int = 0, sink: bool = False, output_gate: bool = False,
                 names: Optional[Dict[str, str]] = None):
        if n_kv_heads <= 0 or n_q_heads % n_kv_heads:
            raise ValueError("the number of query heads must be a multiple of the number of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= head_dim:
            raise ValueError("rot_dims must be even and at most head_dim")
        self.hidden_size, self.n_q, self.n_kv, self.head_dim = hidden_size, n_q_heads, n_kv_heads, head_dim
        self.value_dim = int(value_dim) if value_dim else head_dim
        self.eps = float(eps)
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.norm_weight = bool(norm_weight)
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.softcap = float(softcap) if softcap else None
        self.window = int(window) if window else None
        self.keep_first = int(keep_first or 0) if self.window else 0
        self.sink, self.output_gate = bool(sink), bool(output_gate)
        self.names = dict(DEFAULT_NAMES, **(names or {}))
        self.w_in: Optional[torch.Tensor] = None        # [W_q; W_k; W_v; (W_g)]
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm = self.k_norm = None
        self.inv_freq: Optional[torch.Tensor] = None
        self._max_groups: Optional[int] = None          # groups of warps per block of the split-key kernel, asked once

    # -- sizes of the sections of the fused row
    @property
    def _sections(self):
        q, k, v = self.n_q * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.value_dim
        return q, k, v, (self.n_q * self.value_dim if self.output_gate else 0)

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_tc", "gemm_tc2"])
            if self._flash_ok(dtype):
                mods.append(("attention_flash", {"HEAD_DIM": self.head_dim}))
            if self._tc_ok(dtype):
                mods.append(("attention_tc", {"HEAD_DIM": self.head_dim}))
            if self._flash_ok(dtype) and not (self.keep_first or self.sink or self.softcap) and self.head_dim in (64, 128) \
                    and self.n_q // self.n_kv <= 16:
                mods.append(("attention_decode", {"HEAD_DIM": self.head_dim}))     # long contexts without any of the rules
        return mods

    def _flash_ok(self, dtype) -> bool:
        return self.value_dim == self.head_dim and ops.flash_attention_supported(dtype, self.head_dim)

    def _tc_ok(self, dtype) -> bool:
        return (dtype == torch.bfloat16 and self.value_dim == self.head_dim and self.head_dim in (64, 128)
                and ops.USE_ATTENTION_TC and self.n_q // self.n_kv <= 128)

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.hidden_size
        q, k, v, g = self._sections
        specs = [TensorSpec(n["q"], (q, H)), TensorSpec(n["k"], (k, H)), TensorSpec(n["v"], (v, H)),
                 TensorSpec(n["o"], (H, self.n_q * self.value_dim))]
        if self.output_gate:
            specs.append(TensorSpec(n["g"], (g, H)))
        if self.norm_weight:
            specs += [TensorSpec(n["q_norm"], (self.head_dim,), role="vector", init="norm"),
                      TensorSpec(n["k_norm"], (self.head_dim,), role="vector", init="norm")]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        parts = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]] + ([tensors[n["g"]]] if self.output_gate else [])
        self.w_in = torch.cat(parts, dim=0).contiguous()
        self.w_o = tensors[n["o"]].contiguous()
        if self.norm_weight:
            self.q_norm, self.k_norm = tensors[n["q_norm"]].contiguous(), tensors[n["k_norm"]].contiguous()
        if self.rot_dims:
            j = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            self.inv_freq = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * j / self.rot_dims).to(self.w_in.device)

    def weight_bytes(self) -> int:
        return (self.w_in.numel() + self.w_o.numel()) * self.w_in.element_size()

    def cache_spec(self) -> Optional[PagedCacheSpec]:
        return PagedCacheSpec(self.n_kv, self.head_dim, self.window, value_dim=self.value_dim, keep_first=self.keep_first)

    # -- one step
    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        nq, nk, nv, ng = self._sections
        rows = project(h, self.w_in)
        q = torch.empty((T, nq), dtype=h.dtype, device=h.device)
        group = ctx.groups[cache.group]
        store = not cache.shared and cache.k is not None
        ops.qk_norm_rope_write(rows[:, :nq], rows[:, nq:nq + nk], rows[:, nq + nk:nq + nk + nv], q, self.q_norm, self.k_norm,
                               self.eps, ctx.positions, self.inv_freq, self.rot_dims, group.slot_mapping if store else None,
                               cache.k if store else None, cache.v if store else None, self.n_q, self.n_kv, self.head_dim,
                               self.value_dim, ctx.error_flag)
        attn = torch.empty((T, self.n_q * self.value_dim), dtype=h.dtype, device=h.device)
        gate = rows[:, nq + nk + nv:] if self.output_gate else None
        # the gate rides in the epilogue of the attention kernel; a gate whose rows are not 16-byte aligned gets a pass of its own
        fused = gate is not None and (not self._flash_ok(q.dtype) or ops.gate_fusable(gate))
        self.attend(q, attn, ctx, cache, gate if fused else None)
        if gate is not None and not fused:
            ops.gate_mul(attn, gate)
        return project(attn, self.w_o)

    def attend(self, q: torch.Tensor, out: torch.Tensor, ctx: StepContext, cache: LayerCache,
               gate: Optional[torch.Tensor] = None) -> None:
        """bfloat16 with heads the tensor-core kernels are compiled for (keys and values of one width): those
        kernels, tcgen05 for prompt portions and the split-key kernel for decoded tokens.  float32 and other sizes:
        the general kernel, whose sums depend on a token's position alone; its bfloat16 decode steps share a
        token's keys out over blocks."""
        if self._flash_ok(q.dtype):
            attend_tensor_cores(self, q, out, ctx, cache, keep_first=self.keep_first, sink=self.sink, softcap=self.softcap,
                                gate=gate)
            return
        group = ctx.groups[cache.group]
        splits = 1
        if q.dtype == torch.bfloat16 and ctx.max_query_len == 1:
            keys = ctx.max_context_len if self.window is None else min(self.window + self.keep_first + 1, ctx.max_context_len)
            blocks = max(1, ctx.num_tokens * self.n_kv)
            splits = max(1, min(keys // 128, (2 * ops.sm_count(q.device)) // blocks, 64))
        ops.paged_attention(q, out, cache.k, cache.v, group.block_table, ctx.token_seq, ctx.positions, self.n_q, self.n_kv,
                            self.head_dim, self.window, self.scale, ctx.error_flag, value_dim=self.value_dim, splits=splits,
                            keep_first=self.keep_first, sink=self.sink, softcap=self.softcap, gate=gate)


register_mixer("normed_attention", NormedAttention)
