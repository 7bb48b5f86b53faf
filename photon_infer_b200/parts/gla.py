"""Gated linear attention: a recurrent mixer with a matrix-valued state per head.

``q = W_q h * dim^(-1/2)``, ``k = W_k h`` (heads x dim), ``v = W_v h`` (heads x vdim) and a decay per key channel
``a = sigmoid(z)^(1/tau)`` with ``z = W_a2 (W_a1 h) + b`` (a low-rank projection, laid out heads x dim).  Per head

    S_t = diag(a_t) S_(t-1) + k_t v_t^T,        o_t = S_t^T q_t,

``o_t`` is RMS-normed over vdim with a weight that the heads share, the heads are concatenated, multiplied by
``silu(W_g h)`` and projected by ``W_o``.  The state starts at zero, is 32-bit, and lives in the request's state
slot between steps; decays, their logarithms and the recurrence itself are 32-bit.

One fused product gives ``[q | k | v | g | W_a1 h]``; one kernel forms the decay logits from the low-rank part,
runs the recurrence over the tokens of a step and applies the norm and the gate in its epilogue.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, StateSpec, StepContext, TensorSpec
from .linear import project
from .registry import register_mixer


class GatedLinearAttention(Mixer):
    kernel_modules = ("gla",)
    state_skips_negative_slots = True

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, tau: float, eps: float,
                 decay_rank: Optional[int] = None):
        self.hidden_size, self.heads, self.dim, self.vdim = hidden_size, heads, dim, vdim
        self.tau, self.eps = float(tau), float(eps)
        self.decay_rank = decay_rank            # None: the weight file decides
        self.w_in = self.w_a2 = self.b_a2 = self.norm = self.w_o = None

    def required_kernels(self, dtype):
        mods = list(self.kernel_modules)
        if dtype == torch.bfloat16:
            mods.extend(["gemm_skinny", "gemm_tc", "gemm_tc2"])
        return mods

    def tensor_specs(self) -> List[TensorSpec]:
        H, n, d, v = self.hidden_size, self.heads, self.dim, self.vdim
        rank = -1 if self.decay_rank is None else self.decay_rank
        return [TensorSpec("q", (n * d, H)), TensorSpec("k", (n * d, H)), TensorSpec("v", (n * v, H)),
                TensorSpec("g", (n * v, H)), TensorSpec("o", (H, n * v)),
                TensorSpec("norm", (v,), role="vector", init="norm"),
                TensorSpec("a1", (rank, H)), TensorSpec("a2", (n * d, rank)),
                TensorSpec("a2.b", (n * d,), role="vector", init="normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
            raise ValueError("the two halves of the decay projection do not fit each other")
        self.decay_rank = tensors["a1"].shape[0]
        self.w_in = torch.cat([tensors[n] for n in ("q", "k", "v", "g", "a1")], dim=0).contiguous()
        self.w_a2 = tensors["a2"].contiguous()
        self.b_a2 = tensors["a2.b"].contiguous()
        self.norm = tensors["norm"].contiguous()
        self.w_o = tensors["o"].contiguous()

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_a2, self.w_o))

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.heads, self.dim, self.vdim), torch.float32)

    def forward(self, h: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        T = h.shape[0]
        nd, nv = self.heads * self.dim, self.heads * self.vdim
        fused = project(h, self.w_in)                                    # [T, 2 nd + 2 nv + rank]
        q, k = fused[:, :nd], fused[:, nd:2 * nd]
        v, g = fused[:, 2 * nd:2 * nd + nv], fused[:, 2 * nd + nv:2 * nd + 2 * nv]
        low = fused[:, 2 * nd + 2 * nv:]
        out = torch.empty((T, nv), dtype=h.dtype, device=h.device)
        # long bfloat16 prompt portions run their chunks side by side; everything else (and the float32 run, whose sums
        # depend on nothing but the token's place in its request) goes token by token
        skip = 0
        lens = list(ctx.host_query_lens)
        if h.dtype == torch.bfloat16 and lens and max(lens) >= CHUNKED_MIN_TOKENS and ops.gla_chunked_supported(self.dim, self.vdim, self.decay_rank or 64):
            skip = CHUNKED_MIN_TOKENS
            slots = self._host_slots(ctx)
            t = 0
            for s, m in enumerate(lens):
                if m >= skip:
                    ops.gla_chunked(q, k, v, g, low, self.w_a2, self.b_a2, self.norm, self.eps, self.tau, self.dim ** -0.5,
                                    t, m, slots[s], cache.state, out, self.heads, self.dim, self.vdim, ctx.error_flag)
                t += m
        if skip == 0 or min(lens) < skip:
            ops.gla_recurrent(q, k, v, g, low, self.w_a2, self.b_a2, self.norm, self.eps, self.tau, self.dim ** -0.5,
                              ctx.cu_tokens, ctx.state_slots, cache.state, out, ctx.num_seqs, self.heads, self.dim, self.vdim,
                              ctx.error_flag, skip_from=skip)
        return project(out, self.w_o)


    @staticmethod
    def _host_slots(ctx: StepContext):
        """The requests' state slots on the host (the chunked path takes a request's slot as a launch argument)."""
        if ctx.host_state_slots:
            return list(ctx.host_state_slots)
        return ctx.state_slots.cpu().tolist()


#: A request that brings at least this many tokens to a bfloat16 step runs chunk-parallel.
CHUNKED_MIN_TOKENS = 128

register_mixer("gla", GatedLinearAttention)
register_mixer("gla_2", GatedLinearAttention)
