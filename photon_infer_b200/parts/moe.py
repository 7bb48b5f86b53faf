"""Mixture of experts: ``experts`` small gated feed-forward layers, of which every token uses ``top``, and an
optional shared expert of the same form that every token uses.

Router logits ``z = W_r h + b`` in 32-bit; the ``top`` experts with the largest logits are chosen and weighted
with the softmax over the chosen logits only; the output is the weighted sum of their outputs plus the shared
expert's.  An expert is ``W_down (act(W_gate h) * (W_up h))`` without biases.

On the device the (token, choice) pairs are sorted by expert without a round trip to the host; two grouped
products walk the sorted rows (the first gathers its rows of ``h`` and applies the gated activation in its
epilogue, the second leaves 32-bit rows), and one kernel forms every token's weighted sum in the order of its
choices and adds the shared expert's output.  That is the float32 path and the one for a middling number of
rows.  A bfloat16 decode step (a handful of pairs) skips the sort and runs one matrix-vector product per pair;
a bfloat16 step with many rows hands the sorted rows to the library's grouped product.  The experts' matrices are stacked into ``[E, 2 ff, H]`` and
``[E, H, ff]`` when loaded.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, StepContext, TensorSpec
from .linear import project
from .registry import register_feed_forward


class MoEFeedForward(FeedForward):
    kernel_modules = ("moe", "elementwise")

    def required_kernels(self, dtype):
        return list(self.kernel_modules) + (["gemm_skinny", "gemm_tc", "gemm_tc2"] if dtype == torch.bfloat16 else [])

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, shared_size: Optional[int] = None,
                 activation: str = "silu", shared_activation: Optional[str] = None):
        if not 1 <= top <= experts:
            raise ValueError("a token uses between one and all of the experts")
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}")
        self.hidden_size, self.experts, self.top = hidden_size, experts, top
        self.expert_size, self.shared_size = expert_size, shared_size
        self.activation = activation
        self.shared_activation = shared_activation or activation
        self.w_router = self.b_router = self.w_gate_up = self.w_down = None
        self.shared_gate_up = self.shared_down = None

    def tensor_specs(self) -> List[TensorSpec]:
        H, F = self.hidden_size, self.expert_size
        specs = [TensorSpec("router", (self.experts, H)), TensorSpec("router.b", (self.experts,), role="vector", init="normal")]
        for e in range(self.experts):
            specs += [TensorSpec(f"e{e}.gate", (F, H)), TensorSpec(f"e{e}.up", (F, H)), TensorSpec(f"e{e}.down", (H, F))]
        if self.shared_size:
            S = self.shared_size
            specs += [TensorSpec("shared.gate", (S, H)), TensorSpec("shared.up", (S, H)), TensorSpec("shared.down", (H, S))]
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = self.experts
        self.w_router = tensors["router"].contiguous()
        self.b_router = tensors["router.b"].contiguous()
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0) for e in range(E)]).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(E)]).contiguous()
        if self.shared_size:
            self.shared_gate_up = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0).contiguous()
            self.shared_down = tensors["shared.down"].contiguous()

    def weight_bytes(self) -> int:
        """What a step reads at most: the router, the shared expert and every expert once."""
        ws = [self.w_router, self.w_gate_up, self.w_down] + ([self.shared_gate_up, self.shared_down] if self.shared_size else [])
        return sum(w.numel() * w.element_size() for w in ws)

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, H = h.shape
        n = T * self.top
        ids, weights, counts = ops.moe_route(h, self.w_router, self.b_router, self.top)
        shared = None
        if self.shared_size:
            shared = project(ops.linear_swiglu(h, self.shared_gate_up, self.shared_activation), self.shared_down)
        out = torch.empty((T, H), dtype=h.dtype, device=h.device)
        if n <= GEMV_MAX_PAIRS and ops.moe_gemv_supported(h, self.w_gate_up) and self.expert_size % 8 == 0:
            # a decode step: nothing is sorted, every pair streams its expert's matrices once
            act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
            ops.moe_gemv(h, self.top, ids, self.w_gate_up, act, glu=True, activation=self.activation)
            y = torch.empty((n, H), dtype=torch.float32, device=h.device)
            ops.moe_gemv(act, 1, ids, self.w_down, y)
            ops.moe_combine(y, None, weights, shared, out)
            return out
        offsets, srt, place, tiles, num_tiles, max_tiles = ops.moe_align(ids, counts)
        if h.dtype == torch.bfloat16 and n >= GROUPED_LIBRARY_PAIRS and H % 8 == 0 and self.expert_size % 8 == 0:
            # many bfloat16 rows: the library's grouped product over the rows gathered in sorted order
            xs = ops.moe_gather(h, srt, self.top)
            gate_up = torch._grouped_mm(xs, self.w_gate_up.transpose(1, 2), offs=offsets[1:])
            act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
            ops.swiglu(gate_up, act, self.activation)
            y = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=offsets[1:])
            ops.moe_combine(y, place, weights, shared, out)
            return out
        act = torch.empty((n, self.expert_size), dtype=h.dtype, device=h.device)
        ops.moe_gemm(h, srt, self.top, self.w_gate_up, act, tiles, num_tiles, max_tiles, glu=True, activation=self.activation)
        y = torch.empty((n, H), dtype=torch.float32, device=h.device)
        ops.moe_gemm(act, None, 1, self.w_down, y, tiles, num_tiles, max_tiles)
        ops.moe_combine(y, place, weights, shared, out)
        return out


#: Up to this many (token, choice) pairs a bfloat16 step runs one matrix-vector product per pair.
GEMV_MAX_PAIRS = 64
#: From this many pairs on a bfloat16 step hands the sorted rows to the library's grouped product.
GROUPED_LIBRARY_PAIRS = 256

register_feed_forward("moe", MoEFeedForward)
