"""Steps between layers that work on the residual stream itself.

``loop_add``: ``x <- x + x0 (from the second pass on) + s[t]``, see ``LoopAdd``.

``loop_input``: the entrance of a block of layers that is run several times with the same weights.  Before
every pass ``x <- W [x ; x0] + s[t]``, with ``x0`` the embedding output, ``W [H, 2H]`` (the columns of ``x``
first) and ``s [times, H]`` one vector per pass, ``t`` the number of the pass.  The sum that was pending on the
stream is applied first, in 32-bit; the product takes its operands in the run dtype and leaves a 32-bit
result, to which the pass vector is added.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import StepContext, StreamPart, TensorSpec, delta_pair
from .registry import register_stream_part


class LoopInput(StreamPart):
    kernel_modules = ("elementwise",)

    def __init__(self, hidden_size: int, times: int, weight_name: str = "in", step_name: str = "step"):
        self.hidden_size = hidden_size
        self.times = times
        self.weight_name, self.step_name = weight_name, step_name
        self.weight: Optional[torch.Tensor] = None
        self.steps: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        H = self.hidden_size
        return [TensorSpec(self.weight_name, (H, 2 * H)), TensorSpec(self.step_name, (self.times, H), role="vector", init="normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.weight_name].contiguous()
        self.steps = tensors[self.step_name].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, residual, delta, first, index: int, ctx: StepContext) -> torch.Tensor:
        if not 0 <= index < self.times:
            raise IndexError(f"pass {index} of a block that runs {self.times} times")
        T, H = residual.shape
        d1, d2 = delta_pair(delta)
        both = torch.empty((T, 2 * H), dtype=self.weight.dtype, device=residual.device)
        ops.stream_concat(residual, d1, d2, first, both)
        out = ops.linear(both, self.weight, out_dtype=torch.float32)
        ops.scale_bias_rows(out, 1.0, self.steps[index])
        return out


class LoopAdd(StreamPart):
    """The entrance of a block of layers that is run several times, without a projection: before every pass but the
    first the embedding output is added to the stream, and before every pass (the first too) the pass's vector
    ``s[t]`` (``s [times, H]``).  Everything is summed in 32-bit, after what was pending on the stream."""
    kernel_modules = ("elementwise",)

    def __init__(self, hidden_size: int, times: int, step_name: str = "step"):
        self.hidden_size = hidden_size
        self.times = times
        self.step_name = step_name
        self.steps: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.step_name, (self.times, self.hidden_size), role="vector", init="normal")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.steps = tensors[self.step_name].contiguous()

    def weight_bytes(self) -> int:
        return self.hidden_size * self.steps.element_size()

    def forward(self, residual, delta, first, index: int, ctx: StepContext) -> torch.Tensor:
        if not 0 <= index < self.times:
            raise IndexError(f"pass {index} of a block that runs {self.times} times")
        d1, d2 = delta_pair(delta)
        ops.stream_add(residual, d1, d2, first if index > 0 else None, self.steps[index])
        return residual


register_stream_part("loop_input", LoopInput)
register_stream_part("loop_add", LoopAdd)
