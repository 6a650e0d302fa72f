"""RMSNorm with the residual add fused in.

out = x * rsqrt(mean(x^2) + eps) * weight, eps inside the root, the weight used
as it is (crates/airun-cuda/kernels/ops.cu:12-41); with ``delta`` the sum
x + delta is formed first and, unless only some rows are wanted, stored back as
the new residual (ops.cu:47-78).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from ..weights.loader import WeightSpec
from .base import Norm, register_part


class RMSNorm(Norm):
    device_driven = True

    def __init__(self, prefix: str, size: int, eps: float, dtype=None, device=None,
                 weight_name: str = "weight"):
        self.prefix, self.size, self.eps = prefix, int(size), float(eps)
        # weight_name "": the tensor is called by the prefix itself
        self.name = f"{prefix}.{weight_name}" if (prefix and weight_name) else (prefix or weight_name)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), storage="float32", init="norm")]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def forward(self, ctx, x, out, delta=None, rows=None) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows)

    def fusable(self):
        """(weight, eps) for products that fold this norm in (out = x * rsqrt(mean x^2 + eps) * weight)."""
        return self.weight, self.eps


register_part("norm", "rmsnorm", RMSNorm)


class DynamicTanh(Norm):
    """out = tanh(alpha * x) * weight + bias: a norm that takes no mean or variance of the row.  ``alpha`` is
    one learnt number, ``weight`` and ``bias`` are vectors; all three are kept in float32.  The tensors are
    ``<prefix>`` (or ``<prefix>.<weight_name>``), ``<prefix>.<bias_name>`` and ``<prefix>.<alpha_name>``.
    Like RMSNorm it carries out the residual add on the way (x += delta), and it can add one more row to
    every token (``add_vec``: an offset of the residual stream that belongs to a pass over the layers)."""
    device_driven = True
    takes_add_vec = True

    def __init__(self, prefix: str, size: int, dtype=None, device=None, weight_name: str = "",
                 bias_name: str = "b", alpha_name: str = "alpha"):
        self.prefix, self.size = prefix, int(size)
        self.name = f"{prefix}.{weight_name}" if weight_name else prefix
        self.bias_name, self.alpha_name = f"{prefix}.{bias_name}", f"{prefix}.{alpha_name}"
        self.weight = self.bias = self.alpha = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.size,), storage="float32", init="norm"),
                WeightSpec(self.bias_name, (self.size,), storage="float32", init="normal"),
                WeightSpec(self.alpha_name, (), storage="float32", init="norm")]

    def load_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight, self.bias = tensors[self.name], tensors[self.bias_name]
        self.alpha = tensors[self.alpha_name].reshape(1)

    def forward(self, ctx, x, out, delta=None, rows=None, add_vec=None) -> None:
        ops.dyt_norm(x, self.alpha, self.weight, self.bias, out, delta=delta, rows=rows, add_vec=add_vec)


register_part("norm", "dynamic_tanh", DynamicTanh)
