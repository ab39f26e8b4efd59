"""RMSNorm, fused with the residual add that precedes it.

Parity with InfiniLM: `csrc/models/minicpm4/minicpm4_for_causal_lm.cpp:43,45,52,54,86,99`
(`RMSNorm(hidden_size, rms_norm_eps)` used through `forward_inplace(hidden, residual)`):
y = x / sqrt(mean(x^2) + eps) * w, no bias.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Norm, register_part
from .spec import WeightSpec


class RMSNorm(Norm):
    """params: size, eps, weight_offset (default 0: y = x / rms * w; with 1 the stored weight is a deviation from one:
    y = x / rms * (1 + w), the sum made in float32 when the weights are loaded), name (local tensor name, default "weight")."""
    fusable_rms = True
    graph_safe = True

    def __init__(self, params, prefix, dtype):
        super().__init__(params, prefix, dtype)
        self.size, self.eps = int(params["size"]), float(params["eps"])
        self.offset = float(params.get("weight_offset", 0.0))
        self.name = str(params.get("name", "weight"))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        init = ("ones_normal", 0.01) if self.offset == 0.0 else ("normal", 0.05)
        return [WeightSpec(self.name, (self.size,), role="vector", init=init)]

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.name]
        if w.dtype not in (torch.float32, torch.bfloat16):
            w = w.to(torch.float32)
        if self.dtype == torch.float32 or self.offset != 0.0:
            w = w.to(torch.float32)
        if self.offset != 0.0:
            w = w + self.offset                   # in float32: 1 + w keeps every bit of a weight stored in bfloat16
        self.weight = w.contiguous()

    def add_norm(self, resid, branch, branch_scale, out, rows=None, vec=None):
        ops.add_rmsnorm(resid, branch, branch_scale, self.weight, self.eps, out, rows, vec)
        return out


    def norm_add(self, resid, branch, scale, copy=None):
        """resid (f32 [T,H]) += scale * norm(branch): the norm sits on the branch, not on the stream; `copy` receives the
        new stream in the compute dtype."""
        ops.norm_add(resid, branch, self.weight, self.eps, scale, copy)


register_part("norm", "rmsnorm", RMSNorm)
