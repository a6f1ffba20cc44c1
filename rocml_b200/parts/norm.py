"""RMSNorm, fused with the residual addition that precedes it."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from ..config.specs import NormSpec
from ..weights.decl import TensorDecl
from .base import BuildEnv, DeferredNorm, Norm, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w, statistics in 32-bit
    (rocml-kernels/kernels/rmsnorm.hip:18-41); the weight multiplies directly.  With the spec's
    ``weight_offset`` the factor is w + offset: the sum is formed once, at load time, in 32-bit
    (a bfloat16 weight near zero plus one would lose its low bits in bfloat16), and the kernels
    read a 32-bit weight."""

    graph_safe = True

    def __init__(self, spec: NormSpec, size: int, env: BuildEnv):
        self.eps = float(spec.eps)
        self.offset = float(getattr(spec, "weight_offset", 0.0))
        self.size = size
        self.env = env
        self.weight: Optional[torch.Tensor] = None

    def declare(self, prefix: str) -> List[TensorDecl]:
        return [TensorDecl(f"{prefix}.weight", (self.size,), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], prefix: str) -> None:
        self.weight = tensors[f"{prefix}.weight"]
        if self.offset:
            self.weight = (self.weight.float() + self.offset).contiguous()

    def weight_bytes(self) -> int:
        if self.weight is None:
            return self.size * (4 if self.env.mode == "float32" else 2)
        return self.weight.numel() * self.weight.element_size()

    def workspace_bytes(self, n_tokens: int) -> int:
        return n_tokens * self.size * (4 if self.env.mode == "float32" else 2)

    deferrable = True     # a product's epilogue can prepare this norm's input (see parts.base.DeferredNorm)

    def forward(self, resid, delta, n_rows: Optional[int] = None, rows=None, write_back=True):
        if isinstance(delta, DeferredNorm):
            # the part before has added its result into the residual already
            if delta.norm is self and rows is None:
                return delta            # and prepared this norm's rows: nothing to launch
            delta = None
        n = (rows.numel() if rows is not None else resid.shape[0]) if n_rows is None else n_rows
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=resid.device)
        if delta is None:
            write_back = False          # nothing is added: the residual stays as it is
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows=rows, n_rows=n, write_back=write_back)
        return out

    def forward_with(self, other: "RMSNorm", resid, delta, n_rows: Optional[int] = None):
        """This norm and ``other`` of the same rows in one kernel (they share the rows' statistics when their eps
        agree, and differ by their weights): returns (rows of this norm, rows of the other)."""
        if isinstance(delta, DeferredNorm):
            delta = None
        if other.eps != self.eps or other.size != self.size or other.weight.dtype != self.weight.dtype:
            first = self.forward(resid, delta, n_rows)
            return first, other.forward(resid, None, n_rows)
        n = resid.shape[0] if n_rows is None else n_rows
        out = torch.empty((n, self.size), dtype=self.env.act_dtype, device=resid.device)
        out2 = torch.empty_like(out)
        kernels.add_rmsnorm(resid, delta, self.weight, self.eps, out, n_rows=n, write_back=delta is not None,
                            weight2=other.weight, out2=out2)
        return out, out2
