"""Layer norm with weight and bias: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, in float32.

Two uses, one kernel (csrc/mixers.cu): ``plan_add`` norms a sublayer's output (float32, in the slot of products that
wait for the stream) and adds it to the stream, writing the new stream also as the next product's activations;
``plan`` / ``forward`` norm rows of the stream into activations (the model's last norm, over the wanted rows).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..weights import VECTOR, TensorDecl
from .base import ResidualStream, register
from .program import record


@register("norm", "layernorm")
class LayerNorm:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        return {spec.weight_name: TensorDecl((spec.size,), VECTOR, init="ones"),
                spec.bias_name: TensorDecl((spec.size,), VECTOR, init="zeros")}

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        self.weight = weights.get(prefix + spec.weight_name, VECTOR)
        self.bias = weights.get(prefix + spec.bias_name, VECTOR)

    def weight_bytes(self) -> int:
        return 4 * (self.weight.numel() + self.bias.numel())

    def plan(self, program, out_scale: float = 1.0, wanted_rows: bool = False) -> None:
        """One record: rows of the stream (all, or the wanted ones) normed into activations."""
        if out_scale != 1.0:
            raise ValueError("a layer norm has a bias; a factor on its output is not built")
        program.emit_records([record("layernorm", "x", "hw" if wanted_rows else "h", n=self.spec.size, eps=self.spec.eps,
                                     vec=self.weight, bias=self.bias, wanted_rows=wanted_rows)], keep=(self.weight, self.bias))

    def plan_add(self, program, also_activations: bool = True) -> None:
        """One record: stream += LN(the product that waits in the delta slot); the new stream also as activations."""
        program.emit_records([record("layernorm", "delta", "h" if also_activations else None, n=self.spec.size, eps=self.spec.eps,
                                     vec=self.weight, bias=self.bias)], keep=(self.weight, self.bias))

    def forward(self, residual: ResidualStream, ctx, out_scale: float = 1.0, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Norm every row, or only ``rows`` (int32 indices), of the stream into activations."""
        from .. import kernels
        if out_scale != 1.0:
            raise ValueError("a layer norm has a bias; a factor on its output is not built")
        x = residual.value()
        n = rows.numel() if rows is not None else x.shape[0]
        out = self.runtime.empty(n, self.spec.size)
        kernels.layernorm(x, self.weight, self.bias, self.spec.eps, out=out, rows=rows)
        return out
