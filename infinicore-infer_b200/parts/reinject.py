"""A step between two layers that feeds the embedding's output in again: x <- W [x | x0] + b.

x0 is what the embedding left (the model keeps a copy when a run-order entry asks for this step); b is one row of a
table, chosen by the specification (the number of the pass that the step opens).  One record: the two streams side by
side as a product's operand, the product into the stream, the row added.
"""
from __future__ import annotations

from typing import Dict

from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import record


@register("stream", "reinject")
class Reinject:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d = spec.hidden_size
        decls = {spec.weight_name: TensorDecl((d, 2 * d))}
        if spec.step_name is not None:
            decls[spec.step_name] = TensorDecl((spec.steps, d), VECTOR, init="zeros")
        return decls

    def __init__(self, spec, weights, prefix: str, runtime, shared=None):
        self.spec = spec
        shared = shared if shared is not None else {}
        load = lambda name, role: shared[name] if name in shared else shared.setdefault(name, weights.get(prefix + name, role))
        self.weight = load(spec.weight_name, MATRIX)
        self.steps = load(spec.step_name, VECTOR) if spec.step_name is not None else None
        if self.steps is not None and not 0 <= spec.step_index < self.steps.shape[0]:
            raise ValueError(f"step {spec.step_index} of a table of {self.steps.shape[0]}")

    needs_embedding_output = True

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def plan(self, program) -> None:
        d = self.spec.hidden_size
        row = self.steps[self.spec.step_index] if self.steps is not None else None
        program.emit_records([record("reinject", "x0", "x", n=d, k=2 * d, w=self.weight, vec=row)], keep=(self.weight, self.steps))
