"""The block whose norms sit on the sublayers' outputs: x += norm_a(mixer(x)); x += norm_b(feed_forward(x)).

The sublayers read the stream itself, so what a product takes as activations is the stream in the activation type: the
norm that adds a sublayer's output writes it along (one kernel), and a block that finds the activations not to be the
stream (the first of a model) casts once.  A layer may have no feed-forward.
"""
from __future__ import annotations

from typing import Dict

from ..weights import TensorDecl
from .base import part_class, register
from .program import record


@register("block", "postnorm")
class PostNormBlock:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        out = {}
        for sub, prefix, family in _children(spec):
            for name, decl in part_class(family, sub).tensor_decls(sub).items():
                out[prefix + name] = decl
        return out

    @staticmethod
    def cache_need(spec):
        return part_class("mixer", spec.mixer).cache_need(spec.mixer)

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        ask = getattr(part_class("mixer", spec.mixer), "state_need", None)
        return ask(spec.mixer, writes_cache) if ask is not None else None

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec = spec
        build = lambda family, sub, p: part_class(family, sub)(sub, weights, prefix + p, runtime)
        self.mixer = build("mixer", spec.mixer, spec.mixer_prefix)
        self.mixer_norm = build("norm", spec.mixer_norm, spec.mixer_norm_prefix)
        self.feed_forward = self.ffn_norm = None
        if spec.feed_forward is not None:
            self.feed_forward = build("feed_forward", spec.feed_forward, spec.ffn_prefix)
            self.ffn_norm = build("norm", spec.ffn_norm, spec.ffn_norm_prefix)
        for part in (self.mixer, self.feed_forward):
            if part is not None and not hasattr(part, "plan_delta"):
                raise TypeError(f"{type(part).__name__} cannot leave its output for a norm to add (no plan_delta)")
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not hasattr(norm, "plan_add"):
                raise TypeError(f"{type(norm).__name__} cannot norm a sublayer's output into the stream (no plan_add)")

    def weight_bytes(self) -> int:
        parts = (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward)
        return sum(p.weight_bytes() for p in parts if p is not None and hasattr(p, "weight_bytes"))

    def plan(self, program, view, writes_cache: bool = True, state_view=None) -> None:
        hidden = program.hidden_size
        if not program.h_holds_stream:
            program.emit_records([record("cast", "x", "h", n=hidden)])
        self.mixer.plan_delta(program, view, writes_cache, state_view=state_view)
        self.mixer_norm.plan_add(program)
        if self.feed_forward is not None:
            self.feed_forward.plan_delta(program)
            self.ffn_norm.plan_add(program)
        program.h_holds_stream = True


def _children(spec):
    out = [(spec.mixer, spec.mixer_prefix, "mixer"), (spec.mixer_norm, spec.mixer_norm_prefix, "norm")]
    if spec.feed_forward is not None:
        out += [(spec.feed_forward, spec.ffn_prefix, "feed_forward"), (spec.ffn_norm, spec.ffn_norm_prefix, "norm")]
    return out
