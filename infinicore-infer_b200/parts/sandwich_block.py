"""The block with a norm before and after each sublayer: x += norm_b(mixer(norm_a(x))); x += norm_d(ff(norm_c(x))).

The norm after a sublayer adds into the stream (``plan_add``); the norm before the next sublayer, of this layer or of
the next, joins that kernel where it follows directly (``plan_after_add``), so a sublayer boundary is one kernel.  A layer
may have no feed-forward.
"""
from __future__ import annotations

from typing import Dict

from ..weights import TensorDecl
from .base import part_class, register


@register("block", "sandwich")
class SandwichBlock:
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
        self.mixer_norm = build("norm", spec.mixer_norm, spec.mixer_norm_prefix)
        self.mixer = build("mixer", spec.mixer, spec.mixer_prefix)
        self.mixer_post_norm = build("norm", spec.mixer_post_norm, spec.mixer_post_norm_prefix)
        self.feed_forward = self.ffn_norm = self.ffn_post_norm = None
        if spec.feed_forward is not None:
            self.ffn_norm = build("norm", spec.ffn_norm, spec.ffn_norm_prefix)
            self.feed_forward = build("feed_forward", spec.feed_forward, spec.ffn_prefix)
            self.ffn_post_norm = build("norm", spec.ffn_post_norm, spec.ffn_post_norm_prefix)
        for part in (self.mixer, self.feed_forward):
            if part is not None and not hasattr(part, "plan_delta"):
                raise TypeError(f"{type(part).__name__} cannot leave its output for a norm to add (no plan_delta)")
        for norm in (self.mixer_post_norm, self.ffn_post_norm):
            if norm is not None and not hasattr(norm, "plan_add"):
                raise TypeError(f"{type(norm).__name__} cannot norm a sublayer's output into the stream (no plan_add)")

    def weight_bytes(self) -> int:
        parts = (self.mixer_norm, self.mixer, self.mixer_post_norm, self.ffn_norm, self.feed_forward, self.ffn_post_norm)
        return sum(p.weight_bytes() for p in parts if p is not None and hasattr(p, "weight_bytes"))

    def plan(self, program, view, writes_cache: bool = True, state_view=None) -> None:
        _plan_norm(self.mixer_norm, program)
        self.mixer.plan_delta(program, view, writes_cache, state_view=state_view)
        self.mixer_post_norm.plan_add(program)
        if self.feed_forward is not None:
            _plan_norm(self.ffn_norm, program)
            self.feed_forward.plan_delta(program)
            self.ffn_post_norm.plan_add(program)


def _plan_norm(norm, program) -> None:
    if hasattr(norm, "plan_after_add"):
        norm.plan_after_add(program)
    else:
        norm.plan(program)


def _children(spec):
    out = [(spec.mixer_norm, spec.mixer_norm_prefix, "norm"), (spec.mixer, spec.mixer_prefix, "mixer"),
           (spec.mixer_post_norm, spec.mixer_post_norm_prefix, "norm")]
    if spec.feed_forward is not None:
        out += [(spec.ffn_norm, spec.ffn_norm_prefix, "norm"), (spec.feed_forward, spec.ffn_prefix, "feed_forward"),
                (spec.ffn_post_norm, spec.ffn_post_norm_prefix, "norm")]
    return out
