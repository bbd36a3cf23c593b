"""A state-space mixer with input-dependent step sizes (a selective scan).

    [x | z] = W_in h;  x <- silu(conv(x));  [dt part | B | C] = W_x x;  dt = softplus(W_dt dt part + b)
    S <- exp(dt A) S + dt x B,  y = S C + D x  per channel;  out = W_o (y silu(z))          A = -exp(A_log)

The in-projection in float32 rows; the convolution with its activation (``causal_conv``: float32 for the scan and the
activation type for the product), whose last taps - 1 inputs per request are state; the small projection; the scan with
the step sizes formed inside it, everything in float32, from and into the request's state slot; the output product.
Kernels: csrc/blocks.cu.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import StateSlot
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import ACT, record


@register("mixer", "selective_scan")
class SelectiveScan:
    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d, E, N, K = spec.hidden_size, spec.inner, spec.state_size, spec.dt_rank
        b = spec.bias_suffix
        return {spec.in_name: TensorDecl((2 * E, d)),
                spec.conv_name: TensorDecl((E, spec.conv_taps), VECTOR, init="taps"),
                spec.conv_name + b: TensorDecl((E,), VECTOR, init="zeros"),
                spec.x_name: TensorDecl((K + 2 * N, E)),
                spec.dt_name: TensorDecl((E, K)),
                spec.dt_name + b: TensorDecl((E,), VECTOR, init="zeros"),
                spec.a_log_name: TensorDecl((E, N), VECTOR, init="zeros"),
                spec.d_name: TensorDecl((E,), VECTOR, init="ones"),
                spec.o_name: TensorDecl((d, E))}

    @staticmethod
    def cache_need(spec):
        return StateSlot((spec.inner, spec.state_size), "float32")

    @staticmethod
    def state_need(spec, writes_cache: bool = True):
        """The convolution's tails: the last taps - 1 inputs of every channel."""
        return StateSlot((spec.conv_taps - 1, spec.inner), "float32") if spec.conv_taps > 1 else None

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        b = spec.bias_suffix
        vec = lambda name: weights.get(prefix + name, VECTOR)
        self.w_in = weights.get(prefix + spec.in_name, MATRIX)
        self.w_x = weights.get(prefix + spec.x_name, MATRIX)
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        self.taps, self.conv_bias = vec(spec.conv_name), vec(spec.conv_name + b)
        self.w_dt = weights.get(prefix + spec.dt_name, MATRIX)      # float32 rows meet it unrounded (csrc/blocks.cu: scan_steps)
        self.dt_bias, self.skip = vec(spec.dt_name + b), vec(spec.d_name)
        self.A = (-torch.exp(vec(spec.a_log_name).to(torch.float32))).contiguous()

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_x, self.w_o, self.w_dt, self.A))

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None) -> None:
        """Five records: in-projection, convolution, small projection, scan, output product into the delta slot."""
        s = self.spec
        E, N, K = s.inner, s.state_size, s.dt_rank
        tails = state_view.state if state_view is not None else None
        if s.conv_taps > 1 and tails is None:
            raise ValueError("a convolution of more than one tap needs its tails' state")
        program.emit_records([
            record("linear", "h", "tmp", n=2 * E, k=s.hidden_size, w=self.w_in),
            record("causal_conv", "tmp", "o", out2_slot="mix", n=E, ld=2 * E, q_off=0, taps=s.conv_taps, conv_q=self.taps,
                   bias=self.conv_bias, act=ACT["silu"], state=tails),
            record("linear", "o", "scan", n=K + 2 * N, k=E, w=self.w_x),
            record("selective_scan", "mix", "act", in2_slot="scan", n=E, k=N, rank=K, w2=self.w_dt, b2=self.dt_bias, decay=self.A,
                   vec=self.skip, q_off=0, g_off=E, ld=2 * E, state=view.state),
            record("linear", "act", "delta", n=s.hidden_size, k=E, w=self.w_o),
        ], keep=(self.w_in, self.w_x, self.w_o, self.taps, self.conv_bias, self.w_dt, self.dt_bias, self.skip, self.A, tails, view.state))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True, state_view=None) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache, state_view), ctx, h,
                              self.spec.hidden_size, result_slot="delta")
