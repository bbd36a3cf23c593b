"""Linear attention as a recurrence with a float32 state per request and head.

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t

One fused product [q | k | v | gate (| decay projection)] of the mixer's input in float32; the recurrence over each
request's rows, from and into the request's state slot (csrc/mixers.cu: ``linear_scan``); an RMS norm of the output,
times an activation of the gate (``norm_gate``); the output product.  The decay is a constant per head or
sigmoid(W2 (W1 h) + b2) ** (1 / tau) per key channel; both, like the state, in float32.  ``LinearAttentionSpec`` names
every choice.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..cache import StateSlot
from ..weights import MATRIX, VECTOR, TensorDecl
from .base import register
from .program import ACT, record


@register("mixer", "linear_attention")
class LinearAttention:
    @staticmethod
    def _widths(spec):
        return spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim

    @staticmethod
    def tensor_decls(spec) -> Dict[str, TensorDecl]:
        d = spec.hidden_size
        nk, nv = LinearAttention._widths(spec)
        decls = {spec.q_name: TensorDecl((nk, d)), spec.k_name: TensorDecl((nk, d)), spec.v_name: TensorDecl((nv, d)),
                 spec.gate_name: TensorDecl((nv, d)), spec.o_name: TensorDecl((d, nv)),
                 spec.norm_name: TensorDecl((spec.v_head_dim if spec.norm_per_head else nv,), VECTOR, init="ones")}
        if spec.decay is None:
            decls[spec.decay_down_name] = TensorDecl((spec.decay_rank, d))
            decls[spec.decay_up_name] = TensorDecl((nk, spec.decay_rank))
            decls[spec.decay_up_name + spec.bias_suffix] = TensorDecl((nk,), VECTOR, init="zeros")
        return decls

    @staticmethod
    def cache_need(spec):
        return StateSlot((spec.num_heads, spec.head_dim, spec.v_head_dim), "float32")

    def __init__(self, spec, weights, prefix: str, runtime):
        self.spec, self.runtime = spec, runtime
        if spec.decay is None and spec.decay_rank <= 0:
            raise ValueError("a linear attention needs constant decays or a decay projection")
        if spec.decay is not None and len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        names = [spec.q_name, spec.k_name, spec.v_name, spec.gate_name] + ([spec.decay_down_name] if spec.decay is None else [])
        self.w_in = weights.get_rows([prefix + n for n in names], MATRIX)
        self.w_o = weights.get(prefix + spec.o_name, MATRIX)
        self.norm = weights.get(prefix + spec.norm_name, VECTOR)
        self.decay = self.w2 = self.b2 = None
        if spec.decay is None:
            self.w2 = weights.get(prefix + spec.decay_up_name, MATRIX)
            self.b2 = weights.get(prefix + spec.decay_up_name + spec.bias_suffix, VECTOR)
        else:
            self.decay = torch.tensor(spec.decay, dtype=torch.float64).to(torch.float32).to(runtime.device)

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o, self.w2) if t is not None)

    def plan_delta(self, program, view, writes_cache: bool = True, state_view=None) -> None:
        """Three records: the fused product (h -> float32 rows), the recurrence with norm and gate (-> o), the output product
        into the delta slot."""
        s = self.spec
        nk, nv = self._widths(s)
        ld = self.w_in.shape[0]
        program.emit_records([
            record("linear", "h", "tmp", n=ld, k=s.hidden_size, w=self.w_in),
            record("linear_attention", "tmp", "o", heads=s.num_heads, head_dim=s.head_dim, v_head_dim=s.v_head_dim, ld=ld,
                   q_off=0, k_off=nk, v_off=2 * nk, g_off=2 * nk + nv, r_off=2 * nk + 2 * nv, act=ACT[s.qkv_act], q_scale=s.q_scale,
                   gate_act=ACT[s.gate_act], per_head_norm=s.norm_per_head, eps=s.norm_eps, vec=self.norm, decay=self.decay,
                   w2=self.w2, b2=self.b2, rank=s.decay_rank if s.decay is None else 0, tau=s.decay_tau, state=view.state),
            record("linear", "o", "delta", n=s.hidden_size, k=nv, w=self.w_o),
        ], keep=(self.w_in, self.w_o, self.norm, self.decay, self.w2, self.b2, view.state))

    def forward(self, h: torch.Tensor, ctx, view, writes_cache: bool = True) -> torch.Tensor:
        """The part alone: its own records over ``h``; float32 ``[T, hidden]``."""
        from .program import run_part_alone
        return run_part_alone(self.runtime, lambda program: self.plan_delta(program, view, writes_cache), ctx, h,
                              self.spec.hidden_size, result_slot="delta")
