"""Linear attention with a matrix state per head and request.

Per head, with q and the write vector b of ``key_dim`` channels and v of ``value_dim``:

    S_t = diag(a_t) S_(t-1) + b_t v_t^T          o_t = S_t^T q_t

The spec's ``gate`` says where a and b come from: one constant per head and a key projection
("fixed_decay": S decays uniformly, b = act(W_k x)), or a forget gate per channel with a learnt
floor that also sets the write strength ("forget": a = floor + (1 - floor) sigmoid(W_f x + bias),
b = 1 - a; no key, no other scale).  The outputs are RMS-normed (all heads together with one weight
over the row, or each head by itself with one weight of head size), optionally multiplied by
sigmoid(W_g x), and projected by W_o.

The state starts at zero when a request takes a slot, is 32-bit, and is carried from step to
step in the slot's row of a ``StateSpec`` cache.  One product makes all projections of a step
(rows of W_q, then W_k or W_f, then W_v, then W_g), one kernel walks every request's tokens in
order (prompt portions and single tokens alike), one kernel norms and gates.  Gates, decays, the
state and the norm are 32-bit whatever the compute dtype.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import ParamSpec, Part, StateSpec, register_mixer


@register_mixer("linear_recurrence")
class LinearRecurrence(Part):
    graph_safe = True
    kernels = ("gemm", "linear_scan", "rownorm")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        s = spec
        if s.gate not in ("fixed_decay", "forget"):
            raise ValueError(f"gate '{s.gate}' is not known (fixed_decay, forget)")
        if s.gate == "fixed_decay" and len(s.decay) != s.num_heads:
            raise ValueError(f"{len(s.decay)} decays for {s.num_heads} heads")
        if s.out_norm not in ("all", "per_head"):
            raise ValueError(f"out_norm '{s.out_norm}' is not known (all, per_head)")
        for a in (s.q_activation, s.k_activation, s.v_activation):
            if a not in ("none", "silu"):
                raise ValueError(f"activation '{a}' is not implemented here (none, silu)")
        self.qk = s.num_heads * s.key_dim
        self.vv = s.num_heads * s.value_dim
        self.decay = None
        if s.gate == "fixed_decay":
            self.decay = torch.tensor([float(d) for d in s.decay], dtype=torch.float32, device=rt.device)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H = spec.hidden_size
        qk, vv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        p = {"q": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "o": ParamSpec((H, vv))}
        if spec.gate == "fixed_decay":
            p["k"] = ParamSpec((qk, H))
        else:
            p["f"] = ParamSpec((qk, H))
            p["f_bias"] = ParamSpec((qk,), role="vector", init="normal")
            p["floor"] = ParamSpec((qk,), role="vector", init="normal")
        if spec.out_gate:
            p["g"] = ParamSpec((vv, H))
        p["norm"] = ParamSpec((vv if spec.out_norm == "all" else spec.value_dim,), role="vector", init="ones")
        return p

    def load(self, tensors):
        s = self.spec
        second = tensors["k"] if s.gate == "fixed_decay" else tensors["f"]
        rows = [tensors["q"], second, tensors["v"]] + ([tensors["g"]] if s.out_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_out = tensors["o"].contiguous()
        self.norm = tensors["norm"]
        self.f_bias = tensors.get("f_bias")
        self.floor = tensors.get("floor")

    def cache_spec(self):
        s = self.spec
        return StateSpec((s.num_heads, s.value_dim, s.key_dim))     # key channels contiguous

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops = self.spec, self.rt.ops
        proj = ops.linear(x, self.w_in)                               # [T, q | k or f | v | g]
        o = self.rt.empty(x.shape[0], self.vv, dtype=torch.float32)
        ops.linear_scan(proj, 0, self.qk, 2 * self.qk, s.num_heads, s.key_dim, s.value_dim, s.gate,
                        self.decay, self.f_bias, self.floor, s.q_activation, s.k_activation, s.v_activation,
                        cache.state, ctx, o)
        gate = proj[:, 2 * self.qk + self.vv:] if s.out_gate else None
        y = self.rt.empty(x.shape[0], self.vv)
        ops.rows_norm_gate(o, self.norm, 1 if s.out_norm == "all" else s.num_heads, s.eps, gate, y)
        return ops.linear(y, self.w_out)
