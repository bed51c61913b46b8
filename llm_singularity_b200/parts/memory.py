"""A matrix memory per head and request with an exponential input gate (the mLSTM cell).

Per head, with q (scaled by ``key_dim^-1/2``) and k of ``key_dim`` channels, v of ``value_dim``, the
log gates ``i = cap tanh((W_i x + b_i) / cap)``, ``f = logsigmoid(cap tanh((W_f x + b_f) / cap))`` and
a running maximum m (0 when a request begins):

    m_t = max(f + m_(t-1), i)
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T           n_t likewise with k alone
    o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)

Each head's o is brought to unit rms, the heads are concatenated, multiplied by one weight and by
``sigmoid(W_g x)``, and projected by W_o.

n is S with a value column of ones, so the walk is the one of linear attention
(``csrc/linear_scan.cu``) with two numbers per token and head given from outside and one more
column; a kernel before it makes those numbers (it walks the chain of maxima in order), a kernel
behind it divides, norms and gates.  The state (S with n as its last column, and m) is 32-bit,
starts at zero when a request takes a slot and is carried in the slot's rows of two ``StateSpec``
caches.  Gates, maxima, exponentials, the state and the norm are 32-bit whatever the compute dtype.
"""
from __future__ import annotations

from typing import Dict

import torch

from .base import CompositeCacheSpec, ParamSpec, Part, StateSpec, register_mixer


@register_mixer("matrix_memory")
class MatrixMemory(Part):
    graph_safe = True
    kernels = ("gemm", "matrix_memory", "linear_scan")

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if not spec.gate_cap > 0:
            raise ValueError(f"gate_cap must be positive, got {spec.gate_cap}")
        self.qk = spec.num_heads * spec.key_dim
        self.vv = spec.num_heads * spec.value_dim

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        H, n = spec.hidden_size, spec.num_heads
        qk, vv = n * spec.key_dim, n * spec.value_dim
        p = {"q": ParamSpec((qk, H)), "k": ParamSpec((qk, H)), "v": ParamSpec((vv, H)), "o": ParamSpec((H, vv)),
             "i": ParamSpec((n, H)), "i_bias": ParamSpec((n,), role="vector", init="normal"),
             "f": ParamSpec((n, H)), "f_bias": ParamSpec((n,), role="vector", init="normal"),
             "norm": ParamSpec((vv,), role="vector", init="ones")}
        if spec.out_gate:
            p["g"] = ParamSpec((vv, H))
        return p

    def load(self, tensors):
        rows = [tensors["q"], tensors["k"], tensors["v"]] + ([tensors["g"]] if self.spec.out_gate else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_gates = torch.cat([tensors["i"], tensors["f"]], dim=0).contiguous()
        self.w_out = tensors["o"].contiguous()
        self.norm = tensors["norm"]
        self.i_bias, self.f_bias = tensors["i_bias"], tensors["f_bias"]

    def cache_spec(self):
        s = self.spec
        return CompositeCacheSpec((StateSpec((s.num_heads, s.value_dim + 1, s.key_dim)),     # S, and n behind it
                                   StateSpec((s.num_heads,))))                               # m

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        s, ops = self.spec, self.rt.ops
        T, n = x.shape[0], s.num_heads
        proj = ops.linear(x, self.w_in)                                   # [T, q | k | v | g]
        raw = ops.linear(x, self.w_gates, out_dtype=torch.float32)        # [T, i | f]
        gates = self.rt.empty(3, T, n, dtype=torch.float32)               # keep, write, floor
        ops.memory_gates(raw, self.i_bias, self.f_bias, s.gate_cap, cache[1].state, ctx, gates)
        walked = self.rt.empty(T, n * (s.value_dim + 1), dtype=torch.float32)
        ops.linear_scan(proj, 0, self.qk, 2 * self.qk, n, s.key_dim, s.value_dim, "given", None, None, None,
                        "none", "none", "none", cache[0].state, ctx, walked, keep=gates[0], write=gates[1],
                        ones=True, q_scale=float(s.key_dim) ** -0.5)
        gate = proj[:, 2 * self.qk + self.vv:] if s.out_gate else None
        y = self.rt.empty(T, self.vv)
        ops.memory_output(walked, gates[2], self.norm, gate, s.eps, y)
        return ops.linear(y, self.w_out)
