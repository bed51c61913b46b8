"""The Fogezen decoder in plain, slow arithmetic: one function per mechanism, float64, no cache.

A whole sequence goes in; where a mechanism carries something from one token to the next it is
walked token by token.  Nothing here is shared with the engine's parts or kernels.  ``cfg`` is the
dictionary that config.json holds, ``W`` maps tensor names to float64 tensors.

Notation: ``x`` is the residual stream [T, width]; ``h`` is what a sublayer reads; a linear map
stored [out, in] is applied as ``h @ M.T``; ``pos`` are the tokens' places in their sequence.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ small functions
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w)


def turn_neighbours(v, pos, dims, base):
    """Dims (2i, 2i+1), i < dims/2, of the last axis turn by ``pos * base^(-2i/dims)``; the dims
    from ``dims`` on stay.  ``v``: [T, heads, n]."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=F64)
    ang = pos.to(F64)[:, None] * torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def visible(pos, chunk=None):
    """[T, T] truth table: query i sees key j if j is not later and, with ``chunk``, if both lie in
    the same stretch of ``chunk`` places counted from the start of the sequence."""
    i, j = pos[:, None], pos[None, :]
    ok = j <= i
    if chunk is not None:
        ok = ok & (torch.div(i, chunk, rounding_mode="floor") == torch.div(j, chunk, rounding_mode="floor"))
    return ok


def softmax_heads(q, k, v, scale, ok):
    """q [T, H, D], k [T, G, D], v [T, G, V]; head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~ok, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


# ------------------------------------------------------------------------- mixers
def biased_attention(h, W, p, m, pos):
    """Softmax attention over all earlier places, with biased projections, no rotation, and a
    query that grows with the logarithm of its place in steps of ``every``."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, V)
    qt = m.get("q_temp")
    if qt is not None:
        steps = torch.div(pos + 1, int(qt["every"]), rounding_mode="floor").to(F64)
        q = q * (1.0 + float(qt["coef"]) * torch.log(steps + 1.0))[:, None, None]
    o = softmax_heads(q, k, v, float(m["scale"]), visible(pos))
    return o.reshape(T, H * V) @ W[p + "o"].T


def chunked_gated_attention(h, W, p, m, eps, pos):
    """Softmax attention inside stretches of ``mask.size`` places; queries and keys are brought to
    unit rms per head (one weight for all heads) and then turned; a sigmoid gate of the input
    multiplies the heads' outputs."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ W[p + "q"].T).reshape(T, H, D), eps) * W[p + "q.norm"]
    k = unit_rms((h @ W[p + "k"].T).reshape(T, G, D), eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    rot = m.get("rot")
    if rot is not None:
        q = turn_neighbours(q, pos, int(rot["dims"]), float(rot["base"]))
        k = turn_neighbours(k, pos, int(rot["dims"]), float(rot["base"]))
    chunk = m["mask"]["size"] if m.get("mask") else None
    o = softmax_heads(q, k, v, float(m["scale"]), visible(pos, chunk))
    o = o.reshape(T, H * V) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def matrix_memory(h, W, p, m, eps, state=None):
    """A matrix memory per head with exponential input gate and a running maximum m that keeps the
    exponentials in range.  state = (S [H, D, V], n [H, D], m [H]); all zero at the start."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[p + "q"].T).reshape(T, H, D) / math.sqrt(D)
    k = (h @ W[p + "k"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    gi = cap * torch.tanh((h @ W[p + "i"].T + W[p + "i.b"]) / cap)                      # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[p + "f"].T + W[p + "f.b"]) / cap))
    if state is None:
        S, n, mx = torch.zeros(H, D, V, dtype=F64), torch.zeros(H, D, dtype=F64), torch.zeros(H, dtype=F64)
    else:
        S, n, mx = state
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, write = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + write[:, None, None] * (k[t][:, :, None] * v[t][:, None, :])
        n = keep[:, None] * n + write[:, None] * k[t]
        mx = new
        dot = (n * q[t]).sum(-1)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / (torch.maximum(dot.abs(), torch.exp(-mx)) + 1e-6)[:, None]
    y = unit_rms(o, eps).reshape(T, H * V) * W[p + "norm"]
    y = y * torch.sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T, (S, n, mx)


def side_by_side(h, W, p, m, eps, pos):
    """Both mixers read h; each result is normed over the width with its own weight; half the sum."""
    left = chunked_gated_attention(h, W, p + "left.", m["left"], eps, pos)
    right, _ = matrix_memory(h, W, p + "right.", m["right"], eps)
    return 0.5 * (unit_rms(left, eps) * W[p + "left.out"] + unit_rms(right, eps) * W[p + "right.out"])


def gated_feed_forward(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# -------------------------------------------------------------------------- model
def run_order(cfg):
    """[(layer, pass or None)]: the layers in the order they run; a looped stretch runs ``times``
    times in a row, and the first layer of each pass carries the pass's number."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(L)]
    a, b, n = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(a)]
    for t in range(n):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, L)]


def layer(x, cfg, W, i, pos):
    entry = cfg["layers"][i]
    eps, mult, p = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0)), f"l{i}."
    h = norm_around_zero(x, W[p + "norm1"], eps)
    if entry["type"] == "attention":
        y = biased_attention(h, W, p + "mix.", entry["mixer"], pos)
    elif entry["type"] == "parallel":
        y = side_by_side(h, W, p + "mix.", entry["mixer"], eps, pos)
    else:
        raise ValueError(entry["type"])
    x = x + mult * norm_around_zero(y, W[p + "norm1b"], eps)
    if entry.get("mlp") is not None:
        y = gated_feed_forward(norm_around_zero(x, W[p + "norm2"], eps), W, p + "mlp.")
        x = x + mult * norm_around_zero(y, W[p + "norm2b"], eps)
    return x


def forward(cfg, W, tokens, streams=None):
    """Logits [T, vocab] of one whole sequence.  ``streams``: a list that receives the residual
    stream after every layer run."""
    W = {n: t.to(F64) for n, t in W.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(len(ids))
    x = W["embed"][ids] * float(cfg.get("embedding", {}).get("scale", 1.0))
    for i, t in run_order(cfg):
        if t is not None:
            x = x + W["loop.step"][t]
        x = layer(x, cfg, W, i, pos)
        if streams is not None:
            streams.append(x.clone())
    return norm_around_zero(x, W["final.norm"], float(cfg["norm"]["eps"])) @ W["embed"].T
