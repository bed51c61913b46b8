"""The Ridotar decoder in plain, slow arithmetic: one function per mechanism, float64, no cache.

A whole sequence goes in, token by token where a mechanism carries something from one token to
the next; nothing here is shared with the engine's parts or kernels.  ``cfg`` is the dictionary
that config.json holds, ``W`` maps tensor names to float64 tensors.

Notation: ``x`` is the residual stream [T, width]; ``h`` is what a sublayer reads; a linear map
stored [out, in] is applied as ``h @ M.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ------------------------------------------------------------------ small functions
def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def grouped_rms_norm(x, weight, groups, eps):
    """The last axis in ``groups`` equal consecutive parts, each brought to unit rms; then the weight."""
    shape = x.shape
    parts = x.reshape(*shape[:-1], groups, shape[-1] // groups)
    return rms_unit(parts, eps).reshape(shape) * weight


def rotate_adjacent_pairs(v, positions, dims, base):
    """Dims (2i, 2i+1), i < dims/2, of the last axis turn by ``positions * base^(-2i/dims)``;
    the dims from ``dims`` on stay.  ``v``: [T, ..., n], ``positions``: [T]."""
    out = v.clone()
    i = torch.arange(dims // 2, dtype=F64)
    freq = torch.pow(torch.tensor(float(base), dtype=F64), -2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]                  # [T, dims/2]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * torch.cos(ang) - b * torch.sin(ang)
    out[..., 1:dims:2] = b * torch.cos(ang) + a * torch.sin(ang)
    return out


# ------------------------------------------------------------------------- mixers
def lightning_mixer(h, W, p, m, eps, state=None):
    """Linear attention with one fixed decay per head.  State per head [dim, vdim], from zero."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, D)
    k = silu(h @ W[p + "k"].T).reshape(T, H, D)
    v = silu(h @ W[p + "v"].T).reshape(T, H, V)
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms_unit(o.reshape(T, H * V), eps) * W[p + "norm"]
    y = y * torch.sigmoid(h @ W[p + "g"].T)
    return y @ W[p + "o"].T, S


def hgrn2_mixer(h, W, p, m, eps, state=None):
    """Linear attention whose forget gate f also gives the write strength 1 - f.  f has a floor."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, D)
    v = (h @ W[p + "v"].T).reshape(T, H, V)
    floor = W[p + "lower"]
    f = floor + (1.0 - floor) * torch.sigmoid(h @ W[p + "f"].T + W[p + "f.b"])
    f = f.reshape(T, H, D)
    S = torch.zeros(H, D, V, dtype=F64) if state is None else state
    o = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms_unit(o, eps) * W[p + "norm"]                 # per head, over vdim
    return y.reshape(T, H * V) @ W[p + "o"].T, S


def latent_kv(h, W, p, m, eps, positions):
    """What a latent-attention layer caches: the normed latent [T, kv_rank] and the rotated key part
    [T, rot_dim] that all heads share."""
    R, rd = m["kv_rank"], m["rot_dim"]
    down = h @ W[p + "dkv"].T
    c = rms_unit(down[:, :R], eps) * W[p + "dkv.norm"]
    kr = rotate_adjacent_pairs(down[:, R:R + rd], positions, m["rot"]["dims"], m["rot"]["base"])
    return c, kr


def latent_attention_mixer(h, W, p, m, eps, positions, c, kr):
    """Causal softmax attention with keys and values made per head from the latent ``c`` [S, kv_rank]
    and the shared rotated key part ``kr`` [S, rot_dim]; the queries (the last T of the S places)
    come through a latent of their own."""
    T, S = h.shape[0], c.shape[0]
    H, D, rd, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, D + rd)
    q_plain = q[..., :D]
    q_rot = rotate_adjacent_pairs(q[..., D:], positions, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ W[p + "uk"].T).reshape(S, H, D)
    val = (c @ W[p + "uv"].T).reshape(S, H, V)
    out = torch.zeros(T, H, V, dtype=F64)
    for t in range(T):
        n = S - T + t + 1                                 # keys at places 0 .. n-1 are seen
        s = torch.einsum("hd,shd->hs", q_plain[t], k_plain[:n]) + q_rot[t] @ kr[:n].T
        w = torch.softmax(s * m["scale"], dim=-1)
        out[t] = torch.einsum("hs,shv->hv", w, val[:n])
    return out.reshape(T, H * V) @ W[p + "o"].T


# ------------------------------------------------------------------- feed-forward
def moe_feed_forward(h, W, p, f):
    """Sigmoid scores, the ``top`` largest chosen, each chosen expert fed ``score * h``."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ W[p + "router"].T)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            u = s[t, e] * h[t]
            a = silu(W[p + f"e{e}.gate"] @ u) * (W[p + f"e{e}.up"] @ u)
            out[t] += W[p + f"e{e}.down"] @ a
    return out


# --------------------------------------------------------------------------- model
def model_norm(x, weight, cfg):
    return grouped_rms_norm(x, weight, cfg["norm"]["groups"], cfg["norm"]["eps"])


def forward(cfg, W, tokens, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer if asked)."""
    W = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in W.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = W["embed"][tokens]
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        L, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        h = x
        if kind == "lightning":
            y, _ = lightning_mixer(h, W, L + "mix.", m, eps)
        elif kind == "hgrn2":
            y, _ = hgrn2_mixer(h, W, L + "mix.", m, eps)
        elif kind == "latent_attention":
            if "kv_from" in m:
                c, kr = kept[m["kv_from"]]
            else:
                c, kr = kept[i] = latent_kv(h, W, L + "mix.", m, eps, positions)
            y = latent_attention_mixer(h, W, L + "mix.", m, eps, positions, c, kr)
        else:
            raise ValueError(kind)
        y = y * torch.sigmoid(h @ W[L + "rg1"].T + W[L + "rg1.b"])
        x = model_norm(alpha * x + y, W[L + "norm1"], cfg)
        if layer.get("mlp") is not None:
            h = x
            y = moe_feed_forward(h, W, L + "mlp.", layer["mlp"])
            y = y * torch.sigmoid(h @ W[L + "rg2"].T + W[L + "rg2.b"])
            x = model_norm(alpha * x + y, W[L + "norm2"], cfg)
        if cfg.get("token_side"):
            d = cfg["token_side"]["dim"]
            e = W["side.embed"][tokens][:, i * d:(i + 1) * d]
            g = gelu_tanh(x @ W[L + "side.gate"].T) * e
            x = x + rms_unit(g @ W[L + "side.proj"].T, eps) * W[L + "side.norm"]
        after.append(x)
    logits = model_norm(x, W["final.norm"], cfg) @ W["embed"].T
    return (logits, torch.stack(after)) if keep_layers else logits
