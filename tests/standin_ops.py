"""Dense-tensor stand-ins for the kernel entry points, for tests without a GPU.

The product has no CPU path: ``llm_singularity_b200.kernels`` refuses to run
without its compiled CUDA libraries.  These functions mirror the signatures of
that module so that host-side logic (cache manager, block tables, step
metadata, scheduler, entry point) can be driven end to end on the CPU box where
the tests are written.  They are handed to ``Runtime(ops=...)`` explicitly by
tests and are never imported by the package.
"""
from __future__ import annotations

import torch


def prepare(names, verbose=False):
    return None


def scatter_i32(dst, idx, val):
    dst.view(-1)[idx.long()] = val


def move_i32(dst, dst_idx, src, src_idx):
    dst[dst_idx.long()] = src[src_idx.long()]


def embedding(table, ids, out):
    out.copy_(table[ids.long()].float())


def _rms(x, w, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def add_rmsnorm(residual, delta, weight, eps, out):
    if delta is not None:
        residual += delta.float()
    out.copy_(_rms(residual, weight, eps).to(out.dtype))


def gather_add_rmsnorm(residual, delta, rows, weight, eps, out):
    x = residual[rows.long()]
    if delta is not None:
        x = x + delta[rows.long()].float()
    out.copy_(_rms(x, weight, eps).to(out.dtype))


ACTIVATIONS = {"silu": 1, "gelu_tanh": 2, "none": 3}


def _act(g, name):
    if name == "silu":
        return g / (1 + torch.exp(-g))
    if name == "gelu_tanh":
        return 0.5 * g * (1 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    assert name == "none"
    return g


def linear(x, w, out_dtype=None, gated=False, activation="silu"):
    y = x.float() @ w.float().T
    if gated:
        y = _act(y[:, 0::2], activation) * y[:, 1::2]
    return y.to(out_dtype or x.dtype)


def swiglu(gate_up, out):
    g, u = gate_up[:, 0::2].float(), gate_up[:, 1::2].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store=True):
    T = qkv.shape[0]
    pos = ctx.positions.long()
    q = qkv[:, :nh * hd].view(T, nh, hd)
    k = qkv[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    if inv_freq is not None:
        half = rotary_dim // 2
        ang = pos.float()[:, None] * inv_freq[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        for x in (q, k):
            x0, x1 = x[..., :half].float().clone(), x[..., half:rotary_dim].float().clone()
            x[..., :half] = (x0 * cos - x1 * sin).to(x.dtype)
            x[..., half:rotary_dim] = (x0 * sin + x1 * cos).to(x.dtype)
    if store:
        ps = cache.page_size
        rows = ctx.table_rows.long()[ctx.token_req.long()]
        pages = cache.block_table[rows, pos // ps].long()
        assert (pages >= 0).all(), "write into a page that is not held"
        off = pos % ps
        cache.k_pages[pages, :, off, :] = k
        cache.v_pages[pages, :, off, :] = v


def rope_store_attention(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store, scale, window, out):
    rope_kv_store(qkv, nh, nkv, hd, ctx, cache, inv_freq, rotary_dim, store)
    paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out)


def paged_attention(qkv, nh, nkv, hd, ctx, cache, scale, window, out):
    T = qkv.shape[0]
    q = qkv[:, :nh * hd].view(T, nh, hd).float()
    ps = cache.page_size
    group = nh // nkv
    q_start = ctx.q_start.tolist()
    for r in range(ctx.n_requests):
        row = int(ctx.table_rows[r])
        kv_len = int(ctx.kv_len[r])
        n = q_start[r + 1] - q_start[r]
        lo_all = 0
        if window:
            lo_all = max(0, (kv_len - n) - window + 1)
        idx = torch.arange(lo_all, kv_len)
        pages = cache.block_table[row, idx // ps].long()
        assert (pages >= 0).all(), "read of a page that is not held"
        K = cache.k_pages[pages, :, idx % ps, :].float()     # [len, nkv, hd]
        V = cache.v_pages[pages, :, idx % ps, :].float()
        for i in range(n):
            p = kv_len - n + i
            mask = idx <= p
            if window:
                mask &= idx > p - window
            for h in range(nh):
                s = (K[:, h // group, :] @ q[q_start[r] + i, h]) * scale
                s = s.masked_fill(~mask, float("-inf"))
                w = torch.softmax(s, 0)
                out[q_start[r] + i, h * hd:(h + 1) * hd] = (w @ V[:, h // group, :]).to(out.dtype)


def sample(logits, params, top_k, prev_start, prev_tokens, out, work=None):
    import plain_llama
    for r in range(logits.shape[0]):
        t, p, pen, u = (float(x) for x in params[r])
        prev = ()
        if prev_start is not None:
            prev = prev_tokens[int(prev_start[r]):int(prev_start[r + 1])].tolist()
        out[r] = plain_llama.sample_plain(logits[r].tolist(), t, int(top_k[r]), p, pen, prev, u)


# ------------------------------------------- stand-ins for the kernels of streams normed after the sum
def _sig(z):
    return 1.0 / (1.0 + torch.exp(-z))


def _group_norm(x, w, groups, eps):
    T, n = x.shape
    p = x.reshape(T, groups, n // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    return p.reshape(T, n) * w


def cast_rows(x, out):
    out.copy_(x.to(out.dtype))


def post_group_norm(residual, delta, weight, eps, groups, alpha, out, gate=None, gate_bias=None,
                    keep_sum=False, dtype=None):
    s = alpha * residual
    if delta is not None:
        d = delta.float()
        if gate is not None:
            z = gate.float() + (gate_bias if gate_bias is not None else 0.0)
            d = d * _sig(z)
        s = s + d
    y = _group_norm(s, weight, groups, eps)
    residual.copy_(s if keep_sum else y)
    if out is not None:
        out.copy_(y.to(out.dtype))


def gather_group_norm(residual, rows, weight, eps, groups, out):
    out.copy_(_group_norm(residual[rows.long()], weight, groups, eps).to(out.dtype))


def unit_add(residual, y, weight, eps, out):
    y = y.float()
    residual += y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * weight
    if out is not None:
        out.copy_(residual.to(out.dtype))


def rows_norm_gate(x, weight, groups, eps, gate, out):
    n = x.shape[1]
    y = _group_norm(x, weight.repeat(n // weight.shape[0]), groups, eps)
    if gate is not None:
        y = y * _sig(gate.float())
    out.copy_(y.to(out.dtype))


def token_side_gate(g, table, token_ids, offset, activation, out):
    e = table[token_ids.long()][:, offset:offset + g.shape[1]].float()
    out.copy_((_act(g.float(), activation) * e).to(out.dtype))


def linear_scan(proj, q_off, k_off, v_off, heads, key_dim, value_dim, gate, decay, f_bias, floor,
                q_act, k_act, v_act, state, ctx, out):
    T = proj.shape[0]
    p = proj.float()
    q = _act(p[:, q_off:q_off + heads * key_dim], q_act).view(T, heads, key_dim)
    z = p[:, k_off:k_off + heads * key_dim]
    v = _act(p[:, v_off:v_off + heads * value_dim], v_act).view(T, heads, value_dim)
    if gate == "fixed_decay":
        a = decay[None, :, None].expand(T, heads, key_dim)
        b = _act(z, k_act).view(T, heads, key_dim)
    else:
        a = (floor + (1 - floor) * _sig(z + (f_bias if f_bias is not None else 0.0))).view(T, heads, key_dim)
        b = 1 - a
    q_start = ctx.q_start.tolist()
    for r in range(ctx.n_requests):
        S = state[int(ctx.table_rows[r])]                     # [heads, value_dim, key_dim]
        for t in range(q_start[r], q_start[r + 1]):
            S.copy_(a[t][:, None, :] * S + v[t][:, :, None] * b[t][:, None, :])
            out[t] = torch.einsum("hvd,hd->hv", S, q[t]).reshape(-1)


def _rotate(x, pos, inv_freq, rot_dims, pairing):
    """x [T, ..., n] float; dims below rot_dims turn."""
    if not rot_dims:
        return x
    out = x.clone()
    ang = pos.float()[:, None] * inv_freq[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    cos, sin = torch.cos(ang), torch.sin(ang)
    if pairing == "adjacent":
        a, b = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
        out[..., 0:rot_dims:2] = a * cos - b * sin
        out[..., 1:rot_dims:2] = b * cos + a * sin
    else:
        half = rot_dims // 2
        a, b = x[..., :half], x[..., half:rot_dims]
        out[..., :half] = a * cos - b * sin
        out[..., half:rot_dims] = b * cos + a * sin
    return out


def _rms(x, w, eps):                                                   # noqa: F811 (same as above)
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w


def latent_prep(down, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, inv_freq, rot_dims, pairing,
                ctx, cache, cq, write):
    cq.copy_(_rms(down[:, :q_rank], q_weight, eps).to(cq.dtype))
    if not write:
        return
    pos = ctx.positions.long()
    c = _rms(down[:, q_rank:q_rank + kv_rank], kv_weight, eps)
    kr = _rotate(down[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim], pos, inv_freq, rot_dims, pairing)
    ps = cache.page_size
    rows = ctx.table_rows.long()[ctx.token_req.long()]
    pages = cache.block_table[rows, pos // ps].long()
    assert (pages >= 0).all(), "write into a page that is not held"
    cache.pages[pages, pos % ps] = torch.cat([c, kr], dim=1).to(cache.pages.dtype)


def latent_query_rot(q, qf, heads, plain, rot_dim, kv_rank, inv_freq, rot_dims, pairing, ctx):
    T = q.shape[0]
    part = q.view(T, heads, plain + rot_dim)[:, :, plain:]
    qf[:, :, kv_rank:] = _rotate(part, ctx.positions.long(), inv_freq, rot_dims, pairing)


def batched_nt(a, b, out):
    out.copy_(torch.einsum("mhk,hnk->mhn", a.float(), b.float()).to(out.dtype))


def latent_attention(qf, ctx, cache, kv_rank, rot_dim, scale, out):
    ps = cache.page_size
    q_start = ctx.q_start.tolist()
    for r in range(ctx.n_requests):
        row, kv_len = int(ctx.table_rows[r]), int(ctx.kv_len[r])
        n = q_start[r + 1] - q_start[r]
        idx = torch.arange(kv_len)
        pages = cache.block_table[row, idx // ps].long()
        assert (pages >= 0).all(), "read of a page that is not held"
        rows = cache.pages[pages, idx % ps].float()                   # [len, width]
        for i in range(n):
            p = kv_len - n + i
            s = (qf[q_start[r] + i] @ rows[:p + 1].T) * scale          # [heads, p + 1]
            w = torch.softmax(s, -1)
            out[q_start[r] + i] = (w @ rows[:p + 1, :kv_rank]).to(out.dtype)


def moe_route(logits, top, score, renormalize, ids, weights):
    s = _sig(logits) if score == "sigmoid" else torch.softmax(logits, -1)
    # the largest first, the lower index first among equals
    order = torch.sort(-logits, dim=-1, stable=True).indices[:, :top]
    w = torch.gather(s, 1, order)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    ids.copy_(order.to(torch.int32))
    weights.copy_(w)


def moe_experts(x, ids, weights, w_gate_up, w_down, activation, weight_on, out):
    T = x.shape[0]
    acc = torch.zeros(T, x.shape[1])
    for t in range(T):
        for k in range(ids.shape[1]):
            e, w = int(ids[t, k]), weights[t, k]
            u = (w * x[t].float()).to(x.dtype).float() if weight_on == "input" else x[t].float()
            gu = w_gate_up[e].float() @ u
            a = (_act(gu[0::2], activation) * gu[1::2]).to(x.dtype).float()
            y = w_down[e].float() @ a
            acc[t] += y if weight_on == "input" else w * y
    out.copy_(acc.to(out.dtype))


def moe_routed_experts(x, logits, top, score, renormalize, w_gate_up, w_down, activation, weight_on, out):
    ids = torch.empty(logits.shape[0], top, dtype=torch.int32)
    weights = torch.empty(logits.shape[0], top, dtype=torch.float32)
    moe_route(logits, top, score, renormalize, ids, weights)
    moe_experts(x, ids, weights, w_gate_up, w_down, activation, weight_on, out)
