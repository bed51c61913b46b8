"""The Fogezen design in the engine against tests/plain_fogezen.py (float64, whole sequences, one
function per mechanism, no cache).  Every test makes its own small model (tests/fogezen_util.py).

Covered: each mixer alone, with and without feed-forward; whole prompts against token-by-token
stepping; portions of changing size down to two tokens; batches of unequal requests against each
alone; pages and state slots given back and used again; keys far back, at page borders, among the
first tokens and just inside and just outside a chunk, in prompts and in decoding, with one score
made to stand out; long decoding through many pages and chunks; other sizes; the kernels of the
design one by one against plain functions; greedy generation through the engine's entry point.
"""
import math

import pytest
import torch

import fogezen_util as U
import plain_fogezen as P

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def _setup(tmp_path, cfg, seed, **kw):
    W = U.make_weights(cfg, seed, **kw)
    return W, U.write_model(str(tmp_path / f"m{seed}"), cfg, W)


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
def test_each_mixer_alone(tmp_path, dtype):
    cases = [("attention", True, {}), ("parallel", True, {}), ("attention", False, dict(heads=4, kv=4, dim=32, vdim=32)),
             ("parallel", False, dict(chunk=None, rot=None)), ("parallel", True, dict(heads=2, kv=1, dim=64, vdim=32, chunk=16,
                                                                                      rot=(64, 100.0)))]
    for n, (kind, mlp, kw) in enumerate(cases):
        cfg = U.single(kind, mlp, **kw)
        W, path = _setup(tmp_path, cfg, 100 + n)
        toks = U.tokens_for(cfg, 77, n)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=8)
        whole = U.run_cuts(r, "w", toks, [77])
        assert U.close(whole, want, dtype), (kind, mlp, kw, U.rel_err(whole, want))
        stepped = U.run_cuts(r, "s", toks, [1] * 77)             # the same slot and pages once more
        assert U.close(stepped, want, dtype), (kind, mlp, kw, "token by token", U.rel_err(stepped, want))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_portions_of_any_size(tmp_path, dtype, name, n=150):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 7)
    toks = U.tokens_for(cfg, n, 3)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, pages=12)
    ragged, pattern = [], [2, 15, 1, 16, 17, 31, 2, 2, 33, 5]
    while sum(ragged) < n:
        ragged.append(min(pattern[len(ragged) % len(pattern)], n - sum(ragged)))
    for cuts in ([n], [n - 40] + [1] * 40, ragged, [16] * (n // 16) + [n % 16], [2] * (n // 2)):
        cuts = [c for c in cuts if c]
        got = U.run_cuts(r, "p", toks, cuts)
        assert U.close(got, want, dtype), (cuts[:6], U.rel_err(got, want))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path, dtype, name):
    """Four requests of unequal length stepped together (portions beside single tokens, a request
    left out of some steps, ends at different times, a fifth request taking over a freed slot and
    freed pages) against the plain model of each alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 9)
    lens = {"a": 70, "b": 23, "c": 41, "d": 1, "e": 37}
    toks = {k: U.tokens_for(cfg, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: U.plain_logits(cfg, W, t) for k, t in toks.items()}
    r = U.make_runner(path, dtype, pages=12, slots=4)      # 192 token places for 172 tokens
    plan = [[("a", 33), ("b", 2)], [("a", 1), ("b", 17), ("c", 5)], [("d", 1), ("c", 1), ("a", 1)],
            [("b", 1), ("c", 30), ("a", 20)], [("b", 1), ("a", 1), ("c", 1)], [("b", 1), ("c", 2)],
            [("b", 1), ("e", 3), ("a", 14), ("c", 2)], [("e", 33), ("b", 0)], [("e", 1)]]
    at = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in plan:
        entries, who = [], []
        for k, n in step:
            n = min(n, lens[k] - at[k])
            if n <= 0:
                continue
            if not r.cache.has(k):
                assert r.open(k), f"no slot for {k}"
            entries.append(StepEntry(k, toks[k][at[k]:at[k] + n], list(range(n))))
            who.append((k, n))
        logits = r.step(entries).float().cpu()
        row = 0
        for k, n in who:
            got[k].append(logits[row:row + n].clone())
            row += n
            at[k] += n
            if at[k] == lens[k]:
                r.close(k)
    r.check_kernels()
    assert at == lens
    for k in lens:
        assert U.close(torch.cat(got[k]), want[k], dtype), (k, U.rel_err(torch.cat(got[k]), want[k]))
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_keys_page_borders_chunk_edges_and_first_tokens(tmp_path, dtype):
    """A strongly peaked softmax over a few hundred keys, chunks of 50 against pages of 16: a key
    that is lost, one page or one place off, a first token left out or a chunk edge one token off
    changes the logits by far more than the tolerance."""
    for kind, kw, seed in (("attention", {}, 31), ("parallel", dict(chunk=50), 32)):
        cfg = U.single(kind, mlp=False, **kw)
        W, path = _setup(tmp_path, cfg, seed, sharpen=8.0)
        n = 300
        toks = U.tokens_for(cfg, n, 5)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=20)
        for cuts in ([n], [255, 1, 1, 15, 17, 11], [n - 64] + [1] * 64, [49, 2, 48, 1, 1, 49, 50, 100]):
            got = U.run_cuts(r, "f", toks, cuts)
            assert U.close(got, want, dtype), (kind, cuts[:4], U.rel_err(got, want))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tmp_path, dtype, name="mix_b"):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13)
    n = 140
    toks = U.tokens_for(cfg, n, 8)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, pages=10)
    got = U.run_cuts(r, "l", toks, [3] + [1] * (n - 3))
    assert U.close(got, want, dtype), U.rel_err(got, want)
    assert r.graph_replays > 100                              # single tokens replay a captured step


@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_engine(tmp_path, dtype, name="mix_a"):
    """Greedy generation through Engine (scheduler, portions of 16, three requests at once) gives
    the tokens the plain model picks, wherever its choice is not a near tie."""
    from llm_singularity_b200 import Engine
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 17)
    eng = Engine(path, dtype=dtype, kv_block_size=16, num_kv_blocks=24, max_batch_size=3,
                 max_tokens_per_batch=48, prefill_chunk=16)
    prompts = [U.tokens_for(cfg, n, 40 + n) for n in (5, 37, 18)]
    new = 12
    ids = [eng.add_request(p, max_new_tokens=new) for p in prompts]
    out = {i: [] for i in ids}
    while eng.has_work():
        for rid, tok, _ in eng.step():
            assert tok >= 0
            out[rid].append(tok)
    for rid, p in zip(ids, prompts):
        seq = list(p)
        for tok in out[rid]:
            logits = U.plain_logits(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if (top2[0] - top2[1]) > (0.05 if dtype == "float32" else 0.5):
                assert tok == int(logits.argmax()), (rid, len(seq))
            seq.append(tok)
        assert len(out[rid]) == new


# ----------------------------------------------------------------- kernels against plain functions
def _ctx(q_lens, kv_lens, rows=None):
    from llm_singularity_b200.engine.batch import ContextBuilder
    b = ContextBuilder("cuda", 4096, 64)
    ctx, _ = b.build([[0] * n for n in q_lens], [kv - q for kv, q in zip(kv_lens, q_lens)],
                     rows or list(range(len(q_lens))), [[] for _ in q_lens])
    ctx._keep = b
    return ctx


def _pages(slots, max_kv, nkv, dk, dv, page, dtype, seed=0):
    from llm_singularity_b200.parts import KVCacheView
    per = -(-max_kv // page)
    n = slots * per + 3
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed))[:slots * per].view(slots, per)
    return KVCacheView(torch.zeros(n, nkv, page, dk, dtype=dtype, device="cuda"),
                       torch.zeros(n, nkv, page, dv, dtype=dtype, device="cuda"),
                       perm.to(torch.int32).cuda(), page, None, 0)


def _fill(cache, row, K, V):
    pos = torch.arange(K.shape[0])
    pages = cache.block_table[row].cpu()[pos // cache.page_size].long()
    cache.k_pages[pages, :, pos % cache.page_size, :] = K.to(cache.k_pages.dtype).cuda()
    cache.v_pages[pages, :, pos % cache.page_size, :] = V.to(cache.v_pages.dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh, nkv, dk, dv, chunk, window, page", [(4, 2, 32, 16, 24, 0, 16), (6, 2, 96, 48, 40, 0, 16),
                                                                  (3, 3, 10, 14, 5, 0, 8), (4, 1, 64, 128, 0, 0, 16),
                                                                  (2, 2, 128, 64, 33, 21, 16), (8, 2, 48, 80, 64, 0, 32),
                                                                  (20, 1, 80, 48, 50, 0, 16), (5, 5, 112, 16, 7, 0, 8)])
def test_attention_kernel_one_score_standing_out(dtype, nh, nkv, dk, dv, chunk, window, page):
    """Three requests in one launch (a prompt portion that begins inside a chunk, a single token, a
    longer portion).  All keys are alike but one per request, which every query of that request
    scores high: wherever it is visible the output is its value, wherever it is not the output is
    the mean of the visible values.  The standing-out key is put far back, on a page border, first
    in the sequence, and just inside and just outside the last query's chunk and window."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(dk + dv)
    q_lens, kv_lens = [37, 1, 70], [90, 131, 70]
    ctx = _ctx(q_lens, kv_lens, rows=[2, 0, 1])
    scale = 1.0 / math.sqrt(dk)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    lows = []
    for kv in kv_lens:
        p = kv - 1
        lows.append(max((p // chunk) * chunk if chunk else 0, p - window + 1 if window else 0))
    for targets in ([3, 0, 15], [lo - 1 if lo else 0 for lo in lows], lows, [16, 127, 48], [89, 130, 69]):
        cache = _pages(3, 144, nkv, dk, dv, page, dtype, seed=1)
        qs, outs = [], []
        for r, (ql, kv, tgt) in enumerate(zip(q_lens, kv_lens, targets)):
            Kd = 0.1 * torch.randn(kv, nkv, dk, generator=g)
            Kd[tgt, :, 0] = 6.0
            Vd = torch.randn(kv, nkv, dv, generator=g)
            q = 0.1 * torch.randn(ql, nh, dk, generator=g)
            q[:, :, 0] = 4.0 / scale
            Kd, Vd, q = (t.to(dtype).double() for t in (Kd, Vd, q))
            _fill(cache, [2, 0, 1][r], Kd, Vd)
            pos = torch.arange(kv - ql, kv)
            ok = P.visible(torch.arange(kv), chunk or None)[pos]
            if window:
                ok &= torch.arange(kv)[None, :] > (pos[:, None] - window)
            o = torch.zeros(ql, nh, dv, dtype=torch.float64)
            for h in range(nh):
                s = (q[:, h] @ Kd[:, h // (nh // nkv)].T) * scale
                o[:, h] = torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ Vd[:, h // (nh // nkv)]
            qs.append(q)
            outs.append(o)
        q = torch.cat(qs).reshape(sum(q_lens), nh * dk).to(dtype).cuda()
        gate = torch.randn(sum(q_lens), nh * dv + 6, generator=g).to(dtype).cuda()
        want = torch.cat(outs).reshape(sum(q_lens), nh * dv)
        out = torch.empty(sum(q_lens), nh * dv, dtype=dtype, device="cuda")
        for shape in ((0, 1, 2, 3, 4) if dtype == torch.bfloat16 else (0,)):       # every block shape of the tile kernel
            K.DV_BLOCK_SHAPE = shape
            try:
                out.zero_()
                K.attention_dv(q, nh, nkv, dk, dv, ctx, cache, scale, window, chunk, None, out)
            finally:
                K.DV_BLOCK_SHAPE = 0
            assert (out.double().cpu() - want).abs().max() <= tol * 4, (targets, shape)
        K.attention_dv(q, nh, nkv, dk, dv, ctx, cache, scale, window, chunk, gate[:, 6:], out)
        gated = want * torch.sigmoid(gate[:, 6:].double().cpu())
        assert (out.double().cpu() - gated).abs().max() <= tol * 4, targets
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing", ["adjacent", "half"])
def test_preparation_kernel(dtype, pairing):
    """Biases, head norms, query temperature, rotation of the first dims and the cache write, each
    on and off, against plain arithmetic; positions from two requests that continue mid-sequence."""
    from llm_singularity_b200 import kernels as K
    from llm_singularity_b200.parts.rotary import rotary_inv_freq
    nh, nkv, dk, dv, rot, page = 5, 2, 24, 10, 12, 8
    g = torch.Generator().manual_seed(3)
    q_lens, kv_lens = [9, 1, 4], [40, 33, 4]
    T, ld = sum(q_lens), nh * dk + nkv * dk + nkv * dv + 7
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    for bias, norm, temp, rotate in ((True, False, (0.3, 8), False), (False, True, None, True), (True, True, (0.5, 3), True),
                                     (False, False, None, False)):
        ctx = _ctx(q_lens, kv_lens, rows=[1, 2, 0])
        cache = _pages(3, 48, nkv, dk, dv, page, dtype, seed=2)
        proj = torch.randn(T, ld, generator=g).to(dtype).cuda()
        vec = {n: torch.randn(s, generator=g).cuda() for n, s in (("q_bias", nh * dk), ("k_bias", nkv * dk), ("v_bias", nkv * dv))}
        nrm = {n: (1 + 0.3 * torch.randn(dk, generator=g)).cuda() for n in ("q_norm", "k_norm")}
        inv = rotary_inv_freq(rot, 900.0).float().cuda()
        kw = dict(norm_eps=1e-4)
        if bias:
            kw.update(vec)
        if norm:
            kw.update(nrm)
        if temp:
            kw.update(temp_coef=temp[0], temp_every=temp[1])
        if rotate:
            kw.update(inv_freq=inv, rotary_dim=rot, pairing=pairing)
        q_out = torch.empty(T, nh * dk, dtype=dtype, device="cuda")
        K.attention_prep(proj, 3, 3 + nh * dk, 3 + (nh + nkv) * dk, nh, nkv, dk, dv, ctx, cache, q_out, **kw)
        pos = ctx.positions.cpu()
        x = proj.double().cpu()
        q = x[:, 3:3 + nh * dk].clone()
        k = x[:, 3 + nh * dk:3 + (nh + nkv) * dk].clone()
        v = x[:, 3 + (nh + nkv) * dk:3 + (nh + nkv) * dk + nkv * dv].clone()
        if bias:
            q, k, v = q + vec["q_bias"].double().cpu(), k + vec["k_bias"].double().cpu(), v + vec["v_bias"].double().cpu()
        q, k = q.view(T, nh, dk), k.view(T, nkv, dk)
        if norm:
            q = P.unit_rms(q, 1e-4) * nrm["q_norm"].double().cpu()
            k = P.unit_rms(k, 1e-4) * nrm["k_norm"].double().cpu()
        if temp:
            q = q * (1 + temp[0] * torch.log(torch.div(pos + 1, temp[1], rounding_mode="floor").double() + 1))[:, None, None]
        if rotate:
            if pairing == "adjacent":
                q, k = P.turn_neighbours(q, pos, rot, 900.0), P.turn_neighbours(k, pos, rot, 900.0)
            else:
                ang = pos.double()[:, None] * rotary_inv_freq(rot, 900.0)[None, :]
                c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
                for t in (q, k):
                    a, b = t[..., :rot // 2].clone(), t[..., rot // 2:rot].clone()
                    t[..., :rot // 2], t[..., rot // 2:rot] = a * c - b * s, b * c + a * s
        assert (q_out.double().cpu().view(T, nh, dk) - q).abs().max() <= tol * 8
        t0 = 0
        for r, (ql, kv) in enumerate(zip(q_lens, kv_lens)):
            p = torch.arange(kv - ql, kv)
            pages = cache.block_table[[1, 2, 0][r]].cpu()[p // page].long()
            got_k = cache.k_pages[pages, :, p % page, :].double().cpu()
            got_v = cache.v_pages[pages, :, p % page, :].double().cpu()
            assert (got_k - k[t0:t0 + ql]).abs().max() <= tol * 8
            assert (got_v - v[t0:t0 + ql].view(ql, nkv, dv)).abs().max() <= tol * 8
            t0 += ql
        assert int((cache.k_pages.abs().sum((1, 2, 3)) > 0).sum()) <= 2 + 1 + 1      # no other page touched
    K.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_and_branch_kernels(dtype):
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(1)
    T, H, eps1, eps2, mult = 37, 90, 3e-5, 1e-6, 0.7
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    res = torch.randn(T, H, generator=g).cuda()
    y = torch.randn(T, H, generator=g).to(dtype).cuda()
    w1, w2, step = (torch.randn(H, generator=g).cuda() for _ in range(3))
    want_x = res.double().cpu() + mult * P.unit_rms(y.double().cpu(), eps1) * w1.double().cpu() + step.double().cpu()
    want_h = P.unit_rms(want_x, eps2) * w2.double().cpu()
    rows = torch.tensor([5, 36, 0], dtype=torch.int32, device="cuda")
    picked = torch.empty(3, H, dtype=dtype, device="cuda")
    keep = res.clone()
    K.stream_norm(res, y, w1, eps1, mult, step, rows, w2, eps2, picked)
    assert torch.equal(res, keep) and (picked.double().cpu() - want_h[[5, 36, 0]]).abs().max() <= tol * 4
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    K.stream_norm(res, y, w1, eps1, mult, step, None, w2, eps2, out)
    assert (res.double().cpu() - want_x).abs().max() <= 1e-5 and (out.double().cpu() - want_h).abs().max() <= tol * 4
    res2 = keep.clone()
    K.stream_norm(res2, y, None, 0.0, 2.0, None, None, w2, eps2, out)          # a plain sum, then the norm
    plain = keep.double().cpu() + 2.0 * y.double().cpu()
    assert (res2.double().cpu() - plain).abs().max() <= 1e-5
    assert (out.double().cpu() - P.unit_rms(plain, eps2) * w2.double().cpu()).abs().max() <= tol * 4
    ys = [torch.randn(T, H, generator=g).to(dtype).cuda() for _ in range(3)]
    ws = [torch.randn(H, generator=g).cuda() for _ in range(3)]
    for n in (2, 3):
        K.branch_mean(ys[:n], ws[:n], eps1, out)
        want = sum(P.unit_rms(a.double().cpu(), eps1) * b.double().cpu() for a, b in zip(ys[:n], ws[:n])) / n
        assert (out.double().cpu() - want).abs().max() <= tol * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads, D, V, cap", [(3, 16, 24, 8.0), (2, 64, 32, 15.0), (5, 6, 10, 2.5), (1, 128, 128, 15.0)])
def test_matrix_memory_part_with_carried_state(dtype, heads, D, V, cap):
    """The mixer alone, built from its spec: three requests in changing portions (one of them long
    enough to be walked in segments), slots used again after a request ends, against the plain
    memory walked token by token.  The gate maps are large, so the running maximum moves and the
    floor exp(-m) of the normaliser is the larger term at some places and the smaller at others."""
    from llm_singularity_b200.cache import CacheManager
    from llm_singularity_b200.config.specs import MatrixMemorySpec
    from llm_singularity_b200.engine.batch import ContextBuilder
    from llm_singularity_b200.parts import MIXERS, Runtime
    rt = Runtime("cuda", dtype)
    H, eps = 48, 1e-5
    mem = MIXERS.build(MatrixMemorySpec(hidden_size=H, num_heads=heads, key_dim=D, value_dim=V, gate_cap=cap, eps=eps), rt)
    g = torch.Generator().manual_seed(D)
    W = {}
    for name, ps in type(mem).params(mem.spec).items():
        t = torch.randn(ps.shape, generator=g)
        if len(ps.shape) == 2:
            t = t / math.sqrt(ps.shape[1]) * (4.0 if name in ("i", "f") else 1.0)
        W[name] = t.to(torch.bfloat16).float()
    mem.load({n: t.to(device="cuda", dtype=dtype if t.dim() == 2 else torch.float32) for n, t in W.items()})
    plainW = {"p." + {"i_bias": "i.b", "f_bias": "f.b"}.get(n, n): t.double() for n, t in W.items()}
    m = {"heads": heads, "dim": D, "vdim": V, "gate_cap": cap}
    cache = CacheManager([mem.cache_spec()], 16, 8, 3, 8, rt=rt)
    builder = ContextBuilder("cuda", 4096, 8)
    lens = {"a": 300, "b": 40, "c": 9, "d": 25}
    x = {k: torch.randn(n, H, generator=g).to(torch.bfloat16).double() for k, n in lens.items()}
    want = {k: P.matrix_memory(x[k], plainW, "p.", m, eps)[0] for k in lens}
    plan = [[("a", 270), ("b", 3)], [("b", 1), ("c", 9), ("a", 2)], [("d", 24), ("a", 1), ("b", 36)], [("a", 27), ("d", 1)]]
    at, got = {k: 0 for k in lens}, {k: [] for k in lens}
    for step in plan:
        for k, _ in step:
            if not cache.has(k):
                assert cache.open(k) is not None
        ctx, _ = builder.build([[0] * n for _, n in step], [at[k] for k, _ in step], [cache.slot(k) for k, _ in step],
                               [[] for _ in step])
        rows = torch.cat([x[k][at[k]:at[k] + n] for k, n in step]).to(dtype).cuda()
        y = mem.forward(rows, ctx, cache.view(0, ctx)).double().cpu()
        o = 0
        for k, n in step:
            got[k].append(y[o:o + n])
            o += n
            at[k] += n
            if at[k] == lens[k]:
                cache.close(k)
    assert at == lens
    # 32-bit: every value.  bfloat16: where q is nearly orthogonal to the normaliser and to the memory's
    # columns the rounded projections leave little of the output; nearly all values must be close and
    # the mean error small.
    for k in lens:
        scale = want[k].abs().max().item()
        err = (torch.cat(got[k]) - want[k]).abs()
        if dtype == torch.float32:
            assert err.max() <= 2e-4 * scale, (k, scale)
        else:
            assert (err > 4e-2 * scale).double().mean() <= 0.01 and err.mean() <= 4e-3 * scale, (k, scale, err.mean())
    rt.ops.check_status()


# ------------------------------------------------------------------------ as a user runs it
@pytest.mark.parametrize("dtype", DTYPES)
def test_memory_walked_in_segments_and_gates_in_three_kernels(tmp_path, dtype):
    """With segments of 16 tokens every portion of 32 tokens and more is walked segment by segment
    and chained; the portions of 300 and 255 tokens also take the gates' three-kernel form."""
    from llm_singularity_b200 import kernels as K
    old = K.SCAN_SEGMENT
    K.SCAN_SEGMENT = 16
    try:
        cfg = U.CONFIGS["mix_b"]
        W, path = _setup(tmp_path, cfg, 41)
        n = 300
        toks = U.tokens_for(cfg, n, 6)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, pages=20)
        for cuts in ([n], [255, 33, 12], [40, 260]):
            got = U.run_cuts(r, "g", toks, cuts)
            assert U.close(got, want, dtype), (cuts, U.rel_err(got, want))
    finally:
        K.SCAN_SEGMENT = old


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_user_runs_it(tmp_path, dtype):
    """bin/trace_run as a process of its own, fed step by step: seven requests through four slots
    and a pool smaller than their sum (mixed portions and single tokens), then each request in
    portions of changing size; every position against the plain model."""
    import cuttings
    import numpy as np
    import replay_util
    cfg = U.CONFIGS["mix_a"]
    W, path = _setup(tmp_path, cfg, 23)
    seqs = {f"q{i}": U.tokens_for(cfg, n, 60 + i) for i, n in enumerate((5, 70, 33, 1, 100, 64, 21))}
    want = {rid: U.plain_logits(cfg, W, t) for rid, t in seqs.items()}
    for k, (steps, max_tokens) in enumerate((cuttings.mixed(seqs, seed=3), cuttings.portions(seqs))):
        out = str(tmp_path / f"out{k}")
        replay_util.replay_subprocess(path, dtype, steps, out, max_tokens)
        rows = replay_util.collect(steps, out, cfg["vocab"])
        assert len(rows) == sum(len(t) for t in seqs.values())
        for rid, t in seqs.items():
            got = torch.from_numpy(np.stack([rows[(rid, p)] for p in range(len(t))]))
            assert U.close(got, want[rid], dtype), (k, rid, U.rel_err(got, want[rid]))


def test_command_line_serves_the_design(tmp_path):
    """bin/llm-serve-llama picks the design by config.json and generates greedily what the plain
    model picks (where its choice is clear)."""
    import json
    import os
    import subprocess
    import sys
    cfg = U.CONFIGS["mix_b"]
    W, path = _setup(tmp_path, cfg, 29)
    prompts = [U.tokens_for(cfg, n, 70 + n) for n in (4, 19)]
    (tmp_path / "p.json").write_text(json.dumps(prompts))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "llm-serve-llama"), "--model-dir", path, "--dtype", "fp32",
           "--prompt-ids", str(tmp_path / "p.json"), "--max-new-tokens", "6", "--ignore-eos",
           "--num-kv-blocks", "16", "--max-batch-size", "2"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr
    outs = [json.loads(line)["tokens"] for line in res.stdout.splitlines()]
    assert len(outs) == 2 and all(len(o) == 6 for o in outs)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            logits = U.plain_logits(cfg, W, seq)[-1]
            top2 = torch.topk(logits, 2).values
            if top2[0] - top2[1] > 0.05:
                assert tok == int(logits.argmax())
            seq.append(tok)
