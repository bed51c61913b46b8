"""The Ridotar design in the engine against tests/plain_ridotar.py (float64, whole sequences, one
function per mechanism, no cache).  Every test makes its own small model (tests/ridotar_util.py).

Covered: each mixer alone, with and without the routed feed-forward and the per-token input;
whole prompts against token-by-token stepping; portions of changing size down to two tokens;
batches of unequal requests against each alone; pages and state slots given back and used again;
keys far back, at page borders and among the first tokens under a peaked softmax; long decoding
through many pages; other sizes; greedy generation through the engine's entry point and scheduler.
The same bodies run on the CPU with stand-in kernels in tests/test_ridotar_host.py, which checks
everything but the kernels.
"""
import pytest
import torch

import ridotar_util as U

GPU = dict(device="cuda:0", ops=None)


def _setup(tmp_path, cfg, seed, **kw):
    W = U.make_weights(cfg, seed, **kw)
    return W, U.write_model(str(tmp_path / f"m{seed}"), cfg, W)


# ------------------------------------------------------------------ bodies (device-agnostic)
def body_single_mixers(tmp_path, dtype, device, ops):
    for n, (kind, mlp, side) in enumerate([("lightning", False, False), ("hgrn2", False, True),
                                           ("latent_attention", False, False), ("hgrn2", True, False),
                                           ("latent_attention", True, True)]):
        cfg = U.single(kind, mlp, side)
        W, path = _setup(tmp_path, cfg, 100 + n)
        toks = U.tokens_for(cfg, 45, n)
        want = U.plain_logits(cfg, W, toks)
        r = U.make_runner(path, dtype, device, ops, pages=8)
        whole = U.run_cuts(r, "w", toks, [45])
        assert U.close(whole, want, dtype), (kind, mlp, side, U.rel_err(whole, want))
        stepped = U.run_cuts(r, "s", toks, [1] * 45)             # the same slot and pages once more
        assert U.close(stepped, want, dtype), (kind, mlp, side, "token by token", U.rel_err(stepped, want))


def body_portions(tmp_path, dtype, device, ops, name="mix_a", n=150):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 7)
    toks = U.tokens_for(cfg, n, 3)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, device, ops, pages=12)
    ragged, pattern = [], [2, 15, 1, 16, 17, 31, 2, 2, 33, 5]
    while sum(ragged) < n:
        ragged.append(min(pattern[len(ragged) % len(pattern)], n - sum(ragged)))
    for cuts in ([n], [n - 40] + [1] * 40, ragged, [16] * (n // 16) + [n % 16]):
        cuts = [c for c in cuts if c]
        got = U.run_cuts(r, "p", toks, cuts)
        assert U.close(got, want, dtype), (cuts[:6], U.rel_err(got, want))
    r.cache.check_invariants()


def body_mixed_batches(tmp_path, dtype, device, ops, name="mix_a"):
    """Four requests of unequal length stepped together (portions beside single tokens, a request
    left out of some steps, ends at different times, a fifth request taking over a freed slot and
    freed pages) against the plain model of each alone."""
    from llm_singularity_b200.engine.batch import StepEntry
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 9)
    lens = {"a": 70, "b": 23, "c": 41, "d": 1, "e": 37}
    toks = {k: U.tokens_for(cfg, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    want = {k: U.plain_logits(cfg, W, t) for k, t in toks.items()}
    r = U.make_runner(path, dtype, device, ops, pages=12, slots=4)      # 192 token places for 172 tokens
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


def body_far_keys_and_borders(tmp_path, dtype, device, ops):
    """A strongly peaked softmax over a few hundred keys: a key that is lost, one page or one place
    off, or a first token left out changes the logits by far more than the tolerance."""
    cfg = U.single("latent_attention", mlp=False, side=False)
    W, path = _setup(tmp_path, cfg, 31, sharpen=8.0)
    n = 300
    toks = U.tokens_for(cfg, n, 5)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, device, ops, pages=20)
    for cuts in ([n], [255, 1, 1, 15, 17, 11], [n - 64] + [1] * 64):
        assert U.close(U.run_cuts(r, "f", toks, cuts), want, dtype), cuts[:4]


def body_long_decode(tmp_path, dtype, device, ops, name="mix_b"):
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 13)
    n = 140
    toks = U.tokens_for(cfg, n, 8)
    want = U.plain_logits(cfg, W, toks)
    r = U.make_runner(path, dtype, device, ops, pages=10)
    got = U.run_cuts(r, "l", toks, [3] + [1] * (n - 3))
    assert U.close(got, want, dtype), U.rel_err(got, want)


def body_greedy(tmp_path, dtype, device, ops, name="mix_a"):
    """Greedy generation through Engine (scheduler, portions of 16, three requests at once) gives
    the tokens the plain model picks, wherever its choice is not a near tie."""
    from llm_singularity_b200 import Engine
    cfg = U.CONFIGS[name]
    W, path = _setup(tmp_path, cfg, 17)
    eng = Engine(path, dtype=dtype, device=device, ops=ops, kv_block_size=16, num_kv_blocks=24, max_batch_size=3,
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


# ----------------------------------------------------------------------------------- GPU tests
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_mixer_alone(tmp_path, dtype):
    body_single_mixers(tmp_path, dtype, **GPU)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_portions_of_any_size(tmp_path, dtype, name):
    body_portions(tmp_path, dtype, name=name, **GPU)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix_a", "mix_b", "mix_c"])
def test_mixed_batches_with_slots_and_pages_used_again(tmp_path, dtype, name):
    body_mixed_batches(tmp_path, dtype, name=name, **GPU)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_page_borders_and_first_tokens(tmp_path, dtype):
    body_far_keys_and_borders(tmp_path, dtype, **GPU)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(tmp_path, dtype):
    body_long_decode(tmp_path, dtype, **GPU)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(tmp_path, dtype):
    body_greedy(tmp_path, dtype, **GPU)


# ----------------------------------------------------------------- kernels against plain functions
def _plain_rows(x, w, groups, eps):
    import plain_ridotar as P
    return P.grouped_rms_norm(x.double(), w.double(), groups, eps)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_kernels(dtype):
    import plain_ridotar as P
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(1)
    T, n, groups, eps, alpha = 37, 90, 5, 3e-5, 1.7
    x = torch.randn(T, n, generator=g)
    delta = torch.randn(T, n, generator=g).to(dtype)
    wide = torch.randn(T, n + 14, generator=g).to(dtype)
    gate, bias, w = wide[:, 14:], torch.randn(n, generator=g), 1 + 0.3 * torch.randn(n, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    s = alpha * x.double() + delta.double() * torch.sigmoid(gate.double() + bias.double())
    want = _plain_rows(s, w, groups, eps)
    res, out = x.cuda(), torch.empty(T, n, dtype=dtype, device="cuda")
    K.post_group_norm(res, delta.cuda(), w.cuda(), eps, groups, alpha, out, gate=wide.cuda()[:, 14:], gate_bias=bias.cuda())
    assert (res.cpu().double() - want).abs().max() < 1e-5
    assert (out.cpu().double() - want).abs().max() < tol
    res = x.cuda()
    K.post_group_norm(res, delta.cuda(), w.cuda(), eps, groups, 1.0, out, keep_sum=True)
    assert (res.cpu().double() - (x.double() + delta.double())).abs().max() < 1e-5
    assert (out.cpu().double() - _plain_rows(x.double() + delta.double(), w, groups, eps)).abs().max() < tol
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    some = torch.empty(4, n, dtype=dtype, device="cuda")
    K.gather_group_norm(x.cuda(), rows.cuda(), w.cuda(), eps, groups, some)
    assert (some.cpu().double() - _plain_rows(x[rows.long()], w, groups, eps)).abs().max() < tol
    res = x.cuda()
    K.unit_add(res, delta.cuda(), w.cuda(), eps, out)
    want = x.double() + P.rms_unit(delta.double(), eps) * w.double()
    assert (res.cpu().double() - want).abs().max() < 1e-5 and (out.cpu().double() - want).abs().max() < tol
    w_head = 1 + 0.3 * torch.randn(n // groups, generator=g)
    K.rows_norm_gate(x.cuda(), w_head.cuda(), groups, eps, wide.cuda()[:, 14:], out)
    want = _plain_rows(x, w_head.repeat(groups), groups, eps) * torch.sigmoid(gate.double())
    assert (out.cpu().double() - want).abs().max() < tol


@pytest.mark.gpu
def test_router_picks_the_largest_and_the_lower_index_of_equals():
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(2)
    T, E, top = 50, 37, 5
    z = torch.randn(T, E, generator=g)
    z[3, 10] = z[3, 30] = 9.0                     # a tie at the top: 10 before 30
    z[4] = 0.0                                    # all equal: 0, 1, 2, 3, 4
    for score, renorm in (("sigmoid", False), ("softmax", True)):
        ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
        w = torch.empty(T, top, dtype=torch.float32, device="cuda")
        K.moe_route(z.cuda(), top, score, renorm, ids, w)
        order = torch.sort(-z, dim=-1, stable=True).indices[:, :top]
        assert torch.equal(ids.cpu().long(), order)
        s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, -1)
        want = torch.gather(s, 1, order)
        if renorm:
            want = want / want.sum(-1, keepdim=True)
        assert (w.cpu() - want).abs().max() < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weight_on", ["input", "output"])
@pytest.mark.parametrize("sizes", [(75, 40, 28, 6, 2), (300, 64, 48, 5, 3)])
def test_routed_experts_kernels(dtype, weight_on, sizes):
    """Tokens spread unevenly over experts (one expert gets none, one gets most), more rows than a
    tile for one of them, against a loop over tokens."""
    from llm_singularity_b200 import kernels as K
    import plain_ridotar as P
    g = torch.Generator().manual_seed(4)
    T, H, F, E, top = sizes          # the second set is one the grouped tensor-core product takes in bfloat16
    x = torch.randn(T, H, generator=g).to(dtype)
    wg, wu = (torch.randn(E, F, H, generator=g) / 6).to(dtype), (torch.randn(E, F, H, generator=g) / 6).to(dtype)
    wd = (torch.randn(E, H, F, generator=g) / 5).to(dtype)
    ids = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(T)])      # expert 5 idle
    most = 2 * T // 3                # two thirds of the tokens choose expert 2 first: more rows than a tile
    ids[:most, 0] = 2
    for k in range(1, top):
        ids[:most, k] = torch.where(ids[:most, k] == 2, ids[:most, k].new_tensor(3 if k == 1 else 0), ids[:most, k])
    wts = torch.rand(T, top, generator=g) + 0.2
    want = torch.zeros(T, H, dtype=torch.float64)
    for t in range(T):
        for k in range(top):
            e, s = int(ids[t, k]), wts[t, k].double()
            u = x[t].double() * (s if weight_on == "input" else 1.0)
            y = wd[e].double() @ (P.silu(wg[e].double() @ u) * (wu[e].double() @ u))
            want[t] += y if weight_on == "input" else s * y
    gate_up = torch.stack([wg, wu], dim=2).reshape(E, 2 * F, H).contiguous()
    out = torch.empty(T, H, dtype=dtype, device="cuda")
    K.moe_experts(x.cuda(), ids.to(torch.int32).cuda(), wts.cuda(), gate_up.cuda(), wd.cuda(), "silu", weight_on, out)
    K.check_status()
    scale = want.abs().max()
    assert (out.cpu().double() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2) * scale


@pytest.mark.gpu
@pytest.mark.parametrize("tensor_cores", [False, True])
def test_latent_attention_kernels(tensor_cores):
    """Both attention kernels over a latent cache against a loop: prompt portions whose 64-row tiles
    straddle tokens (five heads), single tokens with the keys split over blocks, a request that
    starts in the middle of a page, pages in scrambled order."""
    from types import SimpleNamespace
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(6)
    H, R, rd, ps = 5, 128, 32, 16
    width = R + rd
    old = K.LATENT_TENSOR_CORES
    K.LATENT_TENSOR_CORES = tensor_cores
    try:
        for q_lens, kv_lens in (([70, 1, 33], [200, 150, 33]), ([1, 1], [333, 17])):
            n_req, T = len(q_lens), sum(q_lens)
            n_pages = sum(-(-n // ps) for n in kv_lens) + 3
            pages = torch.randn(n_pages, ps, width, generator=g).to(torch.bfloat16)
            order = torch.randperm(n_pages, generator=g).tolist()
            table = torch.full((n_req + 2, 32), -1, dtype=torch.int32)
            rows = [2, 0, 3][:n_req]
            for r in range(n_req):
                for i in range(-(-kv_lens[r] // ps)):
                    table[rows[r], i] = order.pop()
            qf = 0.3 * torch.randn(T, H, width, generator=g)
            starts = [0]
            for n in q_lens:
                starts.append(starts[-1] + n)
            ctx = SimpleNamespace(q_start=torch.tensor(starts, dtype=torch.int32).cuda(),
                                  kv_len=torch.tensor(kv_lens, dtype=torch.int32).cuda(),
                                  table_rows=torch.tensor(rows, dtype=torch.int32).cuda(),
                                  n_requests=n_req, n_tokens=T, max_q_len=max(q_lens))
            cache = SimpleNamespace(pages=pages.cuda(), block_table=table.cuda(), page_size=ps)
            out = torch.empty(T, H, R, dtype=torch.bfloat16, device="cuda")
            K.latent_attention(qf.cuda(), ctx, cache, R, rd, 0.11, out)
            K.check_status()
            for r in range(n_req):
                idx = torch.arange(kv_lens[r])
                keys = pages[table[rows[r], idx // ps].long(), idx % ps].double()
                for i in range(q_lens[r]):
                    p = kv_lens[r] - q_lens[r] + i
                    s = (qf[starts[r] + i].double() @ keys[:p + 1].T) * 0.11
                    want = torch.softmax(s, -1) @ keys[:p + 1, :R]
                    got = out[starts[r] + i].cpu().double()
                    assert (got - want).abs().max() < 0.03, (tensor_cores, q_lens, r, i)
    finally:
        K.LATENT_TENSOR_CORES = old


@pytest.mark.gpu
@pytest.mark.parametrize("tensor_cores", [False, True])
def test_per_head_products(tensor_cores):
    """out[m, h] = a[m, h] @ b[h].T with strided views and sizes that fill no tile."""
    from llm_singularity_b200 import kernels as K
    g = torch.Generator().manual_seed(8)
    old = K.LATENT_TENSOR_CORES
    K.LATENT_TENSOR_CORES = tensor_cores
    try:
        for M, H, Kd, N in ((70, 3, 20, 40), (1, 5, 128, 96), (130, 2, 72, 130)):
            wide = torch.randn(M, H, Kd + 12, generator=g)
            b = (torch.randn(H, N, Kd, generator=g) / 4).to(torch.bfloat16)
            want = torch.einsum("mhk,hnk->mhn", wide[:, :, :Kd].double(), b.double())
            for a_dtype, out_dtype in ((torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16)):
                a = wide.to(a_dtype).cuda()[:, :, :Kd]
                out_wide = torch.zeros(M, H, N + 5, dtype=out_dtype, device="cuda")
                K.batched_nt(a, b.cuda(), out_wide[:, :, :N])
                got = out_wide[:, :, :N].cpu().double()
                assert (got - want).abs().max() < 0.06 * want.abs().max(), (M, H, Kd, N, a_dtype)
                assert float(out_wide[:, :, N:].abs().max()) == 0.0
    finally:
        K.LATENT_TENSOR_CORES = old


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix_a", "mix_b"])
def test_recurrences_walked_in_segments(tmp_path, dtype, name):
    """Portions longer than two segments are walked segment by segment, side by side, and chained:
    with segments of 16 tokens every cutting of the portions test goes that way (portions of 150,
    110 and 33 tokens beside shorter ones that are walked whole)."""
    from llm_singularity_b200 import kernels as K
    old = K.SCAN_SEGMENT
    K.SCAN_SEGMENT = 16
    try:
        body_portions(tmp_path, dtype, name=name, **GPU)
        body_mixed_batches(tmp_path, dtype, name=name, **GPU)
    finally:
        K.SCAN_SEGMENT = old


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(tmp_path, dtype):
    """bin/trace_run as a process of its own, fed step by step: seven requests through four slots
    and a pool smaller than their sum (mixed portions and single tokens), then each request in
    portions of changing size; every position against the plain model."""
    import cuttings
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
            got = torch.from_numpy(__import__("numpy").stack([rows[(rid, p)] for p in range(len(t))]))
            assert U.close(got, want[rid], dtype), (k, rid, U.rel_err(got, want[rid]))


@pytest.mark.gpu
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
