"""Small Fogezen models for the tests: configurations that differ in every size, random weights
made here (not by the engine), and helpers that step the engine and compare with tests/plain_fogezen.py.

The sizes are chosen so that nothing passes by two sizes being equal or a count being one: key and
value sizes differ, kv heads are one, several or as many as the heads, fewer dims rotate than a
head has, chunks are shorter than a page in one model and span several pages in another, a layer
has no feed-forward, the loop starts at the first layer in one model and is absent in another.
"""
import json
import math
import os

import torch

import plain_fogezen


def _att(heads, kv, dim, vdim, temp=None, scale=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale or 1.0 / math.sqrt(dim)}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _left(heads, kv, dim, vdim, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": 1.0 / math.sqrt(dim)}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def _right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # the loop begins with the first layer; a layer without feed-forward; key and value sizes differ
    "mix_a": {
        "architecture": "Fogezen", "vocab": 211, "width": 72, "norm": {"eps": 2e-5}, "embedding": {"scale": 7.5},
        "residual_mult": 0.7, "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [
            _layer("parallel", {"left": _left(4, 2, 32, 16, chunk=24, rot=(16, 5000.0)), "right": _right(3, 16, 24, 8.0)}, 40),
            _layer("attention", _att(6, 3, 16, 32, temp=(0.4, 20)), 56),
            _layer("attention", _att(2, 2, 48, 48, temp=(0.25, 7)), None),
        ]},
    # sizes that fill whole tiles: the tensor-core paths in bfloat16 (heads of 64 and 128)
    "mix_b": {
        "architecture": "Fogezen", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
        "residual_mult": 0.5, "loop": {"start": 1, "stop": 3, "times": 3},
        "layers": [
            _layer("attention", _att(4, 1, 64, 64, temp=(0.3, 16)), 128),
            _layer("parallel", {"left": _left(4, 2, 64, 32, chunk=40, rot=(64, 10000.0)), "right": _right(2, 64, 32, 15.0)}, 64),
            _layer("attention", _att(2, 1, 128, 64), 128),
            _layer("parallel", {"left": _left(2, 1, 32, 64, chunk=16, rot=(16, 300.0)), "right": _right(4, 16, 48, 4.0)}, 96),
        ]},
    # nothing a multiple of eight, no loop, chunks shorter than a page, no multipliers
    "mix_c": {
        "architecture": "Fogezen", "vocab": 53, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
        "residual_mult": 1.0,
        "layers": [
            _layer("parallel", {"left": _left(3, 1, 10, 14, chunk=5, rot=(6, 700.0)), "right": _right(5, 6, 10, 20.0)}, 30),
            _layer("attention", _att(5, 5, 12, 6), 18),
            _layer("parallel", {"left": _left(2, 2, 14, 6), "right": _right(1, 26, 22, 2.5)}, None),
        ]},
}


def single(kind, mlp=True, **kw):
    """A one-layer model of one mixer kind."""
    if kind == "attention":
        mixer = _att(kw.get("heads", 6), kw.get("kv", 2), kw.get("dim", 24), kw.get("vdim", 40), temp=kw.get("temp", (0.5, 9)))
    else:
        mixer = {"left": _left(kw.get("heads", 4), kw.get("kv", 2), kw.get("dim", 24), kw.get("vdim", 40),
                               chunk=kw.get("chunk", 50), rot=kw.get("rot", (12, 2000.0))),
                 "right": _right(3, 20, 12, kw.get("cap", 6.0))}
    return {"architecture": "Fogezen", "vocab": 97, "width": 56, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5},
            "residual_mult": 0.8, "layers": [_layer(kind, mixer, 44 if mlp else None)]}


def make_weights(cfg, seed, sharpen=3.0):
    """Random bfloat16-representable weights, name -> float32 tensor.  Query and key maps of the
    attention mixers are scaled up so that the softmax is peaked and one wrong or missing key shows;
    the gate maps of the memory are scaled up so that the gates move, and its forget bias is positive
    so that the memory reaches far back; stored norm weights are near zero where one is added."""
    from llm_singularity_b200.config.fogezen import FogezenConfig
    from llm_singularity_b200.engine.runner import expected_tensors_of
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, role, init) in expected_tensors_of(FogezenConfig.from_dict(cfg).to_model_spec()).items():
        if name == "loop.step":
            t = 0.5 * torch.randn(shape, generator=g)
        elif init == "ones":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = (0.3 if "norm" in name else 0.5) * torch.randn(shape, generator=g)
            if name.endswith("right.f.b"):
                t = t + 3.0
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith((".mix.q", ".mix.k", ".left.q", ".left.k")):
                t = t * sharpen
            if name.endswith((".right.i", ".right.f")):
                t = t * 3.0
        out[name] = t.to(torch.bfloat16).float()
    return out


def write_model(path, cfg, weights, dtype=torch.bfloat16):
    from llm_singularity_b200.weights.safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    write_safetensors(os.path.join(path, "model.safetensors"), {n: t.to(dtype) for n, t in weights.items()})
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    return path


def tokens_for(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def plain_logits(cfg, weights, tokens):
    return plain_fogezen.forward(cfg, weights, tokens).float()


def make_runner(path, dtype, pages=64, slots=4, page_size=16, **kw):
    from llm_singularity_b200.engine.runner import ModelRunner
    return ModelRunner(path, dtype=dtype, device="cuda:0", page_size=page_size, num_pages=pages,
                       max_requests=slots, max_model_len=pages * page_size, **kw)


def run_cuts(runner, rid, tokens, cuts):
    """One request alone, its tokens in portions of the given sizes, every place wanted."""
    from llm_singularity_b200.engine.batch import StepEntry
    assert sum(cuts) == len(tokens)
    assert runner.open(rid)
    at, rows = 0, []
    for c in cuts:
        rows.append(runner.step([StepEntry(rid, tokens[at:at + c], list(range(c)))]).float().cpu().clone())
        at += c
    runner.close(rid)
    runner.check_kernels()
    return torch.cat(rows)


def position_errors(got, want):
    """Per position: rms over the vocabulary of the difference (means taken off), over the rms of
    the wanted logits."""
    d = got.double() - want.double()
    d = d - d.mean(-1, keepdim=True)
    w = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return position_errors(got, want).max().item()


TOLERANCE = {"float32": 2e-4, "bfloat16": 0.08}


def close(got, want, dtype):
    """32-bit: every position within the tolerance.  bfloat16: under a peaked softmax rounding can
    move most of a query's weight from one key to another of nearly the same score, which changes
    that position by more than rounding; so at most one position in twenty may be outside, and the
    median must lie far inside.  A fault of the cache, the state or the batch shows in 32-bit, where
    no such allowance is made."""
    e = position_errors(got, want)
    if dtype == "float32":
        return bool(e.max() < TOLERANCE[dtype])
    return bool((e > TOLERANCE[dtype]).float().mean() <= 0.05 and e.median() < TOLERANCE[dtype] / 3)
