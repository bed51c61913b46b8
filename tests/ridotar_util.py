"""Small Ridotar models for the tests: configurations that differ in every size, random weights
made here (not by the engine), and helpers that step the engine and compare with tests/plain_ridotar.py.

The sizes avoid round numbers on purpose (widths that are no multiple of 32, three norm groups,
fewer rotating dims than the rotated part is wide, two or three experts per token, a feed-forward
left out in one layer, a layer reading another layer's latent cache) so that nothing passes by
two sizes being equal or a count being one.
"""
import json
import math
import os

import torch

import plain_ridotar


def _lat(heads, dim, vdim, rot_dim, q_rank, kv_rank, dims, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "rot_dim": rot_dim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": dims}, "scale": 1.0 / math.sqrt(dim + rot_dim)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # all three mixers, a shared latent cache two layers on, one layer without feed-forward
    "mix_a": {
        "architecture": "Ridotar", "vocab": 211, "width": 72, "norm": {"eps": 2e-5, "groups": 3},
        "postln_alpha": 1.5, "token_side": {"dim": 10},
        "layers": [
            _layer("latent_attention", _lat(3, 20, 24, 12, 28, 40, 8, 5000.0), _moe(5, 2, 36)),
            _layer("hgrn2", {"heads": 3, "dim": 20, "vdim": 28}, None),
            _layer("latent_attention", _lat(2, 24, 20, 12, 36, 40, 8, 5000.0, kv_from=0), _moe(7, 3, 24)),
            _layer("lightning", {"heads": 3, "dim": 12, "vdim": 40, "decay": [0.5, 0.93, 0.995]}, _moe(5, 2, 36)),
        ]},
    # one norm group, no per-token input, wider heads, top 1 of 3, sizes that fill whole tiles
    "mix_b": {
        "architecture": "Ridotar", "vocab": 160, "width": 128, "norm": {"eps": 1e-6, "groups": 1},
        "postln_alpha": 1.0,
        "layers": [
            _layer("lightning", {"heads": 2, "dim": 64, "vdim": 32, "decay": [0.9, 0.999]}, _moe(3, 1, 64)),
            _layer("hgrn2", {"heads": 1, "dim": 80, "vdim": 48}, _moe(4, 4, 32)),
            _layer("latent_attention", _lat(4, 32, 32, 16, 48, 64, 16, 10000.0), None),
        ]},
    # nothing a multiple of eight: the products, the cache rows and the scans take their plain paths
    "mix_c": {
        "architecture": "Ridotar", "vocab": 53, "width": 100, "norm": {"eps": 1e-5, "groups": 5},
        "postln_alpha": 0.75, "token_side": {"dim": 7},
        "layers": [
            _layer("hgrn2", {"heads": 3, "dim": 10, "vdim": 14}, _moe(3, 3, 30)),
            _layer("latent_attention", _lat(5, 6, 10, 6, 22, 18, 4, 700.0), _moe(3, 2, 30)),
            _layer("lightning", {"heads": 1, "dim": 26, "vdim": 22, "decay": [0.97]}, None),
            _layer("latent_attention", _lat(2, 14, 6, 6, 10, 18, 4, 700.0, kv_from=1), _moe(4, 1, 18)),
        ]},
}


def single(kind, mlp=False, side=True):
    """A one-layer model of one mixer kind (its feed-forward and side input optional)."""
    mixer = {"lightning": {"heads": 3, "dim": 20, "vdim": 12, "decay": [0.7, 0.97, 0.999]},
             "hgrn2": {"heads": 2, "dim": 36, "vdim": 20},
             "latent_attention": _lat(3, 20, 12, 8, 24, 28, 6, 3000.0)}[kind]
    cfg = {"architecture": "Ridotar", "vocab": 97, "width": 56, "norm": {"eps": 1e-5, "groups": 2},
           "postln_alpha": 2.5, "layers": [_layer(kind, mixer, _moe(6, 2, 20) if mlp else None)]}
    if side:
        cfg["token_side"] = {"dim": 6}
    return cfg


def make_weights(cfg, seed, sharpen=3.0):
    """Random bfloat16-representable weights, name -> float32 tensor.  Query and key maps of the
    attention layers are scaled up so that the softmax is peaked and one wrong or missing key
    shows; floors of forget gates lie in [0, 0.9]; norm weights are near one."""
    from llm_singularity_b200.config.ridotar import RidotarConfig
    from llm_singularity_b200.engine.runner import expected_tensors_of
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, (shape, role, init) in expected_tensors_of(RidotarConfig.from_dict(cfg).to_model_spec()).items():
        if name.endswith("lower"):
            t = 0.9 * torch.rand(shape, generator=g)
        elif init == "ones":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed"):
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith("mix.uq") or name.endswith("mix.uk"):
                t = t * sharpen
            if name.endswith("mlp.router"):
                t = t * 4.0                      # scores away from one another: no close calls
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
    return plain_ridotar.forward(cfg, weights, tokens).float()


def make_runner(path, dtype, device="cuda:0", ops=None, pages=64, slots=4, page_size=16, **kw):
    from llm_singularity_b200.engine.runner import ModelRunner
    return ModelRunner(path, dtype=dtype, device=device, ops=ops, page_size=page_size, num_pages=pages,
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
    """32-bit: every position within the tolerance.  bfloat16: rounding can turn a router's close
    call the other way, which changes that position (and, through a recurrent state, those after
    it) by more than rounding; so at most one position in twenty may be outside, and the median
    must lie far inside.  A fault of the cache, the state or the batch shows in 32-bit, where no
    such allowance is made."""
    e = position_errors(got, want)
    if dtype == "float32":
        return bool(e.max() < TOLERANCE[dtype])
    return bool((e > TOLERANCE[dtype]).float().mean() <= 0.05 and e.median() < TOLERANCE[dtype] / 3)
