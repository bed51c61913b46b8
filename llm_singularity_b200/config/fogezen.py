"""FogezenConfig: the Fogezen decoder's configuration, read from config.json keys.

A Fogezen model is a list of layers, each with one of two mixers and a dense gated feed-forward
(tanh form of gelu) or none.  ``attention``: softmax attention over all earlier tokens with biased
projections, no rotation, and a query that grows with the logarithm of its position in steps.
``parallel``: two mixers on the same input whose normed results are averaged; ``left`` is chunked
softmax attention with normed and rotated queries and keys and an output gate, ``right`` a matrix
memory with exponential input gate.  Every sublayer has a norm in front and behind
(``x += mult * norm_b(sublayer(norm(x)))``), and the norms' stored weights are distances from one.
A stretch of layers may run several times in a row with the same weights (``loop``), each pass
with caches of its own and a step vector added to the stream at its start.  The embedding is
scaled on the way in and serves unscaled as the output head.  Every size and constant below comes
from config.json; the tensor names are those of the checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .llama import ConfigError
from .specs import (EmbeddingSpec, GatedMLPSpec, HeadSpec, KVAttentionSpec, LayerCall, MatrixMemorySpec, ModelSpec,
                    NoPositionSpec, ParallelMixerSpec, RMSNormSpec, RotarySpec, SandwichBlockSpec)

MIXER_KINDS = ("attention", "parallel")


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d: Mapping[str, Any], key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where} '{key}' must be a positive integer, got {v!r}")
    return v


@dataclass(frozen=True)
class FogezenAttention:
    """Softmax attention as either mixer has it; what a mixer lacks stays at its default."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float = 0.0            # query temperature (``attention``)
    temp_every: int = 0
    chunk: Optional[int] = None       # mask.size (``left``)
    rot_dims: int = 0                 # 0: no rotation
    rot_base: float = 10000.0


@dataclass(frozen=True)
class FogezenMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class FogezenLayer:
    kind: str
    attention: FogezenAttention       # the mixer itself, or the left one of a parallel pair
    memory: Optional[FogezenMemory] = None
    ff: Optional[int] = None          # None: no feed-forward


@dataclass(frozen=True)
class FogezenConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[FogezenLayer, ...]
    loop_start: int = 0               # layers loop_start .. loop_stop - 1 run loop_times times in a row
    loop_stop: int = 0
    loop_times: int = 0               # 0: no loop

    architecture = "Fogezen"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "FogezenConfig":
        norm = _get(d, "norm", "the model")
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = [cls._parse_layer(i, e) for i, e in enumerate(raw_layers)]
        loop = d.get("loop")
        start = stop = times = 0
        if loop:
            start, stop, times = int(_get(loop, "start", "'loop'")), int(_get(loop, "stop", "'loop'")), \
                _pos_int(loop, "times", "'loop'")
        emb = d.get("embedding") or {}
        cfg = cls(vocab=_pos_int(d, "vocab", "the model"), width=_pos_int(d, "width", "the model"),
                  norm_eps=float(_get(norm, "eps", "'norm'")), embedding_scale=float(emb.get("scale", 1.0)),
                  residual_mult=float(d.get("residual_mult", 1.0)), layers=tuple(layers),
                  loop_start=start, loop_stop=stop, loop_times=times)
        cfg.validate()
        return cfg

    @staticmethod
    def _parse_attention(m: Mapping[str, Any], where: str) -> FogezenAttention:
        heads = _pos_int(m, "heads", where)
        kw = dict(heads=heads, kv_heads=_pos_int(m, "kv_heads", where) if m.get("kv_heads") is not None else heads,
                  dim=_pos_int(m, "dim", where), vdim=_pos_int(m, "vdim", where), scale=float(_get(m, "scale", where)))
        temp, mask, rot = m.get("q_temp"), m.get("mask"), m.get("rot")
        if temp:
            kw.update(temp_coef=float(_get(temp, "coef", where + " q_temp")),
                      temp_every=_pos_int(temp, "every", where + " q_temp"))
        if mask:
            kw["chunk"] = _pos_int(mask, "size", where + " mask")
        if rot:
            kw.update(rot_dims=_pos_int(rot, "dims", where + " rot"), rot_base=float(_get(rot, "base", where + " rot")))
        return FogezenAttention(**kw)

    @classmethod
    def _parse_layer(cls, i: int, entry: Mapping[str, Any]) -> FogezenLayer:
        where = f"layer {i}"
        kind = _get(entry, "type", where)
        if kind not in MIXER_KINDS:
            raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(MIXER_KINDS)})")
        m = _get(entry, "mixer", where)
        mlp, ff = entry.get("mlp"), None
        if mlp is not None:
            if mlp.get("kind", "dense") != "dense":
                raise ConfigError(f"config.json: {where} has a feed-forward of kind '{mlp.get('kind')}' (known: dense)")
            ff = _pos_int(mlp, "ff", where + " mlp")
        if kind == "attention":
            return FogezenLayer(kind, cls._parse_attention(m, where), None, ff)
        right = _get(m, "right", where)
        memory = FogezenMemory(heads=_pos_int(right, "heads", where + " right"), dim=_pos_int(right, "dim", where + " right"),
                               vdim=_pos_int(right, "vdim", where + " right"),
                               gate_cap=float(_get(right, "gate_cap", where + " right")))
        return FogezenLayer(kind, cls._parse_attention(_get(m, "left", where), where + " left"), memory, ff)

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        if self.loop_times and not 0 <= self.loop_start < self.loop_stop <= len(self.layers):
            raise ConfigError(f"loop: layers {self.loop_start} .. {self.loop_stop} - 1 of {len(self.layers)}")
        for i, l in enumerate(self.layers):
            a = l.attention
            if a.heads % a.kv_heads:
                raise ConfigError(f"layer {i}: {a.heads} heads cannot share {a.kv_heads} kv heads")
            if a.rot_dims % 2 or a.rot_dims > a.dim:
                raise ConfigError(f"layer {i}: rot.dims {a.rot_dims} must be even and at most dim {a.dim}")
            if a.rot_dims and a.rot_base <= 0:
                raise ConfigError(f"layer {i}: rot.base must be positive")
            if l.memory is not None and l.memory.gate_cap <= 0:
                raise ConfigError(f"layer {i}: gate_cap must be positive")

    # ------------------------------------------------------------------ writing
    @staticmethod
    def _attention_dict(a: FogezenAttention) -> dict:
        m = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
        if a.temp_every:
            m["q_temp"] = {"coef": a.temp_coef, "every": a.temp_every}
        if a.chunk is not None:
            m["mask"] = {"size": a.chunk}
        if a.rot_dims:
            m["rot"] = {"base": a.rot_base, "dims": a.rot_dims}
        return m

    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = self._attention_dict(l.attention)
            if l.kind == "parallel":
                r = l.memory
                m = {"left": m, "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim, "gate_cap": r.gate_cap}}
            layers.append({"type": l.kind, "mixer": m, "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
             "residual_mult": self.residual_mult, "layers": layers}
        if self.loop_times:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d

    # -------------------------------------------------------------- translation
    def run_order(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, number of the pass that begins with this call or None), in the order the layers run."""
        n = len(self.layers)
        if not self.loop_times:
            return [(i, None) for i in range(n)]
        a, b = self.loop_start, self.loop_stop
        order: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(a)]
        for t in range(self.loop_times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]

    def _attention_spec(self, a: FogezenAttention, left: bool) -> KVAttentionSpec:
        position = NoPositionSpec()
        if a.rot_dims:
            position = RotarySpec(head_dim=a.dim, rotary_dim=a.rot_dims, theta=a.rot_base, pairing="adjacent")
        return KVAttentionSpec(hidden_size=self.width, num_heads=a.heads, num_kv_heads=a.kv_heads, key_dim=a.dim,
                               value_dim=a.vdim, scale=a.scale, chunk=a.chunk, qkv_bias=not left, qk_norm=left,
                               eps=self.norm_eps, temp_coef=a.temp_coef, temp_every=a.temp_every, out_gate=left,
                               position=position)

    def _mixer_spec(self, l: FogezenLayer):
        if l.kind == "attention":
            return self._attention_spec(l.attention, left=False)
        r = l.memory
        memory = MatrixMemorySpec(hidden_size=self.width, num_heads=r.heads, key_dim=r.dim, value_dim=r.vdim,
                                  gate_cap=r.gate_cap, out_gate=True, eps=self.norm_eps)
        return ParallelMixerSpec(hidden_size=self.width, branches=(self._attention_spec(l.attention, left=True), memory),
                                 names=("left", "right"), eps=self.norm_eps)

    @staticmethod
    def _mixer_names(l: FogezenLayer, p: str, b: str):
        """(checkpoint name, (owner path, the part's parameter)) of a layer's mixer."""
        if l.kind == "attention":
            pairs = [("q", "q"), ("q.b", "q_bias"), ("k", "k"), ("k.b", "k_bias"), ("v", "v"), ("v.b", "v_bias"), ("o", "o")]
            return [(p + ck, (b, local)) for ck, local in pairs]
        left = [("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q.norm", "q_norm"), ("k.norm", "k_norm")]
        right = [("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("i", "i"),
                 ("i.b", "i_bias"), ("f", "f"), ("f.b", "f_bias")]
        names = [(p + "left." + ck, (b + ".left", local)) for ck, local in left]
        names += [(p + "right." + ck, (b + ".right", local)) for ck, local in right]
        return names + [(p + "left.out", (b, "left_out")), (p + "right.out", (b, "right_out"))]

    def to_model_spec(self) -> ModelSpec:
        W = self.width
        norm = RMSNormSpec(size=W, eps=self.norm_eps, unit_offset=True)
        names = [("embed", ("embedding", "weight")), ("final.norm", ("head.norm", "weight"))]
        if self.loop_times:
            names.append(("loop.step", ("steps", "table")))
        blocks, ignorable = [], []
        for i, l in enumerate(self.layers):
            p, b = f"l{i}.", f"blocks.{i}"
            ffn = None if l.ff is None else GatedMLPSpec(hidden_size=W, intermediate_size=l.ff, activation="gelu_tanh")
            blocks.append(SandwichBlockSpec(mixer=self._mixer_spec(l), ffn=ffn, mixer_norm=norm, mixer_post_norm=norm,
                                            ffn_norm=norm if ffn is not None else None,
                                            ffn_post_norm=norm if ffn is not None else None,
                                            residual_mult=self.residual_mult))
            names += [(p + "norm1", (b + ".mixer_norm", "weight")), (p + "norm1b", (b + ".mixer_post_norm", "weight"))]
            names += self._mixer_names(l, p + "mix.", b + ".mixer")
            if ffn is not None:
                names += [(p + "norm2", (b + ".ffn_norm", "weight")), (p + "norm2b", (b + ".ffn_post_norm", "weight")),
                          (p + "mlp.gate", (b + ".ffn", "gate_proj")), (p + "mlp.up", (b + ".ffn", "up_proj")),
                          (p + "mlp.down", (b + ".ffn", "down_proj"))]
            else:
                ignorable += [p + "norm2", p + "norm2b"]
        # every run of a layer has a cache of its own: a pass through looped layers shares weights only
        order = tuple(LayerCall(block=i, cache=c, step=t) for c, (i, t) in enumerate(self.run_order()))
        return ModelSpec(
            architecture=self.architecture,
            embedding=EmbeddingSpec(vocab_size=self.vocab, hidden_size=W, scale=self.embedding_scale),
            blocks=tuple(blocks), order=order,
            head=HeadSpec(vocab_size=self.vocab, hidden_size=W, tied=True, norm=norm),
            tensor_names=tuple(names), ignorable=tuple(ignorable),
            step_vectors=self.loop_times)
