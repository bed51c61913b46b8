"""RidotarConfig: the Ridotar decoder's configuration, read from config.json keys.

A Ridotar model is a list of layers, each with one of three mixers (``lightning``: linear
attention with a fixed decay per head; ``hgrn2``: linear attention whose forget gate also sets the
write strength; ``latent_attention``: softmax attention over a cached latent, optionally reading
another layer's cache) and a routed feed-forward or none.  The stream is normed after every sum
(``x <- norm(alpha x + gate * sublayer(x))``, the norm in groups), each layer ends with a narrow
per-token input, and the output head is the embedding table.  Every size and constant below comes
from config.json; the tensor names are those of the checkpoint.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .llama import ConfigError
from .specs import (EmbeddingSpec, GroupRMSNormSpec, HeadSpec, LatentAttentionSpec, LayerCall,
                    LinearRecurrenceSpec, ModelSpec, MoESpec, PostNormBlockSpec, RotarySpec, TokenSideSpec)

MIXER_KINDS = ("lightning", "hgrn2", "latent_attention")


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
class RidotarMoE:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class RidotarLayer:
    kind: str
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...] = ()              # lightning
    rot_dim: int = 0                           # latent attention from here on
    q_rank: int = 0
    kv_rank: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    scale: float = 0.0
    kv_from: Optional[int] = None
    mlp: Optional[RidotarMoE] = None


@dataclass(frozen=True)
class RidotarConfig:
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    alpha: float
    side_dim: int                              # 0: no per-token input
    layers: Tuple[RidotarLayer, ...]

    architecture = "Ridotar"

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RidotarConfig":
        norm = _get(d, "norm", "the model")
        side = d.get("token_side")
        layers = []
        raw_layers = _get(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        for i, entry in enumerate(raw_layers):
            layers.append(cls._parse_layer(i, entry))
        cfg = cls(vocab=_pos_int(d, "vocab", "the model"), width=_pos_int(d, "width", "the model"),
                  norm_eps=float(_get(norm, "eps", "'norm'")), norm_groups=int(norm.get("groups", 1)),
                  alpha=float(d.get("postln_alpha", 1.0)),
                  side_dim=_pos_int(side, "dim", "'token_side'") if side else 0,
                  layers=tuple(layers))
        cfg.validate()
        return cfg

    @staticmethod
    def _parse_layer(i: int, entry: Mapping[str, Any]) -> RidotarLayer:
        where = f"layer {i}"
        kind = _get(entry, "type", where)
        if kind not in MIXER_KINDS:
            raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(MIXER_KINDS)})")
        m = _get(entry, "mixer", where)
        mlp = entry.get("mlp")
        moe = None
        if mlp is not None:
            if mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"config.json: {where} has a feed-forward of kind '{mlp.get('kind')}' (known: moe)")
            router = _get(mlp, "router", where + " mlp")
            moe = RidotarMoE(experts=_pos_int(router, "experts", where + " router"),
                             top=_pos_int(router, "top", where + " router"),
                             ff=_pos_int(_get(mlp, "expert", where + " mlp"), "ff", where + " expert"))
        common = dict(kind=kind, heads=_pos_int(m, "heads", where), dim=_pos_int(m, "dim", where),
                      vdim=_pos_int(m, "vdim", where), mlp=moe)
        if kind == "lightning":
            decay = _get(m, "decay", where)
            decay = tuple(float(x) for x in decay) if isinstance(decay, (list, tuple)) else (float(decay),) * common["heads"]
            return RidotarLayer(decay=decay, **common)
        if kind == "hgrn2":
            return RidotarLayer(**common)
        rot = _get(m, "rot", where)
        kv_from = m.get("kv_from")
        return RidotarLayer(rot_dim=_pos_int(m, "rot_dim", where), q_rank=_pos_int(m, "q_rank", where),
                            kv_rank=_pos_int(m, "kv_rank", where), rot_dims=_pos_int(rot, "dims", where + " rot"),
                            rot_base=float(_get(rot, "base", where + " rot")), scale=float(_get(m, "scale", where)),
                            kv_from=None if kv_from is None else int(kv_from), **common)

    def validate(self) -> None:
        if self.norm_groups <= 0 or self.width % self.norm_groups:
            raise ConfigError(f"norm.groups {self.norm_groups} must divide the width {self.width}")
        if self.norm_eps <= 0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        for i, l in enumerate(self.layers):
            if l.kind == "lightning" and len(l.decay) != l.heads:
                raise ConfigError(f"layer {i}: {len(l.decay)} decays for {l.heads} heads")
            if l.mlp is not None and l.mlp.top > l.mlp.experts:
                raise ConfigError(f"layer {i}: top {l.mlp.top} of {l.mlp.experts} experts")
            if l.kind != "latent_attention":
                continue
            if l.rot_dims % 2 or l.rot_dims > l.rot_dim:
                raise ConfigError(f"layer {i}: rot.dims {l.rot_dims} must be even and at most rot_dim {l.rot_dim}")
            if l.rot_base <= 0:
                raise ConfigError(f"layer {i}: rot.base must be positive")
            if l.kv_from is not None:
                j = l.kv_from
                src = self.layers[j] if 0 <= j < i else None
                if src is None or src.kind != "latent_attention" or src.kv_from is not None:
                    raise ConfigError(f"layer {i}: kv_from {j} must name an earlier latent-attention layer "
                                      f"that has a latent projection of its own")
                if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (l.kv_rank, l.rot_dim, l.rot_dims, l.rot_base):
                    raise ConfigError(f"layer {i}: kv_rank, rot_dim and rotation must equal those of layer {j}")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for l in self.layers:
            m = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim}
            if l.kind == "lightning":
                m["decay"] = list(l.decay)
            elif l.kind == "latent_attention":
                m.update(rot_dim=l.rot_dim, q_rank=l.q_rank, kv_rank=l.kv_rank, scale=l.scale,
                         rot={"base": l.rot_base, "dims": l.rot_dims})
                if l.kv_from is not None:
                    m["kv_from"] = l.kv_from
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            layers.append({"type": l.kind, "mixer": m, "mlp": mlp})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "postln_alpha": self.alpha, "layers": layers}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d

    # -------------------------------------------------------------- translation
    def _mixer_spec(self, l: RidotarLayer):
        W = self.width
        if l.kind == "lightning":
            return LinearRecurrenceSpec(hidden_size=W, num_heads=l.heads, key_dim=l.dim, value_dim=l.vdim,
                                        gate="fixed_decay", decay=l.decay, q_activation="silu",
                                        k_activation="silu", v_activation="silu", out_norm="all",
                                        out_gate=True, eps=self.norm_eps)
        if l.kind == "hgrn2":
            return LinearRecurrenceSpec(hidden_size=W, num_heads=l.heads, key_dim=l.dim, value_dim=l.vdim,
                                        gate="forget", q_activation="silu", v_activation="none",
                                        out_norm="per_head", out_gate=False, eps=self.norm_eps)
        rotary = RotarySpec(head_dim=l.rot_dim, rotary_dim=l.rot_dims, theta=l.rot_base, pairing="adjacent")
        return LatentAttentionSpec(hidden_size=W, num_heads=l.heads, plain_dim=l.dim, rot_dim=l.rot_dim,
                                   value_dim=l.vdim, q_rank=l.q_rank, kv_rank=l.kv_rank, scale=l.scale,
                                   eps=self.norm_eps, reads_only=l.kv_from is not None, position=rotary)

    @staticmethod
    def _mixer_names(l: RidotarLayer):
        """(checkpoint suffix, the part's parameter) of a layer's mixer."""
        if l.kind == "lightning":
            return [("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm")]
        if l.kind == "hgrn2":
            return [("q", "q"), ("f", "f"), ("f.b", "f_bias"), ("lower", "floor"), ("v", "v"),
                    ("o", "o"), ("norm", "norm")]
        names = [("dq", "dq"), ("dq.norm", "dq_norm"), ("uq", "uq"), ("uk", "uk"), ("uv", "uv"), ("o", "o")]
        if l.kv_from is None:
            names += [("dkv", "dkv"), ("dkv.norm", "dkv_norm")]
        return names

    def to_model_spec(self) -> ModelSpec:
        W, L = self.width, len(self.layers)
        norm = GroupRMSNormSpec(size=W, eps=self.norm_eps, groups=self.norm_groups)
        names = [("embed", ("embedding", "weight")), ("final.norm", ("head.norm", "weight"))]
        if self.side_dim:
            names.append(("side.embed", ("embedding", "side_weight")))
        blocks, order, ignorable = [], [], []
        for i, l in enumerate(self.layers):
            p, b = f"l{i}.", f"blocks.{i}"
            ffn = None
            if l.mlp is not None:
                ffn = MoESpec(hidden_size=W, expert_size=l.mlp.ff, num_experts=l.mlp.experts, top=l.mlp.top,
                              activation="silu", score="sigmoid", renormalize=False, weight_on="input")
            side = None
            if self.side_dim:
                side = TokenSideSpec(hidden_size=W, dim=self.side_dim, offset=i * self.side_dim,
                                     activation="gelu_tanh", eps=self.norm_eps)
            blocks.append(PostNormBlockSpec(mixer=self._mixer_spec(l), ffn=ffn, mixer_norm=norm,
                                            ffn_norm=norm if ffn is not None else None, alpha=self.alpha,
                                            gated_residual=True, hidden_size=W, side=side))
            order.append(LayerCall(block=i, cache=i if l.kv_from is None else l.kv_from,
                                   writes_cache=l.kv_from is None))
            names += [(p + "norm1", (b + ".mixer_norm", "weight")), (p + "rg1", (b, "mixer_gate")),
                      (p + "rg1.b", (b, "mixer_gate_bias"))]
            names += [(p + "mix." + ck, (b + ".mixer", local)) for ck, local in self._mixer_names(l)]
            if ffn is not None:
                names += [(p + "norm2", (b + ".ffn_norm", "weight")), (p + "rg2", (b, "ffn_gate")),
                          (p + "rg2.b", (b, "ffn_gate_bias")), (p + "mlp.router", (b + ".ffn", "router"))]
                for e in range(l.mlp.experts):
                    names += [(f"{p}mlp.e{e}.{w}", (b + ".ffn", f"e{e}.{w}")) for w in ("gate", "up", "down")]
            else:
                ignorable += [p + "norm2", p + "rg2", p + "rg2.b"]
            if side is not None:
                names += [(p + "side.gate", (b + ".side", "gate")), (p + "side.proj", (b + ".side", "proj")),
                          (p + "side.norm", (b + ".side", "norm"))]
        return ModelSpec(
            architecture=self.architecture,
            embedding=EmbeddingSpec(vocab_size=self.vocab, hidden_size=W, side_size=L * self.side_dim),
            blocks=tuple(blocks), order=tuple(order),
            head=HeadSpec(vocab_size=self.vocab, hidden_size=W, tied=True, norm=norm),
            tensor_names=tuple(names), ignorable=tuple(ignorable))
