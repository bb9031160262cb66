"""Typed configuration of the Divadra design, read from its own config.json keys.

A small decoder whose config.json lists its layers one by one: each entry names its mixer
(``type``: "parallel" or "mamba2"), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: a
dense one with a squared relu, routed experts that a table over token ids picks, or null for none).
The embedding adds a row of a second table chosen by the token and the one before it and is
RMS-normed.  Every layer is "parallel" with two norms: x += mixer(norm1(x)) + ff(norm2(x)), both of
the same x, and what each sublayer reads, h, is first replaced by h + conv(h), a short causal
convolution over time (``canon.taps``).  The "parallel" mixer runs attention (``left``: one RMS norm
over the whole of q and of k, a rotation of pairs (i, i + r/2) of part of each head, values rotated by
their distance to the query, a given score scale, chunks, sigmoid weights with a bias a head) beside
an RWKV-style recurrent mixer (``right``) and returns half the sum of their RMS-normed outputs; the
"mamba2" mixer is a state-space layer with a scalar decay per head.  Tensors of layer i start with
``l<i>.``.

Every size and every constant that may differ between models comes from config.json (or, for the
width of the recurrent mixer's decay projection, from the tensor's shape); nothing is derived from
one model's values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

from .registry import Architecture, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Divadra"


def _fail(msg: str):
    raise ConfigError(f"{ARCHITECTURE}: {msg}")


def _obj(cfg, key, where="config.json") -> Dict[str, Any]:
    v = cfg.get(key)
    if not isinstance(v, dict):
        _fail(f"{where} lacks the object '{key}'")
    return v


def _int(cfg, key, where, low=1) -> int:
    v = cfg.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        _fail(f"{where}: '{key}' must be an integer, got {v!r}")
    if int(v) < low:
        _fail(f"{where}: '{key}' must be at least {low}, got {v}")
    return int(v)


def _num(cfg, key, where, positive=True) -> float:
    v = cfg.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        _fail(f"{where}: '{key}' must be a number, got {v!r}")
    if positive and not float(v) > 0:
        _fail(f"{where}: '{key}' must be positive, got {v}")
    return float(v)


@dataclass(frozen=True)
class LeftAttention:
    heads: int
    kv_heads: int
    dim: int                          # per-head query/key size
    vdim: int                         # per-head value size
    scale: float                      # factor on q . k
    chunk: int                        # position i sees j <= i with i // chunk == j // chunk; 0: every earlier one
    rot_dims: int                     # rotated dimensions of each query/key head (0: none)
    rot_base: float                   # also the base of the values' rotation


@dataclass(frozen=True)
class RightWkv:
    heads: int
    dim: int


@dataclass(frozen=True)
class ParallelMixer:
    left: LeftAttention
    right: RightWkv


@dataclass(frozen=True)
class Mamba2Mixer:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    taps: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class TableMoeMlp:
    experts: int
    top: int
    expert_ff: int


@dataclass(frozen=True)
class DivadraLayer:
    type: str
    mixer: Union[ParallelMixer, Mamba2Mixer]
    mlp: Union[DenseMlp, TableMoeMlp, None]


@dataclass(frozen=True)
class DivadraConfig:
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: Tuple[DivadraLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()      # config.json as it was read, for writing it out again

    @staticmethod
    def from_dict(cfg: Dict[str, Any]) -> "DivadraConfig":
        vocab, width = _int(cfg, "vocab", "config.json"), _int(cfg, "width", "config.json")
        eps = _num(_obj(cfg, "norm"), "eps", "norm")
        taps = _int(_obj(cfg, "canon"), "taps", "canon")
        if taps > 16:
            _fail(f"canon: 'taps' must be at most 16, got {taps}")
        bg = _obj(_obj(cfg, "embedding"), "bigram", "embedding")
        buckets = _int(bg, "buckets", "embedding.bigram")
        mul_prev, mul_cur = _int(bg, "mul_prev", "embedding.bigram", low=0), _int(bg, "mul_cur", "embedding.bigram", low=0)
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            _fail("'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                _fail(f"{where} must be an object")
            kind = e.get("type")
            m = _obj(e, "mixer", where)
            mw = where + ".mixer"
            if kind == "parallel":
                l, lw = _obj(m, "left", mw), mw + ".left"
                heads = _int(l, "heads", lw)
                kv = _int(l, "kv_heads", lw) if l.get("kv_heads") is not None else heads
                if heads % kv:
                    _fail(f"{lw}: heads {heads} is not a multiple of kv_heads {kv}")
                dim = _int(l, "dim", lw)
                vdim = _int(l, "vdim", lw) if l.get("vdim") is not None else dim
                if vdim % 2:
                    _fail(f"{lw}: vdim {vdim} must be even (the values are rotated in pairs)")
                chunk = _int(_obj(l, "mask", lw), "size", lw + ".mask") if l.get("mask") is not None else 0
                rot_dims, rot_base = 0, 10000.0
                if l.get("rot") is not None:
                    r = _obj(l, "rot", lw)
                    rot_dims, rot_base = _int(r, "dims", lw + ".rot", low=0), _num(r, "base", lw + ".rot")
                    if rot_dims % 2 or rot_dims > dim:
                        _fail(f"{lw}.rot: dims {rot_dims} must be even and at most dim {dim}")
                r_, rw = _obj(m, "right", mw), mw + ".right"
                mixer: Union[ParallelMixer, Mamba2Mixer] = ParallelMixer(
                    LeftAttention(heads, kv, dim, vdim, _num(l, "scale", lw, positive=False), chunk, rot_dims, rot_base),
                    RightWkv(_int(r_, "heads", rw), _int(r_, "dim", rw)))
            elif kind == "mamba2":
                heads, groups = _int(m, "heads", mw), _int(m, "groups", mw) if m.get("groups") is not None else 1
                vdim = _int(m, "vdim", mw)
                ng = _int(m, "norm_groups", mw) if m.get("norm_groups") is not None else 1
                if heads % groups:
                    _fail(f"{mw}: heads {heads} is not a multiple of groups {groups}")
                if (heads * vdim) % ng:
                    _fail(f"{mw}: heads x vdim {heads * vdim} is not a multiple of norm_groups {ng}")
                ctaps = _int(m, "conv", mw)
                if ctaps > 16:
                    _fail(f"{mw}: 'conv' must be at most 16, got {ctaps}")
                mixer = Mamba2Mixer(heads, vdim, _int(m, "state", mw), groups, ng, ctaps)
            else:
                _fail(f"{where}: unknown mixer type {kind!r}; known: parallel, mamba2")
            mlp: Union[DenseMlp, TableMoeMlp, None] = None
            if e.get("mlp") is not None:
                ml, lw = _obj(e, "mlp", where), where + ".mlp"
                if ml.get("kind") == "dense":
                    mlp = DenseMlp(_int(ml, "ff", lw))
                elif ml.get("kind") == "moe":
                    rt = _obj(ml, "router", lw)
                    experts, top = _int(rt, "experts", lw + ".router"), _int(rt, "top", lw + ".router")
                    if top > experts:
                        _fail(f"{lw}.router: top {top} exceeds experts {experts}")
                    mlp = TableMoeMlp(experts, top, _int(_obj(ml, "expert", lw), "ff", lw + ".expert"))
                else:
                    _fail(f"{lw}: unknown kind {ml.get('kind')!r}; known: dense, moe")
            layers.append(DivadraLayer(kind, mixer, mlp))
        return DivadraConfig(vocab, width, eps, taps, buckets, mul_prev, mul_cur, tuple(layers), tuple(cfg.items()))

    def to_dict(self) -> Dict[str, Any]:
        if self.raw:
            return dict(self.raw)

        def mixer(m):
            if isinstance(m, Mamba2Mixer):
                return {"heads": m.heads, "vdim": m.vdim, "state": m.state, "groups": m.groups,
                        "norm_groups": m.norm_groups, "conv": m.taps}
            a = m.left
            left: Dict[str, Any] = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.chunk:
                left["mask"] = {"size": a.chunk}
            left["rot"] = {"dims": a.rot_dims, "base": a.rot_base}
            return {"left": left, "right": {"heads": m.right.heads, "dim": m.right.dim}}

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, DenseMlp):
                return {"kind": "dense", "ff": f.ff}
            return {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.expert_ff}}

        return {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "canon": {"taps": self.canon_taps},
            "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
        }


def model_spec(c: DivadraConfig) -> ModelSpec:
    """Layer by layer into parts; tensor names are the checkpoint's."""
    W = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": c.norm_eps, "names": {"weight": ""}}, name)

    def canon(name: str) -> PartSpec:
        return PartSpec("residual_conv", {"size": W, "taps": c.canon_taps, "names": {"weight": ""}}, name)

    layers = []
    for i, L in enumerate(c.layers):
        p, m = f"l{i}.", L.mixer
        if isinstance(m, ParallelMixer):
            a = m.left
            # (the values' rotation takes the position encoding's base, so the encoding is there even
            # where no dimension of q and k is rotated)
            position: Dict[str, Any] = {"kind": "rotary", "theta": a.rot_base, "rotary_dim": a.rot_dims,
                                        "partial": a.rot_dims < a.dim}
            left = {"kind": "gqa_attention", "params": {
                "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
                "value_dim": a.vdim, "window": None, "chunk": a.chunk, "scale": a.scale,
                "qk_norm": {"eps": c.norm_eps, "whole": True}, "rotate_values": True, "sigmoid": True,
                "position": position,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                          "head_bias": "pb"}}}
            right = {"kind": "wkv", "params": {"hidden_size": W, "num_heads": m.right.heads, "head_dim": m.right.dim,
                                               "eps": c.norm_eps}}
            mixer = PartSpec("side_by_side", {"hidden_size": W, "eps": c.norm_eps, "left": left, "right": right},
                             p + "mix.")
        else:
            mixer = PartSpec("ssd", {"hidden_size": W, "num_heads": m.heads, "value_dim": m.vdim, "state_size": m.state,
                                     "groups": m.groups, "norm_groups": m.norm_groups, "taps": m.taps,
                                     "eps": c.norm_eps}, p + "mix.")
        ffn = None
        if isinstance(L.mlp, DenseMlp):
            ffn = PartSpec("dense_mlp", {"hidden_size": W, "size": L.mlp.ff, "activation": "relu2",
                                         "names": {"up": "up", "down": "down"}}, p + "mlp.")
        elif isinstance(L.mlp, TableMoeMlp):
            f = L.mlp
            ffn = PartSpec("routed_experts",
                           {"hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.expert_ff,
                            "router": "table", "vocab_size": c.vocab,
                            "names": {"table": "table", "expert_gate": "e{e}.gate", "expert_up": "e{e}.up",
                                      "expert_down": "e{e}.down"}},
                           p + "mlp.")
        layers.append(LayerSpec("parallel", norm(p + "norm1"), mixer, norm(p + "norm2") if ffn is not None else None, ffn,
                                pre1=canon(p + "canon1"), pre2=canon(p + "canon2") if ffn is not None else None))
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=W,
        vocab_size=c.vocab,
        embedding=PartSpec("pair_embedding", {"vocab_size": c.vocab, "hidden_size": W, "buckets": c.buckets,
                                              "mul_prev": c.mul_prev, "mul_cur": c.mul_cur, "eps": c.norm_eps,
                                              "names": {"weight": "embed", "pair": "bigram", "norm": "embed.norm"}}, ""),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l, l, True) for l in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False, "names": {"weight": ""}}, "head"),
        # a layer without a feed-forward may still carry the norm and the convolution of one
        ignorable=tuple(n for i, L in enumerate(c.layers) if L.mlp is None for n in (f"l{i}.norm2", f"l{i}.canon2")),
    )


register_architecture(Architecture(ARCHITECTURE, DivadraConfig.from_dict, model_spec, DivadraConfig.to_dict))
