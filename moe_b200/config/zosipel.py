"""Typed configuration of the Zosipel design, read from its own config.json keys.

A small decoder whose config.json lists its layers one by one: each entry names its mixer
(``type``: ``attention``, differential attention with a window, a capped score, a rotation with
YaRN scaling and one output gate a head; or ``latent_attention``, attention over one cached latent
per position with a sink in the softmax), the mixer's sizes (``mixer``) and its feed-forward
(``mlp``: routed experts picked within the best groups, plus a gated shared expert; or null for
none).  Layers are pre-norm with RMS norms whose weights are stored around zero (factor 1 + w).  A
stretch of the layers (``loop``: start, stop, times) may run several times in a row with the same
weights; every pass has cache entries of its own and starts by adding row t of the tensor
``loop.step`` to the stream.  Tensors of layer i start with ``l<i>.``.

Every size and every constant that may differ between models comes from config.json; nothing is
derived from one model's values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

from .registry import Architecture, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Zosipel"


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
class RotScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class DiffAttentionMixer:
    heads: int
    kv_heads: int
    dim: int                          # query/key size of one of a head's two maps
    vdim: int                         # per-head value size
    scale: float                      # factor on q . k
    softcap: Optional[float]          # the scaled score s becomes cap * tanh(s / cap)
    diff: float                       # offset of lambda; the joined maps are multiplied by 1 - diff
    window: Optional[int]             # position i sees j with 0 <= i - j < window; None: every earlier one
    rot_dims: int                     # rotated dimensions of each map (0: none)
    rot_base: float
    rot_scaling: Optional[RotScaling]


@dataclass(frozen=True)
class LatentAttentionMixer:
    heads: int
    dim: int
    vdim: int
    kv_rank: int                      # size of the cached latent
    scale: float


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    groups: int                       # equal groups of neighbouring experts (1: none)
    keep: int                         # groups whose experts may be picked
    expert_ff: int
    shared_ff: int                    # 0: no shared expert


@dataclass(frozen=True)
class ZosipelLayer:
    type: str
    mixer: Union[DiffAttentionMixer, LatentAttentionMixer]
    mlp: Optional[MoeMlp]


@dataclass(frozen=True)
class ZosipelLoop:
    start: int
    stop: int
    times: int


def _attention(m, mw) -> DiffAttentionMixer:
    heads, kv = _int(m, "heads", mw), _int(m, "kv_heads", mw)
    if heads % kv:
        _fail(f"{mw}: heads {heads} is not a multiple of kv_heads {kv}")
    dim, vdim = _int(m, "dim", mw), _int(m, "vdim", mw)
    window = None
    if m.get("mask") is not None:
        window = _int(_obj(m, "mask", mw), "size", mw + ".mask")
    rot_dims, rot_base, scaling = 0, 10000.0, None
    if m.get("rot") is not None:
        r = _obj(m, "rot", mw)
        rot_dims, rot_base = _int(r, "dims", mw + ".rot", low=0), _num(r, "base", mw + ".rot")
        if rot_dims % 2 or rot_dims > dim:
            _fail(f"{mw}.rot: dims {rot_dims} must be even and at most dim {dim}")
        if r.get("scaling") is not None:
            sc, sw = _obj(r, "scaling", mw + ".rot"), mw + ".rot.scaling"
            scaling = RotScaling(_num(sc, "factor", sw), _num(sc, "original", sw), _num(sc, "fast", sw),
                                 _num(sc, "slow", sw))
    softcap = _num(m, "softcap", mw) if m.get("softcap") is not None else None
    diff = _num(m, "diff", mw, positive=False)
    return DiffAttentionMixer(heads, kv, dim, vdim, _num(m, "scale", mw, positive=False), softcap, diff, window,
                              rot_dims, rot_base, scaling)


def _latent(m, mw) -> LatentAttentionMixer:
    return LatentAttentionMixer(_int(m, "heads", mw), _int(m, "dim", mw), _int(m, "vdim", mw), _int(m, "kv_rank", mw),
                                _num(m, "scale", mw, positive=False))


def _mlp(ml, where) -> MoeMlp:
    if ml.get("kind") != "moe":
        _fail(f"{where}: unknown kind {ml.get('kind')!r}; known: moe")
    r, rw = _obj(ml, "router", where), where + ".router"
    experts, top = _int(r, "experts", rw), _int(r, "top", rw)
    if top > experts:
        _fail(f"{rw}: top {top} exceeds experts {experts}")
    groups, keep = 1, 1
    if r.get("groups") is not None:
        g = _obj(r, "groups", rw)
        groups, keep = _int(g, "count", rw + ".groups"), _int(g, "keep", rw + ".groups")
        if experts % groups or keep > groups:
            _fail(f"{rw}.groups: count {groups} must divide experts {experts}, and keep {keep} must not exceed it")
        if top > keep * (experts // groups):
            _fail(f"{rw}: the {keep} kept groups hold fewer than top {top} experts")
    shared = 0
    if ml.get("shared") is not None:
        shared = _int(_obj(ml, "shared", where), "ff", where + ".shared")
    return MoeMlp(experts, top, groups, keep, _int(_obj(ml, "expert", where), "ff", where + ".expert"), shared)


@dataclass(frozen=True)
class ZosipelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZosipelLayer, ...]
    loop: Optional[ZosipelLoop]
    raw: Tuple[Tuple[str, Any], ...] = ()      # config.json as it was read, for writing it out again

    @staticmethod
    def from_dict(cfg: Dict[str, Any]) -> "ZosipelConfig":
        vocab, width = _int(cfg, "vocab", "config.json"), _int(cfg, "width", "config.json")
        eps = _num(_obj(cfg, "norm"), "eps", "norm")
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
            if kind == "attention":
                mixer = _attention(m, where + ".mixer")
            elif kind == "latent_attention":
                mixer = _latent(m, where + ".mixer")
            else:
                _fail(f"{where}: unknown mixer type {kind!r}; known: attention, latent_attention")
            mlp = _mlp(_obj(e, "mlp", where), where + ".mlp") if e.get("mlp") is not None else None
            layers.append(ZosipelLayer(kind, mixer, mlp))
        loop = None
        if cfg.get("loop") is not None:
            lp = _obj(cfg, "loop")
            loop = ZosipelLoop(_int(lp, "start", "loop", low=0), _int(lp, "stop", "loop", low=0), _int(lp, "times", "loop"))
            if not loop.start < loop.stop <= len(layers):
                _fail(f"loop: start {loop.start} and stop {loop.stop} must delimit layers of the {len(layers)}")
        return ZosipelConfig(vocab, width, eps, tuple(layers), loop, tuple(cfg.items()))

    def to_dict(self) -> Dict[str, Any]:
        if self.raw:
            return dict(self.raw)

        def mixer(m):
            if isinstance(m, LatentAttentionMixer):
                return {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale}
            d: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim,
                                 "scale": m.scale, "diff": m.diff}
            if m.softcap is not None:
                d["softcap"] = m.softcap
            if m.window is not None:
                d["mask"] = {"size": m.window}
            if m.rot_dims:
                d["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    d["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            return d

        def mlp(f):
            if f is None:
                return None
            d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": f.expert_ff},
                                 "router": {"experts": f.experts, "top": f.top,
                                            "groups": {"count": f.groups, "keep": f.keep}}}
            if f.shared_ff:
                d["shared"] = {"ff": f.shared_ff}
            return d

        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d

    def run_order(self):
        """[(layer, number of the pass it starts, or None)] in the order the layers run: the layers
        before the loop, the looped stretch ``times`` times, the layers after it."""
        n = len(self.layers)
        if self.loop is None:
            return [(l, None) for l in range(n)]
        a, b = self.loop.start, self.loop.stop
        order = [(l, None) for l in range(a)]
        for t in range(self.loop.times):
            order += [(l, t if l == a else None) for l in range(a, b)]
        return order + [(l, None) for l in range(b, n)]


def model_spec(c: ZosipelConfig) -> ModelSpec:
    """Layer by layer into parts; tensor names are the checkpoint's."""
    W = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": c.norm_eps, "offset": 1.0, "names": {"weight": ""}}, name)

    layers = []
    for i, L in enumerate(c.layers):
        p, m = f"l{i}.", L.mixer
        if isinstance(m, DiffAttentionMixer):
            position: Dict[str, Any] = {"kind": "none"}
            if m.rot_dims:
                position = {"kind": "rotary", "theta": m.rot_base, "rotary_dim": m.rot_dims, "partial": m.rot_dims < m.dim}
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    position.update(kind="rotary_yarn", factor=s.factor, original=s.original, fast=s.fast, slow=s.slow)
            mixer = PartSpec(
                "diff_attention",
                {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                 "value_dim": m.vdim, "qkv_bias": True, "window": m.window, "scale": m.scale, "softcap": m.softcap,
                 "diff": m.diff, "eps": c.norm_eps, "out_gate": True, "position": position,
                 "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                           "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2", "gate": "g"}},
                p + "mix.")
        else:
            mixer = PartSpec(
                "latent_attention",
                {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "kv_rank": m.kv_rank,
                 "scale": m.scale, "eps": c.norm_eps, "sink": True,
                 "names": {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "sink": "sink",
                           "o": "o"}},
                p + "mix.")
        if L.mlp is None:
            layers.append(LayerSpec("prenorm", norm(p + "norm1"), mixer, None, None))
            continue
        f = L.mlp
        ffn = PartSpec(
            "routed_experts",
            {"hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.expert_ff,
             "norm_topk_prob": True, "groups": {"count": f.groups, "keep": f.keep},
             "shared_size": f.shared_ff, "shared_gate": bool(f.shared_ff),
             "names": {"router": "router", "expert_gate": "e{e}.gate", "expert_up": "e{e}.up", "expert_down": "e{e}.down",
                       "shared_gate_proj": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down",
                       "shared_gate": "shared.sg"}},
            p + "mlp.")
        layers.append(LayerSpec("prenorm", norm(p + "norm1"), mixer, norm(p + "norm2"), ffn))
    ignorable = tuple(x for i, L in enumerate(c.layers) if L.mlp is None for x in (f"l{i}.norm2", f"l{i}.norm2.*"))
    times = c.loop.times if c.loop is not None else 0
    schedule = tuple(ScheduleEntry(l, run, True, join=starts) for run, (l, starts) in enumerate(c.run_order()))
    joins = tuple(PartSpec("add_row", {"hidden_size": W, "rows": times, "row": t, "names": {"weight": ""}}, "loop.step")
                  for t in range(times))
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=W,
        vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "names": {"weight": ""}}, "embed"),
        layers=tuple(layers),
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False, "names": {"weight": ""}}, "head"),
        ignorable=ignorable,
        joins=joins,
    )


register_architecture(Architecture(ARCHITECTURE, ZosipelConfig.from_dict, model_spec, ZosipelConfig.to_dict))
