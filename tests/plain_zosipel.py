"""A plain, slow restatement of the Zosipel design in float64 PyTorch on the CPU: one function per
mechanism, whole sequences, no cache.  It shares no code with the library; the tests compare the
library's kernels, cache and step function with it.

Notation: W weights stored [out, in] and applied as W n; n the input of a sublayer; p a position
counted from 0; d the per-head query/key size, dv the value size, r the rotated width, c the latent.
"""
import json
import math
import os
import struct

import torch

F = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> tensor (float tensors widened to float64, integer tables kept)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, rec in head.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[rec["dtype"]]).reshape(rec["shape"])
        out[name] = t.to(F) if t.is_floating_point() else t
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- mechanisms
def silu(z):
    return z * torch.sigmoid(z)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_norm(x, weight, eps):
    """The stream's norm: its weight is stored around zero."""
    return rms(x, eps) * (1.0 + weight)


def yarn_frequencies(rot):
    """(frequency per pair [r/2], factor on cos and sin) of a rotation with optional YaRN scaling."""
    r, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(r // 2, dtype=F)
    f = base ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn(t):                      # the (fractional) pair that makes t turns over the original length
        return r * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn(float(sc["slow"]))), r - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x: [T, heads, d]; the first r dims of each head turn, pair (i, i + r/2); the rest pass."""
    r = int(rot["dims"])
    f, m = yarn_frequencies(rot)
    a = positions.to(F)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * m)[:, None, :], (torch.sin(a) * m)[:, None, :]
    u, v = x[..., : r // 2], x[..., r // 2: r]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., r:]], dim=-1)


def seen_mask(T, window):
    """[T, T] bool: query i sees key j with 0 <= i - j (< window, if there is one)."""
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = i - j >= 0
    if window:
        seen &= i - j < window
    return seen


def softmax_attention(q, k, v, scale, window=None, softcap=None, sink=None):
    """One head: q [T, d], k [T, d], v [T, dv].  ``softcap``: the scaled score s becomes cap tanh(s / cap);
    ``sink``: a number whose exponential joins the denominator (it has no key and no value)."""
    s = (q @ k.T) * scale
    if softcap:
        s = softcap * torch.tanh(s / softcap)
    s = s.masked_fill(~seen_mask(q.shape[0], window), float("-inf"))
    if sink is None:
        return torch.softmax(s, dim=-1) @ v
    m = torch.maximum(s.max(-1, keepdim=True).values, torch.as_tensor(float(sink), dtype=F))
    e = torch.exp(s - m)
    return (e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))) @ v


def differential_lambda(w, p, diff):
    return float(torch.exp((w[p + ".lq1"] * w[p + ".lk1"]).sum()) - torch.exp((w[p + ".lq2"] * w[p + ".lk2"]).sum()) + diff)


def attention_mixer(w, p, m, n, eps):
    """Differential attention on the sublayer input n [T, width]; p is the tensor prefix '<layer>.mix'."""
    T = n.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (n @ w[p + ".q"].T + w[p + ".q.b"]).reshape(T, H * 2, d)          # head by head: [map 1, map 2]
    k = (n @ w[p + ".k"].T + w[p + ".k.b"]).reshape(T, G * 2, d)
    v = (n @ w[p + ".v"].T + w[p + ".v.b"]).reshape(T, G, dv)
    pos = torch.arange(T)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    window = int(m["mask"]["size"]) if m.get("mask") else None
    diff = float(m["diff"])
    lam = differential_lambda(w, p, diff)
    gate = torch.sigmoid(n @ w[p + ".g"].T)                               # [T, H]
    heads = []
    for h in range(H):
        g = h // (H // G)
        a = [softmax_attention(q[:, 2 * h + j], k[:, 2 * g + j], v[:, g], float(m["scale"]), window, m.get("softcap"))
             for j in (0, 1)]
        o = rms(a[0] - lam * a[1], eps) * (1.0 - diff)
        heads.append(o * gate[:, h:h + 1])
    return torch.cat(heads, dim=-1) @ w[p + ".o"].T


def latent_attention_mixer(w, p, m, n, eps):
    """Attention whose keys and values are projections of one small latent per position; no positions."""
    T = n.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (n @ w[p + ".q"].T).reshape(T, H, d)
    c = rms(n @ w[p + ".dkv"].T, eps) * w[p + ".dkv.norm"]
    k = (c @ w[p + ".uk"].T).reshape(T, H, d)
    v = (c @ w[p + ".uv"].T).reshape(T, H, dv)
    heads = [softmax_attention(q[:, h], k[:, h], v[:, h], float(m["scale"]), sink=w[p + ".sink"][h]) for h in range(H)]
    return torch.cat(heads, dim=-1) @ w[p + ".o"].T


def gated_expert(w, p, n):
    return (silu(n @ w[p + ".gate"].T) * (n @ w[p + ".up"].T)) @ w[p + ".down"].T


def route(scores, top, groups, keep):
    """scores [T, E] -> (experts [T, top], weights [T, top]): the best ``top`` experts among those of
    the ``keep`` groups (of ``groups`` equal groups of neighbours) whose best score is largest."""
    T, E = scores.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    if groups and groups > 1 and keep < groups:
        best = scores.reshape(T, groups, E // groups).max(-1).values
        kept = torch.zeros(T, groups, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = kept[:, :, None].expand(T, groups, E // groups).reshape(T, E)
    picked = scores.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    wts = scores.gather(1, picked)
    return picked, wts / (wts.sum(-1, keepdim=True) + 1e-20)


def choice_margin(z, free, mine, groups):
    """How far the router logits z [E] of one token are from giving ``mine`` instead of ``free``: if
    the two choices lie in different sets of groups, the gap between the best logits of the groups
    that were swapped; else the gap between the logits of the experts that were swapped."""
    E = z.numel()
    gs = E // max(groups, 1)
    ga, gb = {e // gs for e in free}, {e // gs for e in mine}
    if groups > 1 and ga != gb and (ga - gb) and (gb - ga):
        best = z.reshape(groups, gs).max(-1).values
        return float(max(best[g] for g in ga - gb) - min(best[g] for g in gb - ga))
    a, b = set(free), set(mine)
    if not (a - b) or not (b - a):
        return 0.0
    return float(max(z[e] for e in a - b) - min(z[e] for e in b - a))


def moe(w, p, ml, n, forced=None, margins=None):
    """Routed experts plus the gated shared one.  ``forced`` [T, top] replaces the choice of experts
    (the weights still come from this function's scores); ``margins`` (a list) then receives, for
    every token whose forced choice differs from the free one, ``choice_margin`` as a fraction of the
    root mean square of the layer's router logits."""
    r = ml["router"]
    E, top = int(r["experts"]), int(r["top"])
    g = r.get("groups") or {}
    z = n @ w[p + ".router"].T
    scores = torch.softmax(z, dim=-1)
    picked, wts = route(scores, top, int(g.get("count", 1)), int(g.get("keep", 1)))
    if forced is not None:
        mine = torch.as_tensor(forced, dtype=torch.int64)
        if margins is not None:
            scale = float(z.pow(2).mean().sqrt().clamp(min=1e-30))
            for t in range(n.shape[0]):
                a, b = sorted(picked[t].tolist()), sorted(mine[t].tolist())
                if a != b:
                    margins.append(choice_margin(z[t], a, b, int(g.get("count", 1))) / scale)
        picked = mine
        wts = scores.gather(1, picked)
        wts = wts / (wts.sum(-1, keepdim=True) + 1e-20)
    out = torch.zeros_like(n)
    for e in range(E):
        hit = picked == e
        rows = hit.any(-1)
        if rows.any():
            out[rows] += gated_expert(w, f"{p}.e{e}", n[rows]) * (wts * hit).sum(-1, keepdim=True)[rows]
    if ml.get("shared"):
        out = out + gated_expert(w, p + ".shared", n) * torch.sigmoid(n @ w[p + ".shared.sg"].T)
    return out


def layer_order(cfg):
    """[(layer, number of the pass it starts, or None)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(l, None) for l in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(l, None) for l in range(a)]
    for t in range(times):
        order += [(l, t if l == a else None) for l in range(a, b)]
    return order + [(l, None) for l in range(b, n)]


def forward(cfg, w, tokens, layers_out=None, forced=None, margins=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every
    layer run; ``forced`` / ``margins``: the routed layers' choices, one entry per RUN of a layer with
    routed experts, in the order they run (see ``moe``)."""
    eps = float(cfg["norm"]["eps"])
    forced = list(forced) if forced is not None else None
    x = w["embed"][torch.tensor(tokens)]
    for run, (l, starts) in enumerate(layer_order(cfg)):
        L, p = cfg["layers"][l], f"l{l}"
        if starts is not None:
            x = x + w["loop.step"][starts]
        n = offset_norm(x, w[p + ".norm1"], eps)
        if L["type"] == "attention":
            x = x + attention_mixer(w, p + ".mix", L["mixer"], n, eps)
        elif L["type"] == "latent_attention":
            x = x + latent_attention_mixer(w, p + ".mix", L["mixer"], n, eps)
        else:
            raise ValueError(L["type"])
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "moe"
            x = x + moe(w, p + ".mlp", L["mlp"], offset_norm(x, w[p + ".norm2"], eps),
                        forced.pop(0) if forced is not None else None, margins)
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T
