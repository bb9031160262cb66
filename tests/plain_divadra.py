"""A plain, slow restatement of the Divadra design in float64 PyTorch on the CPU: one function per
mechanism, whole sequences, no cache and no state carried between calls.  It shares no code with
the library; the tests compare the library's kernels, cache, state and step function with it.

Notation: W weights stored [out, in] and applied as W n; x the residual stream; n a sublayer's
input; p a position counted from 0; H query heads on G key/value heads; d the per-head query/key
size, dv the value size, r the rotated width, C the size of an attention chunk; in a recurrent
mixer S is a head's state; taps the length of a causal convolution over time.
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


# --------------------------------------------------------------------------- small functions
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def causal_taps(u, taps_w, bias=None):
    """u: [T, channels]; taps_w: [channels, taps].  y_t = sum_j taps_w[:, j] * u_(t - taps + 1 + j),
    rows before the first count as zero; the last column multiplies the token's own row."""
    T, _ = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y if bias is None else y + bias


# --------------------------------------------------------------------------- embedding
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the pair table for every token: (previous * mul_prev + token * mul_cur) mod buckets, and
    row number ``buckets`` (the table's last) for a sequence's first token."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (tokens[t - 1] * mul_prev + tok * mul_cur) % buckets)
    return rows


def embedding(cfg, w, tokens):
    b = cfg["embedding"]["bigram"]
    x = w["embed"][torch.tensor(tokens)]
    x = x + w["bigram"][torch.tensor(bigram_rows(tokens, int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])))]
    return unit_rms(x, float(cfg["norm"]["eps"])) * w["embed.norm"]


# --------------------------------------------------------------------------- the left mixer: attention
def rotate_halves(x, positions, r, base, sign=1.0):
    """x: [T, heads, d]; dims (i, i + r/2), i < r/2, turn by the angle sign * p * base^(-2i/r): the pair
    (a, b) becomes (a cos - b sin, b cos + a sin); dims from r on pass."""
    i = torch.arange(r // 2, dtype=F)
    a = sign * positions.to(F)[:, None] * (base ** (-2.0 * i / r))[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    lo, hi = x[..., :r // 2], x[..., r // 2:r]
    out = x.clone()
    out[..., :r // 2] = lo * cos - hi * sin
    out[..., r // 2:r] = hi * cos + lo * sin
    return out


def chunked_sigmoid_attention(q, k, v, scale, chunk, head_bias):
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv].  Query i sees key j <= i of its own chunk
    (i // chunk == j // chunk; every earlier key without chunks).  The weight of a visible key is
    sigmoid(q . k * scale + head_bias[h]); the weights are not normalised."""
    T, H, _ = q.shape
    _, G, dv = v.shape
    out = torch.zeros(T, H, dv, dtype=F)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if chunk:
        seen = seen & ((i // chunk) == (j // chunk))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale + head_bias[h]
        out[:, h] = torch.sigmoid(s).masked_fill(~seen, 0.0) @ v[:, g]
    return out


def attention_mixer(w, p, m, n, eps):
    """The attention mixer on n [T, width]; p is the tensor prefix '<layer>.mix.left'."""
    T = n.shape[0]
    H, d = int(m["heads"]), int(m["dim"])
    G, dv = int(m.get("kv_heads") or H), int(m.get("vdim") or d)
    pos = torch.arange(T)
    # one RMS norm over the whole projection, all heads at once
    q = (unit_rms(n @ w[p + ".q"].T, eps) * w[p + ".q.norm"]).reshape(T, H, d)
    k = (unit_rms(n @ w[p + ".k"].T, eps) * w[p + ".k.norm"]).reshape(T, G, d)
    v = (n @ w[p + ".v"].T).reshape(T, G, dv)
    base = 10000.0
    if m.get("rot"):
        r, base = int(m["rot"]["dims"]), float(m["rot"]["base"])
        q, k = rotate_halves(q, pos, r, base), rotate_halves(k, pos, r, base)
    # values turn by their own position over the whole head; the summed output turns back by the query's
    v = rotate_halves(v, pos, dv, base)
    chunk = int(m["mask"]["size"]) if m.get("mask") else 0
    ctx = chunked_sigmoid_attention(q, k, v, float(m["scale"]), chunk, w[p + ".pb"])
    ctx = rotate_halves(ctx, pos, dv, base, sign=-1.0)
    return ctx.reshape(T, H * dv) @ w[p + ".o"].T


# --------------------------------------------------------------------------- the right mixer: wkv
def wkv_mixer(w, p, m, n, eps, trace=None):
    """The recurrent mixer on n [T, width].  Every projection reads its own blend of the token's
    input and the previous token's; per head o_t = (S + diag(u) k_t v_t^T)^T r_t and then
    S <- diag(w_t) S + k_t v_t^T."""
    T, _ = n.shape
    H, d = int(m["heads"]), int(m["dim"])
    prev = torch.cat([torch.zeros(1, n.shape[1], dtype=F), n[:-1]], dim=0)

    def blend(s):
        return n + (prev - n) * w[p + ".mu." + s]

    r = (blend("r") @ w[p + ".r"].T).reshape(T, H, d)
    k = (blend("k") @ w[p + ".k"].T).reshape(T, H, d)
    v = (blend("v") @ w[p + ".v"].T).reshape(T, H, d)
    gate = silu(blend("g") @ w[p + ".g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(blend("w") @ w[p + ".w1"].T) @ w[p + ".w2"].T + w[p + ".w0"])).reshape(T, H, d)
    u = w[p + ".u"]
    out = torch.zeros(T, H, d, dtype=F)
    S = torch.zeros(H, d, d, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    if trace is not None:
        trace.append(S.clone())
    out = unit_rms(out, eps).reshape(T, H * d) * w[p + ".norm"] * gate
    return out @ w[p + ".o"].T


def side_by_side_mixer(w, p, m, n, eps):
    """Attention (left) and the recurrent mixer (right) read the same input; each output passes an
    RMS norm over the model's width with a weight of its own, and the result is half their sum."""
    a = unit_rms(attention_mixer(w, p + ".left", m["left"], n, eps), eps) * w[p + ".left.out"]
    b = unit_rms(wkv_mixer(w, p + ".right", m["right"], n, eps), eps) * w[p + ".right.out"]
    return 0.5 * (a + b)


# --------------------------------------------------------------------------- the state-space mixer
def ssd_mixer(w, p, m, n, eps, trace=None):
    """Mamba-2 on n [T, width].  The input projection's rows are [z | x | B | C | dt]; x, B and C pass
    a causal convolution with bias and silu; per head h (group g = h // (heads / groups)), with
    dt = softplus(dt + dt_bias): S <- exp(-exp(A_log_h) dt) S + dt B x^T (S: [N, dv]),
    y = S^T C + D_h x; then y * silu(z), an RMS norm in ``norm_groups`` equal parts, W_o."""
    T, _ = n.shape
    H, dv, N, G, NG = int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["norm_groups"])
    inner = H * dv
    proj = n @ w[p + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_taps(xbc, w[p + ".conv"], w[p + ".conv.b"]))
    xs = xbc[:, :inner].reshape(T, H, dv)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + ".dt_bias"])                       # [T, H]
    decay = torch.exp(-torch.exp(w[p + ".A_log"]) * dt)         # [T, H]
    y = torch.zeros(T, H, dv, dtype=F)
    S = torch.zeros(H, N, dv, dtype=F)
    grp = torch.arange(H) // (H // G)
    for t in range(T):
        Bt, Ct = B[t][grp], C[t][grp]                           # [H, N]
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bt[:, :, None] * xs[t][:, None, :]
        y[t] = torch.einsum("hn,hnv->hv", Ct, S) + w[p + ".D"][:, None] * xs[t]
    if trace is not None:
        trace.append(S.clone())
    y = y.reshape(T, inner) * silu(z)
    y = unit_rms(y.reshape(T, NG, inner // NG), eps).reshape(T, inner) * w[p + ".norm"]
    return y @ w[p + ".o"].T


# --------------------------------------------------------------------------- feed-forwards
def squared_relu_ff(w, p, n):
    return torch.relu(n @ w[p + ".up"].T) ** 2 @ w[p + ".down"].T


def silu_glu(w, p, n):
    return (silu(n @ w[p + ".gate"].T) * (n @ w[p + ".up"].T)) @ w[p + ".down"].T


def table_experts(w, p, mlp, n, tokens):
    """Every token takes the experts that row ``token id`` of the table names, each with weight 1 / top."""
    top = int(mlp["router"]["top"])
    table = w[p + ".table"]
    out = torch.zeros_like(n)
    for t, tok in enumerate(tokens):
        for e in table[tok].tolist()[:top]:
            out[t] += silu_glu(w, f"{p}.e{int(e)}", n[t:t + 1])[0] / top
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after
    every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embedding(cfg, w, tokens)
    for l, L in enumerate(cfg["layers"]):
        p = f"l{l}"
        n1 = unit_rms(x, eps) * w[p + ".norm1"]
        n1 = n1 + causal_taps(n1, w[p + ".canon1"])
        if L["type"] == "parallel":
            delta = side_by_side_mixer(w, p + ".mix", L["mixer"], n1, eps)
        elif L["type"] == "mamba2":
            delta = ssd_mixer(w, p + ".mix", L["mixer"], n1, eps)
        else:
            raise ValueError(L["type"])
        mlp = L.get("mlp")
        if mlp:
            n2 = unit_rms(x, eps) * w[p + ".norm2"]
            n2 = n2 + causal_taps(n2, w[p + ".canon2"])
            if mlp["kind"] == "dense":
                delta = delta + squared_relu_ff(w, p + ".mlp", n2)
            elif mlp["kind"] == "moe":
                delta = delta + table_experts(w, p + ".mlp", mlp, n2, tokens)
            else:
                raise ValueError(mlp["kind"])
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.clone())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
