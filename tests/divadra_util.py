"""Small Divadra configurations and weights of the tests' own making.

The weights are drawn here (not by the library's random mode) so that every constant is away from
its neutral value: norm weights, the convolutions' taps, the heads' score biases, the recurrent
mixers' blends, decays, step sizes and skips, the pair table.  Values are rounded to bfloat16 and
stored so, as a checkpoint is: the float32 engine, the bfloat16 engine and the plain implementation
read the same numbers.  Integer tables are stored as int32.
"""
import json
import math
import os

import torch


def left(heads=4, kv_heads=2, dim=32, vdim=32, chunk=None, rot=16, base=10000.0, scale=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if kv_heads is not None:
        m["kv_heads"] = kv_heads
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = {"dims": rot, "base": base}
    return m


def parallel(l, heads=2, dim=32):
    return {"type": "parallel", "mixer": {"left": l, "right": {"heads": heads, "dim": dim}}}


def mamba2(heads=4, vdim=16, state=24, groups=2, norm_groups=2, conv=4):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def dense(ff=96):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# Sizes differ from layer to layer and from one configuration to the next; where one configuration
# has values that coincide or are 1, another has not.
CONFIGS = {
    # both mixers and all three kinds of feed-forward; value heads smaller and larger than key heads;
    # chunks shorter than a page and longer than one (a ring of two pages); part of the head and the
    # whole head rotated; two of six experts and one of five; a layer without a feed-forward
    "mix": dict(vocab=131, width=64, eps=1e-5, taps=3, buckets=61, mul_prev=7, mul_cur=13, rank=5, layers=[
        layer(parallel(left(4, 2, 32, 16, chunk=24, rot=16, base=500.0, scale=0.25), 2, 32), dense(96)),
        layer(mamba2(4, 16, 24, 2, 2, 4), moe(6, 2, 40)),
        layer(parallel(left(2, 2, 16, 48, chunk=70, rot=16, scale=0.3), 4, 16), moe(5, 1, 32)),
        layer(mamba2(2, 32, 16, 1, 1, 2), None)]),
    # what may be absent is absent: no chunks, no rotated part of q and k, kv heads not named; heads of 24
    # and 40 (no multiples of 16); one recurrent head; every expert chosen (2 of 2); taps of 2
    "lean": dict(vocab=97, width=48, eps=1e-6, taps=2, buckets=17, mul_prev=3, mul_cur=5, rank=3, layers=[
        layer(parallel(left(3, None, 24, 24, chunk=None, rot=None, scale=0.2), 1, 40), dense(64)),
        layer(mamba2(3, 8, 40, 3, 3, 3), moe(2, 2, 24))]),
    # ones: one head on one kv head, a chunk of one position (a token sees itself only) and of exactly a
    # page, convolutions of one tap (a factor per channel), one bucket, one expert of one, one group
    "ones": dict(vocab=64, width=32, eps=1e-5, taps=1, buckets=1, mul_prev=1, mul_cur=1, rank=1, layers=[
        layer(parallel(left(1, 1, 64, 64, chunk=64, rot=8), 1, 8), moe(1, 1, 16)),
        layer(parallel(left(1, 1, 24, 40, chunk=1, rot=24), 3, 8), dense(48)),
        layer(mamba2(1, 32, 8, 1, 1, 1), dense(40))]),
    # peaked weights (a large score scale), so that one key more or less in sight changes the result
    "sharp": dict(vocab=80, width=64, eps=1e-5, taps=4, buckets=53, mul_prev=11, mul_cur=29, rank=4, layers=[
        layer(parallel(left(4, 2, 32, 32, chunk=9, rot=16, scale=1.5), 2, 16), dense(64)),
        layer(parallel(left(4, 1, 32, 32, chunk=130, rot=32, scale=1.5), 2, 32), dense(64))]),
    # heads of 128 and 64 (records the tensor-core kernels take), a wider model, chunks of several pages,
    # a state of 64 by 64
    "wide": dict(vocab=203, width=128, eps=1e-5, taps=4, buckets=211, mul_prev=41, mul_cur=37, rank=8, layers=[
        layer(parallel(left(2, 1, 128, 64, chunk=150, rot=64, base=250.0, scale=0.09), 2, 64), moe(4, 2, 64)),
        layer(mamba2(2, 64, 64, 1, 2, 4), dense(160)),
        layer(parallel(left(4, 4, 64, 64, chunk=None, rot=32, scale=0.125), 1, 64), None)]),
    # one layer that sees everything, without a rotated part: the tests make one far key stand out in it
    "far": dict(vocab=70, width=32, eps=1e-5, taps=2, buckets=19, mul_prev=2, mul_cur=3, rank=2, layers=[
        layer(parallel(left(2, 1, 16, 16, chunk=None, rot=None, scale=1.0), 1, 16), dense(48))]),
}


def config_dict(name):
    c = CONFIGS[name]
    return {"architecture": "Divadra", "vocab": c["vocab"], "width": c["width"], "norm": {"eps": c["eps"]},
            "canon": {"taps": c["taps"]},
            "embedding": {"bigram": {"buckets": c["buckets"], "mul_prev": c["mul_prev"], "mul_cur": c["mul_cur"]}},
            "layers": json.loads(json.dumps(c["layers"]))}


def draw_weights(cfg, seed, rank=4):
    """name -> tensor (bfloat16; integer tables int32) for every tensor of the configuration."""
    g = torch.Generator().manual_seed(seed)
    W, taps = cfg["width"], cfg["canon"]["taps"]
    out = {}

    def mat(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(name, n, mean, std):
        out[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    out["bigram"] = (0.7 * torch.randn(cfg["embedding"]["bigram"]["buckets"] + 1, W, generator=g)).to(torch.bfloat16)
    vec("embed.norm", W, 1.0, 0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", W, 1.0, 0.2)
        out[p + "canon1"] = (0.3 * torch.randn(W, taps, generator=g)).to(torch.bfloat16)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            H, G, d, dv = a["heads"], a.get("kv_heads") or a["heads"], a["dim"], a["vdim"]
            mat(p + "mix.left.q", H * d, W), mat(p + "mix.left.k", G * d, W), mat(p + "mix.left.v", G * dv, W, gain=1.5)
            vec(p + "mix.left.q.norm", H * d, 1.0, 0.2), vec(p + "mix.left.k.norm", G * d, 1.0, 0.2)
            vec(p + "mix.left.pb", H, -1.5, 0.7)
            mat(p + "mix.left.o", W, H * dv, gain=1.5)
            H, d = r["heads"], r["dim"]
            for s in "rkvgw":
                out[p + "mix.right.mu." + s] = torch.rand(W, generator=g).to(torch.bfloat16)
            for s in "rkvg":
                mat(p + "mix.right." + s, H * d, W, gain=1.3)
            mat(p + "mix.right.w1", rank, W, gain=1.5), mat(p + "mix.right.w2", H * d, rank, gain=1.5)
            vec(p + "mix.right.w0", H * d, -1.0, 0.8)
            out[p + "mix.right.u"] = (0.5 * torch.randn(H, d, generator=g)).to(torch.bfloat16)
            vec(p + "mix.right.norm", H * d, 1.0, 0.2)
            mat(p + "mix.right.o", W, H * d, gain=1.5)
            vec(p + "mix.left.out", W, 1.0, 0.2), vec(p + "mix.right.out", W, 0.8, 0.2)
        else:
            H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * dv, H * dv + 2 * G * N
            mat(p + "mix.in", 2 * inner + 2 * G * N + H, W, gain=1.3)
            out[p + "mix.conv"] = (0.4 * torch.randn(ch, m["conv"], generator=g) + 0.3).to(torch.bfloat16)
            vec(p + "mix.conv.b", ch, 0.0, 0.2)
            vec(p + "mix.dt_bias", H, -0.5, 0.8), vec(p + "mix.A_log", H, -0.5, 0.6), vec(p + "mix.D", H, 0.8, 0.3)
            vec(p + "mix.norm", inner, 1.0, 0.2)
            mat(p + "mix.o", W, inner, gain=1.5)
        ml = L["mlp"]
        if ml:
            vec(p + "norm2", W, 1.0, 0.2)
            out[p + "canon2"] = (0.3 * torch.randn(W, taps, generator=g)).to(torch.bfloat16)
            if ml["kind"] == "dense":
                mat(p + "mlp.up", ml["ff"], W, gain=1.5), mat(p + "mlp.down", W, ml["ff"], gain=1.5)
            else:
                E, top = ml["router"]["experts"], ml["router"]["top"]
                for e in range(E):
                    q = p + f"mlp.e{e}"
                    mat(q + ".gate", ml["expert"]["ff"], W, gain=1.5), mat(q + ".up", ml["expert"]["ff"], W, gain=1.5)
                    mat(q + ".down", W, ml["expert"]["ff"], gain=1.5)
                order = torch.rand(cfg["vocab"], E, generator=g).argsort(dim=1)
                out[p + "mlp.table"] = order[:, :top].to(torch.int32).contiguous()
    vec("final.norm", W, 1.0, 0.2)
    mat("head", cfg["vocab"], W)
    return out


def spike_token(w, cfg, token=0):
    """Change drawn weights of a model whose first layer's attention has no rotated part so that every
    query looks at the key of ``token`` wherever it stands, and at nothing else to speak of: only that
    token has a component along feature 0 (in both tables of the embedding, and no convolution mixes
    it into its neighbours), which alone feeds channel 0 of every key head; feature 1 is the same
    positive number for every token and alone feeds channel 0 of every query head; and every head's
    bias is so low that an ordinary key weighs next to nothing.  After the norms over the whole
    projections the score of that key is in the hundreds."""
    for t in ("embed", "bigram"):
        w[t][:, 0] = 0.0
        w[t][:, 1] = 0.0
    w["embed"][token, 0] = 6.0
    w["embed"][:, 1] = 5.0
    for n in ("embed.norm", "l0.norm1"):
        w[n][0] = 1.0
        w[n][1] = 1.0
    w["l0.canon1"][0, :] = 0.0
    a = cfg["layers"][0]["mixer"]["left"]
    d = a["dim"]
    w["l0.mix.left.k"][::d, :] = 0.0
    w["l0.mix.left.k"][:, 0] = 0.0
    w["l0.mix.left.k"][::d, 0] = 30.0
    w["l0.mix.left.q"][::d, :] = 0.0
    w["l0.mix.left.q"][::d, 1] = 30.0
    w["l0.mix.left.q.norm"][::d] = 4.0
    w["l0.mix.left.k.norm"][::d] = 4.0
    w["l0.mix.left.pb"][:] = -9.0


_folders = {}


def model_folder(root, name, seed=11, edit=None, edit_weights=None):
    """Write (once) config.json and model.safetensors of configuration ``name``; ``edit(cfg)`` may
    change the configuration dict first and ``edit_weights(weights, cfg)`` the drawn weights (their
    ``__name__`` tells the folders apart)."""
    from moe_b200.weights.safetensors_io import write_safetensors

    key = (str(root), name, seed, getattr(edit, "__name__", None), getattr(edit_weights, "__name__", None))
    if key not in _folders:
        cfg = config_dict(name)
        if edit is not None:
            edit(cfg)
        d = os.path.join(str(root), "_".join(str(k) for k in key[1:]))
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        w = draw_weights(cfg, seed, CONFIGS[name]["rank"])
        if edit_weights is not None:
            edit_weights(w, cfg)
        write_safetensors(os.path.join(d, "model.safetensors"), w)
        _folders[key] = d
    return _folders[key]


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
