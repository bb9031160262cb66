"""Small Zosipel configurations and weights of the tests' own making.

The weights are drawn here (not by the library's random mode) so that every constant is away from
its neutral value: norm weights (stored around zero), biases, the vectors of lambda, the gates, the
sinks, the vectors added at the start of a pass.  Values are rounded to bfloat16 and stored so, as a
checkpoint is: the float32 engine, the bfloat16 engine and the plain implementation read the same
numbers.
"""
import json
import math
import os

import torch


def attention(heads=4, kv_heads=2, dim=16, vdim=16, window=None, rot=16, base=10000.0, scaling=None, scale=None,
              softcap=None, diff=0.25):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff,
         "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def latent(heads=3, dim=16, vdim=16, rank=24, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank,
                      "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}}


def moe(experts=6, top=2, ff=40, shared=48, groups=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if groups:
        d["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# Sizes differ from layer to layer and from one configuration to the next; where one configuration
# has values that coincide or are 1, another has not.
CONFIGS = {
    # both mixers; a loop in the middle run three times; two key/value heads; value heads larger and
    # smaller than the maps; part of a map and the whole map rotated, with and without YaRN; windows
    # shorter than a page and longer than one (a ring of two pages); experts within two of three groups,
    # within one of two, and without groups; a layer without a feed-forward; one without a shared expert
    "mix": dict(vocab=131, width=64, eps=1e-5, loop=(1, 3, 3), layers=[
        layer(attention(4, 2, 16, 24, window=21, rot=8, base=500.0, scaling=(4.0, 64, 8.0, 1.0), scale=0.3, softcap=8.0, diff=0.2),
              moe(6, 2, 40, 48, groups=(3, 2))),
        layer(latent(3, 24, 16, 40, scale=0.2), moe(8, 3, 32, 0, groups=(2, 1))),
        layer(attention(2, 2, 32, 16, window=70, rot=32, base=10000.0, scale=0.2, softcap=30.0, diff=0.5), None),
        layer(latent(2, 16, 40, 24, scale=0.25), moe(4, 4, 24, 16))]),
    # what may be absent is absent: no loop, no cap, no window, no scaling of the rotation, no groups, no
    # shared expert; as many kv heads as heads; sizes that are no multiples of 16 (and one of 4 only)
    "lean": dict(vocab=97, width=48, eps=1e-6, loop=None, layers=[
        layer(attention(3, 3, 24, 24, window=None, rot=12, base=300.0, scale=0.2, diff=0.1), moe(2, 2, 24, 0)),
        layer(latent(1, 40, 12, 20, scale=0.15), moe(5, 1, 16, 24, groups=(5, 2)))]),
    # ones: one head on one kv head, a window of one position (a token sees itself only) and of exactly a
    # page, a loop run once, one expert of one, a latent of 8, every group kept
    "ones": dict(vocab=64, width=32, eps=1e-5, loop=(0, 2, 1), layers=[
        layer(attention(1, 1, 64, 64, window=64, rot=8, scaling=(2.0, 32, 4.0, 1.0), softcap=5.0, diff=0.3), moe(1, 1, 16, 8)),
        layer(attention(1, 1, 24, 40, window=1, rot=24, diff=0.7), moe(4, 2, 16, 8, groups=(2, 2))),
        layer(latent(1, 8, 8, 8), None)]),
    # peaked attention (a large score scale, no cap), so that one key more or less in sight changes the result
    "sharp": dict(vocab=80, width=64, eps=1e-5, loop=None, layers=[
        layer(attention(4, 2, 32, 32, window=9, rot=16, scale=1.5, diff=0.2), moe(4, 2, 32, 32, groups=(2, 1))),
        layer(attention(4, 1, 32, 32, window=66, rot=32, scale=1.5, diff=0.4), None)]),
    # maps of 64 with values of 128 and latents of 128 and 64 (records the tensor-core kernels take), a
    # wider model, a window of several pages, the whole model looped twice
    "wide": dict(vocab=203, width=128, eps=1e-5, loop=(0, 3, 2), layers=[
        layer(attention(2, 1, 64, 128, window=150, rot=32, base=250.0, scaling=(8.0, 128, 16.0, 2.0), scale=0.09, softcap=15.0, diff=0.35),
              moe(8, 2, 64, 64, groups=(4, 2))),
        layer(latent(4, 32, 48, 128, scale=0.15), moe(4, 2, 48, 0)),
        layer(latent(2, 64, 64, 64, scale=0.125), None)]),
    # one windowed layer with part of a map unrotated: the tests make one key stand out in it, whatever
    # the distance to the query, and move the window's edge
    "edge": dict(vocab=90, width=64, eps=1e-5, loop=None, layers=[
        layer(attention(4, 2, 32, 24, window=67, rot=16, scale=0.5, diff=0.3), moe(3, 1, 24, 16))]),
    # one latent layer, which sees everything: the tests make one far key stand out in it
    "far": dict(vocab=70, width=32, eps=1e-5, loop=None, layers=[
        layer(latent(2, 16, 16, 16, scale=1.0), moe(2, 1, 24, 0))]),
}


def drawn_config(seed):
    """A configuration drawn at random, in the form of ``CONFIGS``' entries: two to six layers of either
    mixer, widths of 64 to 512, maps and heads of 16 to 128 numbers (multiples of 8 only), up to five
    query heads a kv head, latents of 8 to 256, windows of 1 to 257 positions or none, part of a map,
    all of it or nothing rotated, one to 32 experts in one to eight groups, loops of one to four passes
    anywhere in the stack, any of the optional parts absent."""
    import random

    rng = random.Random(seed)
    width = rng.choice([64, 96, 128, 160, 192, 256, 320, 384, 512])
    count = rng.randint(2, 6)
    layers = []
    for _ in range(count):
        if rng.random() < 0.5:
            kv = rng.choice([1, 1, 2, 3, 4])
            heads = kv * rng.choice([1, 2, 3, 4, 5, 8])
            dim = rng.choice([16, 24, 32, 40, 48, 64, 80, 96, 128])
            vdim = rng.choice([dim, 2 * dim, dim // 2, 32, 64, 72])
            rot = rng.choice([dim, dim // 2, dim // 4 * 2, 8, 0]) // 2 * 2
            scaling = None
            if rot and rng.random() < 0.7:
                scaling = (rng.choice([2.0, 4.0, 8.0, 16.0, 40.0]), rng.choice([32, 64, 128, 512, 4096]),
                           rng.choice([32.0, 16.0, 8.0]), rng.choice([1.0, 2.0, 0.5]))
            m = attention(heads, kv, dim, vdim, window=rng.choice([None, 1, 2, 7, 33, 64, 65, 100, 128, 200, 257]), rot=rot,
                          base=rng.choice([100.0, 10000.0, 300000.0, 1e6]), scaling=scaling,
                          scale=rng.choice([None, 0.1, 0.3, 1.7 / math.sqrt(dim)]),
                          softcap=rng.choice([None, 5.0, 30.0, 50.0]), diff=rng.choice([0.0, 0.1, 0.3, 0.8]))
        else:
            m = latent(rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 12, 16]), rng.choice([8, 16, 24, 32, 48, 64, 96, 128]),
                       rng.choice([8, 16, 32, 40, 64, 128]), rng.choice([8, 16, 24, 32, 48, 64, 96, 128, 160, 192, 256]),
                       scale=rng.choice([None, 0.1, 0.25]))
        mlp = None
        if rng.random() < 0.8:
            groups, per = rng.choice([1, 2, 3, 4, 8]), rng.choice([1, 2, 3, 4])
            keep = rng.randint(1, groups)
            grouped = rng.random() < 0.8
            top = rng.randint(1, min(keep * per if grouped else groups * per, 8))
            mlp = moe(groups * per, top, rng.choice([16, 24, 40, 64, 96, 136]), rng.choice([0, 16, 64, 136]),
                      groups=(groups, keep) if grouped else None)
        layers.append(layer(m, mlp))
    loop = None
    if rng.random() < 0.8:
        a = rng.randint(0, count - 1)
        loop = (a, rng.randint(a + 1, count), rng.choice([1, 2, 3, 4]))
    return dict(vocab=rng.choice([50, 257, 600, 1000, 2049]), width=width, eps=rng.choice([1e-5, 1e-6, 1e-3]), loop=loop,
                layers=layers)


def spike_token(w, cfg, token):
    """Change drawn weights of a model whose first layer is latent attention so that every query looks
    at the key of ``token`` wherever it stands: only that token has a component along feature 0,
    which alone feeds the latent's first number, which alone feeds the first key dimension of every
    head; every token has the same component along feature 1, which alone feeds the first query
    dimension of every head."""
    m = cfg["layers"][0]["mixer"]
    w["embed"][:, 0] = 0.0
    w["embed"][token, 0] = 8.0
    w["embed"][:, 1] = 2.0
    if "loop.step" in w:
        w["loop.step"][:, :2] = 0.0
    w["l0.norm1"][:2] = 0.0
    w["l0.mix.dkv"][0, :], w["l0.mix.dkv"][:, 0] = 0.0, 0.0
    w["l0.mix.dkv"][0, 0] = 4.0
    w["l0.mix.dkv.norm"][0] = 1.0
    d = m["dim"]
    for h in range(m["heads"]):
        w["l0.mix.uk"][h * d, :], w["l0.mix.uk"][h * d: (h + 1) * d, 0] = 0.0, 0.0
        w["l0.mix.uk"][h * d, 0] = 4.0
        w["l0.mix.q"][h * d, :] = 0.0
        w["l0.mix.q"][h * d, 1] = 4.0


def spike_attention(w, cfg, token):
    """Change drawn weights of a model whose first layer is differential attention with an unrotated
    last dimension in every map, so that in map 1 of every head every query looks at the key of
    ``token`` while that key is in its window: only that token has a component along feature 0, which
    alone feeds the last dimension of map 1 of every key head; every token has the same component
    along feature 1, which alone feeds the last dimension of map 1 of every query head."""
    m = cfg["layers"][0]["mixer"]
    d = m["dim"]
    assert m.get("rot") is None or m["rot"]["dims"] < d
    w["embed"][:, 0] = 0.0
    w["embed"][token, 0] = 8.0
    w["embed"][:, 1] = 2.0
    if "loop.step" in w:
        w["loop.step"][:, :2] = 0.0
    w["l0.norm1"][:2] = 0.0
    w["l0.mix.k"][:, 0] = 0.0
    w["l0.mix.q"][:, 0] = 0.0
    for g in range(m["kv_heads"]):
        row = g * 2 * d + d - 1
        w["l0.mix.k"][row, :], w["l0.mix.k.b"][row] = 0.0, 0.0
        w["l0.mix.k"][row, 0] = 4.0
    for h in range(m["heads"]):
        row = h * 2 * d + d - 1
        w["l0.mix.q"][row, :], w["l0.mix.q.b"][row] = 0.0, 0.0
        w["l0.mix.q"][row, 1] = 4.0


def config_dict(name):
    c = CONFIGS[name]
    d = {"architecture": "Zosipel", "vocab": c["vocab"], "width": c["width"], "norm": {"eps": c["eps"]},
         "layers": json.loads(json.dumps(c["layers"]))}
    if c["loop"]:
        d["loop"] = dict(zip(("start", "stop", "times"), c["loop"]))
    return d


def draw_weights(cfg, seed):
    """name -> bfloat16 tensor for every tensor of the configuration."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}

    def mat(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(name, n, mean, std):
        out[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def glu(p, ff):
        mat(p + ".gate", ff, W, gain=1.5), mat(p + ".up", ff, W, gain=1.5), mat(p + ".down", W, ff, gain=1.5)

    out["embed"] = torch.randn(cfg["vocab"], W, generator=g).to(torch.bfloat16)
    if cfg.get("loop"):
        out["loop.step"] = (0.5 * torch.randn(cfg["loop"]["times"], W, generator=g)).to(torch.bfloat16)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", W, 0.0, 0.2)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * 2 * d, W), vec(p + "mix.q.b", H * 2 * d, 0.0, 0.3)
            mat(p + "mix.k", G * 2 * d, W), vec(p + "mix.k.b", G * 2 * d, 0.0, 0.3)
            mat(p + "mix.v", G * dv, W, gain=1.5), vec(p + "mix.v.b", G * dv, 0.0, 0.3)
            for r in ("lq1", "lk1", "lq2", "lk2"):
                vec(p + "mix." + r, d, 0.0, 0.6 / d ** 0.25)
            mat(p + "mix.g", H, W, gain=1.5)
            mat(p + "mix.o", W, H * dv, gain=1.5)
        else:
            H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            mat(p + "mix.q", H * d, W)
            mat(p + "mix.dkv", r, W), vec(p + "mix.dkv.norm", r, 1.0, 0.2)
            mat(p + "mix.uk", H * d, r), mat(p + "mix.uv", H * dv, r, gain=1.5)
            vec(p + "mix.sink", H, 0.0, 1.0)
            mat(p + "mix.o", W, H * dv, gain=1.5)
        ml = L["mlp"]
        if ml:
            vec(p + "norm2", W, 0.0, 0.2)
            E = ml["router"]["experts"]
            mat(p + "mlp.router", E, W, gain=2.0)
            for e in range(E):
                glu(p + f"mlp.e{e}", ml["expert"]["ff"])
            if ml.get("shared"):
                glu(p + "mlp.shared", ml["shared"]["ff"])
                mat(p + "mlp.shared.sg", 1, W, gain=1.5)
    vec("final.norm", W, 0.0, 0.2)
    mat("head", cfg["vocab"], W)
    return out


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
        w = draw_weights(cfg, seed)
        if edit_weights is not None:
            edit_weights(w, cfg)
        write_safetensors(os.path.join(d, "model.safetensors"), w)
        _folders[key] = d
    return _folders[key]


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
