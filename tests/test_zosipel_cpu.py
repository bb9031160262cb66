"""Zosipel without a GPU: the configuration reader, the translation into parts, the tensor names
and shapes against the tests' own checkpoints, the order in which looped layers run, and the plain
implementation's own consistency (latent attention by its definition against the form that attends
over the latents alone; the choice of experts within groups against an exhaustive search)."""
import itertools
import json

import pytest
import torch

import plain_zosipel as plain
import zosipel_util as U

F = torch.float64


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("zosipel_cpu")


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_config_parts_and_tensor_names_fit_the_checkpoint(root, name):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore

    d = U.model_folder(root, name)
    arch, typed = parse_config(read_config_json(d))
    assert arch.name == "Zosipel"
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    store.check({n: ts.shape for n, ts in expected_tensors(spec, store).items()}, spec.ignorable)
    assert [l.block for l in spec.layers] == ["prenorm"] * len(typed.layers)
    assert typed.to_dict() == json.load(open(d + "/config.json"))
    for L, ls in zip(typed.layers, spec.layers):
        assert ls.mixer.kind == {"attention": "diff_attention", "latent_attention": "latent_attention"}[L.type]
        assert (ls.ffn is None) == (L.mlp is None) == (ls.norm2 is None)
        assert ls.norm1.params["offset"] == 1.0


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random_are_read_and_fit_their_checkpoints(root, seed):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore

    name = f"drawn{seed}"
    U.CONFIGS[name] = U.drawn_config(seed)
    d = U.model_folder(root, name)
    arch, typed = parse_config(read_config_json(d))
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    store.check({n: ts.shape for n, ts in expected_tensors(spec, store).items()}, spec.ignorable)
    assert typed.to_dict() == json.load(open(d + "/config.json"))
    loop = U.CONFIGS[name]["loop"]
    runs = len(typed.layers) + ((loop[1] - loop[0]) * (loop[2] - 1) if loop else 0)
    assert len(plain.layer_order(json.load(open(d + "/config.json")))) == runs == len(spec.schedule)


def test_a_config_written_from_the_typed_form_reads_back_the_same():
    from moe_b200.config.zosipel import ZosipelConfig

    for name in U.CONFIGS:
        typed = ZosipelConfig.from_dict(U.config_dict(name))
        again = ZosipelConfig.from_dict(ZosipelConfig(typed.vocab, typed.width, typed.norm_eps, typed.layers, typed.loop).to_dict())
        assert again.layers == typed.layers and again.vocab == typed.vocab and again.loop == typed.loop


@pytest.mark.parametrize("bad,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "fewer than top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "must divide"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_config_errors_say_what_is_wrong(bad, word):
    from moe_b200.config import ConfigError, parse_config

    cfg = U.config_dict("mix")
    bad(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_looped_layers_run_in_order_with_a_cache_entry_for_every_run(name):
    from moe_b200.config import parse_config

    cfg = U.config_dict(name)
    arch, typed = parse_config(cfg)
    spec = arch.model_spec(typed)
    order = plain.layer_order(cfg)
    assert [e.layer for e in spec.schedule] == [l for l, _ in order]
    assert [e.cache for e in spec.schedule] == list(range(len(order)))            # no two runs share a cache entry
    assert [e.join for e in spec.schedule] == [t for _, t in order]
    times = cfg["loop"]["times"] if cfg.get("loop") else 0
    assert [(j.kind, j.params["row"], j.prefix) for j in spec.joins] == [("add_row", t, "loop.step") for t in range(times)]
    if cfg.get("loop"):
        a, b = cfg["loop"]["start"], cfg["loop"]["stop"]
        assert len(order) == len(cfg["layers"]) + (times - 1) * (b - a)
        starts = [i for i, (_, t) in enumerate(order) if t is not None]
        assert starts == [a + t * (b - a) for t in range(times)]


def test_a_missing_or_misshapen_tensor_is_named(root):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore, TensorDictStore, WeightError

    d = U.model_folder(root, "mix")
    arch, typed = parse_config(read_config_json(d))
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    t = {n: store.raw(n) for n in store.names()}
    del t["l1.mix.sink"]
    t["l0.mix.lq2"] = torch.zeros(15)
    t["loop.step"] = torch.zeros(2, 64)
    with pytest.raises(WeightError) as e:
        bad = TensorDictStore(t)
        bad.check({n: ts.shape for n, ts in expected_tensors(spec, bad).items()}, spec.ignorable)
    for word in ("l1.mix.sink", "l0.mix.lq2", "loop.step"):
        assert word in str(e.value)


def test_plain_latent_attention_is_attention_over_the_latents_alone(root):
    """The definition (keys and values of every head projected from the latent) against the form the
    library runs: queries carried onto the latent, one shared record a position as key and value, the
    attended latent projected onto the values; the sink's exponential in the denominator of both."""
    cfg, w = plain.read_model(U.model_folder(root, "mix"))
    m, p, eps = cfg["layers"][1]["mixer"], "l1.mix", cfg["norm"]["eps"]
    g = torch.Generator().manual_seed(2)
    n = torch.randn(40, cfg["width"], generator=g, dtype=F)
    ref = plain.latent_attention_mixer(w, p, m, n, eps)
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    c = plain.rms(n @ w[p + ".dkv"].T, eps) * w[p + ".dkv.norm"]
    q = (n @ w[p + ".q"].T).reshape(-1, H, d)
    heads = []
    for h in range(H):
        qc = q[:, h] @ w[p + ".uk"][h * d:(h + 1) * d]                         # [T, r]
        a = plain.softmax_attention(qc, c, c, m["scale"], sink=w[p + ".sink"][h])
        heads.append(a @ w[p + ".uv"][h * dv:(h + 1) * dv].T)
    again = torch.cat(heads, dim=-1) @ w[p + ".o"].T
    assert (ref - again).abs().max() < 1e-12
    # a token's output depends on no later token, and the sink takes weight from every token
    assert (plain.latent_attention_mixer(w, p, m, n[:13], eps) - ref[:13]).abs().max() < 1e-12
    w2 = dict(w)
    w2[p + ".sink"] = w[p + ".sink"] + 3.0
    assert (plain.latent_attention_mixer(w2, p, m, n, eps) - ref).abs().max() > 1e-3


@pytest.mark.parametrize("E,top,groups,keep", [(6, 2, 3, 2), (8, 3, 2, 1), (8, 5, 4, 3), (4, 2, 2, 2), (5, 1, 5, 2), (6, 3, 1, 1)])
def test_plain_choice_within_groups_against_an_exhaustive_search(E, top, groups, keep):
    """Among all sets of ``keep`` groups, the kept one has the largest best scores; among all sets of
    ``top`` experts inside the kept groups, the chosen one has the largest sum of scores."""
    g = torch.Generator().manual_seed(E * 100 + top)
    scores = torch.softmax(2 * torch.randn(50, E, generator=g, dtype=F), dim=-1)
    picked, wts = plain.route(scores, top, groups, keep)
    gs = E // groups
    limited = 0
    for t in range(50):
        s = scores[t]
        best = [float(s[i * gs:(i + 1) * gs].max()) for i in range(groups)]
        kept = max(itertools.combinations(range(groups), min(keep, groups)), key=lambda c: sorted((best[i] for i in c), reverse=True))
        allowed = [e for e in range(E) if e // gs in kept]
        want = max(itertools.combinations(allowed, top), key=lambda c: sum(float(s[e]) for e in c))
        assert sorted(picked[t].tolist()) == sorted(want)
        assert abs(float(wts[t].sum()) - 1.0) < 1e-12
        assert torch.allclose(wts[t], s[picked[t]] / s[picked[t]].sum())
        limited += sorted(want) != sorted(torch.topk(s, top).indices.tolist())
    if 1 < groups and top > keep:
        assert limited > 0                                   # the groups do change choices
    else:
        assert limited == 0                                  # the best ``top`` lie in at most ``top`` groups, the best ones


def test_plain_differential_attention_by_hand_on_two_tokens():
    """Two tokens, one head, no rotation: the second token's two maps written out by hand."""
    g = torch.Generator().manual_seed(9)
    W, d, dv, eps, diff, scale, cap = 6, 4, 3, 1e-5, 0.3, 0.7, 2.0
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "diff": diff, "scale": scale, "softcap": cap}
    w = {"p.q": torch.randn(2 * d, W, generator=g, dtype=F), "p.k": torch.randn(2 * d, W, generator=g, dtype=F),
         "p.v": torch.randn(dv, W, generator=g, dtype=F), "p.q.b": torch.randn(2 * d, generator=g, dtype=F),
         "p.k.b": torch.randn(2 * d, generator=g, dtype=F), "p.v.b": torch.randn(dv, generator=g, dtype=F),
         "p.g": torch.randn(1, W, generator=g, dtype=F), "p.o": torch.eye(dv, dtype=F)}
    for r in ("lq1", "lk1", "lq2", "lk2"):
        w["p." + r] = 0.5 * torch.randn(d, generator=g, dtype=F)
    n = torch.randn(2, W, generator=g, dtype=F)
    out = plain.attention_mixer(w, "p", m, n, eps)
    q, k, v = n @ w["p.q"].T + w["p.q.b"], n @ w["p.k"].T + w["p.k.b"], n @ w["p.v"].T + w["p.v.b"]
    a = []
    for j in (0, 1):
        s = torch.stack([q[1, j * d:(j + 1) * d] @ k[i, j * d:(j + 1) * d] for i in (0, 1)]) * scale
        s = cap * torch.tanh(s / cap)
        e = torch.exp(s - s.max())
        a.append((e / e.sum()) @ v)
    lam = torch.exp(w["p.lq1"] @ w["p.lk1"]) - torch.exp(w["p.lq2"] @ w["p.lk2"]) + diff
    o = a[0] - lam * a[1]
    o = o / torch.sqrt((o * o).mean() + eps) * (1 - diff) * torch.sigmoid(n[1] @ w["p.g"][0])
    assert (out[1] - o).abs().max() < 1e-12
    # the first token sees itself only: both maps return its value
    o0 = v[0] * (1 - lam)
    o0 = o0 / torch.sqrt((o0 * o0).mean() + eps) * (1 - diff) * torch.sigmoid(n[0] @ w["p.g"][0])
    assert (out[0] - o0).abs().max() < 1e-12


def test_plain_window_and_rotation():
    assert plain.seen_mask(5, 2).int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [0, 1, 1, 0, 0], [0, 0, 1, 1, 0], [0, 0, 0, 1, 1]]
    assert plain.seen_mask(3, None).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    # a rotation keeps lengths (times the factor on cos and sin) and leaves the unrotated part alone;
    # the score of a rotated query and key depends on the distance only
    rot = {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    f, mult = plain.yarn_frequencies(rot)
    plainf = 100.0 ** (-2.0 * torch.arange(4, dtype=F) / 8)
    assert float(f[0]) == 1.0 and abs(float(f[-1]) - float(plainf[-1]) / 4.0) < 1e-15 and (f <= plainf).all()
    assert abs(mult - (0.1 * torch.log(torch.tensor(4.0, dtype=F)) + 1)) < 1e-12
    g = torch.Generator().manual_seed(4)
    x = torch.randn(1, 1, 12, generator=g, dtype=F)
    y = torch.randn(1, 1, 12, generator=g, dtype=F)
    a = plain.rotate(x.expand(30, 1, 12), torch.arange(30), rot)
    b = plain.rotate(y.expand(30, 1, 12), torch.arange(30), rot)
    assert torch.equal(a[..., 8:], x.expand(30, 1, 12)[..., 8:])
    assert (a[..., :8].norm(dim=-1) - mult * x[..., :8].norm()).abs().max() < 1e-12
    s = torch.einsum("thd,uhd->tu", a, b)
    assert (s[7, 3] - s[24, 20]).abs() < 1e-10 and (s[7, 3] - s[8, 3]).abs() > 1e-6
