"""Divadra without a GPU: the configuration reader, the translation into parts, the tensor names and
shapes against the tests' own checkpoints, the random-weights mode, and pieces of the plain
implementation worked out by hand."""
import json
import math

import pytest
import torch

import divadra_util as U
import plain_divadra as plain

F = torch.float64


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("divadra_cpu")


@pytest.mark.parametrize("name", sorted(U.CONFIGS))
def test_config_parts_and_tensor_names_fit_the_checkpoint(root, name):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore

    d = U.model_folder(root, name)
    arch, typed = parse_config(read_config_json(d))
    assert arch.name == "Divadra"
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    exp = expected_tensors(spec, store)
    store.check({n: ts.shape for n, ts in exp.items()}, spec.ignorable, integer=[n for n, ts in exp.items() if ts.integer])
    assert [l.block for l in spec.layers] == ["parallel"] * len(typed.layers)
    assert typed.to_dict() == json.load(open(d + "/config.json"))
    assert spec.embedding.kind == "pair_embedding"
    for L, ls in zip(typed.layers, spec.layers):
        assert ls.mixer.kind == {"parallel": "side_by_side", "mamba2": "ssd"}[L.type]
        assert (ls.ffn is None) == (L.mlp is None) == (ls.norm2 is None) == (ls.pre2 is None)
        assert ls.pre1.kind == "residual_conv" and ls.pre1.params["taps"] == typed.canon_taps


def test_a_config_written_from_the_typed_form_reads_back_the_same():
    from moe_b200.config.divadra import DivadraConfig

    for name in U.CONFIGS:
        typed = DivadraConfig.from_dict(U.config_dict(name))
        bare = DivadraConfig(typed.vocab, typed.width, typed.norm_eps, typed.canon_taps, typed.buckets, typed.mul_prev,
                             typed.mul_cur, typed.layers)
        again = DivadraConfig.from_dict(bare.to_dict())
        assert again.layers == typed.layers and again.vocab == typed.vocab and again.buckets == typed.buckets


@pytest.mark.parametrize("bad,word", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(vdim=15), "even"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "unknown kind"),
    (lambda c: c.pop("canon"), "canon"),
    (lambda c: c["embedding"].pop("bigram"), "bigram"),
])
def test_config_errors_say_what_is_wrong(bad, word):
    from moe_b200.config import ConfigError, parse_config

    cfg = U.config_dict("mix")
    bad(cfg)
    with pytest.raises(ConfigError) as e:
        parse_config(cfg)
    assert word in str(e.value)


def test_an_integer_table_is_asked_for_as_one_and_floats_are_refused_in_its_place(root):
    from moe_b200.config import parse_config, read_config_json
    from moe_b200.models.decoder import expected_tensors
    from moe_b200.weights import SafetensorsStore, TensorDictStore, WeightError

    d = U.model_folder(root, "mix")
    arch, typed = parse_config(read_config_json(d))
    spec = arch.model_spec(typed)
    store = SafetensorsStore(d)
    assert store.raw("l1.mlp.table").dtype == torch.int32
    t = {n: store.raw(n) for n in store.names()}
    t["l1.mlp.table"] = t["l1.mlp.table"].to(torch.float32)
    bad = TensorDictStore(t)
    exp = expected_tensors(spec, bad)
    with pytest.raises(WeightError):
        bad.check({n: ts.shape for n, ts in exp.items()}, spec.ignorable, integer=[n for n, ts in exp.items() if ts.integer])


def test_random_weights_give_tables_of_distinct_experts(tmp_path):
    import moe_b200
    from moe_b200.weights import SafetensorsStore

    d = moe_b200.write_random_model(str(tmp_path / "m"), U.config_dict("mix"), seed=3)
    store = SafetensorsStore(d)
    table = store.raw("l1.mlp.table")
    assert table.dtype == torch.int32 and tuple(table.shape) == (131, 2)
    assert int(table.min()) >= 0 and int(table.max()) < 6 and bool((table[:, 0] != table[:, 1]).all())
    cfg, w = plain.read_model(d)
    assert torch.isfinite(plain.forward(cfg, w, [1, 5, 5, 130])).all()


def test_pair_rows_and_convolution_by_hand():
    assert plain.bigram_rows([4, 9, 9, 2], 7, 3, 5) == [7, (4 * 3 + 9 * 5) % 7, (9 * 3 + 9 * 5) % 7, (9 * 3 + 2 * 5) % 7]
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=F)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=F)          # the last column is the token's own
    assert plain.causal_taps(u, w).flatten().tolist() == [1.0, 12.0, 124.0]


def test_sigmoid_attention_in_chunks_by_hand():
    """Three positions, chunks of two: position 2 starts a chunk and sees itself alone; the weights are
    sigmoids that do not sum to one."""
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 2.0]], [[1.0, 1.0]]], dtype=F)
    k = torch.tensor([[[1.0, 1.0]], [[2.0, 0.5]], [[0.0, 3.0]]], dtype=F)
    v = torch.tensor([[[1.0]], [[10.0]], [[100.0]]], dtype=F)
    b = torch.tensor([-0.5], dtype=F)
    out = plain.chunked_sigmoid_attention(q, k, v, 0.5, 2, b).flatten()

    def sg(x):
        return 1.0 / (1.0 + math.exp(-x))

    want = [sg(0.5 * 1.0 - 0.5) * 1.0, sg(0.5 * 2.0 - 0.5) * 1.0 + sg(0.5 * 1.0 - 0.5) * 10.0, sg(0.5 * 3.0 - 0.5) * 100.0]
    assert max(abs(a - c) for a, c in zip(out.tolist(), want)) < 1e-12
    everything = plain.chunked_sigmoid_attention(q, k, v, 0.5, 0, b).flatten()
    assert abs(float(everything[2]) - (sg(0.5 * 2.0 - 0.5) * 1.0 + sg(0.5 * 2.5 - 0.5) * 10.0 + want[2])) < 1e-12


def test_values_arrive_turned_by_their_distance_to_the_query():
    """A value rotated by its position j and turned back by the query's position i is the value rotated by
    j - i: the same for every pair of positions that far apart."""
    g = torch.Generator().manual_seed(1)
    v = torch.randn(1, 1, 8, generator=g, dtype=F)
    a = plain.rotate_halves(plain.rotate_halves(v, torch.tensor([3]), 8, 100.0), torch.tensor([10]), 8, 100.0, sign=-1.0)
    b = plain.rotate_halves(plain.rotate_halves(v, torch.tensor([40]), 8, 100.0), torch.tensor([47]), 8, 100.0, sign=-1.0)
    c = plain.rotate_halves(v, torch.tensor([-7]), 8, 100.0)
    assert (a - b).abs().max() < 1e-12 and (a - c).abs().max() < 1e-12


def test_plain_recurrences_do_not_depend_on_later_tokens(root):
    cfg, w = plain.read_model(U.model_folder(root, "mix"))
    g = torch.Generator().manual_seed(3)
    n = torch.randn(30, cfg["width"], generator=g, dtype=F)
    for p, m, fn in (("l1.mix", cfg["layers"][1]["mixer"], plain.ssd_mixer), ("l0.mix", cfg["layers"][0]["mixer"], plain.side_by_side_mixer)):
        whole, shorter = fn(w, p, m, n, 1e-5), fn(w, p, m, n[:17], 1e-5)
        assert whole.shape == (30, cfg["width"]) and (whole[:17] - shorter).abs().max() < 1e-12
    # the state-space recurrence by hand for one head, one state row, two tokens
    S, dt, a = 0.0, [0.5, 2.0], 0.3
    ys = []
    for t, (B, C, x) in enumerate([(2.0, 1.0, 3.0), (0.5, 4.0, -1.0)]):
        S = math.exp(-a * dt[t]) * S + dt[t] * B * x
        ys.append(C * S + 0.7 * x)
    assert abs(ys[0] - (1.0 * (0.5 * 2.0 * 3.0) + 2.1)) < 1e-12
    assert abs(ys[1] - (4.0 * (math.exp(-0.6) * 3.0 + 2.0 * 0.5 * -1.0) - 0.7)) < 1e-12


def test_experts_by_the_table_weigh_the_same(root):
    cfg, w = plain.read_model(U.model_folder(root, "mix"))
    g = torch.Generator().manual_seed(4)
    n = torch.randn(3, cfg["width"], generator=g, dtype=F)
    toks = [7, 7, 100]
    out = plain.table_experts(w, "l1.mlp", cfg["layers"][1]["mlp"], n, toks)
    e0, e1 = w["l1.mlp.table"][7].tolist()
    want = 0.5 * (plain.silu_glu(w, f"l1.mlp.e{e0}", n[:1]) + plain.silu_glu(w, f"l1.mlp.e{e1}", n[:1]))[0]
    assert (out[0] - want).abs().max() < 1e-12 and e0 != e1
