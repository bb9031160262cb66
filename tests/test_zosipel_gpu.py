"""Zosipel on the GPU against the plain implementation (tests/plain_zosipel.py): every mechanism
alone, whole prompts, decoding through the cache, portions of prompts, unequal batches, slots and
pages used again, windows' and pages' edges, far keys, sinks, long decoding, greedy generation and
the trace program.  Configurations and weights are the tests' own (tests/zosipel_util.py)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import gpu_util as G
import helpers
import plain_zosipel as plain
import zosipel_util as U

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
NAMES = ["mix", "lean", "ones", "sharp", "wide"]
F = torch.float64
DEV = "cuda:0"


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("zosipel")


_engines, _models = {}, {}


def engine_of(root, name, dtype, max_slots=None, use_graphs=None, edit=None, edit_weights=None):
    import moe_b200
    from moe_b200.engine import Engine

    d = U.model_folder(root, name, edit=edit, edit_weights=edit_weights)
    key = (d, dtype, max_slots, use_graphs)
    if key not in _engines:
        _engines[key] = Engine(moe_b200.load_model(d, dtype=dtype), max_tokens=2048, max_slots=max_slots,
                               use_graphs=use_graphs)
    return d, _engines[key]


def model_of(folder):
    if folder not in _models:
        _models[folder] = plain.read_model(folder)
    return _models[folder]


def tol_of(name, dtype):
    """Against the plain implementation.  In bfloat16 queries and keys are rounded to 8 bits before the
    score, whose error is the score's size times 2^-8 or so: with the peaked attention of "sharp" and
    "far" (scores of 10 and more) that is tenths, several times what ordinary scores give."""
    if dtype == "bfloat16" and name in ("sharp", "far"):
        return 3 * G.tol(dtype)
    if dtype == "bfloat16" and name == "ones":
        return 1.5 * G.tol(dtype)         # a width of 32: a rounding is averaged over few terms
    return G.tol(dtype)


def check_schedule(folder, eng, requests, steps, tol, flip):
    """Run ``steps`` (helpers.run_schedule) and compare every wanted place with the plain
    implementation run whole, with the engine's expert choices (a choice may differ from the plain
    implementation's own only where the router logits that decide are within ``flip`` of each other).
    Returns {request: {position: row}} for comparisons between cuts."""
    cfg, w = model_of(folder)
    logits, picks = helpers.run_schedule(eng, steps)
    out, flips, total = {}, 0, 0
    for rid, toks in requests.items():
        forced = [[layer[(rid, i)] for i in range(len(toks))] for layer in picks]
        margins = []
        ref = plain.forward(cfg, w, toks, forced=forced, margins=margins)
        assert not margins or max(margins) < flip, f"{rid}: an expert choice differs at margin {max(margins):.3g}"
        flips, total = flips + len(margins), total + len(toks) * max(len(picks), 1)
        scale = float(ref.abs().max())
        rows = {pos: row for (r, pos), row in logits.items() if r == rid}
        assert rows, rid
        for pos, row in rows.items():
            err = float((row.double() - ref[pos]).abs().max()) / scale
            assert err < tol, f"{rid} at position {pos} of {len(toks)}: relative error {err:.3g}"
        out[rid] = rows
    assert flips <= 0.05 * total, f"expert choices differ too often: {flips} of {total}"
    return out


def portions_schedule(rid, toks, sizes):
    """One request in portions of the given sizes (the last size repeats), logits at every place."""
    steps, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        steps.append({"entries": [(rid, toks[at:at + n], list(range(n)))], "end": [rid] if at + n == len(toks) else []})
        at, i = at + n, i + 1
    return steps


def dev(t, dtype=torch.float32):
    return t.to(dtype).to(DEV).contiguous()


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("H,dv,D,gated", [(4, 24, 32, True), (1, 64, 64, True), (3, 16, 48, False), (2, 128, 128, True),
                                         (5, 6, 24, True), (2, 96, 96, False)])
def test_the_two_maps_are_joined_normed_and_gated(bf16, H, dv, D, gated):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(H * 10 + dv)
    T, lam, eps, mult = 11, 0.37, 1e-5, 0.7
    dt = torch.bfloat16 if bf16 else torch.float32
    ctx = (2 * torch.randn(T, 2 * H, D, generator=g)).to(dt)
    proj = torch.randn(T, 7 + H, generator=g)                              # the gate's logits: the last H columns of a wider row
    pd = dev(proj)
    out = torch.full((T, H * dv), 9.0, dtype=dt, device=DEV)
    core.diff_combine(ctx.to(DEV), out, nh=H, dv=dv, width=D, lam=lam, eps=eps, mult=mult, gate=pd[:, 7:] if gated else None)
    c = ctx.double()
    o = plain.rms(c[:, :H, :dv] - lam * c[:, H:, :dv], eps) * mult
    if gated:
        o = o * torch.sigmoid(proj[:, 7:].double())[:, :, None]
    assert (out.double().cpu() - o.reshape(T, H * dv)).abs().max() < (2e-2 if bf16 else 1e-5)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("H,d,r,D", [(3, 24, 40, 48), (1, 8, 8, 16), (5, 64, 64, 64), (2, 40, 20, 32), (4, 32, 128, 128)])
def test_latent_norm_queries_head_by_head_and_the_transposes(bf16, H, d, r, D):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(H * 100 + r)
    T, eps = 13, 1e-5
    dt = torch.bfloat16 if bf16 else torch.float32
    proj = 3 * torch.randn(T, H * d + r, generator=g)
    wn = 1 + 0.3 * torch.randn(r, generator=g)
    batch = G.make_batch(DEV, [1, 2], [0, 5], [9, 4])
    q_t = torch.full((H, T, d), 7.0, dtype=dt, device=DEV)
    k_new = torch.full((T, 1, D), 7.0, dtype=dt, device=DEV)
    status = core.new_status(DEV)
    core.latent_prepare(dev(proj), batch, nh=H, d=d, r=r, width=D, weight=dev(wn), eps=eps, q_t=q_t, k_new=k_new, status=status)
    core.check_status(status)
    c = plain.rms(proj[:, H * d:].double(), eps) * wn.double()
    tol = 2e-2 if bf16 else 1e-5
    assert (k_new[:, 0, :r].double().cpu() - c).abs().max() < tol * max(1.0, float(c.abs().max()))
    assert D == r or float(k_new[:, 0, r:].abs().max()) == 0.0                          # zero-filled beyond the latent
    q = proj[:, :H * d].reshape(T, H, d).transpose(0, 1)
    assert (q_t.double().cpu() - q.double()).abs().max() < tol * float(q.abs().max())
    # the queries as records of the cache's width, token by token
    if d <= D:
        q_rec = torch.full((T, H, D), 7.0, dtype=dt, device=DEV)
        k_two = torch.full((T, 1, D), 7.0, dtype=dt, device=DEV)
        core.latent_prepare(dev(proj), batch, nh=H, d=d, r=r, width=D, weight=dev(wn), eps=eps, q_t=q_rec, k_new=k_two, status=status,
                            token_major=True)
        assert torch.equal(k_two, k_new)
        assert torch.equal(q_rec[:, :, :d].cpu(), q_t.transpose(0, 1).cpu()) and (D == d or float(q_rec[:, :, d:].abs().max()) == 0.0)
    # [A, B, n] -> [B, A, wider], zero-filled, from either dtype into either
    for src_dt, dst_dt in ((torch.float32, dt), (dt, torch.float32), (dt, dt)):
        src = torch.randn(H, T, r + 3, generator=g).to(src_dt)
        dst = torch.full((T, H, D), 5.0, dtype=dst_dt, device=DEV)
        core.heads_transpose(src.to(DEV)[:, :, 3:], dst, n=r)                          # a slice: rows with a pitch
        want = src[:, :, 3:].transpose(0, 1).to(dst_dt)
        assert torch.equal(dst[:, :, :r].cpu(), want) and (D == r or float(dst[:, :, r:].abs().max()) == 0.0)


def test_a_vector_is_added_to_every_row_with_what_was_pending():
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(1)
    for W in (32, 50, 256):
        x, delta, row = torch.randn(9, W, generator=g), torch.randn(9, W, generator=g), torch.randn(W, generator=g)
        xs = dev(x)
        core.add_row(xs, dev(row), delta=dev(delta))
        assert (xs.cpu() - (x + delta + row)).abs().max() < 1e-6
        xs = dev(x)
        core.add_row(xs, dev(row))
        assert (xs.cpu() - (x + row)).abs().max() < 1e-6


@pytest.mark.parametrize("T", [1, 7, 70, 300])
@pytest.mark.parametrize("E,k,groups,keep", [(6, 2, 3, 2), (8, 3, 2, 1), (8, 5, 4, 3), (16, 4, 4, 1), (5, 1, 5, 2), (12, 6, 6, 3),
                                             (64, 6, 8, 3), (4, 2, 2, 2)])
def test_router_picks_within_the_best_groups_in_every_routing_kernel(T, E, k, groups, keep):
    """Scores are the softmax over all experts, a group's score is its best expert's, the picks are the
    best experts of the kept groups and their weights the picks' scores over their sum."""
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(E * 10 + k + T)
    H = 48
    h, wr = torch.randn(T, H, generator=g), 2.0 * torch.randn(E, H, generator=g) / math.sqrt(H)
    z = h.double() @ wr.double().T
    scores = torch.softmax(z, dim=-1)
    picked, wts = plain.route(scores, k, groups, keep)
    grp = dict(groups=groups, keep=keep) if keep < groups else {}

    def same(idx, wt):
        idx = idx.cpu().long()
        order = idx.argsort(dim=-1)
        ref_order = picked.argsort(dim=-1)
        assert torch.equal(idx.gather(1, order), picked.gather(1, ref_order))
        assert (wt.double().cpu().gather(1, order) - wts.gather(1, ref_order)).abs().max() < 1e-5

    idx = torch.empty((T, k), dtype=torch.int32, device=DEV)
    wt = torch.empty((T, k), dtype=torch.float32, device=DEV)
    core.router(dev(h), dev(wr), k, True, 1.0, idx, wt, **grp)
    same(idx, wt)
    idx2, wt2 = torch.zeros_like(idx), torch.zeros_like(wt)
    core.router_topk(dev(z), k, True, 1.0, idx2, wt2, num_experts=E, **grp)
    same(idx2, wt2)
    if T <= 64:
        status = core.new_status(DEV)
        got = core.route_dispatch(dev(h), dev(wr), k, True, 1.0, status=status, **grp)
        core.check_status(status)
        same(got[0], got[1])
    if keep < groups and k > keep and T >= 70:
        free = torch.topk(scores, k, dim=-1).indices.sort(dim=-1).values
        assert not torch.equal(free, picked.sort(dim=-1).values)                        # the groups do change choices


# ----------------------------------------------------------------------------- the attention kernels with this design's options
def attention_case(kernel, dt, nh, nkv, hd, window, softcap, sinks, before, new, seed, latent=False, edit=None):
    """A window, capped scores and a sink of its own value for every head (``sinks`` [nh] or None), in
    one attention kernel, for sequences with ``before`` cached positions and ``new`` new ones.  With
    ``latent`` the values are the keys (one plane of the cache).  Pages that no sequence has written
    hold huge numbers, so that a key that should be masked shows.  -> (kernel's rows, plain rows)."""
    from moe_b200.cache import KVCache, KVRequest
    from moe_b200.ops import core, tc

    torch.manual_seed(seed)
    B = len(new)
    cache = KVCache({0: KVRequest(nkv, hd, window, values_are_keys=latent)}, {0: None}, max_tokens=64 * 40, max_slots=B + 1,
                    dtype=dt, device=DEV)
    cache.groups[0].storage.fill_(3e30)
    view = cache.view(0)
    slots = [cache.acquire() for _ in range(B)]
    st = core.new_status(DEV)
    K = [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(before, new)]
    V = K if latent else [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(before, new)]
    Q = [(2 * torch.randn(b, nh, hd, device=DEV)).to(dt) for b in new]
    if edit:
        edit(Q, K, V)
    live = [i for i in range(B) if before[i] > 0]
    if live:                                         # the past goes through the cache
        for i in live:
            G.give_pages(cache, slots[i], before[i])
        b0 = G.make_batch(DEV, [slots[i] for i in live], [0] * len(live), [before[i] for i in live])
        core.kv_commit(torch.cat([K[i][:before[i]] for i in live]).contiguous(),
                       torch.cat([V[i][:before[i]] for i in live]).contiguous(), view, b0, st)
    for i in range(B):
        G.give_pages(cache, slots[i], before[i] + new[i])
    b1 = G.make_batch(DEV, slots, before, new)
    q = torch.cat(Q).contiguous()
    kn = torch.cat([K[i][before[i]:] for i in range(B)]).contiguous()
    vn = kn if latent else torch.cat([V[i][before[i]:] for i in range(B)]).contiguous()
    out = torch.full((q.shape[0], nh * hd), float("nan"), device=DEV, dtype=dt)
    scale = 1.3 / math.sqrt(hd)
    kw = dict(nh=nh, window=window, scale=scale, status=st, softcap=softcap, sink=dev(sinks) if sinks is not None else False)
    if kernel == "generic":
        core.attention_generic(q, kn, vn, view, b1, out, use_local=True, **kw)
    elif kernel == "tiled":
        assert core.attention_tiled(q, kn, vn, view, b1, out, use_local=True, **kw)
    elif kernel == "tc":
        assert tc.attention_cached(q, kn, vn, view, b1, out, **kw)
    elif kernel == "tc_prompt":
        assert not any(before)
        assert tc.attention_prefill(q, kn, vn, b1, out, nkv=nkv, hd=hd, **kw)
    else:                                            # one new token each: appended first, then read from the cache
        assert all(n == 1 for n in new)
        core.kv_commit(kn, vn, view, b1, st)
        core.attention_decode(q, view, b1, out, **kw)
    core.check_status(st)
    refs = []
    for i in range(B):
        full_q = torch.zeros(before[i] + new[i], nh, hd, dtype=F)
        full_q[before[i]:] = Q[i].double().cpu()
        k, v = K[i].double().cpu(), V[i].double().cpu()
        heads = [plain.softmax_attention(full_q[:, h], k[:, h // (nh // nkv)], v[:, h // (nh // nkv)], scale, window, softcap or None,
                                         sinks[h].double() if sinks is not None else None)[before[i]:] for h in range(nh)]
        refs.append(torch.cat(heads, dim=-1))
    return out.double().cpu(), torch.cat(refs)


PASTS = [([0, 0, 0], [5, 70, 131]),                       # fresh sequences only: nothing from the cache
         ([10, 100], [7, 30]),
         ([130, 64, 0], [70, 129, 200]),                  # past a page's and a tile's edge; a fresh one among them
         ([700, 128, 127, 129, 1], [300, 1, 5, 257, 128]),
         ([63, 64, 65, 191, 192, 193], [1, 2, 64, 65, 3, 130])]
ONES = [([0, 1, 63, 64, 65, 199, 200, 201, 700], [1] * 9), ([299, 300, 301, 7, 8, 9, 127, 128], [1] * 8)]
# (window, cap, sinks?)
OPTIONS = [(None, 0.0, True), (1, 0.0, True), (9, 5.0, False), (64, 0.0, True), (70, 3.0, False), (75, 30.0, True), (200, 0.0, True),
           (None, 2.0, False)]


def rows_agree(out, ref, before, new, tol):
    assert torch.isfinite(out).all(), (before, new)
    o = 0
    for a, b in zip(before, new):
        err = float((out[o:o + b] - ref[o:o + b]).abs().max())
        assert err < tol * max(float(ref[o:o + b].abs().max()), 0.1), (before, new, a, b, err)
        o += b


def sinks_of(nh, on):
    return torch.linspace(-2.0, 3.0, nh) if on else None


@pytest.mark.parametrize("option", OPTIONS)
@pytest.mark.parametrize("kernel,dt,nh,nkv,hd", [("generic", torch.float32, 3, 1, 48), ("tiled", torch.float32, 4, 2, 96),
                                                 ("tiled", torch.bfloat16, 2, 2, 80), ("tc", torch.bfloat16, 6, 3, 64),
                                                 ("tc", torch.bfloat16, 5, 1, 128)])
def test_window_cap_and_sinks_in_steps_of_several_tokens(kernel, dt, nh, nkv, hd, option):
    window, cap, sink = option
    for n, (before, new) in enumerate(PASTS):
        out, ref = attention_case(kernel, dt, nh, nkv, hd, window, cap, sinks_of(nh, sink), before, new, seed=n + hd)
        rows_agree(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)


@pytest.mark.parametrize("option", OPTIONS)
@pytest.mark.parametrize("hd", [64, 128])
def test_window_cap_and_sinks_in_whole_prompts_on_the_tensor_cores(hd, option):
    window, cap, sink = option
    before, new = [0, 0, 0, 0], [5, 70, 131, 400]
    out, ref = attention_case("tc_prompt", torch.bfloat16, 4, 2, hd, window, cap, sinks_of(4, sink), before, new, seed=hd)
    rows_agree(out, ref, before, new, 2e-2)


@pytest.mark.parametrize("option", OPTIONS)
@pytest.mark.parametrize("dt,nh,nkv,hd", [(torch.float32, 3, 1, 48), (torch.float32, 4, 2, 64), (torch.bfloat16, 6, 1, 128),
                                          (torch.bfloat16, 2, 2, 64), (torch.bfloat16, 4, 2, 80),
                                          # eight and more heads on a kv head: the tensor-core kernel
                                          (torch.bfloat16, 16, 2, 64), (torch.bfloat16, 24, 1, 128), (torch.bfloat16, 9, 1, 64)])
def test_window_cap_and_sinks_in_single_token_steps(dt, nh, nkv, hd, option):
    window, cap, sink = option
    for n, (before, new) in enumerate(ONES):
        out, ref = attention_case("decode", dt, nh, nkv, hd, window, cap, sinks_of(nh, sink), before, new, seed=n + hd)
        rows_agree(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)


@pytest.mark.parametrize("kernel,dt,nh,hd", [("generic", torch.float32, 3, 48), ("tiled", torch.float32, 6, 64), ("tiled", torch.bfloat16, 2, 48),
                                             ("tc", torch.bfloat16, 6, 64), ("tc", torch.bfloat16, 4, 128), ("tc_prompt", torch.bfloat16, 5, 64),
                                             ("decode", torch.float32, 6, 64), ("decode", torch.bfloat16, 3, 128),
                                             ("decode", torch.bfloat16, 16, 128), ("decode", torch.bfloat16, 40, 64),
                                             ("decode", torch.bfloat16, 8, 64)])
def test_many_heads_on_one_record_that_is_key_and_value(kernel, dt, nh, hd):
    """The cache of latent attention: one plane, one record a position, which every head reads as its
    key and as its value; a sink for every head."""
    cases = ONES if kernel == "decode" else [PASTS[0]] if kernel == "tc_prompt" else PASTS
    for n, (before, new) in enumerate(cases):
        out, ref = attention_case(kernel, dt, nh, 1, hd, None, 0.0, sinks_of(nh, True), before, new, seed=n, latent=True)
        rows_agree(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)


@pytest.mark.parametrize("kernel,dt,hd,nh", [("tiled", torch.float32, 64, 2), ("tc", torch.bfloat16, 64, 2), ("tc", torch.bfloat16, 128, 2),
                                             ("decode", torch.float32, 48, 2), ("decode", torch.bfloat16, 64, 2),
                                             ("decode", torch.bfloat16, 64, 12), ("decode", torch.bfloat16, 128, 16)])
def test_a_key_at_the_windows_edge_counts_for_the_last_query_that_sees_it_and_for_no_later_one(kernel, dt, hd, nh):
    """One key of the past is made to stand out (query and key scaled).  With a window of 200 the key at
    610 counts for the queries up to 809 (which then return that key's value, nearly) and for none from
    810 on; the ring of the window has wrapped several times by then."""
    window, far = 200, 610

    def edit(Q, K, V):
        for q in Q:
            q[:, :, 0] = 6.0
        for k in K:
            k[:, :, 0] = 0.0
            k[far, :, 0] = 40.0

    if kernel == "decode":
        for at, seen in ((809, True), (810, False), (700, True), (1200, False)):
            out, ref = attention_case(kernel, dt, nh, 1, hd, window, 0.0, None, [at], [1], seed=at, edit=edit)
            rows_agree(out, ref, [at], [1], 2e-5 if dt == torch.float32 else 2e-2)
    else:
        before, new = [780], [60]                                   # queries 780 ... 839: the edge falls inside the step
        out, ref = attention_case(kernel, dt, nh, 1, hd, window, 0.0, None, before, new, seed=1, edit=edit)
        rows_agree(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)
        # the plain rows do change at the edge: up to 809 they are that key's value
        assert float((ref[29] - ref[30]).abs().max()) > 0.5


# ----------------------------------------------------------------------------- whole prompts, layer by layer
@pytest.mark.parametrize("name", NAMES)
def test_every_layer_run_of_a_whole_prompt_in_32_bit(root, name):
    d, eng = engine_of(root, name, "float32", use_graphs=False)
    cfg, w = model_of(d)
    toks = U.tokens(cfg["vocab"], 150, 1)
    ref_layers = []
    ref = plain.forward(cfg, w, toks, ref_layers)
    eng.model.stream_tap = []
    try:
        s = eng.new_sequence()
        got = eng.step([s], [toks], [list(range(len(toks)))]).cpu()
        eng.release(s)
        tap = eng.model.stream_tap
    finally:
        eng.model.stream_tap = None
    assert len(tap) == len(ref_layers) == len(plain.layer_order(cfg))          # a looped layer counts every time
    for i, (a, b) in enumerate(zip(tap, ref_layers)):
        assert helpers.max_rel_err(a.cpu(), b) < 2e-5, f"layer run {i}"
    assert helpers.max_rel_err(got, ref) < G.tol("float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_of_many_lengths(root, name, dtype):
    """Lengths around a page (64), around the windows, one and two tokens, and past two pages."""
    d, eng = engine_of(root, name, dtype)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"w{n}": U.tokens(V, n, n) for n in (1, 2, 7, 21, 22, 63, 64, 65, 71, 129, 200)}
    check_schedule(d, eng, reqs, helpers.whole_schedule(reqs), tol_of(name, dtype), G.flip(dtype))



@pytest.mark.parametrize("seed", range(10))
def test_configurations_drawn_at_random_whole_decoded_and_batched_in_32_bit(root, seed):
    """Sizes, orders and constants nobody chose: each request whole, with its last 40 tokens one by one,
    and four at a time on four slots, against the plain implementation and against each other."""
    name = f"drawn{seed}"
    U.CONFIGS[name] = U.drawn_config(seed)
    d, eng = engine_of(root, name, "float32", max_slots=4)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"r{i}": U.tokens(V, n, 50 + i + seed) for i, n in enumerate([1, 2, 37, 131, 300, 70])}
    tol, flip = G.tol("float32"), G.flip("float32")
    whole = check_schedule(d, eng, reqs, helpers.whole_schedule(reqs), tol, flip)
    cuts = [check_schedule(d, eng, reqs, helpers.tail_schedule(reqs, 40), tol, flip),
            check_schedule(d, eng, reqs, helpers.batches_schedule(reqs, 4, lambda r: max(1, len(reqs[r]) - 36)), tol, flip)]
    for rid, rows in whole.items():
        scale = max(float(r.abs().max()) for r in rows.values())
        for cut in cuts:
            for pos, row in cut[rid].items():
                assert float((row.double() - rows[pos].double()).abs().max()) / scale < 4 * G.tol_cut("float32"), (rid, pos)
    assert eng.cache.ledger.slots.num_held == 0
    _engines.pop((d, "float32", 4, None))

# ----------------------------------------------------------------------------- the same tokens cut differently
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_decoding_token_by_token_from_the_first_token_and_long_after_the_rings_wrap(root, name, dtype):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 210, 3)
    reqs = {"r": toks}
    tol, flip = tol_of(name, dtype), G.flip(dtype)
    check_schedule(d, eng, reqs, portions_schedule("r", toks, [1]), tol, flip)        # every token alone, 210 steps
    check_schedule(d, eng, reqs, helpers.tail_schedule(reqs, tail=150), tol, flip)    # a prompt of 60, then 150 single steps


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_prompt_and_its_replay_token_by_token_agree_closely(root, dtype):
    """The same tokens whole, in portions and one by one, against each other (not only against the plain
    implementation): what differs is the order of sums and, in bfloat16, which kernel rounds where."""
    d, eng = engine_of(root, "mix", dtype)
    toks = U.tokens(U.CONFIGS["mix"]["vocab"], 140, 5)
    reqs = {"r": toks}
    tol, flip = tol_of("mix", dtype), G.flip(dtype)
    whole = check_schedule(d, eng, reqs, helpers.whole_schedule(reqs), tol, flip)["r"]
    for sizes in ([1], [2], [64, 1], [70, 3]):
        cut = check_schedule(d, eng, reqs, portions_schedule("r", toks, sizes), tol, flip)["r"]
        scale = max(float(r.abs().max()) for r in whole.values())
        worst = max(float((cut[p].double() - whole[p].double()).abs().max()) / scale for p in whole)
        assert worst < 2 * G.tol_cut(dtype), (sizes, worst)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("sizes", [[2], [3, 64, 1, 65, 2, 7], [64], [63, 2, 1, 70], [129, 5]])
def test_portions_of_a_prompt_of_several_sizes(root, name, dtype, sizes):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 150 if sizes == [2] else 200, 4)
    check_schedule(d, eng, {"r": toks}, portions_schedule("r", toks, sizes), tol_of(name, dtype), G.flip(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_few_slots_against_the_plain_implementation(root, name, dtype):
    """Seven requests of unequal lengths on three slots: a batch starts with half of each prompt in one
    step and decodes together, the shorter ones leave earlier, and the next batch takes over slots and
    pages that were given back (twice, so that everything has been used before)."""
    d, eng = engine_of(root, name, dtype, max_slots=3)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"b{i}": U.tokens(V, n, 20 + i) for i, n in enumerate([150, 3, 40, 1, 131, 66, 17])}
    steps = helpers.batches_schedule(reqs, 3, lambda r: len(reqs[r]) // 2)
    for _ in range(2):
        check_schedule(d, eng, reqs, steps, tol_of(name, dtype), G.flip(dtype))
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_gives_every_request_what_it_gets_alone(root, dtype):
    d, eng = engine_of(root, "mix", dtype)
    V = U.CONFIGS["mix"]["vocab"]
    reqs = {f"a{i}": U.tokens(V, n, 30 + i) for i, n in enumerate([90, 7, 65, 30])}
    tol, flip = tol_of("mix", dtype), G.flip(dtype)
    alone = check_schedule(d, eng, reqs, helpers.tail_schedule(reqs, tail=5), tol, flip)
    together = check_schedule(d, eng, reqs, helpers.batches_schedule(reqs, 4, lambda r: len(reqs[r]) - 5), tol, flip)
    for r in reqs:
        scale = max(float(x.abs().max()) for x in alone[r].values())
        for p in alone[r]:
            assert float((alone[r][p].double() - together[r][p].double()).abs().max()) / scale < 2 * G.tol_cut(dtype), (r, p)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_portions_that_go_on_from_different_places(root, dtype):
    """Fresh and continued sequences mixed in one step, each bringing a different number of tokens."""
    d, eng = engine_of(root, "mix", dtype)
    V = U.CONFIGS["mix"]["vocab"]
    reqs = {f"m{i}": U.tokens(V, n, 40 + n) for i, n in enumerate((90, 130, 70))}
    cuts = {"m0": [60, 30], "m1": [5, 64, 61], "m2": [70]}
    at = {r: 0 for r in reqs}
    steps = []
    for step in range(3):
        entries, end = [], []
        for r in reqs:
            if step < len(cuts[r]):
                n = cuts[r][step]
                entries.append((r, reqs[r][at[r]:at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == len(reqs[r]):
                    end.append(r)
        steps.append({"entries": entries, "end": end})
    check_schedule(d, eng, reqs, steps, G.tol(dtype), G.flip(dtype))


# ----------------------------------------------------------------------------- edges that random weights would hide
def with_window(layer, delta):
    def edit(cfg):
        cfg["layers"][layer]["mixer"]["mask"]["size"] += delta
    edit.__name__ = f"window{layer}{delta:+d}"
    return edit


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_window_one_position_longer_or_shorter_would_show(root, dtype):
    """With peaked attention the result moves by far more than the tolerance when the first layer's
    window is one position longer or shorter (the plain implementation says by how much); the engine
    agrees with the windows of the configuration, whole, decoded and in portions.  One window is
    shorter than a page, the other two positions longer than one."""
    d, eng = engine_of(root, "sharp", dtype)
    cfg, w = model_of(d)
    toks = U.tokens(cfg["vocab"], 160, 6)
    ref = plain.forward(cfg, w, toks)
    scale = float(ref.abs().max())
    c = cfg["layers"][0]["mixer"]["mask"]["size"]
    for delta in (-1, +1):
        other = plain.forward(*model_of(U.model_folder(root, "sharp", edit=with_window(0, delta))), toks)
        moved = (other - ref).abs().amax(dim=1) / scale
        assert float(moved[: c - 1].max()) == 0.0                      # while the whole past fits the window nothing differs
        assert float(moved[c + 1:].median()) > max(1e-2, 5 * G.tol(dtype))   # afterwards nearly every place does
    reqs = {"r": toks}
    for steps in (helpers.whole_schedule(reqs), helpers.tail_schedule(reqs, tail=100), portions_schedule("r", toks, [5, 9, 10, 1, 64])):
        check_schedule(d, eng, reqs, steps, tol_of("sharp", dtype), G.flip(dtype))


SPIKE = 5


def spike_in_window(w, cfg):
    U.spike_attention(w, cfg, SPIKE)


def window_of(size):
    def edit(cfg):
        cfg["layers"][0]["mixer"]["mask"]["size"] = size
    edit.__name__ = f"window{size}"
    return edit


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [5, 64, 67])
def test_a_key_counts_for_the_last_position_of_its_window_and_for_none_after(root, dtype, window):
    """The layer's weights are made so that the key of one token outweighs all others in one map of
    every head, at any distance.  That token stands at one place (not the first).  Replacing it moves the
    plain implementation's logits by a large part of their size at every place whose window holds it,
    up to the last one, and by nothing at all from the next place on.  The engine agrees with the plain
    implementation on the original at every place: whole, with the places around the edge decoded one
    by one, and in portions that end just before, at and just after the edge (windows shorter than a
    page, of a page, and three positions longer)."""
    at = 3
    d, eng = engine_of(root, "edge", dtype, edit=window_of(window), edit_weights=spike_in_window)
    cfg, w = model_of(d)
    toks = [t if t != SPIKE else SPIKE + 1 for t in U.tokens(cfg["vocab"], 150, 9)]
    toks[at] = SPIKE
    ref = plain.forward(cfg, w, toks)
    other = plain.forward(cfg, w, toks[:at] + [SPIKE + 1] + toks[at + 1:])
    moved = (other - ref).abs().amax(dim=1) / float(ref.abs().max())
    last = at + window - 1                                               # the last place that sees the key
    assert float(moved[at:last + 1].min()) > 0.15 and float(moved[last + 1:].max()) < 1e-12 and float(moved[:at].max()) < 1e-12
    reqs = {"r": toks}
    tol = tol_of("sharp", dtype)
    for steps in (helpers.whole_schedule(reqs), helpers.tail_schedule(reqs, tail=len(toks) - last + 2),
                  portions_schedule("r", toks, [last - 1, 1, 1, 1, 1, 70]), portions_schedule("r", toks, [last + 1, 2, 64]),
                  portions_schedule("r", toks, [2, last - 1, 3, 1]), portions_schedule("r", toks, [1])):
        check_schedule(d, eng, reqs, steps, tol, G.flip(dtype))




def spike(w, cfg):
    U.spike_token(w, cfg, SPIKE)


def no_sinks(w, cfg):
    for name in w:
        if name.endswith(".sink"):
            w[name] = torch.full_like(w[name], -60.0)


def large_sinks(w, cfg):
    for name in w:
        if name.endswith(".sink"):
            w[name] = torch.full_like(w[name], 3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_among_hundreds_is_seen(root, dtype):
    """The layer of this configuration sees every earlier token, and its weights are made so that the
    key of one token, which stands at the very first place only, outweighs all others.  Without that
    key (another token in its place) the plain implementation's logits move by a large part of their
    size 300 and more places later.  The engine agrees with the plain implementation on the original:
    whole, decoded one by one across five pages, and in portions."""
    d, eng = engine_of(root, "far", dtype, edit_weights=spike)
    cfg, w = model_of(d)
    toks = [SPIKE] + [t if t != SPIKE else SPIKE + 1 for t in U.tokens(cfg["vocab"], 329, 7)]
    ref = plain.forward(cfg, w, toks)
    other = plain.forward(cfg, w, [SPIKE + 1] + toks[1:])
    assert float((other - ref)[300:].abs().amax(dim=1).min()) / float(ref.abs().max()) > 0.1
    reqs = {"r": toks}
    for steps in (helpers.whole_schedule(reqs), helpers.tail_schedule(reqs, tail=40), portions_schedule("r", toks, [100, 64, 3, 129])):
        check_schedule(d, eng, reqs, steps, tol_of("far", dtype), G.flip(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["far", "lean"])
def test_the_sink_counts_once_unscaled_and_most_for_the_first_tokens(root, name, dtype):
    """The first tokens of a sequence have few keys, so the sink's share of the denominator is large:
    with sinks of 3 the plain result is far from the one with sinks that are as good as absent (-60),
    and, where the score scale is not 1, from the one whose sinks are 3 times the scale.  The engine
    agrees with the plain implementation on each, whole and one token at a time."""
    flat = U.CONFIGS[name]["layers"]
    li = next(i for i, L in enumerate(flat) if L["type"] == "latent_attention")
    scale = flat[li]["mixer"]["scale"]
    short = U.tokens(U.CONFIGS[name]["vocab"], 12, 8)
    results = {}
    for edit in (large_sinks, no_sinks):
        d, eng = engine_of(root, name, dtype, edit_weights=edit)
        cfg, w = model_of(d)
        results[edit.__name__] = plain.forward(cfg, w, short)
        check_schedule(d, eng, {"s": short}, helpers.whole_schedule({"s": short}), tol_of(name, dtype), G.flip(dtype))
        check_schedule(d, eng, {"s": short}, portions_schedule("s", short, [1]), tol_of(name, dtype), G.flip(dtype))
    size = float(results["large_sinks"].abs().max())
    assert float((results["large_sinks"] - results["no_sinks"]).abs().max()) / size > 10 * G.tol(dtype)
    if scale != 1.0:
        cfg, w = model_of(U.model_folder(root, name, edit_weights=large_sinks))
        w2 = {k: (v * scale if k.endswith(".sink") else v) for k, v in w.items()}
        assert float((plain.forward(cfg, w2, short) - results["large_sinks"]).abs().max()) / size > 5 * G.tol(dtype)


# ----------------------------------------------------------------------------- the library's entry points
def every_expert(cfg):
    """Nothing to choose: the comparison with the plain implementation's own choices is then exact."""
    for L in cfg["layers"]:
        if L.get("mlp"):
            L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
            L["mlp"]["router"].pop("groups", None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["lean", "mix"])
def test_greedy_generation_through_the_generation_loop(root, name, dtype):
    import moe_b200

    d, eng = engine_of(root, name, dtype, edit=every_expert)
    cfg, w = model_of(d)
    prompts = [U.tokens(cfg["vocab"], n, 60 + n) for n in (5, 70, 1, 23)]
    outs = moe_b200.generate(eng, prompts, max_tokens=12, eos=())
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain.forward(cfg, w, p + o.tokens)[len(p) - 1:-1]
        top = ref.max(dim=-1).values
        margin = (2e-4 if dtype == "float32" else 4e-2) * float(ref.abs().max())
        for j, tok in enumerate(o.tokens):
            assert float(ref[j, tok]) >= float(top[j]) - margin, (p[:3], j, tok)
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_trace_program_replays_steps_on_a_model_folder(root, tmp_path, dtype):
    """bin/trace_run as a user drives it: two requests start together in one step, go on by one token
    each, the shorter one ends earlier; its files against the plain implementation."""
    d = U.model_folder(root, "lean", edit=every_expert)
    cfg, w = model_of(d)
    V = cfg["vocab"]
    a, b = U.tokens(V, 75, 70), U.tokens(V, 9, 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 63, 64, 69]},
                                      {"id": "b", "tokens": b[:7], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[70]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[71]], "want": []}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[72:], "want": [2]}], "end": ["a"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                        "--max-tokens", "84"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    want = {0: ra[[0, 63, 64, 69]], 1: torch.stack([ra[70], rb[7]]), 2: rb[8:9], 3: ra[74:75]}
    import numpy as np

    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        assert got.shape == ref.shape and helpers.max_rel_err(got, ref) < G.tol(dtype), n


def test_model_summary_names_the_parts(root):
    import moe_b200

    d = U.model_folder(root, "mix")
    model = moe_b200.load_model(d, dtype="bfloat16")
    b = model.blocks
    assert b[0].kind == "prenorm" and "weight 1 + w" in b[0].norm1.describe()
    for word in ("differential attention (4 heads of two maps / 2 kv heads", "map size 16", "values of 24", "lambda offset 0.2",
                 "one sigmoid gate a head", "YaRN x4", "capped at 8", "window 21"):
        assert word in b[0].mixer.describe(), word
    for word in ("latent attention (3 heads of 24", "values of 16", "one cached latent of 40", "sink"):
        assert word in b[1].mixer.describe(), word
    assert "within the best 2 of 3 groups" in b[0].ffn.describe() and "shared expert 48 (gated)" in b[0].ffn.describe()
    assert "groups" not in b[3].ffn.describe() and b[2].ffn is None and b[2].norm2 is None
    # one cache entry for every run of a layer; a latent layer caches one record of its latent a position
    assert len(model.spec.schedule) == 1 + 3 * 2 + 1
    assert b[1].mixer.kv_request().num_kv_heads == 1 and b[1].mixer.kv_request().values_are_keys
    assert b[0].mixer.kv_request().num_kv_heads == 4 and b[0].mixer.kv_request().window == 21
