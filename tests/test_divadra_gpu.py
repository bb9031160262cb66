"""Divadra on the GPU against the plain implementation (tests/plain_divadra.py): every mechanism
alone, whole prompts, decoding through cache and state, portions of prompts, unequal batches, slots,
pages and state used again, chunks' and pages' edges, far keys, the first tokens, long decoding,
greedy generation and the trace program.  Configurations and weights are the tests' own
(tests/divadra_util.py)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import divadra_util as U
import gpu_util as G
import helpers
import plain_divadra as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
NAMES = ["mix", "lean", "ones", "sharp", "wide"]
F = torch.float64


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("divadra")


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
    score, whose error is the score's size times 2^-8 or so: with the peaked weights of "sharp" and "far"
    (scores of 10 and more) that is tenths, several times what ordinary scores give."""
    if dtype == "bfloat16" and name in ("sharp", "far"):
        return 3 * G.tol(dtype)
    return G.tol(dtype)


_sens = {}


def sensitivity(folder, toks):
    """Per position: how far the plain result moves (as a fraction of the largest logit) when every weight
    is changed by a relative 2^-8, the spacing of bfloat16 (the larger of two draws).  A position where that
    is much (a recurrent head whose first output nearly cancels before it is divided by its own size, so that
    a rounding may turn its sign) cannot be held to the same bound as the others by any 16-bit implementation."""
    key = (folder, tuple(toks))
    if key not in _sens:
        cfg, w = model_of(folder)
        g = torch.Generator().manual_seed(len(toks))
        ref = plain.forward(cfg, w, toks)
        worst = torch.zeros(len(toks), dtype=F)
        for _ in range(2):
            w2 = {n: (t * (1.0 + 2.0 ** -8 * torch.randn(t.shape, generator=g, dtype=F)) if t.is_floating_point() else t)
                  for n, t in w.items()}
            worst = torch.maximum(worst, (plain.forward(cfg, w2, toks) - ref).abs().amax(dim=1) / float(ref.abs().max()))
        _sens[key] = worst
    return _sens[key]


def allowed(folder, toks, tol):
    """The bound at every position: ``tol``, and for the 16-bit path four times the position's sensitivity on top."""
    if tol < 1e-3:
        return torch.full((len(toks),), tol, dtype=F)
    return tol + 4.0 * sensitivity(folder, toks)


def check_schedule(folder, eng, requests, steps, tol):
    """Run ``steps`` (helpers.run_schedule) and compare every wanted place with the plain
    implementation run whole.  Returns {request: {position: row}} for comparisons between cuts."""
    cfg, w = model_of(folder)
    logits, _ = helpers.run_schedule(eng, steps)
    out = {}
    for rid, toks in requests.items():
        ref = plain.forward(cfg, w, toks)
        scale = float(ref.abs().max())
        bound = allowed(folder, toks, tol)
        rows = {pos: row for (r, pos), row in logits.items() if r == rid}
        assert rows, rid
        for pos, row in rows.items():
            err = float((row.double() - ref[pos]).abs().max()) / scale
            assert err < float(bound[pos]), f"{rid} at position {pos} of {len(toks)}: relative error {err:.3g}"
        out[rid] = rows
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
    return t.to(dtype).cuda().contiguous()


CUTS = [[(0, 0, 10)], [(0, 10, 12), (1, 0, 2)], [(0, 12, 23), (1, 2, 9)]]       # (sequence, from, to) per step


def run_cuts(lens, rows_of, call):
    """Two sequences of unequal lengths in three steps (the second one joins later, and a step brings
    fewer rows than a convolution has taps): ``call(batch, rows)`` -> a tensor [T, ...] whose rows are
    collected per sequence."""
    got = {s: [] for s in lens}
    for step in CUTS:
        batch = G.make_batch("cuda", [s + 1 for s, _, _ in step], [a for _, a, _ in step], [b - a for _, a, b in step])
        out = call(batch, dev(torch.cat([rows_of[s][a:b] for s, a, b in step])))
        o = 0
        for s, a, b in step:
            got[s].append(out[o:o + b - a].double().cpu())
            o += b - a
    return {s: torch.cat(v) for s, v in got.items()}


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("width,taps,residual,act", [(64, 3, True, None), (48, 1, True, None), (40, 4, False, "silu"),
                                                     (300, 2, False, "silu"), (32, 5, True, None)])
def test_causal_convolution_over_steps_with_state(width, taps, residual, act):
    """Rows before a step's first come from the state, rows before a sequence's first are zero, and a
    step of one row a sequence moves the state on in the same launch."""
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(width + taps)
    lens = {0: 23, 1: 9}
    u = {s: torch.randn(n, width, generator=g) for s, n in lens.items()}
    w = 0.5 * torch.randn(width, taps, generator=g)
    b = torch.randn(width, generator=g) if act else None
    state = torch.zeros((3, 7 + max(taps - 1, 1) * width), device="cuda")

    def call(batch, rows):
        out = torch.empty_like(rows)
        core.seq_conv([dict(u=rows, w=dev(w.t()), bias=dev(b) if b is not None else None, offset=7, out32=out)], state, batch,
                      taps=taps, channels=width, residual=residual, act=act)
        if taps > 1 and not batch.all_decode:
            core.conv_state_update(rows, state, batch, taps=taps, channels=width, offset=7)
        return out

    got = run_cuts(lens, u, call)
    # ... then one row at a time for the longer sequence, which takes the state along in the kernel itself
    more = torch.randn(5, width, generator=g)
    tail = []
    for i in range(5):
        batch = G.make_batch("cuda", [1], [23 + i], [1])
        tail.append(call(batch, dev(more[i:i + 1])).double().cpu())
    for s, n in lens.items():
        x = torch.cat([u[s], more]).double() if s == 0 else u[s].double()
        ref = plain.causal_taps(x, w.double(), b.double() if b is not None else None)
        if act:
            ref = plain.silu(ref)
        if residual:
            ref = ref + x
        have = torch.cat([got[s]] + (tail if s == 0 else []))
        assert float((have - ref).abs().max()) < 1e-5, (s, float((have - ref).abs().max()))
    assert float(state[:, :7].abs().max()) == 0.0          # what lies before the offset is someone else's


@pytest.mark.parametrize("vocab,width,buckets,mp,mc", [(50, 64, 7, 3, 5), (33, 40, 1, 1, 1), (70000, 32, 521, 40503, 65599)])
def test_pair_embedding_takes_the_previous_token_from_the_step_or_the_state(vocab, width, buckets, mp, mc):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(vocab)
    table, pair = torch.randn(vocab, width, generator=g), torch.randn(buckets + 1, width, generator=g)
    nw = 1.0 + 0.2 * torch.randn(width, generator=g)
    toks = {0: torch.randint(0, vocab, (23,), generator=g).tolist(), 1: torch.randint(0, vocab, (9,), generator=g).tolist()}
    state = torch.zeros((3, 1), dtype=torch.int32, device="cuda")
    status = core.new_status("cuda")
    got = {0: [], 1: []}
    for step in CUTS:
        batch = G.make_batch("cuda", [s + 1 for s, _, _ in step], [a for _, a, _ in step], [b - a for _, a, b in step],
                             tokens=[toks[s][a:b] for s, a, b in step])
        x = torch.empty((batch.num_tokens, width), device="cuda")
        core.embed_pair(dev(table), dev(pair), dev(nw), 1e-5, batch, x, state, buckets=buckets, mul_prev=mp, mul_cur=mc,
                        status=status)
        o = 0
        for s, a, b in step:
            got[s].append(x[o:o + b - a].double().cpu())
            o += b - a
    core.check_status(status)
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}, "norm": {"eps": 1e-5}}
    w = {"embed": table.double(), "bigram": pair.double(), "embed.norm": nw.double()}
    for s in toks:
        ref = plain.embedding(cfg, w, toks[s])
        assert float((torch.cat(got[s]) - ref).abs().max()) < 1e-5
    assert state[1:, 0].tolist() == [toks[0][-1], toks[1][-1]]


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("nh,nkv,d,dv,rot", [(4, 2, 32, 16, 16), (2, 2, 16, 48, 16), (3, 1, 24, 40, 0), (1, 1, 64, 64, 8),
                                             (5, 5, 18, 6, 18), (2, 1, 128, 64, 64)])
def test_whole_projection_norm_rotations_and_the_turn_back(bf16, nh, nkv, d, dv, rot):
    """q and k normed over all their channels at once, rotated in halves; values rotated over their whole
    width; and a rotated head turned back by the same position is the head again."""
    from moe_b200.ops import core
    from moe_b200.parts.attention import record_width

    g = torch.Generator().manual_seed(nh * 100 + d)
    D = record_width(d, dv, bf16)
    T, eps, base = 11, 1e-5, 300.0
    proj = torch.randn(T, (nh + nkv) * d + nkv * dv + 3, generator=g)
    qn, kn = 1 + 0.3 * torch.randn(nh * d, generator=g), 1 + 0.3 * torch.randn(nkv * d, generator=g)
    starts = [5, 300]
    batch = G.make_batch("cuda", [1, 2], starts, [4, 7])
    pos = torch.tensor([5, 6, 7, 8] + list(range(300, 307)))
    freq = dev(base ** (-2.0 * torch.arange(rot // 2, dtype=F) / max(rot, 1))) if rot else None
    vfreq = dev(base ** (-2.0 * torch.arange(dv // 2, dtype=F) / dv))
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k, v = (torch.full((T, n, D), 7.0, dtype=dt, device="cuda") for n in (nh, nkv, nkv))
    core.whole_prepare(dev(proj), batch, nh=nh, nkv=nkv, d=d, dv=dv, width=D, q=q, k=k, v=v, q_norm=dev(qn), k_norm=dev(kn),
                       eps=eps, freq=freq, rot=rot, vfreq=vfreq, status=core.new_status("cuda"))
    x = proj.double()
    rq = (plain.unit_rms(x[:, :nh * d], eps) * qn.double()).reshape(T, nh, d)
    rk = (plain.unit_rms(x[:, nh * d:(nh + nkv) * d], eps) * kn.double()).reshape(T, nkv, d)
    rv = x[:, (nh + nkv) * d:(nh + nkv) * d + nkv * dv].reshape(T, nkv, dv)
    if rot:
        rq, rk = plain.rotate_halves(rq, pos, rot, base), plain.rotate_halves(rk, pos, rot, base)
    rv = plain.rotate_halves(rv, pos, dv, base)
    # (an angle is the 32-bit product of position and frequency: its rounding grows with the position)
    tol = 2e-2 if bf16 else 5e-5
    for have, ref, n in ((q, rq, d), (k, rk, d), (v, rv, dv)):
        assert float((have[..., :n].double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
        assert float(have[..., n:].abs().max() if n < D else 0.0) == 0.0
    # the turn back: heads filled with rotated values come out as the values were
    ctx = torch.zeros((T, nh, D), dtype=dt, device="cuda")
    vals = torch.randn(T, nh, dv, generator=g)
    ctx[..., :dv] = dev(plain.rotate_halves(vals.double(), pos, dv, base), dt)
    out = torch.empty((T, nh * dv), dtype=dt, device="cuda")
    core.unrotate_pack(ctx, batch.pos, vfreq, out, nh=nh, dv=dv, width=D)
    assert float((out.double().cpu().reshape(T, nh, dv) - vals.double()).abs().max()) < (4e-2 if bf16 else 3e-4)


def attention_case(bf16, nh, nkv, D, chunk, scale, lens, starts, seed, spike=None):
    """Queries, keys and values for sequences that hold ``starts[i]`` positions in the cache and bring
    ``lens[i]`` more; returns what the kernels need and the plain result per sequence."""
    from moe_b200.cache.kv import KVCache, KVRequest
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(seed)
    dt = torch.bfloat16 if bf16 else torch.float32
    cache = KVCache({0: KVRequest(nkv, D, chunk or None)}, {0: None}, 4096, 8, dt, "cuda")
    bias = torch.randn(nh, generator=g) - 1.0
    slots = [cache.acquire() for _ in lens]
    qs, ks, vs, refs = [], [], [], []
    status = core.new_status("cuda")
    for slot, n_old, n_new in zip(slots, starts, lens):
        n = n_old + n_new
        q, k, v = torch.randn(n, nh, D, generator=g), torch.randn(n, nkv, D, generator=g), torch.randn(n, nkv, D, generator=g)
        if spike is not None:          # one key whose score towers over the others for every query
            j = spike(n_old, n_new)
            q[:, :, 1:] *= 0.2
            k[:, :, 0] = 0.0
            k[j] *= 0.05
            k[j, :, 0], q[:, :, 0] = 9.0, 9.0
        q, k, v = (t.to(dt).double() for t in (q, k, v))
        ref = plain.chunked_sigmoid_attention(q, k, v, scale, chunk, bias.double())
        refs.append(ref[n_old:])
        if n_old:                      # what earlier steps left in the cache
            G.give_pages(cache, slot, n_old)
            b0 = G.make_batch("cuda", [slot], [0], [n_old])
            core.kv_commit(dev(k[:n_old], dt), dev(v[:n_old], dt), cache.view(0), b0, status)
        qs.append(q[n_old:]), ks.append(k[n_old:]), vs.append(v[n_old:])
    for slot, n_old, n_new in zip(slots, starts, lens):
        G.give_pages(cache, slot, n_old + n_new)
    batch = G.make_batch("cuda", slots, starts, lens)
    core.check_status(status)
    return cache, batch, dev(torch.cat(qs), dt), dev(torch.cat(ks), dt), dev(torch.cat(vs), dt), torch.cat(refs), dev(bias), status


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("kernel", ["generic", "tiled", "tc"])
@pytest.mark.parametrize("nh,nkv,D,chunk", [(4, 2, 64, 24), (2, 1, 128, 150), (3, 3, 48, 0), (8, 1, 64, 64), (2, 2, 32, 1)])
def test_sigmoid_weights_in_chunks_in_steps_of_several_tokens(bf16, kernel, nh, nkv, D, chunk):
    """Sequences that go on from the cache (one from the middle of a chunk, one from a chunk's first
    position, one from a page's last) and a fresh one, in one step."""
    from moe_b200.ops import core, tc

    if kernel == "tc" and (not bf16 or D not in (64, 128)):
        pytest.skip("the tensor-core kernel takes bfloat16 records of 64 and 128")
    starts, lens = [37, chunk or 64, 63, 0], [70, 9, 130, 40]
    cache, batch, q, k, v, ref, bias, status = attention_case(bf16, nh, nkv, D, chunk, 0.2, lens, starts, D + chunk)
    out = torch.zeros_like(q)
    kw = dict(nh=nh, window=None, scale=0.2, status=status, chunk=chunk, sink=core.SigmoidWeights(bias))
    if kernel == "generic":
        core.attention_generic(q, k, v, cache.view(0), batch, out, use_local=True, **kw)
    elif kernel == "tiled":
        assert core.attention_tiled(q, k, v, cache.view(0), batch, out, use_local=True, **kw)
    else:
        if not tc.attention_cached(q, k, v, cache.view(0), batch, out, **kw):
            pytest.skip("the tensor-core kernel declines this case")
    core.check_status(status)
    err = float((out.double().cpu() - ref).abs().max()) / float(ref.abs().max())
    assert err < (2e-2 if bf16 else 2e-5), err


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("nh,nkv,D,chunk", [(4, 2, 64, 24), (2, 1, 128, 150), (3, 3, 48, 0), (16, 1, 64, 64), (2, 2, 32, 1),
                                            (32, 2, 128, 200)])
def test_sigmoid_weights_in_chunks_for_single_tokens(bf16, nh, nkv, D, chunk):
    """One new token a sequence over the cache, split along the keys and merged: positions in the
    middle of a chunk, at a chunk's first and last position, far into a long sequence."""
    from moe_b200.ops import core

    c = chunk or 64
    starts = [5, c - 1, c, 2 * c + 3, 700]
    lens = [1] * len(starts)
    cache, batch, q, k, v, ref, bias, status = attention_case(bf16, nh, nkv, D, chunk, 0.15, lens, starts, 7 * D + chunk)
    core.kv_commit(k, v, cache.view(0), batch, status)
    out = torch.zeros_like(q)
    batch.max_end = 1024
    core.attention_decode(q, cache.view(0), batch, out.view(len(starts), -1), nh=nh, window=None, scale=0.15, status=status,
                          chunk=chunk, sink=core.SigmoidWeights(bias))
    core.check_status(status)
    err = float((out.double().cpu() - ref).abs().max()) / float(ref.abs().max())
    assert err < (2e-2 if bf16 else 2e-5), err


@pytest.mark.parametrize("where", ["first of its chunk", "last before the chunk", "far back"])
@pytest.mark.parametrize("decode", [False, True])
def test_a_key_that_towers_is_seen_exactly_where_the_chunk_says(where, decode):
    """One key's score exceeds every other's by far, so the output is that key's value if the key is in
    sight and next to nothing if it is not: just inside the chunk, just outside it, and hundreds of
    positions back where nothing limits the sight."""
    from moe_b200.ops import core

    chunk = 0 if where == "far back" else 100
    n_old, n_new = (499, 1) if decode else (380, 120)
    # queries at positions 380 .. 499 (or 499 alone); chunk 4 starts at 400
    j = {"first of its chunk": 400, "last before the chunk": 399, "far back": 3}[where]

    def spike(a, b):
        return j

    # (in a prompt the key at 400 lies among the step's own keys, the one at 399 among them too; for a
    # single token both lie in the cache)
    cache, batch, q, k, v, ref, bias, status = attention_case(False, 2, 1, 32, chunk, 1.0, [n_new], [n_old], 5, spike=spike)
    out = torch.zeros_like(q)
    kw = dict(nh=2, window=None, scale=1.0, status=status, chunk=chunk, sink=core.SigmoidWeights(bias - 12.0))
    # (with the bias lowered every other key weighs next to nothing)
    if decode:
        core.kv_commit(k, v, cache.view(0), batch, status)
        batch.max_end = 512
        core.attention_decode(q, cache.view(0), batch, out.view(1, -1), **kw)
    else:
        assert core.attention_tiled(q, k, v, cache.view(0), batch, out, use_local=True, **kw)
    core.check_status(status)
    size = out.double().abs().amax(dim=(1, 2)).cpu()          # per query: how large its output is
    first_q = n_old
    for i in range(n_new):
        p = first_q + i
        seen = j <= p and (chunk == 0 or p // chunk == j // chunk)
        if seen:
            assert float(size[i]) > 0.5, (where, p)
        else:
            assert float(size[i]) < 0.1, (where, p)


@pytest.mark.parametrize("heads,groups,n,dv,ng", [(4, 2, 24, 16, 2), (2, 1, 16, 32, 1), (1, 1, 8, 40, 1), (3, 3, 40, 8, 3),
                                                  (2, 1, 64, 64, 2), (2, 2, 130, 48, 4), (1, 1, 300, 16, 1)])
@pytest.mark.parametrize("bf16", [False, True])
def test_state_space_recurrence_and_gated_norm_over_steps(heads, groups, n, dv, ng, bf16):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(heads * 10 + n)
    inner, ch = heads * dv, heads * dv + 2 * groups * n
    lens = {0: 23, 1: 9}
    rows = {s: torch.cat([torch.randn(m, ch, generator=g), torch.randn(m, heads, generator=g), torch.randn(m, inner, generator=g)], 1)
            for s, m in lens.items()}                      # [x B C | dt | z]
    dt_bias, a_log, dsk = torch.randn(heads, generator=g), 0.5 * torch.randn(heads, generator=g), torch.randn(heads, generator=g)
    nw = 1 + 0.2 * torch.randn(inner, generator=g)
    state = torch.zeros((3, 5 + heads * n * dv), device="cuda")
    odt = torch.bfloat16 if bf16 else torch.float32

    def call(batch, r):
        y = torch.zeros((r.shape[0], inner), device="cuda")
        core.ssd_scan(r[:, :ch].contiguous(), r[:, ch:ch + heads], dev(dt_bias), dev(a_log), dev(dsk), state, batch, y,
                      heads=heads, groups=groups, n=n, dv=dv, offset=5)
        out = torch.empty((r.shape[0], inner), dtype=odt, device="cuda")
        core.ssd_finish(y, r[:, ch + heads:], dev(nw), 1e-5, batch, out, norm_groups=ng)
        return out

    got = run_cuts(lens, rows, call)
    grp = torch.arange(heads) // (heads // groups)
    for s, m in lens.items():
        r = rows[s].double()
        xs, B = r[:, :inner].reshape(m, heads, dv), r[:, inner:inner + groups * n].reshape(m, groups, n)
        C = r[:, inner + groups * n:ch].reshape(m, groups, n)
        dt = plain.softplus(r[:, ch:ch + heads] + dt_bias.double())
        S = torch.zeros(heads, n, dv, dtype=F)
        y = torch.zeros(m, heads, dv, dtype=F)
        for t in range(m):
            S = torch.exp(-torch.exp(a_log.double()) * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][grp][:, :, None] * xs[t][:, None, :]
            y[t] = torch.einsum("hn,hnv->hv", C[t][grp], S) + dsk.double()[:, None] * xs[t]
        y = y.reshape(m, inner) * plain.silu(r[:, ch + heads:])
        ref = plain.unit_rms(y.reshape(m, ng, inner // ng), 1e-5).reshape(m, inner) * nw.double()
        err = float((got[s] - ref).abs().max()) / float(ref.abs().max())
        assert err < (1e-2 if bf16 else 2e-5), (s, err)


@pytest.mark.parametrize("heads,groups,n,dv,segments", [(2, 1, 24, 16, 4), (3, 3, 64, 40, 3), (1, 1, 130, 64, 8), (2, 2, 16, 8, 2)])
def test_state_space_recurrence_in_segments_side_by_side(heads, groups, n, dv, segments):
    """Long sequences cut into segments that run side by side give what the chain over all tokens gives:
    two sequences of unequal lengths (one shorter than a segment) that go on from a state left by an
    earlier step, and the state they leave behind."""
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(heads * 7 + n)
    inner, ch = heads * dv, heads * dv + 2 * groups * n
    lens = {0: 50 + 650, 1: 20 + 90}
    rows = {s: torch.cat([torch.randn(m, ch, generator=g), torch.randn(m, heads, generator=g) - 1.0], 1) for s, m in lens.items()}
    dt_bias, a_log, dsk = torch.randn(heads, generator=g), 0.5 * torch.randn(heads, generator=g) - 1.0, torch.randn(heads, generator=g)
    got, states = {}, {}
    for name, segs in (("chain", 1), ("segments", segments)):
        state = torch.zeros((3, heads * n * dv), device="cuda")
        outs = {0: [], 1: []}
        for a0, a1, b0, b1, sg in ((0, 50, 0, 20, 1), (50, 700, 20, 110, segs)):
            batch = G.make_batch("cuda", [1, 2], [a0, b0], [a1 - a0, b1 - b0])
            r = dev(torch.cat([rows[0][a0:a1], rows[1][b0:b1]]))
            y = torch.zeros((r.shape[0], inner), device="cuda")
            core.ssd_scan(r[:, :ch].contiguous(), r[:, ch:], dev(dt_bias), dev(a_log), dev(dsk), state, batch, y, heads=heads,
                          groups=groups, n=n, dv=dv, segments=sg)
            outs[0].append(y[:a1 - a0].double().cpu()), outs[1].append(y[a1 - a0:].double().cpu())
        got[name] = {s: torch.cat(v) for s, v in outs.items()}
        states[name] = state.double().cpu()
    grp = torch.arange(heads) // (heads // groups)
    for s, m in lens.items():
        r = rows[s].double()
        xs, B = r[:, :inner].reshape(m, heads, dv), r[:, inner:inner + groups * n].reshape(m, groups, n)
        C = r[:, inner + groups * n:ch].reshape(m, groups, n)
        dt = plain.softplus(r[:, ch:] + dt_bias.double())
        S = torch.zeros(heads, n, dv, dtype=F)
        ref = torch.zeros(m, heads, dv, dtype=F)
        for t in range(m):
            S = torch.exp(-torch.exp(a_log.double()) * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][grp][:, :, None] * xs[t][:, None, :]
            ref[t] = torch.einsum("hn,hnv->hv", C[t][grp], S) + dsk.double()[:, None] * xs[t]
        scale = float(ref.abs().max())
        for name in got:
            assert float((got[name][s] - ref.reshape(m, inner)).abs().max()) / scale < 2e-5, (name, s)
            assert float((states[name][s + 1].reshape(heads, n, dv) - S).abs().max()) / float(S.abs().max()) < 2e-5, (name, s)


@pytest.mark.parametrize("heads,d,segments", [(2, 32, 4), (3, 64, 3), (1, 80, 8), (2, 16, 2)])
def test_recurrent_scan_in_segments_side_by_side(heads, d, segments):
    """The recurrent mixer's scan cut into segments against the chain over all tokens and against the
    recurrence written out: two sequences of unequal lengths that go on from a state left by an earlier
    step, and the state they leave behind."""
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(heads * 5 + d)
    I = heads * d
    lens = {0: 40 + 660, 1: 30 + 75}
    r = {s: torch.randn(m, I, generator=g) / 4 for s, m in lens.items()}
    k = {s: torch.randn(m, I, generator=g) / 4 for s, m in lens.items()}
    v = {s: torch.randn(m, I, generator=g) for s, m in lens.items()}
    w = {s: torch.exp(-torch.exp(torch.randn(m, I, generator=g) - 2.0)) for s, m in lens.items()}
    u = torch.randn(heads, d, generator=g)
    got, states = {}, {}
    for name, segs in (("chain", 1), ("segments", segments)):
        state = torch.zeros((3, 5 + I * d), device="cuda")
        outs = {0: [], 1: []}
        for a0, a1, b0, b1, sg in ((0, 40, 0, 30, 1), (40, 700, 30, 105, segs)):
            batch = G.make_batch("cuda", [1, 2], [a0, b0], [a1 - a0, b1 - b0])
            cat = lambda t: dev(torch.cat([t[0][a0:a1], t[1][b0:b1]]))
            o = torch.zeros((a1 - a0 + b1 - b0, I), device="cuda")
            core.wkv_scan(cat(r), cat(k), cat(v), cat(w), dev(u), state[:, 5:], batch, o, heads=heads, d=d, segments=sg)
            outs[0].append(o[:a1 - a0].double().cpu()), outs[1].append(o[a1 - a0:].double().cpu())
        got[name] = {s: torch.cat(x) for s, x in outs.items()}
        states[name] = state[:, 5:].double().cpu()
    for s, m in lens.items():
        rr, kk, vv, ww = (t[s].double().reshape(m, heads, d) for t in (r, k, v, w))
        S = torch.zeros(heads, d, d, dtype=F)
        ref = torch.zeros(m, heads, d, dtype=F)
        for t in range(m):
            kv = kk[t][:, :, None] * vv[t][:, None, :]
            ref[t] = torch.einsum("hi,hij->hj", rr[t], S + u.double()[:, :, None] * kv)
            S = ww[t][:, :, None] * S + kv
        scale = float(ref.abs().max())
        for name in got:
            assert float((got[name][s] - ref.reshape(m, I)).abs().max()) / scale < 2e-5, (name, s)
            assert float((states[name][s + 1].reshape(heads, d, d) - S).abs().max()) / float(S.abs().max()) < 2e-5, (name, s)


def test_half_the_sum_of_two_normed_rows_squared_relu_and_the_table():
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(3)
    a, b = torch.randn(9, 72, generator=g), 3 * torch.randn(9, 72, generator=g)
    wa, wb = torch.randn(72, generator=g), torch.randn(72, generator=g)
    out = torch.empty((9, 72), device="cuda")
    core.pair_norm_mean(dev(a), dev(wa), dev(b), dev(wb), 1e-5, out)
    ref = 0.5 * (plain.unit_rms(a.double(), 1e-5) * wa.double() + plain.unit_rms(b.double(), 1e-5) * wb.double())
    assert float((out.double().cpu() - ref).abs().max()) < 1e-5
    z = torch.randn(7, 33, generator=g)
    for dt in (torch.float32, torch.bfloat16):
        act = torch.empty((7, 33), dtype=dt, device="cuda")
        core.relu2(dev(z), act)
        assert float((act.double().cpu() - torch.relu(z.double()) ** 2).abs().max()) < (3e-2 if dt == torch.bfloat16 else 1e-6)
    table = torch.rand(40, 6, generator=g).argsort(dim=1)[:, :3].to(torch.int32)
    toks = [[5, 39, 0], [7]]
    batch = G.make_batch("cuda", [1, 2], [0, 4], [3, 1], tokens=toks)
    idx, wt = torch.empty((4, 3), dtype=torch.int32, device="cuda"), torch.empty((4, 3), device="cuda")
    core.table_route(table.cuda(), batch, 3, 6, idx, wt, core.new_status("cuda"))
    assert idx.cpu().tolist() == [table[t].tolist() for t in (5, 39, 0, 7)]
    assert torch.allclose(wt.cpu(), torch.full((4, 3), 1.0 / 3))


# ----------------------------------------------------------------------------- the model, layer by layer
@pytest.mark.parametrize("name", NAMES)
def test_every_layer_of_a_whole_prompt_in_32_bit(root, name):
    d, eng = engine_of(root, name, "float32", use_graphs=False)
    cfg, w = model_of(d)
    toks = U.tokens(cfg["vocab"], 150, 3)
    ref_layers = []
    plain.forward(cfg, w, toks, ref_layers)
    eng.model.stream_tap = []
    s = eng.new_sequence()
    try:
        eng.step([s], [toks], [[len(toks) - 1]])
        taps = [t.double().cpu() for t in eng.model.stream_tap]
    finally:
        eng.model.stream_tap = None
        eng.release(s)
    assert len(taps) == len(ref_layers)
    for i, (have, ref) in enumerate(zip(taps, ref_layers)):
        err = float((have - ref).abs().max()) / float(ref.abs().max())
        assert err < 3e-5, f"layer {i}: {err:.3g}"


# ----------------------------------------------------------------------------- whole prompts, decoding, portions
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_of_many_lengths(root, name, dtype):
    d, eng = engine_of(root, name, dtype)
    cfg, _ = model_of(d)
    requests = {f"r{n}": U.tokens(cfg["vocab"], n, n) for n in (1, 2, 3, 63, 64, 65, 131, 200)}
    check_schedule(d, eng, requests, helpers.whole_schedule(requests), tol_of(name, dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_decoding_from_the_first_token_on_and_a_prompt_against_its_replay(root, name, dtype):
    """Token by token from position 0 for 150 tokens (chunks and pages pass by, rings wrap), and a prompt
    whose tail is decoded, against the plain implementation and against the whole prompt."""
    d, eng = engine_of(root, name, dtype)
    cfg, _ = model_of(d)
    toks = U.tokens(cfg["vocab"], 150, 5)
    tol = tol_of(name, dtype)
    one = check_schedule(d, eng, {"a": toks}, helpers.tail_schedule({"a": toks}, tail=149), tol)["a"]
    tail = check_schedule(d, eng, {"a": toks}, helpers.tail_schedule({"a": toks}, tail=40), tol)["a"]
    whole = check_schedule(d, eng, {"a": toks}, helpers.whole_schedule({"a": toks}), tol)["a"]
    scale = float(torch.stack(list(whole.values())).abs().max())
    bound = allowed(d, toks, G.tol_cut(dtype) * (3 if name == "sharp" else 1))
    for pos in whole:
        for other in (one, tail):
            assert float((other[pos] - whole[pos]).abs().max()) / scale < float(bound[pos]), pos


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "ones", "wide"])
@pytest.mark.parametrize("sizes", [[2], [3], [63, 2], [64], [65, 1, 1, 7], [129]])
def test_portions_of_several_sizes(root, name, dtype, sizes):
    d, eng = engine_of(root, name, dtype)
    cfg, _ = model_of(d)
    toks = U.tokens(cfg["vocab"], 140 if sizes[0] > 3 else 41, 9)
    check_schedule(d, eng, {"a": toks}, portions_schedule("a", toks, sizes), tol_of(name, dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "lean", "wide"])
def test_unequal_requests_batched_against_each_alone_on_slots_used_again(root, name, dtype):
    """Seven requests of unequal lengths on three slots, twice over (so that slots, pages and state are
    used again), batches of three decoded together; then every request alone."""
    d, eng = engine_of(root, name, dtype, max_slots=3)
    cfg, _ = model_of(d)
    lens = [70, 5, 131, 1, 64, 33, 90]
    requests = {f"q{i}": U.tokens(cfg["vocab"], n, 20 + i) for i, n in enumerate(lens)}
    tol = tol_of(name, dtype)
    for _ in range(2):
        together = check_schedule(d, eng, requests, helpers.batches_schedule(requests, 3, lambda r: max(1, len(requests[r]) - 12)), tol)
    alone = check_schedule(d, eng, requests, helpers.whole_schedule(requests), tol)
    for rid in requests:
        scale = float(torch.stack(list(alone[rid].values())).abs().max())
        bound = allowed(d, requests[rid], G.tol_cut(dtype))
        for pos in together[rid]:
            assert float((together[rid][pos] - alone[rid][pos]).abs().max()) / scale < float(bound[pos]), (rid, pos)


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_that_go_on_from_different_places_in_one_step(root, dtype):
    d, eng = engine_of(root, "mix", dtype)
    cfg, _ = model_of(d)
    a, b, c = (U.tokens(cfg["vocab"], n, 40 + n) for n in (120, 75, 30))
    steps = [
        {"entries": [("a", a[:50], list(range(50)))], "end": []},
        {"entries": [("a", a[50:52], [0, 1]), ("b", b[:64], list(range(64)))], "end": []},
        {"entries": [("a", a[52:119], list(range(67))), ("b", b[64:75], list(range(11))), ("c", c, list(range(30)))], "end": ["b", "c"]},
        {"entries": [("a", a[119:], [0])], "end": ["a"]},
    ]
    check_schedule(d, eng, {"a": a, "b": b, "c": c}, steps, tol_of("mix", dtype))


# ----------------------------------------------------------------------------- edges that random weights would hide
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("place", [3, 63, 64, 400])
def test_a_far_key_among_hundreds(root, dtype, place):
    """A token whose key every query looks at, 140 to 540 positions back, at a page's border or not:
    whole, and with the last 40 tokens decoded.  The plain result changes by much when that token is
    replaced, so a key that is lost shows."""
    d, eng = engine_of(root, "far", dtype, edit_weights=U.spike_token)
    cfg, w = model_of(d)
    special = 0                      # (the token that spike_token marks by default)
    toks = [1 + t % (cfg["vocab"] - 1) for t in U.tokens(cfg["vocab"], 545, 77)]
    toks[place] = special
    ref = plain.forward(cfg, w, toks)
    other = list(toks)
    other[place] = 1
    moved = float((plain.forward(cfg, w, other)[-1] - ref[-1]).abs().max()) / float(ref.abs().max())
    assert moved > 0.05, moved       # the test's premise: the far key matters
    tol = tol_of("far", dtype)
    check_schedule(d, eng, {"a": toks}, helpers.whole_schedule({"a": toks}), tol)
    check_schedule(d, eng, {"a": toks}, helpers.tail_schedule({"a": toks}, tail=40), tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [1, 7, 64, 65, 130])
def test_chunks_one_position_longer_or_shorter(root, dtype, chunk):
    """The same weights with another chunk size: a key just inside a chunk in one model is just outside
    in the next, in prompts and in decoding."""
    def edit(cfg):
        for L in cfg["layers"]:
            L["mixer"]["left"]["mask"] = {"size": chunk}
    edit.__name__ = f"chunk{chunk}"
    d, eng = engine_of(root, "sharp", dtype, edit=edit)
    cfg, _ = model_of(d)
    toks = U.tokens(cfg["vocab"], 200, chunk)
    tol = tol_of("sharp", dtype)
    check_schedule(d, eng, {"a": toks}, helpers.whole_schedule({"a": toks}), tol)
    check_schedule(d, eng, {"a": toks}, helpers.tail_schedule({"a": toks}, tail=70), tol)
    check_schedule(d, eng, {"a": toks}, portions_schedule("a", toks, [chunk + 1, 2, 61]), tol)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(root, dtype):
    d, eng = engine_of(root, "mix", dtype)
    cfg, _ = model_of(d)
    toks = U.tokens(cfg["vocab"], 420, 13)
    steps = [{"entries": [("a", toks[:20], [19])], "end": []}]
    steps += [{"entries": [("a", [toks[i]], [0] if i % 7 == 0 or i > 400 else [])], "end": ["a"] if i == 419 else []}
              for i in range(20, 420)]
    check_schedule(d, eng, {"a": toks}, steps, tol_of("mix", dtype))


# ----------------------------------------------------------------------------- through the library's own entry points
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "lean"])
def test_greedy_generation_through_the_entry_point(root, name, dtype):
    import moe_b200

    d, eng = engine_of(root, name, dtype)
    cfg, w = model_of(d)
    prompts = [U.tokens(cfg["vocab"], n, 60 + n) for n in (9, 1, 70, 33)]
    outs = moe_b200.generate(eng, prompts, max_tokens=12, eos=())
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain.forward(cfg, w, p + o.tokens)[len(p) - 1:-1]
        margin = (2e-4 if dtype == "float32" else 4e-2) * float(ref.abs().max())
        for j, tok in enumerate(o.tokens):
            assert float(ref[j, tok]) >= float(ref[j].max()) - margin, (dtype, j, tok)


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_trace_program_replays_a_mixed_schedule(root, dtype, tmp_path):
    d = U.model_folder(root, "mix")
    cfg, w = model_of(d)
    a, b = U.tokens(cfg["vocab"], 80, 1), U.tokens(cfg["vocab"], 30, 2)
    lines = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:25], "want": [24]}], "end": []}]
    for i in range(5):
        lines.append({"step": 1 + i, "entries": [{"id": "a", "tokens": [a[70 + i]], "want": [0]}, {"id": "b", "tokens": [b[25 + i]], "want": [0]}],
                      "end": ["b"] if i == 4 else []})
    lines.append({"step": 6, "entries": [{"id": "a", "tokens": a[75:], "want": [4]}], "end": ["a"]})
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "256"], input="\n".join(json.dumps(x) for x in lines) + "\n", capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(7)]
    ra, rb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)
    import numpy as np

    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, -1).copy()).double()
    got6 = torch.from_numpy(np.fromfile(out / "6.f32", dtype="<f4").reshape(1, -1).copy()).double()
    tol = tol_of("mix", dtype) * float(ra.abs().max())
    assert float((got0 - torch.stack([ra[0], ra[69], rb[24]])).abs().max()) < tol
    assert float((got6[0] - ra[79]).abs().max()) < tol


def test_command_line_generates_and_traces_the_table_s_picks(root, tmp_path):
    import moe_b200

    d = U.model_folder(root, "mix")
    cfg, w = model_of(d)
    env = dict(os.environ, PYTHONPATH=ROOT)
    run = lambda *a: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "moe"), *a], capture_output=True, text=True,
                                    env=env, timeout=900)
    tr = tmp_path / "routes.jsonl"
    r = run("run", d, "--ids", "5,17,3,9", "-n", "6", "--no-stream", "--dtype", "float32", "--trace", str(tr))
    assert r.returncode == 0, r.stderr[-2000:]
    toks = json.loads(r.stdout.strip().splitlines()[-1])
    _, eng = engine_of(root, "mix", "float32")
    assert moe_b200.generate(eng, [[5, 17, 3, 9]], max_tokens=6)[0].tokens == toks
    recs = [json.loads(x) for x in tr.read_text().splitlines()]
    fed = [5, 17, 3, 9] + toks[:-1]
    routed = [i for i, L in enumerate(cfg["layers"]) if L["mlp"] and L["mlp"]["kind"] == "moe"]
    assert len(recs) == 1 + len(fed) * len(routed)
    for x in recs[1:]:
        table = w[f"l{x['layer']}.mlp.table"]
        top = table.shape[1]
        assert [e for e, _ in x["experts"]] == table[fed[x["pos"]]].tolist()
        assert all(abs(wt - 1.0 / top) < 1e-6 for _, wt in x["experts"])


def test_the_summary_names_the_design_s_parts(root):
    d = U.model_folder(root, "mix")
    r = subprocess.run([sys.executable, "-m", "moe_b200", "info", d], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    for word in ("Divadra", "half the sum", "ssd(", "sigmoid weights", "table over token ids", "causal convolution"):
        assert word in r.stdout, word
