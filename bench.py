#!/usr/bin/env python3
"""Decode and prefill throughput of moe_b200 on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default run: the layer sizes of Qwen1.5-MoE-A2.7B with random bfloat16 weights,
8 sequences with 512-token prompts inside a 4096-token context, K decode steps.
A "step" is one decode step (inputs copied from pinned memory, every layer, the
output projection and a greedy pick).  Prints ONE JSON line.

  value    decoded tokens a second, timed on the device with CUDA events
  e2e      the same through moe_b200.generate(): host token lists in and out
  prefill  one 2,048-token prompt: tokens a second and fraction of the bf16 peak
  roofline bytes a decode step must read (every weight it uses once, and the
           cache of the live requests) / its time, against the measured copy bandwidth
  points   decode at batch 1 and 64

The reference (JGalego/Moe) is a Rust CPU engine; it installs only with a Rust
toolchain, which this image lacks, so ``--impl reference`` reports that.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A27B = dict(
    architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe",
    num_hidden_layers=24, hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, head_dim=128,
    num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408, shared_expert_intermediate_size=5632,
    intermediate_size=5632, norm_topk_prob=False, decoder_sparse_step=1, mlp_only_layers=[],
    vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, use_sliding_window=False, tie_word_embeddings=False,
    max_position_embeddings=8192,
)
FULL_LAYERS = 24
# the larger shape of the same architecture (Qwen2-57B-A14B): only with --sweep, to see other sizes
A57B = dict(A27B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
            num_experts=64, num_experts_per_tok=8, moe_intermediate_size=2560, shared_expert_intermediate_size=20480,
            intermediate_size=18944)
CONTEXT, PROMPT_LEN, PREFILL_TOKENS = 4096, 512, 2048


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        self.rows = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def model_numbers(cfg, layers):
    """Parameter counts and per-token work of the configuration."""
    H, V = cfg["hidden_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    E, k, mi, si = cfg["num_experts"], cfg["num_experts_per_tok"], cfg["moe_intermediate_size"], cfg["shared_expert_intermediate_size"]
    attn = (nh + 2 * nkv) * hd * H + H * nh * hd
    expert = 3 * mi * H
    shared = 3 * si * H + H
    router = E * H
    return dict(attn=attn, expert=expert, shared=shared, router=router, head=V * H,
                kv_bytes_per_token_layer=2 * nkv * hd * 2,
                active_per_token=layers * (attn + k * expert + shared + router))


def run_ours(args):
    import torch

    import moe_b200
    from moe_b200.engine.generate import GenerationStats
    from moe_b200.ops import core
    from moe_b200.sampling.params import SamplingParams
    from moe_b200.sampling.sampler import DeviceSampler

    pk = peaks()
    cfg = dict(A57B if (args.sweep and args.shape == "57b") else A27B)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    torch.cuda.set_device(0)
    model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    V = cfg["vocab_size"]
    nums = model_numbers(cfg, layers)
    clocks = ClockSampler()

    def decode_run(B, steps, warmup, sample_clocks=False, prompt_len=PROMPT_LEN):
        """``prompt_len``: one length for all sequences, or (lo, hi) for unequal lengths drawn from a
        seeded generator.  -> (ms per step, launches per step, h2d bytes per step, mean cache tokens a
        sequence, unique experts per layer, clocks)"""
        if isinstance(prompt_len, tuple):
            import random

            rng = random.Random(B)
            lens = [rng.randint(*prompt_len) for _ in range(B)]
        else:
            lens = [prompt_len] * B
        room = sum(-(-(n + steps + warmup + 8) // 64) * 64 for n in lens)
        eng = moe_b200.Engine(model, max_tokens=room, max_slots=B)
        sampler = DeviceSampler(eng.cache.rng_states, eng.rt.device)
        greedy = SamplingParams()
        slots = [eng.new_sequence() for _ in range(B)]
        prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(lens[b])] for b in range(B)]
        b0 = 0
        while b0 < B:                                   # prompts in groups of at most 4,096 tokens, to bound the workspace
            b1, held = b0, 0
            while b1 < B and (b1 == b0 or held + lens[b1] <= 4096) and b1 - b0 < 8:
                held += lens[b1]
                b1 += 1
            eng.step(slots[b0:b1], prompts[b0:b1], [[] for _ in slots[b0:b1]])
            b0 = b1

        def one(i):
            logits = eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(B)], check=False)
            return sampler.sample(logits, eng.last_batch.slots, greedy)

        for i in range(warmup):
            one(i)
        # which experts a step touches (for the byte count), measured on one extra untimed step
        routed = [b.ffn for b in model.blocks if b.ffn.kind == "routed_experts"]
        for r in routed:
            r.trace = []
        one(warmup)
        uniq = sum(len(torch.unique(r.trace[0][0][:B])) for r in routed) / max(len(routed), 1)   # (rows past B: padding)
        for r in routed:
            r.trace = None
        torch.cuda.synchronize()
        if sample_clocks:
            clocks.start()
        l0 = core.launches
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for i in range(steps):
            one(warmup + 1 + i)
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        clk = clocks.stop() if sample_clocks else None
        eng.rt.check()
        launches = (core.launches - l0) / steps
        mean_len = sum(lens) / B + warmup + 1 + steps / 2
        h2d = (3 * B + 4 * B + 2 + B) * 4
        for s in slots:
            eng.release(s)
        del eng
        torch.cuda.empty_cache()
        return ms, launches, h2d, mean_len, uniq, clk

    def decode_bytes(B, mean_len, uniq):
        per_layer = nums["attn"] + nums["shared"] + nums["router"] + uniq * nums["expert"]
        weights = 2 * (layers * per_layer + nums["head"]) + 2 * B * cfg["hidden_size"]   # bf16, + embedding rows
        kv = B * mean_len * nums["kv_bytes_per_token_layer"] * layers
        return weights + kv

    if args.sweep:
        # decode only, one line per batch size (not the benchmark record)
        for b in [int(v) for v in args.sweep.split(",")]:
            plen = (256, 2048) if args.unequal else (args.prompt_len or PROMPT_LEN)
            m, _, _, mean_len, uniq, _ = decode_run(b, max(8, args.steps // 2), args.warmup, prompt_len=plen)
            nb = decode_bytes(b, mean_len, uniq)
            gbs = nb / (m / 1e3) / 1e9
            print(json.dumps({"shape": args.shape, "layers": layers, "batch": b, "cache_tokens": int(mean_len),
                              "experts_per_layer": round(uniq, 1), "bytes_per_step": int(nb), "ms_per_step": round(m, 4),
                              "tokens_per_s": round(b / (m / 1e3), 1), "hbm_gbs": round(gbs, 1),
                              "hbm_frac": round(gbs / pk["hbm_gbs"], 4)}), flush=True)
        return 0

    # ---- headline: batch 8 ---------------------------------------------------------------
    B = 8
    ms, launches, h2d, mean_len, uniq, clk = decode_run(B, args.steps, args.warmup, sample_clocks=True)
    value = B / (ms / 1e3)
    nbytes = decode_bytes(B, mean_len, uniq)
    achieved = nbytes / (ms / 1e3) / 1e9

    # ---- other batch sizes: at least 64 steps each, with clocks and roofline of their own --------
    points, points_detail = {}, {}
    for b in (1, 64):
        n_steps = max(64, args.steps)
        m, _, _, ml, uq, ck = decode_run(b, n_steps, args.warmup, sample_clocks=True)
        points[f"decode_b{b}"] = round(b / (m / 1e3), 1)
        gbs = decode_bytes(b, ml, uq) / (m / 1e3) / 1e9
        points_detail[f"decode_b{b}"] = {"ms_per_step": round(m, 4), "steps": n_steps, "hbm_gbs": round(gbs, 1),
                                         "hbm_frac": round(gbs / pk["hbm_gbs"], 4), "experts_per_layer": round(uq, 1),
                                         "sm_mhz": ck["sm_mhz"], "reasons": ck["reasons"]}

    # ---- prefill of 2,048 tokens ------------------------------------------------------------
    eng = moe_b200.Engine(model, max_tokens=PREFILL_TOKENS + 64, max_slots=1)
    ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]
    times = []
    for it in range(args.warmup + 5):
        s = eng.new_sequence()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([s], [ids], check=False)
        b_.record()
        torch.cuda.synchronize()
        eng.release(s)
        if it >= args.warmup:
            times.append(a.elapsed_time(b_))
    eng.rt.check()
    pf_ms = sorted(times)[len(times) // 2]
    T = PREFILL_TOKENS
    flops = 2 * T * nums["active_per_token"] + 2 * nums["head"] \
        + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) // 2
    # frac: of the burst peak (a cuBLAS product timed alone); frac_sustained: of the peak of a seconds-long
    # loop under the power cap, which is the state this step is measured in, after the decode runs
    prefill = {"value": round(T / (pf_ms / 1e3), 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "frac_sustained": round(flops / (pf_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}
    del eng
    torch.cuda.empty_cache()

    # ---- end to end through the Python entry point ----------------------------------------
    eng = moe_b200.Engine(model, max_tokens=8 * (-(-(PROMPT_LEN + args.steps + 8) // 64) * 64), max_slots=8)
    prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(PROMPT_LEN)] for b in range(8)]
    moe_b200.generate(eng, prompts, max_tokens=4, eos=())                       # warm-up
    st = GenerationStats()
    moe_b200.generate(eng, prompts, max_tokens=args.steps + 1, eos=(), stats=st)
    e2e = {"value": round(st.decode_tokens / max(st.decode_seconds, 1e-9), 1), "unit": "tokens/s",
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": (8 + 1) * 4,
           "prefill_tokens_per_s": round(st.prefill_tokens / max(st.prefill_seconds, 1e-9), 1)}

    out = {
        "metric": "decode tokens/s (batch 8, Qwen1.5-MoE-A2.7B shape, bf16)", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights N(0, 0.02)",
        "config": {
            "model": "Qwen1.5-MoE-A2.7B shape", "layers": layers, "layers_of_model": FULL_LAYERS, "hidden": 2048,
            "heads": 16, "kv_heads": 16, "head_dim": 128, "experts": 60, "top_k": 4, "moe_intermediate": 1408,
            "shared_intermediate": 5632, "vocab": V, "global_batch": B, "seq_len": CONTEXT, "prompt_len": PROMPT_LEN,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights read per step >> 126 MB)",
            "peaks": pk["source"],
        },
        "clocks": clk,
        "e2e": e2e,
        "gpu_launches": int(round(launches * args.steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": int(nbytes),
                     "experts_per_layer": round(uniq, 1), "of": pk["source"]},
        "points": points,
        "points_detail": points_detail,
    }
    print(json.dumps(out))
    return 0


def run_fp32_long(args):
    """The true 32-bit path at the model's layer sizes and a long context: 8 sequences of unequal
    prompts (4,096 to 24,576 tokens, seeded) inside 32,768 positions, a window of 4,096 on the last
    three layers, then 64 decode steps; and the logits of two of the prompts against the bfloat16
    path on the same (bfloat16-representable) weights.  Prints one JSON line; not the benchmark record."""
    import random

    import torch

    import moe_b200

    pk = peaks()
    cfg = dict(A27B, use_sliding_window=True, sliding_window=4096, max_window_layers=21, max_position_embeddings=32768)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    cfg["max_window_layers"] = max(0, layers - 3)
    V = cfg["vocab_size"]
    rng = random.Random(5)
    lens = [rng.randint(4096, 24576) for _ in range(8)] if not args.prompt_len else [args.prompt_len] * 8
    steps = 64
    model = moe_b200.random_model(cfg, seed=0, dtype="float32", device="cuda:0", stored_dtype="bfloat16")
    room = sum(-(-(n + steps + 8) // 64) * 64 for n in lens)
    eng = moe_b200.Engine(model, max_tokens=room, max_slots=8)
    prompts = [[(i * 7 + 13 + 31 * b) % V for i in range(n)] for b, n in enumerate(lens)]
    slots = [eng.new_sequence() for _ in lens]
    last = {}
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for b in range(8):
        last[b] = eng.step([slots[b]], [prompts[b]]).float().clone()     # (the engine runs it in pieces)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    nums = model_numbers(cfg, layers)
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(3):
        eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(8)], check=False)
    a.record()
    for i in range(steps):
        eng.step(slots, [[(i * 13 + 7 * b + 3) % V] for b in range(8)], check=False)
    z.record()
    torch.cuda.synchronize()
    eng.rt.check()
    ms = a.elapsed_time(z) / steps
    full, win = cfg["max_window_layers"], layers - cfg["max_window_layers"]
    kv_tok = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 4
    mean = [n + 3 + steps / 2 for n in lens]
    kv = kv_tok * (full * sum(mean) + win * sum(min(m, 4096) for m in mean))
    uniq = cfg["num_experts"] * (1 - (1 - cfg["num_experts_per_tok"] / cfg["num_experts"]) ** 8)
    weights = 4 * (layers * (nums["attn"] + nums["shared"] + nums["router"] + uniq * nums["expert"]) + nums["head"])
    gbs = (weights + kv) / (ms / 1e3) / 1e9
    out = {"workload": "float32, context 32768, 8 unequal prompts, 64 decode steps", "layers": layers, "prompt_tokens": lens,
           "prefill_tokens_per_s": round(sum(lens) / prefill_s, 1), "prefill_s": round(prefill_s, 2),
           "decode_ms_per_step": round(ms, 3), "decode_tokens_per_s": round(8 / (ms / 1e3), 1),
           "decode_bytes_per_step": int(weights + kv), "decode_hbm_gbs": round(gbs, 1),
           "decode_hbm_frac": round(gbs / pk["hbm_gbs"], 4)}
    # ---- the bfloat16 path on the same weights: the two shortest prompts' last logits --------------
    for s_ in slots:
        eng.release(s_)
    short = sorted(range(8), key=lambda b: lens[b])[:2]
    del eng
    torch.cuda.empty_cache()
    m16 = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    e16 = moe_b200.Engine(m16, max_tokens=sum(-(-(lens[b] + 8) // 64) * 64 for b in short), max_slots=2)
    worst = []
    for n, b in enumerate(short):
        # the first whole, the second in pieces of 2,048 tokens that go on from the cache (the windowed
        # layers' rings wrap on the way)
        e16.max_step_tokens = 8192 if n == 0 else 2048
        s_ = e16.new_sequence()
        lg = e16.step([s_], [prompts[b]]).float()
        e16.release(s_)
        worst.append(round(float((lg - last[b]).abs().max() / last[b].abs().max()), 5))
    out["bf16_vs_fp32_last_logits_rel"] = max(worst)
    out["bf16_vs_fp32_prompts"] = [lens[b] for b in short]
    out["bf16_vs_fp32_each"] = {"whole": worst[0], "pieces_of_2048": worst[1]}
    print(json.dumps(out))
    return 0


def run_long_prompt(args):
    """One prompt of ``--prompt-len`` tokens (32,768 unless given) in bfloat16 through the engine's
    step, which runs it in pieces of at most 8,192 tokens that go on from the cache.  Prints one JSON
    line; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    cfg = dict(A27B, max_position_embeddings=131072)
    layers = args.layers or cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers
    V = cfg["vocab_size"]
    T = args.prompt_len or 32768
    model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
    eng = moe_b200.Engine(model, max_tokens=-(-T // 64) * 64 + 64, max_slots=1)
    ids = [(i * 7 + 13) % V for i in range(T)]
    times = []
    for it in range(3):
        s = eng.new_sequence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        eng.step([s], [ids], check=False)
        b.record()
        torch.cuda.synchronize()
        eng.rt.check()
        eng.release(s)
        times.append(a.elapsed_time(b))
    ms = sorted(times)[1]
    nums = model_numbers(cfg, layers)
    flops = 2 * T * nums["active_per_token"] + 2 * nums["head"] \
        + layers * 4 * cfg["num_attention_heads"] * cfg["head_dim"] * T * (T + 1) // 2
    print(json.dumps({"workload": "bfloat16, one prompt, pieces of %d tokens" % eng.max_step_tokens, "layers": layers,
                      "prompt_tokens": T, "ms": round(ms, 2), "tokens_per_s": round(T / (ms / 1e3), 1),
                      "tflops": round(flops / (ms / 1e3) / 1e12, 1),
                      "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}))
    return 0


def profile_step(args):
    """A small case for a profiler: the model's layer sizes, few layers, graphs off (every kernel is
    a launch of its own); only the steps between cudaProfilerStart and cudaProfilerStop matter."""
    import torch

    import moe_b200

    cfg = dict(A27B)
    V = cfg["vocab_size"]
    if args.profile_step == "sample":
        # the sampling kernels alone, on random logits of the model's vocabulary: greedy, then a
        # temperature with top-p, then with top-k too
        from moe_b200.ops import core

        B = args.batch
        logits = torch.randn(B, V, device="cuda:0") * 2
        slots = torch.arange(B, dtype=torch.int32, device="cuda:0")
        rng = torch.arange(1, B + 2, dtype=torch.int64, device="cuda:0") * 0x9E3779B97F4A7C15 % (1 << 62) | 1
        out = torch.zeros(B, dtype=torch.int32, device="cuda:0")
        last = torch.zeros(B + 1, dtype=torch.int32, device="cuda:0")

        def run(i):
            core.sample(logits, slots, rng, out, last_token=last)
            core.sample(logits, slots, rng, out, temp=0.8, top_p=0.95, last_token=last)
            core.sample(logits, slots, rng, out, temp=0.8, top_k=40, top_p=0.95, last_token=last)
        model = None
    else:
        cfg["num_hidden_layers"] = args.layers or 2
        model = moe_b200.random_model(cfg, seed=0, dtype=args.dtype, device="cuda:0")
    if args.profile_step == "sample":
        pass
    elif args.profile_step == "decode":
        B = args.batch
        eng = moe_b200.Engine(model, max_tokens=B * 1024, max_slots=B, use_graphs=False)
        slots = [eng.new_sequence() for _ in range(B)]
        eng.step(slots, [[(i * 7 + 31 * b) % V for i in range(PROMPT_LEN)] for b in range(B)], [[] for _ in slots])
        run = lambda i: eng.step(slots, [[(i * 13 + 7 * b) % V] for b in range(B)])
    elif args.profile_step == "chunk":
        # a piece of a long prompt: --prompt-len tokens [2048] that go on from 6,144 tokens in the cache
        n, past = args.prompt_len or PREFILL_TOKENS, 6144
        eng = moe_b200.Engine(model, max_tokens=past + n + 64, max_slots=1, use_graphs=False)
        s = eng.new_sequence()
        eng.step([s], [[(i * 7 + 13) % V for i in range(past)]], [[]])
        ids = [(i * 11 + 5) % V for i in range(n)]

        def run(i):
            eng.step([s], [ids])
            eng.truncate(s, past)
    else:
        eng = moe_b200.Engine(model, max_tokens=PREFILL_TOKENS + 64, max_slots=1, use_graphs=False)
        ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

        def run(i):
            s = eng.new_sequence()
            eng.step([s], [ids])
            eng.release(s)
    for i in range(3):
        run(i)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for i in range(max(1, min(args.steps, 2))):
        run(3 + i)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(f"profiled {args.profile_step} step(s)")
    return 0


# Supevik at sizes that resemble a real model's layers, and beside each the library's closest model at
# equal size: Qwen2 MoE without experts (dense SwiGLU layers), as many layers as the Supevik shape has
# layer RUNS, the same width, heads, head size, feed-forward size, window and vocabulary.
SUPEVIK_SHAPES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, ff=5632, window=1024, rot=64, layers=6,
                  loop=(1, 5, 2), vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, ff=11008, window=2048, rot=64, layers=4,
                  loop=(0, 4, 2), vocab=32768),
}


def supevik_config(sh):
    mixer = {"heads": sh["heads"], "kv_heads": sh["kv_heads"], "dim": sh["dim"], "vdim": sh["vdim"],
             "scale": sh["dim"] ** -0.5, "mask": {"size": sh["window"]},
             "rot": {"dims": sh["rot"], "base": 1e6, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    a, b, t = sh["loop"]
    return {"architecture": "Supevik", "vocab": sh["vocab"], "width": sh["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "loop": {"start": a, "stop": b, "times": t},
            "layers": [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": sh["ff"]}}] * sh["layers"]}


def dense_qwen_config(sh):
    a, b, t = sh["loop"]
    runs = sh["layers"] + (b - a) * (t - 1)
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=runs,
                hidden_size=sh["width"], num_attention_heads=sh["heads"], num_key_value_heads=sh["kv_heads"],
                head_dim=sh["dim"], num_experts=0, intermediate_size=sh["ff"], vocab_size=sh["vocab"], rope_theta=1e6,
                rms_norm_eps=1e-5, use_sliding_window=True, sliding_window=sh["window"], max_window_layers=0,
                tie_word_embeddings=False, max_position_embeddings=8192, qkv_bias=True)


def _median_ms(fn, reps=5, warmup=3):
    import torch

    for _ in range(warmup):
        fn()
    times = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def _graph_ms(fn, calls=10, reps=5):
    """Device time of one call of ``fn`` whose kernels are shorter than the host's work to launch them:
    ``calls`` calls captured in a CUDA graph, the median of ``reps`` replays, divided by ``calls``."""
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for _ in range(calls):
                fn()
    torch.cuda.current_stream().wait_stream(side)
    return _median_ms(g.replay, reps=reps, warmup=2) / calls


def supevik_kernels(sh, pk):
    """The new design's own kernels beside the like kernels of the closest model, each alone at 8,192
    tokens (what a call reads and writes exceeds L2), as a fraction of the measured copy bandwidth
    (products: of the measured bf16 peak)."""
    import torch

    from moe_b200.ops import core, tc

    dev = "cuda:0"
    T, H, nh, nkv, d, I = 8192, sh["width"], sh["heads"], sh["kv_heads"], sh["dim"], sh["ff"]
    status = core.new_status(dev)
    r = lambda *s: torch.randn(*s, device=dev)
    x, delta, w, b, al = r(T, H), r(T, H), r(H), r(H), torch.tensor(0.8, device=dev)
    o16 = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    out = {}

    def row(name, ms, nbytes=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if nbytes:
            e["gb_s"] = round(nbytes / ms / 1e6, 0)
            e["of_copy_peak"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)
        if flops:
            e["tflops"] = round(flops / ms / 1e9, 0)
            e["of_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
        out[name] = e

    nb = T * H * (4 + 4 + 4 + 2)
    row("dyt (norm after + sum + norm before)", _median_ms(lambda: core.dyt(x, (al, w, b), delta=delta, post=(al, w, b), out16=o16, status=status)), nb)
    row("rmsnorm (sum + norm)", _median_ms(lambda: core.rmsnorm(x, w, 1e-5, delta=delta, out16=o16, status=status)), nb)
    wq = (nh + 2 * nkv) * d
    proj = r(T, wq + nh * d)
    qkv = r(T, wq)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    q, k, v = (torch.empty((T, n, d), dtype=torch.bfloat16, device=dev) for n in (nh, nkv, nkv))
    freq = torch.rand(sh["rot"] // 2, device=dev)
    nb = T * wq * (4 + 2)
    row("heads_prepare (q/k norm + rotation + split)", _median_ms(lambda: core.heads_prepare(
        proj, pos, seq, nh=nh, nkv=nkv, d=d, dv=d, width=d, q=q, k=k, v=v, q_norm=w[:d].contiguous(), k_norm=b[:d].contiguous(),
        eps=1e-5, freq=freq, rot=sh["rot"], mscale=1.1, status=status)), nb)
    row("rope_split (rotation + split)", _median_ms(lambda: core.rope_split(qkv, pos, freq, nh, nkv, d, sh["rot"], q, k, v)), nb)
    ctx = torch.empty((T, nh, d), dtype=torch.bfloat16, device=dev)
    packed = torch.empty((T, nh * d), dtype=torch.bfloat16, device=dev)
    row("gate_pack (sigmoid gate on the heads)", _median_ms(lambda: core.gate_pack(ctx, packed, nh=nh, dv=d, width=d, gate=proj[:, wq:])),
        T * nh * d * (2 + 4 + 2))
    a16 = torch.randn(T, H, device=dev).to(torch.bfloat16)
    wgu = (torch.randn(2 * I, H, device=dev) / 32).to(torch.bfloat16)
    act = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
    fl = 2.0 * T * 2 * I * H
    row("gate|up product, gelu_tanh epilogue", _median_ms(lambda: tc.gemm_tc(a16, wgu, act, swiglu=True, status=status, act="gelu_tanh")), flops=fl)
    row("gate|up product, silu epilogue", _median_ms(lambda: tc.gemm_tc(a16, wgu, act, swiglu=True, status=status)), flops=fl)
    core.check_status(status)
    return out


def run_supevik(args):
    """``--workload supevik``: prefill and decode of the Supevik design at two sizes, the closest existing
    model at equal size beside it, and the new kernels beside their counterparts.  One JSON line per
    shape; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    names = [args.shape] if args.shape in SUPEVIK_SHAPES else list(SUPEVIK_SHAPES)
    for name in names:
        sh = SUPEVIK_SHAPES[name]
        V = sh["vocab"]
        res = {"workload": "supevik", "shape": name, "sizes": sh, "dtype": "bfloat16", "data": "synthetic, random weights",
               "peaks": pk}
        for label, cfg in (("supevik", supevik_config(sh)), ("qwen2_dense", dense_qwen_config(sh))):
            model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = {"parameters": int(model.num_parameters)}
            eng = moe_b200.Engine(model, max_tokens=64 * (512 + args.steps + 64) + 4096, max_slots=64)
            ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

            def prefill():
                s = eng.new_sequence()
                eng.step([s], [ids], check=False)
                eng.release(s)

            ms = _median_ms(prefill)
            r["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3, 0)}
            for B in (1, 8, 64):
                slots = [eng.new_sequence() for _ in range(B)]
                eng.step(slots, [ids[:PROMPT_LEN]] * B, check=False)
                for i in range(args.warmup):
                    eng.step(slots, [[i % V]] * B, check=False)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for i in range(args.steps):
                    eng.step(slots, [[(i + 5) % V]] * B, check=False)
                b.record()
                torch.cuda.synchronize()
                eng.rt.check()
                ms = a.elapsed_time(b) / args.steps
                r[f"decode_b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 0)}
                for s in slots:
                    eng.release(s)
            res[label] = r
            del eng, model
            torch.cuda.empty_cache()
        res["kernels_at_8192_tokens"] = supevik_kernels(sh, pk)
        print(json.dumps(res), flush=True)
    return 0


# Fogapel at sizes that resemble a real model's layers, and beside each the library's closest model at
# equal size: Qwen2 MoE with as many layers, the same width, heads, head size, experts, expert and shared
# sizes, first layer dense, and vocabulary (every layer of it is attention; its windows are the chunks' size).
FOGAPEL_SHAPES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=1024, rot=64, taps=4, softcap=30.0,
                  wkv_heads=32, wkv_dim=64, ff=5632, limit=7.0, experts=32, top=4, expert_ff=704, shared_ff=2816,
                  order=("wkv", "wkv", "attention", "wkv", "attention", "wkv"), vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, chunk=2048, rot=64, taps=4, softcap=30.0,
                  wkv_heads=64, wkv_dim=64, ff=11008, limit=7.0, experts=32, top=4, expert_ff=1408, shared_ff=5632,
                  order=("wkv", "attention", "wkv", "attention"), vocab=32768),
}


def fogapel_config(sh):
    att = {"heads": sh["heads"], "kv_heads": sh["kv_heads"], "dim": sh["dim"], "vdim": sh["vdim"], "scale": sh["dim"] ** -0.5,
           "softcap": sh["softcap"], "conv": sh["taps"], "mask": {"size": sh["chunk"]}, "rot": {"dims": sh["rot"], "base": 1e6}}
    wkv = {"heads": sh["wkv_heads"], "dim": sh["wkv_dim"]}
    moe = {"kind": "moe", "router": {"experts": sh["experts"], "top": sh["top"]}, "expert": {"ff": sh["expert_ff"]},
           "shared": {"ff": sh["shared_ff"]}}
    dense = {"kind": "dense", "ff": sh["ff"], "limit": sh["limit"]}
    return {"architecture": "Fogapel", "vocab": sh["vocab"], "width": sh["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5},
            "layers": [{"type": t, "mixer": att if t == "attention" else wkv, "mlp": dense if i == 0 else moe}
                       for i, t in enumerate(sh["order"])]}


def moe_qwen_config(sh):
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=len(sh["order"]),
                hidden_size=sh["width"], num_attention_heads=sh["heads"], num_key_value_heads=sh["kv_heads"],
                head_dim=sh["dim"], num_experts=sh["experts"], num_experts_per_tok=sh["top"],
                moe_intermediate_size=sh["expert_ff"], shared_expert_intermediate_size=sh["shared_ff"],
                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[0], intermediate_size=sh["ff"],
                vocab_size=sh["vocab"], rope_theta=1e6, rms_norm_eps=1e-5, use_sliding_window=True,
                sliding_window=sh["chunk"], max_window_layers=0, tie_word_embeddings=False,
                max_position_embeddings=8192, qkv_bias=True)


def fogapel_kernels(sh, pk):
    """The new design's own kernels beside the like kernels of the closest model, each alone at 8,192
    tokens of 4 sequences (what a call reads and writes exceeds L2), as a fraction of the measured copy
    bandwidth (attention: of the measured bf16 peak, counting the products of the keys a query sees)."""
    import torch

    import moe_b200
    from moe_b200.cache.kv import KVCache, KVRequest
    from moe_b200.ops import core, tc

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import gpu_util as G

    dev = "cuda:0"
    B, n = 4, 2048
    T, H, nh, nkv, d = B * n, sh["width"], sh["heads"], sh["kv_heads"], sh["dim"]
    wh, wd = sh["wkv_heads"], sh["wkv_dim"]
    I = wh * wd
    status = core.new_status(dev)
    r = lambda *s: torch.randn(*s, device=dev)
    out = {}

    def row(name, ms, nbytes=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if nbytes:
            e["gb_s"] = round(nbytes / ms / 1e6, 0)
            e["of_copy_peak"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)
        if flops:
            e["tflops"] = round(flops / ms / 1e9, 0)
            e["of_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
        out[name] = e

    batch = G.make_batch(dev, list(range(1, B + 1)), [0] * B, [n] * B)
    # ---- norms -------------------------------------------------------------------------------------
    x, a, b, w, sa, sb = r(T, H), r(T, H), r(T, H), r(H), r(H), r(H)
    o16 = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
    row("rmsnorm_scaled (two scaled outputs + sum + norm)",
        _median_ms(lambda: core.rmsnorm_scaled(x, a, sa, b, sb, w, 1e-5, out16=o16, status=status)), T * H * (4 + 4 + 4 + 4 + 2))
    row("rmsnorm (sum + norm)", _median_ms(lambda: core.rmsnorm(x, w, 1e-5, delta=a, out16=o16, status=status)), T * H * (4 + 4 + 4 + 2))
    # ---- between projection and attention -------------------------------------------------------------
    wq = (nh + 2 * nkv) * d
    proj = r(T, wq)
    q, k, v = (torch.empty((T, m, d), dtype=torch.bfloat16, device=dev) for m in (nh, nkv, nkv))
    freq = torch.rand(sh["rot"] // 2, device=dev)
    taps_w = r(sh["taps"], wq)
    state = torch.zeros((B + 2, (sh["taps"] - 1) * wq), device=dev)
    row("conv_heads_prepare (convolution + rotation + unit norm + split)", _median_ms(lambda: core.conv_heads_prepare(
        proj, batch, nh=nh, nkv=nkv, d=d, dv=d, width=d, q=q, k=k, v=v, taps_w=taps_w, state=state, eps=1e-5, unit_norm=True,
        freq=freq, rot=sh["rot"], status=status)), T * wq * (4 + 2))
    row("rope_split (rotation + split)", _median_ms(lambda: core.rope_split(proj, batch.pos, freq, nh, nkv, d, sh["rot"], q, k, v)),
        T * wq * (4 + 2))
    # ---- attention of whole prompts: keys a query sees, 4 flops a key and dimension -------------------------
    qq, kk, vv = (torch.randn(T, m, d, device=dev).to(torch.bfloat16) for m in (nh, nkv, nkv))
    ctx = torch.empty((T, nh * d), dtype=torch.bfloat16, device=dev)
    c = sh["chunk"]
    seen_chunk = sum(p % c + 1 for p in range(n)) * B
    seen_window = sum(min(p + 1, c) for p in range(n)) * B
    row("tcgen05 attention, chunks + capped scores + sink", _median_ms(lambda: tc.attention_prefill(
        qq, kk, vv, batch, ctx, nh=nh, nkv=nkv, hd=d, window=None, scale=d ** -0.5, status=status, chunk=c,
        softcap=sh["softcap"], sink=True)), flops=4.0 * seen_chunk * nh * d)
    row("tcgen05 attention, window", _median_ms(lambda: tc.attention_prefill(
        qq, kk, vv, batch, ctx, nh=nh, nkv=nkv, hd=d, window=c, scale=d ** -0.5, status=status)), flops=4.0 * seen_window * nh * d)
    # ---- the recurrent mixer ------------------------------------------------------------------------------
    h32, mu = r(T, H), torch.rand(5, H, device=dev)
    wstate = torch.zeros((B + 2, H + I * wd), device=dev)
    mixed = torch.empty((4, T, H), dtype=torch.bfloat16, device=dev)
    xw = torch.empty((T, H), device=dev)
    row("wkv_shift_mix (five blends)", _median_ms(lambda: core.wkv_shift_mix(h32, mu, wstate, batch, mixed, last32=xw)),
        T * H * (4 + 4 * 2 + 4))
    w1, w2t, w0 = r(16, H) / 32, r(16, I) / 4, r(I) - 1
    decay = torch.empty((T, I), device=dev)
    row("wkv_shift_mix with the decay (blends + two projections + exponentials)",
        _median_ms(lambda: core.wkv_shift_mix(h32, mu, wstate, batch, mixed, decay=(w1, w2t, w0, decay))),
        T * H * (4 + 4 * 2) + T * I * 4)
    rr, kk2, vv2 = r(T, I) / 8, r(T, I) / 8, r(T, I)
    o = torch.empty((T, I), device=dev)
    u = r(wh, wd)
    ms = _median_ms(lambda: core.wkv_scan(rr, kk2, vv2, decay, u, wstate[:, H:], batch, o, heads=wh, d=wd))
    row("wkv_scan (4 sequences of 2,048 tokens)", ms, T * I * 4 * 5, flops=6.0 * T * I * wd)
    out["wkv_scan (4 sequences of 2,048 tokens)"]["us_per_token_of_a_sequence"] = round(ms * 1e3 / n, 3)
    one = G.make_batch(dev, list(range(1, 65)), [n] * 64, [1] * 64)
    st64 = torch.zeros((66, H + I * wd), device=dev)
    r1 = lambda: (r(64, I) / 8)
    a1, b1, c1, d1, o1 = r1(), r1(), r1(), torch.rand(64, I, device=dev), torch.empty((64, I), device=dev)
    row("wkv_scan (one token of 64 sequences: the state read and written)",
        _median_ms(lambda: core.wkv_scan(a1, b1, c1, d1, u, st64[:, H:], one, o1, heads=wh, d=wd)), 64 * I * wd * 4 * 2)
    y = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
    gate, nw = r(T, I), r(I)
    row("wkv_finish (head norm + gate)", _median_ms(lambda: core.wkv_finish(o, gate, nw, 1e-5, batch, y, heads=wh, d=wd)),
        T * I * (4 + 4 + 2))
    # ---- the gated pair in the product's epilogue ----------------------------------------------------------
    a16 = torch.randn(T, H, device=dev).to(torch.bfloat16)
    wgu = (torch.randn(2 * sh["ff"], H, device=dev) / 32).to(torch.bfloat16)
    act = torch.empty((T, sh["ff"]), dtype=torch.bfloat16, device=dev)
    fl = 2.0 * T * 2 * sh["ff"] * H
    row("gate|up product, clamped sigmoid epilogue", _median_ms(lambda: tc.gemm_tc(a16, wgu, act, swiglu=True, status=status,
                                                                                 act="clamped_sigmoid", act_param=sh["limit"])), flops=fl)
    row("gate|up product, silu epilogue", _median_ms(lambda: tc.gemm_tc(a16, wgu, act, swiglu=True, status=status)), flops=fl)
    core.check_status(status)
    return out


def run_fogapel(args):
    """``--workload fogapel``: prefill and decode of the Fogapel design at two sizes, the closest existing
    model at equal size beside it, and the new kernels beside their counterparts.  One JSON line per
    shape; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    names = [args.shape] if args.shape in FOGAPEL_SHAPES else list(FOGAPEL_SHAPES)
    for name in names:
        sh = FOGAPEL_SHAPES[name]
        V = sh["vocab"]
        res = {"workload": "fogapel", "shape": name, "sizes": sh, "dtype": "bfloat16", "data": "synthetic, random weights",
               "peaks": pk}
        for label, cfg in (("fogapel", fogapel_config(sh)), ("qwen2_moe", moe_qwen_config(sh))):
            model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = {"parameters": int(model.num_parameters)}
            eng = moe_b200.Engine(model, max_tokens=64 * (512 + args.steps + 64) + 4096, max_slots=64)
            ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

            def prefill():
                s = eng.new_sequence()
                eng.step([s], [ids], check=False)
                eng.release(s)

            ms = _median_ms(prefill)
            r["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3, 0)}
            for B in (1, 8, 64):
                slots = [eng.new_sequence() for _ in range(B)]
                eng.step(slots, [ids[:PROMPT_LEN]] * B, check=False)
                for i in range(args.warmup):
                    eng.step(slots, [[i % V]] * B, check=False)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for i in range(args.steps):
                    eng.step(slots, [[(i + 5) % V]] * B, check=False)
                b.record()
                torch.cuda.synchronize()
                eng.rt.check()
                ms = a.elapsed_time(b) / args.steps
                r[f"decode_b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 0)}
                for s in slots:
                    eng.release(s)
            res[label] = r
            del eng, model
            torch.cuda.empty_cache()
        res["kernels_at_8192_tokens"] = fogapel_kernels(sh, pk)
        print(json.dumps(res), flush=True)
    return 0


# Divadra at sizes that resemble a real model's layers, and beside each the library's closest model at
# equal size: Fogapel (parallel blocks, chunked attention, the same recurrent mixer, dense and routed
# feed-forwards) with as many layers, the same width, heads, head size, chunks, experts, expert size
# and vocabulary; an attention layer where Divadra runs attention beside the recurrent mixer, a
# recurrent layer where Divadra has the state-space mixer.
DIVADRA_SHAPES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, vdim=128, chunk=1024, rot=64, taps=4, wkv_heads=32, wkv_dim=64,
                  ssd_heads=32, ssd_vdim=64, state=128, groups=1, norm_groups=1, conv=4, ff=5632, experts=32, top=4,
                  expert_ff=704, order=("parallel", "mamba2", "parallel", "parallel", "mamba2", "parallel"), vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, chunk=2048, rot=64, taps=4, wkv_heads=64, wkv_dim=64,
                  ssd_heads=64, ssd_vdim=64, state=128, groups=1, norm_groups=1, conv=4, ff=11008, experts=32, top=4,
                  expert_ff=1408, order=("parallel", "mamba2", "parallel", "mamba2"), vocab=32768),
}


def divadra_config(sh):
    left = {"heads": sh["heads"], "kv_heads": sh["kv_heads"], "dim": sh["dim"], "vdim": sh["vdim"], "scale": sh["dim"] ** -0.5,
            "mask": {"size": sh["chunk"]}, "rot": {"dims": sh["rot"], "base": 1e6}}
    par = {"left": left, "right": {"heads": sh["wkv_heads"], "dim": sh["wkv_dim"]}}
    ssd = {"heads": sh["ssd_heads"], "vdim": sh["ssd_vdim"], "state": sh["state"], "groups": sh["groups"],
           "norm_groups": sh["norm_groups"], "conv": sh["conv"]}
    moe = {"kind": "moe", "router": {"experts": sh["experts"], "top": sh["top"]}, "expert": {"ff": sh["expert_ff"]}}
    dense = {"kind": "dense", "ff": sh["ff"]}
    return {"architecture": "Divadra", "vocab": sh["vocab"], "width": sh["width"], "norm": {"eps": 1e-5},
            "canon": {"taps": sh["taps"]}, "embedding": {"bigram": {"buckets": 65521, "mul_prev": 40503, "mul_cur": 65599}},
            "layers": [{"type": t, "mixer": par if t == "parallel" else ssd, "mlp": dense if i == 0 else moe}
                       for i, t in enumerate(sh["order"])]}


def divadra_fogapel_config(sh):
    att = {"heads": sh["heads"], "kv_heads": sh["kv_heads"], "dim": sh["dim"], "vdim": sh["vdim"], "scale": sh["dim"] ** -0.5,
           "softcap": 30.0, "conv": sh["taps"], "mask": {"size": sh["chunk"]}, "rot": {"dims": sh["rot"], "base": 1e6}}
    wkv = {"heads": sh["wkv_heads"], "dim": sh["wkv_dim"]}
    moe = {"kind": "moe", "router": {"experts": sh["experts"], "top": sh["top"]}, "expert": {"ff": sh["expert_ff"]}}
    dense = {"kind": "dense", "ff": sh["ff"], "limit": 7.0}
    return {"architecture": "Fogapel", "vocab": sh["vocab"], "width": sh["width"], "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5},
            "layers": [{"type": "attention" if t == "parallel" else "wkv", "mixer": att if t == "parallel" else wkv,
                        "mlp": dense if i == 0 else moe} for i, t in enumerate(sh["order"])]}


def divadra_kernels(sh, pk):
    """The new design's own kernels beside the like kernels of the closest model, each alone at 8,192
    tokens of 4 sequences (what a call reads and writes exceeds L2), as a fraction of the measured copy
    bandwidth (attention: of the measured bf16 peak, counting the products of the keys a query sees)."""
    import torch

    from moe_b200.ops import core, tc

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import gpu_util as G

    dev = "cuda:0"
    B, n = 4, 2048
    T, H, nh, nkv, d = B * n, sh["width"], sh["heads"], sh["kv_heads"], sh["dim"]
    status = core.new_status(dev)
    r = lambda *s: torch.randn(*s, device=dev)
    out = {}

    def row(name, ms, nbytes=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if nbytes:
            e["gb_s"] = round(nbytes / ms / 1e6, 0)
            e["of_copy_peak"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)
        if flops:
            e["tflops"] = round(flops / ms / 1e9, 0)
            e["of_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
        out[name] = e

    ids = torch.randint(0, sh["vocab"], (T,)).tolist()
    batch = G.make_batch(dev, list(range(1, B + 1)), [0] * B, [n] * B, tokens=[ids[i * n:(i + 1) * n] for i in range(B)])
    one = G.make_batch(dev, list(range(1, 65)), [n] * 64, [1] * 64)
    # ---- embedding ----------------------------------------------------------------------------------
    table = (torch.randn(sh["vocab"], H, device=dev)).to(torch.bfloat16)
    pair = (torch.randn(65522, H, device=dev)).to(torch.bfloat16)
    x, w = torch.empty((T, H), device=dev), r(H)
    prev = torch.zeros((B + 2, 1), dtype=torch.int32, device=dev)
    row("embed_pair (two rows + norm)", _median_ms(lambda: core.embed_pair(table, pair, w, 1e-5, batch, x, prev, buckets=65521,
        mul_prev=40503, mul_cur=65599, status=status)), T * H * (2 + 2 + 4))
    row("embed (one row)", _median_ms(lambda: core.embed(table, batch.token_ids, x, status)), T * H * (2 + 4))
    # ---- norms and the input convolutions ---------------------------------------------------------------
    a, b, ones = r(T, H), r(T, H), torch.ones(H, device=dev)
    o16, o16b = (torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(2))
    o32, o32b = torch.empty((T, H), device=dev), torch.empty((T, H), device=dev)
    row("rmsnorm_scaled (two outputs + sum + norm; the closest model's one norm a layer)",
        _median_ms(lambda: core.rmsnorm_scaled(x, a, ones, b, ones, w, 1e-5, out16=o16, status=status)), T * H * (4 + 4 + 4 + 4 + 2))
    row("rmsnorm (the second norm of the same stream)", _median_ms(lambda: core.rmsnorm(x, w, 1e-5, out32=o32, write_back=False, status=status)),
        T * H * (4 + 4))
    cstate = torch.zeros((B + 2, 2 * (sh["taps"] - 1) * H), device=dev)
    tw = r(sh["taps"], H)
    jobs = [dict(u=o32, w=tw, bias=None, offset=0, out32=a, out16=o16), dict(u=o32b, w=tw, bias=None, offset=(sh["taps"] - 1) * H, out16=o16b)]
    row("seq_conv (both sublayers' inputs: h + conv(h))", _median_ms(lambda: core.seq_conv(jobs, cstate, batch, taps=sh["taps"], channels=H,
        residual=True)), T * H * (4 + 4 + 2 + 4 + 2))
    # ---- between projection and attention -------------------------------------------------------------
    wq = (nh + 2 * nkv) * d
    proj = r(T, wq)
    q, k, v = (torch.empty((T, m, d), dtype=torch.bfloat16, device=dev) for m in (nh, nkv, nkv))
    freq, vfreq = torch.rand(sh["rot"] // 2, device=dev), torch.rand(d // 2, device=dev)
    qn, kn = r(nh * d), r(nkv * d)
    row("whole_prepare (norm over the projection + rotations of q, k, v + split)", _median_ms(lambda: core.whole_prepare(
        proj, batch, nh=nh, nkv=nkv, d=d, dv=d, width=d, q=q, k=k, v=v, q_norm=qn, k_norm=kn, eps=1e-5, freq=freq, rot=sh["rot"],
        vfreq=vfreq, status=status)), T * wq * (4 + 2))
    taps_w = r(sh["taps"], wq)
    state = torch.zeros((B + 2, (sh["taps"] - 1) * wq), device=dev)
    row("conv_heads_prepare (the closest model's: convolution + rotation + unit norm + split)", _median_ms(lambda: core.conv_heads_prepare(
        proj, batch, nh=nh, nkv=nkv, d=d, dv=d, width=d, q=q, k=k, v=v, taps_w=taps_w, state=state, eps=1e-5, unit_norm=True,
        freq=freq, rot=sh["rot"], status=status)), T * wq * (4 + 2))
    # ---- attention of whole prompts: keys a query sees, 4 flops a key and dimension -------------------------
    qq, kk, vv = (torch.randn(T, m, d, device=dev).to(torch.bfloat16) for m in (nh, nkv, nkv))
    ctx = torch.empty((T, nh, d), dtype=torch.bfloat16, device=dev)
    c = sh["chunk"]
    seen = sum(p % c + 1 for p in range(n)) * B
    hb = r(nh)
    row("tcgen05 attention, chunks + sigmoid weights", _median_ms(lambda: tc.attention_prefill(
        qq, kk, vv, batch, ctx, nh=nh, nkv=nkv, hd=d, window=None, scale=d ** -0.5, status=status, chunk=c,
        sink=core.SigmoidWeights(hb))), flops=4.0 * seen * nh * d)
    row("tcgen05 attention, chunks + capped scores + sink (the closest model's)", _median_ms(lambda: tc.attention_prefill(
        qq, kk, vv, batch, ctx, nh=nh, nkv=nkv, hd=d, window=None, scale=d ** -0.5, status=status, chunk=c, softcap=30.0,
        sink=True)), flops=4.0 * seen * nh * d)
    packed = torch.empty((T, nh * d), dtype=torch.bfloat16, device=dev)
    row("unrotate_pack (the turn back of the heads' outputs)", _median_ms(lambda: core.unrotate_pack(ctx, batch.pos, vfreq, packed, nh=nh,
        dv=d, width=d)), T * nh * d * (2 + 2))
    # ---- single tokens over the cache ---------------------------------------------------------------------
    # ---- the two mixers' outputs into one --------------------------------------------------------------------
    row("pair_norm_mean (two norms + half the sum)", _median_ms(lambda: core.pair_norm_mean(a, w, b, w, 1e-5, o32)), T * H * 12)
    # ---- the state-space mixer beside the recurrent one ------------------------------------------------------
    sheads, sdv, N, G_ = sh["ssd_heads"], sh["ssd_vdim"], sh["state"], sh["groups"]
    inner, ch = sheads * sdv, sheads * sdv + 2 * G_ * sh["state"]
    pin = r(T, 2 * inner + 2 * G_ * N + sheads)
    xbc = torch.empty((T, ch), device=dev)
    sstate = torch.zeros((B + 2, (sh["conv"] - 1) * ch + sheads * N * sdv), device=dev)
    cw, cb = r(sh["conv"], ch), r(ch)
    row("seq_conv with bias and silu (x, B, C of the state-space mixer)", _median_ms(lambda: core.seq_conv(
        [dict(u=pin[:, inner:inner + ch], w=cw, bias=cb, offset=0, out32=xbc)], sstate, batch, taps=sh["conv"], channels=ch, act="silu")),
        T * ch * 8)
    dtb, alog, dsk = r(sheads), r(sheads) - 1, r(sheads)
    y = torch.empty((T, inner), device=dev)
    off = (sh["conv"] - 1) * ch
    ms = _median_ms(lambda: core.ssd_scan(xbc, pin[:, inner + ch:], dtb, alog, dsk, sstate, batch, y, heads=sheads, groups=G_, n=N,
                                          dv=sdv, offset=off, segments=1))
    row("ssd_scan (4 sequences of 2,048 tokens)", ms, T * (ch + inner) * 4, flops=4.0 * T * inner * N)
    # one sequence alone: the chain over its tokens, and the same cut into segments that run side by side
    b1 = G.make_batch(dev, [1], [0], [n])
    for label, segs in (("in one chain", 1), ("in 8 segments side by side", 8)):
        row(f"ssd_scan (one sequence of 2,048 tokens, {label})", _median_ms(lambda: core.ssd_scan(
            xbc[:n], pin[:n, inner + ch:], dtb, alog, dsk, sstate, b1, y[:n], heads=sheads, groups=G_, n=N, dv=sdv, offset=off,
            segments=segs)), n * (ch + inner) * 4)
    out["ssd_scan (4 sequences of 2,048 tokens)"]["us_per_token_of_a_sequence"] = round(ms * 1e3 / n, 3)
    st64 = torch.zeros((66, off + sheads * N * sdv), device=dev)
    x1, p1, y1 = r(64, ch), r(64, 2 * inner + 2 * G_ * N + sheads), torch.empty((64, inner), device=dev)
    row("ssd_scan (one token of 64 sequences: the state read and written)", _median_ms(lambda: core.ssd_scan(
        x1, p1[:, inner + ch:], dtb, alog, dsk, st64, one, y1, heads=sheads, groups=G_, n=N, dv=sdv, offset=off)),
        64 * sheads * N * sdv * 4 * 2)
    y16 = torch.empty((T, inner), dtype=torch.bfloat16, device=dev)
    nw = r(inner)
    row("ssd_finish (gate + norm)", _median_ms(lambda: core.ssd_finish(y, pin[:, :inner], nw, 1e-5, batch, y16, norm_groups=sh["norm_groups"])),
        T * inner * (4 + 4 + 2))
    wh, wd = sh["wkv_heads"], sh["wkv_dim"]
    I = wh * wd
    rr, kk2, vv2, decay = r(T, I) / 8, r(T, I) / 8, r(T, I), torch.rand(T, I, device=dev)
    o, u = torch.empty((T, I), device=dev), r(wh, wd)
    wstate = torch.zeros((B + 2, H + I * wd), device=dev)
    ms = _median_ms(lambda: core.wkv_scan(rr, kk2, vv2, decay, u, wstate[:, H:], batch, o, heads=wh, d=wd, segments=1))
    row("wkv_scan (the recurrent mixer's, 4 sequences of 2,048 tokens)", ms, T * I * 4 * 5, flops=6.0 * T * I * wd)
    for label, segs in (("in one chain", 1), ("in 8 segments side by side", 8)):
        row(f"wkv_scan (one sequence of 2,048 tokens, {label})", _median_ms(lambda: core.wkv_scan(
            rr[:n], kk2[:n], vv2[:n], decay[:n], u, wstate[:, H:], b1, o[:n], heads=wh, d=wd, segments=segs)), n * I * 4 * 5)
    out["wkv_scan (the recurrent mixer's, 4 sequences of 2,048 tokens)"]["us_per_token_of_a_sequence"] = round(ms * 1e3 / n, 3)
    st64w = torch.zeros((66, H + I * wd), device=dev)
    r1 = lambda: (r(64, I) / 8)
    a1, b1, c1, d1, o1 = r1(), r1(), r1(), torch.rand(64, I, device=dev), torch.empty((64, I), device=dev)
    row("wkv_scan (one token of 64 sequences: the state read and written)",
        _median_ms(lambda: core.wkv_scan(a1, b1, c1, d1, u, st64w[:, H:], one, o1, heads=wh, d=wd)), 64 * I * wd * 4 * 2)
    yw = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
    gate, nww = r(T, I), r(I)
    row("wkv_finish (the recurrent mixer's head norm + gate)", _median_ms(lambda: core.wkv_finish(o, gate, nww, 1e-5, batch, yw, heads=wh, d=wd)),
        T * I * (4 + 4 + 2))
    # ---- the dense feed-forward's first product and activation ----------------------------------------------
    a16 = torch.randn(T, H, device=dev).to(torch.bfloat16)
    wup = (torch.randn(sh["ff"], H, device=dev) / 32).to(torch.bfloat16)
    wgu = (torch.randn(2 * sh["ff"], H, device=dev) / 32).to(torch.bfloat16)
    act = torch.empty((T, sh["ff"]), dtype=torch.bfloat16, device=dev)

    def up_relu2():
        from moe_b200.parts.feedforward import relu2_linear

        relu2_linear(_Rt(status), a16, wup, act)

    row("up product with the squared relu", _median_ms(up_relu2), flops=2.0 * T * sh["ff"] * H)
    row("gate|up product, clamped sigmoid epilogue (the closest model's)", _median_ms(lambda: tc.gemm_tc(
        a16, wgu, act, swiglu=True, status=status, act="clamped_sigmoid", act_param=7.0)), flops=2.0 * T * 2 * sh["ff"] * H)
    # ---- the experts' choice -------------------------------------------------------------------------------------
    tbl = torch.rand(sh["vocab"], sh["experts"], device=dev).argsort(dim=1)[:, :sh["top"]].to(torch.int32).contiguous()
    idx, wt = torch.empty((T, sh["top"]), dtype=torch.int32, device=dev), torch.empty((T, sh["top"]), device=dev)
    row("table_route (experts by token id)", _median_ms(lambda: core.table_route(tbl, batch, sh["top"], sh["experts"], idx, wt, status)),
        T * sh["top"] * 12)
    core.check_status(status)
    return out


class _Rt:
    """What ``ops.linear`` asks of a runtime, for calling a product outside a model."""

    is_bf16 = True

    def __init__(self, status):
        import torch

        self.status, self.compute_dtype = status, torch.bfloat16


def run_divadra(args):
    """``--workload divadra``: prefill and decode of the Divadra design at two sizes, the closest existing
    model at equal size beside it, and the new kernels beside their counterparts.  One JSON line per
    shape; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    names = [args.shape] if args.shape in DIVADRA_SHAPES else list(DIVADRA_SHAPES)
    for name in names:
        sh = DIVADRA_SHAPES[name]
        V = sh["vocab"]
        res = {"workload": "divadra", "shape": name, "sizes": sh, "dtype": "bfloat16", "data": "synthetic, random weights",
               "peaks": pk}
        for label, cfg in (("divadra", divadra_config(sh)), ("fogapel", divadra_fogapel_config(sh))):
            model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = {"parameters": int(model.num_parameters)}
            eng = moe_b200.Engine(model, max_tokens=64 * (512 + args.steps + 64) + 4096, max_slots=64)
            ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

            def prefill():
                s = eng.new_sequence()
                eng.step([s], [ids], check=False)
                eng.release(s)

            ms = _median_ms(prefill)
            r["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3, 0)}
            for B in (1, 8, 64):
                slots = [eng.new_sequence() for _ in range(B)]
                eng.step(slots, [ids[:PROMPT_LEN]] * B, check=False)
                for i in range(args.warmup):
                    eng.step(slots, [[i % V]] * B, check=False)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for i in range(args.steps):
                    eng.step(slots, [[(i + 5) % V]] * B, check=False)
                b.record()
                torch.cuda.synchronize()
                eng.rt.check()
                ms = a.elapsed_time(b) / args.steps
                r[f"decode_b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 0)}
                for s in slots:
                    eng.release(s)
            res[label] = r
            del eng, model
            torch.cuda.empty_cache()
        res["kernels_at_8192_tokens"] = divadra_kernels(sh, pk)
        print(json.dumps(res), flush=True)
    return 0


# Zosipel at sizes that resemble a real model's layers, and beside each the library's closest model at
# equal size: Qwen2 MoE with as many layers as the Zosipel shape has layer RUNS, the same width, heads,
# experts, expert and shared sizes and vocabulary, every layer routed, heads of twice a map's size (a
# differential head is two maps), windows of the same size on every layer.
ZOSIPEL_SHAPES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=64, vdim=128, window=1024, rot=64, softcap=30.0, diff=0.3,
                  lat_heads=16, lat_dim=128, lat_vdim=128, rank=128, experts=32, top=4, groups=(8, 4), expert_ff=704,
                  shared_ff=2816, order=("latent_attention", "attention", "latent_attention", "latent_attention", "attention",
                                         "latent_attention"), loop=(1, 3, 2), vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=64, vdim=128, window=2048, rot=64, softcap=30.0, diff=0.3,
                  lat_heads=32, lat_dim=128, lat_vdim=128, rank=128, experts=32, top=4, groups=(8, 4), expert_ff=1408,
                  shared_ff=5632, order=("latent_attention", "attention", "latent_attention", "attention"), loop=(0, 2, 2),
                  vocab=32768),
}


def zosipel_config(sh):
    att = {"heads": sh["heads"], "kv_heads": sh["kv_heads"], "dim": sh["dim"], "vdim": sh["vdim"], "scale": sh["dim"] ** -0.5,
           "softcap": sh["softcap"], "diff": sh["diff"], "mask": {"size": sh["window"]},
           "rot": {"dims": sh["rot"], "base": 1e6, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    lat = {"heads": sh["lat_heads"], "dim": sh["lat_dim"], "vdim": sh["lat_vdim"], "kv_rank": sh["rank"],
           "scale": sh["lat_dim"] ** -0.5}
    moe = {"kind": "moe", "router": {"experts": sh["experts"], "top": sh["top"],
                                     "groups": {"count": sh["groups"][0], "keep": sh["groups"][1]}},
           "expert": {"ff": sh["expert_ff"]}, "shared": {"ff": sh["shared_ff"]}}
    a, b, t = sh["loop"]
    return {"architecture": "Zosipel", "vocab": sh["vocab"], "width": sh["width"], "norm": {"eps": 1e-5},
            "loop": {"start": a, "stop": b, "times": t},
            "layers": [{"type": t_, "mixer": att if t_ == "attention" else lat, "mlp": moe} for t_ in sh["order"]]}


def zosipel_qwen_config(sh):
    a, b, t = sh["loop"]
    runs = len(sh["order"]) + (b - a) * (t - 1)
    return dict(architectures=["Qwen2MoeForCausalLM"], model_type="qwen2_moe", num_hidden_layers=runs,
                hidden_size=sh["width"], num_attention_heads=sh["heads"], num_key_value_heads=sh["kv_heads"],
                head_dim=2 * sh["dim"], num_experts=sh["experts"], num_experts_per_tok=sh["top"],
                moe_intermediate_size=sh["expert_ff"], shared_expert_intermediate_size=sh["shared_ff"],
                norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[], intermediate_size=sh["shared_ff"],
                vocab_size=sh["vocab"], rope_theta=1e6, rms_norm_eps=1e-5, use_sliding_window=True,
                sliding_window=sh["window"], max_window_layers=0, tie_word_embeddings=False,
                max_position_embeddings=8192, qkv_bias=True)


def zosipel_kernels(sh, pk):
    """The new design's own kernels beside the like kernels of the closest model, each alone at 8,192
    tokens of 4 sequences (what a call reads and writes exceeds L2), as a fraction of the measured copy
    bandwidth (attention and products: of the measured bf16 peak, counting the products the mechanism
    needs, not the zero-filled part of a record); then the attention of one token of 64 sequences at a
    context of 2,048 (the cache read once; ten calls replayed from a CUDA graph, since a call's kernels
    are shorter than the host's work to launch them)."""
    import torch

    from moe_b200.cache.kv import KVCache, KVRequest
    from moe_b200.ops import core, tc
    from moe_b200.ops.linear import grouped_linear
    from moe_b200.parts.base import Runtime

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import gpu_util as G

    dev = "cuda:0"
    bf = torch.bfloat16
    B, n = 4, 2048
    T, W = B * n, sh["width"]
    H, Gk, d, dv, win = sh["heads"], sh["kv_heads"], sh["dim"], sh["vdim"], sh["window"]
    LH, ld_, lv, rk = sh["lat_heads"], sh["lat_dim"], sh["lat_vdim"], sh["rank"]
    status = core.new_status(dev)
    rt = Runtime(dev, bf)
    r = lambda *s: torch.randn(*s, device=dev)
    out = {}

    def row(name, ms, nbytes=None, flops=None):
        e = {"us": round(ms * 1e3, 1)}
        if nbytes:
            e["gb_s"] = round(nbytes / ms / 1e6, 0)
            e["of_copy_peak"] = round(nbytes / ms / 1e6 / pk["hbm_gbs"], 3)
        if flops:
            e["tflops"] = round(flops / ms / 1e9, 0)
            e["of_bf16_peak"] = round(flops / ms / 1e9 / pk["bf16_tflops"], 3)
        out[name] = e

    batch = G.make_batch(dev, list(range(1, B + 1)), [0] * B, [n] * B)
    freq = torch.rand(sh["rot"] // 2, device=dev)
    # ---- between projection and attention -------------------------------------------------------------
    D = max(2 * d, dv)                                   # one record width for maps and values, as the part chooses it
    nh2, nkv2 = 2 * H, 2 * Gk
    cols = (nh2 + nkv2) * d + nkv2 * dv + H
    proj = r(T, cols)
    q, k, v = (torch.empty((T, m, D), dtype=bf, device=dev) for m in (nh2, nkv2, nkv2))
    row("heads_prepare (rotation of both maps + split into records)", _median_ms(lambda: core.heads_prepare(
        proj, batch.pos, batch.seq_of_token, nh=nh2, nkv=nkv2, d=d, dv=dv, width=D, q=q, k=k, v=v, freq=freq, rot=sh["rot"],
        mscale=1.1, status=status)), T * (cols - H) * 4 + T * (nh2 + 2 * nkv2) * D * 2)
    wq = (H + 2 * Gk) * 2 * d
    qkv = r(T, wq)
    q1, k1, v1 = (torch.empty((T, m, 2 * d), dtype=bf, device=dev) for m in (H, Gk, Gk))
    row("rope_split (rotation + split)", _median_ms(lambda: core.rope_split(qkv, batch.pos, freq, H, Gk, 2 * d, sh["rot"], q1, k1, v1)),
        T * wq * (4 + 2))
    lproj = r(T, LH * ld_ + rk)
    q_t = torch.empty((LH, T, ld_), dtype=bf, device=dev)
    k_new = torch.empty((T, 1, rk), dtype=bf, device=dev)
    wn = r(rk)
    row("latent_prepare (latent norm + record + queries head by head)", _median_ms(lambda: core.latent_prepare(
        lproj, batch, nh=LH, d=ld_, r=rk, width=rk, weight=wn, eps=1e-5, q_t=q_t, k_new=k_new, status=status)),
        T * (LH * ld_ + rk) * (4 + 2))
    qc = r(LH, T, rk)
    ql = torch.empty((T, LH, rk), dtype=bf, device=dev)
    row("heads_transpose (32-bit [heads, tokens] -> 16-bit [tokens, heads])", _median_ms(lambda: core.heads_transpose(qc, ql, n=rk)),
        T * LH * rk * (4 + 2))
    # ---- attention of whole prompts: keys a query sees, 4 flops a key and dimension of the mechanism -------
    seen = sum(min(p + 1, win) for p in range(n)) * B
    causal = n * (n + 1) // 2 * B
    qq, kk, vv = (torch.randn(T, m, D, device=dev).to(bf) for m in (nh2, nkv2, nkv2))
    ctx = torch.empty((T, nh2, D), dtype=bf, device=dev)
    row("tcgen05 attention, two maps a head (window + capped scores)", _median_ms(lambda: tc.attention_prefill(
        qq, kk, vv, batch, ctx, nh=nh2, nkv=nkv2, hd=D, window=win, scale=d ** -0.5, status=status, softcap=sh["softcap"])),
        flops=2.0 * seen * nh2 * (d + dv))
    qs, ks, vs = (torch.randn(T, m, 2 * d, device=dev).to(bf) for m in (H, Gk, Gk))
    ctx1 = torch.empty((T, H, 2 * d), dtype=bf, device=dev)
    row("tcgen05 attention, window", _median_ms(lambda: tc.attention_prefill(
        qs, ks, vs, batch, ctx1, nh=H, nkv=Gk, hd=2 * d, window=win, scale=d ** -0.5, status=status)), flops=4.0 * seen * H * 2 * d)
    sinks = r(LH)
    lq, lk = torch.randn(T, LH, rk, device=dev).to(bf), torch.randn(T, 1, rk, device=dev).to(bf)
    lctx = torch.empty((T, LH, rk), dtype=bf, device=dev)
    row("tcgen05 attention over latents (all heads on one record, sink a head)", _median_ms(lambda: tc.attention_prefill(
        lq, lk, lk, batch, lctx, nh=LH, nkv=1, hd=rk, window=None, scale=ld_ ** -0.5, status=status, sink=sinks)),
        flops=4.0 * causal * LH * rk)
    row("tcgen05 attention, causal", _median_ms(lambda: tc.attention_prefill(
        qs, ks, vs, batch, ctx1, nh=H, nkv=Gk, hd=2 * d, window=None, scale=d ** -0.5, status=status)), flops=4.0 * causal * H * 2 * d)
    # ---- after attention ---------------------------------------------------------------------------------
    packed = torch.empty((T, H * dv), dtype=bf, device=dev)
    row("diff_combine (difference + head norm + gate + pack)", _median_ms(lambda: core.diff_combine(
        ctx, packed, nh=H, dv=dv, width=D, lam=0.4, eps=1e-5, mult=0.7, gate=proj[:, cols - H:])), T * H * dv * (2 + 2 + 2))
    row("gate_pack (sigmoid gate on the heads)", _median_ms(lambda: core.gate_pack(ctx1, packed, nh=H, dv=2 * d, width=2 * d,
                                                                                  gate=proj[:, :H * 2 * d])), T * H * 2 * d * (2 + 4 + 2))
    # ---- the per-head products of latent attention (a group a head) ----------------------------------------
    offsets = (torch.arange(0, LH + 1, dtype=torch.int32, device=dev) * T).contiguous()
    w_qc = (torch.randn(LH, rk, ld_, device=dev) / 16).to(bf)
    row("queries onto the latent (grouped product, a group a head)",
        _median_ms(lambda: grouped_linear(rt, q_t.view(LH * T, ld_), w_qc, offsets, LH * T)), T * LH * (ld_ * 2 + rk * 4),
        flops=2.0 * T * LH * ld_ * rk)
    I = sh["expert_ff"]
    xs = torch.randn(T * sh["top"], W, device=dev).to(bf)
    w_e = (torch.randn(sh["experts"], 2 * I, W, device=dev) / 32).to(bf)
    eo = (torch.arange(0, sh["experts"] + 1, dtype=torch.int32, device=dev) * (T * sh["top"] // sh["experts"])).contiguous()
    row("experts' gate|up (grouped product, a group an expert)",
        _median_ms(lambda: grouped_linear(rt, xs, w_e, eo, T * sh["top"])), flops=2.0 * T * sh["top"] * 2 * I * W)
    # ---- the router's pick ---------------------------------------------------------------------------------
    E, top = sh["experts"], sh["top"]
    logits = r(T, E)
    idx = torch.empty((T, top), dtype=torch.int32, device=dev)
    wt = torch.empty((T, top), dtype=torch.float32, device=dev)
    nb = T * (E * 4 + top * 8)
    row("router pick within the best groups", _median_ms(lambda: core.router_topk(
        logits, top, True, 1.0, idx, wt, num_experts=E, groups=sh["groups"][0], keep=sh["groups"][1])), nb)
    row("router pick", _median_ms(lambda: core.router_topk(logits, top, True, 1.0, idx, wt, num_experts=E)), nb)
    # ---- one token of 64 sequences at a context of 2,048: the cache read once ---------------------------------
    S, ctxlen = 64, 2048

    def decode_case(nh, nkv, hd, window, latent, **kw):
        cache = KVCache({0: KVRequest(nkv, hd, window, values_are_keys=latent)}, {0: None}, max_tokens=S * (ctxlen + 64),
                        max_slots=S + 1, dtype=bf, device=dev)
        cache.groups[0].storage.normal_()
        slots = [cache.acquire() for _ in range(S)]
        for s_ in slots:
            G.give_pages(cache, s_, ctxlen + 1)
        b1 = G.make_batch(dev, slots, [ctxlen] * S, [1] * S)
        q_ = torch.randn(S, nh, hd, device=dev).to(bf)
        o_ = torch.empty((S, nh * hd), dtype=bf, device=dev)
        ms = _graph_ms(lambda: core.attention_decode(q_, cache.view(0), b1, o_, nh=nh, window=window, scale=0.1, status=status, **kw))
        read = min(window or ctxlen + 1, ctxlen + 1)
        return ms, S * read * nkv * hd * 2 * (1 if latent else 2)

    ms, nb = decode_case(LH, 1, rk, None, True, sink=sinks)
    row("decode attention over latents (one record a position)", ms, nb)
    ms, nb = decode_case(nh2, nkv2, D, win, False, softcap=sh["softcap"])
    row("decode attention, two maps a head (window)", ms, nb)
    ms, nb = decode_case(H, Gk, 2 * d, None, False)
    row("decode attention, causal", ms, nb)
    ms, nb = decode_case(H, Gk, 2 * d, win, False)
    row("decode attention, window", ms, nb)
    core.check_status(status)
    return out


def run_zosipel(args):
    """``--workload zosipel``: prefill and decode of the Zosipel design at two sizes, the closest existing
    model at equal size beside it, and the new kernels beside their counterparts.  One JSON line per
    shape; not the benchmark record."""
    import torch

    import moe_b200

    pk = peaks()
    names = [args.shape] if args.shape in ZOSIPEL_SHAPES else list(ZOSIPEL_SHAPES)
    for name in names:
        sh = ZOSIPEL_SHAPES[name]
        V = sh["vocab"]
        res = {"workload": "zosipel", "shape": name, "sizes": sh, "dtype": "bfloat16", "data": "synthetic, random weights",
               "peaks": pk}
        for label, cfg in (("zosipel", zosipel_config(sh)), ("qwen2_moe", zosipel_qwen_config(sh))):
            model = moe_b200.random_model(cfg, seed=0, dtype="bfloat16", device="cuda:0")
            r = {"parameters": int(model.num_parameters)}
            eng = moe_b200.Engine(model, max_tokens=64 * (512 + args.steps + 64) + 4096, max_slots=64)
            ids = [(i * 7 + 13) % V for i in range(PREFILL_TOKENS)]

            def prefill():
                s = eng.new_sequence()
                eng.step([s], [ids], check=False)
                eng.release(s)

            ms = _median_ms(prefill)
            r["prefill_2048"] = {"ms": round(ms, 3), "tokens_per_s": round(PREFILL_TOKENS / ms * 1e3, 0)}
            for B in (1, 8, 64):
                slots = [eng.new_sequence() for _ in range(B)]
                eng.step(slots, [ids[:PROMPT_LEN]] * B, check=False)
                for i in range(args.warmup):
                    eng.step(slots, [[i % V]] * B, check=False)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for i in range(args.steps):
                    eng.step(slots, [[(i + 5) % V]] * B, check=False)
                b.record()
                torch.cuda.synchronize()
                eng.rt.check()
                ms = a.elapsed_time(b) / args.steps
                r[f"decode_b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 0)}
                for s in slots:
                    eng.release(s)
            res[label] = r
            del eng, model
            torch.cuda.empty_cache()
        res["kernels_at_8192_tokens"] = zosipel_kernels(sh, pk)
        print(json.dumps(res), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (reported in config)")
    ap.add_argument("--profile-step", choices=["decode", "prefill", "chunk", "sample"], default=None,
                    help="run a few steps of one kind between cudaProfilerStart/Stop (for ncu "
                         "--profile-from-start off) and print no benchmark line")
    ap.add_argument("--batch", type=int, default=8, help="with --profile-step decode: sequences in the batch")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16",
                    help="with --profile-step: the path whose kernels are wanted")
    ap.add_argument("--shape", choices=["a2.7b", "57b"] + sorted(set(SUPEVIK_SHAPES) | set(FOGAPEL_SHAPES) | set(ZOSIPEL_SHAPES) | set(DIVADRA_SHAPES)), default="a2.7b",
                    help="with --sweep: the layer sizes; with --workload supevik, fogapel, zosipel or divadra: one of its shapes (default: all)")
    ap.add_argument("--prompt-len", type=int, default=0, help="with --sweep: tokens in each prompt (default 512)")
    ap.add_argument("--workload", choices=["fp32-32k", "long-prompt", "supevik", "fogapel", "zosipel", "divadra"], default=None,
                    help="fp32-32k: the true 32-bit path at a context of 32,768; long-prompt: one bfloat16 prompt of "
                         "--prompt-len tokens [32768] run in pieces; supevik, fogapel, zosipel, divadra: that design at two sizes beside "
                         "the closest model at equal size (each prints its own line, no benchmark record)")
    ap.add_argument("--unequal", action="store_true", help="with --sweep: prompts of unequal lengths, 256 to 2,048 tokens")
    ap.add_argument("--sweep", default=None, help="comma-separated batch sizes: print decode throughput for each "
                                                  "and no benchmark line")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "JGalego/Moe is a Rust crate (no Python package, "
                          "no setup.py/pyproject); cargo and rustc are absent from this image and there is no network"}))
        return 0
    if args.gpus != 1:
        print("bench.py: moe_b200 is a single-GPU library; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.profile_step:
        return profile_step(args)
    if args.workload == "long-prompt":
        return run_long_prompt(args)
    if args.workload == "fp32-32k":
        return run_fp32_long(args)
    if args.workload == "supevik":
        return run_supevik(args)
    if args.workload == "fogapel":
        return run_fogapel(args)
    if args.workload == "zosipel":
        return run_zosipel(args)
    if args.workload == "divadra":
        return run_divadra(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
