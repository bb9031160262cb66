"""A recurrent mixer with a matrix-valued state per head and data-dependent decay (RWKV-style
time mixing).

With n_t the layer's normed input, n_(t-1) the previous token's (zeros before the first token)
and a blend x_s = n_t + (n_(t-1) - n_t) * mu_s for each of s in (r, k, v, g, w):
    r = Wr x_r, k = Wk x_k, v = Wv x_v           (heads x dim each)
    gate = silu(Wg x_g)
    w = exp(-exp(W2 tanh(W1 x_w) + w0))          (the decay, per head and key channel, in (0, 1))
per head, with a state S [dim, dim] that starts at zero:
    o_t = (S + diag(u) k_t v_t^T)^T r_t          (the bonus u acts on the current token only)
    S  <- diag(w_t) S + k_t v_t^T
and out = Wo ((o_t / rms(o_t over each head)) * norm_weight * gate).

What a sequence carries from step to step is of fixed size: n of its last token and S of every
head, both 32-bit (``state_request``).  The blends, the decay (its projections included), the scan
and the head norm are 32-bit arithmetic in both dtypes; the bfloat16 path rounds the blends that
feed the r, k, v and gate projections and the normed, gated output that feeds Wo.
"""
from __future__ import annotations

import os

import torch

from ..cache.kv import StateRequest
from ..ops import core
from ..ops.linear import grouped_linear, linear
from .base import Part, TensorSpec, register_part

_STREAMS = ("r", "k", "v", "g", "w")


class WKVMixer(Part):
    category, kind = "mixer", "wkv"
    graph_safe = True
    wants32 = True          # the blends are formed from the 32-bit normed input
    default_names = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w",
                     "r": "r", "k": "k", "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u",
                     "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.hd = int(p["head_dim"])
        self.eps = float(p["eps"])                     # of the per-head norm of the output
        self.rank = p.get("decay_rank")                # None: read from the tensor's shape when bound
        if not (self.nh > 0 and 0 < self.hd <= 256):
            raise ValueError(f"wkv: {self.nh} heads of {self.hd}; the scan takes heads of up to 256")
        self.inner = self.nh * self.hd
        # up to this many tokens a step the blends' kernel forms the decay itself
        self.fused_decay_tokens = int(os.environ.get("MOE_B200_WKV_FUSED_DECAY_MAX", "64"))

    def tensors(self):
        n, W, I = self.names, self.hidden, self.inner
        rank = int(self.rank) if self.rank else 16
        t = {n["mu_" + s]: TensorSpec((W,), vector=True) for s in _STREAMS}
        for s in ("r", "k", "v", "g"):
            t[n[s]] = TensorSpec((I, W))
        t[n["w1"]] = TensorSpec((rank, W))
        t[n["w2"]] = TensorSpec((I, rank))
        t[n["w0"]] = TensorSpec((I,), vector=True)
        t[n["u"]] = TensorSpec((self.nh, self.hd), vector=True)
        t[n["norm"]] = TensorSpec((I,), init="ones", vector=True)
        t[n["o"]] = TensorSpec((W, I))
        return t

    def tensors_in(self, has):
        """The width of the decay's narrow projection is given by its tensors alone (unless the part
        was told ``decay_rank``): any extent is accepted there, and ``bind`` checks that the two agree."""
        t = self.tensors()
        if not self.rank:
            n = self.names
            t[n["w1"]] = TensorSpec((-1, self.hidden))
            t[n["w2"]] = TensorSpec((self.inner, -1))
        return t

    def describe(self):
        return f"wkv({self.nh} heads of {self.hd}, state {self.hd}x{self.hd} a head, decay by a rank-{self.rank or '?'} projection)"

    def kv_request(self):
        return None

    def state_request(self):
        # [the last token's normed input | S of every head]
        return StateRequest((self.hidden + self.nh * self.hd * self.hd,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.mu = torch.stack([tensors[n["mu_" + s]].to(torch.float32) for s in _STREAMS]).contiguous()
        ws = [tensors[n[s]] for s in ("r", "k", "v", "g")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.w_rkvg = torch.stack([w.to(dt) for w in ws]).contiguous()          # [4, inner, hidden]
        # the decay's two small projections stay 32-bit arithmetic in both dtypes
        w1 = tensors[n["w1"]]
        self.w1 = w1.to(torch.float32).contiguous()
        self.w1_3 = None
        if rt.is_bf16 and w1.dtype == torch.bfloat16 and self.hidden % 8 == 0:
            self.w1_3 = torch.cat([w1, w1, w1], dim=1).contiguous()
        w2 = tensors[n["w2"]].to(torch.float32)
        if self.w1.shape[0] != w2.shape[1]:
            raise ValueError(f"wkv: the decay's projections disagree on their inner width ({self.w1.shape[0]} and {w2.shape[1]})")
        self.w2t = w2.t().contiguous()                 # [rank, inner]: the decay kernel reads it by columns
        self.rank = int(self.w1.shape[0])
        self.w0 = tensors[n["w0"]].to(torch.float32).contiguous()
        self.u = tensors[n["u"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.wo = tensors[n["o"]].contiguous()
        self._offsets = {}

    def _group_offsets(self, T, device):
        """Row offsets [0, T, 2T, 3T, 4T] of the four blends in the grouped product."""
        o = self._offsets.get(T)
        if o is None:
            o = self._offsets[T] = torch.arange(0, 5 * T, T, dtype=torch.int32, device=device)[:5].contiguous()
        return o

    def forward(self, rt, h, batch, cache_view, state):
        T, W, I = batch.num_tokens, self.hidden, self.inner
        dev = h.f32.device
        # ---- the five blends (and the state's last-token row) -----------------------------------
        decay = torch.empty((T, I), dtype=torch.float32, device=dev)
        if self.rank <= core.WKV_FUSED_RANK and T <= self.fused_decay_tokens:
            # few tokens: the decay exp(-exp(W2 tanh(W1 x_w) + w0)) in the same launch, its blend in registers
            mixed = rt.empty((4, T, W))
            core.wkv_shift_mix(h.f32, self.mu, state, batch, mixed, decay=(self.w1, self.w2t, self.w0, decay))
        else:
            # many tokens: every block of the fused form would read both projections from L2 (measured
            # 833 us against 104 + 40 + 84 at 8,192 tokens of width 2,048).  The blend stays 32-bit; in
            # bfloat16 its narrow projection runs on the tensor cores without leaving 32-bit accuracy: the
            # blend as three bfloat16 terms (exact) against the (bfloat16, hence exact) rows, three times
            # side by side, accumulated in float32
            mixed = rt.empty((4, T, W))
            xw = torch.empty((T, W), dtype=torch.float32, device=dev)
            core.wkv_shift_mix(h.f32, self.mu, state, batch, mixed, last32=xw)
            low = torch.empty((T, self.rank), dtype=torch.float32, device=dev)
            done = False
            if self.w1_3 is not None:
                from ..ops import tc

                done = tc.gemm_tc(core.split3(xw), self.w1_3, low, bn=64, splits=8, status=rt.status)
            if not done:
                core.gemm_generic(xw, self.w1, low, status=rt.status)
            core.wkv_decay(low, self.w2t, self.w0, decay)
        # ---- r, k, v and the gate: one grouped product, a group a blend ---------------------------
        rkvg = grouped_linear(rt, mixed.view(4 * T, W), self.w_rkvg, self._group_offsets(T, dev), 4 * T)
        # ---- the scan over each sequence's tokens -----------------------------------------------
        o = torch.empty((T, I), dtype=torch.float32, device=dev)
        core.wkv_scan(rkvg[:T], rkvg[T:2 * T], rkvg[2 * T:3 * T], decay, self.u, state[:, W:], batch, o,
                      heads=self.nh, d=self.hd)
        y = rt.empty((T, I))
        core.wkv_finish(o, rkvg[3 * T:], self.norm_w, self.eps, batch, y, heads=self.nh, d=self.hd)
        return linear(rt, y, self.wo)


register_part("mixer", "wkv", WKVMixer)


class SSDMixer(Part):
    """A state-space mixer with one decay number per head and step (Mamba-2).

    With n_t the layer's input, inner = heads * dv, N the state size and G groups of heads that share
    B and C, the input projection's rows are [z: inner | x: inner | B: G N | C: G N | dt: heads].
    x, B and C together pass a causal convolution over time per channel (taps [channels, taps] with a
    bias; the last column multiplies the token's own row) and silu.  Per head h of group
    g = h // (heads / G), with dt = softplus(dt + dt_bias_h) and a state S [N, dv] that starts at zero:
        S  <- exp(-exp(A_log_h) dt) S + dt B_t x_t^T
        y_t = S^T C_t + D_h x_t
    and out = Wo norm(y * silu(z)), the norm an RMS norm over each of ``norm_groups`` equal parts of
    the row, times a weight.

    What a sequence carries from step to step is of fixed size: the convolution's last taps - 1 inputs
    and S of every head, both 32-bit.  The convolution, dt, the decay, the recurrence, the gate and the
    norm are 32-bit arithmetic in both dtypes; the bfloat16 path rounds the input of the two
    projections."""

    category, kind = "mixer", "ssd"
    graph_safe = True
    default_names = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log",
                     "d": "D", "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.dv, self.n = int(p["num_heads"]), int(p["value_dim"]), int(p["state_size"])
        self.groups, self.norm_groups = int(p.get("groups", 1)), int(p.get("norm_groups", 1))
        self.taps = int(p["taps"])
        self.eps = float(p["eps"])
        self.inner = self.nh * self.dv
        self.channels = self.inner + 2 * self.groups * self.n
        if self.nh % self.groups or self.inner % self.norm_groups:
            raise ValueError("ssd: heads must be a multiple of groups, and heads * value_dim of norm_groups")
        if not (0 < self.n <= 512 and 1 <= self.taps <= 16):
            raise ValueError(f"ssd: state of {self.n}, {self.taps} taps; the kernels take up to 512 and 1 to 16")

    def tensors(self):
        n = self.names
        return {
            n["in"]: TensorSpec((2 * self.inner + 2 * self.groups * self.n + self.nh, self.hidden)),
            n["conv"]: TensorSpec((self.channels, self.taps)),
            n["conv_bias"]: TensorSpec((self.channels,), init="zeros", vector=True),
            n["dt_bias"]: TensorSpec((self.nh,), init="zeros", vector=True),
            n["a_log"]: TensorSpec((self.nh,), init="zeros", vector=True),
            n["d"]: TensorSpec((self.nh,), init="ones", vector=True),
            n["norm"]: TensorSpec((self.inner,), init="ones", vector=True),
            n["o"]: TensorSpec((self.hidden, self.inner)),
        }

    def describe(self):
        return (f"ssd({self.nh} heads of {self.dv}, state {self.n}x{self.dv} a head, {self.groups} groups, "
                f"convolution of {self.taps} taps, norm in {self.norm_groups} parts)")

    def kv_request(self):
        return None

    def state_request(self):
        # [the convolution's last taps - 1 inputs | S of every head]
        return StateRequest(((self.taps - 1) * self.channels + self.nh * self.n * self.dv,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.w_in = tensors[n["in"]].contiguous()
        self.taps_w = tensors[n["conv"]].to(torch.float32).t().contiguous()          # [taps, channels]
        self.conv_b = tensors[n["conv_bias"]].to(torch.float32).contiguous()
        self.dt_bias = tensors[n["dt_bias"]].to(torch.float32).contiguous()
        self.a_log = tensors[n["a_log"]].to(torch.float32).contiguous()
        self.d_skip = tensors[n["d"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.wo = tensors[n["o"]].contiguous()

    def forward(self, rt, h, batch, cache_view, state):
        T, I, C = batch.num_tokens, self.inner, self.channels
        proj = linear(rt, h.act, self.w_in)                       # float32 [T, z | x B C | dt]
        mixed = proj[:, I:I + C]
        xbc = torch.empty((T, C), dtype=torch.float32, device=proj.device)
        core.seq_conv([dict(u=mixed, w=self.taps_w, bias=self.conv_b, offset=0, out32=xbc)], state, batch,
                      taps=self.taps, channels=C, act="silu")
        if self.taps > 1 and not batch.all_decode:
            core.conv_state_update(mixed, state, batch, taps=self.taps, channels=C)
        y = torch.empty((T, I), dtype=torch.float32, device=proj.device)
        core.ssd_scan(xbc, proj[:, I + C:I + C + self.nh], self.dt_bias, self.a_log, self.d_skip, state, batch, y,
                      heads=self.nh, groups=self.groups, n=self.n, dv=self.dv, offset=(self.taps - 1) * C)
        out = rt.empty((T, I))
        core.ssd_finish(y, proj[:, :I], self.norm_w, self.eps, batch, out, norm_groups=self.norm_groups)
        return linear(rt, out, self.wo)


class _SubTensors:
    """The tensors of a part that lives inside another: local names with the inner prefix taken off."""

    def __init__(self, outer, prefix, names):
        self._outer, self._prefix, self._names = outer, prefix, list(names)

    def __getitem__(self, local):
        return self._outer[self._prefix + local]

    def __contains__(self, local):
        return local in self._names

    def __iter__(self):
        return iter(self._names)

    def __len__(self):
        return len(self._names)

    def pop(self, local, *default):
        if local not in self._names and default:
            return default[0]
        return self[local]


class SideBySideMixer(Part):
    """Two mixers that read the same input; each output passes an RMS norm over the model's width with
    a weight of its own, and the result is half their sum:
        out = (rmsnorm(left(n)) * w_left + rmsnorm(right(n)) * w_right) / 2
    ``left`` and ``right`` are mixers of any registered kind ({"kind", "params"}); their tensors live
    under ``left.`` / ``right.``.  At most one of them may keep keys and values in pages; state of fixed
    size of both lies side by side in one row a sequence."""

    category, kind = "mixer", "side_by_side"
    default_names = {"left_out": "left.out", "right_out": "right.out"}

    def __init__(self, spec):
        from ..config.spec import PartSpec
        from .base import make_part

        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.eps = float(p["eps"])
        self.subs = []
        for side in ("left", "right"):
            sub = p[side]
            self.subs.append((side + ".", make_part("mixer", PartSpec(sub["kind"], dict(sub["params"]), spec.prefix + side + "."))))
        self.beside = os.environ.get("MOE_B200_SIDE_BY_SIDE_STREAMS", "1") != "0"
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m in self.subs)
        self.wants32 = any(getattr(m, "wants32", False) for _, m in self.subs)
        if sum(m.kv_request() is not None for _, m in self.subs) > 1:
            raise ValueError("side_by_side: only one of the two mixers may keep keys and values in pages")
        if not all(getattr(m, "own_kv", True) for _, m in self.subs):
            raise ValueError("side_by_side: a mixer that reads another layer's cache cannot stand inside")

    def _sub_tensors(self, fn):
        t = {}
        for prefix, m in self.subs:
            for local, ts in fn(m, prefix).items():
                t[prefix + local] = ts
        n = self.names
        t[n["left_out"]] = TensorSpec((self.hidden,), init="ones", vector=True)
        t[n["right_out"]] = TensorSpec((self.hidden,), init="ones", vector=True)
        return t

    def tensors(self):
        return self._sub_tensors(lambda m, prefix: m.tensors())

    def tensors_in(self, has):
        return self._sub_tensors(lambda m, prefix: m.tensors_in(lambda local: has(prefix + local)))

    def describe(self):
        return "half the sum of two normed mixers: " + " | ".join(m.describe() for _, m in self.subs)

    def step_elements(self, num_tokens):
        return float(sum(m.step_elements(num_tokens) for _, m in self.subs) + 2 * self.hidden)

    def kv_request(self):
        for _, m in self.subs:
            if m.kv_request() is not None:
                return m.kv_request()
        return None

    def state_request(self):
        reqs = [m.state_request() for _, m in self.subs]
        if all(r is None for r in reqs):
            return None
        n = 0
        for r in reqs:
            if r is not None:
                if r.dtype != torch.float32 or len(r.shape) != 1:
                    raise ValueError("side_by_side: the mixers' state must be rows of 32-bit floats")
                n += r.shape[0]
        return StateRequest((n,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        for prefix, m in self.subs:
            names = [k[len(prefix):] for k in tensors if k.startswith(prefix) and k not in self.names.values()]
            m.bind(_SubTensors(tensors, prefix, names), rt)
        self.w_left = tensors[self.names["left_out"]].to(torch.float32).contiguous()
        self.w_right = tensors[self.names["right_out"]].to(torch.float32).contiguous()

    def forward(self, rt, h, batch, cache_view, state):
        """The right mixer runs on a second stream beside the left one (inside a captured step: a fork
        and a join); MOE_B200_SIDE_BY_SIDE_STREAMS=0 runs them one after the other."""
        states, at = [], 0
        for _, m in self.subs:
            r = m.state_request()
            states.append(state[:, at:at + r.shape[0]] if r is not None else None)
            at += r.shape[0] if r is not None else 0
        views = [cache_view if m.kv_request() is not None else None for _, m in self.subs]
        (_, left), (_, right) = self.subs
        if self.beside and h.act.is_cuda:
            main = torch.cuda.current_stream()
            side = rt.side_stream(1)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                b = right.forward(rt, h, batch, views[1], states[1])
            a = left.forward(rt, h, batch, views[0], states[0])
            main.wait_stream(side)
            b.record_stream(main)
        else:
            a = left.forward(rt, h, batch, views[0], states[0])
            b = right.forward(rt, h, batch, views[1], states[1])
        out = torch.empty_like(a)
        core.pair_norm_mean(a, self.w_left, b, self.w_right, self.eps, out)
        return out


register_part("mixer", "ssd", SSDMixer)
register_part("mixer", "side_by_side", SideBySideMixer)
