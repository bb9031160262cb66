"""Feed-forward parts: a dense SwiGLU MLP and routed SwiGLU experts with an
optional sigmoid-gated shared expert.

SwiGLU (src/model.rs:26-35):   y = Wd (silu(Wg n) * (Wu n))
Routing (src/model.rs:844-897): softmax over all experts, top k, optional
  renormalisation, scaling factor.
Experts (src/model.rs:902-942): out_i = sum_e w_ie * y_e(n_i).
Shared expert (src/model.rs:956-970): out += sigmoid(Wsg n) * y_s(n).
"""
from __future__ import annotations

import os

import torch

from ..ops import core
from ..ops.linear import grouped_linear, grouped_swiglu_linear, linear, swiglu_linear
from .base import Activations, LazyDelta, Part, TensorSpec, register_part


def _fuse_rows(tensors):
    dt = tensors[0].dtype if all(t.dtype == tensors[0].dtype for t in tensors) else torch.float32
    return torch.cat([t.to(dt) for t in tensors], dim=0).contiguous()


class DenseSwiGLU(Part):
    """y = Wd f(Wg n, Wu n); ``activation`` names f: "silu" (the default) and "gelu_tanh" are
    act(g) * u; "clamped_sigmoid" with its constant ``limit`` L is
    min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1)."""

    category, kind = "ffn", "dense_swiglu"
    graph_safe = True
    wants32 = False
    default_names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.size = int(self.params["size"])
        self.activation = str(self.params.get("activation", "silu"))
        if self.activation not in core.GLU_ACTS:
            raise ValueError(f"dense gated feed-forward: activation '{self.activation}' is none of {sorted(core.GLU_ACTS)}")
        self.limit = float(self.params.get("limit") or 0.0)
        if self.activation == "clamped_sigmoid" and not self.limit > 0:
            raise ValueError("dense gated feed-forward: 'clamped_sigmoid' needs a positive limit")

    def tensors(self):
        n = self.names
        return {
            n["gate"]: TensorSpec((self.size, self.hidden)),
            n["up"]: TensorSpec((self.size, self.hidden)),
            n["down"]: TensorSpec((self.hidden, self.size)),
        }

    def describe(self):
        return (f"dense {'SwiGLU' if self.activation == 'silu' else 'gated ' + self.activation} {self.size}"
                + (f", limit {self.limit:g}" if self.limit else ""))

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.w_gu = _fuse_rows([tensors[n["gate"]], tensors[n["up"]]])
        self.w_down = tensors[n["down"]].contiguous()

    def forward(self, rt, h, batch):
        return linear(rt, swiglu_linear(rt, h.act, self.w_gu, self.activation, self.limit), self.w_down)


def relu2_linear(rt, a, w_up, out=None):
    """relu(a Wu^T)^2 in the compute dtype: in the tensor-core product's epilogue (on the 32-bit
    accumulator) where that kernel takes the product, else the product's 32-bit output and then the
    activation."""
    if out is None:
        out = torch.empty((a.shape[0], w_up.shape[0]), dtype=rt.compute_dtype, device=a.device)
    if rt.is_bf16 and a.dtype == torch.bfloat16 and w_up.dtype == torch.bfloat16:
        from ..ops import tc

        if tc.gemm_tc(a, w_up, out, status=rt.status, act="relu2"):
            return out
    core.relu2(linear(rt, a, w_up), out)
    return out


class DenseMLP(Part):
    """y = Wd f(Wu n), no gate; ``activation`` names f: "relu2" is relu(z)^2.  The activation is 32-bit
    arithmetic on the first product's 32-bit output; the bfloat16 path rounds its result."""

    category, kind = "ffn", "dense_mlp"
    graph_safe = True
    wants32 = False
    default_names = {"up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.size = int(self.params["size"])
        self.activation = str(self.params.get("activation", "relu2"))
        if self.activation != "relu2":
            raise ValueError(f"dense feed-forward: activation '{self.activation}' is none of ['relu2']")

    def tensors(self):
        n = self.names
        return {n["up"]: TensorSpec((self.size, self.hidden)), n["down"]: TensorSpec((self.hidden, self.size))}

    def describe(self):
        return f"dense {self.activation} {self.size}"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.w_up = tensors[self.names["up"]].contiguous()
        self.w_down = tensors[self.names["down"]].contiguous()

    def forward(self, rt, h, batch):
        return linear(rt, relu2_linear(rt, h.act, self.w_up), self.w_down)


class CombineDelta(LazyDelta):
    """The routed experts' outputs before the combine: delta[t] = sum_j w[t, j] * y[pos[t, j]] +
    gate[t] * shared[t].  An RMS norm forms it inside its own kernel."""

    kind = "expert_combine"

    def __init__(self, y, pos_of_pair, topk_w, top_k, shared, shared_gate, tokens, hidden):
        self.y, self.pos_of_pair, self.topk_w, self.top_k = y, pos_of_pair, topk_w, top_k
        self.shared, self.shared_gate, self.tokens, self.hidden = shared, shared_gate, tokens, hidden

    def materialize(self, rt):
        out = rt.empty((self.tokens, self.hidden), torch.float32)
        core.moe_combine(self.y, self.pos_of_pair, self.topk_w, self.top_k, out, shared=self.shared,
                         shared_gate=self.shared_gate)
        return out


class RoutedExperts(Part):
    category, kind = "ffn", "routed_experts"
    graph_safe = True
    wants32 = True   # router logits are computed from the 32-bit normed state
    # {e} in an expert's tensor name is its number; "router_bias" is read only with ``router_bias``
    default_names = {"router": "gate.weight", "router_bias": "gate.bias",
                     "expert_gate": "experts.{e}.gate_proj.weight", "expert_up": "experts.{e}.up_proj.weight",
                     "expert_down": "experts.{e}.down_proj.weight",
                     "shared_gate_proj": "shared_expert.gate_proj.weight", "shared_up": "shared_expert.up_proj.weight",
                     "shared_down": "shared_expert.down_proj.weight", "shared_gate": "shared_expert_gate.weight",
                     "table": "table"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.E = int(p["num_experts"])
        self.k = int(p["top_k"])
        self.size = int(p["expert_size"])
        self.norm_topk = bool(p.get("norm_topk_prob", False))
        self.scale = float(p.get("routed_scaling_factor", 1.0))
        self.shared_size = int(p.get("shared_size", 0) or 0)
        self.shared_gate = bool(p.get("shared_gate", False)) and self.shared_size > 0
        self.router_bias = bool(p.get("router_bias", False))     # logits = Wr n + b
        # "table": no router at all; an integer table [vocab, top_k] names each token id's experts, every
        # one with weight 1 / top_k
        self.table = str(p.get("router", "softmax")) == "table"
        self.vocab = int(p.get("vocab_size", 0) or 0)
        if self.table and (self.vocab <= 0 or p.get("groups") or self.router_bias or p.get("shared_gate")):
            raise ValueError("routing by a table needs the vocabulary's size and takes no router options")
        if self.table:
            self.wants32 = False
        # {"count": g, "keep": m}: the experts form g equal groups of neighbours, a group's score is its
        # best expert's, and only experts of the m best groups may be picked
        grp = p.get("groups") or {}
        self.groups, self.keep = int(grp.get("count", 0) or 0), int(grp.get("keep", 0) or 0)
        if self.groups <= 1 or self.keep >= self.groups:
            self.groups = self.keep = 0                          # every group kept: no limit at all
        elif self.E % self.groups or self.keep < 1 or self.k > self.keep * (self.E // self.groups):
            raise ValueError("router groups: the count must divide the experts, and the kept groups must hold top_k experts")
        self._grp = dict(groups=self.groups, keep=self.keep)
        if not 0 < self.k <= self.E:
            raise ValueError("top_k must lie in 1..num_experts")
        # Set to a list to record every routing decision as (expert ids [T, k], weights [T, k]);
        # the reference's State::trace does the same per token and layer (src/model.rs:157, 943-950).
        self.trace = None
        # measured on a B200: the fused norm + router + dispatch launch wins up to 8 tokens and loses
        # from 16 on, where its single gathering block is the bottleneck
        self.fused_norm_tokens = int(os.environ.get("MOE_B200_NORM_ROUTE_MAX", "8"))
        self.shared_beside = os.environ.get("MOE_B200_SHARED_BESIDE", "1") != "0"
        # up to this many tokens one block picks, inverts and gathers (one launch after the logits);
        # beyond, a warp per token picks and the inversion and the gather are launches of their own
        # (measured on a B200, ms a decode step at 16 / 32 / 64 tokens: 4.65 / 5.89 / 7.38 with one
        # block up to 64 tokens, 4.48 / 5.75 / 7.07 with one block up to 8)
        self.route_dispatch_tokens = int(os.environ.get("MOE_B200_ROUTE_DISPATCH_MAX", "8"))
        # from this many tokens on (a prompt) the router's logits are a tensor-core product of the
        # 32-bit activations split into three bfloat16 terms (35 -> about 15 us at 2,048 tokens)
        self.tc_router_tokens = int(os.environ.get("MOE_B200_TC_ROUTER_MIN", "257"))

    def _expert(self, role, e):
        return self.names[role].format(e=e)

    def tensors(self):
        t = ({self.names["table"]: TensorSpec((self.vocab, self.k), integer=self.E)} if self.table
             else {self.names["router"]: TensorSpec((self.E, self.hidden))})
        for e in range(self.E):
            t[self._expert("expert_gate", e)] = TensorSpec((self.size, self.hidden), sparse=True)
            t[self._expert("expert_up", e)] = TensorSpec((self.size, self.hidden), sparse=True)
            t[self._expert("expert_down", e)] = TensorSpec((self.hidden, self.size), sparse=True)
        return self._common(t)

    def _common(self, t):
        n = self.names
        if self.router_bias:
            t[n["router_bias"]] = TensorSpec((self.E,), init="zeros", vector=True)
        if self.shared_size:
            t[n["shared_gate_proj"]] = TensorSpec((self.shared_size, self.hidden))
            t[n["shared_up"]] = TensorSpec((self.shared_size, self.hidden))
            t[n["shared_down"]] = TensorSpec((self.hidden, self.shared_size))
        if self.shared_gate:
            t[n["shared_gate"]] = TensorSpec((1, self.hidden))
        return t

    def tensors_in(self, has):
        """Three checkpoint layouts of the experts, as the reference reads them (src/model.rs:396-420):
        fused ``experts.gate_up_proj`` [E, 2 size, hidden] (rows [0, size) gate, then up) with
        ``experts.down_proj`` [E, hidden, size]; stacked ``experts.{gate,up,down}_proj`` of three
        dimensions; else one tensor per expert and projection."""
        E, n, H = self.E, self.size, self.hidden
        router = self.names["router"]
        if self.table:
            return self.tensors()
        if has("experts.gate_up_proj"):
            t = {router: TensorSpec((E, H)), "experts.gate_up_proj": TensorSpec((E, 2 * n, H), sparse=True),
                 "experts.down_proj": TensorSpec((E, H, n), sparse=True)}
            return self._common(t)
        if has("experts.gate_proj") and has("experts.up_proj"):
            t = {router: TensorSpec((E, H)), "experts.gate_proj": TensorSpec((E, n, H), sparse=True),
                 "experts.up_proj": TensorSpec((E, n, H), sparse=True),
                 "experts.down_proj": TensorSpec((E, H, n), sparse=True)}
            return self._common(t)
        return self.tensors()

    def describe(self):
        return (f"{self.E} experts of {self.size}, top-{self.k}, "
                + ("named by a table over token ids, equal weights" if self.table else "softmax gate")
                + (" with bias" if self.router_bias else "")
                + (f", within the best {self.keep} of {self.groups} groups" if self.groups else "")
                + (", renormalised" if self.norm_topk else "")
                + (f", scaled by {self.scale:g}" if self.scale != 1.0 else "")
                + (f", shared expert {self.shared_size}" + (" (gated)" if self.shared_gate else "")
                   if self.shared_size else ""))

    def step_elements(self, num_tokens):
        """The router, the shared expert, and the experts that ``num_tokens`` tokens are expected to
        touch if each picks ``top_k`` of them evenly: E (1 - (1 - k/E)^tokens)."""
        dense = sparse = 0
        for ts in self.tensors().values():
            n = 1
            for d in ts.shape:
                n *= d
            if ts.sparse:
                sparse += n
            else:
                dense += n
        touched = 1.0 - (1.0 - self.k / self.E) ** max(num_tokens, 0)
        return dense + sparse * touched

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.route_table = None
        if self.table:
            self.route_table = tensors[n["table"]].to(torch.int32).contiguous()
            self.w_router = None
            dev = self.route_table.device
        else:
            self.w_router = tensors[n["router"]].contiguous()
            dev = self.w_router.device
        self.b_router = tensors[n["router_bias"]].to(torch.float32).contiguous() if self.router_bias else None
        # The device layout is [E, 2 * size, hidden] (rows [0, size) gate, [size, 2 size) up) and
        # [E, hidden, size], whatever the checkpoint's; tensors are fetched one at a time.
        if "experts.gate_up_proj" in tensors:
            self.w_gu = tensors["experts.gate_up_proj"].contiguous()
            self.w_down = tensors["experts.down_proj"].contiguous()
            if self.w_gu.dtype != self.w_down.dtype:
                self.w_gu, self.w_down = self.w_gu.float(), self.w_down.float()
        elif "experts.gate_proj" in tensors:
            g, u, self.w_down = tensors["experts.gate_proj"], tensors["experts.up_proj"], tensors["experts.down_proj"]
            dt = g.dtype if g.dtype == u.dtype == self.w_down.dtype else torch.float32
            self.w_gu = torch.cat([g.to(dt), u.to(dt)], dim=1).contiguous()
            self.w_down = self.w_down.to(dt).contiguous()
        else:
            first = tensors[self._expert("expert_gate", 0)]
            dt = first.dtype
            self.w_gu = torch.empty((self.E, 2 * self.size, self.hidden), dtype=dt, device=dev)
            self.w_down = torch.empty((self.E, self.hidden, self.size), dtype=dt, device=dev)
            for e in range(self.E):
                for role in ("expert_gate", "expert_up", "expert_down"):
                    t = tensors[self._expert(role, e)]
                    if t.dtype != dt:                  # a checkpoint of mixed dtypes: everything in 32-bit
                        self.w_gu, self.w_down, dt = self.w_gu.float(), self.w_down.float(), torch.float32
                    dst = {"expert_gate": self.w_gu[e, : self.size], "expert_up": self.w_gu[e, self.size:],
                           "expert_down": self.w_down[e]}[role]
                    dst.copy_(t)
        self.ws_gu = self.ws_down = self.w_sgate = None
        if self.shared_size:
            self.ws_gu = _fuse_rows([tensors[n["shared_gate_proj"]], tensors[n["shared_up"]]])
            self.ws_down = tensors[n["shared_down"]].contiguous()
        if self.shared_gate:
            self.w_sgate = tensors[n["shared_gate"]].reshape(-1).to(self.w_router.dtype).contiguous()
        # For prompts the router's logits come from the tensor cores: the 32-bit activations as three
        # bfloat16 terms against the (bfloat16, hence exact) router rows, three times side by side.
        self.w_router3 = None
        if rt.is_bf16 and self.w_router is not None and self.w_router.dtype == torch.bfloat16 and self.hidden % 8 == 0:
            rows = [self.w_router] + ([self.w_sgate.reshape(1, -1)] if self.w_sgate is not None else [])
            one = torch.cat(rows, dim=0)
            self.w_router3 = torch.cat([one, one, one], dim=1).contiguous()

    def route(self, rt, h, batch, after_logits=None):
        """-> (topk_idx [T, k] int32, topk_w [T, k] float32, shared_gate [T] float32 or None)
        ``after_logits``: called once the logits' product is launched (or, where logits and picks are one
        launch, after that)."""
        T = h.act.shape[0]
        topk_idx = rt.empty((T, self.k), torch.int32)
        topk_w = rt.empty((T, self.k), torch.float32)
        if self.table:
            core.table_route(self.route_table, batch, self.k, self.E, topk_idx, topk_w, rt.status)
            if after_logits is not None:
                after_logits()
            return topk_idx, topk_w, None
        sg = rt.empty((T,), torch.float32) if self.w_sgate is not None else None
        if self.w_router3 is not None and T >= self.tc_router_tokens:
            from ..ops import tc

            logits = rt.empty((T, self.w_router3.shape[0]), torch.float32)
            if tc.gemm_tc(core.split3(h.f32), self.w_router3, logits, bn=64, splits=8, status=rt.status):
                if after_logits is not None:
                    after_logits()
                core.router_topk(logits, self.k, self.norm_topk, self.scale, topk_idx, topk_w, num_experts=self.E,
                                 shared_gate=sg, seq_of_token=getattr(batch, "seq_of_token", None), bias=self.b_router,
                                 **self._grp)
                return topk_idx, topk_w, sg
        core.router(h.f32, self.w_router, self.k, self.norm_topk, self.scale, topk_idx, topk_w,
                    shared_gate_w=self.w_sgate, shared_gate=sg, seq_of_token=getattr(batch, "seq_of_token", None),
                    bias=self.b_router, **self._grp)
        if after_logits is not None:
            after_logits()
        return topk_idx, topk_w, sg

    def _shared(self, rt, h):
        return linear(rt, swiglu_linear(rt, h.act, self.ws_gu), self.ws_down)

    def forward(self, rt, h, batch):
        return self._run(rt, h, batch, None).materialize(rt)

    def forward_lazy(self, rt, h, batch):
        """The same, the combine left to whoever adds the delta (see ``CombineDelta``)."""
        return self._run(rt, h, batch, None)

    def forward_prenorm(self, rt, x, delta, norm, batch):
        """The block's offer to take the norm before this feed-forward along: for a step of few
        tokens, norm, router and dispatch are one launch.  None if the sizes or the kind of norm do
        not allow it (the block then runs the norm itself and calls ``forward``)."""
        rms = getattr(norm, "rms_params", None)          # the norm says whether it can be run by a neighbour
        if rms is None or x.shape[0] > self.fused_norm_tokens or self.E > 256 or self.b_router is not None or self.table:
            return None
        norm_w, norm_eps = rms()
        routed = core.norm_route(x, delta, norm_w, norm_eps, self.w_router, self.k, self.norm_topk, self.scale,
                                 bf16=rt.is_bf16, shared_gate_w=self.w_sgate,
                                 seq_of_token=getattr(batch, "seq_of_token", None), status=rt.status, **self._grp)
        if routed is None:
            return None
        out32, out16 = routed[:2]
        h = Activations(act=out16 if rt.is_bf16 else out32, f32=out32)
        return self._run(rt, h, batch, routed[2:])

    def _run(self, rt, h, batch, routed):
        T = h.act.shape[0]
        P = T * self.k
        few = T <= 64 and self.E <= 256
        ys = side = None
        if self.ws_gu is not None and few:
            # few tokens: neither branch fills the GPU, so the shared expert runs beside the routed
            # ones on a second stream (inside a captured graph this becomes a fork and a join)
            main = torch.cuda.current_stream()
            side = rt.side_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                ys = self._shared(rt, h)
        if routed is not None:
            topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs = routed
        elif few and T <= self.route_dispatch_tokens and not self.table:
            # pick, table inversion and gather in one launch after the logits
            topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs = core.route_dispatch(
                h.f32, self.w_router, self.k, self.norm_topk, self.scale, shared_gate_w=self.w_sgate,
                seq_of_token=getattr(batch, "seq_of_token", None),
                gather=h.act if h.act.dtype == torch.bfloat16 and T <= 16 else None, status=rt.status,
                bias=self.b_router, **self._grp)
            # (more tokens: the gather by that one block would take longer than a launch of its own)
        else:
            def shared_beside():
                # Many tokens: pick, table inversion and gather are small launches that leave the GPU
                # idle (37 us of a layer at 2,048 tokens), so the shared expert starts beside them on
                # a second stream.  (Not before the logits' product: the shared expert's CTAs fill every
                # SM's shared memory, and that product would wait for them to end.)
                nonlocal ys, side
                main = torch.cuda.current_stream()
                side = rt.side_stream()
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    ys = self._shared(rt, h)

            topk_idx, topk_w, sg = self.route(rt, h, batch,
                                              after_logits=shared_beside if self.ws_gu is not None and side is None and self.shared_beside else None)
            offsets = rt.empty((self.E + 1,), torch.int32)
            sorted_token = rt.empty((P,), torch.int32)
            pos_of_pair = rt.empty((P,), torch.int32)
            core.moe_align(topk_idx, T, self.k, self.E, offsets, sorted_token, pos_of_pair, rt.status)
            xs = None
        if self.trace is not None:
            self.trace.append((topk_idx.clone(), topk_w.clone()))
        act = grouped_swiglu_linear(rt, h.act, self.w_gu, offsets, sorted_token, P, gathered=xs)
        # (the offsets were written before the product above: the second product may start on its weights early)
        y = grouped_linear(rt, act, self.w_down, offsets, P, early_offsets=True)
        if self.ws_gu is not None and side is None:
            ys = self._shared(rt, h)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
            ys.record_stream(torch.cuda.current_stream())
        return CombineDelta(y, pos_of_pair, topk_w, self.k, ys, sg, T, self.hidden)


register_part("ffn", "dense_swiglu", DenseSwiGLU)
register_part("ffn", "dense_mlp", DenseMLP)
register_part("ffn", "routed_experts", RoutedExperts)
