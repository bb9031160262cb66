"""Latent attention: keys and values of every head are projections of ONE small latent per
position, and only the latent is cached.  No position encoding.

With n the layer's normed input, H heads, d the query/key size, dv the value size, r the latent's:
    q = Wq n   [H, d]
    c = rms(Wdkv n) * w_c                        (r numbers; x / sqrt(mean(x^2) + eps), plain weight)
    k_h = Wuk_h c,  v_h = Wuv_h c                (rows of Wuk / Wuv head by head)
    p_hj = exp(scale q_h . k_hj) / (exp(b_h) + sum_j' exp(scale q_h . k_hj')),  j <= position (causal)
    (b_h: the head's sink, a learned number that joins the denominator and carries no value)
    out = Wo [sum_j p_hj v_hj]_h

How it runs.  q_h . (Wuk_h c) = (Wuk_h^T q_h) . c and sum_j p_j Wuv_h c_j = Wuv_h sum_j p_j c_j, so the
attention runs over the cached latents alone: H query heads of r numbers on ONE key/value head
whose keys ARE its values (``KVRequest.values_are_keys``: one plane of the paged cache, r numbers a
position whatever H is).  The attention kernels are the ones every other layer uses, with the
sink's per-head number as one more parameter of their common variant.  Records have one width
D >= r (zero-filled).  Each of the two per-head products runs in one of two forms, chosen when the
weights are bound by the number of weight elements a token then meets (``absorb``: "auto", or True /
False for both sides):

* folded into its neighbour: Wuk_h^T Wq_h (r x hidden a head) stands in the input projection's place,
  so the projection's output row already holds the queries over the latent, and Wo_h Wuv_h (hidden x r
  a head) in the output projection's, which then reads the attended latents as they come; cheaper
  while r (hidden) <= d (hidden + r), resp. dv (hidden + r): a latent no larger than a head.  The folded
  matrices are formed once in float64 from the checkpoint's values and rounded once to the weights'
  dtype.  A latent layer is then norm, projection, ``latent_prepare`` (latent norm, key record,
  append, queries as records), attention, output projection.
* on its own: a grouped product, a group a head, through the kernels the routed experts use; the
  groups' rows lie head by head, which ``latent_prepare`` and ``heads_transpose`` arrange.  Cheaper
  for latents several times a head's size.

32-bit in both dtypes: the latent's norm, scores, softmax and sink.  The bfloat16 path rounds the
queries over the latent, the cached latent, and the attended latent before its product (and, on its
own, the queries before and the values after their per-head product).
"""
from __future__ import annotations

import torch

from ..cache.kv import KVRequest
from ..ops import core
from ..ops.linear import grouped_linear, linear
from .attention import record_width
from .base import Part, TensorSpec, register_part


class LatentAttention(Part):
    category, kind = "mixer", "latent_attention"
    graph_safe = True
    default_names = {"q": "q_proj.weight", "down": "kv_a_proj.weight", "down_norm": "kv_a_norm.weight",
                     "up_k": "k_b_proj.weight", "up_v": "v_b_proj.weight", "sink": "sinks", "o": "o_proj.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.hd = int(p["head_dim"])
        self.vd = int(p.get("value_dim") or self.hd)
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.sink = bool(p.get("sink", False))
        self.absorb = p.get("absorb", "auto")
        if not (self.nh > 0 and self.hd > 0 and self.vd > 0 and 0 < self.rank <= 256):
            raise ValueError(f"latent attention: {self.nh} heads of {self.hd} / {self.vd} on a latent of {self.rank}; "
                             "the attention kernels take latents of up to 256")
        self.width = self.rank                    # of a cached record; set when bound

    def tensors(self):
        n, H, W, r = self.names, self.nh, self.hidden, self.rank
        t = {n["q"]: TensorSpec((H * self.hd, W)), n["down"]: TensorSpec((r, W)),
             n["down_norm"]: TensorSpec((r,), init="ones", vector=True),
             n["up_k"]: TensorSpec((H * self.hd, r)), n["up_v"]: TensorSpec((H * self.vd, r)),
             n["o"]: TensorSpec((W, H * self.vd))}
        if self.sink:
            t[n["sink"]] = TensorSpec((H,), init="zeros", vector=True)
        return t

    def kv_request(self):
        return KVRequest(1, self.width, None, values_are_keys=True)

    def state_request(self):
        return None

    def describe(self):
        return (f"latent attention ({self.nh} heads of {self.hd}, values of {self.vd}, one cached latent of {self.rank} "
                f"a position{', softmax with a sink a head' if self.sink else ''}), no position encoding")

    def step_elements(self, tokens):
        W, H, r = self.hidden, self.nh, self.rank
        fq, fo = self._folds()
        qside = H * r * W if fq else H * self.hd * (W + r)
        oside = H * r * W if fo else H * self.vd * (W + r)
        return float(qside + r * W + r + oside)

    def _folds(self):
        """(fold the queries' product, fold the values' product): by weight elements a token meets."""
        if self.absorb in (True, False):
            return bool(self.absorb), bool(self.absorb)
        W, r = self.hidden, self.rank
        return r * W <= self.hd * (W + r), r * W <= self.vd * (W + r)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n, H, d, dv, r = self.names, self.nh, self.hd, self.vd, self.rank
        self.width = D = record_width(r, r, rt.is_bf16)
        self.fold_q, self.fold_o = self._folds()
        wq, wdown = tensors[n["q"]], tensors[n["down"]]
        dt = wq.dtype if wq.dtype == wdown.dtype else torch.float32
        uk = tensors[n["up_k"]].reshape(H, d, r)
        uv = tensors[n["up_v"]].reshape(H, dv, r)
        wo = tensors[n["o"]]
        if self.fold_q:
            # rows h r ... h r + r - 1: Wuk_h^T Wq_h, the head's queries over the latent
            wq = torch.bmm(uk.double().transpose(1, 2), wq.double().reshape(H, d, self.hidden)).reshape(H * r, self.hidden)
            self.w_qc = None
        else:
            self.w_qc = uk.transpose(1, 2).contiguous()                    # grouped [head, r, d]
        self.w_in = torch.cat([wq.to(dt), wdown.to(dt)], dim=0).contiguous()            # [H (r | d) + r, hidden]
        self.q_cols = r if self.fold_q else d
        if self.fold_o:
            # columns h D ... h D + r - 1: Wo_h Wuv_h (zero beyond r, where the attended records hold zeros)
            ov = torch.bmm(wo.double().reshape(self.hidden, H, dv).transpose(0, 1), uv.double())     # [H, hidden, r]
            full = torch.zeros((self.hidden, H, D), dtype=torch.float64, device=ov.device)
            full[:, :, :r] = ov.transpose(0, 1)
            self.wo = full.reshape(self.hidden, H * D).to(wo.dtype).contiguous()
            self.w_cv = None
        else:
            self.w_cv = uv.contiguous()                                    # grouped [head, dv, r]
            self.wo = wo.contiguous()
        self.w_norm = tensors[n["down_norm"]].to(torch.float32).contiguous()
        self.sinks = tensors[n["sink"]].to(torch.float32).contiguous() if self.sink else False
        self._offsets = {}

    def _head_offsets(self, T, device):
        """Row offsets [0, T, 2T, ..., H T] of the heads in a grouped product."""
        o = self._offsets.get(T)
        if o is None:
            o = self._offsets[T] = (torch.arange(0, self.nh + 1, dtype=torch.int32, device=device) * T).contiguous()
        return o

    def forward(self, rt, h, batch, cache_view, state=None):
        T, D, H, dv, r = batch.num_tokens, self.width, self.nh, self.vd, self.rank
        dev = h.act.device
        proj = linear(rt, h.act, self.w_in)                       # [T, H (r | d) + r] 32-bit
        k_new = rt.empty((T, 1, D))
        # a step of one token a sequence reads its own key from the cache; whole prompts read nothing
        # from it: both may append at once.  A step that goes on from the cache appends afterwards.
        early = batch.all_decode or batch.all_fresh
        kw = dict(nh=H, d=self.q_cols, r=r, width=D, weight=self.w_norm, eps=self.eps, k_new=k_new,
                  commit=cache_view if early else None, status=rt.status)
        q = rt.empty((T, H, D))
        if self.fold_q:
            core.latent_prepare(proj, batch, q_t=q, token_major=True, **kw)
        else:
            q_t = rt.empty((H, T, self.hd))
            core.latent_prepare(proj, batch, q_t=q_t, **kw)
            offsets = self._head_offsets(T, dev)
            qc = grouped_linear(rt, q_t.view(H * T, self.hd), self.w_qc, offsets, H * T)      # [H T, r] 32-bit
            core.heads_transpose(qc.view(H, T, r), q, n=r)
        ctx = rt.empty((T, H, D))
        if batch.all_decode:
            core.attention_decode(q, cache_view, batch, ctx.view(T, H * D), nh=H, window=None, scale=self.scale,
                                  status=rt.status, sink=self.sinks)
        else:
            if getattr(batch, "has_padding", False):
                ctx.zero_()      # rows of no sequence are written by no attention kernel
            done = False
            if rt.is_bf16:
                from ..ops import tc

                if batch.all_fresh:
                    done = tc.attention_prefill(q, k_new, k_new, batch, ctx, nh=H, nkv=1, hd=D, window=None,
                                                scale=self.scale, status=rt.status, sink=self.sinks)
                else:
                    done = tc.attention_cached(q, k_new, k_new, cache_view, batch, ctx, nh=H, window=None,
                                               scale=self.scale, status=rt.status, sink=self.sinks)
            if not done:
                kw = dict(nh=H, window=None, scale=self.scale, use_local=True, status=rt.status, sink=self.sinks)
                if not core.attention_tiled(q, k_new, k_new, cache_view, batch, ctx, **kw):
                    core.attention_generic(q, k_new, k_new, cache_view, batch, ctx, **kw)
            if not early:
                core.kv_commit(k_new, k_new, cache_view, batch, rt.status)
        if self.fold_o:
            return linear(rt, ctx.view(T, H * D), self.wo)
        offsets = self._head_offsets(T, dev)
        c_t = rt.empty((H, T, r))
        core.heads_transpose(ctx, c_t, n=r)
        ov = grouped_linear(rt, c_t.view(H * T, r), self.w_cv, offsets, H * T)      # [H T, dv] 32-bit
        packed = rt.empty((T, H, dv))
        core.heads_transpose(ov.view(H, T, dv), packed, n=dv)
        return linear(rt, packed.view(T, H * dv), self.wo)


register_part("mixer", "latent_attention", LatentAttention)
