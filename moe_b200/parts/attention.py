"""Grouped-query attention with optional q/k/v bias, a position encoding of its own
kind and an optional sliding window (src/model.rs:689-834, Gqa at :42-50).

  q = Wq n + bq, k = Wk n + bk, v = Wv n + bv   (bias by tensor, :707-713)
  rotate q and k heads at the token's position (:729-731); cache k (rotated) and v (:733-734)
  scores over [lo, p], lo = max(0, p + 1 - window) with a window else 0 (:803-808)
  kv head of query head h is h / (heads / kv_heads) (:809); delta = Wo ctx, no bias (:829-833)

A layer with ``own_kv = False`` projects queries only and attends over the cache
entry another layer wrote.

Options beyond that (each a constant of the part; any of them takes the "prepared" path, whose
kernel ``heads_prepare`` stands where the rotation-and-split kernel stands otherwise):
  value_dim   size of a value head dv != head_dim d.  Keys and values are cached in records of one
              width D >= max(d, dv), zero-filled: zeros add nothing to q . k, and the output columns
              beyond dv are dropped.  D is also rounded up to a head size the fast kernels take.
  qk_norm     {"eps": e}: queries and keys are divided by their root mean square over the head,
              x / sqrt(mean(x^2) + e) * w, with one weight vector for all query heads and one for
              all key heads, before the rotation.
  scale       the factor on q . k, instead of 1 / sqrt(d).
  out_gate    the concatenated heads are multiplied by sigmoid(Wg n), n being the same input as
              the other projections'; Wg is one more block of rows of the fused projection.
  a position encoding whose cos and sin carry a factor (``cos_sin_scale``).

Options of the score and the mask, which every attention kernel of the 32-bit arithmetic takes
(``AttnVariant`` in csrc/common.cuh):
  chunk       position i sees j <= i with i // chunk == j // chunk, counted from the sequence's
              first position (instead of a window); the cache keeps a ring of one chunk.
  softcap     the scaled score s becomes cap * tanh(s / cap).
  sink        the softmax's denominator is 1 + sum_j exp(s_j): a term of score 0 without a value.
  o_bias      the output projection has a bias.

A second prepared path, whose kernel ``conv_heads_prepare`` stands in the same place, is taken by
  conv        {"taps": n}: a causal convolution over time on every channel of q, k and v right
              after the projection, y_t = sum_j w[:, j] u_(t - n + 1 + j) (tensors [channels, n]);
              the last n - 1 projected rows of a sequence are its state of fixed size;
  unit_norm   {"eps": e}: after the rotation, query and key heads are divided by their root mean
              square (no weight);
  a rotation of pairs (2i, 2i + 1) (position option ``interleaved``).

A third prepared path, whose kernel ``whole_prepare`` stands in the same place, is taken by
  qk_norm     {"eps": e, "whole": True}: ONE root mean square over all query channels of a token (and
              one over all key channels) before the split into heads, with a weight per channel
              (tensors of the projections' sizes);
  rotate_values  the value of position j is rotated by j over all of its dv dimensions, pair
              (m, m + dv/2) by j * theta^(-2m/dv) (theta: the position encoding's), and cached so; a
              head's output at position i is turned back by -i, so that every value arrives turned
              by its distance to the query;
  sigmoid     the weight of a visible key is sigmoid(score + b_h), b_h a learned number per head
              (tensor role ``head_bias``), and the weights are not normalised over the keys.
"""
from __future__ import annotations

import math
import os

import torch

from ..cache.kv import KVRequest
from ..config.spec import PartSpec
from ..ops import core
from ..ops.linear import linear
from .base import Part, TensorSpec, make_part, register_part


def record_width(d: int, dv: int, bf16: bool) -> int:
    """Width of a cached key/value record for heads of d (queries, keys) and dv (values): in
    bfloat16 the tensor-core attention takes 64 and 128, everything takes multiples of 16."""
    m = max(d, dv)
    if bf16 and m <= 128:
        return 64 if m <= 64 else 128
    return -(-m // 16) * 16


class GQAttention(Part):
    category, kind = "mixer", "gqa_attention"
    graph_safe = True
    default_names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                     "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                     "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "gate": "gate_proj.weight",
                     "o_bias": "o_proj.bias", "q_conv": "q_conv.weight", "k_conv": "k_conv.weight",
                     "v_conv": "v_conv.weight", "head_bias": "head_bias"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.bias = bool(p.get("qkv_bias", False))
        self.window = p.get("window")
        self.own_kv = bool(p.get("own_kv", True))
        self.vd = int(p.get("value_dim") or self.hd)
        self.qk_norm = p.get("qk_norm")
        self.out_gate = bool(p.get("out_gate", False))
        self.fixed_scale = p.get("scale")
        self.chunk = int(p.get("chunk") or 0)
        self.softcap = float(p.get("softcap") or 0.0)
        self.sink = bool(p.get("sink", False))
        self.o_bias = bool(p.get("o_bias", False))
        self.taps = int((p.get("conv") or {}).get("taps", 0) or 0)
        self.unit_norm = p.get("unit_norm")
        self.whole_norm = bool((self.qk_norm or {}).get("whole", False))
        self.rotate_values = bool(p.get("rotate_values", False))
        self.sigmoid = bool(p.get("sigmoid", False))
        self.whole_path = self.whole_norm or self.rotate_values or self.sigmoid
        pos = dict(p.get("position") or {"kind": "none"})
        self.position = make_part("position", PartSpec(pos.pop("kind"), pos, spec.prefix))
        # the prepared path: a kernel of its own between projection and attention, records of width D
        self.cos_sin_scale = float(getattr(self.position, "cos_sin_scale", lambda: 1.0)())
        self.prepared = bool(self.vd != self.hd or self.qk_norm or self.out_gate or self.hd % 16
                             or self.cos_sin_scale != 1.0)
        self.conv_path = bool(self.taps or self.unit_norm or getattr(self.position, "interleaved", False))
        self.variant = dict(chunk=self.chunk, softcap=self.softcap, sink=self.sink)
        self.plain_scores = not (self.chunk or self.softcap or self.sink)    # what the fused decode kernel computes
        if self.whole_path:
            if (self.conv_path or self.out_gate or self.bias or self.sink or not self.own_kv or self.cos_sin_scale != 1.0
                    or (self.qk_norm and not self.whole_norm)):
                raise ValueError("whole-projection norm, rotated values and sigmoid weights go with none of: convolution, "
                                 "unit norm, pairs (2i, 2i + 1), output gate, biases, sink, another layer's cache, "
                                 "scaled cos and sin, a per-head q/k norm")
            if self.rotate_values and self.vd % 2:
                raise ValueError("rotated values need an even value size")
            if not (0 < self.hd <= 256 and 0 < self.vd <= 256):
                raise ValueError(f"head sizes {self.hd} / {self.vd}: the attention kernels take up to 256")
            self.prepared = False
            self.plain_scores = False
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.chunk < 0 or self.softcap < 0 or self.taps < 0 or self.taps > 16:
            raise ValueError("chunk and softcap must not be negative; a convolution has 1 to 16 taps")
        if self.chunk and self.window is not None:
            raise ValueError("a layer's mask is a window or chunks, not both")
        if self.conv_path:
            if not self.own_kv or self.qk_norm or self.out_gate or self.cos_sin_scale != 1.0:
                raise ValueError("the convolution path takes none of own_kv=False, qk_norm, out_gate, scaled cos and sin")
            if not (0 < self.hd <= 256 and 0 < self.vd <= 256):
                raise ValueError(f"head sizes {self.hd} / {self.vd}: the attention kernels take up to 256")
            self.prepared = False
        elif (self.chunk or self.softcap or self.sink) and not self.prepared and not self.whole_path:
            self.prepared = True          # the path whose every step takes the kernels with these options
        if self.prepared:
            if not self.own_kv:
                raise ValueError("a layer that reads another layer's cache takes none of value_dim, qk_norm, out_gate")
            if not (0 < self.hd <= 256 and 0 < self.vd <= 256):
                raise ValueError(f"head sizes {self.hd} / {self.vd}: the attention kernels take up to 256")
        elif not self.conv_path and not self.whole_path and (self.hd % 16 or not 16 <= self.hd <= 256):
            raise ValueError(f"head_dim {self.hd}: the attention kernels take multiples of 16 from 16 to 256")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive")
        self.width = self.hd          # of a cached record; the prepared path sets it when bound

    def tensors(self):
        n = self.names
        t = {
            n["q"]: TensorSpec((self.nh * self.hd, self.hidden)),
            n["o"]: TensorSpec((self.hidden, self.nh * self.vd)),
        }
        if self.own_kv:
            t[n["k"]] = TensorSpec((self.nkv * self.hd, self.hidden))
            t[n["v"]] = TensorSpec((self.nkv * self.vd, self.hidden))
        if self.bias:
            t[n["q_bias"]] = TensorSpec((self.nh * self.hd,), vector=True)
            if self.own_kv:
                t[n["k_bias"]] = TensorSpec((self.nkv * self.hd,), vector=True)
                t[n["v_bias"]] = TensorSpec((self.nkv * self.vd,), vector=True)
        if self.qk_norm:
            t[n["q_norm"]] = TensorSpec((self.nh * self.hd if self.whole_norm else self.hd,), init="ones", vector=True)
            t[n["k_norm"]] = TensorSpec((self.nkv * self.hd if self.whole_norm else self.hd,), init="ones", vector=True)
        if self.sigmoid:
            t[n["head_bias"]] = TensorSpec((self.nh,), init="zeros", vector=True)
        if self.out_gate:
            t[n["gate"]] = TensorSpec((self.nh * self.vd, self.hidden))
        if self.o_bias:
            t[n["o_bias"]] = TensorSpec((self.hidden,), init="zeros", vector=True)
        if self.taps:
            t[n["q_conv"]] = TensorSpec((self.nh * self.hd, self.taps))
            t[n["k_conv"]] = TensorSpec((self.nkv * self.hd, self.taps))
            t[n["v_conv"]] = TensorSpec((self.nkv * self.vd, self.taps))
        t.update(self.position.tensors())
        return t

    def kv_request(self):
        # (chunks: no query looks further back than its chunk's start, so a ring of one chunk is enough)
        return KVRequest(self.nkv, self.width, self.window if not self.chunk else self.chunk)

    @property
    def channels(self):
        return (self.nh + self.nkv) * self.hd + self.nkv * self.vd

    def describe(self):
        d = f"GQA({self.nh} q / {self.nkv} kv heads, head_dim={self.hd}{', bias' if self.bias else ''})"
        if self.vd != self.hd:
            d += f", value heads of {self.vd}"
        if self.qk_norm:
            d += ", q/k RMS norm" + (" over the whole projection" if self.whole_norm else "")
        if self.rotate_values:
            d += ", values rotated by their distance"
        if self.sigmoid:
            d += ", sigmoid weights with a bias a head"
        if self.out_gate:
            d += ", sigmoid output gate"
        if self.taps:
            d += f", convolution of {self.taps} taps on q, k, v"
        d += f", {self.position.describe()}"
        if self.unit_norm:
            d += ", q/k unit RMS after the rotation"
        if self.softcap:
            d += f", scores capped at {self.softcap:g}"
        if self.sink:
            d += ", softmax with a sink"
        if self.chunk:
            d += f", chunks of {self.chunk}"
        if self.window:
            d += f", window {self.window}"
        if not self.own_kv:
            d += ", reads another layer's cache"
        return d

    def state_request(self):
        """The last taps - 1 projected rows [q | k | v] of a sequence, which the convolution of its next
        tokens reads."""
        if self.taps > 1:
            from ..cache.kv import StateRequest

            return StateRequest(((self.taps - 1) * self.channels,), torch.float32)
        return None

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        roles = ["q", "k", "v"] if self.own_kv else ["q"]
        ws = [tensors[n[r]] for r in roles]
        if self.out_gate:
            ws.append(tensors[n["gate"]])        # the gate's rows ride in the same product
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.wqkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.bqkv = None
        if self.bias:
            bs = [tensors[n[r + "_bias"]].to(torch.float32) for r in roles]
            if self.out_gate:
                bs.append(torch.zeros(self.nh * self.vd, dtype=torch.float32, device=bs[0].device))
            self.bqkv = torch.cat(bs).contiguous()
        self.wo = tensors[n["o"]].contiguous()
        self.bo = tensors[n["o_bias"]].to(torch.float32).contiguous() if self.o_bias else None
        self.taps_w = None
        if self.taps:
            # [taps, channels]: a tap's factors for all channels side by side
            self.taps_w = torch.cat([tensors[n[r + "_conv"]].to(torch.float32) for r in ("q", "k", "v")], dim=0).t().contiguous()
        self.q_norm_w = self.k_norm_w = None
        if self.qk_norm:
            self.q_norm_w = tensors[n["q_norm"]].to(torch.float32).contiguous()
            self.k_norm_w = tensors[n["k_norm"]].to(torch.float32).contiguous()
        self.position.bind(tensors, rt)
        self.scale = (float(self.fixed_scale) if self.fixed_scale is not None
                      else self.position.attention_scale() / math.sqrt(self.hd))
        if self.prepared or self.conv_path or self.whole_path:
            self.width = record_width(self.hd, self.vd, rt.is_bf16)
        self.vfreq = None
        if self.rotate_values:
            from .rope import rotary_inv_freq

            self.vfreq = rotary_inv_freq(float(getattr(self.position, "theta", 10000.0)), self.vd).to(rt.device)
        if self.sigmoid:
            self.variant = dict(self.variant, sink=core.SigmoidWeights(tensors[n["head_bias"]].to(torch.float32).contiguous()))
        # Single-token steps append in heads_prepare and attend with the split kernel, whose merge gates
        # and packs (three launches).  MOE_B200_PREPARED_FUSED=1 takes the fused decode kernel instead
        # (two launches); measured slower on a B200 at widths of 2,048 and 4,096 (0.61 against 0.55 ms a
        # step at one sequence, 1.33 against 1.27 at 64), so it is off by default.
        self._fused_decode = os.environ.get("MOE_B200_PREPARED_FUSED", "0") == "1"

    def _forward_prepared(self, rt, h, batch, cache_view):
        """Projection (queries, keys, values and gate logits in one product) -> per-head norm,
        rotation, split and append -> attention over records of width D -> gate and packing ->
        output projection."""
        T, D, nh, nkv = batch.num_tokens, self.width, self.nh, self.nkv
        proj = linear(rt, h.act, self.wqkv, bias=self.bqkv)
        table, rot = self.position.rotary_table()
        g0 = (nh + nkv) * self.hd + nkv * self.vd
        gate = proj[:, g0:g0 + nh * self.vd] if self.out_gate else None
        prep = dict(nh=nh, nkv=nkv, d=self.hd, dv=self.vd, width=D, q_norm=self.q_norm_w, k_norm=self.k_norm_w,
                    eps=float(self.qk_norm["eps"]) if self.qk_norm else 0.0, freq=table, rot=rot,
                    mscale=self.cos_sin_scale, status=rt.status)
        if batch.all_decode and self._fused_decode:
            # one token a sequence: the prepared heads stay 32-bit in one row [q | k | v], and ONE more
            # launch appends key and value, attends over the cache split along the keys, merges the
            # splits, multiplies by the gate and packs the heads
            row = torch.empty((T, nh + 2 * nkv, D), dtype=torch.float32, device=proj.device)
            core.heads_prepare(proj, batch.pos, batch.seq_of_token, q=row[:, :nh], k=row[:, nh:nh + nkv],
                               v=row[:, nh + nkv:], **prep)
            packed = rt.empty((T, nh * self.vd))
            if self.plain_scores and core.attention_decode_fused(
                    row.view(T, -1), None, 0, cache_view, batch, packed, nh=nh, window=self.window, scale=self.scale,
                    status=rt.status, gate=gate, dv=self.vd):
                return linear(rt, packed, self.wo, bias=self.bo)
            self._fused_decode = False       # a head size the fused kernel does not take
        q = rt.empty((T, nh, D))
        k_new, v_new = rt.empty((T, nkv, D)), rt.empty((T, nkv, D))
        ctx = rt.empty((T, nh, D))
        if getattr(batch, "has_padding", False) and not batch.all_decode:
            ctx.zero_()      # rows of no sequence are written by no attention kernel
        # a step of one token a sequence reads its own key from the cache; whole prompts read nothing
        # from it: both may append at once.  A step that goes on from the cache appends afterwards.
        early = batch.all_decode or batch.all_fresh
        core.heads_prepare(proj, batch.pos, batch.seq_of_token, q=q, k=k_new, v=v_new,
                           commit=(cache_view, batch) if early else None, **prep)
        return self._attend_prepared(rt, batch, cache_view, q, k_new, v_new, ctx, gate, early)

    def _forward_conv(self, rt, h, batch, cache_view, state):
        """Projection -> convolution over time (with the sequence's state), rotation of pairs
        (2i, 2i + 1), unit norm, split and append -> attention over records of width D -> packing ->
        output projection."""
        T, D, nh, nkv = batch.num_tokens, self.width, self.nh, self.nkv
        proj = linear(rt, h.act, self.wqkv, bias=self.bqkv)
        table, rot = self.position.rotary_table()
        q = rt.empty((T, nh, D))
        k_new, v_new = rt.empty((T, nkv, D)), rt.empty((T, nkv, D))
        ctx = rt.empty((T, nh, D))
        if getattr(batch, "has_padding", False) and not batch.all_decode:
            ctx.zero_()
        early = batch.all_decode or batch.all_fresh
        core.conv_heads_prepare(proj, batch, nh=nh, nkv=nkv, d=self.hd, dv=self.vd, width=D, q=q, k=k_new, v=v_new,
                                taps_w=self.taps_w, state=state, eps=float((self.unit_norm or {}).get("eps", 0.0)),
                                unit_norm=bool(self.unit_norm), freq=table, rot=rot,
                                commit=cache_view if early else None, status=rt.status)
        if self.taps > 1:
            core.conv_state_update(proj, state, batch, taps=self.taps, channels=self.channels)
        return self._attend_prepared(rt, batch, cache_view, q, k_new, v_new, ctx, None, early)

    def _forward_whole(self, rt, h, batch, cache_view):
        """Projection -> norm over the whole of q and of k, rotation of q and k, rotation of the values,
        split and append -> attention over records of width D -> the output turned back and packed ->
        output projection."""
        T, D, nh, nkv = batch.num_tokens, self.width, self.nh, self.nkv
        proj = linear(rt, h.act, self.wqkv)
        table, rot = self.position.rotary_table()
        q = rt.empty((T, nh, D))
        k_new, v_new = rt.empty((T, nkv, D)), rt.empty((T, nkv, D))
        ctx = rt.empty((T, nh, D))
        if getattr(batch, "has_padding", False) and not batch.all_decode:
            ctx.zero_()
        early = batch.all_decode or batch.all_fresh
        core.whole_prepare(proj, batch, nh=nh, nkv=nkv, d=self.hd, dv=self.vd, width=D, q=q, k=k_new, v=v_new,
                           q_norm=self.q_norm_w, k_norm=self.k_norm_w, eps=float(self.qk_norm["eps"]) if self.qk_norm else 0.0,
                           freq=table, rot=rot, vfreq=self.vfreq, commit=cache_view if early else None, status=rt.status)
        return self._attend_prepared(rt, batch, cache_view, q, k_new, v_new, ctx, None, early)

    def _attend_prepared(self, rt, batch, cache_view, q, k_new, v_new, ctx, gate, early):
        """Attention over prepared records of width D, packing (and gate), output projection."""
        T, D, nh, nkv = batch.num_tokens, self.width, self.nh, self.nkv
        if batch.all_decode and self.rotate_values:
            # (the merge of the splits leaves whole records; the turn back packs them)
            core.attention_decode(q, cache_view, batch, ctx, nh=nh, window=self.window, scale=self.scale,
                                  status=rt.status, **self.variant)
        elif batch.all_decode:
            # (the merge of the splits multiplies by the gate and packs the heads)
            packed = rt.empty((T, nh * self.vd))
            core.attention_decode(q, cache_view, batch, packed, nh=nh, window=self.window, scale=self.scale,
                                  status=rt.status, gate=gate, dv=self.vd, **self.variant)
            return linear(rt, packed, self.wo, bias=self.bo)
        else:
            done = False
            if rt.is_bf16:
                from ..ops import tc

                if batch.all_fresh:
                    done = tc.attention_prefill(q, k_new, v_new, batch, ctx, nh=nh, nkv=nkv, hd=D, window=self.window,
                                                scale=self.scale, status=rt.status, **self.variant)
                else:
                    done = tc.attention_cached(q, k_new, v_new, cache_view, batch, ctx, nh=nh, window=self.window,
                                               scale=self.scale, status=rt.status, **self.variant)
            if not done:
                kw = dict(nh=nh, window=self.window, scale=self.scale, use_local=True, status=rt.status, **self.variant)
                if not core.attention_tiled(q, k_new, v_new, cache_view, batch, ctx, **kw):
                    core.attention_generic(q, k_new, v_new, cache_view, batch, ctx, **kw)
            if not early:
                core.kv_commit(k_new, v_new, cache_view, batch, rt.status)
        if self.rotate_values:
            packed = rt.empty((T, nh * self.vd))
            core.unrotate_pack(ctx, batch.pos, self.vfreq, packed, nh=nh, dv=self.vd, width=D)
        elif self.out_gate or D != self.vd:
            packed = rt.empty((T, nh * self.vd))
            core.gate_pack(ctx, packed, nh=nh, dv=self.vd, width=D, gate=gate)
        else:
            packed = ctx.view(T, nh * D)
        return linear(rt, packed, self.wo, bias=self.bo)

    def forward(self, rt, h, batch, cache_view, state=None):
        if self.conv_path:
            return self._forward_conv(rt, h, batch, cache_view, state)
        if self.whole_path:
            return self._forward_whole(rt, h, batch, cache_view)
        if self.prepared:
            return self._forward_prepared(rt, h, batch, cache_view)
        T = batch.num_tokens
        nkv = self.nkv if self.own_kv else 0
        qkv = linear(rt, h.act, self.wqkv, bias=self.bqkv)
        table, rot = self.position.rotary_table()
        if table is None and hasattr(self.position, "apply"):
            self.position.apply(rt, qkv, self.nh, nkv, self.hd, batch.pos)
        ctx = rt.empty((T, self.nh * self.hd))
        if getattr(batch, "has_padding", False) and not batch.all_decode:
            ctx.zero_()      # rows of no sequence are written by no attention kernel
        if batch.all_decode and self.own_kv:
            # one token per sequence: rotation, append, attention split along the keys and the
            # merge in ONE launch where the head size allows it
            if core.attention_decode_fused(qkv, table, rot, cache_view, batch, ctx, nh=self.nh, window=self.window,
                                           scale=self.scale, status=rt.status):
                return linear(rt, ctx, self.wo, bias=self.bo)
            # else: rotate and append in one launch, then attend over the cache alone
            q = rt.empty((T, self.nh, self.hd))
            core.rope_commit(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, cache_view, batch, rt.status)
            core.attention_decode(q, cache_view, batch, ctx, nh=self.nh, window=self.window, scale=self.scale,
                                  status=rt.status)
            return linear(rt, ctx, self.wo, bias=self.bo)
        q = rt.empty((T, self.nh, self.hd))
        k_new = rt.empty((T, max(nkv, 1), self.hd))
        v_new = rt.empty((T, max(nkv, 1), self.hd))
        # whole prompts read nothing from the cache, so their keys and values may go there at once
        early = batch.all_fresh and self.own_kv and not batch.all_decode
        committed = early and core.rope_split(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, k_new, v_new,
                                              commit=(cache_view, batch), status=rt.status)
        if not committed:
            core.rope_split(qkv, batch.pos, table, self.nh, nkv, self.hd, rot, q, k_new, v_new)
        if batch.all_decode:
            # a layer that reads another layer's cache: queries only
            core.attention_decode(q, cache_view, batch, ctx, nh=self.nh, window=self.window, scale=self.scale,
                                  status=rt.status)
        else:
            done = False
            if batch.all_fresh and self.own_kv and rt.is_bf16:
                # whole prompts: nothing is read from the cache; tensor-core kernel
                from ..ops import tc

                done = tc.attention_prefill(q, k_new, v_new, batch, ctx, nh=self.nh, nkv=self.nkv, hd=self.hd,
                                            window=self.window, scale=self.scale, status=rt.status)
            elif self.own_kv and rt.is_bf16:
                # keys of earlier steps from the pages of the cache, keys of this step from its own
                # buffers; the same tensor-core kernel
                from ..ops import tc

                done = tc.attention_cached(q, k_new, v_new, cache_view, batch, ctx, nh=self.nh, window=self.window,
                                           scale=self.scale, status=rt.status)
            if not done:
                # the same on the CUDA cores in 32-bit arithmetic, 64 queries to a block (the plain
                # kernel where that one declines)
                kw = dict(nh=self.nh, window=self.window, scale=self.scale, use_local=self.own_kv, status=rt.status)
                if not core.attention_tiled(q, k_new, v_new, cache_view, batch, ctx, **kw):
                    core.attention_generic(q, k_new, v_new, cache_view, batch, ctx, **kw)
            if self.own_kv and not committed:
                core.kv_commit(k_new, v_new, cache_view, batch, rt.status)
        return linear(rt, ctx, self.wo, bias=self.bo)


register_part("mixer", "gqa_attention", GQAttention)
