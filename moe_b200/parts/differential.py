"""Differential attention: every head runs two softmax attentions ("maps") over the same values
and takes their difference.

With n the layer's normed input, H heads on G key/value heads, d the query/key size of a map and dv
the value size:
    q = Wq n + bq   [H, 2, d]      k = Wk n + bk   [G, 2, d]      v = Wv n + bv   [G, dv]
    (checkpoint rows head by head, map 1 then map 2 inside a head)
    both maps of q and k are rotated at the token's position (the position part's kind and constants)
    a_m = softmax over the seen keys of f(scale q_m . k_m) v,  m = 1, 2; f caps the score (``softcap``),
          a window bounds what is seen; query head h reads key/value head h // (H / G)
    lambda = exp(sum lq1 * lk1) - exp(sum lq2 * lk2) + diff       (four learned vectors of d; one number a layer)
    o = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - diff)  over the head's dv values
    o <- o * sigmoid(Wg n)_h  (one gate logit a head; optional);  out = Wo [o_1 ... o_H]

How it runs.  The maps are heads of their own for everything the library already has: the fused
projection's rows are re-ordered when bound to [map 1 of all heads | map 2 of all heads] for queries
and for keys, so that 2H query heads on 2G key heads keep the usual rule "query head i reads key head
i // (2H / 2G)", and the value rows stand twice, once per map.  Projection, rotation, split, append,
cache, ring of the window and every attention kernel are the ones of ``GQAttention``'s prepared
path (records of one width D >= max(d, dv)).  One kernel of its own, ``diff_combine``, joins the two
maps, normalises, gates and packs the heads for the output projection.  The cache holds the values
once per map, which is what it costs not to give the cache a head count of its own for values.

32-bit in both dtypes: positions, angles and the rotation, scores, cap, softmax, lambda, the
difference, the head's norm and the gate's sigmoid.  The bfloat16 path rounds the queries, the cache
and each map's output (as every attention kernel stores it) before the difference is formed.
"""
from __future__ import annotations

import torch

from ..cache.kv import KVRequest
from ..config.spec import PartSpec
from ..ops import core
from ..ops.linear import linear
from .attention import record_width
from .base import Part, TensorSpec, make_part, register_part


class DifferentialAttention(Part):
    category, kind = "mixer", "diff_attention"
    graph_safe = True
    default_names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                     "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
                     "lq1": "lambda_q1", "lk1": "lambda_k1", "lq2": "lambda_q2", "lk2": "lambda_k2",
                     "gate": "gate_proj.weight"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv = int(p["num_heads"]), int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])                       # of one map
        self.vd = int(p.get("value_dim") or self.hd)
        self.bias = bool(p.get("qkv_bias", False))
        self.window = p.get("window")
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.diff = float(p["diff"])
        self.eps = float(p["eps"])
        self.out_gate = bool(p.get("out_gate", False))
        pos = dict(p.get("position") or {"kind": "none"})
        self.position = make_part("position", PartSpec(pos.pop("kind"), pos, spec.prefix))
        self.cos_sin_scale = float(getattr(self.position, "cos_sin_scale", lambda: 1.0)())
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (0 < self.hd <= 256 and 0 < self.vd <= 256):
            raise ValueError(f"head sizes {self.hd} / {self.vd}: the attention kernels take up to 256")
        if self.window is not None and self.window <= 0:
            raise ValueError("window must be positive")
        if getattr(self.position, "interleaved", False):
            raise ValueError("differential attention rotates pairs (i, i + r/2)")
        self.width = max(self.hd, self.vd)                 # of a cached record; set when bound
        self.variant = dict(softcap=self.softcap)

    def tensors(self):
        n, H, G, d, dv, W = self.names, self.nh, self.nkv, self.hd, self.vd, self.hidden
        t = {n["q"]: TensorSpec((H * 2 * d, W)), n["k"]: TensorSpec((G * 2 * d, W)), n["v"]: TensorSpec((G * dv, W)),
             n["o"]: TensorSpec((W, H * dv))}
        if self.bias:
            t[n["q_bias"]] = TensorSpec((H * 2 * d,), vector=True)
            t[n["k_bias"]] = TensorSpec((G * 2 * d,), vector=True)
            t[n["v_bias"]] = TensorSpec((G * dv,), vector=True)
        for r in ("lq1", "lk1", "lq2", "lk2"):
            t[n[r]] = TensorSpec((d,), vector=True)
        if self.out_gate:
            t[n["gate"]] = TensorSpec((H, W))
        t.update(self.position.tensors())
        return t

    def kv_request(self):
        return KVRequest(2 * self.nkv, self.width, self.window)

    def state_request(self):
        return None

    def describe(self):
        d = (f"differential attention ({self.nh} heads of two maps / {self.nkv} kv heads, map size {self.hd}, values of "
             f"{self.vd}{', bias' if self.bias else ''}), lambda offset {self.diff:g}")
        if self.out_gate:
            d += ", one sigmoid gate a head"
        d += f", {self.position.describe()}"
        if self.softcap:
            d += f", scores capped at {self.softcap:g}"
        if self.window:
            d += f", window {self.window}"
        return d

    def _maps_first(self, t, heads, size):
        """Rows [head][map][size] -> [map][head][size]."""
        rest = t.shape[1:]
        return t.reshape(heads, 2, size, *rest).transpose(0, 1).reshape(2 * heads * size, *rest)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n, H, G, d, dv = self.names, self.nh, self.nkv, self.hd, self.vd
        ws = [self._maps_first(tensors[n["q"]], H, d), self._maps_first(tensors[n["k"]], G, d),
              tensors[n["v"]], tensors[n["v"]]]
        if self.out_gate:
            ws.append(tensors[n["gate"]])          # the gate's rows ride in the same product
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.wqkv = torch.cat([w.to(dt) for w in ws], dim=0).contiguous()
        self.bqkv = None
        if self.bias:
            bv = tensors[n["v_bias"]].to(torch.float32)
            bs = [self._maps_first(tensors[n["q_bias"]].to(torch.float32), H, d),
                  self._maps_first(tensors[n["k_bias"]].to(torch.float32), G, d), bv, bv]
            if self.out_gate:
                bs.append(torch.zeros(H, dtype=torch.float32, device=bv.device))
            self.bqkv = torch.cat(bs).contiguous()
        self.wo = tensors[n["o"]].contiguous()
        l = {r: tensors[n[r]].to(torch.float32) for r in ("lq1", "lk1", "lq2", "lk2")}
        # one number a layer, formed once in 32-bit
        self.lam = float((torch.exp((l["lq1"] * l["lk1"]).sum()) - torch.exp((l["lq2"] * l["lk2"]).sum())
                          + torch.tensor(self.diff, dtype=torch.float32, device=l["lq1"].device)).item())
        self.position.bind(tensors, rt)
        self.width = record_width(d, dv, rt.is_bf16)

    def forward(self, rt, h, batch, cache_view, state=None):
        T, D, H = batch.num_tokens, self.width, self.nh
        nh, nkv, d, dv = 2 * H, 2 * self.nkv, self.hd, self.vd
        proj = linear(rt, h.act, self.wqkv, bias=self.bqkv)
        table, rot = self.position.rotary_table()
        g0 = (nh + nkv) * d + nkv * dv
        gate = proj[:, g0:g0 + H] if self.out_gate else None
        q = rt.empty((T, nh, D))
        k_new, v_new = rt.empty((T, nkv, D)), rt.empty((T, nkv, D))
        # a step of one token a sequence reads its own key from the cache; whole prompts read nothing
        # from it: both may append at once.  A step that goes on from the cache appends afterwards.
        early = batch.all_decode or batch.all_fresh
        core.heads_prepare(proj, batch.pos, batch.seq_of_token, q=q, k=k_new, v=v_new, nh=nh, nkv=nkv, d=d, dv=dv,
                           width=D, freq=table, rot=rot, mscale=self.cos_sin_scale,
                           commit=(cache_view, batch) if early else None, status=rt.status)
        if batch.all_decode:
            ctx = rt.empty((T, nh, D))
            core.attention_decode(q, cache_view, batch, ctx.view(T, nh * D), nh=nh, window=self.window, scale=self.scale,
                                  status=rt.status, **self.variant)
        else:
            ctx = rt.empty((T, nh, D))
            if getattr(batch, "has_padding", False):
                ctx.zero_()      # rows of no sequence are written by no attention kernel
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
        packed = rt.empty((T, H * dv))
        core.diff_combine(ctx, packed, nh=H, dv=dv, width=D, lam=self.lam, eps=self.eps, mult=1.0 - self.diff, gate=gate)
        return linear(rt, packed, self.wo)


register_part("mixer", "diff_attention", DifferentialAttention)
