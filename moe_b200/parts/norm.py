"""Norms of the residual stream.

RMSNorm: s = 1/sqrt(mean(x^2) + eps), out = x * s * w (src/model.rs:211-216).
DynamicTanh: out = tanh(alpha x) * w + b with a scalar alpha; no statistic of x enters.
Both add a pending delta to the 32-bit stream inside their kernel before they normalise it."""
from __future__ import annotations

import torch

from ..ops import core
from .base import Activations, LazyDelta, Part, TensorSpec, register_part


class RMSNorm(Part):
    category, kind = "norm", "rmsnorm"
    graph_safe = True
    lazy_kinds = ("expert_combine", "scaled_pair")      # deltas this norm forms inside its own kernel
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.eps = float(self.params["eps"])
        # a weight stored around zero: the factor is offset + w (the sum is formed once, in 32-bit, when bound)
        self.offset = float(self.params.get("offset", 0.0) or 0.0)

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.size,), init="zeros" if self.offset else "ones", vector=True)}

    def describe(self):
        return f"RMSNorm eps {self.eps:g}" + (f", weight {self.offset:g} + w" if self.offset else "")

    def rms_params(self):
        """(weight, eps): what a neighbour needs to run this norm inside a kernel of its own (a
        feed-forward that fuses the norm before it with its first step asks for this; a norm
        that is no plain RMS norm simply has no such method)."""
        return self.weight, self.eps

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.names["weight"]].to(torch.float32).contiguous()
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def normed32(self, rt, t):
        out = rt.empty(t.shape, torch.float32)
        core.rmsnorm(t, self.weight, self.eps, out32=out, write_back=False, status=rt.status)
        return out

    def forward_pair(self, rt, x, delta, other):
        """This norm and ``other`` (an RMS norm of the same size and eps with a weight of its own) of the
        same x + delta in one kernel with one statistic: (Activations, Activations), both 32-bit only, or
        None where that is not possible (the caller then runs the two norms one after the other)."""
        if (not isinstance(other, RMSNorm) or other.eps != self.eps or other.size != self.size
                or not isinstance(delta, LazyDelta) or delta.kind != "scaled_pair"):
            return None
        b, combine = delta.b, None
        if isinstance(b, LazyDelta):
            if b.kind == "expert_combine" and b.shared_gate is None:
                b, combine = None, (b.y, b.pos_of_pair, b.topk_w, b.top_k, b.shared)
            else:
                b = b.materialize(rt)
        o1, o2 = rt.empty(x.shape, torch.float32), rt.empty(x.shape, torch.float32)
        core.rmsnorm_scaled(x, delta.a, delta.sa, b, delta.sb, self.weight, self.eps, out32=o1, write_back=True,
                            status=rt.status, combine=combine, second=(other.weight, o2))
        return Activations(act=o1, f32=o1), Activations(act=o2, f32=o2)

    def forward(self, rt, x, delta=None, rows=None, want32=False, write_back=True) -> Activations:
        """Normalise ``x (+ delta)``; with ``delta`` the sum is written back into ``x``
        (unless ``rows`` selects a subset, which leaves ``x`` alone)."""
        n = x.shape[0] if rows is None else rows.numel()
        out32 = out16 = None
        if rt.is_bf16:
            out16 = rt.empty((n, self.size), torch.bfloat16)
            if want32:
                out32 = rt.empty((n, self.size), torch.float32)
        else:
            out32 = rt.empty((n, self.size), torch.float32)
        if isinstance(delta, LazyDelta) and delta.kind == "scaled_pair":
            # two sublayers' outputs times their per-channel factors, the residual sum and the norm
            b, combine = delta.b, None
            if isinstance(b, LazyDelta):
                if b.kind == "expert_combine" and b.shared_gate is None:
                    # the experts' combine inside this kernel too
                    b, combine = None, (b.y, b.pos_of_pair, b.topk_w, b.top_k, b.shared)
                else:
                    b = b.materialize(rt)
            core.rmsnorm_scaled(x, delta.a, delta.sa, b, delta.sb, self.weight, self.eps, rows=rows, out32=out32,
                                out16=out16, write_back=write_back, status=rt.status, combine=combine)
            return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)
        if isinstance(delta, LazyDelta):
            if delta.kind != "expert_combine" or not core.rmsnorm_combine(
                    x, delta, self.weight, self.eps, rows=rows, out32=out32, out16=out16, write_back=write_back,
                    status=rt.status):
                delta = delta.materialize(rt)
            else:
                return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)
        core.rmsnorm(x, self.weight, self.eps, delta=delta, rows=rows, out32=out32, out16=out16,
                     write_back=write_back, status=rt.status)
        return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)


class DynamicTanh(Part):
    """tanh(alpha * x) * weight + shift.  Where the delta it is handed is the output of a sublayer
    that has a Dynamic Tanh of its own in front of the residual sum (``PostNormDelta`` of kind
    ``post_dyt``), both norms and the sum are one kernel."""

    category, kind = "norm", "dyt"
    graph_safe = True
    lazy_kinds = ("post_dyt",)
    default_names = {"weight": "weight", "shift": "bias", "alpha": "alpha"}

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])

    def tensors(self):
        n = self.names
        return {n["weight"]: TensorSpec((self.size,), init="ones", vector=True),
                n["shift"]: TensorSpec((self.size,), init="zeros", vector=True),
                n["alpha"]: TensorSpec((), init="ones", vector=True)}

    def describe(self):
        return "Dynamic Tanh"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.weight = tensors[n["weight"]].to(torch.float32).contiguous()
        self.shift = tensors[n["shift"]].to(torch.float32).contiguous()
        self.alpha = tensors[n["alpha"]].to(torch.float32).reshape(()).contiguous()

    def triple(self):
        return self.alpha, self.weight, self.shift

    def normed32(self, rt, t):
        out = rt.empty(t.shape, torch.float32)
        core.dyt(t, self.triple(), out32=out, write_back=False, status=rt.status)
        return out

    def forward(self, rt, x, delta=None, rows=None, want32=False, write_back=True) -> Activations:
        n = x.shape[0] if rows is None else rows.numel()
        out32 = out16 = None
        if rt.is_bf16:
            out16 = rt.empty((n, self.size), torch.bfloat16)
            if want32:
                out32 = rt.empty((n, self.size), torch.float32)
        else:
            out32 = rt.empty((n, self.size), torch.float32)
        post = None
        if isinstance(delta, LazyDelta):
            if delta.kind == "post_dyt":
                post, delta = delta.norm.triple(), delta.tensor
            else:
                delta = delta.materialize(rt)
        core.dyt(x, self.triple(), delta=delta, post=post, rows=rows, out32=out32, out16=out16, write_back=write_back,
                 status=rt.status)
        return Activations(act=out16 if rt.is_bf16 else out32, f32=out32)


class ChannelScale(Part):
    """A per-channel factor on a sublayer's output ("layer scale")."""

    category, kind = "scale", "channel_scale"
    graph_safe = True
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.size,), init="ones", vector=True)}

    def describe(self):
        return "per-channel scale"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.names["weight"]].to(torch.float32).contiguous()

    def vector(self, rt):
        return self.weight


register_part("scale", "channel_scale", ChannelScale)
register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "dyt", DynamicTanh)
