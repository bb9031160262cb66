"""A short causal convolution over time on what a sublayer reads.

With h_t the sublayer's (normed) input at position t of a sequence and taps w [width, taps]:
    h_t  <-  h_t + sum_j w[:, j] * h_(t - taps + 1 + j)       (rows before the sequence's start are zero)
so the last column of w multiplies the token's own row.  What a sequence carries from step to step
is its last taps - 1 inputs, 32-bit, which the block that owns the part keeps in its state.  The
arithmetic is 32-bit in both dtypes; the bfloat16 path rounds the result that feeds a matrix product.
"""
from __future__ import annotations

import torch

from ..ops import core
from .base import Activations, Part, TensorSpec, register_part


class ResidualConv(Part):
    category, kind = "inconv", "residual_conv"
    graph_safe = True
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(self.params["size"])
        self.taps = int(self.params["taps"])
        if not 1 <= self.taps <= 16:
            raise ValueError(f"residual_conv: {self.taps} taps; the kernel takes 1 to 16")

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.size, self.taps))}

    def describe(self):
        return f"h + causal convolution of {self.taps} taps"

    def state_floats(self) -> int:
        return (self.taps - 1) * self.size

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        # [taps, width]: a tap's factors for all channels side by side
        self.weight_t = tensors[self.names["weight"]].to(torch.float32).t().contiguous()


def run_input_convs(rt, items, batch, state):
    """``items``: for each sublayer (conv part or None, its input Activations, whether the sublayer wants
    the 32-bit form), or None for a sublayer that is absent.  Returns the inputs with h + conv(h) in
    the place of h, both convolutions in one launch where their shapes agree, and moves the state on
    ([first conv's rows | second conv's rows] in a slot's row)."""
    jobs, outs, offset = [], [], 0
    for it in items:
        if it is None:
            outs.append(None)
            continue
        conv, h, want32 = it
        if conv is None:
            outs.append(h)
            continue
        T = h.f32.shape[0]
        o32 = rt.empty((T, conv.size), torch.float32) if (want32 or not rt.is_bf16) else None
        o16 = rt.empty((T, conv.size), torch.bfloat16) if rt.is_bf16 else None
        jobs.append((conv, dict(u=h.f32, w=conv.weight_t, bias=None, offset=offset, out32=o32, out16=o16)))
        offset += conv.state_floats()
        outs.append(Activations(act=o16 if rt.is_bf16 else o32, f32=o32))
    same = len(jobs) == 2 and jobs[0][0].taps == jobs[1][0].taps and jobs[0][0].size == jobs[1][0].size
    groups = [jobs] if same else [[j] for j in jobs]
    for grp in groups:
        conv = grp[0][0]
        core.seq_conv([j for _, j in grp], state, batch, taps=conv.taps, channels=conv.size, residual=True)
    if not batch.all_decode:       # (a step of one token a sequence moves the state on in the same launch)
        for conv, j in jobs:
            if conv.taps > 1:
                core.conv_state_update(j["u"], state, batch, taps=conv.taps, channels=conv.size, offset=j["offset"])
    return outs


register_part("inconv", "residual_conv", ResidualConv)
