"""How a mixer, a feed-forward and their norms are arranged in a layer.

Pre-norm with two residual sums (src/model.rs:669-684):
    n = norm1(x); x += mixer(n); n = norm2(x); x += ffn(n)
The residual stream ``x`` is float32.  The last sum of a block is left pending
and folded into the next norm (of the next block, or the final one), which
reads and writes the stream once instead of twice.  The feed-forward (with its
norm) may be absent: x += mixer(norm1(x)) is then the whole layer.

"Sandwich": a norm before AND after each sublayer, and the feed-forward optional:
    x += post1(mixer(norm1(x)));  x += post2(ffn(norm2(x)))
A sublayer's output is handed on together with its post-norm (``PostNormDelta``), so the next norm
before a sublayer may form post-norm, residual sum and its own norm in one kernel.

"Parallel": ONE norm, whose output both sublayers read, and one residual sum; each sublayer's output
may be multiplied by a per-channel factor first, and the feed-forward is optional:
    n = norm1(x);  x += scale1 * mixer(n) + scale2 * ffn(n)
The two outputs are handed on unscaled and unsummed (``ScaledPairDelta``): the next norm forms the
scaling, the sums and itself in one kernel.  With ``norm2`` the feed-forward reads a norm of its own of
the SAME x: x += mixer(norm1(x)) + ffn(norm2(x)).  With ``pre1`` / ``pre2`` (parts of category
"inconv") what a sublayer reads, h, is first replaced by h + conv(h), a causal convolution over time
on each channel; the last taps - 1 inputs of every sequence are state of the block, which the cache
keeps per scheduled run of the layer (``state_request``, handed to ``forward`` as ``block_state``).
"""
from __future__ import annotations

import os

from ..config.spec import LayerSpec
import torch

from .base import PostNormDelta, ScaledPairDelta, delta_for, make_part


class PreNormBlock:
    category, kind = "block", "prenorm"

    def __init__(self, layer: LayerSpec):
        self.layer = layer
        if (layer.ffn is None) != (layer.norm2 is None):
            raise ValueError("a pre-norm block has a feed-forward with its norm, or neither")
        self.norm1 = make_part("norm", layer.norm1)
        self.mixer = make_part("mixer", layer.mixer)
        self.norm2 = make_part("norm", layer.norm2) if layer.norm2 is not None else None
        self.ffn = make_part("ffn", layer.ffn) if layer.ffn is not None else None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def forward(self, rt, x, pending, batch, cache_view, state):
        """x: [T, hidden] float32 stream; pending: a delta not yet added (or None).
        Returns (x, pending)."""
        h = self.norm1.forward(rt, x, delta=delta_for(self.norm1, pending, rt),
                               want32=getattr(self.mixer, "wants32", False))
        delta = self.mixer.forward(rt, h, batch, cache_view, state)
        if self.ffn is None:          # a layer without a feed-forward: its mixer's output is what is pending
            return x, delta
        # a feed-forward may offer to run the norm before it itself (fused with its first
        # kernels); it returns None where it cannot, and nothing has happened then
        prenorm = getattr(self.ffn, "forward_prenorm", None)
        if prenorm is not None:
            out = prenorm(rt, x, delta, self.norm2, batch)
            if out is not None:
                return x, out
        h = self.norm2.forward(rt, x, delta=delta, want32=getattr(self.ffn, "wants32", False))
        # (its delta may come back uncombined, for the next norm to finish: base.LazyDelta)
        return x, getattr(self.ffn, "forward_lazy", self.ffn.forward)(rt, h, batch)


class SandwichBlock:
    category, kind = "block", "sandwich"

    def __init__(self, layer: LayerSpec):
        if layer.post1 is None or (layer.ffn is None) != (layer.norm2 is None) or (layer.ffn is None) != (layer.post2 is None):
            raise ValueError("a sandwich block has a norm after its mixer, and a feed-forward with both its norms or none")
        self.layer = layer
        self.norm1 = make_part("norm", layer.norm1)
        self.mixer = make_part("mixer", layer.mixer)
        self.post1 = make_part("norm", layer.post1)
        self.ffn = self.norm2 = self.post2 = None
        if layer.ffn is not None:
            self.norm2 = make_part("norm", layer.norm2)
            self.ffn = make_part("ffn", layer.ffn)
            self.post2 = make_part("norm", layer.post2)

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.post1, self.norm2, self.ffn, self.post2) if p is not None]

    def forward(self, rt, x, pending, batch, cache_view, state):
        h = self.norm1.forward(rt, x, delta=delta_for(self.norm1, pending, rt),
                               want32=getattr(self.mixer, "wants32", False))
        pending = PostNormDelta(self.mixer.forward(rt, h, batch, cache_view, state), self.post1)
        if self.ffn is None:
            return x, pending
        h = self.norm2.forward(rt, x, delta=delta_for(self.norm2, pending, rt),
                               want32=getattr(self.ffn, "wants32", False))
        return x, PostNormDelta(self.ffn.forward(rt, h, batch), self.post2)


class ParallelBlock:
    category, kind = "block", "parallel"

    def __init__(self, layer: LayerSpec):
        if layer.post1 is not None or layer.post2 is not None:
            raise ValueError("a parallel block has its norms before the sublayers")
        if layer.ffn is None and (layer.scale2 is not None or layer.norm2 is not None or layer.pre2 is not None):
            raise ValueError("a parallel block without a feed-forward has no factor, norm or convolution for it")
        self.layer = layer
        self.norm1 = make_part("norm", layer.norm1)
        self.mixer = make_part("mixer", layer.mixer)
        self.ffn = make_part("ffn", layer.ffn) if layer.ffn is not None else None
        self.norm2 = make_part("norm", layer.norm2) if layer.norm2 is not None else None
        self.scale1 = make_part("scale", layer.scale1) if layer.scale1 is not None else None
        self.scale2 = make_part("scale", layer.scale2) if layer.scale2 is not None else None
        self.pre1 = make_part("inconv", layer.pre1) if layer.pre1 is not None else None
        self.pre2 = make_part("inconv", layer.pre2) if layer.pre2 is not None else None
        self._ones = None
        # MOE_B200_FFN_BESIDE=0: a block with two norms runs its feed-forward after its mixer, not beside it
        self._beside = os.environ.get("MOE_B200_FFN_BESIDE", "1") != "0"

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn, self.scale1, self.scale2, self.pre1, self.pre2)
                if p is not None]

    def state_request(self):
        """What the input convolutions keep per sequence: [pre1's rows | pre2's rows], 32-bit."""
        from ..cache.kv import StateRequest

        n = sum(p.state_floats() for p in (self.pre1, self.pre2) if p is not None)
        return StateRequest((n,), torch.float32) if n else None

    def _factor(self, rt, scale, like):
        if scale is not None:
            return scale.vector(rt)
        if self._ones is None:
            self._ones = torch.ones(like.shape[1], dtype=torch.float32, device=like.device)
        return self._ones

    def forward(self, rt, x, pending, batch, cache_view, state, block_state=None):
        from .conv import run_input_convs

        mix32 = getattr(self.mixer, "wants32", False)
        ffn32 = getattr(self.ffn, "wants32", False)
        convs = self.pre1 is not None or self.pre2 is not None
        both = None
        if convs and self.norm2 is not None and self.pre1 is not None and self.pre2 is not None:
            # two norms of the same x whose outputs only the convolutions read: one kernel, one statistic
            pair = getattr(self.norm1, "forward_pair", None)
            both = pair(rt, x, delta_for(self.norm1, pending, rt), self.norm2) if pair is not None else None
        if both is not None:
            h, h2 = both
        else:
            h = self.norm1.forward(rt, x, delta=delta_for(self.norm1, pending, rt),
                                   want32=mix32 or (ffn32 and self.norm2 is None) or convs)
            # (norm1 has written the sum back: a second norm reads the same x, with nothing pending)
            h2 = self.norm2.forward(rt, x, want32=ffn32 or convs) if self.norm2 is not None else h
        if convs:
            if self.norm2 is None and self.ffn is not None and (self.pre1 is None) != (self.pre2 is None):
                raise ValueError("a parallel block with one norm convolves both sublayers' input or neither")
            h, h2 = run_input_convs(rt, [(self.pre1, h, mix32), (self.pre2, h2, ffn32) if self.ffn is not None else None],
                                    batch, block_state)
        if self.ffn is not None and self.norm2 is not None and self._beside and x.is_cuda:
            # the two sublayers share nothing but the stream they read: the feed-forward runs on a second
            # stream beside the mixer (inside a captured step: a fork and a join)
            main = torch.cuda.current_stream()
            side = rt.side_stream(2)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                b = self.ffn.forward(rt, h2, batch)
            a = self.mixer.forward(rt, h, batch, cache_view, state)
            main.wait_stream(side)
            b.record_stream(main)
            return x, ScaledPairDelta(a, self._factor(rt, self.scale1, a), b, self._factor(rt, self.scale2, a))
        a = self.mixer.forward(rt, h, batch, cache_view, state)
        if self.ffn is None:
            return x, ScaledPairDelta(a, self._factor(rt, self.scale1, a))
        # (a feed-forward may hand its output on uncombined, for the next norm to finish: base.LazyDelta)
        b = getattr(self.ffn, "forward_lazy", self.ffn.forward)(rt, h2, batch)
        return x, ScaledPairDelta(a, self._factor(rt, self.scale1, a), b, self._factor(rt, self.scale2, a))


_BLOCKS = {"prenorm": PreNormBlock, "sandwich": SandwichBlock, "parallel": ParallelBlock}


def register_block(kind: str, cls) -> None:
    _BLOCKS[kind] = cls


def make_block(layer: LayerSpec):
    if layer.block not in _BLOCKS:
        raise KeyError(f"no block arrangement '{layer.block}'; registered: {', '.join(sorted(_BLOCKS))}")
    return _BLOCKS[layer.block](layer)
