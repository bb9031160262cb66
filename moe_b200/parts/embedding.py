"""Token embedding and the output projection.

x_i = embed[token_i] (src/model.rs:662-665; an id outside the vocabulary is an
error here, the reference wraps it).  logits = W_lm norm(x) on the requested
rows only; W_lm is the embedding when the model ties them (src/model.rs:350).
"""
from __future__ import annotations

import torch

from ..ops import core
from ..ops.linear import linear
from .base import Part, TensorSpec, register_part


class TokenEmbedding(Part):
    category, kind = "embedding", "token_embedding"
    graph_safe = True
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.hidden = int(self.params["hidden_size"])
        self.scale = float(self.params.get("scale", 1.0))   # x = embed[token] * scale

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.vocab, self.hidden))}

    def describe(self):
        return "token embedding" + (f" x {self.scale:g}" if self.scale != 1.0 else "")

    def step_elements(self, num_tokens):
        return float(num_tokens * self.hidden)            # one row a token

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.names["weight"]].contiguous()

    def forward(self, rt, token_ids, num_tokens, batch=None):
        """With a batch that carries ``last_token`` (the per-slot table of the tokens sampled last),
        a token id of -1 is read from there."""
        x = rt.empty((num_tokens, self.hidden), torch.float32)
        last = getattr(batch, "last_token", None)
        if last is not None:
            core.embed(self.weight, token_ids, x, rt.status, last, batch.seq_of_token, batch.slots, scale=self.scale)
        else:
            core.embed(self.weight, token_ids, x, rt.status, scale=self.scale)
        return x


class PairEmbedding(TokenEmbedding):
    """x = rmsnorm(embed[token] + pair[row]) * w: beside the token's own row, a row of a second table
    chosen by the token and the one before it, row = (previous * mul_prev + token * mul_cur) mod
    buckets; a sequence's first token takes row number ``buckets`` (the table's last).  The norm's
    statistics are 32-bit.  The token a sequence saw last is state of fixed size (``state_request``),
    handed to ``forward`` as ``state``."""

    kind = "pair_embedding"
    default_names = {"weight": "weight", "pair": "pair", "norm": "norm"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.buckets, self.mul_prev, self.mul_cur = int(p["buckets"]), int(p["mul_prev"]), int(p["mul_cur"])
        self.eps = float(p["eps"])
        if self.buckets < 1 or self.scale != 1.0:
            raise ValueError("pair_embedding: at least one bucket, and no scale")

    def tensors(self):
        n = self.names
        return {n["weight"]: TensorSpec((self.vocab, self.hidden)), n["pair"]: TensorSpec((self.buckets + 1, self.hidden)),
                n["norm"]: TensorSpec((self.hidden,), init="ones", vector=True)}

    def describe(self):
        return f"token embedding + a row by (previous, token) of {self.buckets} buckets, RMS-normed"

    def step_elements(self, num_tokens):
        return float(2 * num_tokens * self.hidden + self.hidden)

    def state_request(self):
        from ..cache.kv import StateRequest

        return StateRequest((1,), torch.int32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.pair = tensors[self.names["pair"]].to(self.weight.dtype).contiguous()
        self.norm_w = tensors[self.names["norm"]].to(torch.float32).contiguous()

    def forward(self, rt, token_ids, num_tokens, batch=None, state=None):
        x = rt.empty((num_tokens, self.hidden), torch.float32)
        core.embed_pair(self.weight, self.pair, self.norm_w, self.eps, batch, x, state, buckets=self.buckets,
                        mul_prev=self.mul_prev, mul_cur=self.mul_cur, status=rt.status)
        return x


class LMHead(Part):
    category, kind = "head", "lm_head"
    graph_safe = True
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.hidden = int(self.params["hidden_size"])
        self.tied = bool(self.params.get("tied", False))

    def tensors(self):
        return {} if self.tied else {self.names["weight"]: TensorSpec((self.vocab, self.hidden))}

    def describe(self):
        return "output projection" + (" (the embedding)" if self.tied else "")

    def step_elements(self, num_tokens):
        return float(self.vocab * self.hidden)            # the whole matrix, tied or not

    def bind(self, tensors, rt, embedding: TokenEmbedding = None):
        super().bind(tensors, rt)
        self.weight = embedding.weight if self.tied else tensors[self.names["weight"]].contiguous()

    def forward(self, rt, h):
        """h: Activations of the wanted rows -> logits [rows, vocab] float32."""
        return linear(rt, h.act, self.weight)


class ConcatLinearJoin(Part):
    """x <- W [x; x0]: the stream is joined with the embedding output x0 and projected back to the
    model's width (W: [hidden, 2 hidden], the stream's columns first).  A model that runs a stretch of
    its layers several times does this at the start of every pass.  The two halves share one buffer
    in the compute dtype, whose right half is filled once per step (``remember``); the left half
    takes the stream with whatever was still pending, in the kernel of the norm that would have
    added it."""

    category, kind = "join", "concat_linear"
    graph_safe = True
    lazy_kinds = ("post_dyt",)
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.hidden, 2 * self.hidden))}

    def describe(self):
        return "join with the embedding output, projected 2:1"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors[self.names["weight"]].contiguous()
        self._both = None

    def _halves(self, rt):
        return self.hidden, ("out16" if rt.is_bf16 else "out32")

    def remember(self, rt, x0):
        H, key = self._halves(rt)
        self._both = rt.empty((x0.shape[0], 2 * H))
        core.dyt(x0, None, write_back=False, status=rt.status, **{key: self._both[:, H:]})

    def forward(self, rt, x, pending):
        from .base import LazyDelta

        H, key = self._halves(rt)
        post = None
        if isinstance(pending, LazyDelta):
            if pending.kind == "post_dyt":
                post, pending = pending.norm.triple(), pending.tensor
            else:
                pending = pending.materialize(rt)
        core.dyt(x, None, delta=pending, post=post, write_back=False, status=rt.status, **{key: self._both[:, :H]})
        return linear(rt, self._both, self.weight)


class AddRowJoin(Part):
    """x <- x + w[row]: one row of a learned table [rows, hidden] is added to every token's stream (a
    model that runs a stretch of its layers several times adds row t at the start of pass t).  The
    sum is 32-bit and takes along whatever was still pending."""

    category, kind = "join", "add_row"
    graph_safe = True
    default_names = {"weight": "weight"}

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.params["hidden_size"])
        self.rows = int(self.params["rows"])
        self.row = int(self.params["row"])
        if not 0 <= self.row < self.rows:
            raise ValueError(f"add_row: row {self.row} of a table of {self.rows}")

    def tensors(self):
        return {self.names["weight"]: TensorSpec((self.rows, self.hidden), vector=True)}

    def describe(self):
        return f"adds row {self.row} of a table of {self.rows} vectors"

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.vector = tensors[self.names["weight"]][self.row].to(torch.float32).contiguous()

    def remember(self, rt, x0):
        pass

    def forward(self, rt, x, pending):
        from .base import LazyDelta

        if isinstance(pending, LazyDelta):
            pending = pending.materialize(rt)
        core.add_row(x, self.vector, delta=pending)
        return x


register_part("join", "concat_linear", ConcatLinearJoin)
register_part("join", "add_row", AddRowJoin)
register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "pair_embedding", PairEmbedding)
register_part("head", "lm_head", LMHead)
