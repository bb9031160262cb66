"""Python face of the kernel library ``core``: argument checks, then one C call.

Every function launches on the current CUDA stream and returns at once.  There
is no fallback: a tensor on the CPU, a dtype the kernels do not take or a
library that cannot be built raises.
"""
from __future__ import annotations

import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from . import build

DT_F32, DT_BF16 = 0, 1
# the gate's activation of a gated feed-forward (ACT_* in csrc/common.cuh)
GLU_ACTS = {"silu": 0, "gelu_tanh": 1, "clamped_sigmoid": 2}
# what an ungated product's output may pass in the tensor-core kernel's epilogue
PLAIN_ACTS = {"relu2": 3}


class KernelError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = build.load("core")
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        sig = {
            "moe_embed": [P, I, P, P, I, I, I, P, P, P, P, F, P],
            "moe_dyt": [P, P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P],
            "moe_heads_prepare": [P, I, P, P, P, P, F, P, I, F, I, I, I, I, I, I, P, P, P, LL, LL, I, P, P, P, P, P, I, I, I, I, P, P],
            "moe_gate_pack": [P, P, I, I, I, I, I, P, I, P],
            "moe_latent_prepare": [P, I, P, P, P, F, I, I, I, I, I, P, P, I, P, P, P, P, P, I, I, I, I, P, I, P],
            "moe_heads_transpose": [P, I, LL, LL, I, I, I, I, P, I, P],
            "moe_diff_combine": [P, P, I, I, I, I, I, F, F, F, P, I, P],
            "moe_add_row": [P, P, P, LL, I, P],
            "moe_rmsnorm": [P, P, P, P, P, P, I, I, I, F, I, P, P],
            "moe_rmsnorm_combine": [P, P, P, P, I, P, P, P, P, P, P, I, I, I, F, I, P, P],
            "moe_add_inplace": [P, P, LL, P],
            "moe_gemm_generic": [P, I, I, P, I, P, I, LL, P, I, I, P, P, I, I, I, I, P, P],
            "moe_rope_split": [P, P, P, I, I, I, I, I, P, P, P, I, P, P, P, P, P, P, I, I, I, I, P, P],
            "moe_kv_commit": [P, P, P, P, I, P, P, P, P, P, I, I, I, I, I, I, I, P, P],
            "moe_attention_generic": [P, P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, F, I, P, P],
            "moe_router": [P, P, P, I, P, I, I, I, I, I, F, P, P, P, P, P, LL, P, I, I, P],
            "moe_router_logits": [P, P, P, I, I, I, I, P, P, LL, P],
            "moe_router_topk": [P, P, I, I, I, I, I, F, P, P, P, P, I, I, P],
            "moe_split3": [P, P, LL, I, P],
            "moe_route_dispatch": [P, P, I, I, I, I, I, F, P, P, P, P, P, P, P, P, I, P, P, I, I, P],
            "moe_rope_commit": [P, P, P, I, I, I, I, I, P, P, P, I, P, P, P, I, I, I, I, P, P],
            "moe_attention_decode": [P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, I, P, I, F, I, P, P],
            "moe_attention_tiled": [P, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, I, F, I, P, P],
            "moe_conv_heads_prepare": [P, I, P, I, P, LL, P, P, P, P, F, I, P, I, I, I, I, I, I, I, P, P, P, LL, LL, I, P, P,
                                       P, P, I, I, I, I, P, P],
            "moe_conv_state_update": [P, I, P, LL, I, I, P, P, I, P],
            "moe_wkv_shift_mix": [P, P, I, P, LL, P, P, P, P, I, I, P, I, P, P, P, P, I, I, P, P],
            "moe_wkv_decay": [P, P, P, I, I, I, P, P],
            "moe_wkv_scan": [P, P, P, P, LL, P, P, LL, P, P, I, I, I, P, I, I, P, P, P],
            "moe_wkv_finish": [P, P, LL, P, F, P, I, I, I, P, I, P],
            "moe_rmsnorm_scaled": [P, P, P, P, P, P, P, P, P, I, I, I, F, I, P, P, P, P, I, P, P, P, P],
            "moe_attention_decode_fused": [P, P, I, P, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, P, I, I, P, P],
            "moe_norm_route": [P, P, P, F, I, I, P, P, P, P, I, I, I, I, F, P, P, P, P, P, P, P, P, P, P, I, I, P],
            "moe_align": [P, I, I, I, P, P, P, P, P],
            "moe_swiglu": [P, P, I, LL, I, I, F, P],
            "moe_combine": [P, P, P, I, P, P, P, I, I, P],
            "moe_sample": [P, I, I, P, P, P, I, F, I, F, F, P, P, P, LL, I, P],
            "moe_logprobs": [P, I, I, P, I, P, P, P, P],
            "moe_seed_rng": [P, P, P, I, P],
            "moe_table_update": [P, I, P, I, P],
            "moe_whole_prepare": [P, I, P, P, P, P, F, P, I, P, I, I, I, I, I, I, P, P, P, LL, LL, I, P, P, P, P, P, I, I, I, I,
                                  P, P],
            "moe_unrotate_pack": [P, P, P, I, I, I, I, P, I, P],
            "moe_seq_conv": [I, P, LL, P, P, P, P, P, P, LL, P, P, P, P, P, I, I, LL, P, P, P, P, I, I, I, I, P],
            "moe_embed_pair": [P, P, I, P, F, P, P, I, I, I, I, I, I, P, P, P, P, P, P, P, P],
            "moe_pair_norm_mean": [P, P, P, P, F, I, I, P, P],
            "moe_relu2": [P, P, I, LL, P],
            "moe_table_route": [P, I, P, P, P, P, I, I, I, I, P, P, P, P],
            "moe_ssd_scan": [P, LL, P, LL, P, P, P, P, LL, P, P, I, I, I, I, I, P, I, I, P, P, P],
            "moe_ssd_finish": [P, P, LL, P, F, P, I, I, I, P, I, P],
        }
        for name, argtypes in sig.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = c_int
        L.moe_router_scratch_floats.argtypes = [I, I, I, I]
        L.moe_router_scratch_floats.restype = LL
        L.moe_set_pdl.argtypes = [c_int]
        L.moe_set_pdl.restype = None
        if os.environ.get("MOE_B200_PDL", "1") == "0":      # programmatic dependent launch off
            L.moe_set_pdl(0)
        L.moe_set_norm_route_cluster.argtypes = [c_int]
        L.moe_set_norm_route_cluster.restype = None
        L.moe_set_decode_grouped.argtypes = [c_int]
        L.moe_set_decode_grouped.restype = None
        if os.environ.get("MOE_B200_NORM_ROUTE_CLUSTER", "1") == "0":   # ticket form also for few tokens
            L.moe_set_norm_route_cluster(0)
        _lib = L
    return _lib


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current stream's handle.  (``torch.cuda.current_stream()`` builds a Python object on
    every call, which with hundreds of launches a step is milliseconds of host time.)"""
    if _raw_stream is not None and _raw_device is not None:
        return _raw_stream(_raw_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, not {t.dtype}")


def _p(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _chk(t: torch.Tensor, name: str, dtype=None, dims: Optional[int] = None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got {tuple(t.shape)}")
    return t


launches = 0   # kernels launched through this module since import (benchmarks read the difference)


def _ok(code: int, what: str):
    global launches
    launches += 1
    if code != 0:
        try:
            msg = torch.cuda.cudart().cudaGetErrorString(code)
        except Exception:
            msg = "?"
        raise KernelError(f"{what}: CUDA error {code} ({msg})")


# --------------------------------------------------------------------------- status word
STATUS_BITS = {
    1: "a token id lies outside the vocabulary",
    2: "a page table entry lies outside the page pool",
    4: "routing produced an expert id outside the expert range",
    8: "a bounded wait inside a kernel ran out",
    16: "a gather index lies outside its tensor",
}


# Where a bounded wait ran out (status[1]; the first one of a step): kernel and role, barrier.
WAIT_SITES = {
    0x10: "tensor-core product, one CTA a tile", 0x20: "tensor-core product, persistent",
    0x30: "tensor-core product, pairs of CTAs", 0x40: "tensor-core prompt attention",
}
WAIT_ROLES = {
    0x1: "producer: a free stage", 0x2: "producer: its own copies in flight", 0x3: "MMA issuer: a free accumulator",
    0x4: "MMA issuer: a loaded stage", 0x5: "epilogue: a finished accumulator",
}
WAIT_ROLES_ATTENTION = {
    0x1: "producer: a free key stage", 0x2: "producer: a free value stage", 0x3: "producer: its own copies in flight",
    0x4: "MMA issuer: the queries", 0x5: "MMA issuer: a key tile",
    0x7: "MMA issuer: a value tile", 0x8: "MMA issuer: P", 0x9: "softmax: the scores", 0xa: "softmax: its partner's maximum",
    0xb: "softmax: the last P V product", 0xc: "softmax: its partner's sum", 0xd: "softmax: the final P V product",
}


def wait_site(code: int) -> str:
    kernel, role = code & 0xf0, code & 0xf
    roles = WAIT_ROLES_ATTENTION if kernel == 0x40 else WAIT_ROLES
    return f"{WAIT_SITES.get(kernel, 'kernel ?')}, {roles.get(role, 'wait ?')} (site 0x{code:02x})"


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor):
    """Read the status word (synchronises) and raise if a kernel flagged a fault."""
    v, site = (int(x) for x in status[:2].tolist())
    if v:
        status.zero_()
        msg = "; ".join(m for b, m in STATUS_BITS.items() if v & b) or f"status {v}"
        if v & 8 and site:
            msg += f" [{wait_site(site)}]"
        raise KernelError(msg)


# --------------------------------------------------------------------------- kernels
def embed(table, token_ids, out, status, last_token=None, seq_of_token=None, slots=None, scale=1.0):
    """out[t] = table[token_ids[t]] * scale; with ``last_token`` (a per-slot table the sampler fills) a
    token id of -1 stands for the token sampled last for the row's sequence."""
    _chk(table, "table", dims=2), _chk(token_ids, "token_ids", torch.int32, 1), _chk(out, "out", torch.float32, 2)
    T, H = out.shape
    if token_ids.numel() < T or table.shape[1] != H:
        raise KernelError("embed: shape mismatch")
    if last_token is not None:
        _chk(last_token, "last_token", torch.int32, 1), _chk(seq_of_token, "seq_of_token", torch.int32, 1)
        _chk(slots, "slots", torch.int32, 1)
    _ok(lib().moe_embed(_p(table), _dt(table), _p(token_ids), _p(out), T, H, table.shape[0], _p(status),
                        _p(last_token), _p(seq_of_token), _p(slots), float(scale), _stream()), "embed")


def rmsnorm(x, weight, eps, *, delta=None, rows=None, out32=None, out16=None, write_back=True, status=None):
    """y = rmsnorm(x[r] (+ delta[r])) for r in rows (or every row).

    With ``delta`` and ``write_back`` the sum is stored back into ``x`` (the
    32-bit residual stream).  ``out32`` / ``out16`` receive y in float32 /
    bfloat16; either may be None."""
    _chk(x, "x", torch.float32, 2), _chk(weight, "weight", torch.float32, 1)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if weight.numel() != H:
        raise KernelError("rmsnorm: weight size")
    if delta is not None:
        _chk(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError("rmsnorm: delta shape")
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
    for o, dt in ((out32, torch.float32), (out16, torch.bfloat16)):
        if o is not None:
            _chk(o, "out", dt, 2)
            if o.shape[0] < n_out or o.shape[1] != H:
                raise KernelError("rmsnorm: output shape")
    _ok(lib().moe_rmsnorm(_p(x), _p(delta), _p(weight), _p(rows), _p(out32), _p(out16), n_out, S, H, float(eps),
                          1 if (write_back and rows is None) else 0, _p(status), _stream()), "rmsnorm")


def rmsnorm_combine(x, cd, weight, eps, *, rows=None, out32=None, out16=None, write_back=True, status=None) -> bool:
    """``rmsnorm`` whose delta is still the uncombined output of routed experts (``cd``: y,
    pos_of_pair, topk_w, top_k, shared, shared_gate): combined inside the norm's kernel.  False,
    with nothing launched, if the rows are not whole 16-byte units."""
    _chk(x, "x", torch.float32, 2), _chk(weight, "weight", torch.float32, 1), _chk(cd.y, "y", torch.float32, 2)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if weight.numel() != H or cd.y.shape[1] != H or cd.pos_of_pair.numel() < S * cd.top_k:
        raise KernelError("rmsnorm_combine: shapes")
    code = lib().moe_rmsnorm_combine(_p(x), _p(cd.y), _p(cd.pos_of_pair), _p(cd.topk_w), cd.top_k, _p(cd.shared),
                                     _p(cd.shared_gate), _p(weight), _p(rows), _p(out32), _p(out16), n_out, S, H,
                                     float(eps), 1 if (write_back and rows is None) else 0, _p(status), _stream())
    if code == -1:
        return False
    _ok(code, "rmsnorm_combine")
    return True


def dyt(x, pre=None, *, delta=None, post=None, rows=None, out32=None, out16=None, write_back=True, status=None):
    """Dynamic Tanh with the pending residual sum in front of it:
        x += tanh(pa * delta) * pw + pb   (``post`` = (pa, pw, pb); without it x += delta; stored
                                           back into ``x`` with ``write_back`` unless ``rows`` selects)
        out = tanh(a * x) * w + b         (``pre`` = (a, w, b); None: out = x)
    alpha is a 0-dim float32 tensor on the device.  ``out32`` / ``out16`` may be column slices of wider
    buffers (unit stride along the row)."""
    _chk(x, "x", torch.float32, 2)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if delta is not None:
        _chk(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError("dyt: delta shape")
    elif post is not None:
        raise KernelError("dyt: a norm after the sublayer needs that sublayer's output")
    for nm in (pre, post):
        if nm is not None:
            a, w, b = nm
            if a.dtype != torch.float32 or a.numel() != 1 or not a.is_cuda:
                raise KernelError("dyt: alpha must be one float32 on the device")
            _chk(w, "weight", torch.float32, 1), _chk(b, "shift", torch.float32, 1)
            if w.numel() != H or b.numel() != H:
                raise KernelError("dyt: weight size")
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
    ld = None
    for o, dt in ((out32, torch.float32), (out16, torch.bfloat16)):
        if o is not None:
            if not o.is_cuda or o.dtype != dt or o.dim() != 2 or o.stride(1) != 1 or o.shape[0] < n_out or o.shape[1] != H:
                raise KernelError("dyt: output shape, dtype or layout")
            if ld is not None and ld != o.stride(0):
                raise KernelError("dyt: the two outputs must have the same row pitch")
            ld = o.stride(0)
    if ld is None:
        ld = H
    pa, pw, pb = post if post is not None else (None, None, None)
    a, w, b = pre if pre is not None else (None, None, None)
    _ok(lib().moe_dyt(_p(x), _p(delta), _p(pa), _p(pw), _p(pb), _p(a), _p(w), _p(b), _p(rows), _p(out32), _p(out16),
                      ld, n_out, S, H, 1 if (write_back and rows is None) else 0, _p(status), _stream()), "dyt")


def heads_prepare(proj, pos, seq_of_token, *, nh, nkv, d, dv, width, q, k, v, q_norm=None, k_norm=None, eps=0.0,
                  freq=None, rot=0, mscale=1.0, commit=None, status=None):
    """From a step's 32-bit projection rows [q heads | k heads | v heads | ...]: per-head RMS norm of
    queries and keys (``q_norm`` / ``k_norm`` weights of size d, or None), rotation of the first ``rot``
    dimensions with ``freq`` and cos/sin scaled by ``mscale``, split into q [T, nh, width] and k, v
    [T, nkv, width], zero-filled beyond d (dv); the three may be views into one buffer [T, nh + 2 nkv,
    width] (a token pitch of their own).  ``commit=(view, batch)`` also appends keys and values to that
    cache layer."""
    _chk(proj, "proj", torch.float32, 2), _chk(pos, "pos", torch.int32, 1)
    T = proj.shape[0]
    for t, n in ((q, nh), (k, nkv), (v, nkv)):
        if (not t.is_cuda or t.dtype != q.dtype or tuple(t.shape) != (T, n, width) or t.stride(2) != 1
                or t.stride(1) != width or t.stride(0) < n * width):
            raise KernelError("heads_prepare: q, k, v must be [T, heads, width] with dense heads, of one dtype")
    if k.stride(0) != v.stride(0):
        raise KernelError("heads_prepare: keys and values must have the same token pitch")
    if proj.shape[1] < (nh + nkv) * d + nkv * dv:
        raise KernelError("heads_prepare: projection width")
    for wn in (q_norm, k_norm):
        if wn is not None:
            _chk(wn, "head norm weight", torch.float32, 1)
            if wn.numel() != d:
                raise KernelError("heads_prepare: head norm weight size")
    if rot:
        _chk(freq, "freq", torch.float32, 1)
        if freq.numel() < rot // 2:
            raise KernelError("heads_prepare: frequency table too short")
    kc = vc = se = sl = tb = None
    ts = ring = ps = npg = 0
    if commit is not None:
        view, batch = commit
        g = view.group
        if k.dtype != g.dtype or g.num_kv_heads != nkv or g.head_dim != width:
            raise KernelError("heads_prepare: the cache layer differs from the keys in dtype or shape")
        kc, vc, se, sl, tb = view.k, view.v, batch.seq_end, batch.slots, g.table
        ts, ring, ps, npg = g.table.stride(0), g.ring, g.page_size, g.num_pages
    _ok(lib().moe_heads_prepare(_p(proj), proj.stride(0), _p(pos), _p(seq_of_token), _p(q_norm), _p(k_norm), float(eps),
                                _p(freq) if rot else None, int(rot), float(mscale), T, nh, nkv, d, dv, width, _p(q),
                                _p(k), _p(v), q.stride(0), k.stride(0), _dt(q), _p(kc), _p(vc), _p(se), _p(sl), _p(tb), ts, ring, ps, npg,
                                _p(status), _stream()), "heads_prepare")


def gate_pack(ctx, out, *, nh, dv, width, gate=None):
    """out[t, h * dv + j] = ctx[t, h, j] * sigmoid(gate[t, h * dv + j]); ``gate``: a column slice
    [T, nh * dv] of a float32 projection (unit stride along the row), or None for the packing alone."""
    _chk(ctx, "ctx"), _chk(out, "out", dims=2)
    T = out.shape[0]
    if ctx.numel() < T * nh * width or out.shape[1] != nh * dv or out.dtype != ctx.dtype:
        raise KernelError("gate_pack: shapes or dtypes")
    ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != (T, nh * dv):
            raise KernelError("gate_pack: gate shape, dtype or layout")
        ld = gate.stride(0)
    _ok(lib().moe_gate_pack(_p(ctx), _p(gate), ld, T, nh, dv, width, _p(out), _dt(out), _stream()), "gate_pack")


def latent_prepare(proj, batch, *, nh, d, r, width, weight, eps, q_t, k_new, commit=None, status=None,
                   token_major=False):
    """From a step's 32-bit projection rows [q heads (nh x d) | latent (r)]: the latent divided by its
    root mean square, times ``weight``, into ``k_new`` [T, width] (zero-filled beyond r) and, with
    ``commit`` (a cache view), appended to that cache layer; the queries head by head into ``q_t``
    [nh, T, d], or with ``token_major`` token by token into ``q_t`` [T, nh, width] (zero-filled
    beyond d)."""
    _chk(proj, "proj", torch.float32, 2), _chk(weight, "latent norm weight", torch.float32, 1)
    T = proj.shape[0]
    _chk(q_t, "q_t"), _chk(k_new, "k_new")
    if (proj.shape[1] < nh * d + r or weight.numel() != r or q_t.numel() != nh * T * (width if token_major else d)
            or k_new.numel() != T * width or q_t.dtype != k_new.dtype or width < r or (token_major and width < d)):
        raise KernelError("latent_prepare: shapes or dtypes")
    kc = vc = se = sl = tb = None
    ts = ring = ps = npg = 0
    if commit is not None:
        g = commit.group
        if k_new.dtype != g.dtype or g.num_kv_heads != 1 or g.head_dim != width:
            raise KernelError("latent_prepare: the cache layer differs from the latent in dtype or shape")
        kc, vc, se, sl, tb = commit.k, commit.v, batch.seq_end, batch.slots, g.table
        ts, ring, ps, npg = g.table.stride(0), g.ring, g.page_size, g.num_pages
    _ok(lib().moe_latent_prepare(_p(proj), proj.stride(0), _p(batch.pos), _p(batch.seq_of_token), _p(weight), float(eps),
                                 T, nh, d, r, width, _p(q_t), _p(k_new), _dt(k_new), _p(kc), _p(vc), _p(se), _p(sl),
                                 _p(tb), ts, ring, ps, npg, _p(status), 1 if token_major else 0, _stream()),
        "latent_prepare")


def heads_transpose(src, dst, *, n):
    """dst[b, a, :n] = src[a, b, :n], zero beyond n; src: [A, B, >= n] with unit stride along the last
    axis (any pitch of the other two), dst: dense [B, A, wd >= n]; float32 or bfloat16 on either side."""
    if (src.dim() != 3 or dst.dim() != 3 or not dst.is_contiguous() or src.stride(2) != 1 or src.shape[2] < n
            or dst.shape[2] < n or (dst.shape[0], dst.shape[1]) != (src.shape[1], src.shape[0])):
        raise KernelError("heads_transpose: shapes")
    A, B = src.shape[0], src.shape[1]
    _ok(lib().moe_heads_transpose(_p(src), _dt(src), src.stride(0), src.stride(1), A, B, int(n), dst.shape[2], _p(dst),
                                  _dt(dst), _stream()), "heads_transpose")


def diff_combine(ctx, out, *, nh, dv, width, lam, eps, mult, gate=None):
    """Joins the two maps of differential attention: with a1 = ctx[t, h, :dv] and a2 = ctx[t, nh + h, :dv]
    (ctx: [T, 2 nh, width]), o = a1 - lam a2, o / sqrt(mean(o^2) + eps) * mult * sigmoid(gate[t, h]) into
    out[t, h * dv : (h + 1) * dv]; ``gate``: a float32 column slice [T, nh] of a projection, or None."""
    _chk(ctx, "ctx"), _chk(out, "out", dims=2)
    T = out.shape[0]
    if ctx.numel() < T * 2 * nh * width or out.shape[1] != nh * dv or out.dtype != ctx.dtype or width < dv:
        raise KernelError("diff_combine: shapes or dtypes")
    ld = 0
    if gate is not None:
        if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (T, nh):
            raise KernelError("diff_combine: gate shape, dtype or layout")
        ld = gate.stride(0)
    _ok(lib().moe_diff_combine(_p(ctx), _p(gate), ld, T, nh, dv, width, float(lam), float(eps), float(mult), _p(out),
                               _dt(out), _stream()), "diff_combine")


def add_row(x, row, delta=None):
    """x[t, :] += delta[t, :] + row[:] in 32-bit (``delta`` may be None)."""
    _chk(x, "x", torch.float32, 2), _chk(row, "row", torch.float32, 1)
    if row.numel() != x.shape[1]:
        raise KernelError("add_row: the row's width")
    if delta is not None:
        _chk(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError("add_row: the delta's shape")
    _ok(lib().moe_add_row(_p(x), _p(delta), _p(row), x.shape[0], x.shape[1], _stream()), "add_row")


def conv_heads_prepare(proj, batch, *, nh, nkv, d, dv, width, q, k, v, taps_w=None, state=None, eps=0.0,
                       unit_norm=False, freq=None, rot=0, commit=None, status=None):
    """From a step's 32-bit projection rows [q heads | k heads | v heads]: a causal convolution over
    time on every channel (``taps_w`` float32 [taps, channels]; earlier rows come from the step or,
    before it, from ``state`` [slots + 1, >= (taps - 1) * channels]; None: no convolution), the
    rotation of pairs (2i, 2i + 1) of the first ``rot`` dimensions of query and key heads, their
    division by the head's root mean square (``unit_norm``), and the split into q [T, nh, width] and
    k, v [T, nkv, width], zero-filled.  ``commit=view`` also appends keys and values to that cache
    layer.  The state is not changed: ``conv_state_update`` does that afterwards."""
    _chk(proj, "proj", torch.float32, 2)
    T = proj.shape[0]
    channels = (nh + nkv) * d + nkv * dv
    for t, n in ((q, nh), (k, nkv), (v, nkv)):
        if (not t.is_cuda or t.dtype != q.dtype or tuple(t.shape) != (T, n, width) or t.stride(2) != 1
                or t.stride(1) != width or t.stride(0) < n * width):
            raise KernelError("conv_heads_prepare: q, k, v must be [T, heads, width] with dense heads, of one dtype")
    if k.stride(0) != v.stride(0) or proj.shape[1] < channels:
        raise KernelError("conv_heads_prepare: token pitch of keys and values, or projection width")
    taps = 1
    if taps_w is not None:
        _chk(taps_w, "taps", torch.float32, 2)
        taps = taps_w.shape[0]
        if taps_w.shape[1] != channels:
            raise KernelError("conv_heads_prepare: a tap has one factor per channel")
        if taps > 1:
            _chk(state, "state", torch.float32, 2)
    if rot:
        _chk(freq, "freq", torch.float32, 1)
        if freq.numel() < rot // 2:
            raise KernelError("conv_heads_prepare: frequency table too short")
    kc = vc = se = tb = None
    ts = ring = ps = npg = 0
    if commit is not None:
        g = commit.group
        if k.dtype != g.dtype or g.num_kv_heads != nkv or g.head_dim != width:
            raise KernelError("conv_heads_prepare: the cache layer differs from the keys in dtype or shape")
        kc, vc, se, tb = commit.k, commit.v, batch.seq_end, g.table
        ts, ring, ps, npg = g.table.stride(0), g.ring, g.page_size, g.num_pages
    _ok(lib().moe_conv_heads_prepare(_p(proj), proj.stride(0), _p(taps_w), taps, _p(state),
                                     state.stride(0) if state is not None else 0, _p(batch.pos), _p(batch.seq_of_token),
                                     _p(batch.cu_seqlens), _p(batch.slots), float(eps), 1 if unit_norm else 0,
                                     _p(freq) if rot else None, int(rot), T, nh, nkv, d, dv, width, _p(q), _p(k), _p(v),
                                     q.stride(0), k.stride(0), _dt(q), _p(kc), _p(vc), _p(se), _p(tb), ts, ring, ps, npg,
                                     _p(status), _stream()), "conv_heads_prepare")


def conv_state_update(proj, state, batch, *, taps, channels, offset=0):
    """state[slot] <- the last ``taps - 1`` rows of ``proj`` that each sequence of the step holds by now.
    ``proj``: float32 [T, >= channels] (a column slice is fine); the rows live from float ``offset`` on
    in a slot's row of ``state``."""
    _chk(state, "state", torch.float32, 2)
    if (proj.dtype != torch.float32 or not proj.is_cuda or proj.dim() != 2 or proj.stride(1) != 1
            or proj.shape[1] < channels or offset + (taps - 1) * channels > state.shape[1]):
        raise KernelError("conv_state_update: the rows must be float32 [T, >= channels] and fit the state")
    _ok(lib().moe_conv_state_update(_p(proj), proj.stride(0), state.data_ptr() + 4 * int(offset), state.stride(0),
                                    int(taps), int(channels), _p(batch.cu_seqlens), _p(batch.slots), batch.num_seqs,
                                    _stream()), "conv_state_update")


WKV_FUSED_RANK = 32      # widest narrow projection of the decay that ``wkv_shift_mix`` forms itself


def wkv_shift_mix(h32, mu, state, batch, out, last32=None, decay=None):
    """out[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]; the row before a step's first is ``state[slot,
    :width]`` (zeros at position 0), which afterwards holds the sequence's last row of the step.
    ``last32`` (float32 [T, width]) receives the last blend instead of ``out``; or ``decay=(w1, w2t, w0,
    out)`` (w1 [rank <= 32, width], w2t [rank, inner], w0 [inner], out float32 [T, inner]) turns it into
    exp(-exp(w0 + w2t^T tanh(w1 x))) in the same launch."""
    _chk(h32, "h", torch.float32, 2), _chk(mu, "mu", torch.float32, 2)
    if not state.is_cuda or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1:
        raise KernelError("wkv_shift_mix: the state must be float32 rows (a column slice is fine)")
    T, W = h32.shape
    _chk(out, "out", dims=3)
    elsewhere = 1 if (last32 is not None or decay is not None) else 0
    if mu.shape[1] != W or out.shape[1:] != (T, W) or out.shape[0] < mu.shape[0] - elsewhere or state.shape[1] < W:
        raise KernelError("wkv_shift_mix: shapes")
    if last32 is not None:
        _chk(last32, "last32", torch.float32, 2)
        if tuple(last32.shape) != (T, W) or decay is not None:
            raise KernelError("wkv_shift_mix: shapes")
    w1 = w2t = w0 = dout = None
    rank = inner = 0
    if decay is not None:
        w1, w2t, w0, dout = decay
        for t in (w1, w2t, w0, dout):
            _chk(t, "decay", torch.float32)
        rank, inner = w1.shape[0], w2t.shape[1]
        if (rank > WKV_FUSED_RANK or w1.shape[1] != W or w2t.shape[0] != rank or w0.numel() != inner
                or tuple(dout.shape) != (T, inner)):
            raise KernelError("wkv_shift_mix: the decay's shapes")
    _ok(lib().moe_wkv_shift_mix(_p(h32), _p(mu), mu.shape[0], _p(state), state.stride(0), _p(batch.seq_of_token),
                                _p(batch.pos), _p(batch.cu_seqlens), _p(batch.slots), T, W, _p(out), _dt(out), _p(last32),
                                _p(w1), _p(w2t), _p(w0), rank, inner, _p(dout), _stream()),
        "wkv_shift_mix")


def wkv_decay(low, w2t, w0, out):
    """out[t, i] = exp(-exp(w0[i] + sum_q w2t[q, i] tanh(low[t, q]))): float32 throughout; ``w2t`` is the
    second projection transposed, [rank, inner]."""
    _chk(low, "low", torch.float32, 2), _chk(w2t, "w2t", torch.float32, 2), _chk(w0, "w0", torch.float32, 1)
    _chk(out, "out", torch.float32, 2)
    T, R = low.shape
    inner = w2t.shape[1]
    if w2t.shape[0] != R or w0.numel() != inner or tuple(out.shape) != (T, inner):
        raise KernelError("wkv_decay: shapes")
    _ok(lib().moe_wkv_decay(_p(low), _p(w2t), _p(w0), T, inner, R, _p(out), _stream()), "wkv_decay")


def wkv_scan(r, k, v, w, u, state, batch, out, *, heads, d, segments=None):
    """Per sequence and head, tokens in order: o_t = (S + diag(u) k_t v_t^T)^T r_t, then
    S <- diag(w_t) S + k_t v_t^T.  r, k, v, w: float32 [T, heads * d] of one row pitch
    (column slices of one buffer are fine); ``state``: float32 [slots + 1, >= heads * d * d], S of every
    slot; out: float32 [T, heads * d].  ``segments``: into how many pieces that run side by side every
    sequence's tokens are cut (None: ``scan_segments`` decides)."""
    T = out.shape[0]
    for t in (r, k, v, w):
        if (not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or tuple(t.shape) != (T, heads * d)
                or t.stride(1) != 1 or t.stride(0) != r.stride(0)):
            raise KernelError("wkv_scan: r, k, v and the decay must be float32 [T, heads * d] of one row pitch")
    _chk(u, "u", torch.float32), _chk(out, "out", torch.float32, 2)
    if u.numel() != heads * d or state.dtype != torch.float32 or state.stride(1) != 1:
        raise KernelError("wkv_scan: constants or state")
    segs = scan_segments(batch, heads * -(-d // 64), out.device) if segments is None else int(segments)
    seg_len, ends, decays = 0, None, None
    if segs > 1:
        longest = int(getattr(batch, "max_new", 0) or 0) or T
        seg_len = -(-(-(-longest // segs)) // 16) * 16
        ends = torch.empty((batch.num_seqs, segs, heads, d, d), dtype=torch.float32, device=out.device)
        decays = torch.empty((batch.num_seqs, segs, heads, d), dtype=torch.float32, device=out.device)
    _ok(lib().moe_wkv_scan(_p(r), _p(k), _p(v), _p(w), r.stride(0), _p(u), _p(state), state.stride(0),
                           _p(batch.cu_seqlens), _p(batch.slots), batch.num_seqs, heads, d, _p(out), segs, seg_len, _p(ends),
                           _p(decays), _stream()), "wkv_scan")


def wkv_finish(o, gate, norm_w, eps, batch, out, *, heads, d):
    """out = o / rms(o over each head) * norm_w * silu(gate), rounded to ``out``'s dtype."""
    _chk(o, "o", torch.float32, 2), _chk(norm_w, "norm weight", torch.float32, 1), _chk(out, "out", dims=2)
    T = o.shape[0]
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or tuple(gate.shape) != (T, heads * d) or out.shape != o.shape:
        raise KernelError("wkv_finish: shapes")
    _ok(lib().moe_wkv_finish(_p(o), _p(gate), gate.stride(0), _p(norm_w), float(eps), _p(batch.seq_of_token), T, heads, d,
                             _p(out), _dt(out), _stream()), "wkv_finish")


def rmsnorm_scaled(x, a, sa, b, sb, weight, eps, *, rows=None, out32=None, out16=None, write_back=True, status=None,
                   combine=None, second=None):
    """y = rmsnorm(x[r] + a[r] * sa + b[r] * sb) with per-channel scales sa, sb (``b``, ``sb`` may be
    None); with ``write_back`` (and no ``rows``) the sum is stored back into ``x``.  Instead of ``b``,
    ``combine`` may bring routed experts' outputs before their combine (y, pos_of_pair, topk_w, top_k,
    shared; no gate on the shared expert): b[t] = sum_j w[t, j] y[pos[t, j]] + shared[t] is formed here.
    ``second=(weight2, out32b)``: a second RMS norm of the same rows with another weight (the statistic is
    the same), into a float32 tensor of its own."""
    _chk(x, "x", torch.float32, 2), _chk(weight, "weight", torch.float32, 1)
    _chk(a, "a", torch.float32, 2), _chk(sa, "sa", torch.float32, 1)
    S, H = x.shape
    n_out = S if rows is None else rows.numel()
    if a.shape != x.shape or sa.numel() != H or weight.numel() != H:
        raise KernelError("rmsnorm_scaled: shapes")
    if b is not None:
        _chk(b, "b", torch.float32, 2), _chk(sb, "sb", torch.float32, 1)
        if b.shape != x.shape or sb.numel() != H:
            raise KernelError("rmsnorm_scaled: shapes")
    if rows is not None:
        _chk(rows, "rows", torch.int32, 1)
    for o, dt in ((out32, torch.float32), (out16, torch.bfloat16)):
        if o is not None:
            _chk(o, "out", dt, 2)
            if o.shape[0] < n_out or o.shape[1] != H:
                raise KernelError("rmsnorm_scaled: output shape")
    cy = cpos = cw = cshared = None
    top_k = 0
    if combine is not None:
        cy, cpos, cw, top_k, cshared = combine
        _chk(cy, "y", torch.float32, 2), _chk(cpos, "pos_of_pair", torch.int32), _chk(cw, "topk_w", torch.float32)
        _chk(sb, "sb", torch.float32, 1)
        if b is not None or cy.shape[1] != H or cpos.numel() < S * top_k or cw.numel() < S * top_k or sb.numel() != H:
            raise KernelError("rmsnorm_scaled: the experts' outputs")
        if cshared is not None:
            _chk(cshared, "shared", torch.float32, 2)
            if cshared.shape != x.shape:
                raise KernelError("rmsnorm_scaled: the shared expert's output")
    w2 = o2 = None
    if second is not None:
        w2, o2 = second
        _chk(w2, "second weight", torch.float32, 1), _chk(o2, "second output", torch.float32, 2)
        if w2.numel() != H or o2.shape[0] < n_out or o2.shape[1] != H:
            raise KernelError("rmsnorm_scaled: the second norm's weight or output")
    _ok(lib().moe_rmsnorm_scaled(_p(x), _p(a), _p(sa), _p(b), _p(sb), _p(weight), _p(rows), _p(out32), _p(out16), n_out,
                                 S, H, float(eps), 1 if (write_back and rows is None) else 0, _p(status), _p(cy), _p(cpos),
                                 _p(cw), int(top_k), _p(cshared), _p(w2), _p(o2), _stream()),
        "rmsnorm_scaled")


def add_inplace(a, b):
    _chk(a, "a", torch.float32), _chk(b, "b", torch.float32)
    if a.numel() != b.numel():
        raise KernelError("add_inplace: sizes differ")
    _ok(lib().moe_add_inplace(_p(a), _p(b), a.numel(), _stream()), "add_inplace")


def gemm_generic(a, w, out, *, bias=None, a_rows=None, group_offsets=None, status=None, m=None):
    """out[i, :] = a[row(i), :] @ w[g(i)].T (+ bias); the plain kernel, any sizes.

    a: [S, K]; w: [N, K] or [G, N, K]; out: [M, N].  ``a_rows`` int32[M] gathers
    rows of a; ``group_offsets`` int32[G+1] splits the M rows into groups."""
    _chk(a, "a", dims=2), _chk(out, "out", dims=2)
    if not w.is_cuda or not w.is_contiguous():
        raise KernelError("gemm: weight must be a contiguous CUDA tensor")
    if w.dim() == 2:
        G, (N, K) = 1, w.shape
    elif w.dim() == 3:
        G, N, K = w.shape
    else:
        raise KernelError("gemm: weight must be [N, K] or [G, N, K]")
    M = out.shape[0] if m is None else m
    if a.shape[1] != K or out.shape[1] != N or M > out.shape[0]:
        raise KernelError(f"gemm: shapes a{tuple(a.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if a_rows is None and a.shape[0] < M:
        raise KernelError("gemm: a has fewer rows than out")
    if a_rows is not None:
        _chk(a_rows, "a_rows", torch.int32, 1)
        if a_rows.numel() < M:
            raise KernelError("gemm: a_rows too short")
    if group_offsets is not None:
        _chk(group_offsets, "group_offsets", torch.int32, 1)
        if group_offsets.numel() != G + 1:
            raise KernelError("gemm: group_offsets must have G + 1 entries")
    elif G != 1:
        raise KernelError("gemm: a stacked weight needs group_offsets")
    if bias is not None:
        _chk(bias, "bias", torch.float32, 1)
        if bias.numel() != N:
            raise KernelError("gemm: bias size")
    _ok(lib().moe_gemm_generic(_p(a), _dt(a), a.stride(0), _p(a_rows), a.shape[0], _p(w), _dt(w), N * K, _p(out),
                               _dt(out), out.stride(0), _p(bias), _p(group_offsets), G, M, N, K, _p(status),
                               _stream()), "gemm_generic")


def rope_split(qkv, pos, inv_freq, nh, nkv, hd, rot, q, k, v, commit=None, status=None):
    """Rotate and split a step's projections.  ``commit=(view, batch)``: also append the keys and
    values to that cache layer in the same launch (only for a step whose attention reads nothing
    from the cache); returns False if this was asked for and the sizes do not allow it (nothing is
    launched then), else True."""
    _chk(qkv, "qkv", torch.float32, 2), _chk(pos, "pos", torch.int32, 1)
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd:
        raise KernelError("rope_split: qkv width")
    for t, n in ((q, nh), (k, nkv), (v, nkv)):
        _chk(t, "q/k/v")
        if t.numel() < T * n * hd or t.dtype != q.dtype:
            raise KernelError("rope_split: output size or dtype")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
        if inv_freq.numel() < rot // 2:
            raise KernelError("rope_split: inv_freq too short")
    if commit is not None:
        view, batch = commit
        g = view.group
        if k.dtype != g.dtype or g.num_kv_heads != nkv or g.head_dim != hd:
            raise KernelError("rope_split: the cache layer differs from the keys in dtype or shape")
        code = lib().moe_rope_split(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q),
                                    _p(k), _p(v), _dt(q), _p(view.k), _p(view.v), _p(batch.seq_of_token),
                                    _p(batch.seq_end), _p(batch.slots), _p(g.table), g.table.stride(0), g.ring,
                                    g.page_size, g.num_pages, _p(status), _stream())
        if code == -1:
            return False
        _ok(code, "rope_split")
        return True
    _ok(lib().moe_rope_split(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q), _p(k), _p(v),
                             _dt(q), None, None, None, None, None, None, 0, 0, 0, 0, None, _stream()), "rope_split")
    return True


def kv_commit(k_new, v_new, view, batch, status):
    """Append the step's keys and values to the cache layer ``view``."""
    g = view.group
    T = batch.num_tokens
    if k_new.dtype != g.dtype:
        raise KernelError("kv_commit: cache dtype differs from the keys'")
    _ok(lib().moe_kv_commit(_p(k_new), _p(v_new), _p(view.k), _p(view.v), _dt(k_new), _p(batch.seq_of_token),
                            _p(batch.pos), _p(batch.seq_end), _p(batch.slots), _p(g.table), g.table.stride(0),
                            g.ring, g.page_size, g.num_pages, T, g.num_kv_heads, g.head_dim, _p(status), _stream()),
        "kv_commit")


class SigmoidWeights:
    """As an attention kernel's ``sink``: the weight of a visible key is sigmoid(score + bias[h]) and the
    weights are not normalised over the keys (``bias``: float32 [heads] or None)."""

    def __init__(self, bias=None):
        self.bias = bias


ATTN_SIGMOID = 2     # AttnVariant.sink in csrc/common.cuh


def _variant(chunk, softcap, sink):
    """(chunk, softcap, sink, the sink's values per head) as the kernels take them: see AttnVariant in
    csrc/common.cuh.  ``sink``: False, True (a term of score 0), a float32 tensor with one number
    per query head (the term's own score), or ``SigmoidWeights``."""
    if isinstance(sink, SigmoidWeights):
        if sink.bias is not None:
            _chk(sink.bias, "head bias", torch.float32, 1)
        return int(chunk or 0), float(softcap or 0.0), ATTN_SIGMOID, _p(sink.bias)
    if isinstance(sink, torch.Tensor):
        _chk(sink, "sink", torch.float32, 1)
        return int(chunk or 0), float(softcap or 0.0), 1, sink.data_ptr()
    return int(chunk or 0), float(softcap or 0.0), 1 if sink else 0, None


def attention_generic(q, k_new, v_new, view, batch, out, *, nh, window, scale, use_local, status, chunk=0,
                      softcap=0.0, sink=False):
    """``chunk``: a position sees the keys of its own chunk of that many positions only (instead of a
    window); ``softcap``: scores pass cap * tanh(s / cap); ``sink``: the softmax's denominator has one
    more term exp(0).  The same three options in every attention kernel."""
    g = view.group
    T = batch.num_tokens
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    _ok(lib().moe_attention_generic(_p(q), _p(k_new), _p(v_new), _p(view.k), _p(view.v), _p(out), _dt(q),
                                    _p(batch.seq_of_token), _p(batch.pos), _p(batch.seq_start), _p(batch.cu_seqlens),
                                    _p(batch.slots), _p(g.table), g.table.stride(0), g.ring, g.page_size,
                                    g.num_pages, T, nh, g.num_kv_heads, g.head_dim, int(window or 0), float(scale),
                                    1 if use_local else 0, _p(status), *_variant(chunk, softcap, sink), _stream()),
        "attention_generic")


def attention_tiled(q, k_new, v_new, view, batch, out, *, nh, window, scale, use_local, status, chunk=0, softcap=0.0,
                    sink=False) -> bool:
    """The same as ``attention_generic`` with 64 queries of a (sequence, head) to a block and the
    keys staged through shared memory (32-bit arithmetic on the CUDA cores).  False, with nothing
    launched, for a layout it does not take (a page size other than 64, unaligned rows)."""
    g = view.group
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    code = lib().moe_attention_tiled(_p(q), _p(k_new), _p(v_new), _p(view.k), _p(view.v), _p(out), _dt(q),
                                     _p(batch.cu_seqlens), _p(batch.seq_start), _p(batch.slots), _p(g.table),
                                     g.table.stride(0), g.ring, g.page_size, g.num_pages, batch.num_seqs,
                                     batch.num_tokens, nh, g.num_kv_heads, g.head_dim, int(window or 0), float(scale),
                                     1 if use_local else 0, _p(status), *_variant(chunk, softcap, sink), _stream())
    if code == -1:
        return False
    _ok(code, "attention_tiled")
    return True


def _router_bias(bias, E):
    if bias is not None:
        _chk(bias, "router bias", torch.float32, 1)
        if bias.numel() != E:
            raise KernelError("router: one bias per expert")
    return bias


def router(h32, w_router, top_k, norm_topk, scale, topk_idx, topk_w, *, shared_gate_w=None, shared_gate=None,
           seq_of_token=None, bias=None, groups=0, keep=0):
    """``bias``: float32 [E], added to the logits before the softmax and the pick.  ``groups``, ``keep``:
    the experts form ``groups`` equal groups of neighbours, and only experts of the ``keep`` groups
    whose best score is largest may be picked (0: no groups)."""
    _chk(h32, "h", torch.float32, 2), _chk(w_router, "router weight", dims=2)
    T, H = h32.shape
    E = w_router.shape[0]
    if w_router.shape[1] != H:
        raise KernelError("router: weight shape")
    _chk(topk_idx, "topk_idx", torch.int32), _chk(topk_w, "topk_w", torch.float32)
    if topk_idx.numel() < T * top_k or topk_w.numel() < T * top_k:
        raise KernelError("router: output size")
    if shared_gate_w is not None:
        _chk(shared_gate_w, "shared gate weight")
        if shared_gate_w.dtype != w_router.dtype or shared_gate_w.numel() != H:
            raise KernelError("router: the shared gate weight must have the router's dtype and width")
        _chk(shared_gate, "shared_gate", torch.float32)
    logits = torch.empty((T, E + (1 if shared_gate_w is not None else 0)), dtype=torch.float32, device=h32.device)
    need = lib().moe_router_scratch_floats(T, H, E, 1 if shared_gate_w is not None else 0)
    scratch = torch.empty((need,), dtype=torch.float32, device=h32.device) if need else None
    _ok(lib().moe_router(_p(h32), _p(w_router), _p(shared_gate_w), _dt(w_router), _p(seq_of_token), T, H, E, top_k,
                         1 if norm_topk else 0, float(scale), _p(logits), _p(topk_idx), _p(topk_w), _p(shared_gate),
                         _p(scratch), need, _p(_router_bias(bias, E)), int(groups), int(keep), _stream()), "router")


def split3(x32: torch.Tensor) -> torch.Tensor:
    """[T, H] float32 -> [T, 3 H] bfloat16 with x = p0 + p1 + p2 exactly (three terms of 8 bits)."""
    _chk(x32, "x", torch.float32, 2)
    T, H = x32.shape
    out = torch.empty((T, 3 * H), dtype=torch.bfloat16, device=x32.device)
    _ok(lib().moe_split3(_p(x32), _p(out), T, H, _stream()), "split3")
    return out


def router_topk(logits, top_k, norm_topk, scale, topk_idx, topk_w, *, num_experts, shared_gate=None, seq_of_token=None,
                bias=None, groups=0, keep=0):
    """Picks and weights from logits [T, E (+ 1 row for the shared gate)] that are already there."""
    _chk(logits, "logits", torch.float32, 2)
    T = logits.shape[0]
    gate_row = logits.shape[1] == num_experts + 1
    if logits.shape[1] not in (num_experts, num_experts + 1) or (gate_row and shared_gate is None):
        raise KernelError("router_topk: logits must have one column per expert (and one for the shared gate)")
    _ok(lib().moe_router_topk(_p(logits), _p(seq_of_token), T, num_experts, 1 if gate_row else 0, top_k,
                              1 if norm_topk else 0, float(scale), _p(topk_idx), _p(topk_w), _p(shared_gate),
                              _p(_router_bias(bias, num_experts)), int(groups), int(keep), _stream()),
        "router_topk")


_SMS = {}


_DECODE_CTAS = None


def decode_splits(device, num_tokens: int, nkv: int, max_end: int = 0) -> int:
    """Key splits of the decode attention: about four small CTAs per SM (each is a chain of
    dependent loads, so many must be in flight), but no more than leave each of a CTA's four warps
    a tile of 32 keys of the longest sequence (``max_end``, 0 if unknown): with a short context and
    one sequence, 32 splits of one tile each cost more in the merge than they gain."""
    idx = torch.device(device).index or 0
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(device).multi_processor_count
    global _DECODE_CTAS
    if _DECODE_CTAS is None:
        _DECODE_CTAS = int(os.environ.get("MOE_B200_DECODE_CTAS", "4"))
    per_sm = _DECODE_CTAS
    n = max(1, min(32, (per_sm * _SMS[idx]) // max(1, num_tokens * nkv)))
    if max_end > 0:
        n = min(n, max(1, -(-max_end // 32) // 4))
    return n


def _head_blocks(nh: int, nkv: int, group_view=None, dtype=None) -> int:
    """Blocks along the heads of the decode attention's grid: a kv head's query heads two at a time, or,
    where the tensor-core kernel for groups of eight and more heads takes the step (bfloat16, records of
    64 or 128, pages of 64), sixteen at a time."""
    group = max(1, nh // max(nkv, 1))
    if (group_view is not None and dtype == torch.bfloat16 and group >= 8 and group_view.head_dim in (64, 128)
            and group_view.page_size == 64 and group_view.ring % 64 == 0):
        return nkv * -(-group // 16)
    return nkv * (1 if group == 1 else -(-group // 2))


def _gate_args(out, T, nh, hd, gate, dv):
    """(gate pointer, its row pitch, dv) of a merge that writes [T, nh * dv] instead of [T, nh * hd]."""
    if not dv:
        if gate is not None:
            raise KernelError("attention: a gate needs the value width dv")
        return None, 0, 0
    if not 0 < dv <= hd or out.numel() < T * nh * dv:
        raise KernelError("attention: dv or the packed output's size")
    if gate is None:
        return None, 0, int(dv)
    if gate.dtype != torch.float32 or gate.dim() != 2 or gate.stride(1) != 1 or tuple(gate.shape) != (T, nh * dv):
        raise KernelError("attention: gate shape, dtype or layout")
    return gate.data_ptr(), gate.stride(0), int(dv)


def attention_decode(q, view, batch, out, *, nh, window, scale, status, gate=None, dv=0, chunk=0, softcap=0.0,
                     sink=False):
    """Attention of one new token per sequence over the cache alone (its own key already
    appended); split along the keys and merged.  With ``dv`` the merge writes [T, nh * dv], the
    first dv columns of every head, times sigmoid(``gate``) (a float32 column slice [T, nh * dv])
    if given."""
    g = view.group
    T = batch.num_tokens
    if q.dtype != g.dtype or out.dtype != q.dtype:
        raise KernelError("attention: dtypes of queries, cache and output must agree")
    gp, gld, gdv = _gate_args(out, T, nh, g.head_dim, gate, dv)
    nsplit = decode_splits(q.device, T, _head_blocks(nh, g.num_kv_heads, g, q.dtype), getattr(batch, "max_end", 0))
    partial = torch.empty(T * nh * nsplit * (g.head_dim + 2), dtype=torch.float32, device=q.device)
    _ok(lib().moe_attention_decode(_p(q), _p(view.k), _p(view.v), _p(out), _p(partial), _dt(q),
                                   _p(batch.seq_of_token), _p(batch.pos), _p(batch.slots), _p(g.table),
                                   g.table.stride(0), g.ring, g.page_size, g.num_pages, T, nh, g.num_kv_heads,
                                   g.head_dim, int(window or 0), float(scale), nsplit, gp, gld, gdv, _p(status),
                                   *_variant(chunk, softcap, sink), _stream()),
        "attention_decode")


_TICKETS = {}


def _tickets(device, n: int) -> torch.Tensor:
    """Zeroed counters that kernels with a 'last CTA finishes the job' step use and leave zero."""
    idx = torch.device(device).index or 0
    t = _TICKETS.get(idx)
    if t is None or t.numel() < n:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the ticket array must be sized before a CUDA graph is captured")
        t = _TICKETS[idx] = torch.zeros(max(n, 1 << 14), dtype=torch.int32, device=device)
    return t


def attention_decode_fused(qkv, inv_freq, rot, view, batch, out, *, nh, window, scale, status, gate=None, dv=0) -> bool:
    """One token per sequence, ONE launch: rotate the step's q/k/v rows, append key and value to
    the cache layer ``view``, attend over the cache split along the keys, merge.  False (nothing
    launched) if the head size is not one the fast kernel takes.  ``gate`` / ``dv``: as in
    ``attention_decode``."""
    _chk(qkv, "qkv", torch.float32, 2)
    g = view.group
    T = batch.num_tokens
    gp, gld, gdv = _gate_args(out, T, nh, g.head_dim, gate, dv)
    if qkv.shape[1] != (nh + 2 * g.num_kv_heads) * g.head_dim or out.dtype != g.dtype:
        raise KernelError("attention_decode_fused: shapes or dtypes do not fit the cache")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
    nsplit = decode_splits(qkv.device, T, _head_blocks(nh, g.num_kv_heads), getattr(batch, "max_end", 0))
    partial = torch.empty(T * nh * nsplit * (g.head_dim + 2), dtype=torch.float32, device=qkv.device)
    tickets = _tickets(qkv.device, T * g.num_kv_heads)
    code = lib().moe_attention_decode_fused(_p(qkv), _p(inv_freq) if rot else None, rot, _p(view.k), _p(view.v),
                                            _p(out), _p(partial), _p(tickets), _dt(out), _p(batch.seq_of_token),
                                            _p(batch.pos), _p(batch.slots), _p(g.table), g.table.stride(0), g.ring,
                                            g.page_size, g.num_pages, T, nh, g.num_kv_heads, g.head_dim,
                                            int(window or 0), float(scale), nsplit, gp, gld, gdv, _p(status), _stream())
    if code == -1:
        return False
    _ok(code, "attention_decode_fused")
    return True


def moe_align(topk_idx, num_tokens, top_k, num_experts, offsets, sorted_token, pos_of_pair, status):
    for t in (topk_idx, offsets, sorted_token, pos_of_pair):
        _chk(t, "align", torch.int32)
    if offsets.numel() != num_experts + 1 or sorted_token.numel() < num_tokens * top_k:
        raise KernelError("moe_align: output size")
    _ok(lib().moe_align(_p(topk_idx), num_tokens, top_k, num_experts, _p(offsets), _p(sorted_token), _p(pos_of_pair),
                        _p(status), _stream()), "moe_align")


def swiglu(gu, act, fn="silu", param=0.0):
    """act = fn(gu[:, :I]) * gu[:, I:]; ``fn`` is one of ``GLU_ACTS``, ``param`` its constant if it has
    one (the limit of "clamped_sigmoid": min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1))."""
    _chk(gu, "gu", torch.float32, 2), _chk(act, "act", dims=2)
    rows, two_i = gu.shape
    if two_i % 2 or act.shape != (rows, two_i // 2):
        raise KernelError("swiglu: shapes")
    _ok(lib().moe_swiglu(_p(gu), _p(act), _dt(act), rows, two_i // 2, GLU_ACTS[fn], float(param), _stream()), "swiglu")


def moe_combine(y, pos_of_pair, topk_w, top_k, out, *, shared=None, shared_gate=None):
    _chk(y, "y", torch.float32, 2), _chk(out, "out", torch.float32, 2)
    T, H = out.shape
    _ok(lib().moe_combine(_p(y), _p(pos_of_pair), _p(topk_w), top_k, _p(shared), _p(shared_gate), _p(out), T, H,
                          _stream()), "moe_combine")


_sample_ws = {}


def sample(logits, slots, rng_states, out_tokens, *, temp=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, history=None,
           last_token=None, kernel=None):
    """One token per row of ``logits``.  ``kernel="global"`` takes the kernel that works over global
    memory whatever the vocabulary (otherwise only a vocabulary too large for a cluster's shared
    memory does)."""
    _chk(logits, "logits", torch.float32, 2), _chk(out_tokens, "out_tokens", torch.int32, 1)
    R, V = logits.shape
    if temp > 0:
        _chk(slots, "slots", torch.int32, 1), _chk(rng_states, "rng_states", torch.int64, 1)
    if last_token is not None:
        _chk(last_token, "last_token", torch.int32, 1), _chk(slots, "slots", torch.int32, 1)
        if slots.numel() < R:
            raise KernelError("sample: fewer slots than rows")
    hl = 0
    if history is not None:
        _chk(history, "history", torch.int32, 2)
        hl = history.shape[1]
    if out_tokens.numel() < R:
        raise KernelError("sample: fewer places for tokens than rows")
    ws = _sample_ws.get(logits.device)
    if ws is None or ws.numel() < 2 * R:       # zeroed once; the kernels leave it zeroed
        ws = _sample_ws[logits.device] = torch.zeros(max(2 * R, 512), dtype=torch.int64, device=logits.device)
    _ok(lib().moe_sample(_p(logits), R, V, _p(slots), _p(rng_states), _p(history), hl, float(temp), int(top_k),
                         float(top_p), float(repeat_penalty), _p(out_tokens), _p(last_token), _p(ws), ws.numel() * 8,
                         1 if kernel == "global" else 0, _stream()), "sample")


def logprobs(logits, tokens, top: int):
    """What the model thought of the committed ``tokens`` [rows], from the raw ``logits`` [rows, vocab]:
    (logprob [rows] float32, ids [rows, top] int32, logprobs [rows, top] float32), the ``top`` most
    likely tokens strongest first (reference: src/generate.rs:91-105)."""
    _chk(logits, "logits", torch.float32, 2), _chk(tokens, "tokens", torch.int32, 1)
    R, V = logits.shape
    if tokens.numel() < R or not 0 <= top <= 64:
        raise KernelError("logprobs: fewer tokens than rows, or more than 64 alternatives")
    lp = torch.empty(R, dtype=torch.float32, device=logits.device)
    ids = torch.empty((R, top), dtype=torch.int32, device=logits.device)
    lps = torch.empty((R, top), dtype=torch.float32, device=logits.device)
    _ok(lib().moe_logprobs(_p(logits), R, V, _p(tokens), top, _p(lp), _p(ids) if top else None,
                           _p(lps) if top else None, _stream()), "logprobs")
    return lp, ids, lps


def seed_rng(rng_states, slots, seeds):
    _chk(rng_states, "rng_states", torch.int64, 1), _chk(slots, "slots", torch.int32, 1)
    _chk(seeds, "seeds", torch.int64, 1)
    _ok(lib().moe_seed_rng(_p(rng_states), _p(slots), _p(seeds), slots.numel(), _stream()), "seed_rng")


def table_update(table, updates, n):
    """table[slot, index] = page for the first n (slot, index, page) triples of ``updates``."""
    _chk(table, "table", torch.int32, 2), _chk(updates, "updates", torch.int32)
    if updates.numel() < 3 * n:
        raise KernelError("table_update: updates too short")
    _ok(lib().moe_table_update(_p(table), table.stride(0), _p(updates), n, _stream()), "table_update")


def rope_commit(qkv, pos, inv_freq, nh, nkv, hd, rot, q, view, batch, status):
    """Decode step: rotate, write the queries, and append keys and values straight into the
    cache layer ``view`` (one launch instead of rope_split + kv_commit)."""
    _chk(qkv, "qkv", torch.float32, 2), _chk(pos, "pos", torch.int32, 1)
    g = view.group
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or nkv != g.num_kv_heads or hd != g.head_dim or q.dtype != g.dtype:
        raise KernelError("rope_commit: shapes or dtypes do not fit the cache")
    if rot:
        _chk(inv_freq, "inv_freq", torch.float32, 1)
    _ok(lib().moe_rope_commit(_p(qkv), _p(pos), _p(inv_freq) if rot else None, T, nh, nkv, hd, rot, _p(q), _p(view.k),
                              _p(view.v), _dt(q), _p(batch.seq_of_token), _p(batch.slots), _p(g.table),
                              g.table.stride(0), g.ring, g.page_size, g.num_pages, _p(status), _stream()),
        "rope_commit")


def norm_route(x, delta, norm_w, eps, w_router, top_k, norm_topk, scale, *, bf16, shared_gate_w=None,
               seq_of_token=None, status=None, groups=0, keep=0):
    """Few tokens: ``x += delta``, RMS norm, router logits, pick, table inversion and gather of the
    normalised bfloat16 rows in ONE launch.  Returns None (nothing launched) for sizes the kernel
    does not take, else (out32 or None, out16 or None, topk_idx, topk_w, shared_gate, offsets,
    sorted_token, pos_of_pair, gathered or None)."""
    _chk(x, "x", torch.float32, 2), _chk(norm_w, "norm weight", torch.float32, 1), _chk(w_router, "router weight", dims=2)
    T, H = x.shape
    E = w_router.shape[0]
    if T > 64 or E > 256 or T * top_k > 4096 or norm_w.numel() != H or w_router.shape[1] != H:
        return None
    dev = x.device
    out16 = torch.empty((T, H), dtype=torch.bfloat16, device=dev) if bf16 else None
    out32 = None if bf16 else torch.empty((T, H), dtype=torch.float32, device=dev)
    P_ = T * top_k
    topk_idx = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    topk_w = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    sg = torch.empty((T,), dtype=torch.float32, device=dev) if shared_gate_w is not None else None
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    sorted_token = torch.empty((P_,), dtype=torch.int32, device=dev)
    pos_of_pair = torch.empty((P_,), dtype=torch.int32, device=dev)
    xs = torch.empty((P_, H), dtype=torch.bfloat16, device=dev) if bf16 and (H * 2) % 16 == 0 else None
    ticket = _tickets(dev, 1)
    code = lib().moe_norm_route(_p(x), _p(delta), _p(norm_w), float(eps), H, T, _p(out32), _p(out16), _p(w_router),
                                _p(shared_gate_w), _dt(w_router), E, top_k, 1 if norm_topk else 0, float(scale),
                                _p(seq_of_token), _p(topk_idx), _p(topk_w), _p(sg), _p(offsets), _p(sorted_token),
                                _p(pos_of_pair), _p(xs), _p(ticket), _p(status), int(groups), int(keep), _stream())
    if code == -1:
        return None
    _ok(code, "norm_route")
    return out32, out16, topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs


def route_dispatch(h32, w_router, top_k, norm_topk, scale, *, shared_gate_w=None, seq_of_token=None, gather=None,
                   status=None, bias=None, groups=0, keep=0):
    """Few tokens (<= 64) and <= 256 experts: router logits, then pick + table inversion + gather in
    ONE more launch.  Returns (topk_idx, topk_w, shared_gate, offsets, sorted_token, pos_of_pair,
    gathered) where ``gathered[p] = gather[sorted_token[p]]`` (or None)."""
    _chk(h32, "h", torch.float32, 2), _chk(w_router, "router weight", dims=2)
    T, H = h32.shape
    E = w_router.shape[0]
    dev = h32.device
    rows = E + (1 if shared_gate_w is not None else 0)
    logits = torch.empty((T, rows), dtype=torch.float32, device=dev)
    _ok(lib().moe_router_logits(_p(h32), _p(w_router), _p(shared_gate_w), _dt(w_router), T, H, E, _p(logits), None, 0,
                                _stream()), "router_logits")
    P_ = T * top_k
    topk_idx = torch.empty((T, top_k), dtype=torch.int32, device=dev)
    topk_w = torch.empty((T, top_k), dtype=torch.float32, device=dev)
    sg = torch.empty((T,), dtype=torch.float32, device=dev) if shared_gate_w is not None else None
    offsets = torch.empty((E + 1,), dtype=torch.int32, device=dev)
    sorted_token = torch.empty((P_,), dtype=torch.int32, device=dev)
    pos_of_pair = torch.empty((P_,), dtype=torch.int32, device=dev)
    xs, row_bytes = None, 0
    if gather is not None:
        _chk(gather, "gather", dims=2)
        row_bytes = gather.shape[1] * gather.element_size()
        if row_bytes % 16:
            gather, row_bytes = None, 0
        else:
            xs = torch.empty((P_, gather.shape[1]), dtype=gather.dtype, device=dev)
    _ok(lib().moe_route_dispatch(_p(logits), _p(seq_of_token), T, E, 1 if shared_gate_w is not None else 0, top_k,
                                 1 if norm_topk else 0, float(scale), _p(topk_idx), _p(topk_w), _p(sg), _p(offsets),
                                 _p(sorted_token), _p(pos_of_pair), _p(gather), _p(xs), row_bytes, _p(status),
                                 _p(_router_bias(bias, E)), int(groups), int(keep), _stream()), "route_dispatch")
    return topk_idx, topk_w, sg, offsets, sorted_token, pos_of_pair, xs


def whole_prepare(proj, batch, *, nh, nkv, d, dv, width, q, k, v, q_norm=None, k_norm=None, eps=0.0, freq=None, rot=0,
                  vfreq=None, commit=None, status=None):
    """From a step's 32-bit projection rows [q heads | k heads | v heads]: an RMS norm over ALL query
    channels at once and over all key channels (``q_norm`` [nh * d], ``k_norm`` [nkv * d]; None: no norm),
    the rotation of the first ``rot`` dimensions of query and key heads (pairs (i, i + rot/2)), the
    rotation of every value head over all its dimensions by the token's position (``vfreq`` [dv / 2]; None:
    values pass), and the split into q [T, nh, width] and k, v [T, nkv, width], zero-filled.
    ``commit=view`` also appends keys and values to that cache layer."""
    _chk(proj, "proj", torch.float32, 2)
    T = proj.shape[0]
    for t, n in ((q, nh), (k, nkv), (v, nkv)):
        if (not t.is_cuda or t.dtype != q.dtype or tuple(t.shape) != (T, n, width) or t.stride(2) != 1
                or t.stride(1) != width or t.stride(0) < n * width):
            raise KernelError("whole_prepare: q, k, v must be [T, heads, width] with dense heads, of one dtype")
    if k.stride(0) != v.stride(0) or proj.shape[1] < (nh + nkv) * d + nkv * dv:
        raise KernelError("whole_prepare: token pitch of keys and values, or projection width")
    for w, n in ((q_norm, nh * d), (k_norm, nkv * d)):
        if w is not None:
            _chk(w, "norm weight", torch.float32, 1)
            if w.numel() != n:
                raise KernelError("whole_prepare: a norm weight has one factor per channel of the projection")
    if rot:
        _chk(freq, "freq", torch.float32, 1)
        if freq.numel() < rot // 2:
            raise KernelError("whole_prepare: frequency table too short")
    if vfreq is not None:
        _chk(vfreq, "vfreq", torch.float32, 1)
        if dv % 2 or vfreq.numel() < dv // 2:
            raise KernelError("whole_prepare: rotated values need an even width and dv / 2 frequencies")
    kc = vc = se = sl = tb = None
    ts = ring = ps = npg = 0
    if commit is not None:
        g = commit.group
        if k.dtype != g.dtype or g.num_kv_heads != nkv or g.head_dim != width:
            raise KernelError("whole_prepare: the cache layer differs from the keys in dtype or shape")
        kc, vc, se, sl, tb = commit.k, commit.v, batch.seq_end, batch.slots, g.table
        ts, ring, ps, npg = g.table.stride(0), g.ring, g.page_size, g.num_pages
    _ok(lib().moe_whole_prepare(_p(proj), proj.stride(0), _p(batch.pos), _p(batch.seq_of_token), _p(q_norm), _p(k_norm),
                                float(eps), _p(freq) if rot else None, int(rot), _p(vfreq), T, nh, nkv, d, dv, width,
                                _p(q), _p(k), _p(v), q.stride(0), k.stride(0), _dt(q), _p(kc), _p(vc), _p(se), _p(sl),
                                _p(tb), ts, ring, ps, npg, _p(status), _stream()), "whole_prepare")


def unrotate_pack(ctx, pos, vfreq, out, *, nh, dv, width):
    """out[t, h * dv + :] = head h of ctx [T, nh, width] turned back by the token's position: pair
    (m, m + dv/2) by -pos * vfreq[m]; the record's columns beyond dv are dropped."""
    _chk(ctx, "ctx", dims=3), _chk(out, "out", dims=2), _chk(vfreq, "vfreq", torch.float32, 1)
    T = ctx.shape[0]
    if (ctx.shape[1:] != (nh, width) or out.dtype != ctx.dtype or tuple(out.shape) != (T, nh * dv) or dv % 2
            or vfreq.numel() < dv // 2 or width < dv):
        raise KernelError("unrotate_pack: shapes or dtypes")
    _ok(lib().moe_unrotate_pack(_p(ctx), _p(pos), _p(vfreq), T, nh, dv, width, _p(out), _dt(out), _stream()),
        "unrotate_pack")


SEQ_CONV_ACTS = {None: 0, "silu": 1}


def seq_conv(jobs, state, batch, *, taps, channels, residual=False, act=None):
    """A causal convolution over time on every channel, for one or two inputs of one shape in a launch.
    ``jobs``: a list of dicts with ``u`` (float32 [T, >= channels], the step's rows; a column slice is
    fine), ``w`` (float32 [taps, channels]), ``bias`` (float32 [channels] or None), ``offset`` (where the
    job's (taps - 1) * channels floats start in a row of ``state``) and ``out32`` / ``out16`` ([T, channels]
    or None).  y_t = act(sum_j w[j] u_(t - taps + 1 + j) + bias) (+ u_t with ``residual``); rows before
    the step come from the state (the last taps - 1 rows of the sequence, oldest first).  In a step of
    one token a sequence the state is moved on here; otherwise the caller runs ``conv_state_update``."""
    if not 1 <= len(jobs) <= 2:
        raise KernelError("seq_conv: one or two jobs")
    if taps > 1:
        _chk(state, "state", torch.float32, 2)
    args = []
    T = jobs[0]["u"].shape[0]
    for j in jobs:
        u, w = j["u"], j["w"]
        if (u.dtype != torch.float32 or not u.is_cuda or u.dim() != 2 or u.stride(1) != 1 or u.shape[0] != T
                or u.shape[1] < channels):
            raise KernelError("seq_conv: the rows must be float32 [T, >= channels]")
        _chk(w, "taps", torch.float32, 2)
        if tuple(w.shape) != (taps, channels):
            raise KernelError("seq_conv: a tap has one factor per channel")
        if j.get("bias") is not None:
            _chk(j["bias"], "bias", torch.float32, 1)
        o32, o16 = j.get("out32"), j.get("out16")
        for o, dt in ((o32, torch.float32), (o16, torch.bfloat16)):
            if o is not None:
                _chk(o, "out", dt, 2)
                if tuple(o.shape) != (T, channels):
                    raise KernelError("seq_conv: output shape")
        st = None
        if taps > 1:
            off = int(j.get("offset", 0))
            if off + (taps - 1) * channels > state.shape[1]:
                raise KernelError("seq_conv: the state's row is too short")
            st = state.data_ptr() + 4 * off
        args += [_p(u), u.stride(0), _p(w), _p(j.get("bias")), st, _p(o32), _p(o16)]
    if len(jobs) == 1:
        args += [None, 0, None, None, None, None, None]
    _ok(lib().moe_seq_conv(len(jobs), *args, int(taps), int(channels), state.stride(0) if taps > 1 else 0,
                           _p(batch.seq_of_token), _p(batch.pos), _p(batch.cu_seqlens), _p(batch.slots), T,
                           1 if residual else 0, SEQ_CONV_ACTS[act], 1 if (batch.all_decode and taps > 1) else 0,
                           _stream()), "seq_conv")


def embed_pair(table, pair, norm_w, eps, batch, out, prev_state, *, buckets, mul_prev, mul_cur, status):
    """out = rmsnorm(table[token] + pair[(previous * mul_prev + token * mul_cur) mod buckets]) * norm_w, row
    ``buckets`` of ``pair`` at a sequence's first position; ``prev_state`` (int32 [slots + 1]) holds the
    token every sequence saw last and is moved on."""
    _chk(table, "table", dims=2), _chk(pair, "pair", dims=2), _chk(norm_w, "norm weight", torch.float32, 1)
    _chk(out, "out", torch.float32, 2), _chk(prev_state, "prev_state", torch.int32)
    T, H = out.shape
    if table.dtype != pair.dtype or table.shape[1] != H or pair.shape != (buckets + 1, H) or norm_w.numel() != H:
        raise KernelError("embed_pair: shapes or dtypes")
    _ok(lib().moe_embed_pair(_p(table), _p(pair), _dt(table), _p(norm_w), float(eps), _p(batch.token_ids), _p(out), T, H,
                             table.shape[0], int(buckets), int(mul_prev), int(mul_cur), _p(prev_state),
                             _p(batch.seq_of_token), _p(batch.pos), _p(batch.cu_seqlens), _p(batch.slots),
                             _p(getattr(batch, "last_token", None)), _p(status), _stream()), "embed_pair")


def pair_norm_mean(a, wa, b, wb, eps, out):
    """out = (rmsnorm(a) * wa + rmsnorm(b) * wb) / 2 over the last axis, 32-bit."""
    for t in (a, b, out):
        _chk(t, "rows", torch.float32, 2)
    _chk(wa, "wa", torch.float32, 1), _chk(wb, "wb", torch.float32, 1)
    T, H = a.shape
    if b.shape != a.shape or out.shape != a.shape or wa.numel() != H or wb.numel() != H:
        raise KernelError("pair_norm_mean: shapes")
    _ok(lib().moe_pair_norm_mean(_p(a), _p(wa), _p(b), _p(wb), float(eps), T, H, _p(out), _stream()), "pair_norm_mean")


def relu2(x, out):
    """out = relu(x)^2, rounded to ``out``'s dtype."""
    _chk(x, "x", torch.float32), _chk(out, "out")
    if out.numel() != x.numel():
        raise KernelError("relu2: sizes differ")
    _ok(lib().moe_relu2(_p(x), _p(out), _dt(out), x.numel(), _stream()), "relu2")


def table_route(table, batch, top_k, num_experts, topk_idx, topk_w, status):
    """topk_idx[t, :] = table[token id of row t, :top_k]; every weight 1 / top_k; rows of no sequence get
    no expert."""
    _chk(table, "table", torch.int32, 2), _chk(topk_idx, "topk_idx", torch.int32, 2)
    _chk(topk_w, "topk_w", torch.float32, 2)
    T = topk_idx.shape[0]
    if table.shape[1] < top_k or tuple(topk_idx.shape) != (T, top_k) or tuple(topk_w.shape) != (T, top_k):
        raise KernelError("table_route: shapes")
    _ok(lib().moe_table_route(_p(table), table.shape[1], _p(batch.token_ids), _p(batch.seq_of_token), _p(batch.slots),
                              _p(getattr(batch, "last_token", None)), T, table.shape[0], int(top_k), int(num_experts),
                              _p(topk_idx), _p(topk_w), _p(status), _stream()), "table_route")


def scan_segments(batch, blocks_per_sequence: int, device) -> int:
    """Into how many segments a sequence's tokens are cut for ``ssd_scan`` and ``wkv_scan``: one where the launch fills
    the GPU anyway or the sequences are short; else enough to fill it, of at least 128 tokens each, eight
    at most.  (``MOE_B200_SCAN_SEGMENTS``: 0 this rule, n > 0 that many.)"""
    forced = int(os.environ.get("MOE_B200_SCAN_SEGMENTS", "0"))
    longest = int(getattr(batch, "max_new", 0) or 0)
    if forced > 0:
        return max(1, min(forced, 64))
    if longest < 256:
        return 1
    idx = torch.device(device).index or 0
    if idx not in _SMS:
        _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    room = (2 * _SMS[idx]) // max(1, batch.num_seqs * blocks_per_sequence)
    return max(1, min(8, room, longest // 128))


def ssd_scan(xbc, dt_raw, dt_bias, a_log, dskip, state, batch, y, *, heads, groups, n, dv, offset=0, segments=None):
    """Per sequence and head, tokens in order: dt = softplus(dt_raw + dt_bias), S <- exp(-exp(a_log) dt) S +
    dt B x^T, y = S^T C + dskip x.  ``xbc``: float32 [T, heads * dv + 2 groups n] = [x | B | C]; ``dt_raw``:
    float32 [T, heads] (a column slice is fine); ``state``: float32 [slots + 1, ...] whose rows hold
    heads * n * dv floats from ``offset``; y: float32 [T, heads * dv].  ``segments``: into how many pieces
    that run side by side every sequence's tokens are cut (None: ``scan_segments`` decides)."""
    _chk(xbc, "xbc", torch.float32, 2), _chk(y, "y", torch.float32, 2)
    for t in (dt_bias, a_log, dskip):
        _chk(t, "per-head constant", torch.float32, 1)
    T = y.shape[0]
    if (dt_raw.dtype != torch.float32 or dt_raw.dim() != 2 or dt_raw.stride(1) != 1 or tuple(dt_raw.shape) != (T, heads)
            or xbc.shape != (T, heads * dv + 2 * groups * n) or y.shape[1] != heads * dv or state.dtype != torch.float32
            or state.stride(1) != 1 or offset + heads * n * dv > state.shape[1] or dt_bias.numel() != heads):
        raise KernelError("ssd_scan: shapes")
    segs = scan_segments(batch, heads * -(-dv // 64), y.device) if segments is None else int(segments)
    seg_len, ends, decays = 0, None, None
    if segs > 1:
        longest = int(getattr(batch, "max_new", 0) or 0) or T
        seg_len = -(-(-(-longest // segs)) // 16) * 16
        ends = torch.empty((batch.num_seqs, segs, heads, n, dv), dtype=torch.float32, device=y.device)
        decays = torch.empty((batch.num_seqs, segs, heads), dtype=torch.float32, device=y.device)
    _ok(lib().moe_ssd_scan(_p(xbc), xbc.stride(0), _p(dt_raw), dt_raw.stride(0), _p(dt_bias), _p(a_log), _p(dskip),
                           state.data_ptr() + 4 * offset, state.stride(0), _p(batch.cu_seqlens), _p(batch.slots),
                           batch.num_seqs, heads, groups, n, dv, _p(y), segs, seg_len, _p(ends), _p(decays), _stream()),
        "ssd_scan")


def ssd_finish(y, z, norm_w, eps, batch, out, *, norm_groups):
    """out = norm(y * silu(z)): an RMS norm over each of ``norm_groups`` equal parts of the row, times
    ``norm_w``, rounded to ``out``'s dtype.  ``z``: float32 [T, inner], a column slice is fine."""
    _chk(y, "y", torch.float32, 2), _chk(norm_w, "norm weight", torch.float32, 1), _chk(out, "out", dims=2)
    T, inner = y.shape
    if (z.dtype != torch.float32 or z.stride(1) != 1 or tuple(z.shape) != (T, inner) or out.shape != y.shape
            or norm_w.numel() != inner or inner % norm_groups):
        raise KernelError("ssd_finish: shapes")
    _ok(lib().moe_ssd_finish(_p(y), _p(z), z.stride(0), _p(norm_w), float(eps), _p(batch.seq_of_token), T, inner,
                             int(norm_groups), _p(out), _dt(out), _stream()), "ssd_finish")
