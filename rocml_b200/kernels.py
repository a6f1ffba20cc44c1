"""Python face of the CUDA kernel library: one thin function per kernel.

Each function checks devices, element types and layouts, passes raw pointers and the
current CUDA stream to the C entry point, and turns a non-zero return into
``KernelError``.  Nothing here computes; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes
import functools
import inspect
from typing import Optional

import torch

from .csrc.build import library
from .errors import KernelError
from .profile import cost as _cost
from .profile import profiler as _profiler

F32, BF16 = 0, 1
PAGE = 64  # tokens per cache page (RB_PAGE in csrc/common.cuh)

_CODES = {
    10001: "a size the kernel does not take",
    10002: "an element type combination that is not built",
    10003: "a pointer or stride that breaks an alignment rule",
    10004: "a bounded wait inside a kernel ran out",
    10005: "a CUDA driver entry point could not be found",
    10006: "a file could not be read",
}

_c = ctypes
_vp, _i, _ll, _f = _c.c_void_p, _c.c_int, _c.c_longlong, _c.c_float


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {dt} is not supported by the kernels (float32 or bfloat16)")


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("kernel arguments must live on a CUDA device; there is no CPU path")
    return _vp(t.data_ptr())


def _stream():
    # the raw handle of torch's current stream on the current device, without building a Stream object
    return _vp(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


launch_count = 0  # kernel launches issued through this module (graph replays are counted by the engine)


def _check(rc: int, what: str):
    global launch_count
    launch_count += 1
    if rc != 0:
        if rc in _CODES:
            raise KernelError(f"{what}: {_CODES[rc]} (code {rc})")
        raise KernelError(f"{what}: CUDA error {rc}")


# ---- profiling: each wrapper below can be timed with what it had to move and compute ------------------

def _profiled(cost_of):
    """While a profiler is active (rocml_b200.profile), bracket the wrapped launch with a pair of CUDA
    events and file its bytes and operations: ``cost_of(a)`` gets the call's arguments by name and
    returns (bytes, flops).  A wrapper that returns False launched nothing and files nothing."""
    def deco(fn):
        sig = inspect.signature(fn)

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            prof = _profiler.ACTIVE
            if prof is None:
                return fn(*args, **kwargs)
            start = prof.begin()
            result = fn(*args, **kwargs)
            if result is not False:
                bound = sig.bind(*args, **kwargs)
                bound.apply_defaults()
                nbytes, flops = cost_of(bound.arguments, prof.facts)
                prof.end(start, fn.__name__, nbytes, flops)
            return result
        return wrapper
    return deco


def _esz(t) -> int:
    return t.element_size()


def _n_in(x) -> int:
    return x.shape[0] if x.dim() == 3 else 1


def _rows(a, x="x") -> int:
    return a[x].shape[0] if a.get("m") is None else a["m"]


def _attention_cost(a, facts, q="q"):
    window = a.get("window") or None
    n = a["n_seqs"]
    q_lens, kv_lens = facts.q_lens[:n], facts.kv_lens[:n]
    return _cost.attention(q_lens, kv_lens, a["nq"], a["nkv"], a["hd"], _esz(a["k_cache"]), window)


def _i32(t: torch.Tensor, name: str):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")
    return _ptr(t)


_sigs_done = False


def _lib():
    global _sigs_done
    lib = library()
    if not _sigs_done:
        lib.rb_embedding.argtypes = [_vp, _vp, _i, _vp, _i, _i, _i, _vp, _vp]
        lib.rb_add_rmsnorm.argtypes = [_vp, _vp, _i, _ll, _vp, _i, _vp, _i, _vp, _i, _i, _f, _i, _vp, _vp, _vp, _i, _ll, _vp]
        lib.rb_silu_mul.argtypes = [_vp, _i, _i, _ll, _vp, _i, _i, _i, _i, _vp]
        lib.rb_cast.argtypes = [_vp, _i, _vp, _i, _ll, _vp]
        lib.rb_qk_norm_rope_cache.argtypes = [_vp, _i, _i, _ll, _i, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _f,
                                              _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _i, _vp, _i, _i, _i, _i, _vp, _i, _vp,
                                              _vp, _vp, _vp]
        lib.rb_rope_table.argtypes = [_vp, _vp, _i, _i, _f, _vp, _vp]
        lib.rb_gemm_generic.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _ll, _vp]
        lib.rb_attention_generic.argtypes = [_vp, _i, _vp, _i, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i,
                                             _i, _i, _i, _f, _i, _i, _f, _i, _i, _vp, _vp, _i, _vp]
        lib.rb_attention_merge.argtypes = [_vp, _vp, _vp, _i, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp]
        lib.rb_argmax.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _i, _vp]
        lib.rb_attention_prefill.argtypes = [_vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _i,
                                             _f, _i, _i, _f, _vp]
        lib.rb_attention_prefill_tc5.argtypes = [_vp, _i, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _i,
                                                 _i, _i, _i, _f, _i, _i, _f, _i, _vp, _vp, _ll, _i, _vp]
        lib.rb_attention_decode.argtypes = [_vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i, _f, _i,
                                            _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _i, _ll, _ll, _i, _vp]
        lib.rb_attention_decode_fused.argtypes = [_vp, _i, _ll, _i, _vp, _vp, _i, _f, _vp, _i, _vp, _i, _ll, _f, _i,
                                                  _vp, _vp, _vp, _i, _vp, _vp,
                                                  _vp, _i, _i, _i, _i, _f, _i, _i, _i, _vp, _vp, _vp, _vp, _i,
                                                  _i, _f, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _ll, _ll, _vp]
        lib.rb_sample.argtypes = [_vp, _ll, _i, _i, _vp, _vp, _vp, _vp]
        lib.rb_gemm_tcgen05.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _i, _ll, _i, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_add.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_gated_pair.argtypes = [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _vp, _i, _ll, _f, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_qkv_rope.argtypes = [_vp, _vp, _vp, _i, _i, _i, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _i, _vp,
                                                 _vp, _i, _f, _vp, _i, _i, _i, _vp, _vp]
        lib.rb_gemm_tcgen05_residual.argtypes = [_vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp, _ll, _vp, _i, _vp, _ll, _vp,
                                                 _ll, _i, _vp, _vp]
        lib.rb_hold.argtypes = [_ll, _vp]
        lib.rb_embedding_pos.argtypes = [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _f, _vp, _vp, _vp, _vp]
        lib.rb_residual_inject.argtypes = [_vp, _vp, _i, _ll, _vp, _vp, _i, _i, _i, _vp]
        lib.rb_postnorm_add_norm.argtypes = [_vp, _vp, _i, _ll, _vp, _vp, _i, _vp, _f, _vp, _f, _i, _vp, _i, _i, _i, _vp]
        lib.rb_gated_act.argtypes = [_vp, _i, _i, _ll, _ll, _vp, _i, _ll, _i, _i, _i, _f, _f, _i, _vp]
        lib.rb_router_logits.argtypes = [_vp, _i, _ll, _vp, _vp, _i, _i, _i, _i, _vp]
        lib.rb_gemm_tcgen05_grouped.argtypes = [_vp, _vp, _vp, _i, _i, _i, _i, _i, _ll, _ll, _vp, _i, _i, _f, _f, _vp, _vp]
        lib.rb_scale.argtypes = [_vp, _ll, _f, _vp]
        lib.rb_latent_prep.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _vp, _i, _f, _vp, _i, _vp, _vp, _i, _vp, _vp,
                                       _vp, _i, _i, _vp]
        lib.rb_moe_route.argtypes = [_vp, _i, _vp, _i, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp]
        lib.rb_moe_plan.argtypes = [_vp, _i, _i, _i, _vp, _vp, _vp]
        lib.rb_moe_gather.argtypes = [_vp, _i, _i, _vp, _vp, _vp, _i, _i, _vp, _vp, _vp]
        lib.rb_moe_combine.argtypes = [_vp, _ll, _vp, _vp, _i, _i, _vp, _i, _vp, _i, _ll, _vp, _i, _vp]
        lib.rb_grouped_matmul.argtypes = [_vp, _i, _ll, _i, _vp, _i, _ll, _vp, _i, _ll, _i, _i, _i, _i, _i, _vp, _i,
                                          _vp, _i, _i, _f, _f, _vp]
        lib.rb_head_gate.argtypes = [_vp, _ll, _i, _vp, _ll, _i, _vp, _i, _vp, _i, _i, _ll, _ll, _i, _i, _i, _vp]
        lib.rb_decay_scan.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _i,
                                      _vp, _i, _vp]
        lib.rb_decay_step.argtypes = lib.rb_decay_scan.argtypes
        lib.rb_decay_scan_blocks.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _vp, _vp, _vp, _vp, _i,
                                             _i, _vp, _vp, _i, _vp]
        lib.rb_group_norm_gate.argtypes = [_vp, _i, _vp, _i, _i, _ll, _i, _i, _vp, _i, _f, _i, _i, _i, _vp, _i, _i, _vp,
                                           _i, _vp]
        lib.rb_postln.argtypes = [_vp, _vp, _i, _ll, _vp, _vp, _f, _f, _vp, _i, _vp, _i, _i, _vp, _vp, _vp, _vp]
        lib.rb_token_shift.argtypes = [_vp, _vp, _vp, _vp, _vp, _i, _i, _vp, _i, _i, _vp]
        lib.rb_causal_conv.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp, _i, _vp]
        lib.rb_ssm_scan.argtypes = [_vp, _i, _i, _i, _i, _vp, _i, _i, _ll, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp,
                                    _vp, _i, _i, _vp, _i, _vp]
        lib.rb_ssm_scan_blocks.argtypes = [_vp, _i, _i, _i, _i, _vp, _i, _i, _ll, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp,
                                           _vp, _i, _i, _vp, _vp, _vp, _vp, _i, _vp]
        lib.rb_gate_group_norm.argtypes = [_vp, _i, _vp, _i, _i, _ll, _i, _i, _vp, _f, _i, _i, _i, _vp, _i, _i, _vp, _i, _vp]
        lib.rb_latent_rot_prep.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _i, _vp, _vp, _i, _i, _vp,
                                           _vp, _vp, _vp, _i, _i, _vp]
        lib.rb_latent_q_rot.argtypes = [_vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _i, _i, _vp, _i, _vp]
        lib.rb_wide_norm_rope_cache.argtypes = [_vp, _i, _i, _ll, _i, _i, _i, _i, _i, _i, _vp, _vp, _f, _vp, _vp, _i, _i, _vp,
                                                _i, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _vp]
        lib.rb_talk_mix.argtypes = [_vp, _i, _vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _i, _vp]
        lib.rb_gemm_tcgen05_set_wait.argtypes = [_ll, _i]
        lib.rb_gemm_tcgen05_set_wait.restype = None
        _sigs_done = True
    return lib


# ---- embedding --------------------------------------------------------------------------------

@_profiled(lambda a, facts: _cost.embedding(a["out"].shape[0], a["out"].shape[1], _esz(a["table"])))
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, status: Optional[torch.Tensor] = None):
    """out[t, :] = float32(table[ids[t], :]); out is [T, H] float32."""
    T, H = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embedding: out must be contiguous float32, table contiguous")
    if table.shape[1] != H or ids.numel() < T:
        raise KernelError("embedding: shapes do not fit")
    rc = _lib().rb_embedding(_i32(ids, "ids"), _ptr(table), dtype_code(table.dtype), _ptr(out), T, H,
                             table.shape[0], _ptr(status), _stream())
    _check(rc, "embedding")


# ---- fused residual add + RMSNorm ---------------------------------------------------------------

def _n_partials(delta) -> int:
    """How many partial sums a delta (None, [S, T, H], or a pair of such) brings."""
    if delta is None:
        return 0
    if isinstance(delta, (tuple, list)):
        return sum(d.shape[0] for d in delta if d is not None)
    return delta.shape[0]


@_profiled(lambda a, facts: _cost.add_norm(
    a["n_rows"] if a["n_rows"] is not None else (a["rows"].numel() if a["rows"] is not None else a["resid"].shape[0]),
    a["resid"].shape[1], _n_partials(a["delta"]), _esz(a["out"]),
    bool(a["write_back"]) and a["delta"] is not None, _esz(a["weight"])))
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                write_back: bool = True, weight2: Optional[torch.Tensor] = None, out2: Optional[torch.Tensor] = None):
    """resid [T, H] float32 (+= sum of delta [S, T, H] float32); out[i] = rmsnorm(row) * weight.
    ``delta`` may also be a pair of such tensors (the results of a layer's two sublayers): the first one's partial sums
    are added in their order, then the second one's.

    With ``rows`` (int32 indices, -1 = skip) output row i comes from source row rows[i].  ``weight2`` and
    ``out2`` (like ``weight`` and ``out``): a second norm of the same rows with the same eps, whose output differs
    by its weight only."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous() or not out.is_contiguous():
        raise KernelError("add_rmsnorm: resid must be contiguous float32, out contiguous")
    delta_b = None
    if isinstance(delta, (tuple, list)):
        delta, delta_b = delta
    n_delta, stride, n_delta_b, stride_b = 0, 0, 0, 0
    for d in (delta, delta_b):
        if d is not None and (d.dtype != torch.float32 or not d.is_contiguous() or d.dim() != 3 or
                              d.shape[1] < T or d.shape[2] != H):
            raise KernelError("add_rmsnorm: delta must be contiguous float32 [S, >=T, H]")
    if delta is None:
        delta, delta_b = delta_b, None
    if delta is not None:
        n_delta, stride = delta.shape[0], delta.stride(0)
    if delta_b is not None:
        n_delta_b, stride_b = delta_b.shape[0], delta_b.stride(0)
    n = (rows.numel() if rows is not None else T) if n_rows is None else n_rows
    if out.shape[-1] != H or out.numel() < n * H or weight.numel() != H:
        raise KernelError("add_rmsnorm: shapes do not fit")
    if (weight2 is None) != (out2 is None):
        raise KernelError("add_rmsnorm: a second weight comes with a second output")
    if weight2 is not None and (weight2.dtype != weight.dtype or weight2.numel() != H or out2.dtype != out.dtype or
                                not out2.is_contiguous() or out2.shape != out.shape):
        raise KernelError("add_rmsnorm: the second weight and output must look like the first")
    rc = _lib().rb_add_rmsnorm(_ptr(resid), _ptr(delta), n_delta, stride, _ptr(weight), dtype_code(weight.dtype),
                               _ptr(out), dtype_code(out.dtype), None if rows is None else _i32(rows, "rows"),
                               n, H, float(eps), 1 if write_back else 0, _ptr(weight2), _ptr(out2), _ptr(delta_b), n_delta_b,
                               stride_b, _stream())
    _check(rc, "add_rmsnorm")


def _partials(x: torch.Tensor, what: str):
    """(n partial sums, stride between them, row stride) of [T, N] or [S, T, N]."""
    if x.dim() == 3:
        if x.stride(2) != 1:
            raise KernelError(f"{what}: inner stride must be 1")
        return x.shape[0], x.stride(0), x.stride(1)
    if x.stride(1) != 1:
        raise KernelError(f"{what}: inner stride must be 1")
    return 1, 0, x.stride(0)


@_profiled(lambda a, facts: _cost.silu_mul(a["out"].shape[0], a["out"].shape[1], _n_in(a["x"]), _esz(a["x"]), _esz(a["out"])))
def silu_mul(x: torch.Tensor, out: torch.Tensor, paired: bool = False):
    """x [T, 2I] = [gate | up], or [S, T, 2I] partial sums to be added first -> out [T, I] = silu(gate) * up.
    ``paired``: gates and ups alternate in blocks of 16 columns instead of lying in two halves."""
    n_in, in_stride, row_stride = _partials(x, "silu_mul")
    T, I2 = x.shape[-2], x.shape[-1]
    if I2 % 2 or tuple(out.shape) != (T, I2 // 2) or row_stride != I2 or not out.is_contiguous():
        raise KernelError("silu_mul: shapes do not fit")
    _check(_lib().rb_silu_mul(_ptr(x), dtype_code(x.dtype), n_in, in_stride, _ptr(out), dtype_code(out.dtype), T,
                              I2 // 2, 1 if paired else 0, _stream()), "silu_mul")


@_profiled(lambda a, facts: (a["x"].numel() * (_esz(a["x"]) + _esz(a["out"])), 0))
def cast(x: torch.Tensor, out: torch.Tensor):
    if x.numel() != out.numel() or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("cast: shapes do not fit")
    _check(_lib().rb_cast(_ptr(x), dtype_code(x.dtype), _ptr(out), dtype_code(out.dtype), x.numel(), _stream()), "cast")


# ---- q/k norm + rotary + cache write --------------------------------------------------------------

@_profiled(lambda a, facts: _cost.qk_norm_rope(a["n_tokens"], a["nq"], a["nkv"], a["hd"], _n_in(a["proj"]), _esz(a["proj"]),
                                                  _esz(a["q_out"]), bool(a["write_kv"])))
def qk_norm_rope_cache(proj: torch.Tensor, q_out: torch.Tensor, n_tokens: int, nq: int, nkv: int, hd: int,
                       q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                       inv_freq: Optional[torch.Tensor], rot_dim: int, positions: torch.Tensor,
                       slot_of_token: torch.Tensor, block_table: Optional[torch.Tensor],
                       k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor], write_kv: bool = True,
                       cos_sin: Optional[torch.Tensor] = None, v_head_dim: Optional[int] = None,
                       padded_head_dim: Optional[int] = None, interleaved: bool = False,
                       gates: Optional[torch.Tensor] = None, post_norm: bool = False,
                       v_first: Optional[torch.Tensor] = None, v_lambda: Optional[torch.Tensor] = None,
                       v_out: Optional[torch.Tensor] = None):
    """``cos_sin`` (from rope_table, float32 [T, rot_dim / 2, 2]) replaces the kernel's own sincosf.
    proj [T, nq*hd (+ nkv*hd + nkv*vd) (+ gates)] (or [S, T, ...] partial sums): q normalised and rotated into
    q_out (rows of nq*hdp, any row stride; it may be ``proj`` itself when nothing is padded); k (normalised,
    rotated) and v written to their pages.  ``v_head_dim`` (vd): the value heads' width when it is not hd;
    ``padded_head_dim`` (hdp): the width of every head in q_out and in the cache (zeros beyond a head's own);
    ``interleaved``: rotation pairs are neighbours (2i, 2i + 1) instead of (i, i + rot_dim / 2); ``gates``
    (float32 [T, n]): the sigmoid of the row's last n columns.  ``post_norm``: q and k are divided by their root
    mean square over the head (eps inside the root, no weight) after the rotation.  ``v_out`` (float32 [T, nkv * vd])
    receives the value heads as projected; ``v_first`` (such rows of an earlier layer) and ``v_lambda`` (float32,
    one number on the device): the cache receives (1 - lambda) v + lambda v_first."""
    vd = hd if v_head_dim is None else int(v_head_dim)
    hdp = max(hd, vd) if padded_head_dim is None else int(padded_head_dim)
    n_gate = 0 if gates is None else gates.shape[-1]
    width = nq * hd + (nkv * (hd + vd) if write_kv else 0)
    n_in, in_stride, row_stride = _partials(proj, "qk_norm_rope_cache")
    if proj.shape[-1] < width + n_gate:
        raise KernelError(f"qk_norm_rope_cache: projections must be at least {width + n_gate} wide")
    if gates is not None and (gates.dtype != torch.float32 or not gates.is_contiguous() or gates.shape[0] < n_tokens):
        raise KernelError("qk_norm_rope_cache: gates must be contiguous float32 [T, n]")
    if q_out.stride(-1) != 1 or q_out.shape[-1] < nq * hdp:
        raise KernelError("qk_norm_rope_cache: q_out rows must hold nq * hdp elements with unit stride")
    if hdp != hd and q_out.data_ptr() == proj.data_ptr():
        raise KernelError("qk_norm_rope_cache: padded heads cannot be written over the projections")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("qk_norm_rope_cache: give both norm weights or neither")
    wd = dtype_code(q_norm_w.dtype) if q_norm_w is not None else F32
    if q_norm_w is not None and (k_norm_w.dtype != q_norm_w.dtype or q_norm_w.numel() != hd or k_norm_w.numel() != hd):
        raise KernelError("qk_norm_rope_cache: norm weights must share a type and be [head_dim]")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2):
        raise KernelError("qk_norm_rope_cache: inv_freq must be float32 [rot_dim / 2]")
    if write_kv:
        if k_cache is None or v_cache is None or block_table is None:
            raise KernelError("qk_norm_rope_cache: cache tensors missing")
        if k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype or not k_cache.is_contiguous() or \
                tuple(k_cache.shape[1:]) != (nkv, PAGE, hdp):
            raise KernelError("qk_norm_rope_cache: cache must be [pages, nkv, 64, hdp] of the activations' type")
    for name, t in (("v_first", v_first), ("v_out", v_out)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.shape[0] < n_tokens or
                              t.shape[-1] != nkv * vd or not write_kv):
            raise KernelError(f"qk_norm_rope_cache: {name} must be contiguous float32 [T, nkv * vd] of a layer that writes its cache")
    if (v_first is None) != (v_lambda is None) or (v_lambda is not None and (v_lambda.dtype != torch.float32 or v_lambda.numel() != 1)):
        raise KernelError("qk_norm_rope_cache: v_first comes with v_lambda, one float32 number")
    max_pages = block_table.shape[1] if block_table is not None else 0
    rc = _lib().rb_qk_norm_rope_cache(
        _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, _ptr(q_out), dtype_code(q_out.dtype),
        q_out.stride(-2), n_tokens, nq, nkv, hd, _ptr(q_norm_w), _ptr(k_norm_w), wd, float(eps), _ptr(inv_freq),
        rot_dim, _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        None if block_table is None else _i32(block_table, "block_table"), max_pages, _ptr(k_cache), _ptr(v_cache),
        1 if write_kv else 0, _ptr(cos_sin), vd, hdp, 1 if interleaved else 0, n_gate, _ptr(gates),
        1 if post_norm else 0, _ptr(v_first), _ptr(v_lambda), _ptr(v_out), _stream())
    _check(rc, "qk_norm_rope_cache")


@_profiled(lambda a, facts: _cost.rope_table(a["n_tokens"], a["inv_freq"].numel()))
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, n_tokens: int, magnitude: float = 1.0) -> torch.Tensor:
    """float32 [T, half, 2]: (cos, sin) of positions[t] * inv_freq[i], full-precision sincosf, both times ``magnitude``."""
    half = inv_freq.numel()
    out = torch.empty((n_tokens, half, 2), dtype=torch.float32, device=inv_freq.device)
    _check(_lib().rb_rope_table(_i32(positions, "positions"), _ptr(inv_freq), n_tokens, half, float(magnitude), _ptr(out),
                                _stream()),
           "rope_table")
    return out


# ---- matrix products ---------------------------------------------------------------------------------

@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], _esz(a["w"]), _esz(a["x"]), _esz(a["out"]),
                                         _n_in(a["out"])))
def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 m: Optional[int] = None):
    """out[M, N] = x[M, K] . w[N, K]^T (+ bias float32 [N]) on the CUDA cores, 32-bit accumulation.
    ``out`` float32 [S, M, N] with S > 1 (32-bit x and w, at most 16 rows): S partial sums over parts of K,
    to be added in order by the consumer (bias in the first)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    splits, split_stride = 1, 0
    if out.dim() == 3:
        splits, split_stride = out.shape[0], out.stride(0)
        if out.dtype != torch.float32 or out.stride(2) != 1 or out.shape[2] != N:
            raise KernelError("gemm_generic: partial output must be float32 [S, M, N]")
        ldo = out.stride(1)
    else:
        if out.shape[1] != N or out.stride(1) != 1:
            raise KernelError("gemm_generic: shapes or strides do not fit")
        ldo = out.stride(0)
    if x.shape[1] != K or x.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("gemm_generic: shapes or strides do not fit")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_generic: bias must be float32 [N]")
    rc = _lib().rb_gemm_generic(_ptr(x), dtype_code(x.dtype), _ptr(w), dtype_code(w.dtype), _ptr(bias), _ptr(out),
                                dtype_code(out.dtype), M, N, K, x.stride(0), ldo, splits, split_stride, _stream())
    _check(rc, "gemm_generic")


# ---- attention ------------------------------------------------------------------------------------------

@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_generic(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                      n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                      chunk: int = 0, n_chunks: int = 1, part_acc: Optional[torch.Tensor] = None,
                      part_ml: Optional[torch.Tensor] = None, keep: int = 0, sink: Optional[float] = None, cross: int = 0):
    """q rows [T, >= nq*hd] (row stride free) -> out rows [T, >= nq*hd]; keys and values from the pages.
    ``keep``: the keys at positions below it stay visible beside the window; ``sink``: a score that adds
    exp(sink) to every row's denominator and brings no value (None: no such term).  ``cross`` (n > 1, the cache's
    own number of key/value heads): every query head's weights are applied to the values of EVERY stored head;
    ``nkv`` = n * n then counts (key head, value head) pairs, ``nq`` = n * query heads the results, pair
    (a, m) at a * n + m with the results of key head a's queries in their order, and q holds nq / n heads."""
    if q.stride(-1) != 1 or out.stride(-1) != 1 or q.dtype != out.dtype or k_cache.dtype != q.dtype:
        raise KernelError("attention_generic: strides or types do not fit")
    stored = nkv // cross if cross > 1 else nkv
    if tuple(k_cache.shape[1:]) != (stored, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_generic: cache must be [pages, nkv, 64, hd]")
    rc = _lib().rb_attention_generic(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), dtype_code(q.dtype), _ptr(k_cache), _ptr(v_cache),
        _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"),
        _i32(kv_len, "kv_len"), n_seqs, max_q_len, nq, nkv, hd, float(scale), int(window), int(keep), _sink(sink),
        int(chunk), int(n_chunks), _ptr(part_acc), _ptr(part_ml), int(cross), _stream())
    _check(rc, "attention_generic")


NO_SINK = -3.0e38     # RB_NO_SINK of csrc/common.cuh


def _sink(sink: Optional[float]) -> float:
    return NO_SINK if sink is None else float(sink)


PREFILL_L2_BYTES = 96 << 20     # keys and values that stay in the 126 MB L2 cache beside everything else


def prefill_heads_first(n_seqs: int, nkv: int, hd: int, max_kv_len: int, window: int = 0) -> bool:
    """Whether a prompt step's attention starts the longest blocks of all heads first (best balance) or
    runs one head after another (the blocks that run together share keys and values): the first while
    the bfloat16 keys and values of the step's contexts fit the L2 cache (measured: 26 % faster at 2,048
    tokens, 6 % at 16,384, 6 % slower at 32,768, where 134 MB are read by every query tile)."""
    span = min(max_kv_len, abs(window)) if window else max_kv_len      # a window, or blocks of -window positions
    return n_seqs * nkv * span * hd * 4 <= PREFILL_L2_BYTES


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_prefill_tc5(q: torch.Tensor, n_tokens: int, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                          n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                          max_kv_len: Optional[int] = None, keep: int = 0, sink: Optional[float] = None,
                          gate: Optional[torch.Tensor] = None, cross: int = 0) -> bool:
    """bfloat16 flash attention with tcgen05 (accumulators in tensor memory, TMA loads), head sizes 64, 128 and 256.
    ``cross`` (n > 1, the cache's own number of key/value heads): as in ``attention_generic``.
    ``keep``: beside a window the keys at positions below it stay visible; ``sink``: a score whose exponential
    joins every row's denominator.  ``gate``: bfloat16 [T, nq * hd] columns of the projection rows (a view with
    unit stride along a row); the result is multiplied by their sigmoid before it is written.
    ``max_kv_len`` (the longest context of the step; the longest query if not given) only decides the
    order in which blocks start: the longest blocks of all heads first while the keys and values that
    the step reads fit the L2 cache, one head after another beyond.  Returns False when the kernel
    does not take the head size or the alignment."""
    if hd not in (64, 128, 256) or q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            q.stride(-1) != 1 or out.stride(-1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        return False
    if gate is not None and (gate.dtype != torch.bfloat16 or gate.dim() != 2 or gate.stride(1) != 1 or gate.shape != (n_tokens, nq * hd)):
        return False
    if tuple(k_cache.shape[1:]) != (nkv // cross if cross > 1 else nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_prefill_tc5: cache must be [pages, nkv, 64, hd]")
    if cross > 1 and gate is not None:
        return False
    rc = _lib().rb_attention_prefill_tc5(
        _ptr(q), q.stride(0), n_tokens, _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0],
        _i32(block_table, "block_table"), block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"),
        _i32(kv_len, "kv_len"), n_seqs, max_q_len, nq, nkv, hd, float(scale), int(window), int(keep), _sink(sink),
        1 if prefill_heads_first(n_seqs, nkv, hd, max_q_len if max_kv_len is None else max_kv_len, window) else 0,
        _ptr(status_word(q.device)), _ptr(gate), gate.stride(0) if gate is not None else 0, int(cross), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_prefill_tc5")
    return True


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                      n_seqs: int, max_q_len: int, nq: int, nkv: int, hd: int, scale: float, window: int = 0,
                      keep: int = 0, sink: Optional[float] = None) -> bool:
    """bfloat16 flash attention on the tensor cores for any number of query tokens per sequence.
    ``keep``: beside a window the keys at positions below it stay visible; ``sink``: a score whose exponential
    joins every row's denominator.
    Returns False when the kernel does not take the head size or the alignment."""
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or \
            q.stride(-1) != 1 or out.stride(-1) != 1:
        return False
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_prefill: cache must be [pages, nkv, 64, hd]")
    rc = _lib().rb_attention_prefill(
        _ptr(q), q.stride(0), _ptr(out), out.stride(0), _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"),
        block_table.shape[1], _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs,
        max_q_len, nq, nkv, hd, float(scale), int(window), int(keep), _sink(sink), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_prefill")
    return True


_sm_count = {}


def decode_split(n_seqs: int, n_kv_groups: int, n_pages: int, device=0):
    """(blocks per sequence, pages per block) for decode attention.  Three blocks of the kernel fit a
    multiprocessor; the split is the finest that still runs as ONE wave (blocks per sequence times
    sequences times key/value head groups within the resident slots), because a second, partly filled
    wave costs a whole block's latency.  A large batch therefore walks many pages per block (one
    partial result and one merge for all of them) and a single sequence spreads over the device.
    Contexts beyond 4,096 tokens in a batch of four or more, and batches too large for one block a
    (sequence, head group): see below.  Up to 16 blocks per sequence form a thread-block cluster and
    merge through shared memory, which is so much quicker than through global memory that a finer
    split is always cut back to 16."""
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(key).multi_processor_count
    slots = 3 * _sm_count[key]
    pairs = n_seqs * n_kv_groups
    if (4 <= n_seqs <= 256 and n_pages > 64) or \
            (2 <= n_seqs <= 256 and n_pages >= 8 and slots < pairs <= slots + slots // 3):
        # several long contexts, which may differ a lot in length, or a few more (sequence, head group)
        # pairs than blocks run at once (the second, thinly filled wave would take nearly as long as the
        # first; with more pairs than that, waves of whole sequences measured faster): one wave of blocks
        # a head group, which share the pages of all sequences equally (pages per block 0 says so to the
        # kernel)
        return max(1, min(1024, slots // max(1, n_kv_groups))), 0
    blocks = max(1, min(n_pages, slots // max(1, pairs)))
    # more than 16 blocks would merge through global memory, which costs more than the longer blocks
    # of a cluster do (one sequence of 8,192 tokens: 15 us with 16 blocks of 8 pages, 26 us with 43 of 3;
    # at 32,000 tokens 38 against 41)
    blocks = min(blocks, DECODE_CLUSTER_MAX)
    ppb = -(-n_pages // blocks)
    return -(-n_pages // ppb), ppb


DECODE_CLUSTER_MAX = 16

_counters = {}
_COUNTER_INTS = 1 << 20


def decode_counters(device) -> torch.Tensor:
    """Zeroed int32 work space of the decode attention kernel (one counter per sequence and head
    group); the kernel leaves it zeroed, so one buffer per device serves every launch."""
    key = torch.device(device).index or 0
    if key not in _counters:
        _counters[key] = torch.zeros(_COUNTER_INTS, dtype=torch.int32, device=device)
    return _counters[key]


def _check_parts(part_acc, part_ml, n_chunks: int, what: str) -> None:
    """The kernel numbers a row's partial results up to n_chunks - 1 and strides by n_chunks."""
    if n_chunks > 1 and (part_acc is None or part_ml is None or part_acc.shape[2] < n_chunks
                         or part_ml.shape[2] < n_chunks or part_acc.shape[2] != part_ml.shape[2]):
        raise KernelError(f"{what}: work space for {n_chunks} partial results a row is needed")


@_profiled(lambda a, facts: _attention_cost(a, facts))
def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                     n_seqs: int, nq: int, nkv: int, hd: int, scale: float, window: int, n_chunks: int,
                     part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                     pages_per_block: int = 1, keep: int = 0, sink: Optional[float] = None,
                     gate: Optional[torch.Tensor] = None, cross: int = 0) -> bool:
    """``cross`` (n > 1, the cache's own number of key/value heads): as in ``attention_generic``.  ``keep``: the keys at positions below it stay visible beside the window (not with ``pages_per_block`` 0);
    ``sink``: a score whose exponential joins every row's denominator.  ``gate``: [T, nq * hd] or [S, T, nq * hd]
    (partial sums, added in order) columns of the projection rows, bfloat16 or float32, unit stride along a row: the
    result is multiplied by their sigmoid before it is written.
    bfloat16 decode attention, one query token per sequence; a block takes ``pages_per_block``
    pages of 64 keys, ``n_chunks`` blocks cover the longest sequence and are merged by the kernel
    itself; part_acc / part_ml [T, nq, >= n_chunks, ...] are its work space when n_chunks > 1.
    ``pages_per_block`` 0: ``n_chunks`` blocks a key/value head group share the pages of all sequences
    equally, whatever their lengths (see ``decode_split``).  Returns False when the kernel does not
    take the head size or the alignment (use attention_generic)."""
    if n_seqs * nq > _COUNTER_INTS:
        return False
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or q.stride(-1) != 1 or out.stride(-1) != 1:
        return False
    if tuple(k_cache.shape[1:]) != (nkv // cross if cross > 1 else nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_decode: cache must be [pages, nkv, 64, hd]")
    if cross > 1 and gate is not None:
        return False
    _check_parts(part_acc, part_ml, n_chunks, "attention_decode")
    g_n, g_in, g_row = 0, 0, 0
    if gate is not None:
        if gate.dtype not in (torch.bfloat16, torch.float32) or gate.dim() not in (2, 3) or gate.stride(-1) != 1 or \
                gate.shape[-1] != nq * hd:
            return False
        g_n, g_in, g_row = (gate.shape[0], gate.stride(0), gate.stride(1)) if gate.dim() == 3 else (1, 0, gate.stride(0))
    rc = _lib().rb_attention_decode(
        _ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"), block_table.shape[1],
        _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs, nq, nkv, hd, float(scale),
        int(window), int(keep), _sink(sink), int(n_chunks), int(pages_per_block), _ptr(part_acc), _ptr(part_ml),
        _ptr(decode_counters(q.device)), _ptr(out),
        out.stride(0), _ptr(gate), 1 if gate is not None and gate.dtype == torch.float32 else 0, g_n, g_in, g_row, int(cross),
        _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_decode")
    return True


@_profiled(lambda a, facts: tuple(map(sum, zip(_attention_cost(a, facts), (a["proj"].numel() * 4, 0)))))
def attention_decode_fused(proj: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                           block_table: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, kv_len: torch.Tensor,
                           n_seqs: int, nq: int, nkv: int, hd: int, q_norm_w: Optional[torch.Tensor],
                           k_norm_w: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                           write_kv: bool, scale: float, window: int, n_chunks: int,
                           part_acc: Optional[torch.Tensor], part_ml: Optional[torch.Tensor],
                           pages_per_block: int = 1, rowscale=None, row_width: int = 0, keep: int = 0,
                           sink: Optional[float] = None, rot_dim: int = 0, post_norm: bool = False,
                           v_first: Optional[torch.Tensor] = None, v_lambda: Optional[torch.Tensor] = None,
                           v_keep: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None) -> bool:
    """attention_decode for head size 128 that takes the step's projections as the matrix product left
    them: ``proj`` float32 [S, T, (nq + 2 nkv) * 128] partial sums (or [T, ...]; only the nq query heads
    when ``write_kv`` is off).  The kernel adds them, applies the per-head norm and the rotation
    (``cos_sin`` float32 [T, 64, 2] from rope_table) to the queries, and writes the new token's key and
    value into its page before reading it: the work of qk_norm_rope_cache, without a kernel in between.
    ``rowscale`` = (sumsq float32 [G, >= T], eps) with ``row_width``: the rows the projection was made
    from were residual * norm weight; the sums are scaled by rsqrt(sum / row_width + eps) first.
    ``keep``, ``sink`` and ``gate`` as in attention_decode.  ``rot_dim`` (0: the whole head): only the first
    rot_dim dimensions of a head turn and ``cos_sin`` is [T, rot_dim / 2, 2]; ``post_norm``: queries and keys are divided
    by their root mean square after the rotation; ``v_keep``: float32 [T, nkv * 128], receives the new values as projected;
    ``v_first`` and ``v_lambda`` (float32 [1]): such rows of an earlier layer, blended into what is cached.  With any
    of these the rows may hold further columns after the heads.
    Returns False when the kernel does not take the sizes (use the two kernels)."""
    if hd != 128 or proj.dtype != torch.float32 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 \
            or out.stride(-1) != 1 or n_seqs * nq > _COUNTER_INTS:
        return False
    width = (nq + (2 * nkv if write_kv else 0)) * hd
    n_in, in_stride, row_stride = _partials(proj, "attention_decode_fused")
    if proj.shape[-1] != width and (gate is None or proj.shape[-1] < width):
        raise KernelError(f"attention_decode_fused: projections must be {width} wide")
    rot = int(rot_dim) or hd
    if rot % 8 or rot > hd:
        return False
    for name, t in (("v_first", v_first), ("v_keep", v_keep)):
        if t is not None and (t.dtype != torch.float32 or not t.is_contiguous() or t.numel() < n_seqs * nkv * hd):
            raise KernelError(f"attention_decode_fused: {name} must be contiguous float32 [T, nkv * 128]")
    if v_first is not None and (v_lambda is None or v_lambda.dtype != torch.float32):
        raise KernelError("attention_decode_fused: v_first needs v_lambda, float32 [1]")
    g_n, g_in, g_row = 0, 0, 0
    if gate is not None:
        if gate.dtype not in (torch.bfloat16, torch.float32) or gate.dim() not in (2, 3) or gate.stride(-1) != 1 or \
                gate.shape[-1] != nq * hd:
            return False
        g_n, g_in, g_row = (gate.shape[0], gate.stride(0), gate.stride(1)) if gate.dim() == 3 else (1, 0, gate.stride(0))
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hd) or k_cache.shape != v_cache.shape:
        raise KernelError("attention_decode_fused: cache must be [pages, nkv, 64, hd]")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("attention_decode_fused: give both norm weights or neither")
    w_f32 = 0
    if q_norm_w is not None:
        if q_norm_w.dtype != k_norm_w.dtype or q_norm_w.numel() != hd or k_norm_w.numel() != hd:
            raise KernelError("attention_decode_fused: norm weights must share a type and be [head_dim]")
        w_f32 = 1 if q_norm_w.dtype == torch.float32 else 0
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.numel() < n_seqs * rot):
        raise KernelError("attention_decode_fused: cos_sin must be float32 [T, rot_dim / 2, 2]")
    _check_parts(part_acc, part_ml, n_chunks, "attention_decode_fused")
    rc = _lib().rb_attention_decode_fused(
        _ptr(proj), n_in, in_stride, row_stride, _ptr(q_norm_w), _ptr(k_norm_w), w_f32, float(eps), _ptr(cos_sin),
        1 if write_kv else 0, *_row_scale(rowscale, n_seqs, "attention_decode_fused"), int(row_width),
        _ptr(k_cache), _ptr(v_cache), _i32(block_table, "block_table"), block_table.shape[1],
        _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), _i32(kv_len, "kv_len"), n_seqs, nq, nkv, hd, float(scale),
        int(window), int(n_chunks), int(pages_per_block), _ptr(part_acc), _ptr(part_ml),
        _ptr(decode_counters(out.device)), _ptr(out), out.stride(0), int(keep), _sink(sink), rot, 1 if post_norm else 0,
        _ptr(v_first), _ptr(v_lambda), _ptr(v_keep), _ptr(gate), 1 if gate is not None and gate.dtype == torch.float32 else 0,
        g_n, g_in, g_row, _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "attention_decode_fused")
    return True


@_profiled(lambda a, facts: (a["part_acc"].numel() * 4 + a["part_ml"].numel() * 4 + a["n_tokens"] * a["nq"] * a["hd"] * _esz(a["out"]), 0))
def attention_merge(part_acc: torch.Tensor, part_ml: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                    slot_of_token: torch.Tensor, n_tokens: int, nq: int, hd: int, chunk: int, n_chunks: int,
                    window: int = 0, keep: int = 0, sink: Optional[float] = None):
    rc = _lib().rb_attention_merge(_ptr(part_acc), _ptr(part_ml), _ptr(out), out.stride(0), dtype_code(out.dtype),
                                   _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"), n_tokens,
                                   nq, hd, chunk, n_chunks, int(window), int(keep), _sink(sink), _stream())
    _check(rc, "attention_merge")


# ---- sampling ---------------------------------------------------------------------------------------------

_ARGMAX_SLICES = 64


@_profiled(lambda a, facts: _cost.sample(a["logits"].shape[0] if a["rows"] is None else a["rows"], a["logits"].shape[1]))
def argmax(logits: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None):
    """out[r] = index of the first largest value of logits[r, :]; logits float32 [R, V].  Wide rows
    are searched by 64 blocks each, through a small work space."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32:
        raise KernelError("argmax: logits float32 with unit inner stride, out int32")
    R = logits.shape[0] if rows is None else rows
    V = logits.shape[1]
    sv = si = None
    slices = 1
    if V > 8192:
        slices = _ARGMAX_SLICES
        sv = torch.empty((R, slices), dtype=torch.float32, device=logits.device)
        si = torch.empty((R, slices), dtype=torch.int32, device=logits.device)
    _check(_lib().rb_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _ptr(sv), _ptr(si), slices, _stream()),
           "argmax")


@_profiled(lambda a, facts: _cost.sample(a["n"], a["logits"].shape[1]))
def sample(logits: torch.Tensor, n: int, rows: torch.Tensor, history: Optional[torch.Tensor], out: torch.Tensor):
    """One token per row of float32 logits [>= n, V].  ``rows`` holds n records of 8 x 32 bits
    {temperature f32, top_k i32 (0 off), top_p f32 (< 0 off), u f32, penalty f32 (<= 0 off),
    hist_begin i32, hist_len i32, 0} (an int32 tensor with the floats bit-cast); ``history``
    int32 ids.  The repeat penalty edits the logits in place."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or out.dtype != torch.int32 or rows.numel() < 8 * n:
        raise KernelError("sample: logits float32 with unit inner stride, out int32, 8 words per row")
    _check(_lib().rb_sample(_ptr(logits), logits.stride(0), n, logits.shape[1], _i32(rows, "rows"),
                            None if history is None else _i32(history, "history"), _ptr(out), _stream()), "sample")


# ---- tensor-core matrix product (tcgen05) ----------------------------------------------------------------

_status = {}


def status_word(device) -> torch.Tensor:
    """One int32 per device where kernels record a bounded wait that ran out (or a bad token id)."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def raise_for_status(value: int, device=None) -> None:
    """Raise if ``value``, a copy of a device's status word, records a failure; the word itself
    is cleared so that the next step starts clean."""
    if value != 0:
        key = torch.device(device).index or 0 if device is not None else None
        for k, word in _status.items():
            if key is None or k == key:
                word.zero_()
        raise KernelError(f"a kernel reported failure: {_CODES.get(value, 'code ' + str(value))} (code {value})")


def check_status(device) -> None:
    """Read the device's status word (this synchronises) and raise if a kernel recorded a failure."""
    key = torch.device(device).index or 0
    if key in _status:
        raise_for_status(int(_status[key].item()), device)


def hold(microseconds: float) -> None:
    """Keep the current stream busy for about that long (at most a second; not counted as a launch): what is
    enqueued behind it starts when it ends.  The profiler holds the GPU back with it while the host
    enqueues a step."""
    rc = _lib().rb_hold(int(microseconds), _stream())
    if rc != 0:
        raise KernelError(f"hold: CUDA error {rc}")


def set_wait_limit(cycles: int = 0, withhold_first_stage: bool = False) -> None:
    """How long (in clock cycles; 0 restores the default of about two seconds) a warp of the tensor-core
    products waits on a barrier before it gives up, records the failure in the status word and lets
    its block unwind.  ``withhold_first_stage`` is for tests of that path only: few-token products then
    never request their first K block, so the wait for it must run out (with a limit of microseconds
    this takes microseconds and leaves the device usable); they compute nothing useful while it is set."""
    _lib().rb_gemm_tcgen05_set_wait(int(cycles), 1 if withhold_first_stage else 0)


@_profiled(lambda a, facts: (_cost.gated_linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, _esz(a["out"])) if a["gated"] else
                         _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, _esz(a["out"]), _n_in(a["out"]))))
def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 m: Optional[int] = None, stages: int = 0, gated: bool = False, act: str = "silu") -> bool:
    """out = x . w^T on the tensor cores; x, w bfloat16, out bfloat16 [M, N] or float32 [M, N] or
    float32 [S, M, N] (S partial sums over K, to be added by the consumer).  Returns False when the
    kernel refuses the layout (K or a row stride not a multiple of 8, a pointer off 16 bytes);
    the caller then uses the plain kernel.

    ``gated``: w's rows alternate in blocks of 16 between a gate and an up projection of the same
    16 outputs, and out is bfloat16 [M, N / 2] = act(gate) * up, computed in the epilogue (``act`` "silu", or
    "gelu_tanh" for more than 128 rows)."""
    if gated and act not in ("silu", "gelu_tanh"):
        raise KernelError(f"gemm_tcgen05: activation {act!r} is not built into the product")
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05: x and w must be bfloat16, K-major, with matching K")
    if out.dim() == 3:
        splits, split_stride, ldo = out.shape[0], out.stride(0), out.stride(1)
        if out.shape[2] != N or out.stride(2) != 1 or out.dtype != torch.float32:
            raise KernelError("gemm_tcgen05: partial output must be float32 [S, M, N]")
    else:
        splits, split_stride, ldo = 1, 0, out.stride(0)
        if out.shape[1] != (N // 2 if gated else N) or out.stride(1) != 1:
            raise KernelError("gemm_tcgen05: output must be [M, N] (or [M, N / 2] when gated) with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05: bias must be float32 [N]")
    rc = _lib().rb_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0),
                                ldo, splits, split_stride, stages, (1 + GATED_ACTS[act]) if gated else 0,
                                _ptr(status_word(x.device)), _stream())
    if rc == 10003:
        return False
    _check(rc, "gemm_tcgen05")
    return True


def _row_scale(rowscale, m: int, what: str):
    """(pointer, groups, stride, eps) of a deferred 1/RMS: ``rowscale`` = (sumsq float32 [G, >= M], eps)."""
    if rowscale is None:
        return None, 0, 0, 0.0
    sumsq, eps = rowscale
    if sumsq.dtype != torch.float32 or sumsq.dim() != 2 or sumsq.stride(1) != 1 or sumsq.shape[1] < m:
        raise KernelError(f"{what}: the rows' sums of squares must be float32 [groups, >= rows]")
    return _ptr(sumsq), sumsq.shape[0], sumsq.stride(0), float(eps)


@_profiled(lambda a, facts: _cost.gated_linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 2))
def gemm_tcgen05_gated_pair(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, bias: Optional[torch.Tensor] = None,
                            m: Optional[int] = None, rowscale=None) -> bool:
    """h = silu(gate) * up for at most 32 rows, w's rows alternating in blocks of 16 between gate and
    up, with the sum over K done in two halves by two blocks that form a thread-block cluster: the
    second hands its half to the first through shared memory, so no partial sums go through global
    memory.  h is bfloat16 [M, N / 2].  ``rowscale`` = (sumsq float32 [G, >= M], eps): x's rows are
    residual * norm weight, not yet divided by their RMS; column m of sumsq sums to row m's sum of
    squares over K values, and the product is scaled by rsqrt(sum / K + eps) before the bias.
    Returns False when the kernel refuses the sizes or the layout."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_gated_pair: x and w must be bfloat16, K-major, with matching K")
    if h.dtype != torch.bfloat16 or h.shape[1] != N // 2 or h.stride(1) != 1:
        raise KernelError("gemm_tcgen05_gated_pair: h must be bfloat16 [M, N / 2] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_gated_pair: bias must be float32 [N]")
    if M > 32 or N % 32 or K <= 64:
        return False
    rc = _lib().rb_gemm_tcgen05_gated_pair(_ptr(x), _ptr(w), _ptr(bias), _ptr(h), M, N, K, x.stride(0), h.stride(0),
                                           *_row_scale(rowscale, M, "gemm_tcgen05_gated_pair"), 0,
                                           _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_gated_pair")
    return True


@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 4, 1, True))
def gemm_tcgen05_add(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, bias: Optional[torch.Tensor] = None,
                     m: Optional[int] = None) -> bool:
    """resid += x . w^T (+ bias) for many rows (more than 256, N at least 256): the product is added into
    the float32 residual stream in its own epilogue, so no delta goes through memory.  Returns False
    when the kernel refuses the sizes or the layout (write a delta instead)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_add: x and w must be bfloat16, K-major, with matching K")
    if resid.dtype != torch.float32 or resid.shape[1] != N or resid.stride(1) != 1 or resid.shape[0] < M:
        raise KernelError("gemm_tcgen05_add: resid must be float32 [>= M, N] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_add: bias must be float32 [N]")
    if M <= 256 or N < 256:
        return False
    rc = _lib().rb_gemm_tcgen05_add(_ptr(x), _ptr(w), _ptr(bias), _ptr(resid), M, N, K, x.stride(0), resid.stride(0), 0,
                                    _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_add")
    return True


@_profiled(lambda a, facts: tuple(map(sum, zip(_cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 4, 1, True),
                                                       (_rows(a) * a["w"].shape[0] * 2 if a["xhat"] is not None else 0, 0)))))
def gemm_tcgen05_residual(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, splits: int,
                          bias: Optional[torch.Tensor] = None, next_w: Optional[torch.Tensor] = None,
                          xhat: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None,
                          m: Optional[int] = None) -> bool:
    """resid += x . w^T (+ bias) for at most 64 rows, the sum over K in ``splits`` (4, 8, 16) parts by
    the blocks of a thread-block cluster that exchange their parts through shared memory.  For the
    norm that follows: ``xhat`` bfloat16 [M, N] = resid * next_w (the row's 1/RMS is applied by the
    consumer) and ``sumsq`` float32 [ceil(N / 128) * splits, >= M], whose column m sums to the sum of
    squares of row m.  Returns False when the kernel refuses the sizes or the layout."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_residual: x and w must be bfloat16, K-major, with matching K")
    if resid.dtype != torch.float32 or resid.shape[1] != N or resid.stride(1) != 1:
        raise KernelError("gemm_tcgen05_residual: resid must be float32 [M, N] with unit inner stride")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_residual: bias must be float32 [N]")
    if xhat is not None:
        if next_w is None or next_w.numel() != N or next_w.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_tcgen05_residual: xhat needs the norm's weight [N], float32 or bfloat16")
        if xhat.dtype != torch.bfloat16 or xhat.shape[1] != N or xhat.stride(1) != 1:
            raise KernelError("gemm_tcgen05_residual: xhat must be bfloat16 [M, N] with unit inner stride")
    if sumsq is not None and (sumsq.dtype != torch.float32 or sumsq.stride(1) != 1 or sumsq.shape[1] < M
                              or sumsq.shape[0] != ((N + 127) // 128) * splits):
        raise KernelError("gemm_tcgen05_residual: sumsq must be float32 [ceil(N / 128) * splits, >= M]")
    if M > 64 or splits not in (4, 8, 16) or (K + 63) // 64 < splits:
        return False
    rc = _lib().rb_gemm_tcgen05_residual(
        _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0), splits, _ptr(resid), resid.stride(0), _ptr(next_w),
        1 if (next_w is not None and next_w.dtype == torch.float32) else 0, _ptr(xhat),
        xhat.stride(0) if xhat is not None else 0, _ptr(sumsq), sumsq.stride(0) if sumsq is not None else 0, 0,
        _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_residual")
    return True


@_profiled(lambda a, facts: _cost.linear(_rows(a), a["w"].shape[0], a["w"].shape[1], 2, 2, 2))
def gemm_tcgen05_qkv_rope(x: torch.Tensor, w: torch.Tensor, q_out: torch.Tensor, nq: int, nkv: int,
                          q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                          cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slot_of_token: torch.Tensor,
                          block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                          v_cache: Optional[torch.Tensor], bias: Optional[torch.Tensor] = None,
                          m: Optional[int] = None) -> bool:
    """A prompt's q | k | v projection (more than 256 rows, heads of 128) with the per-head norm, the
    rotation and the cache write done in the product's epilogue: q_out bfloat16 [M, nq * 128] receives the
    queries, the keys and values go into their pages.  w is [(nq + 2 nkv) * 128, K], or [nq * 128, K] for
    a layer that only reads a cache (then the cache arguments are unused).  ``cos_sin`` float32
    [M, 64, 2] from rope_table, or None for no rotation.  Returns False when the kernel does not take
    the sizes (run the product and qk_norm_rope_cache instead)."""
    M = x.shape[0] if m is None else m
    N, K = w.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() \
            or x.shape[1] != K:
        raise KernelError("gemm_tcgen05_qkv_rope: x and w must be bfloat16, K-major, with matching K")
    writes = N == (nq + 2 * nkv) * 128
    if M <= 256 or N % 256 or not (writes or N == nq * 128) or K % 8:
        return False
    if q_out.dtype != torch.bfloat16 or q_out.stride(1) != 1 or q_out.shape[1] < nq * 128:
        raise KernelError("gemm_tcgen05_qkv_rope: q_out must be bfloat16 rows of nq * 128 with unit inner stride")
    if writes:
        if k_cache is None or v_cache is None or block_table is None:
            raise KernelError("gemm_tcgen05_qkv_rope: cache tensors missing")
        if k_cache.dtype != torch.bfloat16 or not k_cache.is_contiguous() or tuple(k_cache.shape[1:]) != (nkv, PAGE, 128) \
                or k_cache.shape != v_cache.shape or not v_cache.is_contiguous():
            raise KernelError("gemm_tcgen05_qkv_rope: cache must be bfloat16 [pages, nkv, 64, 128]")
    if (q_norm_w is None) != (k_norm_w is None):
        raise KernelError("gemm_tcgen05_qkv_rope: give both norm weights or neither")
    w_f32 = 0
    if q_norm_w is not None:
        if q_norm_w.dtype != k_norm_w.dtype or q_norm_w.numel() != 128 or k_norm_w.numel() != 128:
            raise KernelError("gemm_tcgen05_qkv_rope: norm weights must share a type and be [128]")
        w_f32 = 1 if q_norm_w.dtype == torch.float32 else 0
    if cos_sin is not None and (cos_sin.dtype != torch.float32 or cos_sin.numel() < M * 128):
        raise KernelError("gemm_tcgen05_qkv_rope: cos_sin must be float32 [M, 64, 2]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_qkv_rope: bias must be float32 [N]")
    rc = _lib().rb_gemm_tcgen05_qkv_rope(
        _ptr(x), _ptr(w), _ptr(bias), M, N, K, x.stride(0), _ptr(q_out), q_out.stride(0), _ptr(k_cache), _ptr(v_cache),
        _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        None if block_table is None else _i32(block_table, "block_table"),
        block_table.shape[1] if block_table is not None else 0, _ptr(q_norm_w), _ptr(k_norm_w), w_f32, float(eps),
        _ptr(cos_sin), nq, nkv, 0, _ptr(status_word(x.device)), _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "gemm_tcgen05_qkv_rope")
    return True



# ---- embedding with a multiplier and sinusoid positions; additions between layers ------------------------------

@_profiled(lambda a, facts: _cost.embedding(a["out"].shape[0], a["out"].shape[1], _esz(a["table"])))
def embedding_pos(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float, positions: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], copy: Optional[torch.Tensor] = None,
                  status: Optional[torch.Tensor] = None):
    """out[t, i] = float32(table[ids[t], i]) * scale + (sin | cos)(positions[t] * inv_freq[i // 2]) for even | odd i
    (nothing is added without ``inv_freq``); ``copy`` receives the same rows."""
    T, H = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or not table.is_contiguous() or table.shape[1] != H:
        raise KernelError("embedding_pos: out must be contiguous float32 [T, H], table contiguous [vocab, H]")
    if copy is not None and (copy.dtype != torch.float32 or not copy.is_contiguous() or copy.shape != out.shape):
        raise KernelError("embedding_pos: copy must look like out")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() < (H + 1) // 2):
        raise KernelError("embedding_pos: inv_freq must be float32 [ceil(H / 2)]")
    rc = _lib().rb_embedding_pos(_i32(ids, "ids"), _ptr(table), dtype_code(table.dtype), _ptr(out), _ptr(copy), T, H,
                                 table.shape[0], float(scale), _i32(positions, "positions"), _ptr(inv_freq),
                                 _ptr(status), _stream())
    _check(rc, "embedding_pos")


@_profiled(lambda a, facts: (a["resid"].numel() * 4 * (2 + (a["delta"].shape[0] if a["delta"] is not None else 0)
                                                       + (1 if a["other"] is not None else 0)), a["resid"].numel() * 3))
def residual_inject(resid: torch.Tensor, delta: Optional[torch.Tensor] = None, other: Optional[torch.Tensor] = None,
                    vec: Optional[torch.Tensor] = None):
    """resid [T, H] float32 += sum of delta [S, T, H] (+ other [T, H] float32) (+ vec [H], every row)."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("residual_inject: resid must be contiguous float32")
    n_delta, stride = 0, 0
    if delta is not None:
        if delta.dtype != torch.float32 or delta.dim() != 3 or tuple(delta.shape[1:]) != (T, H) or \
                not delta[0].is_contiguous():
            raise KernelError("residual_inject: delta must be float32 [S, T, H]")
        n_delta, stride = delta.shape[0], delta.stride(0)
    if other is not None and (other.dtype != torch.float32 or not other.is_contiguous() or other.shape != resid.shape):
        raise KernelError("residual_inject: other must look like resid")
    if vec is not None and (vec.numel() != H or not vec.is_contiguous()):
        raise KernelError("residual_inject: vec must be [H]")
    rc = _lib().rb_residual_inject(_ptr(resid), _ptr(delta), n_delta, stride, _ptr(other), _ptr(vec),
                                   dtype_code(vec.dtype) if vec is not None else F32, T, H, _stream())
    _check(rc, "residual_inject")


@_profiled(lambda a, facts: _cost.add_norm(a["resid"].shape[0], a["resid"].shape[1],
                                           a["top"] if a["row_of"] is not None else a["delta"].shape[0],
                                           _esz(a["out"]) if a["out"] is not None else 0, True, _esz(a["w_post"])))
def postnorm_add_norm(resid: torch.Tensor, delta: torch.Tensor, w_post: torch.Tensor, eps_post: float,
                      w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0, out: Optional[torch.Tensor] = None,
                      row_of: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None, top: int = 0):
    """resid [T, H] float32 += rmsnorm(d) * w_post; with ``w_next`` and ``out`` [T, H]: out = rmsnorm(resid) * w_next
    (the next sublayer's input).  d is the sum of ``delta`` [S, T, H] float32, or, with ``row_of`` (int32 [T, top],
    -1: none) and ``weights`` (float32 [T, top]), row t's weighted sum of the rows ``delta`` [R, H] it names."""
    T, H = resid.shape
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("postnorm_add_norm: resid must be contiguous float32")
    if row_of is not None:
        if delta.dtype != torch.float32 or delta.dim() != 2 or delta.shape[1] != H or delta.stride(1) != 1 or \
                weights is None or weights.dtype != torch.float32 or top < 1 or row_of.numel() < T * top or \
                weights.numel() < T * top or not weights.is_contiguous():
            raise KernelError("postnorm_add_norm: rows to sum must be float32 [R, H] with int32 places and float32 weights [T, top]")
        n_delta, stride = 1, delta.stride(0)
    else:
        if delta.dtype != torch.float32 or delta.dim() != 3 or delta.shape[1] < T or delta.shape[2] != H or \
                delta.stride(2) != 1 or delta.stride(1) != H:
            raise KernelError("postnorm_add_norm: delta must be float32 [S, >= T, H] with dense rows")
        n_delta, stride = delta.shape[0], delta.stride(0)
    if (w_next is None) != (out is None):
        raise KernelError("postnorm_add_norm: give both the next norm's weight and its output or neither")
    if w_post.numel() != H or (w_next is not None and (w_next.numel() != H or w_next.dtype != w_post.dtype)):
        raise KernelError("postnorm_add_norm: the norms' weights must be [H] of one type")
    if out is not None and (not out.is_contiguous() or out.shape[-1] != H or out.numel() < T * H):
        raise KernelError("postnorm_add_norm: out must be contiguous [T, H]")
    rc = _lib().rb_postnorm_add_norm(_ptr(resid), _ptr(delta), n_delta, stride,
                                     None if row_of is None else _i32(row_of, "row_of"), _ptr(weights), int(top),
                                     _ptr(w_post), float(eps_post), _ptr(w_next), float(eps_next), dtype_code(w_post.dtype),
                                     _ptr(out), dtype_code(out.dtype) if out is not None else F32, T, H, _stream())
    _check(rc, "postnorm_add_norm")


GATED_ACTS = {"silu": 0, "clamped_swish": 1, "gelu_tanh": 2}


@_profiled(lambda a, facts: _cost.silu_mul(a["out"].shape[0] if a["rows"] is None else a["rows"], a["out"].shape[1],
                                           _n_in(a["x"]), _esz(a["x"]), _esz(a["out"])))
def gated_act(x: torch.Tensor, out: torch.Tensor, kind: str = "silu", limit: float = 0.0, alpha: float = 1.0,
              rows: Optional[int] = None, paired: bool = False):
    """x [R, 2I] = [gate | up] (or [S, R, 2I] partial sums, added first) -> out [R, I].  ``kind`` "silu":
    silu(gate) * up; "clamped_swish": g = min(gate, limit), u = clamp(up, -limit, limit),
    g * sigmoid(alpha * g) * (u + 1).  ``paired``: gates and ups alternate in blocks of 16 columns."""
    if kind not in GATED_ACTS:
        raise KernelError(f"gated_act: unknown kind {kind!r} (known: {sorted(GATED_ACTS)})")
    n_in, in_stride, row_stride = _partials(x, "gated_act")
    R, I2 = x.shape[-2], x.shape[-1]
    n = R if rows is None else rows
    if I2 % 2 or out.shape[-1] != I2 // 2 or out.stride(-1) != 1 or out.shape[0] < n or n > R:
        raise KernelError("gated_act: shapes do not fit")
    _check(_lib().rb_gated_act(_ptr(x), dtype_code(x.dtype), n_in, in_stride, row_stride, _ptr(out), dtype_code(out.dtype),
                               out.stride(0), n, I2 // 2, GATED_ACTS[kind], float(limit), float(alpha),
                               1 if paired else 0, _stream()),
           "gated_act")


@_profiled(lambda a, facts: (a["x"].numel() * 8, a["x"].numel()))
def scale_(x: torch.Tensor, factor: float):
    """x *= factor in place (contiguous float32)."""
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_: x must be contiguous float32")
    _check(_lib().rb_scale(_ptr(x), x.numel(), float(factor), _stream()), "scale_")


# ---- latent attention: between the projection and the attention ---------------------------------------------------

@_profiled(lambda a, facts: (a["n_tokens"] * (a["proj"].shape[-1] * _esz(a["proj"]) * _n_in(a["proj"])
                                              + (a["q_width"] + a["rank"]) * _esz(a["cache"]) + a["n_gate"] * 4),
                             a["n_tokens"] * (a["rank"] * 6 + a["n_gate"] * 8)))
def latent_prep(proj: torch.Tensor, n_tokens: int, q_width: int, rank: int, n_gate: int, norm_w: torch.Tensor, eps: float,
                q_out: Optional[torch.Tensor], gate_out: Optional[torch.Tensor], cache: torch.Tensor,
                positions: torch.Tensor, slot_of_token: torch.Tensor, block_table: torch.Tensor):
    """proj [T, >= q_width + rank + n_gate] (or [S, T, ...] float32 partial sums) = [queries | latent | gate logits].
    The latent is RMS-normalised (32-bit) with ``norm_w`` and written to each token's place in ``cache``
    [pages, 1, 64, rank]; the queries go to ``q_out`` [T, q_width] in the cache's type when given; sigmoid of the
    gate logits to ``gate_out`` float32 [T, n_gate]."""
    n_in, in_stride, row_stride = _partials(proj, "latent_prep")
    if proj.shape[-1] < q_width + rank + n_gate:
        raise KernelError("latent_prep: projection rows are too narrow")
    if tuple(cache.shape[1:]) != (1, PAGE, rank) or not cache.is_contiguous():
        raise KernelError("latent_prep: cache must be [pages, 1, 64, rank]")
    if norm_w.numel() != rank:
        raise KernelError("latent_prep: the latent norm's weight must be [rank]")
    if q_out is not None and (q_out.dtype != cache.dtype or q_out.stride(-1) != 1 or q_out.shape[-1] < q_width):
        raise KernelError("latent_prep: q_out must hold q_width elements a row in the cache's type")
    if n_gate and (gate_out is None or gate_out.dtype != torch.float32 or not gate_out.is_contiguous()
                   or gate_out.shape[-1] != n_gate):
        raise KernelError("latent_prep: gate_out must be contiguous float32 [T, n_gate]")
    rc = _lib().rb_latent_prep(
        _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, q_width, rank, n_gate, _ptr(norm_w),
        dtype_code(norm_w.dtype), float(eps), _ptr(q_out), q_out.stride(0) if q_out is not None else 0, _ptr(gate_out),
        _ptr(cache), dtype_code(cache.dtype), _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        _i32(block_table, "block_table"), block_table.shape[1], n_tokens, _stream())
    _check(rc, "latent_prep")


# ---- routed experts -----------------------------------------------------------------------------------------------

@_profiled(lambda a, facts: _cost.linear(a["n_tokens"], a["w"].shape[0], a["w"].shape[1], 4, _esz(a["x"]), 4))
def router_logits(x: torch.Tensor, w: torch.Tensor, z: torch.Tensor, n_tokens: int):
    """z [T, E] float32 = x [T, K] . w [E, K]^T with 32-bit FMA; w float32, x bfloat16 or float32."""
    E, K = w.shape
    if w.dtype != torch.float32 or not w.is_contiguous() or z.dtype != torch.float32 or z.stride(1) != 1 or \
            z.shape[1] != E or x.shape[1] != K or x.stride(1) != 1 or x.shape[0] < n_tokens or z.shape[0] < n_tokens:
        raise KernelError("router_logits: w must be contiguous float32 [E, K], z float32 [T, E], x [T, K]")
    _check(_lib().rb_router_logits(_ptr(x), dtype_code(x.dtype), x.stride(0), _ptr(w), _ptr(z), z.stride(0), n_tokens, E, K,
                                   _stream()), "router_logits")


@_profiled(lambda a, facts: (a["n_tokens"] * (a["z"].shape[1] * 4 + a["top"] * 12), a["n_tokens"] * a["z"].shape[1] * 8))
def moe_route(z: torch.Tensor, bias: Optional[torch.Tensor], slot_of_token: torch.Tensor, n_tokens: int, top: int,
              ids: torch.Tensor, weights: torch.Tensor, place: torch.Tensor, counts: torch.Tensor,
              n_groups: int = 1, keep_groups: int = 1, renormalize: bool = False, norm_eps: float = 0.0):
    """z float32 [T, >= E] router logits -> per token the ``top`` experts by sigmoid(z) + bias (``ids`` int32 [T, top],
    -1 for padding tokens), their weights sigmoid(z) (float32 [T, top]) and each choice's place among its expert's
    rows (``place``); ``counts`` int32 [E], zero on entry, ends as the rows of every expert (E is its length; z may
    have more columns).  ``n_groups`` > 1: the experts form equal groups of neighbours, a group's score is the sum of
    its two largest scores, and only experts of the ``keep_groups`` best groups can be chosen.  ``renormalize``: the
    weights are divided by their sum + ``norm_eps``."""
    E = counts.numel()
    if z.shape[1] < E:
        raise KernelError("moe_route: fewer router logits than experts")
    if z.dtype != torch.float32 or z.stride(1) != 1:
        raise KernelError("moe_route: router logits must be float32 with unit inner stride")
    for t, name in ((ids, "ids"), (place, "place")):
        if t.dtype != torch.int32 or not t.is_contiguous() or t.numel() < n_tokens * top:
            raise KernelError(f"moe_route: {name} must be contiguous int32 [T, top]")
    if weights.dtype != torch.float32 or not weights.is_contiguous() or weights.numel() < n_tokens * top:
        raise KernelError("moe_route: weights must be contiguous float32 [T, top]")
    if counts.dtype != torch.int32 or counts.numel() != E or (bias is not None and bias.numel() != E):
        raise KernelError("moe_route: counts (int32) and bias must be [E]")
    rc = _lib().rb_moe_route(_ptr(z), z.stride(0), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
                             _i32(slot_of_token, "slot_of_token"), n_tokens, E, top, _ptr(ids), _ptr(weights),
                             _ptr(place), _ptr(counts), int(n_groups), int(keep_groups), 1 if renormalize else 0,
                             float(norm_eps), _stream())
    _check(rc, "moe_route")


@_profiled(lambda a, facts: ((a["counts"].numel() * 2 + a["tile_group"].numel()) * 4, 0))
def moe_plan(counts: torch.Tensor, tile_rows: int, starts: torch.Tensor, tile_group: torch.Tensor):
    """Every expert's rows start at a multiple of ``tile_rows``: ``starts`` int32 [E + 1]; ``tile_group`` int32
    [max tiles] names each tile's expert (-1: unused)."""
    E = counts.numel()
    if starts.dtype != torch.int32 or starts.numel() != E + 1 or tile_group.dtype != torch.int32:
        raise KernelError("moe_plan: starts must be int32 [E + 1], tile_group int32")
    _check(_lib().rb_moe_plan(_ptr(counts), E, int(tile_rows), tile_group.numel(), _ptr(starts), _ptr(tile_group),
                              _stream()), "moe_plan")


@_profiled(lambda a, facts: (a["n_tokens"] * a["x"].shape[1] * _esz(a["x"]) * (1 + a["top"]), 0))
def moe_gather(x: torch.Tensor, ids: torch.Tensor, place: torch.Tensor, starts: torch.Tensor, n_tokens: int, top: int,
               rows: torch.Tensor, row_of: torch.Tensor):
    """Copy token t's row of ``x`` [T, H] to each of its ``top`` places in ``rows`` [R, H]; ``row_of`` int32 [T, top]
    receives the places (-1 for padding tokens)."""
    if x.dtype != rows.dtype or not x.is_contiguous() or not rows.is_contiguous() or x.shape[1] != rows.shape[1]:
        raise KernelError("moe_gather: x and rows must be contiguous, of one type and width")
    _check(_lib().rb_moe_gather(_ptr(x), dtype_code(x.dtype), x.shape[1], _ptr(ids), _ptr(place), _ptr(starts), n_tokens,
                                top, _ptr(rows), _ptr(row_of), _stream()), "moe_gather")


@_profiled(lambda a, facts: (a["n_tokens"] * a["out"].shape[1] * 4 * (1 + a["top"]), a["n_tokens"] * a["out"].shape[1] * 2 * a["top"]))
def moe_combine(y: torch.Tensor, row_of: torch.Tensor, weights: torch.Tensor, n_tokens: int, top: int, out: torch.Tensor,
                extra: Optional[torch.Tensor] = None, extra_gate: Optional[torch.Tensor] = None):
    """out [T, H] float32 = sum over a token's choices j of weights[t, j] * y[row_of[t, j]] (y float32 [R, H]), plus,
    with ``extra`` (float32 [S, T, H] partial sums), sigmoid(extra_gate[t]) * sum_s extra[s, t] (``extra_gate``: a
    float32 column, one logit a token, any row stride; None: no gate)."""
    if y.dtype != torch.float32 or out.dtype != torch.float32 or y.stride(1) != 1 or not out.is_contiguous() or \
            y.shape[1] != out.shape[1]:
        raise KernelError("moe_combine: y and out must be float32 of one width")
    n_extra = stride = gate_ld = 0
    if extra is not None:
        if extra.dtype != torch.float32 or extra.dim() != 3 or extra.shape[2] != out.shape[1] or extra.shape[1] < n_tokens \
                or extra.stride(2) != 1 or extra.stride(1) != out.shape[1]:
            raise KernelError("moe_combine: extra must be float32 [S, T, H] with dense rows")
        n_extra, stride = extra.shape[0], extra.stride(0)
        if extra_gate is not None:
            if extra_gate.dtype != torch.float32 or extra_gate.dim() != 1 or extra_gate.shape[0] < n_tokens:
                raise KernelError("moe_combine: extra_gate must be a float32 column of T logits")
            gate_ld = extra_gate.stride(0)
    _check(_lib().rb_moe_combine(_ptr(y), y.stride(0), _ptr(row_of), _ptr(weights), n_tokens, top, _ptr(out),
                                 out.shape[1], _ptr(extra), n_extra, stride,
                                 _ptr(extra_gate) if extra is not None else None, gate_ld, _stream()), "moe_combine")


# ---- linear attention with a fixed decay per head ------------------------------------------------------------------

UNIT_ACTS = {"none": 0, "silu": 1, "sigmoid": 2}


@_profiled(lambda a, facts: _cost.decay_scan(a["n_tokens"], a["n_seqs"], a["heads"], a["dim"], a["vdim"], _n_in(a["proj"]),
                                             _esz(a["proj"])))
def decay_scan(proj: torch.Tensor, n_tokens: int, q_off: int, k_off: int, v_off: int, heads: int, dim: int, vdim: int,
               qk_act: str, v_act: str, k_scale: float, decay: torch.Tensor, state: torch.Tensor, seq_slot: torch.Tensor,
               cu_q: torch.Tensor, n_seqs: int, out: torch.Tensor, one_token_each: bool = False):
    """The step's tokens through S = decay[h] * S + k v^T, o = S^T q for every (sequence, head).
    ``one_token_each``: every sequence brings exactly one token (a decode step); the kernel then streams the state
    through registers instead of staging it in shared memory (rounding differs, nothing else).  ``proj`` [T, N] (or
    [S, T, N] float32 partial sums) holds q and k (heads * dim columns from q_off and k_off) and v (heads * vdim from
    v_off); ``qk_act`` / ``v_act``: "none" or "silu"; k is multiplied by ``k_scale``.  ``state`` float32
    [slots, heads, dim, vdim] is read and written in place for the slots of ``seq_slot``; ``out`` float32
    [T, heads * vdim]."""
    n_in, in_stride, row_stride = _partials(proj, "decay_scan")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError("decay_scan: state must be contiguous float32 [slots, heads, dim, vdim]")
    if decay.dtype != torch.float32 or decay.numel() != heads or not decay.is_contiguous():
        raise KernelError("decay_scan: decay must be float32 [heads]")
    if out.dtype != torch.float32 or out.stride(-1) != 1 or out.shape[-1] != heads * vdim or out.shape[0] < n_tokens:
        raise KernelError("decay_scan: out must be float32 [T, heads * vdim]")
    if max(q_off, k_off) + heads * dim > proj.shape[-1] or v_off + heads * vdim > proj.shape[-1]:
        raise KernelError("decay_scan: the projection rows are too narrow")
    fn = _lib().rb_decay_step if one_token_each else _lib().rb_decay_scan
    rc = fn(_ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, q_off, k_off, v_off, heads,
            dim, vdim, UNIT_ACTS[qk_act], UNIT_ACTS[v_act], float(k_scale), _ptr(decay), _ptr(state),
            _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), n_seqs, _ptr(out), out.stride(0), _stream())
    _check(rc, "decay_scan")


DECAY_BLOCK = 64        # tokens a block of decay_scan_blocks
DECAY_BLOCKS_MAX_HEAD = 128


@_profiled(lambda a, facts: _cost.decay_scan(a["n_tokens"], a["n_seqs"], a["heads"], a["dim"], a["vdim"], _n_in(a["proj"]),
                                             _esz(a["proj"])))
def decay_scan_blocks(proj: torch.Tensor, n_tokens: int, q_off: int, k_off: int, v_off: int, heads: int, dim: int, vdim: int,
                      qk_act: str, v_act: str, k_scale: float, decay: torch.Tensor, state: torch.Tensor,
                      seq_slot: torch.Tensor, cu_q: torch.Tensor, n_seqs: int, out: torch.Tensor, work: torch.Tensor) -> bool:
    """``decay_scan`` for prompts: blocks of 64 tokens run side by side (each block's own sum, the states the blocks
    start from along every sequence, each block's outputs).  ``work``: float32 [blocks, heads, dim, vdim] with
    blocks >= n_tokens // 64 + n_seqs.  False, and nothing launched, for head sizes beyond 128."""
    if dim > DECAY_BLOCKS_MAX_HEAD or vdim > DECAY_BLOCKS_MAX_HEAD:
        return False
    n_in, in_stride, row_stride = _partials(proj, "decay_scan_blocks")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError("decay_scan_blocks: state must be contiguous float32 [slots, heads, dim, vdim]")
    if decay.dtype != torch.float32 or decay.numel() != heads or not decay.is_contiguous():
        raise KernelError("decay_scan_blocks: decay must be float32 [heads]")
    if out.dtype != torch.float32 or out.stride(-1) != 1 or out.shape[-1] != heads * vdim or out.shape[0] < n_tokens:
        raise KernelError("decay_scan_blocks: out must be float32 [T, heads * vdim]")
    if max(q_off, k_off) + heads * dim > proj.shape[-1] or v_off + heads * vdim > proj.shape[-1]:
        raise KernelError("decay_scan_blocks: the projection rows are too narrow")
    if work.dtype != torch.float32 or not work.is_contiguous() or tuple(work.shape[1:]) != (heads, dim, vdim) or \
            work.shape[0] < n_tokens // DECAY_BLOCK + n_seqs:
        raise KernelError("decay_scan_blocks: work must be float32 [n_tokens // 64 + n_seqs, heads, dim, vdim]")
    rc = _lib().rb_decay_scan_blocks(_ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, q_off, k_off, v_off,
                                     heads, dim, vdim, UNIT_ACTS[qk_act], UNIT_ACTS[v_act], float(k_scale), _ptr(decay),
                                     _ptr(state), _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), n_seqs, work.shape[0],
                                     _ptr(work), _ptr(out), out.stride(0), _stream())
    _check(rc, "decay_scan_blocks")
    return True


@_profiled(lambda a, facts: (a["n_tokens"] * a["o"].shape[1] * (4 + _esz(a["proj"]) * _n_in(a["proj"]) + _esz(a["out"])),
                             a["n_tokens"] * a["o"].shape[1] * 8))
def group_norm_gate(o: torch.Tensor, proj: torch.Tensor, g_off: int, weight: Optional[torch.Tensor], eps: float, groups: int,
                    gate_act: str, out: torch.Tensor, slot_of_token: torch.Tensor, n_tokens: int):
    """out [T, W] = o / rms(o over each of ``groups`` equal column groups, eps inside the root) (* weight [W]) *
    act(gate), the gate being columns g_off .. g_off + W of ``proj`` (partial sums added first); ``gate_act`` "none",
    "silu" or "sigmoid".  o float32; out in the activations' type."""
    W = o.shape[1]
    n_in, in_stride, row_stride = _partials(proj, "group_norm_gate")
    if o.dtype != torch.float32 or o.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != W or g_off + W > proj.shape[-1]:
        raise KernelError("group_norm_gate: o must be float32 [T, W], out [T, W], the gate inside the projection rows")
    if weight is not None and (weight.numel() != W or not weight.is_contiguous()):
        raise KernelError("group_norm_gate: the weight must be [W]")
    rc = _lib().rb_group_norm_gate(_ptr(o), o.stride(0), _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride,
                                   g_off, _ptr(weight), dtype_code(weight.dtype) if weight is not None else F32, float(eps),
                                   groups, W, UNIT_ACTS[gate_act], _ptr(out), dtype_code(out.dtype), out.stride(0),
                                   _i32(slot_of_token, "slot_of_token"), n_tokens, _stream())
    _check(rc, "group_norm_gate")


@_profiled(lambda a, facts: (a["n_tokens"] * a["heads"] * (a["in_w"] + a["out_w"]) * _esz(a["x"]), a["n_tokens"] * a["heads"] * a["out_w"]))
def head_gate(x: torch.Tensor, out: torch.Tensor, gate: Optional[torch.Tensor], heads: int, in_w: int, out_w: int, n_tokens: int,
              raw: Optional[torch.Tensor] = None, per_value: bool = False):
    """out[t, h, :out_w] = x[t, h, :out_w] * gate: an attention result's heads (``in_w`` wide, of which ``out_w`` are
    values and the rest padding) times a gate formed in 32-bit.  ``gate``: float32 [T, heads] (one a head) or, with
    ``per_value``, [T, heads * out_w] (one a value).  ``raw`` instead: such columns of the projection rows ([T, n] or
    [S, T, n] partial sums, any row stride), of which the kernel takes the sigmoid.  Neither: the heads are only narrowed."""
    if x.dtype != out.dtype or x.stride(-1) != 1 or out.stride(-1) != 1 or x.shape[-1] < heads * in_w or \
            out.shape[-1] < heads * out_w:
        raise KernelError("head_gate: shapes or types do not fit")
    gate_w = out_w if per_value else 1
    if gate is not None and (gate.dtype != torch.float32 or not gate.is_contiguous() or gate.shape[-1] != heads * gate_w):
        raise KernelError("head_gate: gate must be contiguous float32 [T, heads] or [T, heads * out_w]")
    n_in, in_stride, row_stride = 1, 0, 0
    if raw is not None:
        if gate is not None or raw.stride(-1) != 1 or raw.shape[-1] != heads * gate_w:
            raise KernelError("head_gate: raw gate columns must be [.., T, heads (* out_w)] with unit stride, and no finished gate beside them")
        n_in, in_stride, row_stride = (raw.shape[0], raw.stride(0), raw.stride(1)) if raw.dim() == 3 else (1, 0, raw.stride(0))
    _check(_lib().rb_head_gate(_ptr(x), x.stride(0), in_w, _ptr(out), out.stride(0), out_w, _ptr(gate), gate_w, _ptr(raw),
                               dtype_code(raw.dtype) if raw is not None else F32, n_in, in_stride, row_stride, heads,
                               n_tokens, dtype_code(x.dtype), _stream()), "head_gate")


# ---- many small products in one launch ----------------------------------------------------------------------------

@_profiled(lambda a, facts: (a["w"].numel() * _esz(a["w"]) + a["m"] * a["w"].shape[0] * (a["w"].shape[2] * _esz(a["x"])
                                                                                           + a["w"].shape[1] * _esz(a["out"])),
                             2 * a["m"] * a["w"].shape[0] * a["w"].shape[1] * a["w"].shape[2]))
def head_matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, m: int, row_scale: Optional[torch.Tensor] = None,
                x_group_stride: Optional[int] = None, out_group_stride: Optional[int] = None):
    """Per-head products: out[t, g * N : (g + 1) * N] = x[t, g * K : (g + 1) * K] . w[g]^T for w [G, N, K]; rows may be
    strided.  ``row_scale`` float32 [T, G] multiplies head g's result for row t.  ``x_group_stride`` / ``out_group_stride``:
    head g reads from column g * x_group_stride and writes from column g * out_group_stride instead (heads that sit
    in wider rows: only part of each head is read, or the results leave room behind them)."""
    G, N, K = w.shape
    xs = K if x_group_stride is None else int(x_group_stride)
    os_ = N if out_group_stride is None else int(out_group_stride)
    if x.stride(-1) != 1 or out.stride(-1) != 1 or xs < K or os_ < N or x.shape[-1] < (G - 1) * xs + K or \
            out.shape[-1] < (G - 1) * os_ + N or not w.is_contiguous():
        raise KernelError("head_matmul: shapes or strides do not fit")
    if row_scale is not None and (row_scale.dtype != torch.float32 or not row_scale.is_contiguous() or row_scale.shape[-1] != G):
        raise KernelError("head_matmul: row_scale must be contiguous float32 [T, G]")
    rc = _lib().rb_grouped_matmul(_ptr(x), dtype_code(x.dtype), x.stride(0), xs, _ptr(w), dtype_code(w.dtype), N * K,
                                  _ptr(out), dtype_code(out.dtype), out.stride(0), os_, m, N, K, G, None, 0,
                                  _ptr(row_scale), G, 0, 0.0, 1.0, _stream())
    _check(rc, "head_matmul")


def _tile_cost(a, facts):
    """The weights of the groups a step touches (``used``; all of them if not said), the rows in and out; the rows'
    operations (``rows_used`` of them, the buffer's otherwise)."""
    G, N, K = a["w"].shape
    used = G if a.get("used") is None else min(G, a["used"])
    rows = a["x"].shape[0] if a.get("rows_used") is None else a["rows_used"]
    return (int(used * N * K * _esz(a["w"])) + rows * (K * _esz(a["x"]) + a["out"].shape[1] * _esz(a["out"])),
            2 * rows * N * K)


@_profiled(_tile_cost)
def tile_matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, tile_rows: int,
                act: Optional[str] = None, limit: float = 0.0, alpha: float = 1.0, used: Optional[float] = None,
                rows_used: Optional[int] = None) -> bool:
    """Products by tiles of sorted rows: rows i * tile_rows .. of ``x`` [R, K] are multiplied with
    w[tile_group[i]] ([G, N, K]) into the same rows of ``out`` [R, N]; a tile of group -1 is skipped.
    With ``act`` (bfloat16 on the tensor cores only; w's gate and up rows interleaved in blocks of 16) out is
    [R, N / 2], the gated activation of the product (see ``gated_act``); False is returned, and nothing
    launched, when the operands do not take that kernel.  ``used`` (groups that have rows) and ``rows_used`` (rows
    that hold a token) only tell a profiler what the launch had to read and compute."""
    G, N, K = w.shape
    R = x.shape[0]
    if x.stride(1) != 1 or out.stride(1) != 1 or x.shape[1] != K or out.shape[1] != (N // 2 if act else N) or \
            out.shape[0] != R or not w.is_contiguous() or R % tile_rows or tile_group.numel() < R // tile_rows:
        raise KernelError("tile_matmul: shapes or strides do not fit")
    if act is not None and act not in GATED_ACTS:
        raise KernelError(f"tile_matmul: unknown activation {act!r}")
    rc = _lib().rb_grouped_matmul(_ptr(x), dtype_code(x.dtype), x.stride(0), 0, _ptr(w), dtype_code(w.dtype), N * K,
                                  _ptr(out), dtype_code(out.dtype), out.stride(0), 0, R, N, K, G,
                                  _i32(tile_group, "tile_group"), int(tile_rows), None, 0,
                                  0 if act is None else GATED_ACTS[act] + 1, float(limit), float(alpha), _stream())
    if act is not None and rc == 10001:
        return False
    _check(rc, "tile_matmul")
    return True


@_profiled(_tile_cost)
def tile_matmul_tc5(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_group: torch.Tensor, act: Optional[str] = None,
                    limit: float = 0.0, alpha: float = 1.0, used: Optional[float] = None,
                    rows_used: Optional[int] = None) -> bool:
    """``tile_matmul`` for tiles of 128 rows on the tcgen05 tensor cores (the persistent product, each row tile
    taking its group's weight): x bfloat16 [R, K], w bfloat16 [G, N, K], out bfloat16 or float32 [R, N].  With
    ``act`` every group's rows of w alternate in blocks of 16 between gate and up, and out is bfloat16 [R, N / 2]
    = the gated activation (see ``gated_act``).  Returns False when the kernel refuses the sizes or the alignment."""
    G, N, K = w.shape
    R = x.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or not w.is_contiguous() or \
            x.shape[1] != K or out.stride(1) != 1 or out.shape[0] != R or out.shape[1] != (N // 2 if act else N):
        raise KernelError("tile_matmul_tc5: x and w must be bfloat16, K-major, out [R, N] (or [R, N / 2] when gated)")
    if R % 128 or tile_group.numel() < R // 128:
        raise KernelError("tile_matmul_tc5: rows must come in tiles of 128, each with its group")
    if act is not None and act not in GATED_ACTS:
        raise KernelError(f"tile_matmul_tc5: unknown activation {act!r}")
    rc = _lib().rb_gemm_tcgen05_grouped(_ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), R, N, K, G, x.stride(0),
                                        out.stride(0), _i32(tile_group, "tile_group"), 1 if act else 0,
                                        GATED_ACTS.get(act, 0), float(limit), float(alpha), _ptr(status_word(x.device)),
                                        _stream())
    if rc in (10001, 10003):
        return False
    _check(rc, "tile_matmul_tc5")
    return True


# ---- a layer whose norm follows the sum; the blend with the token before ---------------------------------------------

def _f32vec(t: Optional[torch.Tensor], n: int, what: str):
    if t is None:
        return None
    if t.dtype != torch.float32 or not t.is_contiguous() or t.numel() != n:
        raise KernelError(f"{what} must be contiguous float32 with {n} numbers")
    return _ptr(t)


@_profiled(lambda a, facts: (a["resid"].shape[1] * ((a["n_rows"] or a["resid"].shape[0]) * (8 + 4 * _n_partials(a["delta"])
                             + (_esz(a["out"]) if a["out"] is not None else 0)) + 8), 6 * (a["n_rows"] or a["resid"].shape[0]) * a["resid"].shape[1]))
def postln(resid: torch.Tensor, delta: Optional[torch.Tensor], gain: Optional[torch.Tensor], weight: torch.Tensor, alpha: float,
           eps: float, out: Optional[torch.Tensor], slot_of_token: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
           next_mu: Optional[torch.Tensor] = None, next_kept: Optional[torch.Tensor] = None,
           next_out: Optional[torch.Tensor] = None):
    """resid [T, H] float32 <- rmsnorm(alpha * resid + gain * sum_s delta[s]) * weight, in place; ``delta`` float32
    [S, >= T, H] partial sums (or None), ``gain`` and ``weight`` float32 [H]; ``out`` [T, H] also receives the rows in its
    own type.  Rows whose slot is -1 are left alone.  ``next_out`` [T, H] (with ``next_mu`` float32 [H] and ``next_kept``
    float32 [slots, H]; only in a step of one token a sequence): the new row blended with the row its sequence's slot
    kept, row + (kept - row) * mu, as ``token_shift`` would; the slot then keeps the new row."""
    T, H = resid.shape
    n = T if n_rows is None else n_rows
    if resid.dtype != torch.float32 or not resid.is_contiguous():
        raise KernelError("postln: resid must be contiguous float32")
    n_delta, stride = 0, 0
    if delta is not None:
        if delta.dtype != torch.float32 or not delta.is_contiguous() or delta.dim() != 3 or delta.shape[1] < n or delta.shape[2] != H:
            raise KernelError("postln: delta must be contiguous float32 [S, >= T, H]")
        n_delta, stride = delta.shape[0], delta.stride(0)
    if out is not None and (not out.is_contiguous() or out.shape[-1] != H or out.numel() < n * H):
        raise KernelError("postln: out must be contiguous [T, H]")
    if next_out is not None and (next_mu is None or next_kept is None or slot_of_token is None or not next_out.is_contiguous() or
                                 next_out.shape[-1] != H or next_out.numel() < n * H or next_kept.dtype != torch.float32 or
                                 not next_kept.is_contiguous() or next_kept.shape[-1] != H or
                                 (out is not None and out.dtype != next_out.dtype)):
        raise KernelError("postln: next_out [T, H] comes with next_mu [H], next_kept float32 [slots, H] and the rows' slots")
    rc = _lib().rb_postln(_ptr(resid), _ptr(delta), n_delta, stride, _f32vec(gain, H, "postln: gain"),
                          _f32vec(weight, H, "postln: weight"), float(alpha), float(eps), _ptr(out),
                          dtype_code(out.dtype) if out is not None else (dtype_code(next_out.dtype) if next_out is not None else F32),
                          None if slot_of_token is None else _i32(slot_of_token, "slot_of_token"), n, H,
                          _f32vec(next_mu, H, "postln: next_mu") if next_out is not None else None,
                          _ptr(next_kept) if next_out is not None else None, _ptr(next_out), _stream())
    _check(rc, "postln")


@_profiled(lambda a, facts: (a["x"].shape[1] * (a["n_tokens"] * (4 + _esz(a["out"])) + 4 + 8 * a["n_seqs"]), 2 * a["n_tokens"] * a["x"].shape[1]))
def token_shift(x: torch.Tensor, mu: torch.Tensor, kept: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, n_seqs: int,
                max_q_len: int, out: torch.Tensor, n_tokens: int):
    """out[t] = x[t] + (x[t - 1] - x[t]) * mu over each sequence's rows of the step; the row before a sequence's first is
    ``kept[slot]`` (float32 [slots, H]), which then receives the sequence's last row.  x float32 [T, H]."""
    H = x.shape[1]
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous() or out.shape[-1] != H or out.shape[0] < n_tokens:
        raise KernelError("token_shift: x must be contiguous float32 [T, H], out contiguous [T, H]")
    if kept.dtype != torch.float32 or not kept.is_contiguous() or kept.shape[-1] != H:
        raise KernelError("token_shift: kept must be contiguous float32 [slots, H]")
    rc = _lib().rb_token_shift(_ptr(x), _f32vec(mu, H, "token_shift: mu"), _ptr(kept), _i32(seq_slot, "seq_slot"),
                               _i32(cu_q, "cu_q"), n_seqs, max_q_len, _ptr(out), dtype_code(out.dtype), H, _stream())
    _check(rc, "token_shift")


# ---- a state-space mixer ------------------------------------------------------------------------------------------------

CONV_MAX_TAPS = 16


@_profiled(lambda a, facts: (a["n_tokens"] * a["channels"] * (4 + _esz(a["proj"]) * _n_in(a["proj"])) + a["channels"] * 4 * (a["taps"] + 1),
                             2 * a["n_tokens"] * a["channels"] * a["taps"]))
def causal_conv(proj: torch.Tensor, n_tokens: int, col0: int, channels: int, taps: int, weight: torch.Tensor,
                bias: Optional[torch.Tensor], act: str, kept: Optional[torch.Tensor], seq_slot: torch.Tensor, cu_q: torch.Tensor,
                n_seqs: int, max_q_len: int, out: torch.Tensor):
    """out float32 [T, channels] = act(bias + causal convolution with ``taps`` taps) of columns col0 .. col0 + channels of
    ``proj`` ([T, N] or [S, T, N] float32 partial sums).  ``weight`` float32 [channels, taps] (the last tap is the current
    token's); ``kept`` float32 [slots, taps - 1, channels]: the inputs before each sequence's first token of the step, read
    and then replaced by the step's last ones."""
    n_in, in_stride, row_stride = _partials(proj, "causal_conv")
    if taps < 1 or taps > CONV_MAX_TAPS or col0 + channels > proj.shape[-1]:
        raise KernelError(f"causal_conv: 1 to {CONV_MAX_TAPS} taps, and the channels inside the projection rows")
    if weight.dtype != torch.float32 or not weight.is_contiguous() or tuple(weight.shape) != (channels, taps):
        raise KernelError("causal_conv: weight must be contiguous float32 [channels, taps]")
    if taps > 1 and (kept is None or kept.dtype != torch.float32 or not kept.is_contiguous() or tuple(kept.shape[1:]) != (taps - 1, channels)):
        raise KernelError("causal_conv: kept must be contiguous float32 [slots, taps - 1, channels]")
    if out.dtype != torch.float32 or out.stride(-1) != 1 or out.shape[-1] < channels or out.shape[0] < n_tokens:
        raise KernelError("causal_conv: out must be float32 [T, channels]")
    rc = _lib().rb_causal_conv(_ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, col0, channels, taps, _ptr(weight),
                               _f32vec(bias, channels, "causal_conv: bias"), UNIT_ACTS[act], _ptr(kept), _i32(seq_slot, "seq_slot"),
                               _i32(cu_q, "cu_q"), n_seqs, max_q_len, _ptr(out), out.stride(0), _stream())
    _check(rc, "causal_conv")


@_profiled(lambda a, facts: (a["n_tokens"] * 4 * (a["u"].shape[1] + a["heads"] * a["p"]) + 8 * a["n_seqs"] * a["heads"] * a["n"] * a["p"],
                             6 * a["n_tokens"] * a["heads"] * a["n"] * a["p"]))
def ssm_scan(u: torch.Tensor, n_tokens: int, x_off: int, b_off: int, c_off: int, proj: torch.Tensor, dt_off: int,
             dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor, heads: int, groups: int, n: int, p: int,
             state: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, n_seqs: int, out: torch.Tensor,
             one_token_each: bool = False):
    """The step's tokens through S = exp(-exp(a_log[h]) dt) S + dt B x^T, y = S^T C + skip[h] x for every (sequence, head),
    dt = softplus(raw + dt_bias[h]).  ``one_token_each``: every sequence brings exactly one token (a decode step); the kernel
    then streams the state through registers instead of staging it in shared memory (rounding differs, nothing else).  ``u`` float32 [T, >=]: x (heads * p columns from x_off), B and C (groups * n columns
    from b_off and c_off; head h reads group h // (heads / groups)); raw: column dt_off + h of ``proj`` ([T, N] or partial
    sums).  ``state`` float32 [slots, heads, n, p], read and written in place; ``out`` float32 [T, heads * p]."""
    n_in, in_stride, row_stride = _partials(proj, "ssm_scan")
    if u.dtype != torch.float32 or u.stride(-1) != 1 or max(b_off, c_off) + groups * n > u.shape[-1] or x_off + heads * p > u.shape[-1]:
        raise KernelError("ssm_scan: u must be float32 rows that hold x, B and C")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, n, p):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, heads, n, p]")
    if out.dtype != torch.float32 or out.stride(-1) != 1 or out.shape[-1] != heads * p or out.shape[0] < n_tokens:
        raise KernelError("ssm_scan: out must be float32 [T, heads * p]")
    if dt_off + heads > proj.shape[-1] or heads % groups:
        raise KernelError("ssm_scan: the step sizes must lie inside the projection rows, and groups divide heads")
    rc = _lib().rb_ssm_scan(_ptr(u), u.stride(0), x_off, b_off, c_off, _ptr(proj), dtype_code(proj.dtype), n_in, in_stride,
                            row_stride, dt_off, _f32vec(dt_bias, heads, "ssm_scan: dt_bias"), _f32vec(a_log, heads, "ssm_scan: a_log"),
                            _f32vec(skip, heads, "ssm_scan: skip"), heads, groups, n, p, _ptr(state), _i32(seq_slot, "seq_slot"),
                            _i32(cu_q, "cu_q"), n_seqs, 1 if one_token_each else 0, _ptr(out), out.stride(0), _stream())
    _check(rc, "ssm_scan")


SSM_BLOCK = 64        # tokens a block of ssm_scan_blocks


@_profiled(lambda a, facts: (a["n_tokens"] * 4 * (a["u"].shape[1] + a["heads"] * a["p"]) + 8 * a["n_seqs"] * a["heads"] * a["n"] * a["p"],
                             a["n_tokens"] * a["heads"] * (4 * a["n"] * a["p"] + 2 * SSM_BLOCK * (a["n"] + a["p"]))))
def ssm_scan_blocks(u: torch.Tensor, n_tokens: int, x_off: int, b_off: int, c_off: int, proj: torch.Tensor, dt_off: int,
                    dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor, heads: int, groups: int, n: int, p: int,
                    state: torch.Tensor, seq_slot: torch.Tensor, cu_q: torch.Tensor, n_seqs: int, out: torch.Tensor,
                    work: torch.Tensor, block_decay: torch.Tensor, cb: torch.Tensor):
    """``ssm_scan`` for prompts: blocks of 64 tokens run side by side (C . B per block and group, each block's own sum, the
    states the blocks start from along every sequence, each block's outputs).  ``work``: float32 [blocks, heads, n, p],
    ``block_decay``: float32 [blocks, heads], ``cb``: float32 [blocks, groups, 64, 64], blocks >= n_tokens // 64 + n_seqs.  The results differ from ``ssm_scan`` by rounding only."""
    n_in, in_stride, row_stride = _partials(proj, "ssm_scan_blocks")
    if u.dtype != torch.float32 or u.stride(-1) != 1 or max(b_off, c_off) + groups * n > u.shape[-1] or x_off + heads * p > u.shape[-1]:
        raise KernelError("ssm_scan_blocks: u must be float32 rows that hold x, B and C")
    if state.dtype != torch.float32 or not state.is_contiguous() or tuple(state.shape[1:]) != (heads, n, p):
        raise KernelError("ssm_scan_blocks: state must be contiguous float32 [slots, heads, n, p]")
    if out.dtype != torch.float32 or out.stride(-1) != 1 or out.shape[-1] != heads * p or out.shape[0] < n_tokens:
        raise KernelError("ssm_scan_blocks: out must be float32 [T, heads * p]")
    if dt_off + heads > proj.shape[-1] or heads % groups:
        raise KernelError("ssm_scan_blocks: the step sizes must lie inside the projection rows, and groups divide heads")
    blocks = work.shape[0]
    if work.dtype != torch.float32 or not work.is_contiguous() or tuple(work.shape[1:]) != (heads, n, p) or \
            blocks < n_tokens // SSM_BLOCK + n_seqs or block_decay.dtype != torch.float32 or not block_decay.is_contiguous() or \
            tuple(block_decay.shape) != (blocks, heads) or cb.dtype != torch.float32 or not cb.is_contiguous() or \
            tuple(cb.shape) != (blocks, groups, SSM_BLOCK, SSM_BLOCK):
        raise KernelError("ssm_scan_blocks: work must be float32 [n_tokens // 64 + n_seqs, heads, n, p], block_decay [blocks, heads], "
                          "cb [blocks, groups, 64, 64]")
    rc = _lib().rb_ssm_scan_blocks(_ptr(u), u.stride(0), x_off, b_off, c_off, _ptr(proj), dtype_code(proj.dtype), n_in, in_stride,
                                   row_stride, dt_off, _f32vec(dt_bias, heads, "ssm_scan_blocks: dt_bias"),
                                   _f32vec(a_log, heads, "ssm_scan_blocks: a_log"), _f32vec(skip, heads, "ssm_scan_blocks: skip"),
                                   heads, groups, n, p, _ptr(state), _i32(seq_slot, "seq_slot"), _i32(cu_q, "cu_q"), n_seqs, blocks,
                                   _ptr(work), _ptr(block_decay), _ptr(cb), _ptr(out), out.stride(0), _stream())
    _check(rc, "ssm_scan_blocks")


@_profiled(lambda a, facts: (a["n_tokens"] * a["y"].shape[1] * (4 + _esz(a["proj"]) * _n_in(a["proj"]) + _esz(a["out"])),
                             a["n_tokens"] * a["y"].shape[1] * 8))
def gate_group_norm(y: torch.Tensor, proj: torch.Tensor, z_off: int, weight: Optional[torch.Tensor], eps: float, groups: int,
                    gate_act: str, out: torch.Tensor, slot_of_token: torch.Tensor, n_tokens: int):
    """out [T, W] = rmsnorm over each of ``groups`` equal parts of (y * act(z)) (eps inside the root) (* weight float32 [W]):
    the gate first, then the norm.  z: columns z_off .. z_off + W of ``proj`` (partial sums added first).  y float32."""
    W = y.shape[1]
    n_in, in_stride, row_stride = _partials(proj, "gate_group_norm")
    if y.dtype != torch.float32 or y.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != W or z_off + W > proj.shape[-1] or W % groups:
        raise KernelError("gate_group_norm: y must be float32 [T, W], out [T, W], the gate inside the projection rows")
    rc = _lib().rb_gate_group_norm(_ptr(y), y.stride(0), _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, z_off,
                                   _f32vec(weight, W, "gate_group_norm: weight"), float(eps), groups, W, UNIT_ACTS[gate_act],
                                   _ptr(out), dtype_code(out.dtype), out.stride(0), _i32(slot_of_token, "slot_of_token"),
                                   n_tokens, _stream())
    _check(rc, "gate_group_norm")


# ---- latent attention with a query latent and a rotated key part ------------------------------------------------------------

@_profiled(lambda a, facts: (a["n_tokens"] * ((a["q_rank"] + a["rank"] + a["rot"]) * (_esz(a["proj"]) * _n_in(a["proj"]) + _esz(a["cache"]))), 0))
def latent_rot_prep(proj: torch.Tensor, n_tokens: int, q_rank: int, rank: int, rot: int, n_gate: int, q_norm_w: Optional[torch.Tensor],
                    norm_w: torch.Tensor, eps: float, cq_out: Optional[torch.Tensor], gate_out: Optional[torch.Tensor],
                    cache: torch.Tensor, cos_sin: Optional[torch.Tensor], positions: torch.Tensor, slot_of_token: torch.Tensor,
                    block_table: torch.Tensor):
    """proj rows = [query latent (q_rank) | latent (rank) | rotated key part (rot) | gate logits (n_gate)] ([T, N] or partial
    sums).  The query latent, RMS-normalised with ``q_norm_w``, goes to ``cq_out`` [T, q_rank]; the latent, normalised with
    ``norm_w``, then the key part turned by ``cos_sin`` (rotate-half pairs), then zeros go to the token's row of ``cache``
    [pages, 1, 64, dp]; sigmoid of the gate logits to ``gate_out`` float32 [T, n_gate]."""
    n_in, in_stride, row_stride = _partials(proj, "latent_rot_prep")
    dp = cache.shape[-1]
    if proj.shape[-1] < q_rank + rank + rot + n_gate or dp < rank + rot:
        raise KernelError("latent_rot_prep: projection rows or cache rows are too narrow")
    if tuple(cache.shape[1:3]) != (1, PAGE) or not cache.is_contiguous():
        raise KernelError("latent_rot_prep: cache must be [pages, 1, 64, dp]")
    if q_rank and (cq_out is None or cq_out.dtype != cache.dtype or cq_out.stride(-1) != 1 or cq_out.shape[-1] < q_rank):
        raise KernelError("latent_rot_prep: cq_out must hold q_rank elements a row in the cache's type")
    if n_gate and (gate_out is None or gate_out.dtype != torch.float32 or not gate_out.is_contiguous() or gate_out.shape[-1] != n_gate):
        raise KernelError("latent_rot_prep: gate_out must be contiguous float32 [T, n_gate]")
    if rot and (cos_sin is None or cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.numel() < n_tokens * rot):
        raise KernelError("latent_rot_prep: cos_sin must be float32 [T, rot / 2, 2]")
    rc = _lib().rb_latent_rot_prep(
        _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, q_rank, rank, rot, n_gate,
        _f32vec(q_norm_w, q_rank, "latent_rot_prep: q_norm_w") if q_rank else None, _f32vec(norm_w, rank, "latent_rot_prep: norm_w"),
        float(eps), _ptr(cq_out), cq_out.stride(0) if cq_out is not None else 0, _ptr(gate_out), _ptr(cache), dp,
        dtype_code(cache.dtype), _ptr(cos_sin), _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"),
        _i32(block_table, "block_table"), block_table.shape[1], n_tokens, _stream())
    _check(rc, "latent_rot_prep")


@_profiled(lambda a, facts: (a["n_tokens"] * a["heads"] * (a["folded"].shape[-1] // a["heads"] - a["rank"]) * 2 * _esz(a["q"]), 0))
def latent_q_rot(q: torch.Tensor, heads: int, dim: int, rot: int, rank: int, cos_sin: Optional[torch.Tensor], folded: torch.Tensor,
                 slot_of_token: torch.Tensor, n_tokens: int):
    """Head h of ``q`` [T, heads * (dim + rot)] is [dim plain | rot rotated]: the rotated entries, turned by ``cos_sin``
    (rotate-half pairs), go to folded[t, h * dp + rank : + rot] and zeros behind them up to dp = folded.shape[-1] / heads."""
    dp = folded.shape[-1] // heads
    if q.dtype != folded.dtype or q.stride(-1) != 1 or folded.stride(-1) != 1 or q.shape[-1] < heads * (dim + rot) or dp < rank + rot:
        raise KernelError("latent_q_rot: shapes or types do not fit")
    rc = _lib().rb_latent_q_rot(_ptr(q), q.stride(0), heads, dim, rot, rank, dp, _ptr(cos_sin), _ptr(folded), folded.stride(0),
                                dtype_code(q.dtype), _i32(slot_of_token, "slot_of_token"), n_tokens, _stream())
    _check(rc, "latent_q_rot")


# ---- attention with a norm over whole projections and head weights mixed after the softmax -----------------------------------

@_profiled(lambda a, facts: (a["n_tokens"] * ((a["nq"] + a["nkv"]) * a["hd"] + a["nkv"] * a["vd"]) * (_esz(a["proj"]) * _n_in(a["proj"]) + _esz(a["q_out"])), 0))
def wide_norm_rope_cache(proj: torch.Tensor, q_out: torch.Tensor, n_tokens: int, nq: int, nkv: int, hd: int, vd: int, hdp: int,
                         q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float, factor: Optional[torch.Tensor],
                         cos_sin: Optional[torch.Tensor], rot_dim: int, interleaved: bool, positions: torch.Tensor,
                         slot_of_token: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor):
    """proj rows = [q (nq * hd) | k (nkv * hd) | v (nkv * vd)] ([T, N] or partial sums).  q and k are RMS-normalised over their
    whole width with ``q_norm_w`` / ``k_norm_w`` (float32, that wide; None: no norm), the first ``rot_dim`` entries of every
    head turn by ``cos_sin`` (neighbouring pairs when ``interleaved``), query head h is multiplied by ``factor[h]``; q goes to
    ``q_out`` [T, nq * hdp], k and v to their pages [pages, nkv, 64, hdp], heads padded with zeros."""
    n_in, in_stride, row_stride = _partials(proj, "wide_norm_rope_cache")
    if proj.shape[-1] < (nq + nkv) * hd + nkv * vd:
        raise KernelError("wide_norm_rope_cache: projection rows are too narrow")
    if q_out.stride(-1) != 1 or q_out.shape[-1] < nq * hdp or k_cache.dtype != q_out.dtype or v_cache.dtype != q_out.dtype:
        raise KernelError("wide_norm_rope_cache: q_out rows must hold nq * hdp elements of the cache's type")
    if tuple(k_cache.shape[1:]) != (nkv, PAGE, hdp) or k_cache.shape != v_cache.shape or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("wide_norm_rope_cache: caches must be [pages, nkv, 64, hdp]")
    if rot_dim and (cos_sin is None or cos_sin.dtype != torch.float32 or not cos_sin.is_contiguous() or cos_sin.numel() < n_tokens * rot_dim):
        raise KernelError("wide_norm_rope_cache: cos_sin must be float32 [T, rot_dim / 2, 2]")
    rc = _lib().rb_wide_norm_rope_cache(
        _ptr(proj), dtype_code(proj.dtype), n_in, in_stride, row_stride, nq, nkv, hd, vd, hdp,
        _f32vec(q_norm_w, nq * hd, "wide_norm_rope_cache: q_norm_w"), _f32vec(k_norm_w, nkv * hd, "wide_norm_rope_cache: k_norm_w"),
        float(eps), _f32vec(factor, nq, "wide_norm_rope_cache: factor"), _ptr(cos_sin) if rot_dim else None, rot_dim,
        1 if interleaved else 0, _ptr(q_out), q_out.stride(0), _ptr(k_cache), _ptr(v_cache), dtype_code(q_out.dtype),
        _i32(positions, "positions"), _i32(slot_of_token, "slot_of_token"), _i32(block_table, "block_table"),
        block_table.shape[1], n_tokens, _stream())
    _check(rc, "wide_norm_rope_cache")


@_profiled(lambda a, facts: (a["n_tokens"] * a["nq"] * (a["nkv"] * a["hdp"] + a["vd"]) * _esz(a["o"]), 2 * a["n_tokens"] * a["nq"] * a["nq"] * a["vd"]))
def talk_mix(o: torch.Tensor, mix: torch.Tensor, out: torch.Tensor, nq: int, nkv: int, hdp: int, vd: int, slot_of_token: torch.Tensor,
             n_tokens: int):
    """out[t, h, :vd] = sum_g mix[h, g] * o[t, pair(g, m(h)), :vd]: ``o`` [T, nq * nkv * hdp] holds, for every query head g and
    stored value head m, head g's weights applied to m's values (pair (a, m) of key head a at a * nkv + m, its queries in
    order); m(h) is head h's own key/value head; ``mix`` float32 [nq, nq]."""
    if o.dtype != out.dtype or o.stride(-1) != 1 or out.stride(-1) != 1 or o.shape[-1] < nq * nkv * hdp or out.shape[-1] < nq * vd:
        raise KernelError("talk_mix: shapes or types do not fit")
    rc = _lib().rb_talk_mix(_ptr(o), o.stride(0), _f32vec(mix, nq * nq, "talk_mix: mix"), _ptr(out), out.stride(0), nq, nkv, hdp, vd,
                            dtype_code(o.dtype), _i32(slot_of_token, "slot_of_token"), n_tokens, _stream())
    _check(rc, "talk_mix")
