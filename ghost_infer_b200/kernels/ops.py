"""Typed Python wrappers over the kernel library's C entry points.

Each wrapper checks shapes, dtypes, devices and contiguity on the host (the reference validates
token ids, capacity and sizes before any launch: src/model.rs:974-982, src/cuda.rs:8644-8652), then
launches on torch's current stream.  Tensors are torch tensors on a CUDA device; nothing here runs on
the CPU and nothing falls back to library code.
"""
from __future__ import annotations

import contextlib
import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Dict, Optional, Tuple

import torch

from .library import KernelError, last_error, load

F32, BF16 = 0, 1
GEMM_STORE, GEMM_ACCUM_F32 = 0, 1

_DT = {torch.float32: F32, torch.bfloat16: BF16}


class SettleT(ctypes.Structure):
    """gi_settle_t: where a deferred product left its partial sums and how it had cut its work."""
    _fields_ = [("partials", c_void_p), ("tile_first_cta", c_void_p), ("tile_last_cta", c_void_p),
                ("cta_first_tile", c_void_p), ("nt", c_int)]


_bound = None


def _bind():
    global _bound
    if _bound is not None:
        return _bound
    lib = load()
    P, I, L, F = c_void_p, c_int, c_long, c_float
    sigs = {
        "gi_embed": [P, P, I, P, I, I, I, P],
        "gi_rmsnorm": [P, I, P, P, I, P, I, I, F, P],
        "gi_rmsnorm_settle": [P, I, P, P, I, P, I, I, F, SettleT, P],
        "gi_settle": [P, SettleT, P, I, I, P],
        "gi_gemm_stream_geometry": [I, I, I, ctypes.POINTER(c_int), ctypes.POINTER(c_int), ctypes.POINTER(c_int)],
        "gi_silu_mul": [P, P, I, I, I, I, P],
        "gi_gemm_skinny_bf16": [P, I, P, P, I, I, I, L, L, L, P],
        "gi_gemm_generic": [P, I, I, P, I, P, I, I, I, I, L, L, L, P],
        "gi_rope_table": [P, P, P, I, I, P],
        "gi_rope_cache_write": [P, I, L, P, P, P, P, I, P, P, I, I, I, I, I, I, I, P],
        "gi_rope_cache_write_settle": [P, I, L, P, P, P, P, I, P, P, I, I, I, I, I, I, I, SettleT, P],
        "gi_attn_prefill_generic": [P, L, P, L, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_decode_generic": [P, L, P, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, P],
        "gi_gemm_stream_bf16": [P, I, P, P, P, P, I, I, I, I, L, L, L, I, P],
        "gi_gemm_stream_bf16_ex": [P, I, P, P, P, P, I, I, I, I, L, L, L, I, P, I, I, L, I, I, P],
        "gi_gemm_stream_status": [P],
        "gi_gemm_tc_bf16": [P, I, P, P, I, I, I, L, L, L, I, P],
        "gi_gemm_tc_status": [P],
        "gi_attn_prefill_tc": [P, L, P, L, P, P, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_prefill_t5": [P, L, P, L, L, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, P],
        "gi_attn_prefill_t5_status": [P],
        "gi_attn_prefill_t5_ex": [P, L, P, L, L, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, F, P, I, P],
        "gi_attn_prefill_t5_ex2": [P, L, P, L, L, L, P, P, L, P, I, P, P, P, I, I, I, I, I, F, I, F, P, I, I, P],
        "gi_attn_prefill_tc_ex2": [P, L, P, L, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P, I, I, P],
        "gi_attn_decode_tc": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, P],
        "gi_attn_decode_tc_ex": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, P],
        "gi_attn_decode_tc_merged": [P, L, P, P, P, I, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P],
        "gi_attn_decode_tc_rope": [P, L, P, P, P, I, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P, I, SettleT, P],
        "gi_attn_decode_kr": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, I, P],
        "gi_gemm_tc_qkv_rope": [P, P, P, I, I, I, L, L, L, P, P, P, P, I, P, P, I, I, I, I, P],
        "gi_sample": [P, P, L, I, I, F, I, F, P, P, P],
        "gi_embed_scaled": [P, P, I, P, I, I, I, F, P],
        "gi_act_mul": [P, P, I, I, I, I, I, P],
        "gi_attn_prefill_generic_ex": [P, L, P, L, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P, I, P],
        "gi_attn_decode_generic_ex": [P, L, P, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, F, P, I, P],
        "gi_attn_prefill_tc_ex": [P, L, P, L, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P, I, P],
        "gi_attn_decode_kr_ex": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, F, P, I, P],
        "gi_attn_decode_kr_ex2": [P, L, P, P, P, L, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, F, P, I, I, P],
        "gi_kv_store": [P, I, L, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, P],
        "gi_mamba2_conv": [P, P, I, L, P, P, I, P, L, I, P, P, I, I, I, I, I, I, P],
        "gi_mamba2_conv_update": [P, I, L, P, L, I, P, P, I, I, I, I, I, P],
        "gi_mamba2_scan": [P, P, P, I, L, P, P, P, I, P, L, I, P, P, I, I, I, I, I, P],
        "gi_mamba2_gate_norm": [P, I, P, P, I, L, P, I, I, I, I, F, P],
        "gi_moe_route": [P, P, P, P, I, L, P, P, I, I, I, I, I, P],
        "gi_moe_plan": [P, P, P, P, P, I, I, P],
        "gi_moe_gemm_gate_up": [P, I, P, L, P, I, L, P, P, I, I, I, I, I, I, P],
        "gi_moe_gather_rows": [P, P, I, L, P, I, I, I, P],
        "gi_moe_experts_tc": [P, P, P, P, L, P, L, P, I, I, I, P, P, I, P],
        "gi_moe_experts_tc_clamped": [P, P, P, P, L, P, L, P, I, I, I, F, F, P, P, I, P],
        "gi_moe_gemm_down": [P, P, I, L, P, I, L, P, I, I, I, I, P],
        "gi_moe_combine": [P, P, P, P, P, P, I, I, I, P],
        "gi_moe_route_scored": [P, P, P, P, I, L, P, P, I, I, I, I, I, I, P],
        "gi_moe_gemm_rows": [P, P, I, L, P, I, L, P, I, I, I, I, I, P],
        "gi_moe_gather_rows_scaled": [P, P, I, L, P, P, I, I, I, P],
        "gi_attn_prefill_generic_ex2": [P, L, P, L, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P, I, L, P],
        "gi_attn_decode_generic_ex2": [P, L, P, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, F, P, I, L, P],
        "gi_layernorm": [P, I, P, P, I, P, I, I, F, P],
        "gi_layernorm_settle": [P, I, P, P, I, P, I, I, F, SettleT, P],
        "gi_bias_act": [P, P, I, L, P, I, I, I, I, P, P, I, P],
        "gi_latent_prepare": [P, P, I, L, P, P, I, F, P, I, P, P, P, I, P, I, I, I, I, I, P],
        "gi_latent_query_rot": [P, L, P, L, I, P, I, I, I, I, I, I, P],
        "gi_bmm_heads": [P, L, L, P, L, L, I, P, I, L, L, L, I, I, I, I, I, P],
        "gi_rope_table_scaled": [P, P, P, I, I, F, P],
        "gi_attn_latent_tc": [P, L, P, P, P, L, P, P, I, P, P, P, P, I, I, I, I, I, F, I, I, P],
        "gi_gemm_tc_bf16_bias": [P, I, P, P, P, I, I, I, L, L, L, I, P],
        "gi_moe_experts_tc_ungated": [P, P, P, P, L, P, L, P, I, I, I, P, P, I, P],
        "gi_cast_rows": [P, I, P, L, P],
        "gi_postnorm_add": [P, P, P, P, I, I, I, F, P],
        "gi_cast_rows_zero": [P, I, P, P, L, P],
        "gi_postnorm_add_ex": [P, P, P, P, I, I, I, F, P, I, I, P],
        "gi_axpy": [P, P, F, L, P],
        "gi_qk_prepare": [P, L, I, P, L, P, P, P, P, P, I, F, P, I, I, P, P, P, I, P, P, I, I, I, I, I, I, P],
        "gi_gate_mul": [P, P, P, L, I, I, I, I, P],
        "gi_norm_gate": [P, I, P, P, L, P, I, I, I, I, I, I, F, P],
        "gi_side_gate": [P, P, L, I, P, L, I, P, I, I, I, P],
        "gi_act_rows": [P, P, L, I, I, I, P],
        "gi_linear_state": [P, P, L, P, L, P, L, P, L, P, L, I, P, P, P, L, I, P, P, I, I, I, I, I, I, I, F, F, I, I, P],
        "gi_linear_state_gated": [P, P, L, P, L, P, L, P, L, P, L, I, P, P, P, P, P, L, I, P, P, I, I, I, I, I, I, I, F, F, I, I, P],
        "gi_mlstm_gates": [P, P, P, P, L, P, L, P, P, L, I, P, P, F, F, P, L, I, P, P, I, I, I, P],
        "gi_stream_expand": [P, P, I, I, I, P],
        "gi_stream_sum": [P, P, P, I, I, I, P],
        "gi_hyper_read": [P, I, P, P, P, I, P, I, I, I, F, P],
        "gi_hyper_read_conv": [P, I, P, P, P, I, P, I, I, I, F, P, P, I, P, L, I, P, I, P],
        "gi_input_conv": [P, P, I, P, I, P, L, I, P, I, I, I, P],
        "gi_hyper_write": [P, P, P, P, I, I, P, P, P, P, L, I, P, I, I, I, I, P],
        "gi_scale_rows": [P, F, L, P],
        "gi_head_prepare": [P, L, I, P, L, P, P, P, P, P, I, I, I, I, F, P, I, I, P, P, P, I, P, P, I, I, I, I, I, P],
        "gi_head_gate": [P, P, I, P, L, I, I, I, P],
        "gi_scaled_norm_gate": [P, I, P, P, P, L, P, I, I, I, I, F, P],
        "gi_clamped_glu": [P, P, L, I, I, I, F, F, P],
        "gi_clamped_glu_rows": [P, P, L, I, I, I, F, F, I, P],
        "gi_gemm_stream_bf16_clamped": [P, P, P, P, P, I, I, I, I, L, L, L, F, F, P],
        "gi_gemm_tc_bf16_clamped": [P, P, P, I, I, I, L, L, L, I, F, F, P],
        "gi_moe_route_shares": [P, P, P, P, I, L, P, P, I, I, I, I, I, I, P, F, P],
        "gi_moe_gemm_gate_up_clamped": [P, I, P, L, P, I, L, P, P, I, I, I, I, I, I, F, F, P],
        "gi_attn_prefill_generic_ex3": [P, L, P, L, I, P, P, P, I, P, P, P, I, I, I, I, I, F, I, I, F, P, I, L, I, P],
        "gi_attn_decode_generic_ex3": [P, L, P, P, P, L, I, P, P, P, I, P, P, I, I, I, I, F, I, I, I, I, F, P, I, L, I, P],
    }
    for name, argtypes in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.gi_gemm_stream_scratch_floats.restype = c_long
    if os.environ.get("GHOST_INFER_PDL") in ("0", "1"):         # the process-wide default of set_pdl
        lib.gi_set_pdl(int(os.environ["GHOST_INFER_PDL"]))
    _bound = lib
    return lib


launches = 0   # kernels launched through this module since import (benchmarks report the difference)


def _check(lib, rc: int, n: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(last_error(lib) or f"kernel entry point failed with code {rc}")
    launches += n


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor, what: str) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: torch.Tensor, what: str, settles: bool = False) -> None:
    """`settles`: the kernel about to read `t` adds pending partial sums itself; any other kernel must not meet them."""
    if not t.is_cuda:
        raise KernelError(f"{what} must live on a CUDA device; there is no CPU path")
    if not settles and type(t) is Carrier and t.__dict__.get("_gi_pending") is not None:
        raise KernelError(f"{what}: partial sums of a deferred product are pending for this tensor; "
                          f"only a kernel that settles them (or ops.settle) may read it")


def _rows(t: torch.Tensor, what: str) -> int:
    """Leading dimension (in elements) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what} must be 2-D with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _i32(t: Optional[torch.Tensor], what: str):
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{what} must be a contiguous int32 tensor")
    _cuda(t, what)
    return t.data_ptr()


# ---- time per kind of operation ----------------------------------------------------------------------------
# The reference sums wall-clock time into eight named buckets ("embed", "norm+quant", "qkv matmul", "rope+cache",
# "attention", "out matmul", "ffn matmul", "logits"), switched on by GHOST_INFER_PROFILE, synchronising after each
# operation and running without its CUDA graph meanwhile (src/profile.rs:7-46, src/cuda.rs:8054-8063, :9993-9996).
# Here the parts name the bucket of what they launch (`with ops.bucket("attention"):`), and while profiling is on a
# pair of CUDA events brackets each such stretch on the launching stream: device time, no synchronisation inside a
# step.  Steps are then launched kernel by kernel (no graph replay, no dependent launch, which would let one bucket's
# kernels run inside another's stretch).  Off, `bucket` hands out one shared do-nothing context.
BUCKETS = ("embed", "norm", "qkv matmul", "rope+cache", "attention", "conv", "scan", "gated norm", "out matmul", "ffn matmul",
           "router", "experts", "logits", "sampling")


class _NoBucket:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_BUCKET = _NoBucket()
_profile_marks: Optional[list] = None      # (bucket, start event, end event) while profiling
_profile_pdl_was: Optional[bool] = None


class _Bucket:
    __slots__ = ("name", "start")

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.start.record()
        return self

    def __exit__(self, *exc):
        end = torch.cuda.Event(enable_timing=True)
        end.record()
        if _profile_marks is not None:
            _profile_marks.append((self.name, self.start, end))
        return False


def bucket(name: str):
    """A context for the launches of one kind of operation; it costs nothing unless profiling is on."""
    return _NO_BUCKET if _profile_marks is None else _Bucket(name)


def profiling() -> bool:
    return _profile_marks is not None


def profile_start() -> None:
    """From now on the device time of every bucketed stretch is recorded (steps run without graph and dependent launch)."""
    global _profile_marks, _profile_pdl_was
    if _profile_marks is None:
        _profile_pdl_was = get_pdl()
        set_pdl(False)
    _profile_marks = []


def profile_stop() -> Dict[str, float]:
    """Stops recording.  Returns milliseconds of device time per bucket, in the order of BUCKETS (others after)."""
    global _profile_marks, _profile_pdl_was
    marks, _profile_marks = _profile_marks or [], None
    if _profile_pdl_was is not None:
        set_pdl(_profile_pdl_was)
        _profile_pdl_was = None
    torch.cuda.synchronize()
    totals: Dict[str, float] = {}
    for name, a, b in marks:
        totals[name] = totals.get(name, 0.0) + a.elapsed_time(b)
    order = [n for n in BUCKETS if n in totals] + sorted(n for n in totals if n not in BUCKETS)
    return {n: totals[n] for n in order}


# ------------------------------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """x[t] = table[tokens[t]] * scale as float32 rows."""
    lib = _bind()
    _cuda(table, "embedding table")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelError("the embedding table must be a contiguous [vocab, width] matrix")
    n, (vocab, d) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((n, d), dtype=torch.float32, device=table.device)
    _check(lib, lib.gi_embed_scaled(out.data_ptr(), table.data_ptr(), _dt(table, "embedding table"), _i32(tokens, "tokens"),
                                    n, d, vocab, float(scale), _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    lib = _bind()
    _cuda(x, "rmsnorm input", settles=True)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("rmsnorm input must be a contiguous float32 [rows, width] matrix")
    d = x.shape[1]
    if weight.numel() != d or not weight.is_contiguous():
        raise KernelError(f"rmsnorm weight has {weight.numel()} values, the rows are {d} wide")
    n = x.shape[0] if rows is None else rows.numel()
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    pending = _take_pending(x)
    if pending is not None and (pending[1] or d % 4 != 0):
        x.__dict__["_gi_pending"] = pending         # not this kernel's kind of sums: the plain way
        settle(x)
        pending = None
    if pending is not None:
        pending = pending[0]
        # a deferred product left partial sums for this stream: add them while the rows are read anyway (and write
        # the settled rows back; with a selection of rows nothing is written back: the selection may name a row twice,
        # and the stream's other rows stay unsettled, so whoever selects rows must be the stream's last reader)
        _check(lib, lib.gi_rmsnorm_settle(out.data_ptr(), _dt(out, "rmsnorm output"), x.data_ptr(), weight.data_ptr(),
                                          _dt(weight, "rmsnorm weight"), _i32(rows, "rows"), n, d, float(eps), pending,
                                          _stream()))
        return out
    _check(lib, lib.gi_rmsnorm(out.data_ptr(), _dt(out, "rmsnorm output"), x.data_ptr(), weight.data_ptr(),
                               _dt(weight, "rmsnorm weight"), _i32(rows, "rows"), n, d, float(eps), _stream()))
    return out


# ---- deferred accumulation into the residual stream ---------------------------------------------------
# The decode product cuts tiles of W between blocks; adding such a tile's partial sums into the residual
# stream needs an exchange between blocks at the kernel's end.  When the stream's next reader is a norm, which
# reads every row anyway, the product leaves the partial sums in scratch and the norm adds them (in a fixed
# order).  What is pending travels with the tensor itself: only a `Carrier` can have sums pending, the record
# is an attribute of that object (so it dies with it and no other tensor at the same address inherits it),
# any torch operation on it settles first, and a kernel wrapper that does not settle refuses it.
_METADATA = frozenset((
    "get:shape", "get:dtype", "get:device", "get:is_cuda", "get:ndim", "get:layout", "get:requires_grad", "get:is_cpu",
    "get:is_meta", "get:names", "get:grad_fn", "get:is_leaf", "get:_base",
    "data_ptr", "stride", "size", "dim", "numel", "nelement", "element_size", "storage_offset", "is_contiguous",
    "is_floating_point", "is_complex", "get_device", "__len__", "ndimension", "__repr__", "__format__"))


class Carrier(torch.Tensor):
    """A device tensor that a deferred product may leave partial sums for (the residual stream of a step; the
    q/k/v rows on their way to the kernel that rotates and stores).  Shares its storage with the plain tensor
    it was made from.  Reading its sizes, strides and address is free; every other torch operation on it first
    adds what is pending (one kernel launch), so that no reader can see rows without their sums."""

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        name = getattr(func, "__name__", "")
        if name == "__get__":
            name = "get:" + getattr(getattr(func, "__self__", None), "__name__", "")
        if name not in _METADATA:
            for a in args:
                if type(a) is Carrier and a.__dict__.get("_gi_pending") is not None:
                    settle(a)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **(kwargs or {}))


def as_carrier(t: torch.Tensor) -> torch.Tensor:
    """`t` as a tensor that deferred products may leave partial sums for (same storage)."""
    return t if type(t) is Carrier else t.as_subclass(Carrier)


_pending_scratch: Dict[int, torch.Tensor] = {}
_defer_target: Optional[torch.Tensor] = None


def _take_pending(x: torch.Tensor):
    if type(x) is not Carrier:
        return None
    return x.__dict__.pop("_gi_pending", None)


@contextlib.contextmanager
def defer_into(x: torch.Tensor):
    """Inside, a product accumulated into `x` (this very object, a `Carrier`) may leave partial sums pending.
    Whoever reads `x` next settles them: `rmsnorm` while it reads the rows, anything else through `settle`."""
    global _defer_target
    prev = _defer_target
    _defer_target = x if (TUNE["defer_residual"] and type(x) is Carrier and x.is_cuda) else None
    try:
        yield
    finally:
        _defer_target = prev


_defer_store = False


@contextlib.contextmanager
def defer_store():
    """Inside, a decode product that stores bfloat16 rows may leave the tiles cut between blocks as partial sums
    (its result is then a `Carrier`).  `rope_cache_write` adds them while it reads the rows."""
    global _defer_store
    prev = _defer_store
    _defer_store = bool(TUNE["defer_residual"])
    try:
        yield
    finally:
        _defer_store = prev


def has_pending(x: torch.Tensor) -> bool:
    return type(x) is Carrier and x.__dict__.get("_gi_pending") is not None


def settle(x: torch.Tensor) -> None:
    """Adds pending partial sums (if any) to every row of the matrix `x`."""
    pending = _take_pending(x)
    if pending is None:
        return
    lib = _bind()
    rec, store = pending
    if store:
        raise KernelError("partial sums of a stored product are pending: only rope_cache_write settles those")
    _check(lib, lib.gi_settle(x.data_ptr(), rec, None, x.shape[0], x.shape[1], _stream()))


def drop_pending(x: torch.Tensor) -> None:
    """Forgets partial sums pending for `x` (the stream is not read again)."""
    _take_pending(x)


def _defer_ok(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    return (_defer_target is not None and out is _defer_target and out.dtype == torch.float32
            and out.is_contiguous() and out.shape[1] % 4 == 0 and out.shape[1] <= 8192 and out.data_ptr() % 16 == 0
            and not has_pending(out))


def _gemm_stream_deferred(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = 4) -> torch.Tensor:
    lib = _bind()
    key = a.device.index if a.device.index is not None else torch.cuda.current_device()
    if key not in _pending_scratch:
        _pending_scratch[key] = torch.empty(int(lib.gi_gemm_stream_scratch_floats()), dtype=torch.float32, device=a.device)
    scratch = _pending_scratch[key]
    m, k = a.shape
    n = w.shape[0]
    _, counters = _stream_buffers(a.device)
    _check(lib, lib.gi_gemm_stream_bf16_ex(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), scratch.data_ptr(),
                                           counters.data_ptr(), counters.numel(), m, n, k, a.stride(0), w.stride(0),
                                           out.stride(0), -1, *_next_weights(w, mode), _stream()))
    n_ctas, kb, nt = c_int(0), c_int(0), c_int(0)
    lib.gi_gemm_stream_geometry(m, n, k, ctypes.byref(n_ctas), ctypes.byref(kb), ctypes.byref(nt))
    tabs = _settle_tables(a.device, (n + 127) // 128, kb.value, n_ctas.value)
    out.__dict__["_gi_pending"] = (SettleT(scratch.data_ptr(), tabs[0].data_ptr(), tabs[1].data_ptr(), tabs[2].data_ptr(), nt.value),
                                   mode == SKINNY_STORE_DEFER)
    return out


_settle_tabs: Dict[tuple, tuple] = {}


def _settle_tables(device: torch.device, n_tiles: int, kb_per_tile: int, n_ctas: int):
    """Which blocks held pieces of which tile, as the streamed product cuts its work: block c takes the units
    [c * U / G, (c + 1) * U / G) of the U = tiles x K-blocks units.  Built once per shape, kept on the device."""
    key = (str(device), n_tiles, kb_per_tile, n_ctas)
    if key not in _settle_tabs:
        units = n_tiles * kb_per_tile
        starts = [c * units // n_ctas for c in range(n_ctas + 1)]
        import bisect
        cta_of = lambda u: bisect.bisect_right(starts, u) - 1
        first = [cta_of(t * kb_per_tile) for t in range(n_tiles)]
        last = [cta_of((t + 1) * kb_per_tile - 1) for t in range(n_tiles)]
        first_tile = [starts[c] // kb_per_tile for c in range(n_ctas)]
        _settle_tabs[key] = tuple(torch.tensor(v, dtype=torch.int32, device=device) for v in (first, last, first_tile))
    return _settle_tabs[key]


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """silu(gate) * up over rows [gate | up], or, `interleaved`, rows of blocks [8 gate | 8 up]."""
    lib = _bind()
    _cuda(gate_up, "gate/up rows")
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("gate/up rows must be a contiguous [rows, 2 * width] matrix")
    n, f = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((n, f), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib, lib.gi_silu_mul(out.data_ptr(), gate_up.data_ptr(), _dt(gate_up, "gate/up rows"), n, f, int(interleaved),
                                _stream()))
    return out


def gemm_generic(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T with 32-bit accumulation on CUDA cores."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    if out is None:
        if accumulate:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    ldo = _rows(out, "output")
    if out.shape != (m, n):
        raise KernelError(f"matrix product: output is {tuple(out.shape)}, wanted {(m, n)}")
    mode = GEMM_ACCUM_F32 if accumulate else GEMM_STORE
    _check(lib, lib.gi_gemm_generic(out.data_ptr(), _dt(out, "output"), mode, a.data_ptr(), _dt(a, "activations"),
                                    w.data_ptr(), _dt(w, "weights"), m, n, k, lda, ldw, ldo, _stream()))
    return out


SKINNY_STORE_BF16, SKINNY_STORE_F32, SKINNY_ACCUM_F32, SKINNY_SWIGLU, SKINNY_ACCUM_DEFER, SKINNY_STORE_DEFER = 0, 1, 2, 3, 4, 5
ACT_GELU = 0x100        # or-ed into SKINNY_SWIGLU: the gate's activation is gelu (tanh form) instead of silu
SKINNY_MAX_ROWS = 64


def skinny_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the decode product kernel takes these operands: bfloat16, at most 64 rows, 16-byte rows."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and 0 < a.shape[0] <= SKINNY_MAX_ROWS and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T for M <= 64, bfloat16 operands, tensor cores, bound by the bytes of w.
    mode SKINNY_SWIGLU: w's rows are interleaved [8 gate | 8 up] and out is [M, N / 2] = silu(gate) * up."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the decode product kernel takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if (mode & 0xff) == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode & 0xff, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    _check(lib, lib.gi_gemm_skinny_bf16(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, ldo, _stream()))
    return out


# Choices measured on a B200; benchmarks may override them to try alternatives.
TUNE = {"small_skinny": False, "attn_waves": 1.0, "attn_tile_keys": 16, "defer_residual": True, "attn_prefill_tcgen05": True, "prefetch_units": 16,
        "attn_merge_inside": False, "attn_own_slices": False, "attn_stages_hd64": 2, "attn_stages_hd128": 3, "attn_rope_inside": False, "stream_whole_percent": 80,
        "attn_keys_on_rows": True, "attn_kr_warps": 6, "attn_kr_stages": 2, "qkv_rope_epilogue": True, "attn_min_slice": 256,
        "attn_general_tc": True, "bmm_heads_tc": True, "attn_latent_tc": True}
USE_STREAM = True    # decode products through the persistent stream-K kernel (else the mma.sync kernel)


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch: consecutive kernels of a stream that support it overlap one's start with
    the other's end (and the decode product prefetches weights meanwhile).  Process-wide; on unless switched off
    here or by GHOST_INFER_PDL=0 in the environment."""
    lib = _bind()
    lib.gi_set_pdl(int(bool(on)))


def get_pdl() -> bool:
    return bool(_bind().gi_get_pdl())


_STREAM_COUNTERS = 8192
_stream_scratch = {}


def _stream_buffers(device: torch.device):
    """Scratch of the streamed product, one set per device, allocated once (its address is baked into graphs)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _stream_scratch:
        lib = _bind()
        n = int(lib.gi_gemm_stream_scratch_floats())
        _stream_scratch[key] = (torch.empty(n, dtype=torch.float32, device=device),
                                torch.zeros(_STREAM_COUNTERS, dtype=torch.int32, device=device))
    return _stream_scratch[key]


_whole_percent = 80    # what the library was last told (its own default)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None,
                pdl: Optional[bool] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T for M <= 64: persistent, TMA-fed, tcgen05, stream-K balanced; the decode
    step's product.  Modes as gemm_skinny's."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the streamed product takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if (mode & 0xff) == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode & 0xff, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    scratch, counters = _stream_buffers(a.device)
    if (n + 127) // 128 > counters.numel():
        raise KernelError(f"the streamed product takes at most {counters.numel() * 128} rows of weights")
    global _whole_percent
    if _whole_percent != int(TUNE["stream_whole_percent"]):
        _whole_percent = int(TUNE["stream_whole_percent"])
        lib.gi_gemm_stream_whole_tiles(_whole_percent)
    _check(lib, lib.gi_gemm_stream_bf16_ex(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), scratch.data_ptr(),
                                           counters.data_ptr(), counters.numel(), m, n, k, lda, ldw, ldo,
                                           -1 if pdl is None else int(pdl), *_next_weights(w, mode), _stream()))
    return out


# ---- which matrix the next streamed product reads -----------------------------------------------------
# A decode step runs the same products in the same order every time.  Each streamed product remembers which
# matrix followed it the last time and tells its kernel, which asks the L2 cache for that matrix's first units
# while it drains, so the memory does not idle across the kernel boundary.  A wrong guess only costs bandwidth.
_followed_by: Dict[int, tuple] = {}            # weights' address -> (weak reference to the next weights, that product's mode)
_last_streamed: Optional[int] = None


def _next_weights(w: torch.Tensor, mode: int):
    """(pointer, rows, columns, row stride, mode, units ahead) of the product that followed `w`'s last time, or nothing."""
    global _last_streamed
    here = w.data_ptr()
    if _last_streamed is not None and _last_streamed != here:
        if len(_followed_by) > 4096:                     # models come and go: forget the weights that are gone
            for key in [k for k, (ref, _) in _followed_by.items() if ref() is None]:
                del _followed_by[key]
        _followed_by[_last_streamed] = (weakref.ref(w), mode)
    _last_streamed = here
    ref, next_mode = _followed_by.get(here, (None, 0))
    nxt = ref() if ref is not None else None
    ahead = int(TUNE["prefetch_units"])
    if (nxt is None or ahead <= 0 or nxt.dtype != torch.bfloat16 or nxt.dim() != 2 or nxt.stride(1) != 1
            or nxt.device != w.device):
        return None, 0, 0, 0, 0, 0
    return nxt.data_ptr(), nxt.shape[0], nxt.shape[1], nxt.stride(0), next_mode, ahead


_timeline_buf: Optional[torch.Tensor] = None


def stream_timeline_start(slots: int, device="cuda") -> None:
    """From now on each streamed product's blocks note the nanosecond clock at eight places of their life, launch n
    into slot n mod `slots` (a launch captured in a CUDA graph keeps its slot).  For timelines of a decode step."""
    global _timeline_buf
    lib = _bind()
    _timeline_buf = torch.zeros((slots, 256, 8), dtype=torch.int64, device=device)
    lib.gi_gemm_stream_timeline.restype = c_long
    lib.gi_gemm_stream_timeline.argtypes = [c_void_p, c_int]
    lib.gi_gemm_stream_timeline(_timeline_buf.data_ptr(), slots)


def stream_timeline_stop():
    """Stops the stamping.  Returns (stamps [slots, 256 blocks, 8 events] as an int64 array, launches stamped).
    Events: 0 entry, 1 set up, 2 the SM's number, 3 dependency wait over, 4 first stage landed, 5 last load issued,
    6 last product issued, 7 last epilogue done."""
    global _timeline_buf
    lib = _bind()
    lib.gi_gemm_stream_timeline.restype = c_long
    lib.gi_gemm_stream_timeline.argtypes = [c_void_p, c_int]
    n = int(lib.gi_gemm_stream_timeline(None, 0))
    torch.cuda.synchronize()
    out = _timeline_buf.cpu().numpy() if _timeline_buf is not None else None
    _timeline_buf = None
    return out, n


def gemm_stream_status() -> int:
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_gemm_stream_status(ctypes.byref(status)), 0)
    return status.value


def _decode_product(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor]) -> torch.Tensor:
    """The streamed product has a fixed cost of a few microseconds (set-up, and partial sums that cross blocks)
    and then runs at the memory's speed; the register-fed kernel starts faster and streams slower.  Alone, the
    latter wins for at most 8 rows against less than 64 MB of weights; inside a decode step with dependent
    launch the streamed one wins everywhere (it fetches weights while its predecessor drains), so it is the
    default and `TUNE["small_skinny"]` switches the other choice on."""
    small = TUNE["small_skinny"] and a.shape[0] <= 8 and w.shape[0] * w.shape[1] * 2 < (64 << 20)
    if USE_STREAM and not small and (w.shape[0] + 127) // 128 <= _STREAM_COUNTERS:
        if mode == SKINNY_ACCUM_F32:
            if _defer_ok(a, w, out):
                return _gemm_stream_deferred(a, w, out)
            settle(out)          # something is pending for this stream already: add it before adding more
        if mode == SKINNY_STORE_BF16 and _defer_store and out is None and w.shape[0] % 8 == 0:
            out = as_carrier(torch.empty((a.shape[0], w.shape[0]), dtype=torch.bfloat16, device=a.device))
            return _gemm_stream_deferred(a, w, out, SKINNY_STORE_DEFER)
        return gemm_stream(a, w, mode, out)
    return gemm_skinny(a, w, mode, out)


TC_TILE_N = 256     # width of the tensor-core product's output tile (128 or 256)


def tc_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tcgen05 product takes these operands: bfloat16, rows 16 bytes apart, 16-byte aligned."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2 and w.dim() == 2
            and a.shape[0] > 0 and a.shape[1] % 8 == 0 and a.stride(1) == 1 and w.stride(1) == 1
            and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(a: torch.Tensor, w: torch.Tensor, mode: int, out: Optional[torch.Tensor] = None,
            tile_n: Optional[int] = None) -> torch.Tensor:
    """out[M, N] (op)= a[M, K] @ w[N, K]^T on tcgen05 tensor cores with TMA-fed operands; modes as gemm_skinny's."""
    lib = _bind()
    _cuda(a, "activations")
    _cuda(w, "weights")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tensor-core product takes bfloat16 operands")
    lda, ldw = _rows(a, "activations"), _rows(w, "weights")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"matrix product: activations are {k} wide, the weights take {kw}")
    cols = n // 2 if (mode & 0xff) == SKINNY_SWIGLU else n
    want = {SKINNY_STORE_BF16: torch.bfloat16, SKINNY_SWIGLU: torch.bfloat16}.get(mode & 0xff, torch.float32)
    if out is None:
        if mode == SKINNY_ACCUM_F32:
            raise KernelError("matrix product: accumulation needs an output to add to")
        out = torch.empty((m, cols), dtype=want, device=a.device)
    if out.shape != (m, cols) or out.dtype != want:
        raise KernelError(f"matrix product: output is {tuple(out.shape)} {out.dtype}, wanted {(m, cols)} {want}")
    ldo = _rows(out, "output")
    _check(lib, lib.gi_gemm_tc_bf16(out.data_ptr(), mode, a.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, ldo,
                                    int(tile_n or TC_TILE_N), _stream()))
    return out


def qkv_rope_ok(h: torch.Tensor, w: torch.Tensor, memory, head_dim: int, rotary_dim: int) -> bool:
    """Whether the prompt step's q/k/v product can rotate and store in its epilogue (`gemm_tc_qkv_rope`): the
    tensor-core product takes the operands, heads of 64 or 128 values rotated whole, a bfloat16 cache or none to write."""
    if not (TUNE["qkv_rope_epilogue"] and tc_ok(h, w) and h.shape[0] > SKINNY_MAX_ROWS and head_dim in (64, 128)
            and rotary_dim == head_dim):
        return False
    if memory.writes and memory.k is not None:
        return memory.k.dtype == torch.bfloat16 and memory.k.is_contiguous() and memory.v.is_contiguous()
    return True


def gemm_tc_qkv_rope(h: torch.Tensor, w: torch.Tensor, table: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                     block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor], vcache: Optional[torch.Tensor],
                     n_heads: int, n_kv: int, head_dim: int, write_cache: bool) -> torch.Tensor:
    """The packed [q | k | v] rows of a prompt step, h @ w^T, with the rotation by `table` (pairs (i, i + half), the
    whole head) and the cache write in the product's epilogue: the queries' columns of the result are rotated, the
    keys' and values' columns are not written (they went to the cache; with `write_cache` false, nowhere).  The same
    bits as the plain product followed by `rope_cache_write`."""
    lib = _bind()
    _cuda(h, "activations")
    _cuda(w, "weights")
    if h.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("the tensor-core product takes bfloat16 operands")
    lda, ldw = _rows(h, "activations"), _rows(w, "weights")
    m, k = h.shape
    n, kw = w.shape
    if k != kw or n != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v product: activations {tuple(h.shape)}, weights {tuple(w.shape)}, wanted {(n_heads + 2 * n_kv) * head_dim} rows of weights")
    if table.dtype != torch.float32 or not table.is_contiguous() or table.numel() != m * (head_dim // 2) * 2:
        raise KernelError("the table of angles must hold tokens x head_dim / 2 float32 (cos, sin) pairs")
    if write_cache:
        if kcache is None or vcache is None or block_table is None:
            raise KernelError("cache write without a cache")
        if kcache.dtype != torch.bfloat16 or vcache.dtype != torch.bfloat16:
            raise KernelError(f"the cache is {kcache.dtype}, the step runs in bfloat16")
        if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    out = torch.empty((m, n), dtype=torch.bfloat16, device=h.device)
    _check(lib, lib.gi_gemm_tc_qkv_rope(
        out.data_ptr(), h.data_ptr(), w.data_ptr(), m, n, k, lda, ldw, _rows(out, "output"), table.data_ptr(),
        _i32(positions, "positions"), _i32(slots, "slots"), _i32(block_table, "block table"),
        block_table.shape[1] if block_table is not None else 0,
        kcache.data_ptr() if (write_cache and kcache is not None) else None,
        vcache.data_ptr() if (write_cache and vcache is not None) else None,
        n_heads, n_kv, head_dim, int(write_cache), _stream()))
    return out


def gemm_tc_tail_tiles(on: bool) -> None:
    """The tensor-core product cuts the columns of an unfilled last round of blocks into narrower tiles that fit one
    round (on by default); off, every tile has the full width.  Process-wide; for measurements and tests."""
    lib = _bind()
    lib.gi_gemm_tc_tail_tiles(int(bool(on)))


def gemm_tc_status() -> int:
    """0 if every wait inside the tensor-core product was met since the last call; synchronises the device."""
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_gemm_tc_status(ctypes.byref(status)), 0)
    return status.value


def check_status() -> None:
    """Raises if any bounded wait inside the tensor-core kernels ran out since the last call (the kernel then left
    through its normal exit with its work undone: the results of that launch are not to be trusted).  Reads and
    clears the kernels' status words; synchronises the device."""
    bad = []
    for name, fn in (("prompt product", gemm_tc_status), ("decode product", gemm_stream_status),
                     ("prompt attention", attn_prefill_t5_status)):
        code = fn()
        if code:
            bad.append(f"{name} (wait {code})")
    if bad:
        raise KernelError("a wait inside a kernel ran out of tries: " + ", ".join(bad) + "; results since the last check are not to be trusted")


def _tc_out_ok(out: Optional[torch.Tensor], mode: int, cols: int) -> bool:
    """The tensor-core product stores 16 bytes at a time: output rows must start on 16-byte boundaries."""
    align = 8 if mode in (SKINNY_STORE_BF16, SKINNY_SWIGLU) else 4
    if out is None:
        return cols % align == 0
    return out.stride(1) == 1 and out.stride(0) % align == 0 and out.data_ptr() % 16 == 0


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """float32 [tokens, pairs, 2]: (cos, sin) of position * frequency, angles formed in 32-bit, both times `magnitude`."""
    lib = _bind()
    _cuda(positions, "positions")
    if inv_freq.dtype != torch.float32 or not inv_freq.is_contiguous():
        raise KernelError("the rotary frequency table must be contiguous float32")
    n, half = positions.numel(), inv_freq.numel()
    table = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(lib, lib.gi_rope_table_scaled(table.data_ptr(), _i32(positions, "positions"), inv_freq.data_ptr(), n, 2 * half,
                                         float(magnitude), _stream()))
    return table


def rope_cache_write(qkv: torch.Tensor, table: Optional[torch.Tensor], positions: torch.Tensor, slots: torch.Tensor,
                     block_table: Optional[torch.Tensor], kcache: Optional[torch.Tensor],
                     vcache: Optional[torch.Tensor], n_heads: int, n_kv: int, head_dim: int,
                     rotary_dim: int, adjacent: bool, write_cache: bool) -> None:
    """Rotates the q and k parts of the packed rows by the angles of `table` (q in place, k into the cache)
    and copies v into the cache."""
    lib = _bind()
    _cuda(qkv, "q/k/v rows", settles=True)
    ld = _rows(qkv, "q/k/v rows")
    n = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v rows are {qkv.shape[1]} wide, wanted {(n_heads + 2 * n_kv) * head_dim}")
    if rotary_dim:
        if table is None or table.dtype != torch.float32 or table.numel() != n * (rotary_dim // 2) * 2:
            raise KernelError("the table of angles must hold tokens x rotary_dim / 2 float32 (cos, sin) pairs")
    if write_cache:
        if kcache is None or vcache is None or block_table is None:
            raise KernelError("cache write without a cache")
        if kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype:
            raise KernelError(f"the cache is {kcache.dtype}, the step runs in {qkv.dtype}")
        if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    max_pages = block_table.shape[1] if block_table is not None else 0
    args = (qkv.data_ptr(), _dt(qkv, "q/k/v rows"), ld, table.data_ptr() if table is not None else None,
            _i32(positions, "positions"), _i32(slots, "slots"), _i32(block_table, "block table"), max_pages,
            kcache.data_ptr() if kcache is not None else None, vcache.data_ptr() if vcache is not None else None,
            n, n_heads, n_kv, head_dim, rotary_dim, int(adjacent), int(write_cache))
    pending = _take_pending(qkv)
    if pending is not None:       # the product left partial sums instead of some of these rows' values
        if not pending[1]:
            raise KernelError("rope_cache_write met partial sums of an accumulating product")
        _check(lib, lib.gi_rope_cache_write_settle(*args, pending[0], _stream()))
    else:
        _check(lib, lib.gi_rope_cache_write(*args, _stream()))


def attn_prefill_generic(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                         max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                         window: Optional[int], out: torch.Tensor, *, v_dim: Optional[int] = None, softcap: float = 0.0,
                         sinks: Optional[torch.Tensor] = None, chunk: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """`v_dim`: width of a value head when it is not the keys' (`vcache` is then [pages, kv heads, 64, v_dim]);
    `softcap` > 0: scores become cap * tanh(score / cap); `sinks` float32 [heads]: a term exp(sink) in each head's
    softmax denominator without key or value; `chunk`: a query sees keys of its own chunk floor(pos / chunk) only;
    `keep_first`: with a window, the sequence's first so many positions stay visible as well."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if kcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and attention output must share a dtype")
    _check(lib, lib.gi_attn_prefill_generic_ex3(
        out.data_ptr(), ldo, q.data_ptr(), ldq, _dt(q, "queries"), kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), int(v_dim or head_dim), float(softcap or 0.0), _sinks_ptr(sinks, n_heads),
        int(chunk or 0), int(v_dim or head_dim), int(keep_first or 0), _stream()))
    return out


def attn_decode_generic(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                        seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                        head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                        part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                        own_tiles: int = 0, *, v_dim: Optional[int] = None, softcap: float = 0.0,
                        sinks: Optional[torch.Tensor] = None, chunk: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """`v_dim`, `softcap`, `sinks`, `chunk`, `keep_first`: as `attn_prefill_generic`'s.
    `own_tiles` > 0: slice s of a sequence is tiles [s * own_tiles, (s + 1) * own_tiles) of its own span (32 keys a
    tile), whatever `n_splits` is, which must then cover the longest sequence; 0: every span is cut into `n_splits`
    equal slices."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if kcache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and attention output must share a dtype")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * int(v_dim or head_dim):
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    _check(lib, lib.gi_attn_decode_generic_ex3(
        out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
        part_ml.data_ptr() if part_ml is not None else None, q.data_ptr(), ldq, _dt(q, "queries"),
        kcache.data_ptr(), vcache.data_ptr(), _i32(block_table, "block table"), block_table.shape[1],
        _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"), n_seqs, n_heads, n_kv, head_dim, float(scale),
        int(window or 0), int(n_splits), int(own_tiles), int(v_dim or head_dim), float(softcap or 0.0),
        _sinks_ptr(sinks, n_heads), int(chunk or 0), int(v_dim or head_dim), int(keep_first or 0), _stream()), 2 if n_splits > 1 else 1)
    return out


def _sinks_ptr(sinks: Optional[torch.Tensor], n_heads: int):
    if sinks is None:
        return None
    if sinks.dtype != torch.float32 or not sinks.is_contiguous() or sinks.numel() != n_heads:
        raise KernelError(f"attention sinks must be {n_heads} contiguous float32 values, one per head")
    _cuda(sinks, "attention sinks")
    return sinks.data_ptr()


def attn_prefill_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                    max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                    window: Optional[int], out: torch.Tensor) -> torch.Tensor:
    """As attn_prefill_generic, for bfloat16 and head size 64 or 128, on tensor cores."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core prefill attention takes bfloat16 queries, cache and output")
    _check(lib, lib.gi_attn_prefill_tc(
        out.data_ptr(), ldo, q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), _stream()))
    return out


def attn_prefill_t5(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                    max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float,
                    window: Optional[int], out: torch.Tensor, *, softcap: float = 0.0, sinks: Optional[torch.Tensor] = None,
                    chunk: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """As attn_prefill_generic, for bfloat16 and head size 64 or 128 (keys and values alike), on tcgen05 tensor cores with
    TMA-fed operands.  `q` is the whole packed [tokens, (H + 2 KV) * head_dim] matrix (its first columns are the queries), or
    rows of the queries alone.  `softcap`, `sinks`, `chunk`, `keep_first`: as `attn_prefill_generic`'s."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tcgen05 prefill attention takes bfloat16 queries, cache and output")
    if not kcache.is_contiguous() or not vcache.is_contiguous() or q.shape[1] not in ((n_heads + 2 * n_kv) * head_dim, n_heads * head_dim):
        raise KernelError("the tcgen05 prefill attention takes the packed q/k/v rows (or the queries alone) and contiguous cache pages")
    _check(lib, lib.gi_attn_prefill_t5_ex2(
        out.data_ptr(), ldo, q.data_ptr(), ldq, q.shape[0], q.shape[1], kcache.data_ptr(), vcache.data_ptr(), kcache.shape[0],
        _i32(block_table, "block table"), block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"),
        _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"), n_seqs, max_q_len, n_heads, n_kv, head_dim,
        float(scale), int(window or 0), float(softcap or 0.0), _sinks_ptr(sinks, n_heads), int(chunk or 0), int(keep_first or 0),
        _stream()))
    return out


def attn_prefill_t5_pairing(mode: int) -> None:
    """Query tiles two to a block in the tcgen05 prompt attention: 0 never, 1 where the launch then is one round of
    blocks (the default), 2 always.  Process-wide; for measurements and tests."""
    _bind().gi_attn_prefill_t5_pairing(int(mode))


def attn_prefill_t5_status() -> int:
    lib = _bind()
    status = ctypes.c_int(0)
    _check(lib, lib.gi_attn_prefill_t5_status(ctypes.byref(status)), 0)
    return status.value


def attn_decode_tc_ok(q: torch.Tensor, kcache: torch.Tensor, head_dim: int) -> bool:
    """Whether the tensor-core decode attention takes these operands: bfloat16, head size 64 or 128, 16-byte rows."""
    return (q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and head_dim in (64, 128)
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


_ATTN_COUNTERS = 1 << 16
_attn_counters: Dict[int, torch.Tensor] = {}


def _attn_merge_counters(device: torch.device) -> torch.Tensor:
    """Arrival counters of the decode attention's merge, one set per device, allocated once (their address is baked
    into recorded steps) and zero between launches (the kernel leaves them so)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _attn_counters:
        _attn_counters[key] = torch.zeros(_ATTN_COUNTERS, dtype=torch.int32, device=device)
    return _attn_counters[key]


def attn_decode_tc(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                   seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                   head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                   tile_keys: Optional[int] = None, own_tiles: int = 0, merge_inside: Optional[bool] = None,
                   stages: Optional[int] = None, rope: Optional[Tuple[torch.Tensor, int]] = None) -> torch.Tensor:
    """`tile_keys`: 32 (one block per SM, deep rings) or 16 (two blocks per SM); default TUNE["attn_tile_keys"].
    `own_tiles` > 0: slices of that many tiles of each sequence's own span (`n_splits` must then cover the longest
    sequence); 0: every span is cut into `n_splits` equal slices.  `merge_inside`: the slices are merged by the block
    that finishes last instead of by a second kernel (default TUNE["attn_merge_inside"]).
    `rope` = (table of angles [sequences, pairs, 2], rotary size): `q` holds the packed [q | k | v] rows as the
    product left them (partial sums may be pending); the kernel rotates q and k by the table, pairs (i, i + half),
    and stores k and v at each sequence's newest position itself, instead of `rope_cache_write` before it."""
    lib = _bind()
    _cuda(q, "queries", settles=rope is not None)
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core decode attention takes bfloat16 queries, cache and output")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * head_dim:
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    tile_keys = int(tile_keys or TUNE["attn_tile_keys"])
    if own_tiles and n_splits * own_tiles * tile_keys < 1:
        raise KernelError("attention: slices of no keys")
    chunks = (n_heads // max(1, n_kv) + 15) // 16
    inside = TUNE["attn_merge_inside"] if merge_inside is None else merge_inside
    counters = None
    if inside and n_splits > 1 and n_seqs * n_kv * chunks <= _ATTN_COUNTERS:
        counters = _attn_merge_counters(q.device)
    args = (out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
            part_ml.data_ptr() if part_ml is not None else None,
            counters.data_ptr() if counters is not None else None, counters.numel() if counters is not None else 0,
            q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
            _i32(block_table, "block table"), block_table.shape[1], _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"),
            n_seqs, n_heads, n_kv, head_dim, float(scale), int(window or 0), int(n_splits), int(own_tiles),
            tile_keys, int(stages if stages is not None else attn_decode_stages(head_dim)))
    n_launches = 2 if (n_splits > 1 and counters is None) else 1
    if rope is None and counters is None and TUNE["attn_keys_on_rows"] and n_heads // max(1, n_kv) <= 8:
        # the keys of a tile on the rows of the products, up to 8 heads on their columns (a wider group would need
        # two blocks that read the same keys: it keeps the kernel with 16 heads on the rows)
        return attn_decode_kr(q, kcache, vcache, block_table, seq_slots, seq_lens, n_seqs, n_heads, n_kv, head_dim, scale,
                              window, n_splits, out, part_o, part_ml, own_tiles=own_tiles)
    if rope is None:
        _check(lib, lib.gi_attn_decode_tc_merged(*args, _stream()), n_launches)
        return out
    table, rotary_dim = rope
    if q.shape[0] < n_seqs or q.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise KernelError(f"q/k/v rows are {tuple(q.shape)}, wanted {n_seqs} rows of {(n_heads + 2 * n_kv) * head_dim}")
    if table.dtype != torch.float32 or not table.is_contiguous() or table.numel() != q.shape[0] * (rotary_dim // 2) * 2:
        raise KernelError("the table of angles must hold rows x rotary_dim / 2 float32 (cos, sin) pairs")
    if tuple(kcache.shape[1:]) != (n_kv, 64, head_dim) or not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}], got {tuple(kcache.shape)}")
    pending = _take_pending(q)
    if pending is not None and not pending[1]:
        raise KernelError("the decode attention met partial sums of an accumulating product")
    settle_t = pending[0] if pending is not None else SettleT(None, None, None, None, 0)
    _check(lib, lib.gi_attn_decode_tc_rope(*args, table.data_ptr(), int(rotary_dim), settle_t, _stream()), n_launches)
    return out


def sample(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
           rng_state: Optional[torch.Tensor] = None, state_index: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of `logits` (float32).  temperature <= 0: the highest logit, first on ties."""
    lib = _bind()
    _cuda(logits, "logits")
    if logits.dtype != torch.float32:
        raise KernelError("logits must be float32")
    ld = _rows(logits, "logits")
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    if rng_state is not None:
        if rng_state.dtype != torch.int64 or not rng_state.is_contiguous():
            raise KernelError("generator states must be a contiguous int64 tensor")
        _cuda(rng_state, "generator states")
    _check(lib, lib.gi_sample(out.data_ptr(), logits.data_ptr(), ld, n, vocab, float(temperature), int(top_k),
                              float(top_p), rng_state.data_ptr() if rng_state is not None else None,
                              _i32(state_index, "state index"), _stream()))
    return out


# ------------------------------------------------------------------------------------------------
# Dispatchers: the one place where a kernel is chosen for an operation.
def linear(h: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, accumulate: bool = False) -> torch.Tensor:
    want = out.dtype if out is not None else (out_dtype or h.dtype)
    if accumulate and out is not None and not (skinny_ok(h, w) and USE_STREAM):
        settle(out)
    mode = SKINNY_ACCUM_F32 if accumulate else {torch.bfloat16: SKINNY_STORE_BF16, torch.float32: SKINNY_STORE_F32}.get(want)
    if mode is not None:
        if skinny_ok(h, w):
            return _decode_product(h, w, mode, out)
        if tc_ok(h, w) and _tc_out_ok(out, mode, w.shape[0]):
            return gemm_tc(h, w, mode, out)
    return gemm_generic(h, w, out=out, out_dtype=out_dtype, accumulate=accumulate)


def swiglu_interleaved(h: torch.Tensor, w_interleaved: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """act(Wgate h) * (Wup h) where `w_interleaved` holds gate and up rows in blocks [8 gate | 8 up]; `act` "silu" or
    "gelu_tanh" (in the products' epilogues, or as a step of its own where no such product takes the operands)."""
    mode = SKINNY_SWIGLU | (ACT_GELU if act == "gelu_tanh" else 0)
    if act not in ("silu", "gelu_tanh"):
        raise KernelError(f"unknown activation \"{act}\" (silu, gelu_tanh)")
    if skinny_ok(h, w_interleaved) and USE_STREAM and (w_interleaved.shape[0] + 127) // 128 <= _STREAM_COUNTERS and not (
            TUNE["small_skinny"] and act != "silu"):
        return _decode_product(h, w_interleaved, mode, None)
    if tc_ok(h, w_interleaved) and w_interleaved.shape[0] % 16 == 0 and h.shape[0] > SKINNY_MAX_ROWS:
        return gemm_tc(h, w_interleaved, mode)
    gu = linear(h, w_interleaved, out_dtype=h.dtype)
    return act_mul(gu, act, interleaved=True)


def attn_decode_stages(head_dim: int) -> int:
    """Depth of each warp's ring of key/value tiles in the tensor-core decode attention."""
    return int(TUNE["attn_stages_hd64"] if head_dim == 64 else TUNE["attn_stages_hd128"])


def attn_decode_blocks_per_sm(head_dim: int, fast: bool) -> float:
    """How many blocks of the decode attention one SM holds (its shared memory decides: a block's rings of key and
    value tiles are 96 KB at head size 128 and 64 KB at head size 64 with 16-key tiles), times TUNE["attn_waves"]:
    the slice count fills that many places once."""
    if not fast:
        per_sm = 2
    elif TUNE["attn_keys_on_rows"]:
        # the kernel with a tile's keys on the rows of its products: 8 rows of queries, and each warp's ring of
        # `stages` x (16 keys + 16 values); 80 registers a thread at head size 64, up to 127 at 128
        warps, stages = int(TUNE["attn_kr_warps"]), int(TUNE["attn_kr_stages"])
        smem = 8 * head_dim * 2 + warps * stages * 2 * 16 * head_dim * 2 + 1152
        regs = 65536 // (warps * 32 * (80 if head_dim == 64 else 128))
        per_sm = max(1, min(regs, (227 * 1024) // smem))
    elif TUNE["attn_tile_keys"] == 16:
        # a block's shared memory: 16 rows of queries, and four warps' rings of `stages` x (16 keys + 16 values)
        smem = 16 * head_dim * 2 + 4 * attn_decode_stages(head_dim) * 2 * 16 * head_dim * 2 + 1152
        regs = 4 if head_dim == 64 else 3          # blocks per SM that the registers allow (121 and 168 a thread)
        per_sm = min(regs, (227 * 1024) // smem)
    else:
        per_sm = 1
    return per_sm * TUNE["attn_waves"]


OWN_LENGTH_TILES = 8      # 32-bit decode attention: a slice is this many 32-key tiles of the sequence's own span


def attn_decode_plan(n_seqs: int, max_kv_len: int, sm_count: int, n_heads: int, n_kv: int, head_dim: int,
                     window: Optional[int], dtype: torch.dtype, kv_lens=None):
    """How the decode attention cuts contexts into slices, as (slices in the launch, tiles per slice).

    bfloat16, few sequences: tiles per slice 0 = every sequence is cut into the same number of slices, as many as
    fill the GPU once (blocks that wait for a second round cost more than longer slices), at least 256 positions of the
    longest sequence's present length each (measured at batch 1 to 4 of the 8B shape with 2,048 cached positions: 8
    slices beat 16 and 4, and 32, which the length bucket's upper end alone would allow, cost 3.5 % of the step).
    bfloat16, so many sequences that one slice each fills more than half the GPU, and their lengths (`kv_lens`) known:
    slices of a fixed number of tiles of each sequence's own span, the shortest for which all blocks still find a
    place at once; long sequences are then cut and short ones are not, so that no block is much longer than the rest.
    float32: slices of a fixed length counted from the start of the sequence's own span, so that a sequence's
    sums are formed in the same order whatever else the step holds (the reference sizes its slices from the
    token's own span for the same reason, src/cuda.rs:1639-1644, :8432-8437); the launch holds as many slices as
    the longest sequence needs, and shorter ones leave theirs empty."""
    if dtype == torch.float32:
        span = max_kv_len if not window else min(max_kv_len, int(window) + 31)
        tiles = (span + 31) // 32 + (1 if window else 0)
        return max(1, (tiles + OWN_LENGTH_TILES - 1) // OWN_LENGTH_TILES), OWN_LENGTH_TILES
    fast = dtype == torch.bfloat16 and head_dim in (64, 128)
    # heads of a group that one block takes: 16 in the tensor-core kernels (groups of more than 8 heads go to the one
    # that has the heads on the rows of its tile), 8 in the plain kernel
    rows_per_block = 16 if fast else 8
    group = n_heads // n_kv
    chunks = (group + rows_per_block - 1) // rows_per_block
    blocks = max(1, n_seqs * n_kv * chunks)
    places = int(attn_decode_blocks_per_sm(head_dim, fast) * sm_count)
    if 2 * blocks <= places or not fast:
        # slices of at least TUNE["attn_min_slice"] positions of the longest sequence as it is now (a plan is kept while
        # the sequences grow to the end of their length bucket, up to twice as long)
        longest = max_kv_len if not kv_lens else min(max_kv_len, max(int(n) for n in kv_lens))
        return int(max(1, min(places // blocks, 32, longest // int(TUNE["attn_min_slice"])))), 0
    if kv_lens is not None and TUNE["attn_own_slices"] and blocks < places:
        tile = int(TUNE["attn_tile_keys"])
        span = (lambda n: n) if not window else (lambda n: min(n, int(window) + 2 * tile))
        # the lengths a little ahead of now: the plan is kept while the sequences grow
        lens = [span(min(int(n) + 64, max_kv_len)) for n in kv_lens]
        idle = max(0, n_seqs - len(lens))                    # padding rows: one tile each
        longest = span(max_kv_len)
        unit = max(1, 256 // tile)
        own = unit
        while own * tile < longest:
            need = (sum((n + own * tile - 1) // (own * tile) for n in lens) + idle) * n_kv * chunks
            if need <= places:
                return max(1, (longest + own * tile - 1) // (own * tile)), own
            own += unit
    return 1, 0


def attn_decode_kr(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                   seq_slots: torch.Tensor, seq_lens: torch.Tensor, n_seqs: int, n_heads: int, n_kv: int,
                   head_dim: int, scale: float, window: Optional[int], n_splits: int, out: torch.Tensor,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None, own_tiles: int = 0,
                   warps: Optional[int] = None, stages: Optional[int] = None) -> torch.Tensor:
    """The tensor-core decode attention with a tile's 16 keys on the rows of its products and up to 8 heads of a group on
    their columns (wider groups take several blocks per kv head).  Same operands and scratch as `attn_decode_tc`;
    `warps` per block (4, 6 or 8) and `stages` of each warp's ring (2 or 3) default to TUNE's."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core decode attention takes bfloat16 queries, cache and output")
    if n_splits > 1:
        if part_o is None or part_ml is None:
            raise KernelError("attention slices need scratch memory")
        if part_o.dtype != torch.float32 or part_o.numel() < n_seqs * n_heads * n_splits * head_dim:
            raise KernelError("attention scratch for outputs is too small")
        if part_ml.dtype != torch.float32 or part_ml.numel() < n_seqs * n_heads * n_splits * 2:
            raise KernelError("attention scratch for maxima and sums is too small")
    _check(lib, lib.gi_attn_decode_kr(
        out.data_ptr(), ldo, part_o.data_ptr() if part_o is not None else None,
        part_ml.data_ptr() if part_ml is not None else None, q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(),
        _i32(block_table, "block table"), block_table.shape[1], _i32(seq_slots, "slots"), _i32(seq_lens, "lengths"),
        n_seqs, n_heads, n_kv, head_dim, float(scale), int(window or 0), int(n_splits), int(own_tiles),
        int(warps or TUNE["attn_kr_warps"]), int(stages or TUNE["attn_kr_stages"]), _stream()), 2 if n_splits > 1 else 1)
    return out


def attn_rope_inside_ok(qkv: torch.Tensor, memory, step, head_dim: int) -> bool:
    """Whether a step's rotation and cache write can be left to its attention kernel (`attention(..., rope=)`): a
    decode step on the tensor-core kernel that writes its own cache."""
    return bool(TUNE["attn_rope_inside"] and step.is_decode and memory.k is not None and memory.writes
                and attn_decode_tc_ok(qkv, memory.k, head_dim) and qkv.shape[0] == step.n_seqs)


def attention(qkv: torch.Tensor, memory, step, n_heads: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int], out: torch.Tensor, plan=None, rope=None) -> torch.Tensor:
    """Attention of a step's tokens over the cache (which already holds the step's own keys and values).
    The queries are the first n_heads * head_dim columns of the packed rows `qkv`.  `plan`: what
    `attn_decode_plan` gave for a decode step (worked out here when absent).  `rope` = (table, rotary size), only
    where `attn_rope_inside_ok` holds: the rows are not rotated and the cache lacks the step's keys and values;
    the kernel does both."""
    if memory.k is None:
        raise KernelError("attention needs a cache to read from")
    if rope is not None and not attn_rope_inside_ok(qkv, memory, step, head_dim):
        raise KernelError("this step's attention cannot rotate and store by itself")
    if step.is_decode:
        fast = attn_decode_tc_ok(qkv, memory.k, head_dim)
        if plan is None:
            plan = attn_decode_plan(step.n_seqs, step.max_kv_len, step.sm_count, n_heads, n_kv, head_dim, window, qkv.dtype)
        n_splits, own_tiles = plan
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty((step.n_seqs * n_heads * n_splits * head_dim,), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((step.n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
        if fast:
            return attn_decode_tc(qkv, memory.k, memory.v, memory.block_table, step.seq_slots, step.seq_lens,
                                  step.n_seqs, n_heads, n_kv, head_dim, scale, window, n_splits, out, part_o, part_ml,
                                  own_tiles=own_tiles, rope=rope)
        return attn_decode_generic(qkv, memory.k, memory.v, memory.block_table, step.seq_slots, step.seq_lens,
                                   step.n_seqs, n_heads, n_kv, head_dim, scale, window, n_splits, out, part_o, part_ml,
                                   own_tiles=own_tiles)
    if attn_decode_tc_ok(qkv, memory.k, head_dim) and out.stride(0) % 2 == 0:
        # tcgen05 (scores and output in tensor memory); mma.sync when that is switched off or the rows do not suit TMA
        t5 = (TUNE["attn_prefill_tcgen05"] and head_dim in (64, 128) and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
              and qkv.shape[1] == (n_heads + 2 * n_kv) * head_dim and memory.k.is_contiguous())
        kernel = attn_prefill_t5 if t5 else attn_prefill_tc
    else:
        kernel = attn_prefill_generic
    return kernel(qkv, memory.k, memory.v, memory.block_table, step.cu_seqlens, step.seq_slots,
                  step.seq_pos0, step.n_seqs, step.max_q_len, n_heads, n_kv, head_dim, scale, window, out)


# ------------------------------------------------------------------------------------------------
# Attention without rotation whose values may be blended with another layer's and have a width of their own.
def kv_store(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, memory, n_heads: int, n_kv: int,
             head_dim: int, v_dim: int, first: Optional[torch.Tensor] = None, blend: Optional[torch.Tensor] = None,
             copy_to: Optional[torch.Tensor] = None) -> None:
    """Keys and values of packed rows [q | k | v] into `memory`'s pages, unrotated.  `first` [tokens, kv heads * v_dim]
    and `blend` (one float32 on the device): the values become (1 - blend) v + blend first beforehand (also in the rows);
    `copy_to`: receives the rows' own values."""
    lib = _bind()
    _cuda(qkv, "q/k/v rows")
    ld = _rows(qkv, "q/k/v rows")
    n = qkv.shape[0]
    vw = n_kv * v_dim
    if qkv.shape[1] != (n_heads + n_kv) * head_dim + vw:
        raise KernelError(f"q/k/v rows are {qkv.shape[1]} wide, wanted {(n_heads + n_kv) * head_dim + vw}")
    for t, what in ((first, "the first layer's values"), (copy_to, "the copy of the values")):
        if t is not None and (t.dtype != qkv.dtype or tuple(t.shape) != (n, vw) or not t.is_contiguous()):
            raise KernelError(f"{what} must be contiguous [{n}, {vw}] {qkv.dtype}")
    if first is not None and (blend is None or blend.dtype != torch.float32 or blend.numel() != 1 or not blend.is_cuda):
        raise KernelError("blending values needs its weight as one float32 on the device")
    write = bool(memory.writes and memory.k is not None)
    if write:
        if memory.k.dtype != qkv.dtype or memory.v.dtype != qkv.dtype:
            raise KernelError(f"the cache is {memory.k.dtype}, the step runs in {qkv.dtype}")
        if (tuple(memory.k.shape[1:]) != (n_kv, 64, head_dim) or tuple(memory.v.shape[1:]) != (n_kv, 64, v_dim)
                or not memory.k.is_contiguous() or not memory.v.is_contiguous()):
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}] and [.., {v_dim}], got "
                              f"{tuple(memory.k.shape)} and {tuple(memory.v.shape)}")
    bt = memory.block_table
    _check(lib, lib.gi_kv_store(
        qkv.data_ptr(), _dt(qkv, "q/k/v rows"), ld, first.data_ptr() if first is not None else None,
        blend.data_ptr() if first is not None else None, copy_to.data_ptr() if copy_to is not None else None,
        _i32(positions, "positions"), _i32(slots, "slots"), _i32(bt, "block table"), bt.shape[1] if bt is not None else 0,
        memory.k.data_ptr() if write else None, memory.v.data_ptr() if write else None, n, n_heads, n_kv, head_dim, v_dim,
        int(write), _stream()))


def attention_general(qkv: torch.Tensor, memory, step, n_heads: int, n_kv: int, head_dim: int, v_dim: int, scale: float,
                      out: torch.Tensor, *, window: Optional[int] = None, chunk: Optional[int] = None, softcap: float = 0.0,
                      sinks: Optional[torch.Tensor] = None, plan=None, keep_first: int = 0) -> torch.Tensor:
    """Attention of a step's tokens over the cache with any of: values of another width than the keys, capped scores,
    a sink per head, chunks of positions, a window (which may keep the first `keep_first` positions visible as well).
    The cache already holds the step's own keys and values."""
    if memory.k is None:
        raise KernelError("attention needs a cache to read from")
    keep_first = int(keep_first or 0) if window else 0
    opts = dict(v_dim=v_dim, softcap=softcap, sinks=sinks, chunk=chunk)
    if keep_first:
        opts["keep_first"] = keep_first
    if step.is_decode:
        if plan is None:
            plan = attn_general_decode_plan(step.n_seqs, step.max_kv_len, step.sm_count, n_heads, n_kv, window, chunk, qkv.dtype,
                                            head_dim, v_dim, keep_first=keep_first)
        kind, n_splits, own_tiles = plan
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty((step.n_seqs * n_heads * n_splits * v_dim,), dtype=torch.float32, device=qkv.device)
            part_ml = torch.empty((step.n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qkv.device)
        if kind == "tensor cores":
            lib = _bind()
            _cuda(qkv, "queries")
            if qkv.dtype != torch.bfloat16 or memory.k.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
                raise KernelError("the tensor-core decode attention takes bfloat16 queries, cache and output")
            _check(lib, lib.gi_attn_decode_kr_ex2(
                out.data_ptr(), _rows(out, "attention output"), part_o.data_ptr() if part_o is not None else None,
                part_ml.data_ptr() if part_ml is not None else None, qkv.data_ptr(), _rows(qkv, "queries"), memory.k.data_ptr(),
                memory.v.data_ptr(), _i32(memory.block_table, "block table"), memory.block_table.shape[1],
                _i32(step.seq_slots, "slots"), _i32(step.seq_lens, "lengths"), step.n_seqs, n_heads, n_kv, head_dim, float(scale),
                int(window or 0), int(n_splits), int(own_tiles), v_dim, float(softcap or 0.0), _sinks_ptr(sinks, n_heads),
                int(chunk or 0), keep_first, _stream()), 2 if n_splits > 1 else 1)
            return out
        return attn_decode_generic(qkv, memory.k, memory.v, memory.block_table, step.seq_slots, step.seq_lens, step.n_seqs,
                                   n_heads, n_kv, head_dim, scale, window, n_splits, out, part_o, part_ml, own_tiles=own_tiles,
                                   **opts)
    if (TUNE["attn_general_tc"] and TUNE["attn_prefill_tcgen05"] and qkv.dtype == torch.bfloat16 and memory.k.dtype == torch.bfloat16
            and head_dim == v_dim and head_dim in (64, 128) and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0
            and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0
            and qkv.shape[1] in ((n_heads + 2 * n_kv) * head_dim, n_heads * head_dim)
            and memory.k.is_contiguous() and memory.v.is_contiguous()):
        # keys and values of one of the two sizes the tcgen05 kernel takes: scores and output in tensor memory
        return attn_prefill_t5(qkv, memory.k, memory.v, memory.block_table, step.cu_seqlens, step.seq_slots, step.seq_pos0,
                               step.n_seqs, step.max_q_len, n_heads, n_kv, head_dim, scale, window, out, softcap=softcap,
                               sinks=sinks, chunk=chunk, keep_first=keep_first)
    if (TUNE["attn_general_tc"] and qkv.dtype == torch.bfloat16 and memory.k.dtype == torch.bfloat16 and head_dim % 8 == 0
            and v_dim % 8 == 0 and head_dim <= 128 and v_dim <= 128 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0
            and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
        return attn_prefill_tc_general(qkv, memory.k, memory.v, memory.block_table, step.cu_seqlens, step.seq_slots,
                                       step.seq_pos0, step.n_seqs, step.max_q_len, n_heads, n_kv, head_dim, scale, window, out,
                                       **opts)
    return attn_prefill_generic(qkv, memory.k, memory.v, memory.block_table, step.cu_seqlens, step.seq_slots, step.seq_pos0,
                                step.n_seqs, step.max_q_len, n_heads, n_kv, head_dim, scale, window, out, **opts)


def attn_prefill_tc_general(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                            cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, seq_pos0: torch.Tensor, n_seqs: int,
                            max_q_len: int, n_heads: int, n_kv: int, head_dim: int, scale: float, window: Optional[int],
                            out: torch.Tensor, *, v_dim: Optional[int] = None, softcap: float = 0.0,
                            sinks: Optional[torch.Tensor] = None, chunk: Optional[int] = None, keep_first: int = 0) -> torch.Tensor:
    """`attn_prefill_generic` with its options on tensor cores: bfloat16, key and value sizes multiples of 8 up to 128."""
    lib = _bind()
    _cuda(q, "queries")
    ldq, ldo = _rows(q, "queries"), _rows(out, "attention output")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("the tensor-core prefill attention takes bfloat16 queries, cache and output")
    if not kcache.is_contiguous() or not vcache.is_contiguous():
        raise KernelError("the tensor-core prefill attention takes contiguous cache pages")
    _check(lib, lib.gi_attn_prefill_tc_ex2(
        out.data_ptr(), ldo, q.data_ptr(), ldq, kcache.data_ptr(), vcache.data_ptr(), _i32(block_table, "block table"),
        block_table.shape[1], _i32(cu_seqlens, "cu_seqlens"), _i32(seq_slots, "slots"), _i32(seq_pos0, "start positions"),
        n_seqs, max_q_len, n_heads, n_kv, head_dim, float(scale), int(window or 0), int(v_dim or head_dim),
        float(softcap or 0.0), _sinks_ptr(sinks, n_heads), int(chunk or 0), int(keep_first or 0), _stream()))
    return out


def attn_general_tc_ok(dtype: torch.dtype, head_dim: int, v_dim: int) -> bool:
    """Whether `attention_general` has tensor-core kernels for these sizes: bfloat16, multiples of 8 up to 128."""
    return bool(TUNE["attn_general_tc"] and dtype == torch.bfloat16 and head_dim % 8 == 0 and v_dim % 8 == 0
                and 0 < head_dim <= 128 and 0 < v_dim <= 128)


def attn_general_decode_plan(n_seqs: int, max_kv_len: int, sm_count: int, n_heads: int, n_kv: int, window: Optional[int],
                             chunk: Optional[int], dtype: torch.dtype, head_dim: Optional[int] = None,
                             v_dim: Optional[int] = None, kv_lens=None, keep_first: int = 0):
    """(kernel, slices in the launch, tiles per slice) for one-token steps of `attention_general`.
    "tensor cores" (bfloat16, sizes the kernel takes): the cut `attn_decode_plan` makes for the keys-on-rows kernel, over
    the span a token can see.  "plain": slices of eight 32-key tiles counted from the start of that span (the last
    `window` positions, the token's chunk, or everything), so that a sequence's sums are formed in the same order
    whatever else the step holds."""
    limit = window or chunk
    keep_first = int(keep_first or 0) if window else 0
    if head_dim is not None and attn_general_tc_ok(dtype, head_dim, v_dim or head_dim):
        # what a token can see: the window (or chunk) and, in whole tiles of 16, the kept first positions
        reach = int(limit) + (keep_first + 15) // 16 * 16 if limit else None
        seen = min(max_kv_len, reach + 15) if limit else max_kv_len
        lens = [min(int(n), seen) for n in kv_lens] if kv_lens else None
        n_splits, own = attn_decode_plan(n_seqs, seen, sm_count, n_heads, n_kv, 64 if max(head_dim, v_dim or head_dim) <= 64 else 128,
                                         reach, torch.bfloat16, lens)
        return "tensor cores", n_splits, own
    span = max_kv_len
    for limit in (window, chunk):
        if limit:
            span = min(span, int(limit) + 31)
    tiles = (span + 31) // 32 + (1 if (window or chunk) else 0) + (keep_first + 31) // 32
    return "plain", max(1, (tiles + OWN_LENGTH_TILES - 1) // OWN_LENGTH_TILES), OWN_LENGTH_TILES


def act_mul(gate_up: torch.Tensor, act: str, out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """act(gate) * up over rows [gate | up]; `act` "silu" or "gelu_tanh"."""
    lib = _bind()
    _cuda(gate_up, "gate/up rows")
    if gate_up.dim() != 2 or not gate_up.is_contiguous() or gate_up.shape[1] % 2:
        raise KernelError("gate/up rows must be a contiguous [rows, 2 * width] matrix")
    try:
        code = {"silu": 0, "gelu_tanh": 1}[act]
    except KeyError:
        raise KernelError(f"unknown activation \"{act}\" (silu, gelu_tanh)") from None
    n, f = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((n, f), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib, lib.gi_act_mul(out.data_ptr(), gate_up.data_ptr(), _dt(gate_up, "gate/up rows"), n, f, int(interleaved), code,
                               _stream()))
    return out


# ------------------------------------------------------------------------------------------------
# Mamba-2: the steps between its two projections.  `state` is the mixer's per-sequence memory, float32
# [slots + 1, S floats + (taps - 1) * channels].
def _mamba_state(state: torch.Tensor, s_floats: int, channels: int, taps: int):
    if state is None or state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous():
        raise KernelError("the state-space mixer needs its per-sequence state as a contiguous float32 matrix")
    if state.shape[1] != s_floats + (taps - 1) * channels:
        raise KernelError(f"state rows hold {state.shape[1]} floats, wanted {s_floats + (taps - 1) * channels}")
    _cuda(state, "state")


def mamba2_conv(proj: torch.Tensor, conv_w: torch.Tensor, conv_b: torch.Tensor, state: torch.Tensor, step, inner: int,
                channels: int, taps: int, s_floats: int) -> torch.Tensor:
    """silu(conv(x | B | C)) for the step's tokens, [tokens, channels] in the rows' type; then the state takes the step's
    last inputs."""
    lib = _bind()
    _cuda(proj, "projected rows")
    ld = _rows(proj, "projected rows")
    _mamba_state(state, s_floats, channels, taps)
    if tuple(conv_w.shape) != (channels, taps) or not conv_w.is_contiguous() or conv_b.numel() != channels or conv_w.dtype != conv_b.dtype:
        raise KernelError(f"convolution weights must be [{channels}, {taps}] with {channels} biases of the same type")
    out = torch.empty((proj.shape[0], channels), dtype=proj.dtype, device=proj.device)
    _check(lib, lib.gi_mamba2_conv(out.data_ptr(), proj.data_ptr(), _dt(proj, "projected rows"), ld, conv_w.data_ptr(),
                                   conv_b.data_ptr(), _dt(conv_w, "convolution weights"), state.data_ptr(), state.stride(0),
                                   state.shape[0], _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"),
                                   step.n_seqs, step.max_q_len, inner, channels, taps, s_floats, _stream()))
    _check(lib, lib.gi_mamba2_conv_update(proj.data_ptr(), _dt(proj, "projected rows"), ld, state.data_ptr(), state.stride(0),
                                          state.shape[0], _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"),
                                          step.n_seqs, inner, channels, taps, s_floats, _stream()), 1 if taps > 1 else 0)
    return out


def mamba2_scan(xbc: torch.Tensor, proj: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                state: torch.Tensor, step, heads: int, head_dim: int, n_state: int, groups: int, taps: int) -> torch.Tensor:
    """The recurrence over the step's tokens from and into `state`; float32 [tokens, heads * head_dim]."""
    lib = _bind()
    _cuda(xbc, "convolved rows")
    _cuda(proj, "projected rows")
    inner = heads * head_dim
    channels = inner + 2 * groups * n_state
    _mamba_state(state, heads * n_state * head_dim, channels, taps)
    if xbc.dtype != proj.dtype or tuple(xbc.shape) != (proj.shape[0], channels) or not xbc.is_contiguous():
        raise KernelError(f"convolved rows must be contiguous [{proj.shape[0]}, {channels}] of the projected rows' type")
    if proj.shape[1] != 2 * inner + 2 * groups * n_state + heads:
        raise KernelError(f"projected rows are {proj.shape[1]} wide, wanted {2 * inner + 2 * groups * n_state + heads}")
    for t in (dt_bias, a_log, d_skip):
        if t.numel() != heads or t.dtype != dt_bias.dtype or not t.is_contiguous():
            raise KernelError(f"the recurrence's per-head constants must be {heads} values of one type")
    y = torch.empty((proj.shape[0], inner), dtype=torch.float32, device=proj.device)
    _check(lib, lib.gi_mamba2_scan(y.data_ptr(), xbc.data_ptr(), proj.data_ptr(), _dt(proj, "projected rows"),
                                   _rows(proj, "projected rows"), dt_bias.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(),
                                   _dt(dt_bias, "per-head constants"), state.data_ptr(), state.stride(0), state.shape[0],
                                   _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"), step.n_seqs, heads,
                                   head_dim, n_state, groups, _stream()))
    return y


def mamba2_gate_norm(y: torch.Tensor, proj: torch.Tensor, weight: torch.Tensor, parts: int, eps: float,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """rmsnorm in `parts` equal parts of y * silu(z) (z: the first columns of `proj`), times `weight`."""
    lib = _bind()
    _cuda(y, "recurrence output")
    n, inner = y.shape
    if y.dtype != torch.float32 or not y.is_contiguous() or weight.numel() != inner or not weight.is_contiguous():
        raise KernelError("the gated norm takes contiguous float32 rows and one weight per value")
    out = torch.empty((n, inner), dtype=out_dtype, device=y.device)
    _check(lib, lib.gi_mamba2_gate_norm(out.data_ptr(), _dt(out, "normed rows"), y.data_ptr(), proj.data_ptr(),
                                        _dt(proj, "projected rows"), _rows(proj, "projected rows"), weight.data_ptr(),
                                        _dt(weight, "norm weight"), n, inner, int(parts), float(eps), _stream()))
    return out


# ------------------------------------------------------------------------------------------------
# Routed feed-forward.
def moe_route(h: torch.Tensor, w_router: torch.Tensor, top: int, w_shared_gate: Optional[torch.Tensor] = None,
              scores: str = "softmax"):
    """(ids int32 [tokens, top], weights float32 [tokens, top], shared gate float32 [tokens] or None).  `scores`: "softmax"
    (over the chosen logits) or "sigmoid" (each chosen logit's own, not renormalized)."""
    if scores not in ("softmax", "sigmoid"):
        raise KernelError(f"unknown kind of router weights \"{scores}\" (softmax, sigmoid)")
    lib = _bind()
    _cuda(h, "activations")
    ldh = _rows(h, "activations")
    n, width = h.shape
    experts = w_router.shape[0]
    if w_router.dim() != 2 or w_router.shape[1] != width or not w_router.is_contiguous():
        raise KernelError(f"router weights must be contiguous [experts, {width}]")
    if w_shared_gate is not None and (w_shared_gate.numel() != width or w_shared_gate.dtype != w_router.dtype
                                      or not w_shared_gate.is_contiguous()):
        raise KernelError(f"the shared expert's gate must be {width} values of the router's type")
    ids = torch.empty((n, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=h.device)
    sg = torch.empty((n,), dtype=torch.float32, device=h.device) if w_shared_gate is not None else None
    _check(lib, lib.gi_moe_route_scored(ids.data_ptr(), wts.data_ptr(), sg.data_ptr() if sg is not None else None, h.data_ptr(),
                                        _dt(h, "activations"), ldh, w_router.data_ptr(),
                                        w_shared_gate.data_ptr() if w_shared_gate is not None else None,
                                        _dt(w_router, "router weights"), n, width, experts, int(top),
                                        1 if scores == "sigmoid" else 0, _stream()))
    return ids, wts, sg


def moe_plan(ids: torch.Tensor, experts: int):
    """(offsets int32 [experts + 1], perm int32 [entries], inv int32 [entries]) of the stable sort of `ids` by expert."""
    lib = _bind()
    entries = ids.numel()
    dev = ids.device
    offsets = torch.empty((experts + 1,), dtype=torch.int32, device=dev)
    perm = torch.empty((entries,), dtype=torch.int32, device=dev)
    inv = torch.empty((entries,), dtype=torch.int32, device=dev)
    scratch = torch.empty(((entries + 1023) // 1024 * experts + entries,), dtype=torch.int32, device=dev)
    _check(lib, lib.gi_moe_plan(offsets.data_ptr(), perm.data_ptr(), inv.data_ptr(), scratch.data_ptr(), _i32(ids, "expert ids"),
                                entries, int(experts), _stream()), 3)
    return offsets, perm, inv


def moe_gather_rows(h: torch.Tensor, perm: torch.Tensor, top: int, scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The step's rows in the order of the sort by expert: out[r] = h[perm[r] // top], times scale[perm[r]] where `scale`
    (float32, one number per entry: the router's weights) is given."""
    lib = _bind()
    _cuda(h, "activations")
    if scale is not None and (scale.dtype != torch.float32 or scale.numel() != perm.numel() or not scale.is_contiguous()):
        raise KernelError("the rows' scales must be contiguous float32, one per entry")
    out = torch.empty((perm.numel(), h.shape[1]), dtype=h.dtype, device=h.device)
    _check(lib, lib.gi_moe_gather_rows_scaled(out.data_ptr(), h.data_ptr(), _dt(h, "activations"), _rows(h, "activations"),
                                              _i32(perm, "permutation"), scale.data_ptr() if scale is not None else None,
                                              perm.numel(), int(top), h.shape[1], _stream()))
    return out


def moe_rows_product(rows: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, act: Optional[str] = None) -> torch.Tensor:
    """out[r] = W_e rows[r] for rows already sorted by expert (`offsets` on the device), `w` [experts, n, k].  `act` None:
    the sums as float32; "relu2": relu(sum)^2 in the rows' type (an ungated expert's hidden layer)."""
    lib = _bind()
    _cuda(rows, "sorted rows")
    experts, n, k = w.shape
    if act not in (None, "relu2"):
        raise KernelError(f"unknown activation \"{act}\" (relu2)")
    if rows.shape[1] != k or not w.is_contiguous():
        raise KernelError(f"expert weights {tuple(w.shape)} do not fit rows of {rows.shape[1]}")
    entries = rows.shape[0]
    out = torch.empty((entries, n), dtype=torch.float32 if act is None else rows.dtype, device=rows.device)
    _check(lib, lib.gi_moe_gemm_rows(out.data_ptr(), rows.data_ptr(), _dt(rows, "sorted rows"), _rows(rows, "sorted rows"),
                                     w.data_ptr(), _dt(w, "expert weights"), w.stride(0), _i32(offsets, "offsets"), entries,
                                     experts, n, k, 0 if act is None else 1, _stream()))
    return out


def moe_experts(h: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, offsets: torch.Tensor, perm: torch.Tensor,
                top: int, interleaved: bool = False, limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """Every chosen expert's output, float32 [entries (in sorted order), width]: down_e(silu(gate_e h) * (up_e h)), or with
    `limit` > 0 the clamped form down_e(g sigmoid(alpha g) (u + 1)), g = min(gate_e h, limit), u = clamp(up_e h, +-limit).
    `w_gate_up` [experts, 2 f, width] (gate rows, then up rows; or, `interleaved`, blocks [8 gate | 8 up]), `w_down`
    [experts, width, f].  Few entries (one-token steps) take kernels that stream the chosen experts' matrices once."""
    lib = _bind()
    _cuda(h, "activations")
    lda = _rows(h, "activations")
    experts, f2, width = w_gate_up.shape
    f = f2 // 2
    if h.shape[1] != width or tuple(w_down.shape) != (experts, width, f) or not w_gate_up.is_contiguous() or not w_down.is_contiguous():
        raise KernelError(f"expert weights {tuple(w_gate_up.shape)} and {tuple(w_down.shape)} do not fit rows of {h.shape[1]}")
    if w_gate_up.dtype != w_down.dtype:
        raise KernelError("expert weights must share a type")
    entries = perm.numel()
    inter = torch.empty((entries, f), dtype=h.dtype, device=h.device)
    _check(lib, lib.gi_moe_gemm_gate_up_clamped(inter.data_ptr(), _dt(h, "activations"), h.data_ptr(), lda, w_gate_up.data_ptr(),
                                                _dt(w_gate_up, "expert weights"), w_gate_up.stride(0), _i32(offsets, "offsets"),
                                                _i32(perm, "permutation"), entries, int(top), experts, f, width, int(interleaved),
                                                float(limit), float(alpha), _stream()))
    down = torch.empty((entries, width), dtype=torch.float32, device=h.device)
    _check(lib, lib.gi_moe_gemm_down(down.data_ptr(), inter.data_ptr(), _dt(inter, "activations"), f, w_down.data_ptr(),
                                     _dt(w_down, "expert weights"), w_down.stride(0), _i32(offsets, "offsets"), entries,
                                     experts, width, f, _stream()))
    return down


def moe_experts_by_expert(rows: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, host_offsets, limit: float = 0.0,
                          alpha: float = 1.0) -> torch.Tensor:
    """The experts' outputs, float32 [entries, width], for rows already in sorted order, through the tcgen05 products expert
    by expert; `host_offsets`: the experts' offsets as Python integers (the caller has read them back).  bfloat16, gate and
    up rows interleaved in blocks of 8.  `limit` > 0: the clamped form of the gated value (see `moe_experts`)."""
    lib = _bind()
    _cuda(rows, "sorted rows")
    experts, f2, width = w_gate_up.shape
    f = f2 // 2
    entries = rows.shape[0]
    if (rows.dtype != torch.bfloat16 or w_gate_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16 or not rows.is_contiguous()
            or rows.shape[1] != width or tuple(w_down.shape) != (experts, width, f) or not w_gate_up.is_contiguous()
            or not w_down.is_contiguous()):
        raise KernelError("experts on tensor cores take contiguous bfloat16 rows and weights of fitting sizes")
    if len(host_offsets) != experts + 1 or host_offsets[0] != 0 or host_offsets[-1] != entries or any(
            b < a for a, b in zip(host_offsets, host_offsets[1:])):
        raise KernelError("the experts' offsets do not cover the rows")
    hidden = torch.empty((entries, f), dtype=torch.bfloat16, device=rows.device)
    out = torch.empty((entries, width), dtype=torch.float32, device=rows.device)
    scratch, counters = _stream_buffers(rows.device)
    offs = (c_int * (experts + 1))(*[int(x) for x in host_offsets])
    n_live = sum(1 for a, b in zip(host_offsets, host_offsets[1:]) if b > a)
    if limit and limit > 0:
        _check(lib, lib.gi_moe_experts_tc_clamped(out.data_ptr(), hidden.data_ptr(), rows.data_ptr(), w_gate_up.data_ptr(),
                                                  w_gate_up.stride(0), w_down.data_ptr(), w_down.stride(0), offs, experts, width, f,
                                                  float(limit), float(alpha), scratch.data_ptr(), counters.data_ptr(), counters.numel(),
                                                  _stream()), 2 * n_live)
        return out
    _check(lib, lib.gi_moe_experts_tc(out.data_ptr(), hidden.data_ptr(), rows.data_ptr(), w_gate_up.data_ptr(), w_gate_up.stride(0),
                                      w_down.data_ptr(), w_down.stride(0), offs, experts, width, f, scratch.data_ptr(),
                                      counters.data_ptr(), counters.numel(), _stream()), 2 * n_live)
    return out


def moe_experts_by_expert_ungated(rows: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, host_offsets) -> torch.Tensor:
    """`moe_experts_by_expert` for ungated experts: W_down,e relu(W_up,e row)^2 over every expert's stretch of the sorted
    rows, float32 [entries, width]; the squared relu rides in the first product's epilogue.  bfloat16."""
    lib = _bind()
    _cuda(rows, "sorted rows")
    experts, f, width = w_up.shape
    entries = rows.shape[0]
    if (rows.dtype != torch.bfloat16 or w_up.dtype != torch.bfloat16 or w_down.dtype != torch.bfloat16 or not rows.is_contiguous()
            or rows.shape[1] != width or tuple(w_down.shape) != (experts, width, f) or not w_up.is_contiguous()
            or not w_down.is_contiguous() or f % 8 or width % 8):
        raise KernelError("experts on tensor cores take contiguous bfloat16 rows and weights of fitting sizes, multiples of 8")
    if len(host_offsets) != experts + 1 or host_offsets[0] != 0 or host_offsets[-1] != entries or any(
            b < a for a, b in zip(host_offsets, host_offsets[1:])):
        raise KernelError("the experts' offsets do not cover the rows")
    hidden = torch.empty((entries, f), dtype=torch.bfloat16, device=rows.device)
    out = torch.empty((entries, width), dtype=torch.float32, device=rows.device)
    scratch, counters = _stream_buffers(rows.device)
    offs = (c_int * (experts + 1))(*[int(x) for x in host_offsets])
    n_live = sum(1 for a, b in zip(host_offsets, host_offsets[1:]) if b > a)
    _check(lib, lib.gi_moe_experts_tc_ungated(out.data_ptr(), hidden.data_ptr(), rows.data_ptr(), w_up.data_ptr(), w_up.stride(0),
                                              w_down.data_ptr(), w_down.stride(0), offs, experts, width, f, scratch.data_ptr(),
                                              counters.data_ptr(), counters.numel(), _stream()), 2 * n_live)
    return out


def moe_combine(residual: torch.Tensor, down: torch.Tensor, inv: torch.Tensor, wts: Optional[torch.Tensor],
                shared: Optional[torch.Tensor] = None, shared_gate: Optional[torch.Tensor] = None) -> None:
    """residual[t] += sum_k wts[t, k] * down[inv[t, k]] (+ shared_gate[t] * shared[t]); `wts` None: every weight 1."""
    lib = _bind()
    _cuda(residual, "residual stream")
    n, width = residual.shape
    top = inv.numel() // max(n, 1)
    if residual.dtype != torch.float32 or not residual.is_contiguous() or down.dtype != torch.float32 or down.shape[1] != width:
        raise KernelError("expert combine: float32 rows of the stream's width are wanted")
    if shared is not None and (shared.dtype != torch.float32 or tuple(shared.shape) != (n, width) or not shared.is_contiguous()
                               or shared_gate is None):
        raise KernelError("expert combine: the shared expert's output must be float32 [tokens, width] with its gate")
    _check(lib, lib.gi_moe_combine(residual.data_ptr(), down.data_ptr(), _i32(inv, "inverse permutation"),
                                   wts.data_ptr() if wts is not None else None,
                                   shared.data_ptr() if shared is not None else None,
                                   shared_gate.data_ptr() if shared is not None else None, n, width, top, _stream()))


# ---- layers with a latent in place of keys and values per head --------------------------------------------------------
def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """(x - mean) / sqrt(var + eps) * weight per row of the float32 matrix `x` (statistics in 32-bit)."""
    lib = _bind()
    _cuda(x, "layernorm input", settles=True)
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelError("layernorm input must be a contiguous float32 [rows, width] matrix")
    d = x.shape[1]
    if weight.numel() != d or not weight.is_contiguous():
        raise KernelError(f"layernorm weight has {weight.numel()} values, the rows are {d} wide")
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    pending = _take_pending(x)
    if pending is not None and (pending[1] or d % 4 != 0 or d > 4096 or x.data_ptr() % 16 != 0):
        x.__dict__["_gi_pending"] = pending         # not sums this kernel can add: the plain way
        settle(x)
        pending = None
    if pending is not None:
        # a deferred product left partial sums for this stream: they are added while the rows are read anyway
        _check(lib, lib.gi_layernorm_settle(out.data_ptr(), _dt(out, "layernorm output"), x.data_ptr(), weight.data_ptr(),
                                            _dt(weight, "layernorm weight"), _i32(rows, "rows"), n, d, float(eps), pending[0],
                                            _stream()))
        return out
    _check(lib, lib.gi_layernorm(out.data_ptr(), _dt(out, "layernorm output"), x.data_ptr(), weight.data_ptr(),
                                 _dt(weight, "layernorm weight"), _i32(rows, "rows"), n, d, float(eps), _stream()))
    return out


def bias_act(rows: torch.Tensor, bias: Optional[torch.Tensor], act: Optional[str] = None,
             residual: Optional[torch.Tensor] = None, residual_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """act(rows + bias) in the rows' type (`act` None or "relu2": relu squared); with `residual` (float32 rows of the
    stream) its rows also get `residual_bias` added, in the same launch."""
    lib = _bind()
    _cuda(rows, "rows")
    ld = _rows(rows, "rows")
    n, f = rows.shape
    if act not in (None, "relu2"):
        raise KernelError(f"unknown activation \"{act}\" (relu2)")
    wd = bias if bias is not None else residual_bias
    if bias is not None and (bias.numel() != f or not bias.is_contiguous()):
        raise KernelError(f"the bias has {bias.numel()} values, the rows are {f} wide")
    d = 0
    if residual is not None:
        _cuda(residual, "residual stream")
        d = residual.shape[1]
        if (residual.dtype != torch.float32 or not residual.is_contiguous() or residual.shape[0] != n or residual_bias is None
                or residual_bias.numel() != d or not residual_bias.is_contiguous() or (bias is not None and residual_bias.dtype != bias.dtype)):
            raise KernelError("the stream's rows must be contiguous float32, one per row, with a bias of their width and the other bias's type")
    out = torch.empty((n, f), dtype=rows.dtype, device=rows.device)
    _check(lib, lib.gi_bias_act(out.data_ptr(), rows.data_ptr(), _dt(rows, "rows"), ld, bias.data_ptr() if bias is not None else None,
                                _dt(wd, "bias") if wd is not None else F32, n, f, 0 if act is None else 1,
                                residual.data_ptr() if residual is not None else None,
                                residual_bias.data_ptr() if residual is not None else None, d, _stream()))
    return out


ACT_RELU2 = 0x200       # or-ed into SKINNY_STORE_BF16 for the tensor-core product: relu(sum + bias)^2
ACT_GELU_ERF = 0x400    # the same: gelu(sum) in its exact (erf) form, no bias


def linear_act(h: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: str = "relu2") -> torch.Tensor:
    """act(h W^T + bias) in h's type (`act` "relu2": relu squared; "gelu": the exact (erf) form, without a bias).  A prompt
    step's product on the tensor cores adds the bias and applies the activation in its epilogue, on the 32-bit sums; other
    products are followed by `bias_act` or `gelu_rows`."""
    if act not in ("relu2", "gelu") or (act == "gelu" and bias is not None):
        raise KernelError(f"unknown activation \"{act}\" (relu2, or gelu without a bias)")
    flag = ACT_RELU2 if act == "relu2" else ACT_GELU_ERF
    if (tc_ok(h, w) and h.shape[0] > SKINNY_MAX_ROWS and w.shape[0] % 8 == 0
            and (bias is None or (bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == w.shape[0]))):
        lib = _bind()
        _cuda(h, "activations")
        m, k = h.shape
        n = w.shape[0]
        out = torch.empty((m, n), dtype=torch.bfloat16, device=h.device)
        _check(lib, lib.gi_gemm_tc_bf16_bias(out.data_ptr(), SKINNY_STORE_BF16 | flag, h.data_ptr(), w.data_ptr(),
                                             bias.data_ptr() if bias is not None else None, m, n, k, _rows(h, "activations"),
                                             _rows(w, "weights"), n, int(TC_TILE_N), _stream()))
        return out
    if act == "gelu":
        return gelu_rows(linear(h, w, out_dtype=h.dtype))
    return bias_act(linear(h, w, out_dtype=h.dtype), bias, act)


def add_row_bias(residual: torch.Tensor, bias: torch.Tensor) -> None:
    """residual[t, :] += bias for every row of the float32 matrix `residual`."""
    lib = _bind()
    _cuda(residual, "residual stream")
    n, d = residual.shape
    if residual.dtype != torch.float32 or not residual.is_contiguous() or bias.numel() != d or not bias.is_contiguous():
        raise KernelError("the stream's rows must be contiguous float32 with a bias of their width")
    _check(lib, lib.gi_bias_act(None, None, F32, 0, None, _dt(bias, "bias"), n, 0, 0, residual.data_ptr(), bias.data_ptr(), d, _stream()))


def latent_prepare(rows: torch.Tensor, w_query_norm: Optional[torch.Tensor], w_latent_norm: torch.Tensor, eps: float,
                   table: Optional[torch.Tensor], rot: int, positions: torch.Tensor, slots: torch.Tensor, memory,
                   q_rank: int, rank: int, rot_dim: int) -> Optional[torch.Tensor]:
    """From rows [query latent (q_rank) | latent (rank) | rotary key part (rot_dim)]: the RMS-normed query latent (returned,
    in the rows' type; None when q_rank is 0), and the token's cache row [RMS-normed latent | key part, its first `rot`
    numbers turned in neighbouring pairs by `table`] written into `memory`'s pages."""
    lib = _bind()
    _cuda(rows, "latent rows")
    ld = _rows(rows, "latent rows")
    n = rows.shape[0]
    if rows.shape[1] != q_rank + rank + rot_dim:
        raise KernelError(f"latent rows are {rows.shape[1]} wide, wanted {q_rank + rank + rot_dim}")
    write = bool(memory.writes and memory.k is not None)
    if write and (memory.k.dtype != rows.dtype or tuple(memory.k.shape[1:]) != (1, 64, rank + rot_dim) or not memory.k.is_contiguous()):
        raise KernelError(f"the latent cache must be contiguous {rows.dtype} [pages, 1, 64, {rank + rot_dim}], got {memory.k.dtype} {tuple(memory.k.shape)}")
    if w_latent_norm.numel() != rank or (q_rank and (w_query_norm is None or w_query_norm.numel() != q_rank or w_query_norm.dtype != w_latent_norm.dtype)):
        raise KernelError("the latents' norm weights do not fit their sizes")
    cq = torch.empty((n, q_rank), dtype=rows.dtype, device=rows.device) if q_rank else None
    bt = memory.block_table
    _check(lib, lib.gi_latent_prepare(
        cq.data_ptr() if cq is not None else None, rows.data_ptr(), _dt(rows, "latent rows"), ld,
        w_query_norm.data_ptr() if q_rank else None, w_latent_norm.data_ptr(), _dt(w_latent_norm, "norm weights"), float(eps),
        table.data_ptr() if table is not None else None, int(rot), _i32(positions, "positions"), _i32(slots, "slots"),
        _i32(bt, "block table"), bt.shape[1] if bt is not None else 0, memory.k.data_ptr() if write else None, n, q_rank, rank,
        rot_dim, int(write), _stream()))
    return cq


def latent_query_rot(qa: torch.Tensor, q: torch.Tensor, table: Optional[torch.Tensor], rot: int, n_heads: int, dim: int,
                     rot_dim: int, rank: int) -> None:
    """qa[t, h, rank:] = q[t, h, dim:] with its first `rot` numbers turned; q rows [heads][dim + rot_dim], qa rows
    [heads][rank + rot_dim]."""
    lib = _bind()
    _cuda(q, "queries")
    if q.dtype != qa.dtype or q.shape[1] != n_heads * (dim + rot_dim) or qa.shape[1] != n_heads * (rank + rot_dim) or q.shape[0] != qa.shape[0]:
        raise KernelError("latent queries: rows of the wrong sizes")
    _check(lib, lib.gi_latent_query_rot(qa.data_ptr(), _rows(qa, "latent queries"), q.data_ptr(), _rows(q, "queries"),
                                        _dt(q, "queries"), table.data_ptr() if table is not None else None, int(rot), q.shape[0],
                                        n_heads, dim, rot_dim, rank, _stream()))


def bmm_heads(out: torch.Tensor, out_head_stride: int, a: torch.Tensor, a_head_stride: int, w: torch.Tensor, n: int, k: int,
              k_stride: int = 1, row_stride: Optional[int] = None) -> None:
    """out[t, h * out_head_stride + j] = sum_i a[t, h * a_head_stride + i] * w[h][j, i] for j < n, i < k and every head h of
    `w` [heads, ...]: element (j, i) of a head's matrix sits at j * row_stride + i * k_stride (default: [n, k] row-major)."""
    lib = _bind()
    _cuda(a, "rows")
    if a.dtype != out.dtype or a.shape[0] != out.shape[0]:
        raise KernelError("per-head product: rows and outputs must share type and count")
    heads = w.shape[0]
    if not w.is_contiguous():
        raise KernelError("per-head product: the matrices must be contiguous")
    ldw = int(row_stride if row_stride is not None else k)
    _check(lib, lib.gi_bmm_heads(out.data_ptr(), _rows(out, "outputs"), int(out_head_stride), a.data_ptr(), _rows(a, "rows"),
                                 int(a_head_stride), _dt(a, "rows"), w.data_ptr(), _dt(w, "matrices"), w.stride(0), ldw,
                                 int(k_stride), a.shape[0], int(n), int(k), heads, int(TUNE["bmm_heads_tc"]), _stream()))


def attn_latent_tc_ok(dtype: torch.dtype, rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core kernel takes a latent cache of these sizes: bfloat16, rows and values multiples of 8,
    rows up to 576 and values up to 512 numbers."""
    return bool(TUNE["attn_latent_tc"] and dtype == torch.bfloat16 and rank % 8 == 0 and rot_dim % 8 == 0
                and rank + rot_dim <= 576 and rank <= 512)


def attn_latent_decode_plan(n_seqs: int, max_kv_len: int, sm_count: int, n_heads: int, rank: int, rot_dim: int, dtype: torch.dtype):
    """(kernel, slices in the launch, tiles per slice) for one-token steps over a latent cache.
    "tensor cores" (bfloat16, sizes the kernel takes): every context cut into equal slices of 64-key tiles, as many as
    fill the GPU once.  "plain": slices of eight 32-key tiles of each sequence's own span, so that a sequence's sums are
    formed in the same order whatever the step holds."""
    if attn_latent_tc_ok(dtype, rank, rot_dim):
        tiles = (max_kv_len + 63) // 64
        blocks = n_seqs * ((n_heads + 63) // 64)
        # one block per SM (the tiles' ring fills its shared memory): as many slices as make one round of blocks
        return "tensor cores", max(1, min(tiles, sm_count // max(blocks, 1))), 0
    tiles = (max_kv_len + 31) // 32
    return "plain", max(1, (tiles + OWN_LENGTH_TILES - 1) // OWN_LENGTH_TILES), OWN_LENGTH_TILES


def attention_latent(qa: torch.Tensor, memory, step, n_heads: int, rank: int, rot_dim: int, scale: float, out: torch.Tensor,
                     plan=None) -> torch.Tensor:
    """Causal attention of all heads over one shared row per position: `memory.k` holds [latent (rank) | rotary key part
    (rot_dim)] per position, a head's query row in `qa` has the same layout (its unrotated part already carried onto the
    latent), the score is their product times `scale`, and the value is the row's latent: out [tokens, heads * rank]."""
    if memory.k is None:
        raise KernelError("attention needs a cache to read from")
    hd = rank + rot_dim
    if qa.shape[1] != n_heads * hd or out.shape[1] != n_heads * rank:
        raise KernelError("latent attention: rows of the wrong sizes")
    lib = _bind()
    _cuda(qa, "queries")
    if memory.k.dtype != qa.dtype or out.dtype != qa.dtype:
        raise KernelError("queries, cache and attention output must share a dtype")
    if tuple(memory.k.shape[1:]) != (1, 64, hd) or not memory.k.is_contiguous():
        raise KernelError(f"the latent cache must be contiguous [pages, 1, 64, {hd}], got {tuple(memory.k.shape)}")
    bt = memory.block_table
    tc = (attn_latent_tc_ok(qa.dtype, rank, rot_dim) and qa.stride(0) % 8 == 0 and qa.data_ptr() % 16 == 0
          and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0)
    if step.is_decode:
        if plan is None:
            plan = attn_latent_decode_plan(step.n_seqs, step.max_kv_len, step.sm_count, n_heads, rank, rot_dim, qa.dtype)
        kind, n_splits, own_tiles = plan
        if kind == "tensor cores" and not tc:
            raise KernelError("latent attention: the rows do not suit the tensor-core kernel this step was planned for")
        part_o = part_ml = None
        if n_splits > 1:
            part_o = torch.empty((step.n_seqs * n_heads * n_splits * rank,), dtype=torch.float32, device=qa.device)
            part_ml = torch.empty((step.n_seqs * n_heads * n_splits * 2,), dtype=torch.float32, device=qa.device)
        po, pml = (part_o.data_ptr(), part_ml.data_ptr()) if part_o is not None else (None, None)
        if kind == "tensor cores":
            _check(lib, lib.gi_attn_latent_tc(
                out.data_ptr(), _rows(out, "attention output"), po, pml, qa.data_ptr(), _rows(qa, "queries"), memory.k.data_ptr(),
                _i32(bt, "block table"), bt.shape[1], None, _i32(step.seq_slots, "slots"), None, _i32(step.seq_lens, "lengths"),
                step.n_seqs, 1, n_heads, hd, rank, float(scale), int(n_splits), int(own_tiles), _stream()), 2 if n_splits > 1 else 1)
            return out
        _check(lib, lib.gi_attn_decode_generic_ex2(
            out.data_ptr(), _rows(out, "attention output"), po, pml, qa.data_ptr(), _rows(qa, "queries"), _dt(qa, "queries"),
            memory.k.data_ptr(), memory.k.data_ptr(), _i32(bt, "block table"), bt.shape[1],
            _i32(step.seq_slots, "slots"), _i32(step.seq_lens, "lengths"), step.n_seqs, n_heads, 1, hd, float(scale), 0,
            int(n_splits), int(own_tiles), rank, 0.0, None, 0, hd, _stream()), 2 if n_splits > 1 else 1)
        return out
    if tc:
        _check(lib, lib.gi_attn_latent_tc(
            out.data_ptr(), _rows(out, "attention output"), None, None, qa.data_ptr(), _rows(qa, "queries"), memory.k.data_ptr(),
            _i32(bt, "block table"), bt.shape[1], _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"),
            _i32(step.seq_pos0, "start positions"), None, step.n_seqs, step.max_q_len, n_heads, hd, rank, float(scale), 1, 0,
            _stream()))
        return out
    _check(lib, lib.gi_attn_prefill_generic_ex2(
        out.data_ptr(), _rows(out, "attention output"), qa.data_ptr(), _rows(qa, "queries"), _dt(qa, "queries"),
        memory.k.data_ptr(), memory.k.data_ptr(), _i32(bt, "block table"), bt.shape[1],
        _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"), _i32(step.seq_pos0, "start positions"), step.n_seqs,
        step.max_q_len, n_heads, 1, hd, float(scale), 0, rank, 0.0, None, 0, hd, _stream()))
    return out


# ------------------------------------------------------------------------------------------------
# Layers that read the stream itself and norm a sublayer's output; attention with normed, rotated queries and keys.
def cast_rows(x: torch.Tensor, dtype: torch.dtype, zero: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The float32 stream in the activation type; in the 32-bit path the stream itself.  `zero`: float32 rows of the
    stream's shape that are set to zero on the way (what a sublayer will add into)."""
    _cuda(x, "residual stream")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("the stream's rows must be contiguous float32")
    if zero is not None and (zero.dtype != torch.float32 or not zero.is_contiguous() or zero.shape != x.shape or not zero.is_cuda):
        raise KernelError("the rows to set to zero must be contiguous float32 of the stream's shape")
    if dtype == torch.float32:
        if zero is not None:
            zero.zero_()
        return x.as_subclass(torch.Tensor) if type(x) is not torch.Tensor else x
    lib = _bind()
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(lib, lib.gi_cast_rows_zero(out.data_ptr(), _dt(out, "rows"), x.data_ptr(), zero.data_ptr() if zero is not None else None,
                                      x.numel(), _stream()))
    return out


def postnorm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, scale: Optional[torch.Tensor] = None,
                 cast_out: Optional[torch.Tensor] = None, zero_y: bool = False) -> None:
    """x += y / sqrt(mean(y^2) + eps) * weight [* scale] over float32 rows.  `cast_out`: rows of x's shape that receive the
    new x in their own type (what the next sublayer reads); `zero_y`: y is zero afterwards (what it adds into)."""
    lib = _bind()
    _cuda(x, "residual stream")
    _cuda(y, "sublayer output")
    n, d = x.shape
    if (x.dtype != torch.float32 or y.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous()
            or tuple(y.shape) != (n, d)):
        raise KernelError("the stream and the sublayer's output must be contiguous float32 rows of one shape")
    for t, what in ((weight, "the norm's weight"), (scale, "the channel scale")):
        if t is not None and (t.numel() != d or not t.is_contiguous() or t.dtype != weight.dtype):
            raise KernelError(f"{what} must hold {d} values of the norm weight's type")
    if cast_out is not None and (not cast_out.is_cuda or not cast_out.is_contiguous() or tuple(cast_out.shape) != (n, d)
                                 or cast_out.data_ptr() == x.data_ptr()):
        raise KernelError("the rows that take the new stream must be contiguous, of the stream's shape and not the stream itself")
    _check(lib, lib.gi_postnorm_add_ex(x.data_ptr(), y.data_ptr(), weight.data_ptr(), scale.data_ptr() if scale is not None else None,
                                       _dt(weight, "norm weight"), n, d, float(eps),
                                       cast_out.data_ptr() if cast_out is not None else None,
                                       _dt(cast_out, "next input") if cast_out is not None else F32, int(bool(zero_y)), _stream()))


def axpy(out: torch.Tensor, a: torch.Tensor, alpha: float) -> None:
    """out += alpha * a, float32."""
    lib = _bind()
    _cuda(out, "rows")
    _cuda(a, "rows")
    if out.dtype != torch.float32 or a.dtype != torch.float32 or out.shape != a.shape or not out.is_contiguous() or not a.is_contiguous():
        raise KernelError("axpy takes two contiguous float32 tensors of one shape")
    _check(lib, lib.gi_axpy(out.data_ptr(), a.data_ptr(), float(alpha), out.numel(), _stream()))


def qk_prepare(rows: torch.Tensor, out_dtype: torch.dtype, biases, norm_weights, eps: float, table: Optional[torch.Tensor],
               rot: int, adjacent: bool, step, memory, n_heads: int, n_kv: int, head_dim: int, v_dim: int) -> torch.Tensor:
    """Float32 projection rows [q | k | v] (`n_kv` 0: queries only) to queries [tokens, heads * head_dim] of `out_dtype`,
    with keys and values written to `memory`'s pages where the layer owns them.  `biases` (q, k, v) and `norm_weights`
    (q, k) hold tensors or None."""
    lib = _bind()
    _cuda(rows, "projected rows")
    n = rows.shape[0]
    qd, kd, vw = n_heads * head_dim, n_kv * head_dim, n_kv * v_dim
    if rows.dtype != torch.float32 or rows.shape[1] != qd + kd + vw:
        raise KernelError(f"projected rows must be float32 and {qd + kd + vw} wide, got {rows.dtype} {tuple(rows.shape)}")
    ld = _rows(rows, "projected rows")
    write = bool(n_kv > 0 and memory.writes and memory.k is not None)
    params = [t for t in tuple(biases) + tuple(norm_weights) if t is not None]
    wdt = params[0].dtype if params else torch.float32
    for t, size in zip(tuple(biases) + tuple(norm_weights), (qd, kd, vw, qd, kd)):
        if t is not None and (t.dtype != wdt or t.numel() != size or not t.is_contiguous()):
            raise KernelError("biases and norm weights must be contiguous, of one type and of their projection's width")
    if write:
        if memory.k.dtype != out_dtype or memory.v.dtype != out_dtype:
            raise KernelError(f"the cache is {memory.k.dtype}, the step runs in {out_dtype}")
        if (tuple(memory.k.shape[1:]) != (n_kv, 64, head_dim) or tuple(memory.v.shape[1:]) != (n_kv, 64, v_dim)
                or not memory.k.is_contiguous() or not memory.v.is_contiguous()):
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}] and [.., {v_dim}]")
    half = rot // 2
    if half and (table is None or table.dtype != torch.float32 or tuple(table.shape) != (n, half, 2) or not table.is_contiguous()):
        raise KernelError(f"the table of angles must be contiguous float32 [{n}, {half}, 2]")
    q = torch.empty((n, qd), dtype=out_dtype, device=rows.device)
    bt = memory.block_table if memory is not None else None
    ptr = lambda t: t.data_ptr() if t is not None else None
    _check(lib, lib.gi_qk_prepare(
        q.data_ptr(), qd, _dt(q, "queries"), rows.data_ptr(), ld, ptr(biases[0]), ptr(biases[1]), ptr(biases[2]),
        ptr(norm_weights[0]), ptr(norm_weights[1]), _DT[wdt], float(eps), ptr(table) if half else None, half, int(bool(adjacent)),
        _i32(step.positions, "positions"), _i32(step.token_slots, "slots"), _i32(bt, "block table") if write else None,
        bt.shape[1] if (write and bt is not None) else 0, memory.k.data_ptr() if write else None,
        memory.v.data_ptr() if write else None, n, n_heads, n_kv if write or n_kv == 0 else n_kv, head_dim, v_dim, int(write), _stream()))
    return q


def gate_mul(a: torch.Tensor, gate: torch.Tensor, act: str = "sigmoid") -> torch.Tensor:
    """a * sigmoid(gate) or a * silu(gate); `gate` may be a view of wider rows."""
    lib = _bind()
    _cuda(a, "rows")
    _cuda(gate, "gate rows")
    if act not in ("sigmoid", "silu"):
        raise KernelError(f"unknown gate \"{act}\" (sigmoid, silu)")
    if a.dtype != gate.dtype or a.shape != gate.shape or not a.is_contiguous():
        raise KernelError("gated rows must be contiguous and of the gate's type and shape")
    out = torch.empty_like(a)
    _check(lib, lib.gi_gate_mul(out.data_ptr(), a.data_ptr(), gate.data_ptr(), _rows(gate, "gate rows"), _dt(a, "rows"), a.shape[0],
                                a.shape[1], 1 if act == "silu" else 0, _stream()))
    return out


def norm_gate(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, group: int, eps: float, act: str,
              out_dtype: torch.dtype) -> torch.Tensor:
    """y / sqrt(mean over each group of `group` values (y^2) + eps) * weight * act(gate), the weight per value of a group
    (`group` values) or of the row."""
    lib = _bind()
    _cuda(y, "recurrence output")
    _cuda(gate, "gate rows")
    n, inner = y.shape
    if act not in ("sigmoid", "silu"):
        raise KernelError(f"unknown gate \"{act}\" (sigmoid, silu)")
    if y.dtype != torch.float32 or not y.is_contiguous() or gate.dtype != out_dtype or tuple(gate.shape) != (n, inner):
        raise KernelError("the gated norm takes contiguous float32 rows and a gate of the output's type and the rows' shape")
    if weight.numel() not in (group, inner) or not weight.is_contiguous():
        raise KernelError(f"the norm's weight must hold {group} or {inner} values")
    out = torch.empty((n, inner), dtype=out_dtype, device=y.device)
    _check(lib, lib.gi_norm_gate(out.data_ptr(), _dt(out, "normed rows"), y.data_ptr(), gate.data_ptr(), _rows(gate, "gate rows"),
                                 weight.data_ptr(), _dt(weight, "norm weight"), n, inner, int(group),
                                 int(weight.numel() == inner and group != inner), 1 if act == "silu" else 0, float(eps), _stream()))
    return out


def side_gate(gx: torch.Tensor, table: torch.Tensor, tokens: torch.Tensor, col0: int, dim: int) -> torch.Tensor:
    """gelu_tanh(gx) * table[tokens, col0 : col0 + dim], in gx's type."""
    lib = _bind()
    _cuda(gx, "gate rows")
    _cuda(table, "side table")
    n = gx.shape[0]
    if gx.shape[1] != dim or table.dim() != 2 or col0 < 0 or col0 + dim > table.shape[1] or tokens.numel() != n:
        raise KernelError("side gate: the gate rows, the table's slice and the tokens do not fit each other")
    out = torch.empty((n, dim), dtype=gx.dtype, device=gx.device)
    _check(lib, lib.gi_side_gate(out.data_ptr(), gx.data_ptr(), _rows(gx, "gate rows"), _dt(gx, "gate rows"), table.data_ptr(),
                                 _rows(table, "side table"), _dt(table, "side table"), _i32(tokens, "tokens"), n, int(col0), int(dim),
                                 _stream()))
    return out


def gelu_rows(rows: torch.Tensor) -> torch.Tensor:
    """gelu in its exact (erf) form, in the rows' type."""
    lib = _bind()
    _cuda(rows, "rows")
    out = torch.empty(rows.shape, dtype=rows.dtype, device=rows.device)
    _check(lib, lib.gi_act_rows(out.data_ptr(), rows.data_ptr(), _rows(rows, "rows"), _dt(rows, "rows"), rows.shape[0], rows.shape[1],
                                _stream()))
    return out


def linear_state(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, step, heads: int, qk_heads: int,
                 key_dim: int, v_dim: int, decay: torch.Tensor, *, decay_in: Optional[torch.Tensor] = None,
                 dt_bias: Optional[torch.Tensor] = None, beta_in: Optional[torch.Tensor] = None, in_act: bool = False,
                 unit_norm: bool = False, norm_eps: float = 1e-6, q_scale: float = 1.0, delta: bool = False) -> torch.Tensor:
    """The recurrence S <- g S; u = delta ? beta (v - S^T k) : v; S <- S + k u^T; o = S^T q over the step's tokens, from and
    into `state` ([slots + 1, >= heads * key_dim * v_dim] float32).  q, k, v, decay_in, beta_in: views of rows in one type.
    `decay` float32 [heads]: the decay itself, or A_log where `decay_in` (with `dt_bias`) gives the per-token part.
    Returns float32 [tokens, heads * v_dim]."""
    lib = _bind()
    n = q.shape[0]
    for t, what, width in ((q, "queries", qk_heads * key_dim), (k, "keys", qk_heads * key_dim), (v, "values", heads * v_dim),
                           (decay_in, "decay rows", heads), (beta_in, "write strengths", heads)):
        if t is None:
            continue
        _cuda(t, what)
        if t.dtype != q.dtype or tuple(t.shape) != (n, width) or t.stride(1) != 1:
            raise KernelError(f"{what} must be [{n}, {width}] rows of the queries' type, got {t.dtype} {tuple(t.shape)}")
    if state is None or state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < heads * key_dim * v_dim:
        raise KernelError("the recurrence needs its per-sequence state as a contiguous float32 matrix of at least heads x keys x values")
    for t in (decay, dt_bias):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous() or not t.is_cuda):
            raise KernelError(f"the recurrence's per-head constants must be {heads} float32 values on the device")
    o = torch.empty((n, heads * v_dim), dtype=torch.float32, device=q.device)
    ptr = lambda t: t.data_ptr() if t is not None else None
    ldo = lambda t: t.stride(0) if t is not None else 0
    _check(lib, lib.gi_linear_state(
        o.data_ptr(), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), ptr(decay_in), ldo(decay_in),
        ptr(beta_in), ldo(beta_in), _dt(q, "queries"), decay.data_ptr(), ptr(dt_bias), state.data_ptr(), state.stride(0),
        state.shape[0], _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"), step.n_seqs, heads, qk_heads, key_dim,
        v_dim, int(in_act), int(unit_norm), float(norm_eps), float(q_scale), int(delta), int(n), _stream()))
    return o


def linear_state_gated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, step, heads: int, key_dim: int,
                       v_dim: int, decay: torch.Tensor, write: torch.Tensor) -> torch.Tensor:
    """The recurrence S <- decay_t S + k_t (write_t v_t)^T; o_t = S^T q_t with both gates ready made, float32 [tokens, heads],
    from and into `state` ([slots + 1, >= heads * key_dim * v_dim] float32).  Returns float32 [tokens, heads * v_dim]."""
    lib = _bind()
    n = q.shape[0]
    for t, what, width in ((q, "queries", heads * key_dim), (k, "keys", heads * key_dim), (v, "values", heads * v_dim)):
        _cuda(t, what)
        if t.dtype != q.dtype or tuple(t.shape) != (n, width) or t.stride(1) != 1:
            raise KernelError(f"{what} must be [{n}, {width}] rows of the queries' type, got {t.dtype} {tuple(t.shape)}")
    for t, what in ((decay, "decays"), (write, "write strengths")):
        if t.dtype != torch.float32 or tuple(t.shape) != (n, heads) or not t.is_contiguous() or not t.is_cuda:
            raise KernelError(f"{what} must be contiguous float32 [{n}, {heads}] on the device")
    if state is None or state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous() or state.shape[1] < heads * key_dim * v_dim:
        raise KernelError("the recurrence needs its per-sequence state as a contiguous float32 matrix of at least heads x keys x values")
    o = torch.empty((n, heads * v_dim), dtype=torch.float32, device=q.device)
    _check(lib, lib.gi_linear_state_gated(
        o.data_ptr(), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), None, 0, None, 0,
        _dt(q, "queries"), None, None, decay.data_ptr(), write.data_ptr(), state.data_ptr(), state.stride(0), state.shape[0],
        _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"), step.n_seqs, heads, heads, key_dim, v_dim, 0, 0,
        1e-6, 1.0, 0, int(n), _stream()))
    return o


def mlstm_gates(q: torch.Tensor, k: torch.Tensor, gate_i: torch.Tensor, gate_f: torch.Tensor, bias_i: Optional[torch.Tensor],
                bias_f: Optional[torch.Tensor], cap: float, q_scale: float, state: torch.Tensor, state_offset: int, step, heads: int,
                key_dim: int):
    """(keep, put, out_scale), each float32 [tokens, heads], of a matrix memory with a running maximum; the normalizer n and
    the maximum m live in `state` ([slots + 1, ...] float32) from `state_offset` on, heads * (key_dim + 1) floats."""
    lib = _bind()
    n = q.shape[0]
    for t, what, width in ((q, "queries", heads * key_dim), (k, "keys", heads * key_dim), (gate_i, "input gates", heads),
                           (gate_f, "forget gates", heads)):
        _cuda(t, what)
        if t.dtype != q.dtype or tuple(t.shape) != (n, width) or t.stride(1) != 1:
            raise KernelError(f"{what} must be [{n}, {width}] rows of the queries' type, got {t.dtype} {tuple(t.shape)}")
    if gate_i.stride(0) != gate_f.stride(0):
        raise KernelError("the two gates' rows must be equally far apart")
    for t in (bias_i, bias_f):
        if t is not None and (t.dtype != torch.float32 or t.numel() != heads or not t.is_contiguous() or not t.is_cuda):
            raise KernelError(f"a gate's bias must be {heads} float32 values on the device")
    if (state is None or state.dtype != torch.float32 or state.dim() != 2 or not state.is_contiguous()
            or state.shape[1] < state_offset + heads * (key_dim + 1)):
        raise KernelError("the gates need heads x (keys + 1) float32 numbers of per-sequence state")
    keep, put, scale = (torch.empty((n, heads), dtype=torch.float32, device=q.device) for _ in range(3))
    _check(lib, lib.gi_mlstm_gates(
        keep.data_ptr(), put.data_ptr(), scale.data_ptr(), q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), gate_i.data_ptr(),
        gate_f.data_ptr(), gate_i.stride(0), _dt(q, "queries"), bias_i.data_ptr() if bias_i is not None else None,
        bias_f.data_ptr() if bias_f is not None else None, float(cap), float(q_scale), state.data_ptr() + 4 * int(state_offset),
        state.stride(0), state.shape[0], _i32(step.cu_seqlens, "cu_seqlens"), _i32(step.seq_slots, "slots"), step.n_seqs, heads,
        key_dim, _stream()))
    return keep, put, scale


# ---- several copies of the residual stream ------------------------------------------------------------------------------
def stream_expand(e: torch.Tensor, streams: int) -> torch.Tensor:
    """float32 [tokens, streams * d]: every copy of the stream starts as the row of `e` (float32 [tokens, d])."""
    lib = _bind()
    _cuda(e, "embedded tokens")
    if e.dtype != torch.float32 or e.dim() != 2 or not e.is_contiguous():
        raise KernelError("the embedded tokens must be contiguous float32 rows")
    n, d = e.shape
    x = torch.empty((n, streams * d), dtype=torch.float32, device=e.device)
    _check(lib, lib.gi_stream_expand(x.data_ptr(), e.data_ptr(), n, int(streams), d, _stream()))
    return x


def stream_sum(x: torch.Tensor, streams: int, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """float32 [rows, d]: the sum of the copies of the chosen tokens (all tokens without `rows`)."""
    lib = _bind()
    _cuda(x, "residual streams")
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or x.shape[1] % streams:
        raise KernelError("the residual streams must be contiguous float32 rows of streams x width numbers")
    d = x.shape[1] // streams
    n = rows.numel() if rows is not None else x.shape[0]
    out = torch.empty((n, d), dtype=torch.float32, device=x.device)
    _check(lib, lib.gi_stream_sum(out.data_ptr(), x.data_ptr(), _i32(rows, "row selection"), n, int(streams), d, _stream()))
    return out


def hyper_read_conv_ok(d: int, taps: int) -> bool:
    """Whether `hyper_read` can run the input convolution of a one-token step in the same launch."""
    return d % 4 == 0 and 1 <= taps <= 8


def hyper_read(x: torch.Tensor, blend: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
               zero: Optional[torch.Tensor] = None, conv=None):
    """h = rmsnorm(sum_s blend[s] x[:, s]) * weight in `out_dtype`; `zero` (float32 [tokens, d]) is set to zero in the same pass.
    `conv` = (taps_w, state, step), only for a step of one token a sequence and where `hyper_read_conv_ok`: the input
    convolution (`input_conv`) runs in the same launch and (h, h + conv(h)) is returned."""
    lib = _bind()
    _cuda(x, "residual streams")
    streams = blend.numel()
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous() or x.shape[1] % streams:
        raise KernelError("the residual streams must be contiguous float32 rows of streams x width numbers")
    n, d = x.shape[0], x.shape[1] // streams
    if blend.dtype != torch.float32 or not blend.is_contiguous() or not blend.is_cuda or weight.numel() != d or not weight.is_contiguous():
        raise KernelError("hyper_read: the blend must be float32 [streams], the weight [width]")
    if zero is not None and (zero.dtype != torch.float32 or tuple(zero.shape) != (n, d) or not zero.is_contiguous()):
        raise KernelError("hyper_read: the rows to zero must be contiguous float32 [tokens, width]")
    h = torch.empty((n, d), dtype=out_dtype, device=x.device)
    if conv is not None:
        taps_w, state, step = conv
        taps = taps_w.shape[1]
        if not step.is_decode or tuple(taps_w.shape) != (d, taps) or not taps_w.is_contiguous() or not hyper_read_conv_ok(d, taps):
            raise KernelError("hyper_read: the convolution rides along in steps of one token a sequence, with taps [width, taps]")
        sp, sld, srows = _conv_state(state, taps, d)
        c = torch.empty((n, d), dtype=out_dtype, device=x.device)
        _check(lib, lib.gi_hyper_read_conv(h.data_ptr(), _DT[out_dtype], x.data_ptr(), blend.data_ptr(), weight.data_ptr(),
                                           _dt(weight, "norm weight"), zero.data_ptr() if zero is not None else None, n, streams, d,
                                           float(eps), c.data_ptr(), taps_w.data_ptr(), _dt(taps_w, "taps"), sp, sld, srows,
                                           _i32(step.token_slots, "slots"), taps, _stream()))
        return h, c
    _check(lib, lib.gi_hyper_read(h.data_ptr(), _DT[out_dtype], x.data_ptr(), blend.data_ptr(), weight.data_ptr(), _dt(weight, "norm weight"),
                                  zero.data_ptr() if zero is not None else None, n, streams, d, float(eps), _stream()))
    return h


def _conv_state(state: Optional[torch.Tensor], taps: int, d: int):
    if taps <= 1:
        return None, 0, 0
    if state is None or state.dtype != torch.float32 or state.dim() != 2 or state.stride(1) != 1 or state.shape[1] < (taps - 1) * d:
        raise KernelError("the input convolution needs (taps - 1) x width float32 numbers of per-sequence state")
    return state.data_ptr(), state.stride(0), state.shape[0]


def input_conv(h: torch.Tensor, taps_w: torch.Tensor, state: Optional[torch.Tensor], step) -> torch.Tensor:
    """h + conv(h): a causal convolution per channel over the tokens of each sequence (`taps_w` [width, taps], the last tap the
    token's own), inputs older than the step from `state` ([slots + 1, (taps - 1) * width] float32, oldest first)."""
    lib = _bind()
    _cuda(h, "inputs")
    n, d = h.shape
    taps = taps_w.shape[1]
    if not h.is_contiguous() or tuple(taps_w.shape) != (d, taps) or not taps_w.is_contiguous():
        raise KernelError("input_conv: contiguous rows and taps [width, taps] are wanted")
    sp, sld, srows = _conv_state(state, taps, d)
    out = torch.empty_like(h)
    _check(lib, lib.gi_input_conv(out.data_ptr(), h.data_ptr(), _dt(h, "inputs"), taps_w.data_ptr(), _dt(taps_w, "taps"), sp, sld, srows,
                                  _i32(step.token_slots, "slots"), n, d, taps, _stream()))
    return out


def hyper_write(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, share: torch.Tensor, gate: Optional[torch.Tensor] = None,
                gate_bias: Optional[torch.Tensor] = None, h: Optional[torch.Tensor] = None, state: Optional[torch.Tensor] = None,
                taps: int = 1, step=None) -> None:
    """x[:, to] = sum_s mix[s, to] x[:, s] + share[to] * y * sigmoid(gate + gate_bias), all copies at once; with `state`, the
    last `taps` - 1 rows of `h` of every sequence become its convolution state."""
    lib = _bind()
    _cuda(x, "residual streams")
    streams = share.numel()
    n, d = y.shape
    if (x.dtype != torch.float32 or not x.is_contiguous() or tuple(x.shape) != (n, streams * d) or y.dtype != torch.float32
            or not y.is_contiguous() or tuple(mix.shape) != (streams, streams) or mix.dtype != torch.float32 or share.dtype != torch.float32
            or not mix.is_contiguous() or not share.is_contiguous()):
        raise KernelError("hyper_write: float32 streams [tokens, streams x width], rows [tokens, width], mix [streams, streams]")
    ref = gate if gate is not None else h
    if gate is not None and (tuple(gate.shape) != (n, d) or not gate.is_contiguous()):
        raise KernelError("hyper_write: the gate's rows must be contiguous [tokens, width]")
    if h is not None and (tuple(h.shape) != (n, d) or not h.is_contiguous() or (gate is not None and h.dtype != gate.dtype)):
        raise KernelError("hyper_write: the sublayer's inputs must be contiguous [tokens, width] rows of the gate's type")
    sp, sld, srows = _conv_state(state, taps, d) if h is not None else (None, 0, 0)
    _check(lib, lib.gi_hyper_write(
        x.data_ptr(), y.data_ptr(), gate.data_ptr() if gate is not None else None, gate_bias.data_ptr() if gate_bias is not None else None,
        _dt(ref, "rows") if ref is not None else F32, _dt(gate_bias, "gate bias") if gate_bias is not None else F32, mix.data_ptr(),
        share.data_ptr(), h.data_ptr() if h is not None else None, sp, sld, srows, _i32(step.token_slots, "slots"), n, streams, d,
        int(taps), _stream()))


def scale_rows(x: torch.Tensor, c: float) -> torch.Tensor:
    """x *= c in place (float32)."""
    lib = _bind()
    _cuda(x, "rows")
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_rows: contiguous float32 rows are wanted")
    _check(lib, lib.gi_scale_rows(x.data_ptr(), float(c), x.numel(), _stream()))
    return x


# ---- attention normed head by head, gated heads, clamped gated rows -----------------------------------------------------
def head_prepare(rows: torch.Tensor, out_dtype: torch.dtype, biases, norm_weights, norms, eps: float, table: Optional[torch.Tensor],
                 rot_dims: int, adjacent: bool, step, memory, n_heads: int, n_kv: int, head_dim: int, v_dim: int) -> torch.Tensor:
    """The queries of float32 projection rows [q | k | v | ...], prepared head by head, in `out_dtype`; keys and values go to
    the cache (`n_kv` 0: the rows hold queries only).  `biases` (q, k, v) and `norm_weights` (q, k) may hold None; `norms`
    (q, k, v) says which parts are divided by each head's root mean square."""
    lib = _bind()
    _cuda(rows, "projection rows")
    if rows.dtype != torch.float32 or rows.dim() != 2 or rows.stride(1) != 1:
        raise KernelError("head_prepare: float32 projection rows are wanted")
    n = rows.shape[0]
    if rows.shape[1] < (n_heads + n_kv) * head_dim + n_kv * v_dim:
        raise KernelError(f"projection rows of {rows.shape[1]} numbers cannot hold q, k and v")
    if n_kv:
        if memory.k is None or not memory.writes or memory.k.dtype != out_dtype or memory.v.dtype != out_dtype:
            raise KernelError("head_prepare: keys and values need a cache of the step's type that this entry writes")
        if (tuple(memory.k.shape[1:]) != (n_kv, 64, head_dim) or tuple(memory.v.shape[1:]) != (n_kv, 64, v_dim)
                or not memory.k.is_contiguous() or not memory.v.is_contiguous()):
            raise KernelError(f"cache pages must be contiguous [pages, {n_kv}, 64, {head_dim}] and [.., {v_dim}]")
    given = [t for t in tuple(biases) + tuple(norm_weights) if t is not None]
    w_dtype = given[0].dtype if given else torch.float32
    if any(t.dtype != w_dtype or not t.is_contiguous() for t in given):
        raise KernelError("head_prepare: biases and norm weights must share a type")
    ptr = lambda t: t.data_ptr() if t is not None else None
    q = torch.empty((n, n_heads * head_dim), dtype=out_dtype, device=rows.device)
    bt = memory.block_table if n_kv else None
    _check(lib, lib.gi_head_prepare(
        q.data_ptr(), q.stride(0), _DT[out_dtype], rows.data_ptr(), rows.stride(0), ptr(biases[0]), ptr(biases[1]), ptr(biases[2]),
        ptr(norm_weights[0]), ptr(norm_weights[1]), _DT[w_dtype], int(norms[0]), int(norms[1]), int(norms[2]), float(eps),
        table.data_ptr() if (table is not None and rot_dims) else None, int(rot_dims) // 2, int(adjacent),
        _i32(step.positions, "positions"), _i32(step.token_slots, "slots"), _i32(bt, "block table"), bt.shape[1] if bt is not None else 0,
        memory.k.data_ptr() if n_kv else None, memory.v.data_ptr() if n_kv else None, n, n_heads, n_kv, head_dim, v_dim, _stream()))
    return q


def head_gate(a: torch.Tensor, gates: torch.Tensor, n_heads: int, v_dim: int) -> torch.Tensor:
    """a[t, h, :] * sigmoid(gates[t, h]); `gates`: float32 rows with one number per head."""
    lib = _bind()
    _cuda(a, "attention output")
    n = a.shape[0]
    if not a.is_contiguous() or a.shape[1] != n_heads * v_dim or gates.dtype != torch.float32 or gates.stride(1) != 1 or gates.shape[1] < n_heads:
        raise KernelError("head_gate: contiguous heads and float32 gate rows are wanted")
    out = torch.empty_like(a)
    _check(lib, lib.gi_head_gate(out.data_ptr(), a.data_ptr(), _dt(a, "attention output"), gates.data_ptr(), gates.stride(0), n, n_heads,
                                 v_dim, _stream()))
    return out


def scaled_norm_gate(y: torch.Tensor, scale: Optional[torch.Tensor], gate: torch.Tensor, weight: torch.Tensor, n_heads: int,
                     v_dim: int, eps: float, out_dtype: torch.dtype) -> torch.Tensor:
    """Per head: v = y * scale[t, h]; v / sqrt(mean(v^2) + eps) * weight[h] * sigmoid(gate); y, gate float32 rows."""
    lib = _bind()
    _cuda(y, "read-outs")
    n = y.shape[0]
    if (y.dtype != torch.float32 or not y.is_contiguous() or y.shape[1] != n_heads * v_dim or gate.dtype != torch.float32
            or gate.stride(1) != 1 or gate.shape[1] < n_heads * v_dim or weight.numel() != n_heads * v_dim or not weight.is_contiguous()):
        raise KernelError("scaled_norm_gate: float32 read-outs and gate rows of heads x values numbers are wanted")
    if scale is not None and (scale.dtype != torch.float32 or tuple(scale.shape) != (n, n_heads) or not scale.is_contiguous()):
        raise KernelError("scaled_norm_gate: the scales must be contiguous float32 [tokens, heads]")
    out = torch.empty((n, n_heads * v_dim), dtype=out_dtype, device=y.device)
    _check(lib, lib.gi_scaled_norm_gate(out.data_ptr(), _DT[out_dtype], y.data_ptr(), scale.data_ptr() if scale is not None else None,
                                        gate.data_ptr(), gate.stride(0), weight.data_ptr(), _dt(weight, "norm weight"), n, n_heads, v_dim,
                                        float(eps), _stream()))
    return out


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float, interleaved: bool = False) -> torch.Tensor:
    """rows [gate | up] (or, `interleaved`, blocks [8 gate | 8 up]) -> min(gate, limit) * sigmoid(alpha * that) *
    (clamp(up, -limit, limit) + 1), in the rows' type."""
    lib = _bind()
    _cuda(gate_up, "gate/up rows")
    if gate_up.dim() != 2 or gate_up.stride(1) != 1 or gate_up.shape[1] % 2:
        raise KernelError("gate/up rows must be a [rows, 2 * width] matrix")
    n, f = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((n, f), dtype=gate_up.dtype, device=gate_up.device)
    _check(lib, lib.gi_clamped_glu_rows(out.data_ptr(), gate_up.data_ptr(), gate_up.stride(0), _dt(gate_up, "gate/up rows"), n, f,
                                        float(limit), float(alpha), int(interleaved), _stream()))
    return out


def clamped_glu_interleaved(h: torch.Tensor, w_interleaved: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """The clamped gated value of (W_gate h, W_up h) where `w_interleaved` holds gate and up rows in blocks [8 gate | 8 up]: in
    the products' epilogues (streamed for up to 64 rows, tcgen05 tiles above), or as a step of its own where neither product
    takes the operands or there is no positive limit."""
    lib = _bind()
    m, k = h.shape
    n = w_interleaved.shape[0]
    if limit and limit > 0 and n % 16 == 0:
        if skinny_ok(h, w_interleaved) and USE_STREAM and (n + 127) // 128 <= _STREAM_COUNTERS:
            out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=h.device)
            scratch, counters = _stream_buffers(h.device)
            _check(lib, lib.gi_gemm_stream_bf16_clamped(out.data_ptr(), h.data_ptr(), w_interleaved.data_ptr(), scratch.data_ptr(),
                                                        counters.data_ptr(), counters.numel(), m, n, k, h.stride(0), w_interleaved.stride(0),
                                                        out.stride(0), float(limit), float(alpha), _stream()))
            return out
        if tc_ok(h, w_interleaved) and m > SKINNY_MAX_ROWS:
            out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=h.device)
            _check(lib, lib.gi_gemm_tc_bf16_clamped(out.data_ptr(), h.data_ptr(), w_interleaved.data_ptr(), m, n, k, h.stride(0),
                                                    w_interleaved.stride(0), out.stride(0), int(TC_TILE_N), float(limit), float(alpha),
                                                    _stream()))
            return out
    return clamped_glu(linear(h, w_interleaved, out_dtype=h.dtype), limit, alpha, interleaved=True)


def moe_route_shares(h: torch.Tensor, w_router: torch.Tensor, top: int, correction: Optional[torch.Tensor], weight_scale: float):
    """(ids int32 [tokens, top], weights float32 [tokens, top]): shares = softmax over all experts' logits; the `top` largest of
    share + correction are chosen (the lower index on ties); weights = chosen shares / (their sum + 1e-20) * weight_scale."""
    lib = _bind()
    _cuda(h, "activations")
    n, width = h.shape
    experts = w_router.shape[0]
    if w_router.dim() != 2 or w_router.shape[1] != width or not w_router.is_contiguous():
        raise KernelError(f"router weights must be contiguous [experts, {width}]")
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != experts or not correction.is_contiguous()):
        raise KernelError("the router's correction must be float32, one number per expert")
    ids = torch.empty((n, top), dtype=torch.int32, device=h.device)
    wts = torch.empty((n, top), dtype=torch.float32, device=h.device)
    _check(lib, lib.gi_moe_route_shares(ids.data_ptr(), wts.data_ptr(), None, h.data_ptr(), _dt(h, "activations"), _rows(h, "activations"),
                                        w_router.data_ptr(), None, _dt(w_router, "router weights"), n, width, experts, int(top), 2,
                                        correction.data_ptr() if correction is not None else None, float(weight_scale), _stream()))
    return ids, wts
