"""Typed Python wrappers of the CUDA entry points in ``csrc/``.

Every wrapper checks what the kernel cannot (device, dtype, contiguity, sizes it
refuses), passes raw pointers and the current CUDA stream through the C ABI and
raises :class:`KernelError` on a non-zero status.  There is no CPU path: a call
with a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional, Tuple

import torch

from .csrc import builder as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_launches = 0   # kernels launched through these wrappers since the last reset


class KernelError(RuntimeError):
    """A kernel refused its arguments or the launch failed."""


def launches() -> int:
    return _launches


def reset_launches() -> None:
    global _launches
    _launches = 0


def reset_launches_by(n: int) -> None:
    """Take back ``n`` counted launches (calls recorded into a CUDA graph launch nothing)."""
    global _launches
    _launches -= n


def code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


_PROTOTYPES = {
    "elementwise": {
        "zlm_embed": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_void_p],
        "zlm_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_float,
                        c_void_p],
        "zlm_gated_act": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
        "zlm_rmsnorm_strided": [c_void_p, c_long, c_void_p, c_int, c_void_p, c_int, c_long, c_int, c_int, c_int, c_float,
                                c_float, c_void_p],
        "zlm_norm_add_norm": [c_void_p, c_void_p, c_float, c_float, c_void_p, c_void_p, c_float, c_float, c_int, c_void_p,
                              c_int, c_int, c_int, c_void_p],
        "zlm_norm_add_scaled": [c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                                c_void_p],
        "zlm_sum_norm": [c_void_p, c_void_p, c_int, c_float, c_float, c_float, c_void_p, c_void_p, c_int, c_int, c_int,
                         c_void_p],
        "zlm_unary_act": [c_void_p, c_void_p, c_int, c_long, c_int, c_void_p],
        "zlm_sigmoid_mul": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_void_p],
        "zlm_add_row": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "zlm_convert_rows": [c_void_p, c_int, c_long, c_void_p, c_int, c_long, c_int, c_int, c_void_p],
        "zlm_gate_heads": [c_void_p, c_long, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int, c_float, c_void_p],
        "zlm_norm_gate": [c_void_p, c_long, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_float,
                          c_float, c_void_p],
        "zlm_head_norm_gate": [c_void_p, c_long, c_void_p, c_void_p, c_long, c_void_p, c_long, c_int, c_int, c_int, c_int,
                               c_float, c_int, c_float, c_void_p],
        "zlm_scale": [c_void_p, c_long, c_float, c_void_p],
        "zlm_add": [c_void_p, c_void_p, c_long, c_void_p],
        "zlm_convert": [c_void_p, c_int, c_void_p, c_int, c_long, c_void_p],
        "zlm_fill_normal": [c_void_p, c_int, c_long, ctypes.c_ulonglong, c_float, c_float, c_void_p],
    },
    "block_linear": {
        "zlm_block_linear": [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_void_p, c_int, c_long, c_int, c_int,
                             c_int, c_int, c_int, c_void_p, c_long, c_void_p],
    },
    "recurrent": {
        "zlm_causal_conv": [c_void_p, c_int, c_long, c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "zlm_selective_scan": [c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p, c_long, c_void_p, c_long,
                               c_void_p, c_void_p, c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                               c_int, c_int, c_void_p],
        "zlm_gated_scan": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_long, c_void_p, c_long, c_void_p, c_float,
                           c_void_p, c_long, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "linear_attention": {
        "zlm_linear_attention_chunk": [],
        "zlm_linear_attention_segment": [],
        "zlm_linear_attention_segments": [c_int, c_int],
        "zlm_decayed_linear_attention": [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                         c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_int, c_void_p, c_void_p, c_long, c_void_p],
    },
    "moe": {
        "zlm_moe_route": [c_void_p, c_long, c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                          c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p],
        "zlm_moe_max_tiles_scratch": [c_int, c_int],
        "zlm_moe_group": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p],
        "zlm_moe_grouped": [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_long, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p],
        "zlm_moe_gather": [c_void_p, c_int, c_long, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
        "zlm_moe_combine": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_long, c_void_p, c_void_p,
                            c_long, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_generic": {
        "zlm_gemm_generic": [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int,
                             c_int, c_long, c_long, c_long, c_void_p],
    },
    "attention": {
        "zlm_rope_store": [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                           c_void_p, c_int, c_void_p, c_void_p, c_int, c_long, c_void_p],
        "zlm_rope_norm_store": [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_float, c_int,
                                c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                c_int, c_long, c_void_p],
        "zlm_attention_general": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                  c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_long,
                                  c_int, c_void_p, c_long, c_void_p],
        "zlm_qk_prep": [c_void_p, c_int, c_long, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int,
                        c_int, c_float, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                        c_void_p, c_int, c_long, c_void_p],
        "zlm_attention_general_scratch": [c_int, c_int, c_int, c_int, c_int],
    },
    "attention_tc": {
        "zlm_attention_decode": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_int,
                                 c_void_p, c_void_p, c_long, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int,
                                 c_void_p, c_void_p, c_void_p],
        "zlm_attention_decode_flat": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p,
                                      c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_int, c_void_p,
                                      c_void_p, c_long, c_int, c_int, c_int, c_void_p, c_void_p, c_long, c_void_p],
        "zlm_attention_decode_flat_blocks": [c_int, c_int, c_int, c_int],
        "zlm_attention_decode_flat_scratch": [c_int, c_int, c_int, c_int, c_int],
        "zlm_attention_prefill": [c_void_p, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int,
                                  c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_long, c_int, c_void_p],
        "zlm_attention_tc_status": [c_void_p],
        "zlm_attention_tc_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "attention_fmha": {
        "zlm_attention_prefill_fmha": [c_void_p, c_long, c_long, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
                                       c_float, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                       c_void_p, c_long, c_int, c_void_p],
        "zlm_attention_fmha_status": [c_void_p],
        "zlm_attention_fmha_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "gemm_tc": {
        "zlm_gemm_tc": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                        c_long, c_long, c_long, c_int, c_void_p],
        "zlm_gemm_tc_norm": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_long, c_long, c_long, c_int, c_void_p, c_int, c_float, c_void_p, c_long, c_void_p,
                             c_void_p, c_void_p, c_int, c_float, c_void_p],
        "zlm_gemm_tc_unary": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_long, c_long, c_long,
                              c_int, c_void_p],
        "zlm_gemm_tc_swish_clamped": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_long, c_long,
                                      c_long, c_float, c_float, c_void_p],
        "zlm_gemm_tc_groups": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_long, c_long,
                               c_long, c_long, c_float, c_float, c_void_p, c_void_p],
        "zlm_gemm_tc_status": [c_void_p],
        "zlm_gemm_tc_wait_selftest": [c_int, c_void_p, c_void_p],
    },
    "sampling": {
        "zlm_sample_parts_scratch": [c_int],
        "zlm_sample_parts": [c_void_p, c_int, c_int, c_long, c_float, c_int, c_float, c_float, c_float, c_float, c_void_p,
                             c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_long, c_void_p],
        "zlm_argmax": [c_void_p, c_int, c_int, c_long, c_void_p, c_void_p],
        "zlm_sample": [c_void_p, c_int, c_int, c_long, c_float, c_int, c_float, c_float, c_float, c_float, c_void_p,
                       c_int, c_void_p, c_void_p, c_void_p],
    },
}
_functions = {}


def _fn(library: str, name: str):
    f = _functions.get(name)
    if f is None:
        lib = _build.load(library)
        f = getattr(lib, name)
        f.argtypes = _PROTOTYPES[library][name]
        f.restype = c_long if name.endswith("_scratch") else c_int
        _functions[name] = f
    return f


def require(libraries) -> None:
    """Compile (if need be) and load the named kernel libraries, several at a time."""
    _build.build(list(libraries))
    for lib in libraries:
        _build.load(lib)


_STATUS = {-1: "bad argument", -2: "unsupported size or type", -3: "scratch memory too small"}


def _check(status: int, what: str) -> None:
    global _launches
    if status == 0:
        _launches += 1
        return
    if status < 0:
        raise KernelError(f"{what}: {_STATUS.get(status, 'error %d' % status)}")
    raise KernelError(f"{what}: CUDA error {status}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# The handle of the current stream of the current device.  torch.cuda.current_stream() builds a Stream object
# and resolves the device through several Python layers (a few microseconds a call, once per launch); the raw
# getter answers the same question in a fraction of that.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    if _raw_stream is not None and _current_device is not None:
        return _raw_stream(_current_device())
    return torch.cuda.current_stream().cuda_stream


def _cuda(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")


# ------------------------------------------------------------------ elementwise
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[t, :] = float(table[tokens[t], :]) * scale;  out is float32 [T, d]."""
    _cuda(table, "table"); _cuda(tokens, "tokens", torch.int32); _cuda(out, "out", torch.float32)
    T, d = out.shape
    if table.shape[1] != d or tokens.numel() < T:
        raise KernelError("embed: shapes do not match")
    _check(_fn("elementwise", "zlm_embed")(table.data_ptr(), code(table.dtype), tokens.data_ptr(), out.data_ptr(),
                                           T, d, scale, _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, weight_offset: float = 0.0) -> None:
    """out[r] = x[rows[r] or r] * rsqrt(mean(x^2) + eps) * (weight + weight_offset); x is float32."""
    _cuda(x, "x", torch.float32); _cuda(weight, "weight"); _cuda(out, "out")
    n, d = out.shape
    if x.shape[1] != d or weight.numel() != d:
        raise KernelError("rmsnorm: shapes do not match")
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
        if rows.numel() < n:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif x.shape[0] < n:
        raise KernelError("rmsnorm: fewer input rows than output rows")
    _check(_fn("elementwise", "zlm_rmsnorm")(x.data_ptr(), weight.data_ptr(), code(weight.dtype), out.data_ptr(),
                                             code(out.dtype), _ptr(rows), n, d, eps, weight_offset, _stream()),
           "rmsnorm")


ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "swish_clamped": 2}


def gated_act(gu: torch.Tensor, out: torch.Tensor, activation: str = "silu", interleaved: bool = False,
              limit: float = 0.0, slope: float = 1.0) -> None:
    """out[t, j] = act(gate) * up for gu of shape [T, 2I]: gate j, up j in columns (j, I + j), or in columns
    (2j, 2j + 1) when ``interleaved``.  "swish_clamped": g = min(gate, limit), u = clamp(up, -limit, limit),
    out = g * sigmoid(slope * g) * (u + 1)."""
    _cuda(gu, "gu"); _cuda(out, "out", gu.dtype)
    T, I = out.shape
    if gu.shape != (T, 2 * I):
        raise KernelError("gated_act: gu must be [T, 2*I]")
    kind = ACTIVATIONS.get(activation)
    if kind is None:
        raise KernelError(f"gated_act: activation {activation!r} is not known ({', '.join(ACTIVATIONS)})")
    _check(_fn("elementwise", "zlm_gated_act")(gu.data_ptr(), out.data_ptr(), code(gu.dtype), T, I, kind,
                                               int(interleaved), float(limit), float(slope), _stream()), "gated_act")


def _rows(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be on a CUDA device (there is no CPU path)")
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be a matrix with unit column stride")


def _row_stride(t: torch.Tensor) -> int:
    return t.stride(0) if t.shape[0] > 1 else t.shape[1]


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, add: bool = False,
                 weight_offset: float = 0.0) -> None:
    """out[r] = (or += with ``add``) x[r] * rsqrt(mean(x[r]^2) + eps) * (weight + weight_offset).  x is float32;
    x and out may be column slices of wider matrices (rows with a stride of their own); ``add`` needs a float32
    out and is how a norm behind a sublayer is summed into the residual stream."""
    _rows(x, "x"); _rows(out, "out"); _cuda(weight, "weight")
    n, d = x.shape
    if x.dtype != torch.float32 or out.shape != (n, d) or weight.numel() != d or (add and out.dtype != torch.float32):
        raise KernelError("rmsnorm_rows: x must be float32, out of its shape (float32 to add into), weight of its width")
    _check(_fn("elementwise", "zlm_rmsnorm_strided")(
        x.data_ptr(), _row_stride(x), weight.data_ptr(), code(weight.dtype), out.data_ptr(), code(out.dtype),
        _row_stride(out), int(add), n, d, eps, weight_offset, _stream()), "rmsnorm_rows")


def norm_add_norm(branch: torch.Tensor, w1: torch.Tensor, eps1: float, x: torch.Tensor, w2: torch.Tensor, eps2: float,
                  h: torch.Tensor, off1: float = 0.0, off2: float = 0.0) -> bool:
    """x += rmsnorm(branch; w1, eps1) and h = rmsnorm(x; w2, eps2) in one pass over each row: the norm behind a
    sublayer, the residual sum and the norm before the next sublayer.  branch and x float32 [n, d] contiguous; h
    [n, d] in its own type; w1 and w2 of one type.  False, having done nothing, for rows too long for the kernel's
    shared memory."""
    _cuda(branch, "branch", torch.float32); _cuda(x, "x", torch.float32); _cuda(h, "h"); _cuda(w1, "w1"); _cuda(w2, "w2", w1.dtype)
    n, d = x.shape
    if branch.shape != (n, d) or h.shape != (n, d) or w1.numel() != d or w2.numel() != d:
        raise KernelError("norm_add_norm: shapes do not match")
    status = _fn("elementwise", "zlm_norm_add_norm")(branch.data_ptr(), w1.data_ptr(), float(off1), float(eps1), x.data_ptr(),
                                                     w2.data_ptr(), float(off2), float(eps2), code(w1.dtype), h.data_ptr(),
                                                     code(h.dtype), n, d, _stream())
    if status == -2:
        return False
    _check(status, "norm_add_norm")
    return True


def norm_add_scaled(branch: torch.Tensor, weight: torch.Tensor, eps: float, mult: float, x: torch.Tensor,
                    h: Optional[torch.Tensor] = None, weight_offset: float = 0.0) -> None:
    """x += mult * branch / sqrt(mean(branch^2) + eps) * (weight + weight_offset), row by row, and with ``h`` also
    h = x (the new rows, in h's type): the norm behind a sublayer whose input is the residual stream itself.
    branch and x float32 [n, d] contiguous."""
    _cuda(branch, "branch", torch.float32); _cuda(x, "x", torch.float32); _cuda(weight, "weight")
    n, d = x.shape
    if branch.shape != (n, d) or weight.numel() != d:
        raise KernelError("norm_add_scaled: shapes do not match")
    if h is not None:
        _cuda(h, "h")
        if h.shape != (n, d):
            raise KernelError("norm_add_scaled: h must have the shape of x")
    _check(_fn("elementwise", "zlm_norm_add_scaled")(
        branch.data_ptr(), weight.data_ptr(), code(weight.dtype), float(weight_offset), float(eps), float(mult),
        x.data_ptr(), _ptr(h), code(h.dtype) if h is not None else F32, n, d, _stream()), "norm_add_scaled")


def sum_norm(branch: torch.Tensor, weight: torch.Tensor, eps: float, alpha: float, x: torch.Tensor,
             h: Optional[torch.Tensor] = None, weight_offset: float = 0.0) -> None:
    """x = s / sqrt(mean(s^2) + eps) * (weight + weight_offset) with s = alpha * x + branch, row by row and in place,
    and with ``h`` also h = x (the new rows, in h's type): the norm behind a sum, which norms the residual stream
    itself.  branch and x float32 [n, d] contiguous."""
    _cuda(branch, "branch", torch.float32); _cuda(x, "x", torch.float32); _cuda(weight, "weight")
    n, d = x.shape
    if branch.shape != (n, d) or weight.numel() != d:
        raise KernelError("sum_norm: shapes do not match")
    if h is not None:
        _cuda(h, "h")
        if h.shape != (n, d):
            raise KernelError("sum_norm: h must have the shape of x")
    _check(_fn("elementwise", "zlm_sum_norm")(
        branch.data_ptr(), weight.data_ptr(), code(weight.dtype), float(weight_offset), float(eps), float(alpha),
        x.data_ptr(), _ptr(h), code(h.dtype) if h is not None else F32, n, d, _stream()), "sum_norm")


UNARY_ACTIVATIONS = {"relu2": 0, "gelu": 1}


def unary_act(x: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = act(x) element by element (out may be x); "relu2": max(x, 0)^2, "gelu": x (1 + erf(x / sqrt 2)) / 2."""
    _cuda(x, "x"); _cuda(out, "out", x.dtype)
    if activation not in UNARY_ACTIVATIONS or out.shape != x.shape:
        raise KernelError(f"unary_act: activation {activation!r} is not known, or the shapes differ")
    _check(_fn("elementwise", "zlm_unary_act")(x.data_ptr(), out.data_ptr(), code(x.dtype), x.numel(),
                                               UNARY_ACTIVATIONS[activation], _stream()), "unary_act")


def sigmoid_mul(a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> None:
    """out = a * sigmoid(gate); all [T, n] of one type, each may be a column slice of a wider matrix."""
    _rows(a, "a"); _rows(gate, "gate"); _rows(out, "out")
    if a.shape != gate.shape or a.shape != out.shape or a.dtype != gate.dtype or a.dtype != out.dtype:
        raise KernelError("sigmoid_mul: shapes or types do not match")
    T, n = a.shape
    _check(_fn("elementwise", "zlm_sigmoid_mul")(a.data_ptr(), _row_stride(a), gate.data_ptr(), _row_stride(gate),
                                                 out.data_ptr(), _row_stride(out), code(a.dtype), T, n, _stream()),
           "sigmoid_mul")


def convert_rows(src: torch.Tensor, out: torch.Tensor) -> None:
    """out = src, converted to out's type; both [T, n], each may be a column slice of a wider matrix."""
    _rows(src, "src"); _rows(out, "out")
    if src.shape != out.shape:
        raise KernelError("convert_rows: the shapes differ")
    _check(_fn("elementwise", "zlm_convert_rows")(src.data_ptr(), code(src.dtype), _row_stride(src), out.data_ptr(),
                                                  code(out.dtype), _row_stride(out), src.shape[0], src.shape[1], _stream()),
           "convert_rows")


def gate_heads(a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, n_heads: int, mult: float = 1.0) -> None:
    """out[t, h, :] = a[t, h, :] * sigmoid(gate[t, h]) * mult: one gate a head.  a and out [T, n_heads * n], gate
    [T, n_heads], all of one type; each may be a column slice of a wider matrix (out may be a)."""
    _rows(a, "a"); _rows(gate, "gate"); _rows(out, "out")
    T, width = a.shape
    if (n_heads <= 0 or width % n_heads or gate.shape != (T, n_heads) or out.shape != a.shape or a.dtype != gate.dtype
            or a.dtype != out.dtype):
        raise KernelError("gate_heads: a and out must be [T, heads * n] and the gate [T, heads], of one type")
    _check(_fn("elementwise", "zlm_gate_heads")(a.data_ptr(), _row_stride(a), gate.data_ptr(), _row_stride(gate),
                                                out.data_ptr(), _row_stride(out), code(a.dtype), T, n_heads,
                                                width // n_heads, float(mult), _stream()), "gate_heads")


def norm_gate(x: torch.Tensor, weight: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, eps: float,
              mult: float = 1.0) -> None:
    """out[r] = x[r] / sqrt(mean(x[r]^2) + eps) * weight * sigmoid(gate[r]) * mult (no gate: without the sigmoid).
    x float32 rows, weight float32 [d], gate and out rows of one type; each may be a column slice."""
    _rows(x, "x"); _rows(out, "out"); _cuda(weight, "weight", torch.float32)
    n, d = x.shape
    if x.dtype != torch.float32 or out.shape != (n, d) or weight.numel() != d:
        raise KernelError("norm_gate: x must be float32, out of its shape, weight of its width")
    g_stride = 0
    if gate is not None:
        _rows(gate, "gate")
        if gate.shape != (n, d) or gate.dtype != out.dtype:
            raise KernelError("norm_gate: the gate must have out's shape and type")
        g_stride = _row_stride(gate)
    _check(_fn("elementwise", "zlm_norm_gate")(x.data_ptr(), _row_stride(x), weight.data_ptr(), _ptr(gate), g_stride,
                                               out.data_ptr(), _row_stride(out), code(out.dtype), n, d, float(eps),
                                               float(mult), _stream()), "norm_gate")


HEAD_GATES = {None: 0, "sigmoid": 1, "silu": 2}


def head_norm_gate(x: torch.Tensor, weight: Optional[torch.Tensor], gate: Optional[torch.Tensor], out: torch.Tensor,
                   n_heads: int, eps: float, gate_kind: Optional[str] = None, mult: float = 1.0) -> None:
    """Every head of a row normed by itself, with a gate: x float32 [T, n_heads * hd]; out[t, h, :] = x[t, h, :] /
    sqrt(mean(x[t, h, :]^2) + eps) * weight[h, :] * act(gate[t, h, :]) * mult, in out's type.  ``weight`` (float32,
    n_heads * hd) and ``gate`` (out's type) may be None; ``gate_kind``: "sigmoid" or "silu" (g * sigmoid(g)).
    x, gate and out may be column slices."""
    _rows(x, "x"); _rows(out, "out")
    T, d = x.shape
    if gate_kind not in HEAD_GATES:
        raise KernelError(f"head_norm_gate: gate {gate_kind!r} is not known (sigmoid, silu)")
    if x.dtype != torch.float32 or out.shape != (T, d) or n_heads <= 0 or d % n_heads:
        raise KernelError("head_norm_gate: x must be float32 rows of whole heads and out of its shape")
    if weight is not None:
        _cuda(weight, "weight", torch.float32)
        if weight.numel() != d:
            raise KernelError("head_norm_gate: the weight must hold one number for each element of a row")
    if (gate is None) != (gate_kind is None):
        raise KernelError("head_norm_gate: a gate and its kind go together")
    if gate is not None:
        _rows(gate, "gate")
        if gate.dtype != out.dtype or gate.shape != (T, d):
            raise KernelError("head_norm_gate: the gate must have out's type and shape")
    _check(_fn("elementwise", "zlm_head_norm_gate")(
        x.data_ptr(), _row_stride(x), _ptr(weight), _ptr(gate), _row_stride(gate) if gate is not None else 0,
        out.data_ptr(), _row_stride(out), code(out.dtype), T, n_heads, d // n_heads, float(eps), HEAD_GATES[gate_kind],
        float(mult), _stream()), "head_norm_gate")


def add_row(x: torch.Tensor, row: torch.Tensor) -> None:
    """x[t, :] += row for every t; x is float32 [T, d], row holds d elements."""
    _cuda(x, "x", torch.float32); _cuda(row, "row")
    if x.dim() != 2 or row.numel() != x.shape[1]:
        raise KernelError("add_row: the row must be as wide as x")
    _check(_fn("elementwise", "zlm_add_row")(x.data_ptr(), row.data_ptr(), code(row.dtype), x.shape[0], x.shape[1],
                                             _stream()), "add_row")


def scale_(x: torch.Tensor, factor: float) -> None:
    _cuda(x, "x", torch.float32)
    _check(_fn("elementwise", "zlm_scale")(x.data_ptr(), x.numel(), float(factor), _stream()), "scale_")


# ---------------------------------------------------------- block-diagonal product
BLOCK_EPILOGUES = {None: 0, "sigmoid": 1, "sigmoid_gate": 2}


def block_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 epilogue: Optional[str] = None, gate: Optional[torch.Tensor] = None) -> None:
    """out[t, b*N + n] = epi(sum_k x[t, b*K + k] * w[b, n, k] + bias[b*N + n]) for w of shape [B, N, K]: part b of
    a row goes through a matrix of its own (a product per attention head, block-diagonal gates).  ``epilogue``:
    None, "sigmoid", or "sigmoid_gate" (the result times sigmoid(gate[t, b*N + n]), gate float32).  x, out and
    gate may be column slices of wider matrices.  bias is float32."""
    _rows(x, "x"); _rows(out, "out"); _cuda(w, "w")
    if w.dim() != 3:
        raise KernelError("block_linear: w must be [B, N, K]")
    B, N, K = w.shape
    T = x.shape[0]
    if x.shape[1] != B * K or out.shape != (T, B * N):
        raise KernelError(f"block_linear: shapes do not match: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if bias is not None:
        _cuda(bias, "bias", torch.float32)
        if bias.numel() != B * N:
            raise KernelError("block_linear: bias length does not match")
    if epilogue not in BLOCK_EPILOGUES:
        raise KernelError(f"block_linear: epilogue {epilogue!r} is not known")
    gate_stride = 0
    if epilogue == "sigmoid_gate":
        if gate is None:
            raise KernelError("block_linear: the gated epilogue needs a gate")
        _rows(gate, "gate")
        if gate.dtype != torch.float32 or gate.shape != (T, B * N):
            raise KernelError("block_linear: the gate must be float32 of the output's shape")
        gate_stride = _row_stride(gate)
    status = _fn("block_linear", "zlm_block_linear")(
        x.data_ptr(), code(x.dtype), _row_stride(x), w.data_ptr(), code(w.dtype), _ptr(bias), out.data_ptr(),
        code(out.dtype), _row_stride(out), T, B, N, K, BLOCK_EPILOGUES[epilogue], _ptr(gate), gate_stride, _stream())
    _check(status, "block_linear")


# ------------------------------------------------------------------- recurrence
def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor, state: torch.Tensor, step, u: torch.Tensor,
                activation: Optional[str] = None) -> None:
    """u[t, c] = act(bias[c] + sum_j taps[K-1-j, c] * x[t-j, c]) over each sequence of the step; the inputs before the
    step are rows 0..K-2 of the sequence's state [slots, rows >= K - 1, C] (float32; zero for a new sequence).  taps
    [K, C] (one row per tap, the current token's last) and bias [C] are float32; x may be a column slice.
    ``activation``: None or "silu"."""
    _rows(x, "x"); _cuda(u, "u", x.dtype); _cuda(taps, "taps", torch.float32); _cuda(bias, "bias", torch.float32)
    _cuda(state, "state", torch.float32)
    T, C = x.shape
    K = taps.shape[0]
    if (taps.shape != (K, C) or bias.numel() != C or u.shape != (T, C) or state.dim() != 3 or state.shape[2] != C
            or state.shape[1] < K - 1):
        raise KernelError("causal_conv: shapes do not match")
    if activation not in (None, "silu"):
        raise KernelError(f"causal_conv: activation {activation!r} is not known (silu)")
    _check(_fn("recurrent", "zlm_causal_conv")(
        x.data_ptr(), code(x.dtype), _row_stride(x), taps.data_ptr(), bias.data_ptr(), state.data_ptr(), state.stride(0),
        step.seq_of_token.data_ptr(), step.cu_seqlens.data_ptr(), step.slots.data_ptr(), u.data_ptr(), T, C, K,
        1 if activation == "silu" else 0, _stream()), "causal_conv")


def selective_scan(u: torch.Tensor, dt_pre: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, n_states: int,
                   z: torch.Tensor, x: torch.Tensor, a_t: torch.Tensor, d: torch.Tensor, taps: int, state: torch.Tensor,
                   step, out: torch.Tensor) -> None:
    """The selective scan of a state-space layer over the step's sequences.  Per channel c, with N states:
    dt = softplus(dt_pre[t, c]); S[n] <- exp(dt A[c, n]) S[n] + dt u[t, c] B_t[n]; y = sum_n S[n] C_t[n] + d[c] u[t, c];
    out[t, c] = y * silu(z[t, c]).  ``u`` [T, C] (the convolution's output), ``dt_pre`` float32 [T, C], B_t and C_t the
    ``n_states`` columns of ``bc``'s rows from ``b_off`` and ``c_off`` on, ``z`` and ``x`` [T, C] (column slices
    allowed; x: the convolution's inputs), ``a_t`` float32 [N, C] (A transposed and multiplied by log2(e): the kernel
    takes exp2), ``d`` float32 [C].  The state
    [slots, taps - 1 + N, C] float32 holds the convolution's last inputs in its first taps - 1 rows and S behind them;
    both are left as they stand after the step's last token."""
    _cuda(u, "u"); _cuda(dt_pre, "dt_pre", torch.float32); _rows(bc, "bc"); _rows(z, "z"); _rows(x, "x")
    _cuda(a_t, "a_t", torch.float32); _cuda(d, "d", torch.float32); _cuda(state, "state", torch.float32)
    _cuda(out, "out", u.dtype)
    T, C = u.shape
    N = int(n_states)
    if (dt_pre.shape != (T, C) or out.shape != (T, C) or z.shape != (T, C) or x.shape != (T, C) or a_t.shape != (N, C)
            or d.numel() != C or bc.shape[0] != T or max(b_off, c_off) + N > bc.shape[1] or min(b_off, c_off) < 0
            or tuple(state.shape[1:]) != (taps - 1 + N, C) or any(t.dtype != u.dtype for t in (bc, z, x))):
        raise KernelError("selective_scan: shapes or types do not match")
    _check(_fn("recurrent", "zlm_selective_scan")(
        u.data_ptr(), code(u.dtype), dt_pre.data_ptr(), bc.data_ptr(), _row_stride(bc), int(b_off), int(c_off),
        z.data_ptr(), _row_stride(z), x.data_ptr(), _row_stride(x), a_t.data_ptr(), d.data_ptr(), state.data_ptr(),
        state.stride(0), step.cu_seqlens.data_ptr(), step.slots.data_ptr(), out.data_ptr(), step.n_seqs, step.max_new, C,
        N, int(taps), _stream()), "selective_scan")


def gated_scan(u: torch.Tensor, gates: torch.Tensor, gate_block: int, y: torch.Tensor, x: torch.Tensor,
               lam: torch.Tensor, rate: float, state: torch.Tensor, step, out: torch.Tensor) -> None:
    """The recurrence S_t = a_t S_{t-1} + sqrt(1 - a_t^2) i_t u_t with a_t = exp(-rate r_t softplus(lam)), carried in
    row K-1 of the sequence's state, out_t = S_t * gelu_tanh(y_t); it also leaves the last K-1 rows of x (the
    convolution's inputs) in rows 0..K-2 of the state.  gates: float32 [T, 2C], per block of ``gate_block``
    channels first r then i."""
    _cuda(u, "u"); _cuda(out, "out", u.dtype); _cuda(gates, "gates", torch.float32); _cuda(lam, "lam", torch.float32)
    _rows(y, "y"); _rows(x, "x"); _cuda(state, "state", torch.float32)
    T, C = u.shape
    K = state.shape[1]
    if (gates.shape != (T, 2 * C) or y.shape != (T, C) or x.shape != (T, C) or out.shape != (T, C) or lam.numel() != C
            or state.shape[2] != C or y.dtype != u.dtype or x.dtype != u.dtype):
        raise KernelError("gated_scan: shapes or types do not match")
    _check(_fn("recurrent", "zlm_gated_scan")(
        u.data_ptr(), code(u.dtype), gates.data_ptr(), int(gate_block), y.data_ptr(), _row_stride(y), x.data_ptr(),
        _row_stride(x), lam.data_ptr(), float(rate), state.data_ptr(), state.stride(0), step.cu_seqlens.data_ptr(),
        step.slots.data_ptr(), out.data_ptr(), step.n_seqs, step.max_new, C, K, _stream()), "gated_scan")


# ------------------------------------------------------------ mixture of experts
def moe_route(z: Optional[torch.Tensor], correction: Optional[torch.Tensor], top: int, n_groups: int, keep_groups: int,
              group_best: int, ids: torch.Tensor, weights: torch.Tensor, softmax_scores=False,
              renormalize: bool = False, h: Optional[torch.Tensor] = None, router: Optional[torch.Tensor] = None,
              weight_scale: float = 1.0, n_extra: int = 0, extra_out: Optional[torch.Tensor] = None) -> None:
    """Per token: scores = sigmoid(z) (or softmax), chosen by score + correction within the ``keep_groups`` groups
    whose ``group_best`` best choice scores sum highest; ids int32 [T, top], weights float32 [T, top] (the scores
    of the chosen, divided by their sum with ``renormalize``).  ``z``: float32 [T, E] router logits; or None with
    ``h`` [T, d] and ``router`` [E, d] of one type: the logits are then taken inside (float32 sums), which is what
    a step of few tokens wants.  ``softmax_scores`` = 2: the experts with the largest logits are chosen and their
    weights are the softmax over the chosen logits alone (no correction, no groups).  The weights leave multiplied by
    ``weight_scale``.  ``n_extra``: the last columns of ``z`` (or rows of ``router``) are not experts but further
    products of the same rows; with ``router`` their sums are left in ``extra_out`` float32 [T, n_extra]."""
    _cuda(ids, "ids", torch.int32); _cuda(weights, "weights", torch.float32)
    d, h_stride, h_code, z_stride = 0, 0, F32, 0
    if z is not None:
        _rows(z, "z")
        if z.dtype != torch.float32:
            raise KernelError("moe_route: the logits must be float32")
        T, E = z.shape[0], z.shape[1] - n_extra
        z_stride = _row_stride(z)
    else:
        if h is None or router is None:
            raise KernelError("moe_route: the logits, or the rows and the router's matrix, are needed")
        _rows(h, "h"); _cuda(router, "router", h.dtype)
        T, d = h.shape
        E = router.shape[0] - n_extra
        if router.shape != (E + n_extra, d) or E <= 0:
            raise KernelError("moe_route: the router's matrix must be [E, d]")
        h_stride, h_code = _row_stride(h), code(h.dtype)
        if n_extra:
            _cuda(extra_out, "extra_out", torch.float32)
            if extra_out.shape != (T, n_extra):
                raise KernelError("moe_route: the further products go to a float32 [T, n_extra]")
    if correction is not None:
        _cuda(correction, "correction", torch.float32)
        if correction.numel() != E:
            raise KernelError("moe_route: one correction per expert is needed")
    if ids.shape != (T, top) or weights.shape != (T, top):
        raise KernelError("moe_route: ids and weights must be [T, top]")
    _check(_fn("moe", "zlm_moe_route")(_ptr(z), z_stride, _ptr(h), h_code, h_stride, _ptr(router), d, _ptr(correction), T, E,
                                       top, n_groups, keep_groups, group_best, int(softmax_scores), int(renormalize),
                                       float(weight_scale), int(n_extra), _ptr(extra_out) if z is None else None,
                                       ids.data_ptr(), weights.data_ptr(), _stream()), "moe_route")


def moe_max_tiles(n_pairs: int, n_experts: int) -> int:
    return int(_fn("moe", "zlm_moe_max_tiles_scratch")(n_pairs, n_experts))


def moe_group(ids: torch.Tensor, n_experts: int, offs: torch.Tensor, order: torch.Tensor, place: torch.Tensor,
              tile_expert: torch.Tensor, tile_row: torch.Tensor, n_tiles: torch.Tensor,
              n_real: Optional[int] = None) -> None:
    """Group the (token, choice) pairs by expert: ``order`` lists the pairs expert by expert, ``place`` is its
    inverse (where pair p stands in ``order``), ``offs`` [E + 1] says where each expert's run starts, and the runs
    are cut into tiles of rows for the grouped products.  ``n_real``: the experts from there on are identity experts,
    whose runs get no tiles (they have no product)."""
    for t, n in ((ids, "ids"), (offs, "offs"), (order, "order"), (place, "place"), (tile_expert, "tile_expert"),
                 (tile_row, "tile_row"), (n_tiles, "n_tiles")):
        _cuda(t, n, torch.int32)
    P = ids.numel()
    need = moe_max_tiles(P, n_experts)
    if (offs.numel() < n_experts + 1 or order.numel() < P or place.numel() < P or tile_expert.numel() < need
            or tile_row.numel() < need):
        raise KernelError("moe_group: an output is too short")
    _check(_fn("moe", "zlm_moe_group")(ids.data_ptr(), P, n_experts, n_experts if n_real is None else int(n_real),
                                       offs.data_ptr(), order.data_ptr(), place.data_ptr(),
                                       tile_expert.data_ptr(), tile_row.data_ptr(), n_tiles.data_ptr(), _stream()),
           "moe_group")


def moe_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, glu: bool, n_pairs: int, top: int,
                offs: torch.Tensor, order: torch.Tensor, tile_expert: torch.Tensor, tile_row: torch.Tensor,
                n_tiles: torch.Tensor, interleaved: bool = False, skinny: bool = False, limit: float = 0.0,
                slope: float = 1.0) -> None:
    """The experts' products over the grouped pairs.  ``glu``: x [T, K] by token, w [E, 2N, K] (gate rows, then up
    rows; alternating with ``interleaved``), out [P, N] = silu(gate) * up in x's type, rows in grouped order.
    Otherwise: x [P, K] in grouped order, w [E, N, K], out float32 [P, N] with row p the result of pair p.
    ``skinny``: the step has few tokens, so an expert's weights are streamed once against its few rows.
    ``limit`` > 0 (with ``glu``): out = g sigmoid(slope g) (u + 1), g = min(gate, limit), u = clamp(up, -limit, limit)."""
    _rows(x, "x"); _cuda(w, "w"); _rows(out, "out")
    E, NW, K = w.shape
    N = NW // 2 if glu else NW
    if x.shape[1] != K or out.shape != (n_pairs, N) or out.dtype != (x.dtype if glu else torch.float32):
        raise KernelError("moe_grouped: shapes or types do not match")
    _check(_fn("moe", "zlm_moe_grouped")(
        x.data_ptr(), code(x.dtype), _row_stride(x), w.data_ptr(), code(w.dtype), out.data_ptr(), _row_stride(out),
        int(glu), int(interleaved), int(skinny), n_pairs, E, N, K, top, float(limit), float(slope), offs.data_ptr(),
        order.data_ptr(),
        tile_expert.data_ptr(), tile_row.data_ptr(), n_tiles.data_ptr(), _stream()), "moe_grouped")


def moe_gather(x: torch.Tensor, order: torch.Tensor, top: int, rows: torch.Tensor) -> None:
    """rows[s] = x[order[s] // top]: the tokens' rows in grouped order."""
    _rows(x, "x"); _cuda(rows, "rows", x.dtype); _cuda(order, "order", torch.int32)
    P, d = rows.shape
    if x.shape[1] != d or order.numel() < P:
        raise KernelError("moe_gather: shapes do not match")
    _check(_fn("moe", "zlm_moe_gather")(x.data_ptr(), code(x.dtype), _row_stride(x), order.data_ptr(), top,
                                        rows.data_ptr(), P, d, _stream()), "moe_gather")


def gemm_tc_groups(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, host_offs, glu: Optional[str] = None,
                   limit: float = 0.0, slope: float = 1.0) -> bool:
    """One tensor-core product per group of consecutive rows: rows host_offs[g]..host_offs[g+1] of x [P, K] meet
    w[g] ([G, N, K], bf16) and give the same rows of out ([P, N], or [P, N/2] bf16 with ``glu``, whose rows of
    w[g] alternate gate and up).  ``host_offs``: a C array of G + 1 ints on the host.  False, with nothing or only
    some groups done, if the operands are not what TMA can read.  ``limit`` > 0 with ``glu`` "silu": the clamped
    swish of ``gated_act`` with that limit and slope."""
    global _launches
    _cuda(x, "x", torch.bfloat16); _cuda(w, "w", torch.bfloat16); _cuda(out, "out")
    G, N, K = w.shape
    n_out = N // 2 if glu else N
    if x.shape[1] != K or out.shape != (x.shape[0], n_out) or (glu and out.dtype != torch.bfloat16):
        raise KernelError("gemm_tc_groups: shapes or types do not match")
    launched = ctypes.c_int(0)
    status = _fn("gemm_tc", "zlm_gemm_tc_groups")(
        x.data_ptr(), w.data_ptr(), out.data_ptr(), code(out.dtype), GLU_KINDS[glu] if glu else 0, host_offs, G, N, K,
        K, K, n_out, N * K, float(limit), float(slope), ctypes.byref(launched), _stream())
    _launches += launched.value
    if status == -2:
        return False
    if status != 0:
        _check(status, "gemm_tc_groups")
    return True


def moe_combine(y: torch.Tensor, weights: torch.Tensor, out: torch.Tensor, accumulate: bool,
                place: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None, n_real: int = 0,
                h: Optional[torch.Tensor] = None, shared: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None) -> None:
    """out[t] (+)= sum_k weights[t, k] * y[row(t * top + k)], k ascending; all float32.  row(p) = p, or
    ``place[p]`` when y is in grouped order.  ``ids`` int32 [T, top] with ``n_real`` and ``h`` [T, d]: a pair whose
    expert is an identity expert (ids >= n_real) adds weights[t, k] * h[t] instead.  ``shared`` float32 [T, d]: added
    for every token, times sigmoid(gate[t]) when ``gate`` (float32, one number a token, any row stride) is given."""
    _cuda(y, "y", torch.float32); _cuda(weights, "weights", torch.float32); _cuda(out, "out", torch.float32)
    T, top = weights.shape
    d = out.shape[1]
    if y.shape != (T * top, d) or out.shape[0] != T:
        raise KernelError("moe_combine: shapes do not match")
    if place is not None:
        _cuda(place, "place", torch.int32)
        if place.numel() < T * top:
            raise KernelError("moe_combine: one place per pair is needed")
    h_code, h_stride, gate_stride = F32, 0, 0
    if ids is not None:
        _cuda(ids, "ids", torch.int32); _rows(h, "h")
        if ids.numel() < T * top or h.shape != (T, d):
            raise KernelError("moe_combine: the identity experts need every pair's expert and the tokens' rows")
        h_code, h_stride = code(h.dtype), _row_stride(h)
    if shared is not None:
        _cuda(shared, "shared", torch.float32)
        if shared.shape != (T, d):
            raise KernelError("moe_combine: the shared output must be float32 [T, d]")
        if gate is not None:
            if not gate.is_cuda or gate.dtype != torch.float32 or gate.shape[0] != T:
                raise KernelError("moe_combine: the gate must be float32 with one number a token")
            gate_stride = gate.stride(0) if T > 1 else 1
    elif gate is not None:
        raise KernelError("moe_combine: a gate goes with a shared output")
    _check(_fn("moe", "zlm_moe_combine")(y.data_ptr(), weights.data_ptr(), _ptr(place), _ptr(ids), int(n_real), _ptr(h),
                                         h_code, h_stride, _ptr(shared), _ptr(gate), gate_stride, out.data_ptr(), T, d,
                                         top, int(accumulate), _stream()), "moe_combine")


def add_(y: torch.Tensor, x: torch.Tensor) -> None:
    _cuda(y, "y", torch.float32); _cuda(x, "x", torch.float32)
    if y.numel() != x.numel():
        raise KernelError("add_: sizes differ")
    _check(_fn("elementwise", "zlm_add")(y.data_ptr(), x.data_ptr(), y.numel(), _stream()), "add_")


def convert(src: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(src, "src"); _cuda(out, "out")
    if src.numel() != out.numel():
        raise KernelError("convert: sizes differ")
    _check(_fn("elementwise", "zlm_convert")(src.data_ptr(), code(src.dtype), out.data_ptr(), code(out.dtype),
                                             src.numel(), _stream()), "convert")


def fill_normal(out: torch.Tensor, key: int, mean: float, std: float) -> None:
    """out.flat[i] = mean + std * z(key, i) with z the counter-based standard normal value of
    ``ziglm_b200.weights.random_init.normal_values`` (the same bits on the device as there)."""
    _cuda(out, "out")
    _check(_fn("elementwise", "zlm_fill_normal")(out.data_ptr(), code(out.dtype), out.numel(),
                                                 int(key) & 0xFFFFFFFFFFFFFFFF, float(mean), float(std), _stream()),
           "fill_normal")


# ------------------------------------------------------------------------ gemm
def gemm_generic(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 accumulate: bool = False) -> None:
    """out[M,N] (+)= x[M,K] @ w[N,K]^T (+ bias) on the CUDA cores; rows may be strided."""
    for t, n in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"{n} must be on a CUDA device (there is no CPU path)")
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{n} must be a matrix with unit column stride")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm: shapes do not match: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a float32 output")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias length does not match")
    _check(_fn("gemm_generic", "zlm_gemm_generic")(
        x.data_ptr(), code(x.dtype), w.data_ptr(), code(w.dtype), _ptr(bias),
        code(bias.dtype) if bias is not None else F32, out.data_ptr(), code(out.dtype), int(accumulate),
        M, N, K, x.stride(0) if M > 1 else K, w.stride(0) if N > 1 else K, out.stride(0) if M > 1 else N,
        _stream()), "gemm_generic")


# ------------------------------------------------------------------- attention
def rope_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rotary_dim: int,
               inv_freq: Optional[torch.Tensor], positions: torch.Tensor, seq_of_token: torch.Tensor,
               block_table: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
               page_size: int, keys_only: bool = False) -> None:
    """Rotate q and k of qkv[T, (n_heads+2 n_kv) head_dim] in place and store k, v in the cache pages.

    k_pages / v_pages: [n_pages, n_kv, page_size, head_dim] of one layer, or None to store nothing.  With
    ``keys_only`` the rows are [q heads | k heads] and only the keys are stored (``v_pages`` is not touched).
    block_table: int32 [B, stride]; row seq_of_token[t] lists the pages of token t's sequence.
    """
    _cuda(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    T = qkv.shape[0]
    if keys_only:
        v_pages = None
    if qkv.shape[1] != (n_heads + (1 if keys_only else 2) * n_kv) * head_dim:
        raise KernelError("rope_store: qkv width does not match the head counts")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_store: the frequency table must hold rotary_dim/2 entries")
    page_stride = 0
    if k_pages is not None:
        _cuda(k_pages, "k_pages", qkv.dtype)
        if v_pages is not None:
            _cuda(v_pages, "v_pages", qkv.dtype)
        elif not keys_only:
            raise KernelError("rope_store: value pages are needed unless only keys are stored")
        if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or (v_pages is not None and k_pages.shape != v_pages.shape):
            raise KernelError("rope_store: cache pages must be [n_pages, n_kv, page_size, head_dim]")
        page_stride = k_pages.stride(0)
    _check(_fn("attention", "zlm_rope_store")(
        qkv.data_ptr(), code(qkv.dtype), qkv.stride(0), T, n_heads, n_kv, head_dim, rotary_dim, _ptr(inv_freq),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        _ptr(k_pages), _ptr(v_pages), page_size, page_stride, _stream()), "rope_store")


def rope_norm_store(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rotary_dim: int,
                    inv_freq: Optional[torch.Tensor], amplitude: float, norm_dim: int, norm_eps: float,
                    positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                    k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], page_size: int,
                    norm_first: bool = False, q_weight: Optional[torch.Tensor] = None,
                    k_weight: Optional[torch.Tensor] = None) -> None:
    """``rope_store`` with an amplitude on the cosines and sines and a unit RMS norm behind the rotation: every
    q and k head of a row [q heads | k heads | v heads | ...] of qkv is turned, divided by
    sqrt(mean of the squares of its first ``norm_dim`` dimensions + norm_eps) (``norm_dim`` 0: not divided), written
    back and (keys, values) stored in the cache pages.  The row may be wider than the heads.  With ``norm_first`` the
    norm stands before the rotation, and ``q_weight`` / ``k_weight`` (float32 [head_dim], one for all query heads and
    one for all key heads; None: no weight) multiply the normed heads."""
    _rows(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("rope_norm_store: the rows are narrower than the heads")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope_norm_store: the frequency table must hold rotary_dim/2 entries")
    for w in (q_weight, k_weight):
        if w is not None:
            _cuda(w, "norm weight", torch.float32)
            if not norm_first or w.numel() != head_dim:
                raise KernelError("rope_norm_store: a norm weight holds one number for each element of a head and goes "
                                  "with the norm before the rotation")
    page_stride = 0
    if k_pages is not None:
        _cuda(k_pages, "k_pages", qkv.dtype); _cuda(v_pages, "v_pages", qkv.dtype)
        if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("rope_norm_store: cache pages must be [n_pages, n_kv, page_size, head_dim]")
        page_stride = k_pages.stride(0)
    _check(_fn("attention", "zlm_rope_norm_store")(
        qkv.data_ptr(), code(qkv.dtype), _row_stride(qkv), T, n_heads, n_kv, head_dim, rotary_dim, _ptr(inv_freq),
        float(amplitude), int(norm_dim), float(norm_eps), int(bool(norm_first)), _ptr(q_weight), _ptr(k_weight),
        positions.data_ptr(), seq_of_token.data_ptr(),
        block_table.data_ptr(), block_table.stride(0), _ptr(k_pages), _ptr(v_pages), page_size, page_stride, _stream()),
        "rope_norm_store")


def qk_prep(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rotary_dim: int,
            inv_freq: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
            q_count: int, k_count: int, norm_eps: float, mix_mode: int, mix: float, mix_buf: Optional[torch.Tensor],
            value_dim: int, positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
            k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], page_size: int) -> None:
    """What stands between the q|k|v product and attention when q and k are normed as whole vectors, in one kernel:
    rows [q heads | k heads | v heads | ...] of ``qkv`` are changed in place and k, v stored in the cache pages.

    ``q_weight`` / ``k_weight`` (float32, laid out like the q / k heads of a row; None: not normed): q and k, each as
    one vector, are divided by sqrt(mean square + norm_eps), the mean taken over ``q_count`` / ``k_count`` elements (heads
    kept with zeros behind them have fewer true elements), and multiplied by the weight; then the first ``rotary_dim``
    dimensions of every head are turned (pairs i, i + rotary_dim/2).  ``mix_mode`` 1: the values (the first ``value_dim``
    elements of every value head; the rest is zeros the head is kept with) are also left in ``mix_buf``
    [T, n_kv * value_dim]; 2: v <- (1 - mix) v + mix * mix_buf."""
    _rows(qkv, "qkv"); _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    T = qkv.shape[0]
    if qkv.shape[1] < (n_heads + 2 * n_kv) * head_dim:
        raise KernelError("qk_prep: the rows are narrower than the heads")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("qk_prep: the frequency table must hold rotary_dim/2 entries")
    for w, n in ((q_weight, n_heads), (k_weight, n_kv)):
        if w is not None:
            _cuda(w, "norm weight", torch.float32)
            if w.numel() != n * head_dim:
                raise KernelError("qk_prep: a norm weight must be laid out like its heads")
    if mix_mode:
        _cuda(mix_buf, "mix_buf", qkv.dtype)
        if mix_buf.shape != (T, n_kv * value_dim) or not mix_buf.is_contiguous():
            raise KernelError("qk_prep: the buffer of mixed values must be [T, n_kv * value_dim]")
    page_stride = 0
    if k_pages is not None:
        _cuda(k_pages, "k_pages", qkv.dtype); _cuda(v_pages, "v_pages", qkv.dtype)
        if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
            raise KernelError("qk_prep: cache pages must be [n_pages, n_kv, page_size, head_dim]")
        page_stride = k_pages.stride(0)
    _check(_fn("attention", "zlm_qk_prep")(
        qkv.data_ptr(), code(qkv.dtype), _row_stride(qkv), T, n_heads, n_kv, head_dim, rotary_dim, _ptr(inv_freq),
        _ptr(q_weight), _ptr(k_weight), int(q_count), int(k_count), float(norm_eps), int(mix_mode), float(mix),
        _ptr(mix_buf) if mix_mode else None, int(value_dim), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), _ptr(k_pages), _ptr(v_pages), page_size, page_stride, _stream()), "qk_prep")


def linear_attention_chunk() -> int:
    """Tokens of a chunk of ``decayed_linear_attention``: the table of decay powers holds this many plus one a head."""
    return int(_fn("linear_attention", "zlm_linear_attention_chunk")())


def decayed_linear_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, n_heads: int, dim: int,
                             value_dim: int, activation: Optional[str], pows: torch.Tensor, state: torch.Tensor, step,
                             out: torch.Tensor, rotary_dim: int = 0, inv_freq: Optional[torch.Tensor] = None,
                             key_scale: float = 1.0) -> None:
    """Linear attention with a fixed decay per head over the step's sequences: per head S <- a S + k v^T (float32
    [dim, value_dim], carried in ``state`` [slots, n_heads, dim, value_dim]) and o = S^T q.  Head h's q, k, v are the
    columns q_off + h*dim, k_off + h*dim, v_off + h*value_dim of ``proj``'s rows, read through ``activation``
    (None or "silu").  ``pows`` float32 [n_heads, chunk + 1]: decay_h^n.  ``out`` float32 [T, n_heads * value_dim].
    A step with a sequence of more tokens than a segment runs its segments side by side, with their start states in
    the step's scratch; a step of one token a sequence updates the state in place.  ``inv_freq`` (float32
    [rotary_dim / 2]): q and k carry rotary positions, the first ``rotary_dim`` dimensions of every head turned by the
    token's position (dimension i together with i + rotary_dim/2, angle position * inv_freq[i]); ``key_scale``: k times
    a factor behind the rotation.  Both are applied to the float32 copies the kernel works on, so what enters the
    recurrence is not rounded again."""
    _rows(proj, "proj"); _rows(out, "out"); _cuda(pows, "pows", torch.float32); _cuda(state, "state", torch.float32)
    T = proj.shape[0]
    if activation not in (None, "silu"):
        raise KernelError(f"decayed_linear_attention: activation {activation!r} is not known (silu)")
    if out.dtype != torch.float32 or out.shape != (T, n_heads * value_dim):
        raise KernelError("decayed_linear_attention: out must be float32 [T, heads * value_dim]")
    if (max(q_off, k_off) + n_heads * dim > proj.shape[1] or v_off + n_heads * value_dim > proj.shape[1]
            or min(q_off, k_off, v_off) < 0):
        raise KernelError("decayed_linear_attention: the heads lie outside the rows")
    if tuple(state.shape[1:]) != (n_heads, dim, value_dim) or not state.is_contiguous():
        raise KernelError("decayed_linear_attention: the state must be [slots, heads, dim, value_dim]")
    if tuple(pows.shape) != (n_heads, linear_attention_chunk() + 1) or not pows.is_contiguous():
        raise KernelError("decayed_linear_attention: the table of powers must be [heads, chunk + 1]")
    if inv_freq is not None:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() * 2 != rotary_dim or rotary_dim > dim:
            raise KernelError("decayed_linear_attention: the frequency table must hold rotary_dim/2 entries, at most dim/2")
        if activation is not None:
            raise KernelError("decayed_linear_attention: an activation is not combined with a rotation")
    seg_state = None
    if not step.single_token and step.max_new > int(_fn("linear_attention", "zlm_linear_attention_segment")()):
        n = int(_fn("linear_attention", "zlm_linear_attention_segments")(T, step.n_seqs))
        seg_state = step.ws.buf("lin_segment_states", (n, n_heads, dim, value_dim), torch.float32)
    _check(_fn("linear_attention", "zlm_decayed_linear_attention")(
        proj.data_ptr(), code(proj.dtype), _row_stride(proj), q_off, k_off, v_off, n_heads, dim, value_dim,
        1 if activation == "silu" else 0, int(rotary_dim) if inv_freq is not None else 0, _ptr(inv_freq),
        step.positions.data_ptr() if inv_freq is not None else None, float(key_scale), pows.data_ptr(), state.data_ptr(),
        step.slots.data_ptr(),
        step.cu_seqlens.data_ptr(), step.n_seqs, T, 1 if step.single_token and T == step.n_seqs else 0, _ptr(seg_state),
        out.data_ptr(), _row_stride(out), _stream()),
        "decayed_linear_attention")


def attention_general_scratch(n_tokens: int, n_heads: int, n_kv: int, head_dim: int, max_keys: int) -> int:
    """Floats of scratch with which ``attention_general`` spreads a step of few tokens over more blocks (0: none
    is of use)."""
    return int(_fn("attention", "zlm_attention_general_scratch")(n_tokens, n_heads, n_kv, head_dim, max_keys))


def attention_general(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                      window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                      block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_size: int, max_keys: int = 0, scratch: Optional[torch.Tensor] = None,
                      softcap: float = 0.0, keep_first: int = 0, sinks: Optional[torch.Tensor] = None) -> None:
    """out[t, h, :] = softmax(q[t,h] . K[start..pos_t] * scale) @ V over the paged cache; with ``softcap`` c > 0 the
    scaled scores become c * tanh(score / c) before the softmax.  With a window, the first ``keep_first`` positions
    of a sequence stay visible behind it.  ``sinks`` (float32, one per query head): exp(sinks[h]) is added to the
    softmax's denominator; it has no key and no value and is not scaled.

    The queries are the first n_heads*head_dim columns of each row of ``qkv`` (any row stride).
    ``max_keys`` (the most keys a token of the step sees) and ``scratch`` (float32, at least
    ``attention_general_scratch(...)`` elements) let a step of few tokens use more blocks; the result does not
    depend on them.
    """
    _cuda(out, "out", qkv.dtype); _cuda(k_pages, "k_pages", qkv.dtype); _cuda(v_pages, "v_pages", qkv.dtype)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.stride(1) != 1:
        raise KernelError("attention: q must be on the device with unit column stride")
    T = out.shape[0]
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention: widths do not match the head counts")
    if head_dim % 8 or head_dim > 512:
        raise KernelError(f"attention: head size {head_dim} is not supported (a multiple of 8, at most 512)")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if sinks is not None:
        _cuda(sinks, "sinks", torch.float32)
        if sinks.numel() != n_heads:
            raise KernelError("attention: one sink per query head is needed")
    _check(_fn("attention", "zlm_attention_general")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), code(qkv.dtype), T, n_heads, n_kv, head_dim, scale,
        float(softcap or 0.0), int(window or 0), int(keep_first or 0), _ptr(sinks), positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), page_size, k_pages.stride(0), int(max_keys),
        _ptr(scratch), scratch.numel() if scratch is not None else 0, _stream()),
        "attention_general")
    if scratch is not None and max_keys > 0 and scratch.numel() >= attention_general_scratch(
            T, n_heads, n_kv, head_dim, max_keys) > 0:
        global _launches
        _launches += 1          # the fold of the parts is a second launch


def _tc_attention_ok(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and n_kv > 0 and n_heads % n_kv == 0
            and n_heads // n_kv <= 16 and page_size == 64)


def attention_decode(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                     window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                     block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int,
                     n_splits: int, part_o: torch.Tensor, part_ml: torch.Tensor, softcap: float = 0.0,
                     keep_first: int = 0, sinks: Optional[torch.Tensor] = None,
                     head_gate: Optional[torch.Tensor] = None, head_gate_mult: float = 1.0) -> bool:
    """Tensor-core attention for steps of one token per sequence (bf16, head size 64 or 128); ``keep_first`` and
    ``sinks`` as :func:`attention_general` takes them.  ``head_gate`` ([T, n_heads] of the rows' type, a row stride of
    its own): head h of token t leaves multiplied by sigmoid(head_gate[t, h]) * ``head_gate_mult``.

    Each token's query heads are grouped by key/value head so that the cache is read once per group; the keys
    of a sequence are split over ``n_splits`` blocks whose partial results go through the float32 scratch
    ``part_o`` [T*n_heads*n_splits*head_dim] and ``part_ml`` [T*n_heads*n_splits*2].  False if refused.
    """
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    _cuda(part_o, "part_o", torch.float32); _cuda(part_ml, "part_ml", torch.float32)
    T = out.shape[0]
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_decode: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim or qkv.shape[0] < T:
        raise KernelError("attention_decode: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_decode: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if part_o.numel() < T * n_heads * n_splits * head_dim or part_ml.numel() < T * n_heads * n_splits * 2:
        raise KernelError("attention_decode: the scratch is too small for this many splits")
    if sinks is not None:
        _cuda(sinks, "sinks", torch.float32)
        if sinks.numel() != n_heads or not sinks.is_contiguous():
            raise KernelError("attention_decode: one sink per query head is needed")
    if head_gate is not None:
        _rows(head_gate, "head_gate")
        if head_gate.dtype != qkv.dtype or tuple(head_gate.shape) != (T, n_heads):
            raise KernelError("attention_decode: the gates must be [T, n_heads] of the rows' type")
    status = _fn("attention_tc", "zlm_attention_decode")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, n_heads, n_kv, head_dim, scale, float(softcap or 0.0),
        int(window or 0), int(keep_first or 0) if (window or 0) > 0 else 0, _ptr(sinks), _ptr(head_gate),
        _row_stride(head_gate) if head_gate is not None else 0, float(head_gate_mult),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, n_splits, part_o.data_ptr(),
        part_ml.data_ptr(), _stream())
    if status == -2:
        return False
    _check(status, "attention_decode")
    global _launches
    _launches += 1          # the merge of the splits is a second launch
    return True


def _gate_args(gate: Optional[torch.Tensor], n_rows: int, width: int):
    """(pointer, row stride) of a bf16 gate [n_rows, width] that may be a column slice; (None, 0) without one."""
    if gate is None:
        return None, 0
    _rows(gate, "gate")
    if gate.dtype != torch.bfloat16 or gate.shape[0] < n_rows or gate.shape[1] != width:
        raise KernelError("attention: the gate must be bfloat16 with a row per token and a column per output element")
    return gate.data_ptr(), _row_stride(gate)


def attention_decode_flat_blocks(n_tokens: int, n_heads: int, n_kv: int, head_dim: int) -> int:
    """Blocks of one resident wave of the flat decode kernel for a step of ``n_tokens`` (0: sizes it refuses)."""
    return int(_fn("attention_tc", "zlm_attention_decode_flat_blocks")(n_tokens, n_heads, n_kv, head_dim))


def attention_decode_flat_scratch(n_tokens: int, n_heads: int, n_kv: int, head_dim: int, n_blocks: int) -> int:
    """Floats of scratch the flat decode kernel needs with ``n_blocks`` blocks."""
    return int(_fn("attention_tc", "zlm_attention_decode_flat_scratch")(n_tokens, n_heads, n_kv, head_dim, n_blocks))


def attention_decode_flat(qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
                          window: Optional[int], positions: torch.Tensor, seq_of_token: torch.Tensor,
                          block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_size: int,
                          n_blocks: int, counters: torch.Tensor, scratch: torch.Tensor,
                          rope: Optional[Tuple[Optional[torch.Tensor], int, bool]] = None, softcap: float = 0.0,
                          gate: Optional[torch.Tensor] = None) -> bool:
    """Tensor-core attention for steps of one token per sequence, with the pages of all sequences of the
    step divided evenly over ``n_blocks`` blocks (one resident wave), whatever the sequences' lengths.  One
    launch: the block that finishes a sequence's last piece merges the pieces.

    ``scratch``: float32, at least ``attention_decode_flat_scratch(...)`` elements, any content.
    ``counters``: int32, one per (token, kv head), zero before the first call; a call that completes leaves
    them zero (a call that ended with a wait error does not: zero them again).  False if refused.

    ``rope`` = (inv_freq or None, rotary_dim, store): the kernel also does what ``rope_store`` does for the
    step's tokens, so that no kernel runs between the projection and the attention.  The rows of ``qkv`` are
    then [q heads | k heads | v heads] (k and v only with ``store``) as the projection left them; the query
    heads are rotated as they are loaded (``qkv`` itself is left alone) and, with ``store``, the new keys
    (rotated) and values go into the cache pages.  rotary_dim must be a multiple of 32.

    ``gate`` (bf16 [T, n_heads * head_dim], may be a column slice): the output is multiplied by its sigmoid before
    it is rounded.
    """
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(positions, "positions", torch.int32); _cuda(seq_of_token, "seq_of_token", torch.int32)
    _cuda(block_table, "block_table", torch.int32); _cuda(scratch, "scratch", torch.float32)
    _cuda(counters, "counters", torch.int32)
    T = out.shape[0]
    if counters.numel() < T * n_kv:
        raise KernelError("attention_decode_flat: one counter per (token, kv head) is needed")
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_decode_flat: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim or qkv.shape[0] < T:
        raise KernelError("attention_decode_flat: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_decode_flat: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if n_blocks <= 0:
        raise KernelError("attention_decode_flat: the number of blocks must be positive")
    fused, store, rot, inv_freq = 0, 0, 0, None
    if rope is not None:
        inv_freq, rot, store = rope
        fused = 1
        if inv_freq is None:
            rot = 0
        else:
            _cuda(inv_freq, "inv_freq", torch.float32)
            if inv_freq.numel() * 2 != rot:
                raise KernelError("attention_decode_flat: the frequency table must hold rotary_dim/2 entries")
        if qkv.shape[1] < (n_heads + (2 * n_kv if store else 0)) * head_dim:
            raise KernelError("attention_decode_flat: the rows must hold the key and value heads to be stored")
    status = _fn("attention_tc", "zlm_attention_decode_flat")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), T, n_heads, n_kv, head_dim, scale, float(softcap or 0.0),
        int(window or 0),
        positions.data_ptr(), seq_of_token.data_ptr(), block_table.data_ptr(), block_table.stride(0),
        k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, n_blocks, counters.data_ptr(),
        scratch.data_ptr(), scratch.numel(), fused, int(bool(store)), int(rot), _ptr(inv_freq),
        *_gate_args(gate, T, n_heads * head_dim), _stream())
    if status == -2:
        return False
    if status == -1:
        raise KernelError("attention_decode_flat: bad arguments, or the scratch is too small for this many blocks")
    _check(status, "attention_decode_flat")
    return True


def attention_prefill(qkv: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_heads: int, n_kv: int,
                      head_dim: int, scale: float, window: Optional[int], cu_seqlens: torch.Tensor,
                      past_lens: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                      v_pages: torch.Tensor, page_size: int, softcap: float = 0.0) -> bool:
    """Tensor-core attention for prompt steps: sequence b brings tokens cu_seqlens[b]..cu_seqlens[b+1] of the
    packed stream after past_lens[b] cached ones (bf16, head size 64 or 128).  False if refused."""
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(past_lens, "past_lens", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_prefill: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention_prefill: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_prefill: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if cu_seqlens.numel() < n_seqs + 1 or past_lens.numel() < n_seqs:
        raise KernelError("attention_prefill: sequence arrays are too short")
    status = _fn("attention_tc", "zlm_attention_prefill")(
        qkv.data_ptr(), qkv.stride(0), out.data_ptr(), n_seqs, max_new, n_heads, n_kv, head_dim, scale,
        float(softcap or 0.0), int(window or 0), cu_seqlens.data_ptr(), past_lens.data_ptr(), block_table.data_ptr(),
        block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), k_pages.shape[0], page_size, _stream())
    if status == -2:
        return False
    _check(status, "attention_prefill")
    return True


def attention_prefill_fmha(qkv: torch.Tensor, out: torch.Tensor, n_seqs: int, max_new: int, n_heads: int, n_kv: int,
                           head_dim: int, scale: float, window: Optional[int], cu_seqlens: torch.Tensor,
                           past_lens: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, page_size: int, softcap: float = 0.0, keep_first: int = 0,
                           sinks: Optional[torch.Tensor] = None) -> bool:
    """Prompt attention on the tcgen05 tensor cores (tiles of 128 queries, accumulators in tensor memory); same
    arguments as :func:`attention_prefill`, and ``keep_first`` / ``sinks`` as :func:`attention_general` takes them.
    False if refused."""
    if sinks is not None:
        _cuda(sinks, "sinks", torch.float32)
        if sinks.numel() != n_heads or not sinks.is_contiguous():
            raise KernelError("attention_prefill_fmha: one sink per query head is needed")
    _cuda(out, "out", torch.bfloat16); _cuda(k_pages, "k_pages", torch.bfloat16); _cuda(v_pages, "v_pages", torch.bfloat16)
    _cuda(cu_seqlens, "cu_seqlens", torch.int32); _cuda(past_lens, "past_lens", torch.int32)
    _cuda(block_table, "block_table", torch.int32)
    if not qkv.is_cuda or qkv.dtype != torch.bfloat16 or qkv.stride(1) != 1:
        raise KernelError("attention_prefill_fmha: q must be bfloat16 on the device with unit column stride")
    if out.shape[1] != n_heads * head_dim or qkv.shape[1] < n_heads * head_dim:
        raise KernelError("attention_prefill_fmha: widths do not match the head counts")
    if tuple(k_pages.shape[1:]) != (n_kv, page_size, head_dim) or k_pages.shape != v_pages.shape:
        raise KernelError("attention_prefill_fmha: cache pages must be [n_pages, n_kv, page_size, head_dim]")
    if cu_seqlens.numel() < n_seqs + 1 or past_lens.numel() < n_seqs:
        raise KernelError("attention_prefill_fmha: sequence arrays are too short")
    status = _fn("attention_fmha", "zlm_attention_prefill_fmha")(
        qkv.data_ptr(), qkv.stride(0), qkv.shape[0], out.data_ptr(), n_seqs, max_new, n_heads, n_kv, head_dim, scale,
        float(softcap or 0.0), int(window or 0), int(keep_first or 0) if (window or 0) > 0 else 0, _ptr(sinks), cu_seqlens.data_ptr(),
        past_lens.data_ptr(), block_table.data_ptr(), block_table.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
        k_pages.shape[0], page_size, _stream())
    if status == -2:
        return False
    _check(status, "attention_prefill_fmha")
    return True


def attention_fmha_status() -> int:
    """0, or the code of a bounded wait that ran out inside the tcgen05 attention kernel (21 queries, 22 page,
    23 scores, 24 probabilities, 25 output, 26 stage never drained, 4 copies still in flight)."""
    out = ctypes.c_int(0)
    rc = _fn("attention_fmha", "zlm_attention_fmha_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"attention_fmha_status: CUDA error {rc}")
    return out.value


def attention_tc_status() -> int:
    """0, or the code of a bounded wait that ran out inside a tensor-core attention kernel (11 a page never
    landed, 12 a stage never drained, 4 copies still in flight).  Synchronises the device."""
    out = ctypes.c_int(0)
    rc = _fn("attention_tc", "zlm_attention_tc_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"attention_tc_status: CUDA error {rc}")
    return out.value


def decode_splits(n_tokens: int, n_kv: int, max_total: int, page_size: int = 64) -> int:
    """How many blocks share the keys of one sequence in a decode step: enough for two blocks per SM."""
    pages = max(1, -(-max_total // page_size))
    want = -(-296 // max(1, n_tokens * n_kv))
    return max(1, min(want, pages, 64))


def attention_with_rope(step, qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                        scale: float, window: Optional[int], io, inv_freq: Optional[torch.Tensor], rotary_dim: int,
                        store: bool) -> bool:
    """Decode steps on the tensor-core path: rotation, cache write and attention in one kernel.  False when
    the step is not of that kind; the caller then runs ``rope_store`` and ``attention``."""
    if not (step.single_token and _tc_attention_ok(qkv.dtype, n_heads, n_kv, head_dim, io.page_size)):
        return False
    if inv_freq is not None and rotary_dim % 32:
        return False
    n_blocks = attention_decode_flat_blocks(step.n_tokens, n_heads, n_kv, head_dim)
    if n_blocks <= 0:
        return False
    need = attention_decode_flat_scratch(step.n_tokens, n_heads, n_kv, head_dim, n_blocks)
    scratch = step.ws.buf("attn_flat_scratch", (need,), torch.float32)
    counters = step.ws.buf("attn_flat_counters", (step.n_tokens * n_kv,), torch.int32, zeros=True)
    return attention_decode_flat(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions, step.seq_of_token,
                                 io.block_table, io.k_pages, io.v_pages, io.page_size, n_blocks, counters, scratch,
                                 rope=(inv_freq, rotary_dim, store))


def attention(step, qkv: torch.Tensor, out: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, scale: float,
              window: Optional[int], io, softcap: float = 0.0, gate: Optional[torch.Tensor] = None,
              keep_first: int = 0, sinks: Optional[torch.Tensor] = None, head_gate: Optional[torch.Tensor] = None,
              head_gate_mult: float = 1.0, chunk: Optional[int] = None) -> bool:
    """Attention of a step's tokens over the cache of the running layer; picks the kernel.  ``chunk`` (instead of
    ``window``): the positions of a sequence form chunks of that many, counted from its start, and a query sees the
    earlier keys of its own chunk only (the kernels take it as a negative window).  ``softcap`` c > 0:
    the scaled scores become c * tanh(score / c).  ``keep_first``: with a window, the first positions of a sequence
    that stay visible behind it.  ``sinks`` (float32, one per query head): a number in the softmax's denominator that
    belongs to no key.  ``gate`` ([T, n_heads * head_dim] of the step's type): the flat
    decode kernel multiplies its output by sigmoid(gate) before rounding it; the result says whether that was done
    (the caller multiplies when it was not: in a prompt one pass of ``sigmoid_mul`` over coalesced rows costs less
    than the same work in the prompt kernel's epilogue, where every thread walks a row of its own).  ``head_gate``
    ([T, n_heads], instead of ``gate``): one gate a head, times ``head_gate_mult``; the decode kernel that splits a
    sequence's keys applies it where it combines the splits, and the result says so likewise."""
    if gate is not None and head_gate is not None:
        raise KernelError("attention: a gate an element or a gate a head, not both")
    if chunk:
        if window:
            raise KernelError("attention: a window or chunks, not both")
        keep_first = 0
        span = min(step.max_total, int(chunk))        # the most keys a token sees
        window = -int(chunk)
    else:
        keep_first = int(keep_first or 0) if window else 0
        span = min(step.max_total, window + keep_first) if window else step.max_total
    # kept first tokens and sinks: the tcgen05 prompt kernel and the decode kernel that splits a sequence's keys
    # know both, the other tensor-core kernels neither
    plain_only = keep_first > 0 or sinks is not None
    if plain_only and _tc_attention_ok(qkv.dtype, n_heads, n_kv, head_dim, io.page_size):
        if step.single_token:
            n_splits = decode_splits(step.n_tokens, n_kv, span, io.page_size)
            part_o = step.ws.buf("attn_part_o", (step.n_tokens * n_heads * n_splits * head_dim,), torch.float32)
            part_ml = step.ws.buf("attn_part_ml", (step.n_tokens * n_heads * n_splits * 2,), torch.float32)
            if attention_decode(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions, step.seq_of_token,
                                io.block_table, io.k_pages, io.v_pages, io.page_size, n_splits, part_o, part_ml,
                                softcap=softcap, keep_first=keep_first, sinks=sinks, head_gate=head_gate,
                                head_gate_mult=head_gate_mult):
                return head_gate is not None
        elif step.max_new >= 16 and attention_prefill_fmha(
                qkv, out, step.n_seqs, step.max_new, n_heads, n_kv, head_dim, scale, window, step.cu_seqlens,
                step.past_lens, io.block_table, io.k_pages, io.v_pages, io.page_size, softcap=softcap,
                keep_first=keep_first, sinks=sinks):
            return False
    if not plain_only and _tc_attention_ok(qkv.dtype, n_heads, n_kv, head_dim, io.page_size):
        n_blocks = attention_decode_flat_blocks(step.n_tokens, n_heads, n_kv, head_dim) if step.single_token else 0
        if n_blocks > 0:
            need = attention_decode_flat_scratch(step.n_tokens, n_heads, n_kv, head_dim, n_blocks)
            scratch = step.ws.buf("attn_flat_scratch", (need,), torch.float32)
            counters = step.ws.buf("attn_flat_counters", (step.n_tokens * n_kv,), torch.int32, zeros=True)
            if attention_decode_flat(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions,
                                     step.seq_of_token, io.block_table, io.k_pages, io.v_pages, io.page_size,
                                     n_blocks, counters, scratch, softcap=softcap, gate=gate):
                return gate is not None
        if step.single_token:
            n_splits = decode_splits(step.n_tokens, n_kv, span, io.page_size)
            part_o = step.ws.buf("attn_part_o", (step.n_tokens * n_heads * n_splits * head_dim,), torch.float32)
            part_ml = step.ws.buf("attn_part_ml", (step.n_tokens * n_heads * n_splits * 2,), torch.float32)
            if attention_decode(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions,
                                step.seq_of_token, io.block_table, io.k_pages, io.v_pages, io.page_size, n_splits,
                                part_o, part_ml, softcap=softcap):
                return False
        else:
            # prompts: the tcgen05 kernel (tiles of 128 queries); a handful of tokens: the 64-row mma.sync one
            args = (qkv, out, step.n_seqs, step.max_new, n_heads, n_kv, head_dim, scale, window, step.cu_seqlens,
                    step.past_lens, io.block_table, io.k_pages, io.v_pages, io.page_size)
            if step.max_new >= 16 and attention_prefill_fmha(*args, softcap=softcap):
                return False
            if attention_prefill(*args, softcap=softcap):
                return False
    max_keys = span
    need = attention_general_scratch(step.n_tokens, n_heads, n_kv, head_dim, max_keys)
    scratch = step.ws.buf("attn_parts", (need,), torch.float32) if need > 0 else None
    attention_general(qkv, out, n_heads, n_kv, head_dim, scale, window, step.positions, step.seq_of_token,
                      io.block_table, io.k_pages, io.v_pages, io.page_size, max_keys, scratch, softcap=softcap,
                      keep_first=keep_first, sinks=sinks)
    return False


def fast_attention_libraries(dtype: torch.dtype, head_dim: int, n_heads: int = 1, n_kv: int = 1, softcap: float = 0.0,
                             keep_first: int = 0, sinks: bool = False):
    """The sources of the tensor-core attention kernels if they take this shape and these options, else nothing (the
    plain kernel runs)."""
    if keep_first or sinks:
        return ("attention_tc", "attention_fmha") if _tc_attention_ok(dtype, n_heads, n_kv, head_dim, 64) else ()
    return ("attention_tc", "attention_fmha") if _tc_attention_ok(dtype, n_heads, n_kv, head_dim, 64) else ()


def fast_gemm_libraries():
    return ("gemm_tc",)


GLU_KINDS = {"silu": 1, "gelu_tanh": 2}


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
            accumulate: bool = False, splits: int = 0, glu: Optional[str] = None, norm_out=None, row_scale=None):
    """out[T,N] (+)= x[T,K] @ w[N,K]^T (+ bias) on the tcgen05 tensor cores, bf16 operands.

    With ``glu`` ("silu" or "gelu_tanh") the rows of w (and the entries of bias) alternate gate and up rows and
    out is bf16 [T, N/2] holding act(gate + bias) * (up + bias).

    An RMSNorm between two products of a step of few tokens can ride on them.  ``norm_out`` = (gain, offset, hb,
    ssq) on the product before it (``accumulate`` into the float32 residual): it also leaves bf16(x * (gain +
    offset)) in ``hb`` [T, N] and sums of x^2 per tile row of 128 features in ``ssq`` [T, ceil(N/128)] (float32);
    the result is then 2 if it did and 1 if the launch it chose cannot (nothing is written to hb and ssq).
    ``row_scale`` = (ssq, eps) on the product after it, whose x is that ``hb``: every output row t is multiplied
    by 1 / sqrt(sum(ssq[t]) / K + eps) before the bias.

    Returns False, having done nothing, if the operands are not what TMA can read (a row stride that is no
    multiple of 8 elements, a base address off a 16-byte boundary); else a true value.
    """
    for t, n in ((x, "x"), (w, "w"), (out, "out")):
        if not t.is_cuda:
            raise KernelError(f"{n} must be on a CUDA device (there is no CPU path)")
        if t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"{n} must be a matrix with unit column stride")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc: x and w must be bfloat16")
    T, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if glu else N
    if glu and (glu not in GLU_KINDS or N % 2 or out.dtype != torch.bfloat16):
        raise KernelError("gemm_tc: the gated mode needs silu or gelu_tanh, an even row count and a bf16 output")
    if w.shape[1] != K or out.shape != (T, n_out):
        raise KernelError(f"gemm: shapes do not match: x{tuple(x.shape)} w{tuple(w.shape)} out{tuple(out.shape)}")
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulation needs a float32 output")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm: bias length does not match")
    gain = hb = ssq_out = ssq_in = None
    offset, eps, scale_p = 0.0, 0.0, 0
    fused = ctypes.c_int(0)
    if norm_out is not None:
        gain, offset, hb, ssq_out = norm_out
        _cuda(gain, "gain"); _cuda(hb, "hb", torch.bfloat16); _cuda(ssq_out, "ssq", torch.float32)
        if not accumulate or glu or gain.numel() != N or hb.shape != (T, N) or hb.stride(1) != 1 \
                or ssq_out.numel() < T * (-(-N // 128)) or gain.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("gemm_tc: norm_out needs accumulate, a gain of N elements, hb [T, N] and ssq [T, ceil(N/128)]")
    if row_scale is not None:
        ssq_in, eps = row_scale
        _cuda(ssq_in, "ssq", torch.float32)
        if T > 64 or ssq_in.dim() != 2 or ssq_in.shape[0] < T or not ssq_in.is_contiguous():
            raise KernelError("gemm_tc: row_scale needs at most 64 rows and ssq [T, P] contiguous")
        scale_p = ssq_in.shape[1]
    status = _fn("gemm_tc", "zlm_gemm_tc_norm")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), code(bias.dtype) if bias is not None else F32, out.data_ptr(),
        code(out.dtype), int(accumulate), GLU_KINDS[glu] if glu else 0, T, N, K, x.stride(0) if T > 1 else K,
        w.stride(0) if N > 1 else K, out.stride(0) if T > 1 else n_out, int(splits),
        _ptr(gain), code(gain.dtype) if gain is not None else F32, float(offset), _ptr(hb),
        hb.stride(0) if hb is not None and T > 1 else N, _ptr(ssq_out), ctypes.byref(fused), _ptr(ssq_in), scale_p,
        float(eps), _stream())
    if status == -2:
        return False
    _check(status, "gemm_tc")
    return 2 if fused.value else 1


def gemm_tc_swish_clamped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, limit: float, slope: float,
                          bias: Optional[torch.Tensor] = None) -> bool:
    """The gated product on the tensor cores with the clamped swish in its epilogue: the rows of w [2I, K] alternate
    gate and up rows, out [T, I] (bf16) = g * sigmoid(slope * g) * (u + 1) with g = min(gate, limit) and
    u = clamp(up, -limit, limit).  False, having done nothing, if the operands are not what TMA can read."""
    for t, n in ((x, "x"), (w, "w"), (out, "out")):
        _rows(t, n)
        if t.dtype != torch.bfloat16:
            raise KernelError(f"gemm_tc_swish_clamped: {n} must be bfloat16")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or N % 2 or out.shape != (T, N // 2) or not limit > 0:
        raise KernelError("gemm_tc_swish_clamped: shapes do not match, or the limit is not positive")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm_tc_swish_clamped: bias length does not match")
    status = _fn("gemm_tc", "zlm_gemm_tc_swish_clamped")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), code(bias.dtype) if bias is not None else F32, out.data_ptr(), T, N, K,
        _row_stride(x), _row_stride(w), _row_stride(out), float(limit), float(slope), _stream())
    if status == -2:
        return False
    _check(status, "gemm_tc_swish_clamped")
    return True


def gemm_tc_unary(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, activation: str,
                  bias: Optional[torch.Tensor] = None) -> bool:
    """out [T, N] (bf16) = act(x w^T + bias) on the tensor cores, the activation applied to the float32 sums in the
    epilogue ("relu2": max(y, 0)^2; "gelu": the exact, erf form).  False, having done nothing, if the operands are not what TMA can read."""
    _rows(x, "x"); _rows(w, "w"); _rows(out, "out")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_unary: x, w and out must be bfloat16")
    if activation not in UNARY_ACTIVATIONS:
        raise KernelError(f"gemm_tc_unary: activation {activation!r} is not known ({', '.join(UNARY_ACTIVATIONS)})")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (T, N):
        raise KernelError("gemm_tc_unary: shapes do not match")
    if bias is not None:
        _cuda(bias, "bias")
        if bias.numel() != N:
            raise KernelError("gemm_tc_unary: bias length does not match")
    status = _fn("gemm_tc", "zlm_gemm_tc_unary")(
        x.data_ptr(), w.data_ptr(), _ptr(bias), code(bias.dtype) if bias is not None else F32, out.data_ptr(), T, N, K,
        _row_stride(x), _row_stride(w), _row_stride(out), UNARY_ACTIVATIONS[activation] + 1, _stream())
    if status == -2:
        return False
    _check(status, "gemm_tc_unary")
    return True


def gemm_tc_status() -> int:
    """0, or the code of a bounded wait that ran out inside a tensor-core kernel since the last call
    (1 tile never landed, 2 stage never drained, 3 accumulator never completed, 4 copies still in flight).
    Synchronises the device."""
    out = ctypes.c_int(0)
    rc = _fn("gemm_tc", "zlm_gemm_tc_status")(ctypes.byref(out))
    if rc != 0:
        raise KernelError(f"gemm_tc_status: CUDA error {rc}")
    return out.value


WAIT_ERROR_NAMES = {
    1: "a tile never landed", 2: "a stage never drained", 3: "an accumulator never completed",
    4: "copies were still in flight when a block gave up", 11: "a cache page never landed",
    12: "a stage never drained", 21: "the queries never landed", 22: "a cache page never landed",
    23: "the scores never completed", 24: "the probabilities were never consumed", 25: "the output never completed",
    26: "a stage never drained", 27: "a tile address was off its boundary", 90: "a wait ran out on purpose (self-test)",
}


def wait_errors() -> dict:
    """The error words of the bounded waits of every tensor-core library this process has loaded: library name
    -> code (0: none).  Reading a word clears it.  Synchronises the device."""
    out = {}
    for lib, read in (("gemm_tc", gemm_tc_status), ("attention_tc", attention_tc_status),
                      ("attention_fmha", attention_fmha_status)):
        if _build.is_loaded(lib):
            out[lib] = read()
    return out


def wait_selftest(library: str, polls: int = 4096) -> Tuple[int, int]:
    """Run the give-up path of the bounded waits of ``library`` ("gemm_tc", "attention_tc" or "attention_fmha")
    once, on purpose and harmlessly: one block waits, with a limit of ``polls`` polls, on a barrier in its own
    shared memory that nothing arrives on (no copy, no tensor memory, nothing in flight), records code 90 in
    the library's error word and returns.  Result: (what the wait returned: 0 = gave up, the abort flag it
    left).  The library's status call then reports 90 once."""
    if library not in ("gemm_tc", "attention_tc", "attention_fmha"):
        raise KernelError(f"no bounded waits in {library!r}")
    seen = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    _check(_fn(library, f"zlm_{library}_wait_selftest")(int(polls), seen.data_ptr(), _stream()), "wait_selftest")
    torch.cuda.current_stream().synchronize()
    passed, flag = seen.tolist()
    return int(passed), int(flag)


def describe_wait_errors(codes: dict) -> str:
    return "; ".join(f"{lib}: code {c} ({WAIT_ERROR_NAMES.get(c, 'unknown')})" for lib, c in codes.items() if c)


def fast_gemm(linear, x: torch.Tensor, out: torch.Tensor, accumulate: bool, norm_out=None, row_scale=None):
    """Run the product on the tensor-core kernels if they take it (see ``gemm_tc`` for the result); False if
    they do not."""
    if x.dtype != torch.bfloat16 or linear.weight.dtype != torch.bfloat16:
        return False
    if out.dtype not in (torch.float32, torch.bfloat16):
        return False
    return gemm_tc(x, linear.weight, out, bias=linear.bias, accumulate=accumulate, norm_out=norm_out,
                   row_scale=row_scale)


# -------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = the id of the largest logit of row r (lowest id on ties)."""
    _cuda(out, "out", torch.int32)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be a float32 matrix on the device with unit column stride")
    rows, V = logits.shape
    if out.numel() < rows:
        raise KernelError("argmax: the output is too short")
    _check(_fn("sampling", "zlm_argmax")(logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V,
                                         out.data_ptr(), _stream()), "argmax")


def sample(logits: torch.Tensor, out: torch.Tensor, rng: torch.Tensor, temperature: float, top_k: int = 0,
           top_p: float = 1.0, min_p: float = 0.0, repetition_penalty: float = 1.0, presence_penalty: float = 0.0,
           history: Optional[torch.Tensor] = None) -> None:
    """Draw one id per row.  rng: int64 [rows, 2] of (seed, counter).  history: int32 [rows, window], -1 = empty.

    The logits are changed in place when a penalty is on.
    """
    _cuda(out, "out", torch.int32); _cuda(rng, "rng", torch.int64)
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a float32 matrix on the device with unit column stride")
    rows, V = logits.shape
    if out.numel() < rows or rng.numel() < 2 * rows:
        raise KernelError("sample: output or rng too short")
    if not temperature > 0:
        raise KernelError("sample: the temperature must be positive (use argmax for greedy)")
    if top_k > 1024:
        raise KernelError("sample: top_k above 1024 is not supported")
    window = 0
    if history is not None:
        _cuda(history, "history", torch.int32)
        window = history.shape[1]
        if history.shape[0] < rows or window > 1024:
            raise KernelError("sample: history must be [rows, window] with window <= 1024")
    if 1 <= top_k <= 64 and window <= 256:
        # many blocks per row: each finds the k best of its slice, the last one to arrive cuts and draws
        counters, scratch = _sample_scratch(logits.device, rows)
        status = _fn("sampling", "zlm_sample_parts")(
            logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V, temperature, int(top_k), top_p, min_p,
            repetition_penalty, presence_penalty, _ptr(history), window, rng.data_ptr(), out.data_ptr(),
            counters.data_ptr(), scratch.data_ptr(), scratch.numel(), _stream())
        if status != -2:
            _check(status, "sample")
            return
    _check(_fn("sampling", "zlm_sample")(
        logits.data_ptr(), rows, V, logits.stride(0) if rows > 1 else V, temperature, int(top_k), top_p, min_p,
        repetition_penalty, presence_penalty, _ptr(history), window, rng.data_ptr(), out.data_ptr(), _stream()),
        "sample")


_SAMPLE_SCRATCH = {}


def _sample_scratch(device: torch.device, rows: int):
    """Counters and scratch of the many-block sampler, kept per device and grown as needed.  The counters (one
    per row, a buffer of their own so that their place does not move with the number of rows) start at zero
    and every call leaves them zero."""
    counters, scratch = _SAMPLE_SCRATCH.get(device, (None, None))
    need = int(_fn("sampling", "zlm_sample_parts_scratch")(rows))
    if counters is None or counters.numel() < rows:
        counters = torch.zeros(max(rows, 64), dtype=torch.int32, device=device)
    if scratch is None or scratch.numel() < need:
        scratch = torch.empty(max(need, 1), dtype=torch.float32, device=device)
    _SAMPLE_SCRATCH[device] = (counters, scratch)
    return counters, scratch
