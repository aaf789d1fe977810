"""Host-side front end of the scaled-dot custom calls.

Mirrors, for this one path, what XLA does around `__cublas$lt$matmul$f8`:
`GemmBackendConfig` (xla/service/gpu/backend_configs.proto:88-135) carries the per-op
configuration, `ScaledDotCall` plays the part of the thunk for one call site (operands and
results in the order fixed by xla/service/gpu/thunk_emitter.cc:776-862, driven through the FFI
stages like xla/backends/gpu/runtime/custom_call_thunk.cc:451-560), and
`cublas_lt_matmul_f8` is the one-shot convenience wrapper tests and benchmarks use.

Everything goes through the C ABI of libb200_scaled_dot.so by way of XLA FFI call frames; torch
tensors only supply device memory and the stream.
"""

from __future__ import annotations

import ctypes as C
import dataclasses
import enum
from typing import NamedTuple, Optional, Sequence

from . import _native

# XLA PrimitiveType / XLA_FFI_DataType numbers (xla/ffi/api/c_api.h:233-266).
PRED, S8, S32, S64, F16, F32, F64, BF16, F8E5M2, F8E4M3FN = 1, 2, 4, 5, 10, 11, 12, 16, 19, 20
F8E8M0FNU = 33

TARGET_F8 = "b200$scaled_dot$f8"
TARGET_S8 = "b200$dot$s8"
TARGET_MX = "b200$block_scaled_dot$mx"
MX_BLOCK_SIZE = 32  # BlockScalingRewriter::kBlockSizeMXFP8, xla/backends/gpu/transforms/block_scaling_rewriter.h
XLA_WORKSPACE_BYTES = 32 * 1024 * 1024  # GemmConfig::kHopperWorkspace, xla/service/gpu/matmul_utils.h:103

_STAGE_INSTANTIATE, _STAGE_PREPARE, _STAGE_INITIALIZE, _STAGE_EXECUTE = 0, 1, 2, 3


class Epilogue(enum.IntEnum):
    """GemmBackendConfig.Epilogue (backend_configs.proto:106-117)."""

    DEFAULT = 0
    BIAS = 1
    RELU = 2
    BIAS_RELU = 3
    GELU = 4
    GELU_AUX = 5
    BIAS_GELU = 6
    BIAS_GELU_AUX = 7
    SILU = 8
    BIAS_SILU = 9

    @property
    def adds_vector_bias(self) -> bool:
        return self in (Epilogue.BIAS, Epilogue.BIAS_RELU, Epilogue.BIAS_GELU, Epilogue.BIAS_GELU_AUX)


@dataclasses.dataclass
class GemmBackendConfig:
    """The fields of xla.gpu.GemmBackendConfig this path reads."""

    alpha_real: float = 1.0
    alpha_imag: float = 0.0
    beta: float = 0.0
    lhs_contracting_dimensions: Sequence[int] = (1,)
    rhs_contracting_dimensions: Sequence[int] = (0,)
    lhs_batch_dimensions: Sequence[int] = ()      # () or (0,): one leading batch dimension on a, b, c and D
    rhs_batch_dimensions: Sequence[int] = ()
    epilogue: Epilogue = Epilogue.DEFAULT
    damax_output: bool = False
    lhs_stride: Optional[int] = None      # elements between batch entries; only the dense rows * cols the reference writes is accepted
    rhs_stride: Optional[int] = None
    selected_algorithm: int = 0  # 0 automatic; 1 dense; 2 split-K; 3 dense single-CTA; 4 dense CTA-pair


class XlaFfiError(RuntimeError):
    """A non-OK XLA_FFI_Error returned by a handler (code = absl::StatusCode number)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code
        self.message = message


INVALID_ARGUMENT, NOT_FOUND, UNIMPLEMENTED, INTERNAL = 3, 5, 12, 13


class Buffer(NamedTuple):
    """What an XLA_FFI_Buffer carries: element type, dims, device address (0 = not bound yet)."""

    dtype: int
    dims: Sequence[int]
    data: int = 0


def _torch():
    import torch

    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    table = {
        torch.float8_e4m3fn: F8E4M3FN, torch.float8_e5m2: F8E5M2, torch.int8: S8, torch.int32: S32,
        torch.float16: F16, torch.float32: F32, torch.bfloat16: BF16,
    }
    if hasattr(torch, "float8_e8m0fnu"):
        table[torch.float8_e8m0fnu] = F8E8M0FNU
    return table[t]


def as_buffer(x) -> Buffer:
    if isinstance(x, Buffer):
        return x
    if not x.is_contiguous():
        raise ValueError("custom-call operands are dense row-major buffers; got a non-contiguous tensor")
    return Buffer(_dtype_code(x.dtype), tuple(x.shape), x.data_ptr())


def _err_buf():
    return C.create_string_buffer(1024)


class FfiCall:
    """One custom-call site bound to a target registered with the (mock) XLA FFI runtime."""

    def __init__(self, target: str, operands: Sequence, results: Sequence, attrs: dict):
        _native.ensure_registered()
        self._h = _native.mock.mockffi_call_new(target.encode())
        self.target = target
        self._keep = []
        for op in operands:
            b = as_buffer(op)
            dims = (C.c_int64 * max(1, len(b.dims)))(*b.dims)
            _native.mock.mockffi_call_add_arg(self._h, b.dtype, b.data, len(b.dims), dims)
        for r in results:
            b = as_buffer(r)
            dims = (C.c_int64 * max(1, len(b.dims)))(*b.dims)
            _native.mock.mockffi_call_add_ret(self._h, b.dtype, b.data, len(b.dims), dims)
        for name, value in attrs.items():
            self._add_attr(name, value)

    def _add_attr(self, name: str, value) -> None:
        n = name.encode()
        m = _native.mock
        if isinstance(value, tuple) and len(value) == 2 and value[0] in ("i32", "f32", "i64", "f64"):
            kind, v = value
            {"i32": m.mockffi_call_attr_i32, "f32": m.mockffi_call_attr_f32,
             "i64": m.mockffi_call_attr_i64, "f64": m.mockffi_call_attr_f64}[kind](self._h, n, v)
        elif isinstance(value, bool):
            m.mockffi_call_attr_bool(self._h, n, int(value))
        elif isinstance(value, int):
            m.mockffi_call_attr_i64(self._h, n, value)
        elif isinstance(value, float):
            m.mockffi_call_attr_f64(self._h, n, value)
        elif isinstance(value, str):
            m.mockffi_call_attr_str(self._h, n, value.encode())
        elif isinstance(value, (list, tuple)):
            arr = (C.c_int64 * max(1, len(value)))(*value)
            m.mockffi_call_attr_i64_array(self._h, n, arr, len(value))
        else:
            raise TypeError(f"unsupported attribute type for {name}: {type(value)}")

    def _check(self, rc: int, err) -> None:
        if rc != 0:
            raise XlaFfiError(rc, err.value.decode(errors="replace"))

    def invoke_stage(self, stage: int, stream: int = 0, device: int = 0) -> None:
        err = _err_buf()
        self._check(_native.mock.mockffi_call_invoke(self._h, stage, stream, device, err, len(err)), err)

    def instantiate(self) -> None:
        self.invoke_stage(_STAGE_INSTANTIATE)

    def run(self, stream: int = 0, device: int = 0) -> None:
        """instantiate (first time) -> prepare -> initialize -> execute."""
        err = _err_buf()
        self._check(_native.mock.mockffi_call_run(self._h, stream, device, err, len(err)), err)

    def execute(self, stream: int = 0, device: int = 0) -> None:
        err = _err_buf()
        self._check(_native.mock.mockffi_call_execute(self._h, stream, device, err, len(err)), err)

    def set_operand(self, index: int, tensor) -> None:
        _native.mock.mockffi_call_set_arg_data(self._h, index, tensor.data_ptr())

    def set_result(self, index: int, tensor) -> None:
        _native.mock.mockffi_call_set_ret_data(self._h, index, tensor.data_ptr())

    def close(self) -> None:
        if self._h:
            _native.mock.mockffi_call_free(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _config_attrs(cfg: GemmBackendConfig) -> dict:
    if len(cfg.lhs_contracting_dimensions) != 1 or len(cfg.rhs_contracting_dimensions) != 1:
        raise XlaFfiError(INVALID_ARGUMENT, "exactly one contracting dimension per operand")
    batch = {}
    if tuple(cfg.lhs_batch_dimensions) or tuple(cfg.rhs_batch_dimensions):
        batch = {"lhs_batch_dims": list(cfg.lhs_batch_dimensions), "rhs_batch_dims": list(cfg.rhs_batch_dimensions)}
    if cfg.lhs_stride is not None:
        batch["lhs_stride"] = int(cfg.lhs_stride)
    if cfg.rhs_stride is not None:
        batch["rhs_stride"] = int(cfg.rhs_stride)
    return {
        **batch,
        "alpha_real": float(cfg.alpha_real),
        "alpha_imag": float(cfg.alpha_imag),
        "beta": float(cfg.beta),
        "epilogue": ("i32", int(cfg.epilogue)),
        "lhs_contracting_dim": int(cfg.lhs_contracting_dimensions[0]),
        "rhs_contracting_dim": int(cfg.rhs_contracting_dimensions[0]),
        "damax_output": bool(cfg.damax_output),
        "selected_config": int(cfg.selected_algorithm),
    }


class ScaledDotCall(FfiCall):
    """A `b200$scaled_dot$f8` call site.

    operands: a, b, [c], a_scale, b_scale, [bias], [d_scale]; results: D, [amax], [workspace] --
    the arrangement of `__cublas$lt$matmul$f8`.
    """

    def __init__(self, operands: Sequence, results: Sequence, config: GemmBackendConfig):
        super().__init__(TARGET_F8, operands, results, _config_attrs(config))
        self.config = config


class Int8DotCall(FfiCall):
    """A `b200$dot$s8` call site: operands a, b, [a_row_scale, b_col_scale]; results D, [acc s32],
    [workspace].  Rank-3 operands carry one leading batch dimension (`batched=True` sets
    lhs_batch_dims = rhs_batch_dims = {0}; the contracting dimensions then index the rank-3 operand)."""

    def __init__(self, operands: Sequence, results: Sequence, *, lhs_contracting_dim=1, rhs_contracting_dim=0,
                 emit_s32=False, selected_algorithm=0, batched=False):
        attrs = {
            "lhs_contracting_dim": int(lhs_contracting_dim),
            "rhs_contracting_dim": int(rhs_contracting_dim),
            "emit_s32": bool(emit_s32),
            "selected_config": int(selected_algorithm),
        }
        if batched:
            attrs.update({"lhs_batch_dims": [0], "rhs_batch_dims": [0]})
        super().__init__(TARGET_S8, operands, results, attrs)


class BlockScaledDotCall(FfiCall):
    """A `b200$block_scaled_dot$mx` call site: operands a, b, a_scale, b_scale; results D,
    [workspace] -- the arrangement of `__cublas$lt$matmul$mx`
    (xla/service/gpu/thunk_emitter.cc:939-988)."""

    def __init__(self, operands: Sequence, results: Sequence, *, alpha_real: float = 1.0, selected_algorithm: int = 0,
                 block_size: Optional[int] = None):
        attrs = {"alpha_real": float(alpha_real), "selected_config": int(selected_algorithm)}
        if block_size is not None:      # block_scaled_dot_backend_config.block_size: states the block size, allows padded scale columns
            attrs["block_size"] = int(block_size)
        super().__init__(TARGET_MX, operands, results, attrs)


def _current_stream_and_device(t):
    torch = _torch()
    dev = t.device.index if t.device.index is not None else torch.cuda.current_device()
    return torch.cuda.current_stream(dev).cuda_stream, dev


def cublas_lt_matmul_f8(a, b, a_scale, b_scale, *, c=None, bias=None, d_scale=None, out_dtype=None,
                        config: Optional[GemmBackendConfig] = None, workspace=None, out=None, amax_out=None):
    """Runs one scaled dot on the current CUDA stream and returns (D, amax or None).

    a, b: torch float8 tensors; a_scale, b_scale, d_scale: f32 scalar tensors on the device.
    """
    torch = _torch()
    cfg = config or GemmBackendConfig()
    lc, rc = cfg.lhs_contracting_dimensions[0], cfg.rhs_contracting_dimensions[0]
    bo = 1 if tuple(cfg.lhs_batch_dimensions) else 0          # contracting dimensions index the rank-3 operand then
    m, n = a.shape[bo + 1 - (lc - bo)], b.shape[bo + 1 - (rc - bo)]
    out_dtype = out_dtype or torch.bfloat16
    d = out if out is not None else torch.empty(tuple(a.shape[:bo]) + (m, n), dtype=out_dtype, device=a.device)
    operands = [a, b]
    if cfg.beta != 0.0:
        operands.append(c)
    operands += [a_scale, b_scale]
    if cfg.epilogue.adds_vector_bias:
        operands.append(bias)
    if d.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        operands.append(d_scale if d_scale is not None else torch.ones((), dtype=torch.float32, device=a.device))
    results = [d]
    amax = None
    if cfg.damax_output:
        amax = amax_out if amax_out is not None else torch.empty((), dtype=torch.float32, device=a.device)
        results.append(amax)
    if workspace is None:
        workspace = torch.empty(XLA_WORKSPACE_BYTES, dtype=torch.int8, device=a.device)
    results.append(workspace)
    call = ScaledDotCall(operands, results, cfg)
    stream, dev = _current_stream_and_device(a)
    call.run(stream, dev)
    call.close()
    return d, amax


def cublas_lt_matmul_s8(a, b, *, a_row_scale=None, b_col_scale=None, out_dtype=None, emit_s32=False,
                        lhs_contracting_dim=None, rhs_contracting_dim=None, selected_algorithm=0, workspace=None):
    """s8 x s8 dot; returns (D, acc or None).  `workspace` (an int8 tensor) becomes the trailing
    scratch result of the call site, as in XLA.  Rank-3 operands are a batch of dots (leading
    dimension); the contracting dimensions index the operands as given (default: the last of a, the
    first matrix dimension of b)."""
    torch = _torch()
    bo = a.dim() - 2
    lc = bo + 1 if lhs_contracting_dim is None else lhs_contracting_dim
    rc = bo if rhs_contracting_dim is None else rhs_contracting_dim
    m, n = a.shape[2 * bo + 1 - lc], b.shape[2 * bo + 1 - rc]
    lead = tuple(a.shape[:bo])
    out_dtype = out_dtype or (torch.int32 if a_row_scale is None else torch.bfloat16)
    d = torch.empty(lead + (m, n), dtype=out_dtype, device=a.device)
    operands = [a, b] + ([a_row_scale, b_col_scale] if a_row_scale is not None else [])
    results = [d]
    acc = None
    if emit_s32:
        acc = torch.empty(lead + (m, n), dtype=torch.int32, device=a.device)
        results.append(acc)
    if workspace is not None:
        results.append(workspace)
    call = Int8DotCall(operands, results, lhs_contracting_dim=lc, rhs_contracting_dim=rc, emit_s32=emit_s32,
                       selected_algorithm=selected_algorithm, batched=bo == 1)
    stream, dev = _current_stream_and_device(a)
    call.run(stream, dev)
    call.close()
    return d, acc


def cublas_lt_matmul_mx(a, b, a_scale, b_scale, *, out_dtype=None, alpha_real: float = 1.0, workspace=None, out=None,
                        selected_algorithm: int = 0, block_size: Optional[int] = None):
    """Runs one MX block-scaled dot on the current CUDA stream and returns D.

    a: [m, k] or [batch, m, k] float8; b: [n, k] or [batch, n, k] float8 (the contracting dimension is
    the minor one of both, as `__op$block_scaled_dot` fixes it); a_scale / b_scale: [..., rows, k / 32]
    float8_e8m0fnu (uint8 tensors holding the code points are taken as such).  Scale tensors may be
    padded: extra rows always, extra columns when `block_size=32` states the block size (otherwise it
    is implied by the shapes); only the leading [rows, k / 32] corner is used, like the slice in
    xla/backends/gpu/transforms/block_scaling_rewriter.cc:469-518."""
    torch = _torch()
    out_dtype = out_dtype or torch.float32
    lead = tuple(a.shape[:-2])
    d = out if out is not None else torch.empty(lead + (a.shape[-2], b.shape[-2]), dtype=out_dtype, device=a.device)

    def scale_buffer(s):
        if s.dtype == torch.uint8:
            return Buffer(F8E8M0FNU, tuple(s.shape), s.data_ptr())
        return s

    operands = [a, b, scale_buffer(a_scale), scale_buffer(b_scale)]
    results = [d] + ([workspace] if workspace is not None else [])
    call = BlockScaledDotCall(operands, results, alpha_real=alpha_real, selected_algorithm=selected_algorithm, block_size=block_size)
    stream, dev = _current_stream_and_device(a)
    call.run(stream, dev)
    call.close()
    return d


def device_status() -> int:
    """Synchronises the device and returns (and clears) the kernels' error bit mask."""
    bits = C.c_uint32(0)
    err = _err_buf()
    rc = _native.product.b200sd_device_status(C.byref(bits), err, len(err))
    if rc != 0:
        raise XlaFfiError(rc, err.value.decode(errors="replace"))
    return bits.value


def launch_count() -> int:
    return int(_native.product.b200sd_launch_count())


def load_config_table(path: str) -> int:
    """Loads a tuned kernel-choice table (see `python -m xla_b200.autotune`); returns the number of entries."""
    n = C.c_int32(0)
    err = _err_buf()
    rc = _native.product.b200sd_load_config_table(str(path).encode(), C.byref(n), err, len(err))
    if rc != 0:
        raise XlaFfiError(rc, err.value.decode(errors="replace"))
    return n.value


def select_kernel(m: int, n: int, k: int) -> int:
    """What selected_config = 0 resolves to for an FP8 dot of this shape."""
    return int(_native.product.b200sd_select_kernel(m, n, k))


def tuned_kernel_mx(m: int, n: int, k: int) -> int:
    """The tile form (6 / 7) the tuned table holds for an MX block-scaled dot of this shape; 0 when it has none and
    the launch decides."""
    return int(_native.product.b200sd_tuned_kernel_mx(m, n, k))
