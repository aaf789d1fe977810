"""ctypes bindings of libb200_scaled_dot.so and of the FFI test harness libb200_mock_ffi.so."""

from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_DIR = os.path.join(_HERE, "lib")
# B200SD_LIBRARY names another build of the same library (the tuning build with its wait counters).
PRODUCT_LIB = os.environ.get("B200SD_LIBRARY") or os.path.join(LIB_DIR, "libb200_scaled_dot.so")
MOCK_LIB = os.path.join(LIB_DIR, "libb200_mock_ffi.so")


class NativeLibraryMissing(ImportError):
    pass


def _load(path: str) -> C.CDLL:
    if not os.path.exists(path):
        raise NativeLibraryMissing(
            f"{path} has not been built.  Run `python -c 'import __graft_entry__ as g; g.build()'` "
            "(or `make -C xla_b200/csrc`).  There is no fallback implementation."
        )
    return C.CDLL(path, mode=C.RTLD_GLOBAL)


class ScaledDotF8Args(C.Structure):
    """B200SD_ScaledDotF8 of include/b200_scaled_dot.h."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("bias", C.c_void_p),
        ("a_scale", C.c_void_p), ("b_scale", C.c_void_p), ("d_scale", C.c_void_p),
        ("d", C.c_void_p), ("amax", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a_dtype", C.c_int32), ("b_dtype", C.c_int32),
        ("c_dtype", C.c_int32), ("bias_dtype", C.c_int32),
        ("d_dtype", C.c_int32),
        ("lhs_contracting_dim", C.c_int32), ("rhs_contracting_dim", C.c_int32),
        ("epilogue", C.c_int32),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("kernel", C.c_int32),
        ("batch_count", C.c_int32),
    ]


class DotS8Args(C.Structure):
    """B200SD_DotS8 of include/b200_scaled_dot.h."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("a", C.c_void_p), ("b", C.c_void_p),
        ("a_row_scale", C.c_void_p), ("b_col_scale", C.c_void_p),
        ("d", C.c_void_p), ("acc_out", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("d_dtype", C.c_int32),
        ("lhs_contracting_dim", C.c_int32), ("rhs_contracting_dim", C.c_int32),
        ("kernel", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("batch_count", C.c_int64),
    ]


class BlockScaledDotMxArgs(C.Structure):
    """B200SD_BlockScaledDotMx of include/b200_scaled_dot.h."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("a", C.c_void_p), ("b", C.c_void_p), ("a_scale", C.c_void_p), ("b_scale", C.c_void_p),
        ("d", C.c_void_p),
        ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64),
        ("a_dtype", C.c_int32), ("b_dtype", C.c_int32), ("scale_dtype", C.c_int32), ("d_dtype", C.c_int32),
        ("alpha", C.c_float),
        ("batch_count", C.c_int32),
        ("kernel", C.c_int32),
        ("a_scale_rows", C.c_int64), ("a_scale_cols", C.c_int64),
        ("b_scale_rows", C.c_int64), ("b_scale_cols", C.c_int64),
    ]


class ProgressArgs(C.Structure):
    """B200SD_Progress of include/b200_scaled_dot.h."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("counters", C.c_void_p),
        ("rows_per_block", C.c_int32), ("max_ctas", C.c_int32),
        ("num_blocks", C.c_int32), ("increment", C.c_uint32), ("last_increment", C.c_uint32),
    ]


class PeerReduceArgs(C.Structure):
    """B200SD_PeerReduce of include/b200_scaled_dot.h."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("world", C.c_int32), ("rank", C.c_int32), ("emulate_ranks", C.c_int32), ("epoch", C.c_uint32),
        ("d", C.c_void_p * 8), ("stage", C.c_void_p * 8), ("flags", C.c_void_p * 8),
        ("emu_a", C.c_void_p * 8), ("emu_b", C.c_void_p * 8),
        ("d_multicast", C.c_void_p),
        ("peer_wait_ms", C.c_uint32),
        ("pull", C.c_int32),
        ("stage_multicast", C.c_void_p),
    ]


product = _load(PRODUCT_LIB)
mock = _load(MOCK_LIB)

_ERR = (C.c_char_p, C.c_size_t)
product.b200sd_init_device.argtypes = [*_ERR]
product.b200sd_scaled_dot_f8.argtypes = [C.POINTER(ScaledDotF8Args), C.c_void_p, *_ERR]
product.b200sd_dot_s8.argtypes = [C.POINTER(DotS8Args), C.c_void_p, *_ERR]
product.b200sd_check_scaled_dot_f8.argtypes = [C.POINTER(ScaledDotF8Args), *_ERR]
product.b200sd_check_dot_s8.argtypes = [C.POINTER(DotS8Args), *_ERR]
product.b200sd_block_scaled_dot_mx.argtypes = [C.POINTER(BlockScaledDotMxArgs), C.c_void_p, *_ERR]
product.b200sd_check_block_scaled_dot_mx.argtypes = [C.POINTER(BlockScaledDotMxArgs), *_ERR]
product.b200sd_workspace_bytes.argtypes = [C.c_int64, C.c_int64, C.c_int64]
product.b200sd_workspace_bytes.restype = C.c_size_t
product.b200sd_select_kernel.argtypes = [C.c_int64, C.c_int64, C.c_int64]
product.b200sd_tuned_kernel_mx.argtypes = [C.c_int64, C.c_int64, C.c_int64]
product.b200sd_load_config_table.argtypes = [C.c_char_p, C.POINTER(C.c_int32), *_ERR]
product.b200sd_launch_count.restype = C.c_uint64
product.b200sd_device_status.argtypes = [C.POINTER(C.c_uint32), *_ERR]
product.b200sd_wait_probe.argtypes = [C.c_uint64, C.c_void_p, *_ERR]
product.b200sd_ffi_register.argtypes = [C.c_void_p, *_ERR]
product.b200sd_scaled_dot_f8_decode_noalloc.argtypes = [C.POINTER(ScaledDotF8Args), C.c_void_p, *_ERR]
product.b200sd_noalloc_scratch_bytes.restype = C.c_size_t
product.b200sd_scaled_dot_f8_progress.argtypes = [C.POINTER(ScaledDotF8Args), C.POINTER(ProgressArgs), C.c_void_p, *_ERR]
product.b200sd_stream_wait_counter.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, *_ERR]
product.b200sd_scaled_dot_f8_peer_reduce.argtypes = [C.POINTER(ScaledDotF8Args), C.POINTER(PeerReduceArgs), C.c_void_p, *_ERR]
product.b200sd_peer_reduce_flag_words.argtypes = [C.c_int64, C.c_int64, C.c_int32]
product.b200sd_peer_reduce_flag_words.restype = C.c_size_t
product.b200sd_rewrite_hlo.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t, C.c_char_p, C.c_size_t, *_ERR]

mock.mockffi_api.restype = C.c_void_p
mock.mockffi_load_library.argtypes = [C.c_char_p, C.c_char_p, *_ERR]
mock.mockffi_find_handler.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint32), C.POINTER(C.c_int)]
mock.mockffi_call_new.argtypes = [C.c_char_p]
mock.mockffi_call_new.restype = C.c_void_p
mock.mockffi_call_free.argtypes = [C.c_void_p]
for _name in ("mockffi_call_add_arg", "mockffi_call_add_ret"):
    getattr(mock, _name).argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.POINTER(C.c_int64)]
for _name in ("mockffi_call_set_arg_data", "mockffi_call_set_ret_data"):
    getattr(mock, _name).argtypes = [C.c_void_p, C.c_int, C.c_void_p]
mock.mockffi_call_attr_i64.argtypes = [C.c_void_p, C.c_char_p, C.c_int64]
mock.mockffi_call_attr_i32.argtypes = [C.c_void_p, C.c_char_p, C.c_int32]
mock.mockffi_call_attr_f64.argtypes = [C.c_void_p, C.c_char_p, C.c_double]
mock.mockffi_call_attr_f32.argtypes = [C.c_void_p, C.c_char_p, C.c_float]
mock.mockffi_call_attr_bool.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
mock.mockffi_call_attr_str.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
mock.mockffi_call_attr_i64_array.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int64), C.c_size_t]
mock.mockffi_call_invoke.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, *_ERR]
mock.mockffi_call_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, *_ERR]
mock.mockffi_call_execute.argtypes = [C.c_void_p, C.c_void_p, C.c_int, *_ERR]

_registered = False


def ensure_registered() -> None:
    """Registers the product's handler bundles with the mock XLA runtime (once per process)."""
    global _registered
    if _registered:
        return
    err = C.create_string_buffer(512)
    rc = product.b200sd_ffi_register(mock.mockffi_api(), err, len(err))
    if rc != 0:
        raise RuntimeError(f"FFI registration failed ({rc}): {err.value.decode()}")
    _registered = True
