"""Host-only tests of the drop-in boundary: the shared library loads, exports every symbol the
public header declares, registers with an XLA FFI runtime, and validates call frames at the
`instantiate` stage (no device access) the way xla/ffi/api/ffi_test.cc exercises handlers --
by building call frames by hand."""
import ctypes as C
import os
import re

import pytest

import xla_b200
from xla_b200 import _native
from xla_b200.scaled_dot import (BF16, F16, F32, F8E4M3FN, F8E5M2, S8, S32, Buffer, Epilogue, FfiCall,
                                 GemmBackendConfig, Int8DotCall, ScaledDotCall, XlaFfiError)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_every_declared_symbol_is_exported():
    header = open(os.path.join(ROOT, "include", "b200_scaled_dot.h")).read()
    names = set(re.findall(r"\b(b200sd_[a-z0-9_]+)\s*\(", header))
    assert len(names) >= 15
    for n in sorted(names):
        assert hasattr(_native.product, n), f"{n} is declared in the header but not exported"


def test_interface_numbers_are_the_reference_s():
    """Every enum the boundary shares with XLA carries XLA's own numbers: GemmBackendConfig.Epilogue
    (backend_configs.proto:106-117), XLA_FFI_DataType and XLA_FFI_Error_Code (xla/ffi/api/c_api.h),
    as extracted from the reference tree into tests/golden/interface_enums.json."""
    import json

    from oracle import scaled_dot_oracle as o

    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "interface_enums.json")))
    header = open(os.path.join(ROOT, "include", "b200_scaled_dot.h")).read()
    in_header = {k: int(v) for k, v in re.findall(r"\bB200SD_EPILOGUE_([A-Z_]+)\s*=\s*(\d+)", header)}
    assert in_header == golden["epilogue"]["values"]            # all ten, DEFAULT = 0 ... BIAS_SILU = 9
    assert {e.name: int(e) for e in Epilogue} == golden["epilogue"]["values"]
    for name in ("DEFAULT", "BIAS", "RELU", "BIAS_RELU", "GELU", "GELU_AUX", "BIAS_GELU", "BIAS_GELU_AUX"):
        assert getattr(o, "EPI_" + name) == golden["epilogue"]["values"][name]
    types_in_header = {k: int(v) for k, v in re.findall(r"\bB200SD_(S8|S32|F16|F32|BF16|F8E5M2|F8E4M3FN|F8E8M0FNU)\s*=\s*(\d+)", header)}
    assert len(types_in_header) >= 7
    for name, number in types_in_header.items():
        assert golden["data_type"]["values"][name] == number
    for name, number in dict(S8=S8, S32=S32, F16=F16, F32=F32, BF16=BF16, F8E5M2=F8E5M2, F8E4M3FN=F8E4M3FN).items():
        assert golden["data_type"]["values"][name] == number
    kernels_h = open(os.path.join(ROOT, "xla_b200", "csrc", "kernels.h")).read()
    for cname, gname in (("kInvalidArgument", "INVALID_ARGUMENT"), ("kUnimplemented", "UNIMPLEMENTED"), ("kInternal", "INTERNAL"),
                         ("kFailedPrecondition", "FAILED_PRECONDITION"), ("kResourceExhausted", "RESOURCE_EXHAUSTED"),
                         ("kDeadlineExceeded", "DEADLINE_EXCEEDED")):
        assert int(re.search(cname + r"\s*=\s*(\d+)", kernels_h).group(1)) == golden["error_code"]["values"][gname]


def test_call_target_names_are_the_reference_s():
    """The custom-call names this library stands in for (`__cublas$lt$matmul$f8`, `$mx`) or consumes
    (`__op$block_scaled_dot`) and the MX block size, as xla/service/gpu/cublas_cudnn.h:119-131 and
    block_scaling_rewriter.h:86-95 spell them (tests/golden/interface_enums.json)."""
    import json

    from oracle import scaled_dot_oracle as o

    golden = json.load(open(os.path.join(ROOT, "tests", "golden", "interface_enums.json")))
    names = golden["call_targets"]
    assert names["kCublasLtMatmulF8CallTarget"] == "__cublas$lt$matmul$f8" and names["kCublasLtMatmulMxCallTarget"] == "__cublas$lt$matmul$mx"
    rewriter = open(os.path.join(ROOT, "xla_b200", "csrc", "hlo_rewriter.cc")).read()
    assert '\\"' + names["kBlockScaledDotCustomCallTarget"] + '\\"' in rewriter          # the call the rewriter-lite looks for
    evaluator = open(os.path.join(ROOT, "oracle", "hlo_eval.py")).read()
    assert '"' + names["kBlockScaledDotCustomCallTarget"] + '"' in evaluator
    header = open(os.path.join(ROOT, "include", "b200_scaled_dot.h")).read()
    for key in ("kCublasLtMatmulMxCallTarget",):
        assert names[key] in header
    integration = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    for key in ("kCublasLtMatmulF8CallTarget", "kCublasLtMatmulMxCallTarget", "kCublasLtMatmulCallTarget"):
        assert names[key] in integration
    assert o.MX_BLOCK == golden["block_size_mxfp8"] == 32
    # nothing of this library registers under a reference name
    for target in ("b200$scaled_dot$f8", "b200$dot$s8", "b200$block_scaled_dot$mx"):
        assert target not in names.values()


def test_reference_epilogue_numbers_decode_as_the_reference_means_them():
    """A call frame carrying the reference's own numbers: 0 (DEFAULT) is accepted without a bias operand,
    6 (BIAS_GELU) wants the bias, 5 / 7 (the AUX forms) and 8 / 9 (SILU) are UNIMPLEMENTED, 10 is unknown."""
    ops, res = _f8_frame()
    FfiCall("b200$scaled_dot$f8", ops, res, {"epilogue": ("i32", 0)}).instantiate()
    FfiCall("b200$scaled_dot$f8", ops, res, {}).instantiate()                      # absent = DEFAULT
    with pytest.raises(XlaFfiError) as e:
        FfiCall("b200$scaled_dot$f8", ops, res, {"epilogue": ("i32", 6)}).instantiate()
    assert e.value.code == 3 and "operands" in str(e.value)
    FfiCall("b200$scaled_dot$f8", ops + [Buffer(BF16, (256,))], res, {"epilogue": ("i32", 6)}).instantiate()
    FfiCall("b200$scaled_dot$f8", ops + [Buffer(BF16, (256,))], res, {"epilogue": ("i32", 1)}).instantiate()
    for number, with_bias in ((5, False), (7, True), (8, False), (9, False)):
        with pytest.raises(XlaFfiError) as e:
            FfiCall("b200$scaled_dot$f8", ops + ([Buffer(BF16, (256,))] if with_bias else []), res,
                    {"epilogue": ("i32", number)}).instantiate()
        assert e.value.code == 12, (number, str(e.value))
    with pytest.raises(XlaFfiError) as e:
        FfiCall("b200$scaled_dot$f8", ops, res, {"epilogue": ("i32", 10)}).instantiate()
    assert e.value.code == 3


def test_struct_layouts_match_the_header():
    """The ctypes mirrors must have the C structs' sizes (checked through struct_size validation)."""
    err = C.create_string_buffer(256)
    a = _native.ScaledDotF8Args()
    a.struct_size = C.sizeof(a) - 8
    assert _native.product.b200sd_check_scaled_dot_f8(C.byref(a), err, len(err)) == 3
    assert b"struct_size" in err.value
    s = _native.DotS8Args()
    s.struct_size = 8
    assert _native.product.b200sd_check_dot_s8(C.byref(s), err, len(err)) == 3


def test_block_scaled_entry_point_validates_without_a_device():
    """b200sd_check_block_scaled_dot_mx: everything but the pointers, no device access."""
    err = C.create_string_buffer(256)
    chk = _native.product.b200sd_check_block_scaled_dot_mx

    def args(**kw):
        a = _native.BlockScaledDotMxArgs(struct_size=C.sizeof(_native.BlockScaledDotMxArgs), m=256, n=512, k=256, a_dtype=20, b_dtype=19,
                                         scale_dtype=33, d_dtype=16, alpha=1.0, batch_count=0)
        for k_, v in kw.items():
            setattr(a, k_, v)
        return a

    assert chk(C.byref(args()), err, len(err)) == 0, err.value
    assert chk(C.byref(args(batch_count=4, d_dtype=11)), err, len(err)) == 0
    for bad, code in [(dict(struct_size=16), 3), (dict(k=250), 3), (dict(scale_dtype=20), 12), (dict(a_dtype=2), 12), (dict(d_dtype=20), 3),
                      (dict(m=0), 3), (dict(batch_count=-1), 3)]:
        assert chk(C.byref(args(**bad)), err, len(err)) == code, (bad, err.value)
    assert chk(None, err, len(err)) == 3


def test_registration_and_metadata():
    _native.ensure_registered()
    traits, minor = C.c_uint32(0), C.c_int(0)
    for target in (b"b200$scaled_dot$f8", b"b200$dot$s8", b"b200$block_scaled_dot$mx"):
        assert _native.mock.mockffi_find_handler(target, b"CUDA", C.byref(traits), C.byref(minor)) == 1
        assert traits.value & 1           # XLA_FFI_HANDLER_TRAITS_COMMAND_BUFFER_COMPATIBLE
        assert 1 <= minor.value <= 4      # API versions the XLA runtime accepts (ffi_registry.cc:47-65)
    assert _native.mock.mockffi_find_handler(b"b200$scaled_dot$f8", b"Host", None, None) == 0
    # Registering twice is refused, as XLA's registry does.
    err = C.create_string_buffer(256)
    assert _native.product.b200sd_ffi_register(_native.mock.mockffi_api(), err, len(err)) == 6   # ALREADY_EXISTS


def _f8_frame(m=256, k=512, n=256, *, a=F8E4M3FN, b=F8E4M3FN, d=BF16, extra_ops=(), extra_res=(Buffer(S8, (1 << 20,)),),
              lc=1, rc=0):
    a_dims = (m, k) if lc == 1 else (k, m)
    b_dims = (k, n) if rc == 0 else (n, k)
    ops = [Buffer(a, a_dims), Buffer(b, b_dims), Buffer(F32, ()), Buffer(F32, ())] + list(extra_ops)
    return ops, [Buffer(d, (m, n))] + list(extra_res)


@pytest.mark.parametrize("case", [
    # every operand/result arrangement FileCheck'd in gemm_rewriter_fp8_test.cc (lines in comments)
    dict(),                                                                               # :501  a,b,as,bs -> D,ws
    dict(cfg=dict(beta=1.0), ops_insert_c=True),                                           # :1370 matrix bias
    dict(cfg=dict(epilogue=Epilogue.BIAS), extra_ops=[Buffer(BF16, (256,))]),              # :1167 vector bias
    dict(cfg=dict(epilogue=Epilogue.BIAS_RELU), extra_ops=[Buffer(F16, (256,))]),          # :2031
    dict(cfg=dict(epilogue=Epilogue.BIAS_GELU), extra_ops=[Buffer(BF16, (256,))]),         # :2166
    dict(d=F8E4M3FN, extra_ops=[Buffer(F32, ())]),                                         # :1709 d_scale
    dict(d=F8E4M3FN, extra_ops=[Buffer(F32, ())], cfg=dict(damax_output=True),
         extra_res=[Buffer(F32, ()), Buffer(S8, (1 << 20,))]),                             # :2613 amax
    dict(d=F8E4M3FN, cfg=dict(epilogue=Epilogue.BIAS), extra_ops=[Buffer(BF16, (256,)), Buffer(F32, ())]),   # :1971
    dict(d=F8E4M3FN, cfg=dict(epilogue=Epilogue.BIAS_GELU, damax_output=True),
         extra_ops=[Buffer(BF16, (256,)), Buffer(F32, ())],
         extra_res=[Buffer(F32, ()), Buffer(S8, (1 << 20,))]),                             # BASELINE config 1
    dict(d=F8E4M3FN),                                                                      # :313  FP8 result, b_scale doubles as d_scale
    dict(extra_res=[]),                                                                    # no workspace result
    dict(b=F8E5M2, d=F8E5M2, extra_ops=[Buffer(F32, ())]),
    dict(lc=0, rc=1),
])
def test_accepted_arrangements_instantiate(case):
    ops, res = _f8_frame(a=case.get("a", F8E4M3FN), b=case.get("b", F8E4M3FN), d=case.get("d", BF16),
                         extra_ops=case.get("extra_ops", ()),
                         extra_res=case.get("extra_res", (Buffer(S8, (1 << 20,)),)),
                         lc=case.get("lc", 1), rc=case.get("rc", 0))
    if case.get("ops_insert_c"):
        ops.insert(2, Buffer(BF16, (256, 256)))
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(case.get("lc", 1),),
                            rhs_contracting_dimensions=(case.get("rc", 0),), **case.get("cfg", {}))
    ScaledDotCall(ops, res, cfg).instantiate()


def test_batched_frame_instantiates_and_mismatches_are_rejected():
    """gemm_rewriter_fp8_test.cc:941-991: rank-3 operands with one leading batch dimension."""
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,))
    ops = [Buffer(F8E4M3FN, (10, 16, 32)), Buffer(F8E4M3FN, (10, 32, 16)), Buffer(F32, ()), Buffer(F32, ())]
    ScaledDotCall(ops, [Buffer(F32, (10, 16, 16)), Buffer(S8, (1 << 20,))], cfg).instantiate()
    with pytest.raises(XlaFfiError) as e:
        ScaledDotCall(ops, [Buffer(F32, (9, 16, 16)), Buffer(S8, (1 << 20,))], cfg).instantiate()
    assert e.value.code == 3 and "batch" in e.value.message
    with pytest.raises(XlaFfiError) as e:                                   # batch attributes on rank-2 operands
        ScaledDotCall([Buffer(F8E4M3FN, (16, 32)), Buffer(F8E4M3FN, (32, 16)), Buffer(F32, ()), Buffer(F32, ())],
                      [Buffer(F32, (16, 16))], GemmBackendConfig(lhs_batch_dimensions=(0,), rhs_batch_dimensions=(0,))).instantiate()
    assert e.value.code == 3
    cfg2 = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(1,),
                             rhs_batch_dimensions=(0,))
    with pytest.raises(XlaFfiError) as e:                                   # only a LEADING batch dimension is implemented
        ScaledDotCall(ops, [Buffer(F32, (10, 16, 16))], cfg2).instantiate()
    assert e.value.code == 12


@pytest.mark.parametrize("mutate,code,needle", [
    (lambda o, r, c: o.__setitem__(0, Buffer(F8E5M2, (256, 512))) or o.__setitem__(1, Buffer(F8E5M2, (512, 256))), 12, "F8E5M2 x F8E5M2"),
    (lambda o, r, c: o.__setitem__(0, Buffer(BF16, (256, 512))), 3, "F8E4M3FN or F8E5M2"),
    (lambda o, r, c: o.__setitem__(1, Buffer(F8E4M3FN, (500, 256))), 3, "contracting dimensions"),
    (lambda o, r, c: r.__setitem__(0, Buffer(BF16, (256, 128))), 3, "result shape"),
    (lambda o, r, c: r.__setitem__(0, Buffer(S32, (256, 256))), 3, "output type"),
    (lambda o, r, c: o.__setitem__(2, Buffer(F32, (2,))), 3, "f32 scalars"),
    (lambda o, r, c: o.__setitem__(3, Buffer(BF16, ())), 3, "f32 scalars"),
    (lambda o, r, c: o.pop(), 3, "operands"),
    (lambda o, r, c: o.append(Buffer(F32, ())), 3, "operands"),
    (lambda o, r, c: setattr(c, "epilogue", Epilogue.BIAS), 3, "operands"),
    (lambda o, r, c: setattr(c, "epilogue", Epilogue.GELU_AUX), 12, "auxiliary"),
    (lambda o, r, c: setattr(c, "damax_output", True), 3, "amax result"),
    (lambda o, r, c: setattr(c, "lhs_contracting_dimensions", (2,)), 3, "lhs_contracting_dim"),
    (lambda o, r, c: o.__setitem__(0, Buffer(F8E4M3FN, (2, 256, 512))), 12, "rank 2"),
    (lambda o, r, c: (o.__setitem__(0, Buffer(F8E4M3FN, (250, 512))), r.__setitem__(0, Buffer(BF16, (250, 256)))), 3, "multiples of 16"),
    (lambda o, r, c: r.__setitem__(0, Buffer(F8E5M2, (256, 256))) or o.append(Buffer(F32, ())), 12, "type table"),
])
def test_rejected_call_frames(mutate, code, needle):
    """Bad dtypes / dims / attrs surface as XLA_FFI_Error with the right code at instantiate time;
    nothing is launched and nothing faults."""
    ops, res = _f8_frame()
    cfg = GemmBackendConfig()
    mutate(ops, res, cfg)
    with pytest.raises(XlaFfiError) as e:
        ScaledDotCall(ops, res, cfg).instantiate()
    assert e.value.code == code, e.value
    assert needle in e.value.message, e.value.message


def test_attribute_spellings():
    """Integer attributes may arrive as i32 or i64, floats as f32 or f64 (the MLIR dictionary a
    backend_config is parsed into keeps the written width: xla/service/gpu/custom_call_test.cc:554-577)."""
    ops, res = _f8_frame()
    for attrs in (
        {"epilogue": ("i32", 0), "lhs_contracting_dim": ("i32", 1), "rhs_contracting_dim": ("i64", 0), "beta": ("f32", 0.0)},
        {"epilogue": 0, "alpha_real": 1.0},
        {},
    ):
        FfiCall("b200$scaled_dot$f8", ops, res, attrs).instantiate()
    with pytest.raises(XlaFfiError):
        FfiCall("b200$scaled_dot$f8", ops, res, {"alpha_imag": 1.0}).instantiate()


def test_batch_strides_of_the_backend_config():
    """GemmBackendConfig.lhs_stride / rhs_stride (backend_configs.proto:121-122) are what the reference's rewriter
    always writes, rows * cols of one batch entry (gemm_rewriter.cc:705-721): accepted in that form, refused otherwise."""
    ops = [Buffer(F8E4M3FN, (2, 64, 128)), Buffer(F8E4M3FN, (2, 128, 32)), Buffer(F32, ()), Buffer(F32, ())]
    res = [Buffer(BF16, (2, 64, 32))]
    base = {"lhs_batch_dims": [0], "rhs_batch_dims": [0], "lhs_contracting_dim": 2, "rhs_contracting_dim": 1}
    FfiCall("b200$scaled_dot$f8", ops, res, dict(base, lhs_stride=64 * 128, rhs_stride=128 * 32)).instantiate()
    FfiCall("b200$scaled_dot$f8", ops[:1] + ops[1:], res, dict(base, lhs_stride=64 * 128)).instantiate()
    for bad in ({"lhs_stride": 64 * 128 + 16}, {"rhs_stride": 0}):
        with pytest.raises(XlaFfiError) as e:
            FfiCall("b200$scaled_dot$f8", ops, res, dict(base, **bad)).instantiate()
        assert e.value.code == 12 and "stride" in e.value.message
    # rank 2: the same fields describe the one matrix
    ops2, res2 = _f8_frame()
    a_dims, b_dims = ops2[0].dims, ops2[1].dims
    FfiCall("b200$scaled_dot$f8", ops2, res2, {"lhs_stride": a_dims[0] * a_dims[1], "rhs_stride": b_dims[0] * b_dims[1]}).instantiate()
    s8 = [Buffer(S8, (3, 64, 128)), Buffer(S8, (3, 128, 32))]
    Int8DotCall(s8, [Buffer(S32, (3, 64, 32))], batched=True, lhs_contracting_dim=2, rhs_contracting_dim=1).instantiate()
    with pytest.raises(XlaFfiError) as e:
        FfiCall("b200$dot$s8", s8, [Buffer(S32, (3, 64, 32))], dict(base, lhs_stride=1)).instantiate()
    assert e.value.code == 12


def test_int8_frames():
    Int8DotCall([Buffer(S8, (64, 128)), Buffer(S8, (128, 32))], [Buffer(S32, (64, 32))]).instantiate()
    Int8DotCall([Buffer(S8, (64, 128)), Buffer(S8, (128, 32)), Buffer(F32, (64,)), Buffer(F32, (32,))],
                [Buffer(BF16, (64, 32)), Buffer(S32, (64, 32))], emit_s32=True).instantiate()
    # one leading batch dimension, as for the FP8 call; contracting dimensions index the rank-3 operands
    Int8DotCall([Buffer(S8, (3, 64, 128)), Buffer(S8, (3, 128, 32))], [Buffer(S32, (3, 64, 32))], batched=True,
                lhs_contracting_dim=2, rhs_contracting_dim=1).instantiate()
    Int8DotCall([Buffer(S8, (3, 64, 128)), Buffer(S8, (3, 32, 128))], [Buffer(S32, (3, 64, 32)), Buffer(S32, (3, 64, 32))], batched=True,
                lhs_contracting_dim=2, rhs_contracting_dim=2, emit_s32=True).instantiate()
    b3 = [Buffer(S8, (3, 64, 128)), Buffer(S8, (3, 128, 32))]
    for ops, res, kw, code in [
        (b3, [Buffer(S32, (3, 64, 32))], {"lhs_contracting_dim": 2, "rhs_contracting_dim": 1}, 12),        # rank 3 without batch dims
        (b3, [Buffer(S32, (2, 64, 32))], {"batched": True, "lhs_contracting_dim": 2, "rhs_contracting_dim": 1}, 3),
        (b3, [Buffer(S32, (3, 64, 32))], {"batched": True, "lhs_contracting_dim": 0, "rhs_contracting_dim": 1}, 3),   # contracting the batch dimension
        (b3, [Buffer(S32, (3, 64, 32)), Buffer(S32, (64, 32))], {"batched": True, "lhs_contracting_dim": 2, "rhs_contracting_dim": 1, "emit_s32": True}, 3),
        ([Buffer(S8, (64, 128)), Buffer(S8, (128, 32))], [Buffer(S32, (64, 32))], {"batched": True}, 3),   # batch dims on rank 2
    ]:
        with pytest.raises(XlaFfiError) as e:
            Int8DotCall(ops, res, **kw).instantiate()
        assert e.value.code == code, (kw, e.value)
    for ops, res, kw, code in [
        ([Buffer(S8, (64, 128)), Buffer(F8E4M3FN, (128, 32))], [Buffer(S32, (64, 32))], {}, 3),
        ([Buffer(S8, (64, 128)), Buffer(S8, (128, 32)), Buffer(F32, (64,)), Buffer(F32, (32,))], [Buffer(S32, (64, 32))], {}, 3),
        ([Buffer(S8, (64, 128)), Buffer(S8, (128, 32)), Buffer(F32, (63,)), Buffer(F32, (32,))], [Buffer(BF16, (64, 32))], {}, 3),
        ([Buffer(S8, (64, 128)), Buffer(S8, (128, 32))], [Buffer(S8, (64, 32))], {}, 3),
        ([Buffer(S8, (64, 128)), Buffer(S8, (128, 32))], [Buffer(S32, (64, 32))], {"emit_s32": True}, 3),
    ]:
        with pytest.raises(XlaFfiError) as e:
            Int8DotCall(ops, res, **kw).instantiate()
        assert e.value.code == code


def test_block_scaled_frames():
    """`b200$block_scaled_dot$mx` takes what ThunkEmitter::EmitCublasLtMatmulMx takes
    (xla/service/gpu/thunk_emitter.cc:939-988): exactly a, b, a_scale, b_scale and (D, [workspace]); shapes as
    `__op$block_scaled_dot` fixes them (block_scaling_rewriter.h:30-77)."""
    from xla_b200.scaled_dot import BlockScaledDotCall, F8E8M0FNU
    E8 = F8E8M0FNU
    ok = [
        ([Buffer(F8E4M3FN, (8, 128)), Buffer(F8E4M3FN, (16, 128)), Buffer(E8, (8, 4)), Buffer(E8, (16, 4))], [Buffer(F32, (8, 16))]),
        ([Buffer(F8E4M3FN, (4, 16, 256)), Buffer(F8E5M2, (4, 16, 256)), Buffer(E8, (4, 16, 8)), Buffer(E8, (4, 16, 8))],
         [Buffer(BF16, (4, 16, 16)), Buffer(S8, (1 << 20,))]),
        ([Buffer(F8E5M2, (200, 96)), Buffer(F8E4M3FN, (77, 96)), Buffer(E8, (200, 3)), Buffer(E8, (77, 3))], [Buffer(F16, (200, 77))]),
    ]
    for ops, res in ok:
        BlockScaledDotCall(ops, res).instantiate()
    # padded scales (block_scaling_rewriter.cc:469-518): rows always, columns with the block size stated
    pad_rows = [Buffer(F8E4M3FN, (4, 120, 96)), Buffer(F8E4M3FN, (4, 120, 96)), Buffer(E8, (4, 128, 3)), Buffer(E8, (4, 128, 3))]
    pad_both = [Buffer(F8E4M3FN, (4, 120, 96)), Buffer(F8E4M3FN, (4, 120, 96)), Buffer(E8, (4, 128, 4)), Buffer(E8, (4, 128, 4))]
    BlockScaledDotCall(pad_rows, [Buffer(F16, (4, 120, 120))]).instantiate()
    BlockScaledDotCall(pad_both, [Buffer(F16, (4, 120, 120))], block_size=32).instantiate()
    for ops, kw, code in [(pad_both, {}, 3), (pad_both, {"block_size": 16}, 12),
                          (pad_rows[:2] + [Buffer(E8, (4, 100, 3)), Buffer(E8, (4, 128, 3))], {}, 3)]:
        with pytest.raises(XlaFfiError) as e:
            BlockScaledDotCall(ops, [Buffer(F16, (4, 120, 120))], **kw).instantiate()
        assert e.value.code == code
    a, b = Buffer(F8E4M3FN, (8, 128)), Buffer(F8E4M3FN, (16, 128))
    sa, sb, d = Buffer(E8, (8, 4)), Buffer(E8, (16, 4)), Buffer(F32, (8, 16))
    for ops, res, code in [
        ([a, b, sa], [d], 3),                                                     # operand count
        ([a, b, sa, sb, Buffer(F32, ())], [d], 3),                                # a global scale is not part of the $mx call
        ([a, b, sa, sb], [d, Buffer(F32, ()), Buffer(S8, (16,))], 3),             # no amax result
        ([a, b, Buffer(E8, (8, 8)), Buffer(E8, (16, 8))], [d], 3),                # block size 16
        ([a, Buffer(F8E4M3FN, (16, 256)), sa, Buffer(E8, (16, 8))], [d], 3),      # K differs
        ([a, b, Buffer(F8E4M3FN, (8, 4)), Buffer(F8E4M3FN, (16, 4))], [d], 12),   # e4m3 scales (NVFP4-style) not implemented
        ([Buffer(S8, (8, 128)), b, sa, sb], [d], 12),                             # element type
        ([a, b, sa, sb], [Buffer(F8E4M3FN, (8, 16))], 3),                         # result type
        ([a, b, sa, sb], [Buffer(F32, (8, 8))], 3),                               # result shape
        ([Buffer(F8E4M3FN, (8, 100)), Buffer(F8E4M3FN, (16, 100)), Buffer(E8, (8, 3)), Buffer(E8, (16, 3))], [d], 3),   # K % 32
    ]:
        with pytest.raises(XlaFfiError) as e:
            BlockScaledDotCall(ops, res).instantiate()
        assert e.value.code == code, (ops, e.value)


def test_unknown_target_and_wrong_stage():
    with pytest.raises(XlaFfiError) as e:
        FfiCall("__cublas$lt$matmul$f8", [], [], {}).instantiate()
    assert e.value.code == 5          # NOT_FOUND: nothing is registered under the cuBLASLt name


def test_kernel_selection_table():
    """The static stand-in for the autotuner: decode shapes whose 256-column strips leave SMs idle -> split-K (2);
    decode shapes with about one strip per SM, and everything else -> dense (1)."""
    sel = _native.product.b200sd_select_kernel
    assert sel(8192, 8192, 8192) == 1
    assert sel(256, 256, 512) == 1
    for m in (16, 64, 128):
        assert sel(m, 28672, 8192) == 1           # 112 strips on 148 SMs: one CTA per strip streams all of K
        for shard in (14336, 7168, 3584):         # the per-GPU shards of an N-split: too few strips, split K
            assert sel(m, shard, 8192) == 2
            need = _native.product.b200sd_workspace_bytes(m, shard, 8192)
            assert 0 < need <= 32 * 1024 * 1024   # fits the workspace XLA attaches (matmul_utils.h:103)
        assert sel(m, 256 * 150, 8192) == 2       # 150 strips: a second wave of two
    assert sel(16, 256, 256) == 1
    assert _native.product.b200sd_workspace_bytes(8192, 8192, 8192) == 0


def test_missing_library_fails_loudly(tmp_path, monkeypatch):
    monkeypatch.setattr(_native, "PRODUCT_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError):
        _native._load(_native.PRODUCT_LIB)


def test_config_table_overrides_the_static_choice(tmp_path):
    """The persisted-tuning stand-in: exact (type, m, n, k) matches win over the static rule; a bad file changes nothing."""
    import xla_b200

    assert xla_b200.select_kernel(64, 14336, 8192) == 2 and xla_b200.select_kernel(8192, 8192, 8192) == 1
    good = tmp_path / "table.txt"
    good.write_text("# comment\nf8 64 14336 8192 3   # dense single-CTA here\n\ns8 4096 4096 4096 5\nf8 8192 8192 8192 4\n")
    assert xla_b200.load_config_table(good) == 3
    assert xla_b200.select_kernel(64, 14336, 8192) == 3 and xla_b200.select_kernel(8192, 8192, 8192) == 4
    assert xla_b200.select_kernel(128, 14336, 8192) == 2              # no entry: static rule
    bad = tmp_path / "bad.txt"
    bad.write_text("f8 64 14336 8192 9\n")
    with pytest.raises(XlaFfiError) as e:
        xla_b200.load_config_table(bad)
    assert e.value.code == 3 and "bad.txt:1" in e.value.message
    assert xla_b200.select_kernel(64, 14336, 8192) == 3               # still the good table
    with pytest.raises(XlaFfiError):
        xla_b200.load_config_table(tmp_path / "missing.txt")
    with pytest.raises(XlaFfiError):
        (tmp_path / "s8skinny.txt").write_text("s8 64 4096 4096 2\n")
        xla_b200.load_config_table(tmp_path / "s8skinny.txt")
    # the MX block-scaled dot has its own type and its own two tile forms
    assert xla_b200.tuned_kernel_mx(2048, 8192, 4096) == 0
    mx = tmp_path / "mx.txt"
    mx.write_text("mx 2048 8192 4096 7\nmx 8192 8192 8192 6\nf8 2048 8192 4096 4\n")
    assert xla_b200.load_config_table(mx) == 3
    assert xla_b200.tuned_kernel_mx(2048, 8192, 4096) == 7 and xla_b200.tuned_kernel_mx(8192, 8192, 8192) == 6
    assert xla_b200.tuned_kernel_mx(4096, 4096, 4096) == 0 and xla_b200.select_kernel(2048, 8192, 4096) == 4
    for text in ("mx 2048 8192 4096 4\n", "f8 2048 8192 4096 6\n", "s8 256 256 256 7\n", "mxf 256 256 256 6\n"):
        (tmp_path / "badmx.txt").write_text(text)
        with pytest.raises(XlaFfiError):
            xla_b200.load_config_table(tmp_path / "badmx.txt")
    assert xla_b200.tuned_kernel_mx(2048, 8192, 4096) == 7            # a bad file changes nothing
    empty = tmp_path / "empty.txt"
    empty.write_text("# nothing\n")
    assert xla_b200.load_config_table(empty) == 0                     # and back to the static rule for later tests
    assert xla_b200.select_kernel(64, 14336, 8192) == 2 and xla_b200.tuned_kernel_mx(2048, 8192, 4096) == 0


def test_ctypes_mirrors_match_the_header_as_a_c_compiler_sees_it(tmp_path):
    """include/b200_scaled_dot.h compiles as plain C, and every struct has the size and the field offsets of its ctypes mirror."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    pairs = [("B200SD_ScaledDotF8", _native.ScaledDotF8Args), ("B200SD_DotS8", _native.DotS8Args),
             ("B200SD_Progress", _native.ProgressArgs), ("B200SD_PeerReduce", _native.PeerReduceArgs),
             ("B200SD_BlockScaledDotMx", _native.BlockScaledDotMxArgs)]
    lines = ["#include <stdio.h>", "#include <stddef.h>", '#include "b200_scaled_dot.h"', "int main(void) {"]
    for cname, mirror in pairs:
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "abi.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "abi"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    seen = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, mirror in pairs:
        assert int(seen[cname]) == C.sizeof(mirror), cname
        for field, _ in mirror._fields_:
            assert int(seen[f"{cname}.{field}"]) == getattr(mirror, field).offset, f"{cname}.{field}"
