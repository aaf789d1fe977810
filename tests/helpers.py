"""Shared helpers of the GPU parity tests: move oracle inputs to the device, run the custom call
through the FFI boundary, bring results back as the oracle's representation."""
import numpy as np
import torch

from oracle import scaled_dot_oracle as o
import xla_b200
from xla_b200.scaled_dot import Epilogue, GemmBackendConfig

TORCH_OUT = {o.BF16: torch.bfloat16, o.F16: torch.float16, o.F32: torch.float32,
             o.F8E4M3FN: torch.float8_e4m3fn, o.F8E5M2: torch.float8_e5m2}
KIND_DTYPE = {"e4m3fn": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def f8_tensor(codes: np.ndarray, dev, kind="e4m3fn"):
    return torch.from_numpy(np.ascontiguousarray(codes)).to(dev).view(KIND_DTYPE[kind])


def bf16_tensor(bits: np.ndarray, dev):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev).view(torch.bfloat16)


def result_to_oracle_repr(d: torch.Tensor, out_dtype: int) -> np.ndarray:
    if out_dtype in (o.F8E4M3FN, o.F8E5M2):
        return d.view(torch.uint8).cpu().numpy()
    if out_dtype in (o.BF16, o.F16):
        return d.view(torch.int16).cpu().numpy().view(np.uint16)
    return d.cpu().numpy()


def run_scaled_dot(dev, a, b, sa, sb, *, a_kind="e4m3fn", b_kind="e4m3fn", lc=1, rc=0, epilogue=o.EPI_DEFAULT, bias_bits=None,
                   c_f32=None, beta=0.0, alpha=1.0, d_scale=None, out_dtype=o.BF16, want_amax=False, kernel=0):
    """a, b: FP8 code points in their STORAGE layout.  Returns (D in oracle representation, amax)."""
    cfg = GemmBackendConfig(alpha_real=alpha, beta=beta, lhs_contracting_dimensions=(lc,),
                            rhs_contracting_dimensions=(rc,), epilogue=Epilogue(epilogue),
                            damax_output=want_amax, selected_algorithm=kernel)
    d, amax = xla_b200.cublas_lt_matmul_f8(
        f8_tensor(a, dev, a_kind), f8_tensor(b, dev, b_kind),
        torch.tensor(np.float32(sa), device=dev), torch.tensor(np.float32(sb), device=dev),
        c=torch.from_numpy(c_f32).to(dev) if c_f32 is not None else None,
        bias=bf16_tensor(bias_bits, dev) if bias_bits is not None else None,
        d_scale=torch.tensor(np.float32(d_scale), device=dev) if d_scale is not None else None,
        out_dtype=TORCH_OUT[out_dtype], config=cfg)
    torch.cuda.synchronize()
    assert xla_b200.device_status() == 0
    return result_to_oracle_repr(d, out_dtype), (float(amax.item()) if amax is not None else None)


def check_close(exp, got, out_dtype, abs_tol=1e-2, rel_tol=1e-2):
    """The reference's comparison (xla/literal_comparison.cc:456-556): zero mismatches allowed."""
    bad, mabs, mrel = o.near_mismatches(o.output_to_f32(exp, out_dtype), o.output_to_f32(got, out_dtype),
                                        abs_tol, rel_tol)
    assert bad == 0, f"{bad} mismatches (max abs {mabs:.4g}, max rel {mrel:.4g})"
