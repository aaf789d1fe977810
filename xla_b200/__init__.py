"""B200-native replacement for XLA's quantized scaled-dot custom calls.

The product is the shared library `xla_b200/lib/libb200_scaled_dot.so` (hand-written sm_100a
kernels behind XLA FFI handlers, declared in `include/b200_scaled_dot.h`).  This package is the
host-side mirror used to drive it without an XLA build: the custom-call front end over a stand-in
for the XLA side of the FFI (`scaled_dot`), the sharded launch patterns (`sharding`), the runner
that lowers HLO text through the rewriter-lite onto the custom calls (`hlo_runner`) and the offline
kernel-choice tuner (`autotune`).  There is no CPU or PyTorch fallback: importing the native
layer fails loudly when the library has not been built.
"""

from . import _native  # noqa: F401  (fails loudly if the library is missing)
from .scaled_dot import (  # noqa: F401
    Epilogue,
    GemmBackendConfig,
    ScaledDotCall,
    Int8DotCall,
    BlockScaledDotCall,
    cublas_lt_matmul_f8,
    cublas_lt_matmul_s8,
    cublas_lt_matmul_mx,
    device_status,
    launch_count,
    load_config_table,
    select_kernel,
    tuned_kernel_mx,
)
