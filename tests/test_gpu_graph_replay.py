"""A call site recorded into a CUDA graph (how an XLA command buffer records a custom call whose handler
declares XLA_FFI_HANDLER_TRAITS_COMMAND_BUFFER_COMPATIBLE) and replayed with new input data must give the
new data's result every time.  A recorded launch repeats its kernel arguments, so nothing that tells one
launch from the next may live in them: covered here for the three places that keep state between the CTAs
of a launch -- the split-K flags, the stream-K flags and the amax words."""
import numpy as np
import pytest
import torch

from oracle import scaled_dot_oracle as o
import helpers as h
from xla_b200 import _native, device_status
from xla_b200.scaled_dot import Epilogue, GemmBackendConfig, ScaledDotCall, XLA_WORKSPACE_BYTES

pytestmark = pytest.mark.gpu


def _record_and_replay(dev, call, refill, check, replays=3):
    side = torch.cuda.Stream(device=dev)
    refill(0)
    call.run(torch.cuda.current_stream(dev).cuda_stream, dev.index or 0)      # instantiate / initialize outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        call.execute(torch.cuda.current_stream(dev).cuda_stream, dev.index or 0)
    for i in range(1, replays + 1):
        refill(i)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        check(i)
    assert device_status() == 0


def test_split_k_call_replays_with_new_inputs(cuda_device):
    dev = cuda_device
    m, k, n = 64, 4096, 2048
    assert _native.product.b200sd_select_kernel(m, n, k) == 2
    a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=dev)
    b = torch.empty((k, n), dtype=torch.float8_e4m3fn, device=dev)
    sa, sb = torch.empty((), device=dev), torch.empty((), device=dev)
    d = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    ws = torch.empty(XLA_WORKSPACE_BYTES, dtype=torch.int8, device=dev)
    call = ScaledDotCall([a, b, sa, sb], [d, ws], GemmBackendConfig(selected_algorithm=2))
    host = {}

    def refill(i):
        an, bn, s0, s1 = o.make_f8_operands(300 + i, m, k, n)
        host[i] = (an, bn, s0, s1)
        a.copy_(h.f8_tensor(an, dev)); b.copy_(h.f8_tensor(bn, dev))
        sa.fill_(float(s0)); sb.fill_(float(s1))
        d.zero_()

    def check(i):
        an, bn, s0, s1 = host[i]
        exp, _ = o.scaled_dot_f8(an, bn, s0, s1)
        h.check_close(exp, h.result_to_oracle_repr(d, o.BF16), o.BF16)

    _record_and_replay(dev, call, refill, check)
    call.close()


@pytest.mark.parametrize("kernel", [0, 5])
def test_amax_and_stream_k_calls_replay_with_new_inputs(cuda_device, kernel):
    """amax must be THIS replay's maximum (inputs shrink from replay to replay, so a maximum carried over from
    an earlier replay would show), and the stream-K tail (kernel 5) must add this replay's partials only."""
    dev = cuda_device
    m, k, n = 2560, 2048, 2560          # 10 x 10 tiles of 256 x 256 on 74 clusters: one wave, 26 tiles left over, 16 k-blocks each
    a = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=dev)
    b = torch.empty((k, n), dtype=torch.float8_e4m3fn, device=dev)
    sa, sb, ds = (torch.empty((), device=dev) for _ in range(3))
    bias = torch.empty(n, dtype=torch.bfloat16, device=dev)
    d = torch.empty((m, n), dtype=torch.float8_e4m3fn, device=dev)
    amax = torch.empty((), device=dev)
    ws = torch.empty(XLA_WORKSPACE_BYTES, dtype=torch.int8, device=dev)
    cfg = GemmBackendConfig(epilogue=Epilogue.BIAS_GELU, damax_output=True, selected_algorithm=kernel)
    call = ScaledDotCall([a, b, sa, sb, bias, ds], [d, amax, ws], cfg)
    host = {}

    def refill(i):
        an, bn, s0, s1 = o.make_f8_operands(310 + i, m, k, n)
        s0 = np.float32(s0 / (1 + i))                        # every replay's result is smaller than the one before
        bias_bits = o.make_bias_bf16(310 + i, n)
        host[i] = (an, bn, s0, s1, bias_bits)
        a.copy_(h.f8_tensor(an, dev)); b.copy_(h.f8_tensor(bn, dev)); bias.copy_(h.bf16_tensor(bias_bits, dev))
        sa.fill_(float(s0)); sb.fill_(float(s1)); ds.fill_(0.5)
        amax.fill_(1e30)

    def check(i):
        an, bn, s0, s1, bias_bits = host[i]
        rows = np.arange(0, m, 37)                           # a sample of rows keeps the CPU side short; amax from the device result
        exp, _ = o.scaled_dot_f8(np.ascontiguousarray(an[rows]), bn, s0, s1, bias=o.bf16_bits_to_f32(bias_bits),
                                 epilogue=o.EPI_BIAS_GELU, d_scale=0.5, out_dtype=o.F8E4M3FN)
        got = d.view(torch.uint8).cpu().numpy()
        assert o.fp8_within_n_values(exp, got[rows], 1) == 0
        full, full_amax = o.scaled_dot_f8(an, bn, s0, s1, bias=o.bf16_bits_to_f32(bias_bits), epilogue=o.EPI_BIAS_GELU,
                                          out_dtype=o.F32, want_amax=True)
        assert abs(float(amax.item()) - float(full_amax)) <= 1e-2 * float(full_amax), (i, float(amax.item()), float(full_amax))

    _record_and_replay(dev, call, refill, check)
    call.close()
