"""The allocation-free per-tensor quantizer (samq_act_quant_per_tensor_static).

Who needs it: a caller that cannot get device memory where the layer runs — for example a
plugin inside a serving process whose memory was carved up at start-up — and so cannot hand
samq_act_quant_i8 the small workspace its per-tensor mode requires.  This entry point keeps that
scratch in an array built into the library.  The test drives it through the C ABI with ctypes
and checks codes, scale and fake-quant output against the workspace-taking entry point and against
the CPU oracle's per-tensor quantizer, exactly (all three run the same rounding), on two consecutive
calls whose inputs differ, so that anything the first call left in the shared scratch would show up
in the second.  The file name sorts last so a
run that stops at the first failure has already exercised every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _existing(lib, x, n_bits=8):
    from sam_quantization_b200 import _lib
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((1,), dtype=torch.float32, device=x.device)
    fq = torch.empty_like(x)
    ws = torch.empty((64,), dtype=torch.int32, device=x.device)
    code = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[x.dtype]
    _lib.check(lib.samq_act_quant_i8(x.data_ptr(), code, M, K, x.stride(0), None, None, _lib.GRAN_TENSOR, 0, n_bits,
                                     q.data_ptr(), s.data_ptr(), fq.data_ptr(), None, ws.data_ptr(), 256,
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return q, s, fq


def _static(lib, x, n_bits=8):
    from sam_quantization_b200 import _lib
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((1,), dtype=torch.float32, device=x.device)
    fq = torch.empty_like(x)
    code = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[x.dtype]
    _lib.check(lib.samq_act_quant_per_tensor_static(x.data_ptr(), code, M, K, x.stride(0), n_bits,
                                                    q.data_ptr(), s.data_ptr(), fq.data_ptr(),
                                                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    return q, s, fq


def test_static_scratch_variant_matches_workspace_variant(cuda_device):
    from sam_quantization_b200 import _lib
    lib = _lib.load()
    gen = torch.Generator().manual_seed(77)
    big = (torch.randn(1000, 768, generator=gen) * 9).half().to(cuda_device)      # call 1: large maximum
    small = (torch.randn(130, 768, generator=gen) * 0.1).half().to(cuda_device)   # call 2: smaller, fewer rows
    from oracle import oracle as O
    for x in (big, small):
        got = _static(lib, x)
        want = _existing(lib, x)
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g, w)
        q_ref, s_ref, fq_ref = O.quantize_tensor(x.float().cpu().numpy(), "f16")
        assert np.array_equal(got[0].cpu().numpy(), O.saturate_codes(q_ref))
        assert np.array_equal(got[1].cpu().numpy(), s_ref)
        assert np.array_equal(got[2].float().cpu().numpy(), fq_ref)
    for dt in (torch.bfloat16, torch.float32):
        x = torch.randn(257, 100, generator=gen).to(dt).to(cuda_device)           # odd width: scalar path
        got = _static(lib, x)
        for g, w in zip(got, _existing(lib, x)):
            assert torch.equal(g, w)
        q_ref, s_ref, _ = O.quantize_tensor(x.float().cpu().numpy(), "bf16" if dt == torch.bfloat16 else "f32")
        assert np.array_equal(got[0].cpu().numpy(), O.saturate_codes(q_ref))
        assert np.array_equal(got[1].cpu().numpy(), s_ref)


def test_static_scratch_variant_rejects_oversize(cuda_device):
    from sam_quantization_b200 import _lib
    lib = _lib.load()
    x = torch.zeros((8, 16), dtype=torch.float16, device=cuda_device)
    rc = lib.samq_act_quant_per_tensor_static(x.data_ptr(), _lib.F16, 262145, 16, 16, 8, None, None, None, None)
    assert rc == -6
    assert b"262144" in lib.samq_last_error_string()
