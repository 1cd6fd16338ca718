"""The packed int4 path (the format of the reference's native extension, quant/qgemm/kernels/):
the oracle's own consistency on the CPU, and the CUDA entries against the oracle bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O


def test_oracle_int4_packing_round_trip_and_known_bytes():
    codes = np.array([[-8, 7, -1, 0, 3], [1, -2, 5, -6, 7]], np.int8)
    packed = O.pack_int4(codes)
    assert packed.shape == (2, 3)
    # element 2j in the low nibble: (-8, 7) -> 0x78, (-1, 0) -> 0x0F, (3, pad) -> 0x03
    assert packed[0].tolist() == [0x78, 0x0F, 0x03]
    assert np.array_equal(O.unpack_int4(packed, 5), codes)
    rng = np.random.default_rng(0)
    c = rng.integers(-8, 8, size=(17, 64)).astype(np.int8)
    assert np.array_equal(O.unpack_int4(O.pack_int4(c), 64), c)


def test_oracle_int4_quantizer_properties():
    rng = np.random.default_rng(1)
    x = O.rnd(rng.standard_normal((9, 40)).astype(np.float32) * 3, "f16")
    scale = O.rnd(np.abs(x).max(axis=1) / 7.0, "f16")                 # bench_int4.py:13
    q, packed = O.sym_quant_int4(x, scale)
    assert q.min() >= -8 and q.max() <= 7 and np.abs(q).max() == 7
    assert np.array_equal(O.unpack_int4(packed, 40), q)
    # round half to even on exact ties: 2.5 -> 2, 3.5 -> 4, -0.5 -> 0
    ties = np.array([[2.5, 3.5, -0.5, -1.5, 9.0, -9.0]], np.float32)
    qt, _ = O.sym_quant_int4(ties, np.array([1.0], np.float32))
    assert qt[0].tolist() == [2, 4, 0, -2, 7, -8]
    acc = O.matmul_int4(packed, packed)
    assert np.array_equal(acc, q.astype(np.int32) @ q.astype(np.int32).T)
    y = O.sym_dequant_int32(acc, scale, scale)
    want = (scale[:, None] * scale[None, :]).astype(np.float16).astype(np.float32) * acc.astype(np.float16).astype(np.float32)
    assert np.array_equal(y, want.astype(np.float16).astype(np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", [(33, 40, 64), (256, 512, 1280), (200, 72, 100), (5, 7, 2)])
def test_qgemm_surface_equals_oracle(cuda_device, M, N, K):
    """``sym_quant`` / ``matmul`` / ``sym_dequant`` with the reference extension's signatures: packed
    bytes, int32 accumulators and fp16 output equal the oracle exactly."""
    import sam_quantization_b200.qgemm as qgemm
    from sam_quantization_b200 import ops
    g = torch.Generator().manual_seed(M + K)
    xa = (torch.randn(M, K, generator=g) * 2).half()
    xb = torch.randn(N, K, generator=g).half()
    sa = (xa.abs().amax(dim=1, keepdim=True).clamp(min=1e-6) / 7.0)    # bench_int4.py:10-15
    sb = (xb.abs().amax(dim=1, keepdim=True).clamp(min=1e-6) / 7.0)
    qa = qgemm.sym_quant(xa.to(cuda_device), sa.to(cuda_device))
    qb = qgemm.sym_quant(xb.to(cuda_device), sb.to(cuda_device))
    ca, pa = O.sym_quant_int4(xa.float().numpy(), sa.float().numpy())
    cb, pb = O.sym_quant_int4(xb.float().numpy(), sb.float().numpy())
    assert qa.dtype == torch.uint8 and qa.shape == (M, (K + 1) // 2)
    assert np.array_equal(qa.cpu().numpy(), pa) and np.array_equal(qb.cpu().numpy(), pb)
    assert np.array_equal(qgemm.unpack_int4(qa, K).cpu().numpy(), ca)
    assert np.array_equal(qgemm.pack_int4(torch.from_numpy(cb).to(cuda_device)).cpu().numpy(), pb)
    if K % 2 == 0:
        c = qgemm.matmul(qa, qb)
        torch.cuda.synchronize()
        ops.check_status()
        acc = O.matmul_int4(pa, pb)
        assert c.dtype == torch.int32 and np.array_equal(c.cpu().numpy(), acc)
        y = qgemm.sym_dequant(c, sa.to(cuda_device), sb.to(cuda_device), 32)
        assert y.dtype == torch.float16
        assert np.array_equal(y.float().cpu().numpy(), O.sym_dequant_int32(acc, sa.float().numpy(), sb.float().numpy()))
        # and against the fp16 product it approximates (bench_int4.py:86-92)
        ref = xa.float() @ xb.float().t()
        assert (y.float().cpu() - ref).abs().mean() < 0.25 * ref.abs().mean()


@pytest.mark.gpu
def test_qgemm_surface_rejects_what_the_reference_rejects(cuda_device):
    import sam_quantization_b200.qgemm as qgemm
    x = torch.zeros(4, 8, dtype=torch.float16, device=cuda_device)
    s = torch.ones(4, 1, dtype=torch.float16, device=cuda_device)
    with pytest.raises(RuntimeError):
        qgemm.sym_quant(x.cpu(), s.cpu())                              # checkDeviceType
    with pytest.raises(RuntimeError):
        qgemm.sym_quant(x, s[:3])                                      # checkSize
    with pytest.raises(RuntimeError):
        qgemm.sym_quant(x.t(), s)                                      # checkAllContiguous
    q = qgemm.sym_quant(x, s)
    with pytest.raises(RuntimeError, match="Unsupported data type"):
        qgemm.sym_dequant(qgemm.matmul(q, q), s, s, 16)                # only bits == 32 exists


@pytest.mark.gpu
def test_four_bit_weights_survive_packing(cuda_device):
    """A weight quantized with n_bits = 4 (what every YAML of the reference sets) packs to half the
    bytes and unpacks to the same codes; the layer output from the unpacked codes is unchanged."""
    import sam_quantization_b200.qgemm as qgemm
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    g = torch.Generator().manual_seed(4)
    lin = torch.nn.Linear(256, 72).half().to(cuda_device)
    x = torch.randn(50, 256, generator=g).half().to(cuda_device)
    mod = W8A8Linear.from_float(lin, 4)
    assert int(mod.qweight.min()) >= -7 and int(mod.qweight.max()) <= 7
    want = mod(x)
    packed = qgemm.pack_int4(mod.qweight)
    assert packed.numel() * 2 == mod.qweight.numel()
    mod.qweight = qgemm.unpack_int4(packed, 256)
    assert torch.equal(mod(x), want)
