"""K2 parity on the GPU: int32 accumulators bit-exact against the CPU oracle, the fused
epilogue within one rounding step of the output dtype, config 1 against the reference digests."""
import hashlib

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def f32(t):
    return t.detach().float().cpu().numpy()


def rand_codes(rng, shape):
    return rng.integers(-127, 128, size=shape, dtype=np.int8)


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (1, 8, 16), (196, 2304, 768), (300, 520, 400),
                                   (4900, 768, 3072), (4096, 3072, 768), (129, 257 * 8, 1280), (77, 1280, 5120)])
def test_int32_accumulators_exact(cuda_device, M, N, K):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(M * 7 + N)
    a, w = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    acc = ops.gemm_i8(torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device), out_dtype=torch.int32)
    torch.cuda.synchronize()
    ops.check_status()
    assert np.array_equal(acc.cpu().numpy(), O.int32_accumulators(a, w))


def test_extreme_codes_do_not_overflow(cuda_device):
    from sam_quantization_b200 import ops
    M, N, K = 130, 264, 5120
    a = np.full((M, K), -127, np.int8)
    w = np.full((N, K), 127, np.int8)
    w[::2] = -127
    acc = ops.gemm_i8(torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device), out_dtype=torch.int32)
    assert np.array_equal(acc.cpu().numpy(), O.int32_accumulators(a, w))


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("act,use_res,use_bias", [(None, False, True), ("gelu", False, True), (None, True, True),
                                                  ("gelu", True, False)])
def test_fused_epilogue(cuda_device, dt, act, use_res, use_bias):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(3)
    M, N, K = 333, 776, 768
    a, w = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    sa = (rng.random(M) * 0.05 + 0.001).astype(np.float32)
    sw = (rng.random(N) * 0.001 + 0.0001).astype(np.float32)
    bias = O.rnd(rng.standard_normal(N) * 0.5, dt) if use_bias else None
    res = O.rnd(rng.standard_normal((M, N)), dt) if use_res else None
    dev = cuda_device
    y = ops.gemm_i8(torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev),
                    torch.from_numpy(sa).to(dev), torch.from_numpy(sw).to(dev),
                    bias=None if bias is None else torch.from_numpy(bias).to(dev),
                    residual=None if res is None else torch.from_numpy(res).to(TDT[dt]).to(dev),
                    activation=1 if act else 0, out_dtype=TDT[dt])
    torch.cuda.synchronize()
    ops.check_status()
    want = O.dequant_epilogue(O.int32_accumulators(a, w), sa, sw, bias, act, res, dt)
    got = f32(y)
    ulp = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "f32": 2.0 ** -20}[dt]
    if act and dt == "f32":
        ulp = 4e-5           # the kernel's erf-GELU is accurate to 2e-5 relative, not to the last fp32 bit
    assert np.all(np.abs(got - want) <= ulp * np.maximum(np.abs(want), 1e-2) + 1e-6)


def test_per_tensor_scales_and_null_scales(cuda_device):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(4)
    M, N, K = 64, 256, 256
    a, w = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    dev = cuda_device
    y = ops.gemm_i8(torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev),
                    torch.tensor([0.01], device=dev), torch.tensor([0.002], device=dev), a_gran=1, w_gran=1,
                    out_dtype=torch.float32)
    want = O.int32_accumulators(a, w).astype(np.float32) * np.float32(0.01) * np.float32(0.002)
    assert np.allclose(f32(y), want, rtol=1e-6)
    y = ops.gemm_i8(torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev), out_dtype=torch.float32)
    assert np.array_equal(f32(y), O.int32_accumulators(a, w).astype(np.float32))


def test_bad_arguments(cuda_device):
    from sam_quantization_b200 import ops
    from sam_quantization_b200._lib import SamqError
    dev = cuda_device
    a = torch.zeros((8, 24), dtype=torch.int8, device=dev)       # K = 24: row stride not 16-byte aligned
    w = torch.zeros((8, 24), dtype=torch.int8, device=dev)
    with pytest.raises(SamqError):
        ops.gemm_i8(a, w, out_dtype=torch.int32)
    a = torch.zeros((8, 32), dtype=torch.int8, device=dev)
    w = torch.zeros((8, 32), dtype=torch.int8, device=dev)
    with pytest.raises(SamqError):                                 # raw accumulators take no scales
        ops.gemm_i8(a, w, torch.ones(8, device=dev), out_dtype=torch.int32)
    empty = ops.gemm_i8(torch.zeros((0, 32), dtype=torch.int8, device=dev), w, out_dtype=torch.float16)
    assert empty.shape == (0, 8)


def test_config1_against_reference_digests(cuda_device, golden):
    """The single-linear benchmark configuration (ViT-B fc1, one image) end to end through the C ABI: the fake-quant activations and weights
    hash to the digests of the reference's outputs; codes, scales and int32 accumulators equal
    the oracle's; the fp16 layer output is within 1e-2 relative max-abs of the reference's."""
    from sam_quantization_b200 import ops
    g = golden("config1")
    dev = cuda_device
    gen = torch.Generator().manual_seed(1)
    M, K, N = 4096, 768, 3072
    x = torch.randn(M, K, generator=gen)
    idx = torch.randperm(K, generator=gen)[:max(1, K // 100)]
    x[:, idx] *= 20
    w = torch.randn(N, K, generator=gen) * 0.02
    b = torch.randn(N, generator=gen) * 0.01
    x16, w16, b16 = x.half(), w.half(), b.half()
    s, lw, lb, fcs = O.smooth_ln_fcs(np.ones(K, np.float32), np.zeros(K, np.float32), [w16.float().numpy()],
                                     g["act_scales"], 0.5, "f16")
    # online SmoothQuant: x / s with the divisor fused into K1 equals the folded LayerNorm scale
    xs_dev = (x16.to(dev) * torch.from_numpy(lw).half().to(dev))
    a = ops.quantize(xs_dev, 0, fake_quant=True)
    assert hashlib.sha256(a["fq"].cpu().numpy().tobytes()).hexdigest() == str(g["fq_x_sha256"])
    ws = torch.from_numpy(fcs[0]).half().to(dev)
    wq = ops.quantize_weight(ws, 0, fake_quant=True)
    assert hashlib.sha256(wq["fq"].cpu().numpy().tobytes()).hexdigest() == str(g["fq_w_sha256"])
    qx, sx, _ = O.quantize(xs_dev.float().cpu().numpy(), "per_token", "f16")
    qw, sw, _ = O.quantize(fcs[0], "per_channel", "f16")
    assert np.array_equal(a["q"].cpu().numpy(), O.saturate_codes(qx))
    assert np.array_equal(f32(a["scale"]), sx)
    assert np.array_equal(wq["q"].cpu().numpy(), O.saturate_codes(qw))
    assert np.array_equal(f32(wq["scale"]), sw)
    acc = ops.gemm_i8(a["q"], wq["q"], out_dtype=torch.int32)
    assert np.array_equal(acc.cpu().numpy(), O.int32_accumulators(O.saturate_codes(qx), O.saturate_codes(qw)))
    y = ops.gemm_i8(a["q"], wq["q"], a["scale"], wq["scale"], bias=b16.to(dev), out_dtype=torch.float16)
    torch.cuda.synchronize()
    ops.check_status()
    want = g["y_sample"]
    got = f32(y)[::97, ::53]
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-2


@pytest.mark.parametrize("wq,aq,g", [("per_group", "per_token", 128), ("per_group", "per_group_token", 128),
                                     ("per_channel", "per_group_token", 256), ("per_group", "per_tensor", 384),
                                     ("per_group", "per_group_token", 64), ("per_group", "per_token", 32),
                                     ("per_group", "per_group_token", 96)])
def test_grouped_scales_against_oracle(cuda_device, wq, aq, g):
    """Grouped weights and / or activations: per-group int32 partial sums scaled in fp32."""
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(11)
    M, N, K = 203, 392, 768
    x = O.rnd(rng.standard_normal((M, K)).astype(np.float32), "f16")
    x[:, 5] *= 20
    w = O.rnd((rng.standard_normal((N, K)) * 0.02).astype(np.float32), "f16")
    b = O.rnd(rng.standard_normal(N) * 0.01, "f16")
    res = O.rnd(rng.standard_normal((M, N)), "f16")
    dev = cuda_device
    xa = ops.quantize(torch.from_numpy(x).half().to(dev), ops.ACT_GRANULARITY[aq], g if aq == "per_group_token" else None)
    wa = ops.quantize_weight(torch.from_numpy(w).half().to(dev), ops.WEIGHT_GRANULARITY[wq], g if wq == "per_group" else None)
    for act, use_res in ((None, False), ("gelu", True)):
        y = ops.gemm_i8(xa["q"], wa["q"], xa["scale"], wa["scale"], ops.ACT_GRANULARITY[aq], ops.WEIGHT_GRANULARITY[wq], g,
                        bias=torch.from_numpy(b).half().to(dev),
                        residual=torch.from_numpy(res).half().to(dev) if use_res else None,
                        activation=1 if act else 0, out_dtype=torch.float16)
        torch.cuda.synchronize()
        ops.check_status()
        want = O.w8a8_linear_int8(x, w, b, "f16", wq, aq, g, activation=act, residual=res if use_res else None)[0]
        got = f32(y)
        assert np.all(np.abs(got - want) <= 2.0 ** -9 * np.maximum(np.abs(want), 1e-2) + 1e-5), (wq, aq, g, act)


def test_grouped_gemm_rejects_small_groups(cuda_device):
    from sam_quantization_b200 import ops
    from sam_quantization_b200._lib import SamqError
    dev = cuda_device
    a = torch.zeros((8, 256), dtype=torch.int8, device=dev)
    w = torch.zeros((8, 256), dtype=torch.int8, device=dev)
    with pytest.raises(SamqError):
        ops.gemm_i8(a, w, torch.ones(8, device=dev), torch.ones((8, 16), device=dev), 0, 2, 16, out_dtype=torch.float16)


def test_group_size_64_linear_as_in_the_quarot_yaml(cuda_device):
    """group_size 64 (the only group size the reference's configurations use, quant/config/hq44k/quarot.yaml)
    through the module: ViT-H lin2's width, 80 groups per row."""
    from oracle.torch_twin import RefW8A8Linear
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    g = torch.Generator().manual_seed(3)
    lin = torch.nn.Linear(5120, 256).half().to(cuda_device)
    x = torch.randn(300, 5120, generator=g).half().to(cuda_device)
    import copy
    src = copy.deepcopy(lin)
    mine = W8A8Linear.from_float(lin, 8, "per_group", "per_group_token", False, 64)
    twin = RefW8A8Linear.from_float(src, 8, "per_group", "per_group_token", False, 64)
    a, b = mine(x).float(), twin(x).float()
    assert (a - b).abs().max() <= 1e-2 * b.abs().max()


# ---- CTA-pair implementation (tcgen05 cta_group::2) --------------------------------------------

@pytest.fixture
def pair_mode(cuda_device):
    from sam_quantization_b200 import ops
    prev = ops.set_gemm_pair_mode(ops.GEMM_PAIR_ALWAYS)
    yield
    ops.set_gemm_pair_mode(prev)


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (1, 8, 16), (196, 2304, 768), (300, 520, 400), (129, 136, 1280),
                                   (4900, 768, 3072), (4096, 3072, 768), (77, 1280, 5120), (385, 257 * 8, 144)])
def test_pair_int32_accumulators_exact(cuda_device, pair_mode, M, N, K):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(M * 11 + N)
    a, w = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    acc = ops.gemm_i8(torch.from_numpy(a).to(cuda_device), torch.from_numpy(w).to(cuda_device), out_dtype=torch.int32)
    torch.cuda.synchronize()
    ops.check_status()
    assert np.array_equal(acc.cpu().numpy(), O.int32_accumulators(a, w))


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("act,use_res", [(0, False), (1, False), (0, True), (1, True)])
def test_pair_matches_single_cta_bit_for_bit(cuda_device, dt, act, use_res):
    """Same accumulators, same epilogue arithmetic: the two implementations must agree exactly,
    on a shape with ragged M, N and K and more tiles than CTA pairs."""
    from sam_quantization_b200 import ops
    g = torch.Generator(device="cpu").manual_seed(17)
    M, N, K = 9 * 256 + 77, 2304 + 72, 784
    dev = cuda_device
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).to(dev)
    w = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
    sa = (torch.rand(M, generator=g) * 0.05 + 0.001).to(dev)
    sw = (torch.rand(N, generator=g) * 0.001 + 0.0001).to(dev)
    bias = (torch.randn(N, generator=g) * 0.5).to(TDT[dt]).to(dev)
    res = torch.randn((M, N), generator=g).to(TDT[dt]).to(dev) if use_res else None
    outs = []
    for mode in (ops.GEMM_PAIR_NEVER, ops.GEMM_PAIR_ALWAYS):
        prev = ops.set_gemm_pair_mode(mode)
        try:
            outs.append(ops.gemm_i8(a, w, sa, sw, bias=bias, residual=res, activation=act, out_dtype=TDT[dt]))
            torch.cuda.synchronize()
            ops.check_status()
        finally:
            ops.set_gemm_pair_mode(prev)
    assert torch.equal(outs[0], outs[1])


def test_pair_unaligned_output_takes_direct_stores(cuda_device, pair_mode):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(23)
    M, N, K = 300, 250, 256                      # N * 2 bytes is not a multiple of 16: no TMA store
    a, w = rand_codes(rng, (M, K)), rand_codes(rng, (N, K))
    sa = (rng.random(M) * 0.05 + 0.001).astype(np.float32)
    sw = (rng.random(N) * 0.001 + 0.0001).astype(np.float32)
    dev = cuda_device
    y = ops.gemm_i8(torch.from_numpy(a).to(dev), torch.from_numpy(w).to(dev), torch.from_numpy(sa).to(dev),
                    torch.from_numpy(sw).to(dev), out_dtype=torch.float16)
    torch.cuda.synchronize()
    ops.check_status()
    want = O.dequant_epilogue(O.int32_accumulators(a, w), sa, sw, None, None, None, "f16")
    assert np.all(np.abs(f32(y) - want) <= 2.0 ** -10 * np.maximum(np.abs(want), 1e-2) + 1e-6)


# ---- the failure path: a bounded wait that runs out -----------------------------------------------

def test_stalled_pipeline_gives_up_and_reports(cuda_device):
    """A GEMM whose producer never fills one operand stage (a stall made on the host side of the
    launch, no fault involved): the kernel's bounded waits run out after ~1 ms, it returns on its
    own with the status word raised, ``check_status`` raises, and the next GEMM is exact."""
    from sam_quantization_b200 import ops
    from sam_quantization_b200._lib import SamqError
    dev = cuda_device
    g = torch.Generator().manual_seed(12)
    a = torch.randint(-127, 128, (256, 1024), generator=g, dtype=torch.int8).to(dev)
    w = torch.randint(-127, 128, (512, 1024), generator=g, dtype=torch.int8).to(dev)
    want = (a.double() @ w.double().t()).to(torch.int32)
    assert torch.equal(ops.gemm_i8(a, w, out_dtype=torch.int32), want)
    ops.check_status()
    for skip in (1, 6):                                    # a stage of the first trip round the ring, and of the second
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        out = ops.gemm_stall_selftest(a, w, skip_kblock=skip, wait_limit_cycles=2_000_000)
        t1.record()
        torch.cuda.synchronize()                           # the kernel came back by itself
        assert t0.elapsed_time(t1) < 200.0                 # ~1 ms of waiting, nowhere near the 2 s default
        assert int(ops.status_word(dev).item()) == 1
        assert not torch.equal(out, want)                  # the tiles were never completed
        with pytest.raises(RuntimeError, match="bounded wait"):
            ops.check_status()
        ops.check_status()                                 # reading the status cleared it
        assert torch.equal(ops.gemm_i8(a, w, out_dtype=torch.int32), want)
        ops.check_status()
    with pytest.raises(SamqError):
        ops.gemm_stall_selftest(a, w, skip_kblock=99)      # not a k-block of this GEMM
    with pytest.raises(SamqError):
        ops.gemm_stall_selftest(a, w, skip_kblock=0, wait_limit_cycles=10)
