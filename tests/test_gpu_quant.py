"""K1 / K3 parity on the GPU: int8 codes, scales and fake-quant outputs from the CUDA kernels
(called through the C ABI) against the reference fixtures and the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}
ACT = {"per_token": 0, "per_tensor": 1, "per_group_token": 2}


def to_dev(a, dt, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TDT[dt]).to(dev)


def f32(t):
    return t.detach().float().cpu().numpy()


def check_against_oracle(x_np, dt, gran_name, group, dev, divisor=None):
    from sam_quantization_b200 import ops
    x = to_dev(x_np, dt, dev)
    div_t = None if divisor is None else to_dev(divisor, dt, dev)
    out = ops.quantize(x, ACT[gran_name], group, divisor=div_t, codes=True, fake_quant=True, transformed=True)
    xin = O.rnd(x_np, dt)
    if divisor is not None:
        xin = O._div(xin, O.rnd(divisor, dt), dt)
    q, s, fq = O.quantize(xin, gran_name, dt, group)
    assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(out["scale"]).reshape(-1), np.asarray(s, np.float32).reshape(-1))
    assert np.array_equal(f32(out["fq"]), fq)
    assert np.array_equal(f32(out["tx"]), xin)


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_quantizers_match_reference_fixtures(cuda_device, golden, dt):
    from sam_quantization_b200 import ops
    g = golden("quantizers")
    x = to_dev(g[f"{dt}/x"], dt, cuda_device)
    for name, gran, group in (("act_per_token", 0, None), ("act_per_tensor", 1, None), ("act_per_group32", 2, 32)):
        out = ops.quantize(x, gran, group, fake_quant=True)
        assert np.array_equal(f32(out["fq"]), g[f"{dt}/{name}"]), name
    x3 = to_dev(g[f"{dt}/x3"], dt, cuda_device)
    assert np.array_equal(f32(ops.quantize(x3, 0, fake_quant=True)["fq"]), g[f"{dt}/act3_per_token"])
    assert np.array_equal(f32(ops.quantize(x3, 2, 16, fake_quant=True)["fq"]), g[f"{dt}/act3_per_group16"])
    w = to_dev(g[f"{dt}/w"], dt, cuda_device)
    for name, gran, group in (("w_per_channel", 0, None), ("w_per_tensor", 1, None), ("w_per_group32", 2, 32)):
        out = ops.quantize_weight(w, gran, group, fake_quant=True)
        assert np.array_equal(f32(out["fq"]), g[f"{dt}/{name}"]), name


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
@pytest.mark.parametrize("K", [768, 1024, 1280, 3072, 4096, 5120])
def test_per_token_codes_scales_bit_exact(cuda_device, dt, K):
    rng = np.random.default_rng(K)
    x = rng.standard_normal((197, K)).astype(np.float32)
    x[:, rng.permutation(K)[: max(1, K // 100)]] *= 20
    x[7] = 0
    check_against_oracle(x, dt, "per_token", None, cuda_device)


@pytest.mark.parametrize("dt", ["f16", "f32"])
@pytest.mark.parametrize("gran,group", [("per_tensor", None), ("per_group_token", 128), ("per_group_token", 64),
                                        ("per_group_token", 8), ("per_group_token", 384), ("per_group_token", 6)])
def test_other_granularities_bit_exact(cuda_device, dt, gran, group):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((61, 768)).astype(np.float32)
    x[:, 3] *= 20
    check_against_oracle(x, dt, gran, group, cuda_device)


def test_ragged_and_odd_shapes(cuda_device):
    rng = np.random.default_rng(9)
    for M, K in [(1, 8), (3, 7), (33, 100), (5, 8200), (2, 12288)]:
        x = rng.standard_normal((M, K)).astype(np.float32)
        check_against_oracle(x, "f16", "per_token", None, cuda_device)
        check_against_oracle(x, "f32", "per_tensor", None, cuda_device)


def test_smoothquant_divisor(cuda_device):
    rng = np.random.default_rng(10)
    x = rng.standard_normal((64, 768)).astype(np.float32)
    d = (rng.random(768) * 4 + 0.05).astype(np.float32)
    for dt in ("f16", "bf16", "f32"):
        check_against_oracle(x, dt, "per_token", None, cuda_device, divisor=d)
    check_against_oracle(x[:, :100], "f16", "per_token", None, cuda_device, divisor=d[:100])


def test_strided_rows_and_empty(cuda_device):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(11)
    big = torch.from_numpy(rng.standard_normal((40, 2048)).astype(np.float32)).half().to(cuda_device)
    view = big[:, 256:1024]                       # row stride 2048, 768 columns
    out = ops.quantize(view, 0, fake_quant=True)
    q, s, fq = O.quantize(view.float().cpu().numpy(), "per_token", "f16")
    assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(out["scale"]), s)
    empty = torch.empty((0, 768), dtype=torch.float16, device=cuda_device)
    out = ops.quantize(empty, 0)
    assert out["q"].shape == (0, 768) and out["scale"].shape == (0,)


def test_leading_dims_kept(cuda_device):
    from sam_quantization_b200 import ops
    x = torch.randn(2, 3, 5, 64, device=cuda_device, dtype=torch.float16)
    out = ops.quantize(x, 0, fake_quant=True)
    assert out["q"].shape == (2, 3, 5, 64) and out["scale"].shape == (2, 3, 5) and out["fq"].shape == x.shape
    out = ops.quantize(x, 2, 16)
    assert out["scale"].shape == (2, 3, 5, 4)


def test_bad_arguments_raise(cuda_device):
    from sam_quantization_b200 import ops
    from sam_quantization_b200._lib import SamqError
    x = torch.randn(4, 64, device=cuda_device, dtype=torch.float16)
    with pytest.raises(AssertionError):
        ops.quantize(x, 2, 48)
    with pytest.raises(RuntimeError):
        ops.quantize(x.cpu(), 0)
    with pytest.raises(SamqError):
        ops.quantize(x, 1, hadamard=ops.Hadamard("full"))


@pytest.mark.parametrize("n", [16, 64, 1024, 4096])
def test_full_hadamard_pow2_bit_exact(cuda_device, golden, n):
    """Power-of-two online Hadamard (fp32 butterflies in the reference's order, one rounding to
    fp16) then per-token int8: transformed values, codes and scales all exact."""
    from sam_quantization_b200 import ops
    g = golden("hadamard")
    x16 = O.rnd(g[f"hadU/{n}/x"], "f16")
    x = to_dev(x16, "f16", cuda_device)
    out = ops.quantize(x, 0, hadamard=ops.Hadamard("full"), fake_quant=True, transformed=True)
    assert np.array_equal(f32(out["tx"]), g[f"hadU/{n}/y_f16_via_f32"])
    q, s, fq = O.quantize(g[f"hadU/{n}/y_f16_via_f32"], "per_token", "f16")
    assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(out["scale"]), s)
    assert np.array_equal(f32(out["fq"]), fq)


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_full_hadamard_random_rows_with_signs(cuda_device, dt):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(21)
    for n in (1024, 4096, 256):
        x = O.rnd(rng.standard_normal((37, n)).astype(np.float32) * 3, dt)
        signs = (rng.integers(0, 2, n) * 2 - 1).astype(np.int8)
        had = ops.Hadamard("full", signs=torch.from_numpy(signs).to(cuda_device))
        out = ops.quantize(to_dev(x, dt, cuda_device), 0, hadamard=had, transformed=True)
        want = O.hadamard_full_online(x, dt, signs=signs)
        assert np.array_equal(f32(out["tx"]), want)
        q, s, _ = O.quantize(want, "per_token", dt)
        assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
        assert np.array_equal(f32(out["scale"]), s)


def test_partial_hadamard_across_heads(cuda_device):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(22)
    for C, had_dim in ((1024, 64), (1280, 80), (256, 16)):
        x = O.rnd(rng.standard_normal((50, C)).astype(np.float32), "f16")
        out = ops.quantize(to_dev(x, "f16", cuda_device), 0, hadamard=ops.Hadamard("partial", had_dim=had_dim),
                           transformed=True)
        want = O.hadamard_partial_online(x, had_dim, "f16")
        assert np.array_equal(f32(out["tx"]), want)
        q, s, _ = O.quantize(want, "per_token", "f16")
        assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))


@pytest.mark.parametrize("n", [768, 1280, 3072, 5120, 48])
def test_full_hadamard_with_explicit_factor(cuda_device, golden, n):
    """n = had_k * 2^p: the had_k x had_k mix is a small matmul whose fp32 summation order is
    the BLAS's in the reference, so this boundary is toleranced (a few fp32 ulps before the
    fp16 rounding), not bit exact."""
    from sam_quantization_b200 import ops
    g = golden("hadamard")
    for k in (12, 40):
        O.register_hadk(k, g[f"had{k}"])
    hadk, k = O.get_hadK(n)
    rng = np.random.default_rng(n)
    x = O.rnd(rng.standard_normal((9, n)).astype(np.float32), "f16")
    had = ops.Hadamard("full", had_k=k, hadk=torch.from_numpy(hadk).to(cuda_device))
    out = ops.quantize(to_dev(x, "f16", cuda_device), 0, hadamard=had, transformed=True)
    want = O.hadamard_full_online(x, "f16")
    got = f32(out["tx"])
    assert np.abs(got - want).max() <= 2e-3 * np.abs(want).max()
    assert (got != want).mean() < 0.01


# ---- prologue fused into K1: row gather, LayerNorm, bf16 storage read as fp16 ------------------

def test_row_gather_with_padding_rows(cuda_device):
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(31)
    x = O.rnd(rng.standard_normal((50, 768)).astype(np.float32), "f16")
    row_map = np.array([3, -1, 49, 0, 0, -1, 17, 25, 8], np.int32)
    out = ops.quantize(to_dev(x, "f16", cuda_device), 0, row_map=torch.from_numpy(row_map).to(cuda_device),
                       fake_quant=True, transformed=True)
    gathered = np.where(row_map[:, None] >= 0, x[np.maximum(row_map, 0)], 0.0).astype(np.float32)
    q, s, fq = O.quantize(gathered, "per_token", "f16")
    assert out["q"].shape == (9, 768)
    assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(out["scale"]), s)
    assert np.array_equal(f32(out["fq"]), fq)
    assert np.array_equal(f32(out["tx"]), gathered)
    # long rows take the multi-warp layout, odd widths the scalar kernel: same gather
    for K in (5120, 100):
        xk = O.rnd(rng.standard_normal((20, K)).astype(np.float32), "f16")
        rm = np.array([19, -1, 0, 7], np.int32)
        o = ops.quantize(to_dev(xk, "f16", cuda_device), 0, row_map=torch.from_numpy(rm).to(cuda_device))
        qk, sk, _ = O.quantize(np.where(rm[:, None] >= 0, xk[np.maximum(rm, 0)], 0.0).astype(np.float32), "per_token", "f16")
        assert np.array_equal(o["q"].cpu().numpy(), O.saturate_codes(qk)) and np.array_equal(f32(o["scale"]), sk)


def test_bf16_storage_read_as_fp16(cuda_device):
    from sam_quantization_b200 import ops
    xb = (torch.randn(77, 1280, device=cuda_device) * 3).to(torch.bfloat16)
    out = ops.quantize(xb, 0, as_dtype=torch.float16, fake_quant=True)
    ref = ops.quantize(xb.to(torch.float16), 0, fake_quant=True)
    assert out["fq"].dtype == torch.float16
    assert torch.equal(out["q"], ref["q"]) and torch.equal(out["scale"], ref["scale"]) and torch.equal(out["fq"], ref["fq"])


@pytest.mark.parametrize("dt,K", [("f16", 768), ("f16", 1280), ("f16", 1024), ("bf16", 768), ("f32", 1280)])
def test_fused_layernorm_then_quant(cuda_device, dt, K):
    """LayerNorm inside K1 against torch's LayerNorm followed by the plain kernel.  The two
    LayerNorms sum in different orders, so the normalised value may differ in its last bit and a
    code by one step on a handful of elements; everything else must be identical."""
    from sam_quantization_b200 import ops
    g = torch.Generator().manual_seed(K)
    x = (torch.randn(300, K, generator=g) * 2 + 0.3).to(TDT[dt]).to(cuda_device)
    w = (1 + 0.2 * torch.randn(K, generator=g)).to(TDT[dt]).to(cuda_device)
    b = (0.1 * torch.randn(K, generator=g)).to(TDT[dt]).to(cuda_device)
    row_map = torch.arange(299, -1, -1, dtype=torch.int32, device=cuda_device)
    row_map[5] = -1
    out = ops.quantize(x, 0, layer_norm=(w, b, 1e-6), row_map=row_map, transformed=True)
    ln = torch.nn.functional.layer_norm(x, (K,), w, b, 1e-6)
    ln = torch.where(row_map[:, None] >= 0, ln[row_map.clamp(min=0).long()], torch.zeros((), dtype=ln.dtype, device=ln.device))
    ref = ops.quantize(ln, 0)
    tx, lnf = out["tx"].float(), ln.float()
    # fp32 keeps every bit of the statistics' summation-order difference: a few fp32 ulps
    ulp = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7, "f32": 2.0 ** -17}[dt]
    assert float(((tx - lnf).abs() / lnf.abs().clamp(min=2.0 ** -6)).max()) <= 1.01 * ulp
    if dt != "f32":
        assert (tx != lnf).float().mean() < 0.01
    dq = (out["q"].int() - ref["q"].int()).abs()
    assert int(dq.max()) <= 1 and float((dq > 0).float().mean()) < 2e-3
    assert torch.equal(out["q"][5], torch.zeros(K, dtype=torch.int8, device=cuda_device))
    rel = ((out["scale"] - ref["scale"]).abs() / ref["scale"]).max()
    assert float(rel) <= 2 * ulp


def test_hadamard_with_gather_and_bf16_source(cuda_device):
    from sam_quantization_b200 import ops
    xb = (torch.randn(40, 1024, device=cuda_device)).to(torch.bfloat16)
    row_map = torch.tensor([39, -1, 0, 12], dtype=torch.int32, device=cuda_device)
    had = ops.Hadamard("partial", had_dim=64)
    out = ops.quantize(xb, 0, hadamard=had, row_map=row_map, as_dtype=torch.float16, transformed=True)
    src = xb.to(torch.float16)
    g = torch.where(row_map[:, None] >= 0, src[row_map.clamp(min=0).long()], torch.zeros((), dtype=src.dtype, device=src.device))
    ref = ops.quantize(g, 0, hadamard=had, transformed=True)
    assert torch.equal(out["tx"], ref["tx"]) and torch.equal(out["q"], ref["q"]) and torch.equal(out["scale"], ref["scale"])


def test_sign_of_zero_survives(cuda_device):
    """-0.0 and negative values that round to zero come out as -0.0, as the reference's
    div_().round_().mul_() leaves them (the fixtures' digests compare raw bytes)."""
    from sam_quantization_b200 import ops
    x = np.array([[-0.0, 0.0, -1e-4, 1e-4, 5.0, -5.0, -0.0, 0.01] * 16], np.float32)
    for dt in ("f16", "bf16", "f32"):
        out = ops.quantize(to_dev(x, dt, cuda_device), 0, fake_quant=True)
        _, _, fq = O.quantize(O.rnd(x, dt), "per_token", dt)
        got = f32(out["fq"])
        assert np.array_equal(got, fq) and np.array_equal(np.signbit(got), np.signbit(fq))


# ---- the lean kernel (fp16, per-row scale, codes only, K % 256 == 0) ----------------------------

def _lean_rows(M, K, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    x[:, rng.permutation(K)[: max(1, K // 100)]] *= 20
    x[3] = 0                                   # scale floor 1e-5 / 127
    x[4] *= 1e-4                               # subnormal fp16 scale: quotients beyond 127 must saturate
    x[5] *= 3e-3
    x[6] *= 200                                # large values, still finite in fp16
    x[8, 1:] = 0                               # a single non-zero element
    return x


@pytest.mark.parametrize("K", [768, 1024, 1280, 3072, 4096, 5120])
def test_lean_kernel_bit_exact(cuda_device, K):
    from sam_quantization_b200 import ops
    x_np = _lean_rows(301, K, K + 1)
    x = to_dev(x_np, "f16", cuda_device)
    out = ops.quantize(x, 0)                                   # codes + scales only: the lean kernel
    general = ops.quantize(x, 0, fake_quant=True)              # any extra output takes the general kernel
    q, s, _ = O.quantize(O.rnd(x_np, "f16"), "per_token", "f16")
    assert np.array_equal(out["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(out["scale"]), np.asarray(s, np.float32))
    assert torch.equal(out["q"], general["q"]) and torch.equal(out["scale"], general["scale"])


@pytest.mark.parametrize("K", [768, 1280])
def test_lean_kernel_gather_and_bf16_source(cuda_device, K):
    from sam_quantization_b200 import ops
    x_np = _lean_rows(64, K, K + 2)
    x = to_dev(x_np, "f16", cuda_device)
    rm = torch.tensor([63, -1, 0, 4, 4, 3, -1, 17, 25, 8, 6], dtype=torch.int32, device=cuda_device)
    out = ops.quantize(x, 0, row_map=rm)
    ref = ops.quantize(x, 0, row_map=rm, transformed=True)
    assert torch.equal(out["q"], ref["q"]) and torch.equal(out["scale"], ref["scale"])
    assert int(out["q"][1].abs().max()) == 0
    xb = to_dev(x_np, "bf16", cuda_device)
    xb[7] *= 1e-3                                              # values that lose bits in the cast to fp16
    out = ops.quantize(xb, 0, as_dtype=torch.float16, row_map=rm)
    ref = ops.quantize(xb.to(torch.float16), 0, row_map=rm, transformed=True)
    assert torch.equal(out["q"], ref["q"]) and torch.equal(out["scale"], ref["scale"])


@pytest.mark.parametrize("K", [768, 1024, 1280])
def test_lean_kernel_layernorm(cuda_device, K):
    """The lean kernel's LayerNorm sums pairs of lanes' partial sums in another order than the
    general kernel: statistics agree to a few fp32 ulps, codes to one step on a handful of
    elements, padding rows are exact zeros."""
    from sam_quantization_b200 import ops
    g = torch.Generator().manual_seed(K + 3)
    x = (torch.randn(300, K, generator=g) * 2 + 0.3).half().to(cuda_device)
    x[:, 11] *= 30
    w = (1 + 0.2 * torch.randn(K, generator=g)).half().to(cuda_device)
    b = (0.1 * torch.randn(K, generator=g)).half().to(cuda_device)
    rm = torch.arange(299, -1, -1, dtype=torch.int32, device=cuda_device)
    rm[5] = -1
    for row_map in (None, rm):
        out = ops.quantize(x, 0, layer_norm=(w, b, 1e-6), row_map=row_map)
        ref = ops.quantize(x, 0, layer_norm=(w, b, 1e-6), row_map=row_map, transformed=True)
        dq = (out["q"].int() - ref["q"].int()).abs()
        assert int(dq.max()) <= 1 and float((dq > 0).float().mean()) < 1e-3
        assert float(((out["scale"] - ref["scale"]).abs() / ref["scale"]).max()) <= 2.0 ** -10
        if row_map is not None:
            assert int(out["q"][5].abs().max()) == 0
        # against torch's LayerNorm followed by the plain kernel
        ln = torch.nn.functional.layer_norm(x, (K,), w, b, 1e-6)
        if row_map is not None:
            ln = torch.where(row_map[:, None] >= 0, ln[row_map.clamp(min=0).long()], torch.zeros((), dtype=ln.dtype, device=ln.device))
        plain = ops.quantize(ln, 0)
        dq = (out["q"].int() - plain["q"].int()).abs()
        assert int(dq.max()) <= 1 and float((dq > 0).float().mean()) < 2e-3


@pytest.mark.parametrize("n", [4096, 1024])
@pytest.mark.parametrize("with_signs", [False, True])
def test_hadamard_4096_kernel_matches_general_kernel(cuda_device, with_signs, n):
    """The kernel specialised for the 4096-point transform (codes only) against the general
    Hadamard kernel (any extra output selects it) and against the oracle, bit for bit; with a
    row gather, padding rows and a bf16-stored source."""
    from sam_quantization_b200 import ops
    rng = np.random.default_rng(n + int(with_signs))
    x_np = O.rnd(rng.standard_normal((45, n)).astype(np.float32) * 3, "f16")
    x_np[:, rng.permutation(n)[:n // 100]] *= 20
    x_np[3] = 0
    x_np[4] *= 1e-4
    x = to_dev(x_np, "f16", cuda_device)
    signs = None
    if with_signs:
        signs = torch.from_numpy(rng.choice([-1, 1], size=n).astype(np.int8)).to(cuda_device)
    had = ops.Hadamard("full", signs=signs)
    fast = ops.quantize(x, 0, hadamard=had)
    general = ops.quantize(x, 0, hadamard=had, transformed=True)
    assert torch.equal(fast["q"], general["q"]) and torch.equal(fast["scale"], general["scale"])
    if not with_signs:
        tx = O.hadamard_full_online(x_np, "f16")
        q, s, _ = O.quantize(tx, "per_token", "f16")
        assert np.array_equal(fast["q"].cpu().numpy(), O.saturate_codes(q))
        assert np.array_equal(f32(fast["scale"]), np.asarray(s, np.float32))
    rm = torch.tensor([44, -1, 0, 4, 4, 3, -1, 17], dtype=torch.int32, device=cuda_device)
    a = ops.quantize(x, 0, hadamard=had, row_map=rm)
    b = ops.quantize(x, 0, hadamard=had, row_map=rm, transformed=True)
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["scale"], b["scale"]) and int(a["q"][1].abs().max()) == 0
    xb = x.to(torch.bfloat16)
    a = ops.quantize(xb, 0, hadamard=had, as_dtype=torch.float16)
    b = ops.quantize(xb, 0, hadamard=had, as_dtype=torch.float16, transformed=True)
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["scale"], b["scale"])


@pytest.mark.parametrize("n", [4096, 1024])
def test_hadamard_kernels_walk_many_rows(cuda_device, n):
    """More rows than one resident wave of CTAs holds: every CTA of the specialised kernels walks
    several rows (the next row's copies in flight while the current one is transformed), through a
    gather with padding rows; codes and scales equal the general kernel's bit for bit."""
    from sam_quantization_b200 import ops
    g = torch.Generator().manual_seed(n)
    M = 9001 if n == 4096 else 19003
    x = (torch.randn(M, n, generator=g) * 2).half()
    x[:, torch.randperm(n, generator=g)[: n // 100]] *= 20
    x[5] = 0
    x = x.to(cuda_device)
    signs = (torch.randint(0, 2, (n,), generator=g) * 2 - 1).to(torch.int8).to(cuda_device)
    had = ops.Hadamard("full", signs=signs)
    rm = torch.randperm(M, generator=g).to(torch.int32)
    rm[::17] = -1
    rm = rm.to(cuda_device)
    for kw in ({}, {"row_map": rm}):
        fast = ops.quantize(x, 0, hadamard=had, **kw)
        general = ops.quantize(x, 0, hadamard=had, transformed=True, **kw)
        assert torch.equal(fast["q"], general["q"]) and torch.equal(fast["scale"], general["scale"])
    assert int(fast["q"][0].abs().max()) == 0              # a padding row of the gather
    # rows with a pitch: a column slice of a wider tensor
    wide = torch.zeros((1500, n + 64), dtype=torch.float16, device=cuda_device)
    wide[:, 32:32 + n] = x[:1500]
    view = wide[:, 32:32 + n]
    assert not view.is_contiguous()
    a = ops.quantize(view, 0, hadamard=had)
    b = ops.quantize(x[:1500].contiguous(), 0, hadamard=had)
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["scale"], b["scale"])


@pytest.mark.parametrize("had_dim", [64, 80, 8, 128])
def test_hadamard_across_16_heads_kernel_matches_general_kernel(cuda_device, had_dim):
    """The register-only kernel for the transform across 16 heads (codes only) against the general
    Hadamard kernel, bit for bit; ragged row counts, a row gather with padding rows, a bf16 source."""
    from sam_quantization_b200 import ops
    K = 16 * had_dim
    rng = np.random.default_rng(had_dim)
    x_np = O.rnd(rng.standard_normal((67, K)).astype(np.float32) * 2, "f16")
    x_np[:, rng.permutation(K)[: max(1, K // 100)]] *= 20
    x_np[3] = 0
    x_np[4] *= 1e-4
    x = to_dev(x_np, "f16", cuda_device)
    had = ops.Hadamard("partial", had_dim=had_dim)
    fast = ops.quantize(x, 0, hadamard=had)
    general = ops.quantize(x, 0, hadamard=had, transformed=True)
    assert torch.equal(fast["q"], general["q"]) and torch.equal(fast["scale"], general["scale"])
    tx = O.hadamard_partial_online(x_np, had_dim, "f16")
    q, s, _ = O.quantize(tx, "per_token", "f16")
    assert np.array_equal(fast["q"].cpu().numpy(), O.saturate_codes(q))
    assert np.array_equal(f32(fast["scale"]), np.asarray(s, np.float32))
    rm = torch.tensor([66, -1, 0, 4, 4, 3, -1, 17, 25], dtype=torch.int32, device=cuda_device)
    a = ops.quantize(x, 0, hadamard=had, row_map=rm)
    b = ops.quantize(x, 0, hadamard=had, row_map=rm, transformed=True)
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["scale"], b["scale"]) and int(a["q"][1].abs().max()) == 0
    xb = x.to(torch.bfloat16)
    a = ops.quantize(xb, 0, hadamard=had, as_dtype=torch.float16, row_map=rm)
    b = ops.quantize(xb, 0, hadamard=had, as_dtype=torch.float16, row_map=rm, transformed=True)
    assert torch.equal(a["q"], b["q"]) and torch.equal(a["scale"], b["scale"])


def test_layer_norm_and_hadamard_in_one_kernel(cuda_device, K=1024):
    """LayerNorm + sign flip + 1024-point Walsh-Hadamard + per-token quantization as one launch against
    the two-launch route (normalise and gather to an fp16 tensor, then transform and quantize).  The two
    LayerNorms sum in different orders, so a normalised value may differ in its last fp16 bit; codes
    then agree except where such a value sat on a rounding boundary."""
    from sam_quantization_b200 import ops
    g = torch.Generator().manual_seed(K)
    M = 8000                                                   # more row groups than resident CTAs: the kernel's loop runs
    x = (torch.randn(M, K, generator=g) * 2 + 0.3).half().to(cuda_device)
    w = (1 + 0.1 * torch.randn(K, generator=g)).half().to(cuda_device)
    b = (0.1 * torch.randn(K, generator=g)).half().to(cuda_device)
    signs = (torch.randint(0, 2, (K,), generator=g) * 2 - 1).to(torch.int8).to(cuda_device)
    row_map = torch.randperm(M, generator=g)[:7000].to(torch.int32)
    row_map[::13] = -1                                         # padding rows of a window gather
    row_map = row_map.to(cuda_device)
    spec = ops.Hadamard("full", signs=signs)
    assert ops.hadamard_layer_norm_fused(x, spec)
    one = ops.quantize(x, ops.GRAN_ROW, hadamard=spec, layer_norm=(w, b, 1e-6), row_map=row_map)
    tx = ops.quantize(x, ops.GRAN_ROW, codes=False, transformed=True, layer_norm=(w, b, 1e-6), row_map=row_map)["tx"]
    two = ops.quantize(tx, ops.GRAN_ROW, hadamard=spec)
    assert one["q"].shape == (7000, K)
    pad = (row_map < 0)
    assert int(one["q"][pad].abs().max()) == 0                 # zero rows stay zero: the padding comes after the norm
    diff = (one["q"].int() - two["q"].int()).abs()
    assert int(diff.max()) <= 1 and float((diff > 0).float().mean()) < 0.02
    assert torch.allclose(one["scale"], two["scale"], rtol=2e-3)
    # exact when the normalised tensor is the same: no LayerNorm, same kernel family
    assert torch.equal(ops.quantize(tx, ops.GRAN_ROW, hadamard=spec)["q"], two["q"])
    # and against torch's LayerNorm followed by the reference transform in fp32
    ln = torch.nn.functional.layer_norm(x.float(), (K,), w.float(), b.float(), 1e-6).half()
    ln = torch.where(pad[:, None], torch.zeros((), dtype=ln.dtype, device=ln.device), ln[row_map.clamp(min=0).long()])
    ref = ops.quantize(ln, ops.GRAN_ROW, hadamard=spec)
    d2 = (one["q"].int() - ref["q"].int()).abs()
    assert int(d2.max()) <= 2 and float((d2 > 0).float().mean()) < 0.05
