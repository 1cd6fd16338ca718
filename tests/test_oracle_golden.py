"""Pins the CPU oracle (oracle/oracle.py) to outputs of the reference's own functions
(tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
import hashlib

import numpy as np
import pytest

from oracle import oracle as O

DTYPES = ["f16", "bf16", "f32"]


def same(a, b):
    a = np.asarray(a, np.float32)
    b = np.asarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a, b)


@pytest.mark.parametrize("dt", DTYPES)
def test_activation_quantizers_bit_exact(golden, dt):
    g = golden("quantizers")
    x = g[f"{dt}/x"]
    assert same(O.quantize(x, "per_token", dt)[2], g[f"{dt}/act_per_token"])
    assert same(O.quantize(x, "per_tensor", dt)[2], g[f"{dt}/act_per_tensor"])
    assert same(O.quantize(x, "per_group_token", dt, 32)[2], g[f"{dt}/act_per_group32"])
    x3 = g[f"{dt}/x3"]
    assert same(O.quantize(x3, "per_token", dt)[2], g[f"{dt}/act3_per_token"])
    assert same(O.quantize(x3, "per_group_token", dt, 16)[2], g[f"{dt}/act3_per_group16"])


@pytest.mark.parametrize("dt", DTYPES)
def test_weight_quantizers_bit_exact(golden, dt):
    g = golden("quantizers")
    w = g[f"{dt}/w"]
    assert same(O.quantize(w, "per_channel", dt)[2], g[f"{dt}/w_per_channel"])
    assert same(O.quantize(w, "per_tensor", dt)[2], g[f"{dt}/w_per_tensor"])
    assert same(O.quantize(w, "per_group", dt, 32)[2], g[f"{dt}/w_per_group32"])


@pytest.mark.parametrize("dt", DTYPES)
def test_codes_times_scale_is_the_fake_quant(golden, dt):
    """The int8 codes and scales (which the reference never materialises) are consistent with
    its fake-quant output: fq == round_to_dtype(q * s)."""
    g = golden("quantizers")
    x = g[f"{dt}/x"]
    q, s, fq = O.quantize(x, "per_token", dt)
    assert same(O.rnd(q * s[:, None], dt), g[f"{dt}/act_per_token"])
    assert np.array_equal(q, np.rint(q))
    # rows with a normal scale never exceed 127 in fp16 / fp32; the tiny row (index 4) may in
    # fp16 (subnormal scale), and bf16's 8-bit mantissa lets the rounded quotient reach 128
    ok_rows = [i for i in range(x.shape[0]) if i != 4]
    assert np.abs(q[ok_rows]).max() <= (128 if dt == "bf16" else 127)
    assert same(fq, g[f"{dt}/act_per_token"])


@pytest.mark.parametrize("dt", DTYPES)
def test_w8a8_linear_reference_forward(golden, dt):
    g = golden("w8a8_linear")
    x, w, b = g[f"{dt}/x"], g[f"{dt}/w"], g[f"{dt}/b"]
    combos = [("per_channel", "per_token", None, 0), ("per_tensor", "per_tensor", None, 0),
              ("per_group", "per_group_token", 32, 0), ("per_channel", "per_token", None, 1),
              ("per_group", "per_token", 128, 0)]
    for wq, aq, gs, qo in combos:
        want = g[f"{dt}/y/{wq}/{aq}/{gs}/{qo}"]
        got = O.w8a8_linear_reference(x, w, b, dt, wq, aq, gs, bool(qo))
        # the float GEMM's summation order is BLAS's: allow one rounding step of the dtype
        tol = {"f16": 2e-3, "bf16": 1.6e-2, "f32": 1e-5}[dt]
        denom = np.abs(want).max()
        assert np.abs(got - want).max() / denom < tol, (wq, aq, gs, qo)


@pytest.mark.parametrize("dt", DTYPES)
def test_int8_path_matches_reference_layer_within_tolerance(golden, dt):
    """int8 codes -> int32 -> fp32 dequant reproduces the reference layer output within the
    1e-2 relative max-abs bound the north star sets for dequantized layer outputs."""
    g = golden("w8a8_linear")
    x, w, b = g[f"{dt}/x"], g[f"{dt}/w"], g[f"{dt}/b"]
    for wq, aq, gs in [("per_channel", "per_token", None), ("per_tensor", "per_tensor", None),
                       ("per_group", "per_group_token", 32), ("per_group", "per_token", 128)]:
        want = g[f"{dt}/y/{wq}/{aq}/{gs}/0"]
        y = O.w8a8_linear_int8(x, w, b, dt, wq, aq, gs)[0]
        assert np.abs(y - want).max() / np.abs(want).max() < 1e-2


@pytest.mark.parametrize("dt", ["f16", "f32"])
def test_smooth_ln_fcs(golden, dt):
    g = golden("smooth")
    s, lw, lb, fcs = O.smooth_ln_fcs(g[f"{dt}/ln_w"], g[f"{dt}/ln_b"], [g[f"{dt}/fc1_w"], g[f"{dt}/fc2_w"]],
                                     g[f"{dt}/act_scales"], 0.5, dt)
    if dt == "f16":
        assert same(lw, g[f"{dt}/ln_w_s"]) and same(lb, g[f"{dt}/ln_b_s"])
        assert same(fcs[0], g[f"{dt}/fc1_w_s"]) and same(fcs[1], g[f"{dt}/fc2_w_s"])
    else:   # fp32 pow() differs by an ulp between libm implementations
        for a, b in ((lw, g[f"{dt}/ln_w_s"]), (lb, g[f"{dt}/ln_b_s"]), (fcs[0], g[f"{dt}/fc1_w_s"]), (fcs[1], g[f"{dt}/fc2_w_s"])):
            assert np.allclose(a, b, rtol=1e-6, atol=0)


def test_hadamard_tables_and_divisor_order(golden):
    g = golden("hadamard")
    assert np.array_equal(O.paley1(11).astype(np.int8), g["had12"])
    assert np.array_equal(O.paley1(19).astype(np.int8), g["had20"])
    for k in (12, 20, 28, 36, 40):
        H = g[f"had{k}"].astype(np.float64)
        assert np.array_equal(H @ H.T, k * np.eye(k))
    for k in (28, 36, 40):
        O.register_hadk(k, g[f"had{k}"])
    for n in (768, 1024, 1280, 3072, 4096, 5120, 12, 16, 64):
        assert O.get_hadK(n)[1] == int(g[f"hadK_of/{n}"])


def test_matmul_hadU(golden):
    g = golden("hadamard")
    O.register_hadk(40, g["had40"])
    for n in (16, 64, 256, 1024, 4096):          # power of two: same butterfly order -> bit exact
        assert same(O.matmul_hadU(g[f"hadU/{n}/x"]), g[f"hadU/{n}/y"]), n
        got = O.hadamard_full_online(O.rnd(g[f"hadU/{n}/x"], "f16"), "f16")
        assert same(got, g[f"hadU/{n}/y_f16_via_f32"]), n
    for n in (48, 768, 1280, 160):               # explicit hadK factor: matmul order is BLAS's
        want = g[f"hadU/{n}/y"]
        got = O.matmul_hadU(g[f"hadU/{n}/x"])
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max(), n


def test_random_hadamard_matrix(golden):
    g = golden("hadamard")
    for n in (64, 1024, 768):
        signs = g[f"randhad/{n}/signs"].astype(np.float64)
        Q = O.random_hadamard_matrix(n, 123, signs=signs)
        if n != 768:
            assert hashlib.sha256(Q.tobytes()).hexdigest() == str(g[f"randhad/{n}/sha256"])
        assert np.allclose(Q[0], g[f"randhad/{n}/row0"], rtol=0, atol=1e-15)
        assert np.allclose(np.diagonal(Q), g[f"randhad/{n}/diag"], rtol=0, atol=1e-15)
        assert np.allclose(Q @ Q.T, np.eye(n), atol=1e-12)
        # the same signs come out of torch's generator with the reference's seed
        assert np.array_equal(O.random_hadamard_signs(n, 123), signs)


def test_config1_reference_digests(golden):
    """The single-linear benchmark configuration (ViT-B fc1, one image) regenerated from its seeds and pushed through the oracle reproduces
    the digests of the reference's outputs (fake-quant activations and weights bit for bit)."""
    import torch
    g = golden("config1")
    gen = torch.Generator().manual_seed(1)
    M, K, N = 4096, 768, 3072
    x = torch.randn(M, K, generator=gen)
    idx = torch.randperm(K, generator=gen)[:max(1, K // 100)]
    assert np.array_equal(idx.numpy(), g["outlier_idx"])
    x[:, idx] *= 20
    w = torch.randn(N, K, generator=gen) * 0.02
    b = torch.randn(N, generator=gen) * 0.01
    x16 = x.to(torch.float16).float().numpy()
    w16 = w.to(torch.float16).float().numpy()
    s, lw, lb, fcs = O.smooth_ln_fcs(np.ones(K, np.float32), np.zeros(K, np.float32), [w16], g["act_scales"], 0.5, "f16")
    assert same(lw, g["ln_weight_after"])
    assert hashlib.sha256(fcs[0].astype(np.float16).tobytes()).hexdigest() == str(g["w_smoothed_sha256"])
    xs = O.rnd(x16 * lw, "f16")
    qx, sx, fqx = O.quantize(xs, "per_token", "f16")
    assert hashlib.sha256(fqx.astype(np.float16).tobytes()).hexdigest() == str(g["fq_x_sha256"])
    qw, sw, fqw = O.quantize(fcs[0], "per_channel", "f16")
    assert hashlib.sha256(fqw.astype(np.float16).tobytes()).hexdigest() == str(g["fq_w_sha256"])
    assert np.abs(qx).max() <= 127 and np.abs(qw).max() <= 127
    # layer output: int8 path vs the reference's fp16 output sample, 1e-2 relative max-abs
    acc = O.int32_accumulators(O.saturate_codes(qx), O.saturate_codes(qw))
    y = O.dequant_epilogue(acc, sx, sw, O.rnd(b.numpy(), "f16"), None, None, "f16")
    want = g["y_sample"]
    assert np.abs(y[::97, ::53] - want).max() / np.abs(want).max() < 1e-2
