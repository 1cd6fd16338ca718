"""The reference-facing Python surface on the GPU: W8A8Linear, the six quantizer functions,
replace_linear_with_target_and_quantize, SmoothQuant folding, ActQuantWrapper / rotate_sam, and
the encoder against its float twin driven through the reference's arithmetic."""
import copy
import types

import numpy as np
import pytest
import torch

from oracle import oracle as O
from oracle.torch_twin import RefActQuantWrapper, RefW8A8Linear, replace_linears
from tests.golden.make_golden import TINY, tiny_images

pytestmark = pytest.mark.gpu
TDT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(a @ b / (a.norm() * b.norm()))


def rel_err(a, b):
    return float((a.double() - b.double()).abs().max() / b.double().abs().max())


@pytest.mark.parametrize("dt", ["f16", "bf16", "f32"])
def test_w8a8linear_against_reference_outputs(cuda_device, golden, dt):
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    g = golden("w8a8_linear")
    dev = cuda_device
    x = torch.from_numpy(g[f"{dt}/x"]).to(TDT[dt]).to(dev)
    for wq, aq, gs, qo in [("per_channel", "per_token", None, 0), ("per_tensor", "per_tensor", None, 0),
                           ("per_channel", "per_token", None, 1)]:
        lin = torch.nn.Linear(256, 72).to(dev)
        lin.weight.data = torch.from_numpy(g[f"{dt}/w"]).to(TDT[dt]).to(dev)
        lin.bias.data = torch.from_numpy(g[f"{dt}/b"]).to(TDT[dt]).to(dev)
        m = W8A8Linear.from_float(lin, 8, weight_quant=wq, act_quant=aq, quantize_output=bool(qo), group_size=gs)
        y = m(x.clone())
        want = torch.from_numpy(g[f"{dt}/y/{wq}/{aq}/{gs}/{qo}"])
        assert y.dtype == TDT[dt] and y.shape == want.shape
        # 1e-2 relative max-abs on dequantized layer outputs; when the output is fake-quantized
        # again, one flipped rounding is a whole quantization step (max/127), so allow two steps
        assert rel_err(y.float().cpu(), want) < (2e-2 if qo else 1e-2), (wq, aq, qo)
        # the source Linear now holds the fake-quantized weight; m.weight (codes * scale) equals it
        # bit for bit except where bf16's short mantissa let the reference's quotient reach 128,
        # which an int8 code saturates to 127
        if dt == "bf16":
            assert (lin.weight.data != m.weight).float().mean() < 0.02
        else:
            assert torch.equal(lin.weight.data, m.weight)
    assert repr(m) == str(g[f"{dt}/repr"]).replace("weight_quant=per_group", "weight_quant=per_channel").replace(
        "act_quant=per_token, output_quant=None", "act_quant=per_token, output_quant=per_token")


def test_w8a8linear_errors_and_shapes(cuda_device):
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    lin = torch.nn.Linear(64, 32).half().to(cuda_device)
    with pytest.raises(ValueError):
        W8A8Linear.from_float(lin, 8, weight_quant="per_row")
    with pytest.raises(ValueError):
        W8A8Linear.from_float(lin, 8, act_quant="per_row")
    m = W8A8Linear.from_float(lin, 8)
    y = m(torch.randn(2, 5, 7, 64, device=cuda_device, dtype=torch.float16))
    assert y.shape == (2, 5, 7, 32)
    assert m(torch.zeros(0, 64, device=cuda_device, dtype=torch.float16)).shape == (0, 32)


def test_six_quantizer_functions_in_place(cuda_device, golden):
    from sam_quantization_b200.RTN_quantization import per_tensor_channel_group as P
    g = golden("quantizers")
    for dt in ("f16", "bf16", "f32"):
        x = torch.from_numpy(g[f"{dt}/x"]).to(TDT[dt]).to(cuda_device)
        w = torch.from_numpy(g[f"{dt}/w"]).to(TDT[dt]).to(cuda_device)
        for fn, arg, key, extra in [
                (P.quantize_activation_per_token_absmax, x, "act_per_token", ()),
                (P.quantize_activation_per_tensor_absmax, x, "act_per_tensor", ()),
                (P.quantize_activation_per_group_absmax_token_dim, x, "act_per_group32", (32,)),
                (P.quantize_weight_per_channel_absmax, w, "w_per_channel", ()),
                (P.quantize_weight_per_tensor_absmax, w, "w_per_tensor", ()),
                (P.quantize_weight_per_group_absmax_input_features, w, "w_per_group32", (32,))]:
            t = arg.clone()
            r = fn(t, *extra)
            assert r is t                                              # in place, like the reference
            assert np.array_equal(t.float().cpu().numpy(), g[f"{dt}/{key}"]), (dt, key)


def test_four_bit_codes_in_int8_container(cuda_device):
    """n_bits=4 (what most of the reference's YAMLs set): q_max = 7, codes still feed the int8 GEMM."""
    from sam_quantization_b200.RTN_quantization import per_tensor_channel_group as P
    from oracle.torch_twin import fq_rows
    x = torch.randn(33, 256, device=cuda_device, dtype=torch.float16)
    want = fq_rows(x.clone(), 4)
    q, s = P.quantize_activation_codes(x, "per_token", n_bits=4)
    assert int(q.abs().max()) <= 7
    got = P.quantize_activation_per_token_absmax(x.clone(), n_bits=4)
    assert torch.equal(got, want)


def test_replace_linear_walk(cuda_device):
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize

    class Inner(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = torch.nn.Linear(32, 32)
            self.lm_head = torch.nn.Linear(32, 16)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(10, 32)
            self.a = torch.nn.Linear(32, 32)
            self.lm_head = Inner()

    net = Net().half().to(cuda_device)
    replace_linear_with_target_and_quantize(net, W8A8Linear, 8, ["lm_head"])
    assert isinstance(net.a, W8A8Linear)
    assert isinstance(net.lm_head.fc, W8A8Linear)                  # excluded containers are still visited
    assert isinstance(net.lm_head.lm_head, torch.nn.Linear)        # exact child-name match is skipped
    assert isinstance(net.emb, torch.nn.Embedding)


def test_smooth_ln_fcs_matches_reference(cuda_device, golden):
    from sam_quantization_b200.RTN_quantization import smooth_ln_fcs
    g = golden("smooth")
    for dt in ("f16", "f32"):
        C = 64
        ln = torch.nn.LayerNorm(C).to(cuda_device)
        ln.weight.data = torch.from_numpy(g[f"{dt}/ln_w"]).to(TDT[dt]).to(cuda_device)
        ln.bias.data = torch.from_numpy(g[f"{dt}/ln_b"]).to(TDT[dt]).to(cuda_device)
        fc1, fc2 = torch.nn.Linear(C, 96).to(cuda_device), torch.nn.Linear(C, 32).to(cuda_device)
        fc1.weight.data = torch.from_numpy(g[f"{dt}/fc1_w"]).to(TDT[dt]).to(cuda_device)
        fc2.weight.data = torch.from_numpy(g[f"{dt}/fc2_w"]).to(TDT[dt]).to(cuda_device)
        smooth_ln_fcs(ln, [fc1, fc2], torch.from_numpy(g[f"{dt}/act_scales"]), alpha=0.5)
        for got, key in ((ln.weight, "ln_w_s"), (ln.bias, "ln_b_s"), (fc1.weight, "fc1_w_s"), (fc2.weight, "fc2_w_s")):
            want = torch.from_numpy(g[f"{dt}/{key}"])
            # CUDA pow() may differ from the CPU's by an ulp of the dtype
            tol = 2e-3 if dt == "f16" else 1e-6
            assert rel_err(got.float().cpu(), want) <= tol, (dt, key)


def test_hadamard_tables_and_offline_transform(cuda_device, golden):
    from sam_quantization_b200.quarot import hadamard_utils as H
    g = golden("hadamard")
    assert np.array_equal(H.get_had12().numpy().astype(np.int8), g["had12"])
    assert np.array_equal(H.get_had20().numpy().astype(np.int8), g["had20"])
    assert np.array_equal(H.get_had40().numpy().astype(np.int8), g["had40"])
    for n in (768, 1024, 1280, 3072, 4096, 5120, 12, 16, 64):
        assert H.get_hadK(n)[1] == int(g[f"hadK_of/{n}"])
    for n in (16, 64, 256, 1024, 4096):
        x = torch.from_numpy(g[f"hadU/{n}/x"])
        assert np.array_equal(H.matmul_hadU(x).numpy(), g[f"hadU/{n}/y"])
        y = H.matmul_hadU_cuda(x.half().to(cuda_device), None, 1)
        assert np.array_equal(y.float().cpu().numpy(), g[f"hadU/{n}/y_f16_via_f32"])
    for n in (64, 1024):
        Q = H.random_hadamard_matrix(n, "cpu", 123)
        assert np.array_equal(Q[0].numpy(), g[f"randhad/{n}/row0"])
        assert np.array_equal(H.random_hadamard_signs(n, 123).numpy(), g[f"randhad/{n}/signs"])


def _tiny_pair(dev, dtype, attn_dtype, seed=5):
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder(seed=seed, dtype=dtype, attn_dtype=attn_dtype, device=dev, **TINY)
    twin = copy.deepcopy(mine)
    return mine, twin


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_tiny_encoder_rtn_vs_twin_and_reference(cuda_device, golden, dtype):
    """W8A8 on all linears: the CUDA engine against the float twin running the reference's
    fake-quant arithmetic on the same weights (cosine >= 0.999), and against the embeddings the
    reference's own W8A8Linear produced on the CPU (fixture)."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize
    dev = cuda_device
    mine, twin = _tiny_pair(dev, dtype, None)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    img = tiny_images().to(dev, dtype)
    with torch.no_grad():
        a, b = mine(img), twin(img)
    assert cosine(a, b) >= 0.999
    want = torch.from_numpy(golden("encoder_tiny")["w8a8/embedding"])
    assert cosine(a.float().cpu(), want) >= 0.999
    assert rel_err(a.float().cpu(), want) < 5e-2


def test_tiny_encoder_smoothquant(cuda_device):
    from sam_quantization_b200.RTN_quantization import (W8A8Linear, get_act_scales_sam,
                                                        replace_linear_with_target_and_quantize, smooth_sam)
    dev = cuda_device
    mine, twin = _tiny_pair(dev, torch.float16, torch.bfloat16)
    calib = [tiny_images(seed=200 + i).to(dev, torch.float16) for i in range(3)]
    scales = get_act_scales_sam(mine, calib)
    assert set(k.split(".")[-1] for k in scales) == {"qkv", "proj", "lin1", "lin2"}
    smooth_sam(mine, scales, alpha=0.5)
    smooth_sam(twin, scales, alpha=0.5)
    assert torch.equal(mine.image_encoder.blocks[0].norm1.weight, twin.image_encoder.blocks[0].norm1.weight)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    img = tiny_images().to(dev, torch.float16)
    with torch.no_grad():
        assert cosine(mine(img), twin(img)) >= 0.999


def test_tiny_encoder_quarot(cuda_device):
    """rotate_sam on a power-of-two encoder (hidden 64, 4 heads): the fused engine against a twin
    that applies the same recipe with the reference's dense x @ Q, pure-torch Hadamards and
    fake-quant wrappers."""
    from sam_quantization_b200.quarot import rotate_sam, utils as qutils, hadamard_utils as H
    from sam_quantization_b200.quarot import rotation_utils
    dev = cuda_device
    mine, twin = _tiny_pair(dev, torch.float16, torch.bfloat16)
    args = types.SimpleNamespace(hidden_size_image_en=64, num_attention_head_image_en=4, hidden_size_mask_de=256,
                                 num_attention_head_mask_de=8, rotate_mode="hadamard", device=str(dev), seed=123,
                                 fp32_had=True)
    cfg = types.SimpleNamespace(n_bits=8, weight_quant="per_channel", act_quant="per_token", group_size=None,
                                quantize_output=False, quantize_input=True)
    float_model = copy.deepcopy(mine)
    img = tiny_images().to(dev, torch.float16)
    with torch.no_grad():
        y_float = float_model(img)
    # twin: same weight rotation (offline, shared code path is the package's torch/K1 transform),
    # then reference-style wrappers and a dense online Q
    Q = rotation_utils.get_orthogonal_matrix(64, "hadamard", device=str(dev), seed=123)
    rotation_utils.rotate_model(twin, Q, None, args)
    replace_linears(twin, lambda lin: RefActQuantWrapper(lin))
    for name, layer in qutils.find_qlayers(twin, layers=(RefActQuantWrapper,)).items():
        layer.quantize_input = True
        if "lin2" in name:
            layer.online_full_had = True
        if "proj" in name:
            layer.online_partial_had, layer.had_dim = True, 16
    qlayers = rotate_sam(mine, args, cfg)
    assert all(isinstance(v, qutils.ActQuantWrapper) for v in qlayers.values())
    assert qlayers["image_encoder.blocks.0.mlp.lin2"].online_full_had
    assert qlayers["image_encoder.blocks.0.attn.proj"].online_partial_had
    assert qlayers["image_encoder.blocks.0.attn.proj"].had_dim == 16
    with torch.no_grad():
        a, b = mine(img), twin(img)
    assert cosine(a, b) >= 0.999
    # rotation is an exact change of basis: the quantized rotated model still tracks the float model
    assert cosine(a, y_float) >= 0.99


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,W,dim,nh", [(14, 14, 160, 2), (4, 4, 64, 4), (14, 14, 128, 2), (16, 16, 64, 2), (64, 64, 80, 1)])
def test_attention_prep_kernels_against_torch_path(cuda_device, dtype, H, W, dim, nh):
    """The CUDA kernels that build the attention inputs (augmented q / k rows for windows, the
    explicit bias for global attention) against the same attention written with torch ops."""
    from sam_quantization_b200.sam_encoder import Attention
    torch.manual_seed(H * 100 + dim)
    attn = Attention(dim, nh, use_rel_pos=True, input_size=(H, W)).to(cuda_device, dtype)
    with torch.no_grad():
        attn.rel_pos_h.normal_(0, 0.3)
        attn.rel_pos_w.normal_(0, 0.3)
        B = 3
        qkv = torch.randn(B * H * W, 3 * dim, device=cuda_device, dtype=dtype)
        attn.native_prep = True
        attn.window14_kernel = False                  # this test is about the input-building kernels
        a = attn.attend_flat(qkv, B, H, W)
        attn.native_prep = False
        b = attn.attend_flat(qkv, B, H, W)
    assert a.shape == b.shape == (B * H * W, dim)
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    assert rel_err(a.float(), b.float()) < tol
    # over 4096 keys the torch route rounds rel_h + rel_w to 16 bits before the softmax, the kernels do not
    assert cosine(a, b) > (0.9998 if H * W >= 4096 else 0.9999)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,W,dim,nh", [(14, 14, 160, 2), (4, 4, 64, 4), (14, 14, 256, 4), (13, 9, 80, 1)])
def test_windowed_attention_kernel_variants_agree(cuda_device, dtype, H, W, dim, nh):
    """Three routes to the same windowed attention: the one-kernel version, the augmented-row
    version through the library attention, and plain torch ops."""
    from sam_quantization_b200.sam_encoder import Attention
    torch.manual_seed(7 * H + dim)
    attn = Attention(dim, nh, use_rel_pos=True, input_size=(H, W)).to(cuda_device, dtype)
    with torch.no_grad():
        attn.rel_pos_h.normal_(0, 0.3)
        attn.rel_pos_w.normal_(0, 0.3)
        B = 5
        qkv = torch.randn(B * H * W, 3 * dim, device=cuda_device, dtype=dtype)
        attn.window14_kernel = False
        outs = []
        for native, fused in ((True, True), (True, False), (False, False)):
            attn.native_prep, attn.fused_window_kernel = native, fused
            outs.append(attn.attend_flat(qkv, B, H, W).float())
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    assert rel_err(outs[0], outs[2]) < tol and rel_err(outs[1], outs[2]) < tol
    assert cosine(outs[0], outs[2]) > 0.9999


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("H,W,dim,nh,B", [(64, 64, 160, 2, 2), (64, 64, 128, 2, 1), (2, 64, 80, 1, 3), (6, 64, 64, 1, 2),
                                          (14, 14, 160, 2, 7), (14, 14, 128, 2, 3), (16, 16, 80, 1, 2), (5, 3, 64, 1, 4),
                                          (13, 9, 160, 2, 3), (1, 1, 80, 1, 2)])
def test_global_attention_kernel_against_fp32_reference(cuda_device, dtype, H, W, dim, nh, B):
    """The tensor-core attention (scores and bias on chip, online softmax), for whole images and for
    windows, against the same attention in fp32 torch ops and against the library-attention route
    (explicit bias tensor for images, augmented q / k rows for windows)."""
    from sam_quantization_b200 import ops
    from sam_quantization_b200.sam_encoder import Attention
    torch.manual_seed(H + dim + W)
    attn = Attention(dim, nh, use_rel_pos=True, input_size=(H, W)).to(cuda_device, dtype)
    d = dim // nh
    with torch.no_grad():
        attn.rel_pos_h.normal_(0, 0.3)
        attn.rel_pos_w.normal_(0, 0.3)
        qkv = torch.randn(B * H * W, 3 * dim, device=cuda_device, dtype=dtype)
        qkv[:, :dim] *= 2.0                                        # sharper rows: the running maximum must move
        attn.window14_kernel = False
        attn.fused_global_kernel = attn.tc_windows = True
        a = attn.attend_flat(qkv, B, H, W)
        torch.cuda.synchronize()
        ops.check_status()
        attn.fused_global_kernel = attn.tc_windows = False
        b = attn.attend_flat(qkv, B, H, W)
        # fp32 reference from the 16-bit inputs
        q, k, v = qkv.float().view(B, H * W, 3, nh, d).permute(2, 0, 3, 1, 4)
        s = (q * attn.scale) @ k.transpose(-1, -2)
        rq = q.view(B, nh, H, W, d)
        Rh = attn.rel_pos_h.float()[(torch.arange(H)[:, None] - torch.arange(H)[None, :] + H - 1).to(cuda_device)]
        Rw = attn.rel_pos_w.float()[(torch.arange(W)[:, None] - torch.arange(W)[None, :] + W - 1).to(cuda_device)]
        rel_h = torch.einsum("bnhwc,hkc->bnhwk", rq, Rh)
        rel_w = torch.einsum("bnhwc,wkc->bnhwk", rq, Rw)
        s = (s.view(B, nh, H, W, H, W) + rel_h[..., :, None] + rel_w[..., None, :]).view(B, nh, H * W, H * W)
        ref = (s.softmax(-1) @ v).permute(0, 2, 1, 3).reshape(B * H * W, dim)
    assert a.shape == (B * H * W, dim) and a.dtype == dtype
    # the bias terms themselves are 16-bit products (|rel| ~ 5 -> 1e-2 absolute in the logits)
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    assert rel_err(a.float(), ref) < tol
    # the explicit-bias route also rounds rel_h + rel_w to 16 bits in memory: looser on these sharp rows
    tol_b = 8e-2 if dtype == torch.bfloat16 else 1e-2
    assert rel_err(b.float(), ref) < tol_b
    assert rel_err(a.float(), b.float()) < tol_b
    assert cosine(a, ref) > 0.9999
    # keeping the bias in fp32 on chip must not be less accurate than rounding it to 16 bits in memory
    assert 1.0 - cosine(a, ref) <= 1.25 * (1.0 - cosine(b, ref)) + 1e-6


def _fp32_window_attention(qkv, attn, B, H, W, nh, d):
    dim = nh * d
    dev = qkv.device
    q, k, v = qkv.float().view(B, H * W, 3, nh, d).permute(2, 0, 3, 1, 4)
    s = (q * attn.scale) @ k.transpose(-1, -2)
    rq = q.view(B, nh, H, W, d)
    Rh = attn.rel_pos_h.float()[(torch.arange(H)[:, None] - torch.arange(H)[None, :] + H - 1).to(dev)]
    Rw = attn.rel_pos_w.float()[(torch.arange(W)[:, None] - torch.arange(W)[None, :] + W - 1).to(dev)]
    rel_h = torch.einsum("bnhwc,hkc->bnhwk", rq, Rh)
    rel_w = torch.einsum("bnhwc,wkc->bnhwk", rq, Rw)
    s = (s.view(B, nh, H, W, H, W) + rel_h[..., :, None] + rel_w[..., None, :]).view(B, nh, H * W, H * W)
    return (s.softmax(-1) @ v).permute(0, 2, 1, 3).reshape(B * H * W, dim)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("dim,nh,B", [(160, 2, 1), (160, 2, 7), (128, 2, 3), (1280, 16, 25), (768, 12, 40), (80, 1, 401)])
def test_window14_attention_kernel_against_fp32_reference(cuda_device, dtype, dim, nh, B):
    """The persistent tensor-core kernel for 14 x 14 windows (q, k, v read in place, the table
    products from the same MMA as the scores, exact two-pass softmax) against the same attention in
    fp32 torch ops and against the augmented-row route through the library attention.  The larger
    cases give every CTA several (window, head) items, so buffers and barrier phases wrap."""
    from sam_quantization_b200 import ops
    from sam_quantization_b200.sam_encoder import Attention
    H = W = 14
    torch.manual_seed(dim + B)
    attn = Attention(dim, nh, use_rel_pos=True, input_size=(H, W)).to(cuda_device, dtype)
    d = dim // nh
    with torch.no_grad():
        attn.rel_pos_h.normal_(0, 0.3)
        attn.rel_pos_w.normal_(0, 0.3)
        qkv = torch.randn(B * H * W, 3 * dim, device=cuda_device, dtype=dtype)
        qkv[:, :dim] *= 2.0
        assert ops.attn_window14_supported(H, W, d, dtype)
        a = attn.attend_flat(qkv, B, H, W)
        torch.cuda.synchronize()
        ops.check_status()
        a2 = attn.attend_flat(qkv, B, H, W)                        # a second launch reproduces the first bit for bit
        attn.window14_kernel = False
        b = attn.attend_flat(qkv, B, H, W)
        ref = _fp32_window_attention(qkv, attn, B, H, W, nh, d)
    assert a.shape == (B * H * W, dim) and a.dtype == dtype
    assert torch.isfinite(a.float()).all()
    assert torch.equal(a, a2)
    tol = 3e-2 if dtype == torch.bfloat16 else 4e-3
    assert rel_err(a.float(), ref) < tol
    assert cosine(a, ref) > 0.9999
    # the table products stay in fp32 on chip: not less accurate than the route that rounds them to 16 bits
    assert 1.0 - cosine(a, ref) <= 1.25 * (1.0 - cosine(b, ref)) + 1e-6
    # every window separately (a wrong window / head mapping would hide in a global norm)
    per_window = (a.float() - ref).view(B, -1).norm(dim=1) / ref.view(B, -1).norm(dim=1)
    assert float(per_window.max()) < 2 * tol


def test_window14_entry_rejects_bad_arguments(cuda_device):
    import ctypes
    from sam_quantization_b200 import _lib
    lib = _lib.load()
    dev = cuda_device
    qkv = torch.zeros((196, 3 * 80), dtype=torch.bfloat16, device=dev)
    tab = torch.zeros((56, 80), dtype=torch.bfloat16, device=dev)
    out = torch.zeros((196, 80), dtype=torch.bfloat16, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    assert lib.samq_attn_window14(P(qkv), P(tab), 56, _lib.BF16, 1, 1, 80, 0.1, P(out), None, None) == 0
    assert lib.samq_attn_window14(P(qkv), P(tab), 54, _lib.BF16, 1, 1, 80, 0.1, P(out), None, None) != 0      # table not padded to 56 rows
    assert b"56" in lib.samq_last_error_string()
    assert lib.samq_attn_window14(P(qkv), P(tab), 56, _lib.BF16, 1, 1, 96, 0.1, P(out), None, None) != 0      # head widths 64 and 80 only
    assert lib.samq_attn_window14(P(qkv), P(tab), 56, _lib.F32, 1, 1, 80, 0.1, P(out), None, None) != 0
    assert lib.samq_attn_window14(None, P(tab), 56, _lib.BF16, 1, 1, 80, 0.1, P(out), None, None) != 0
    assert lib.samq_attn_window14(P(qkv), P(tab), 56, _lib.BF16, 0, 1, 80, 0.1, P(out), None, None) == 0       # no windows: nothing to do
    torch.cuda.synchronize()


def test_attention_entry_rejects_bad_arguments(cuda_device):
    """Argument checks of the tensor-core attention entries: status codes, no kernel launch."""
    import ctypes
    from sam_quantization_b200 import _lib, ops
    lib = _lib.load()
    dev = cuda_device
    H, W, nh, d = 2, 64, 1, 80
    qkv = torch.zeros((H * W, 3 * nh * d), dtype=torch.bfloat16, device=dev)
    vt = torch.zeros((nh * d, H * W), dtype=torch.bfloat16, device=dev)
    rel = torch.zeros((nh, H * W, 136), dtype=torch.bfloat16, device=dev)
    out = torch.zeros((H * W, nh * d), dtype=torch.bfloat16, device=dev)
    P = lambda t: ctypes.c_void_p(t.data_ptr())

    def call(H_=H, W_=W, d_=d, pitch=136, dtype=_lib.BF16, qkv_=qkv):
        return lib.samq_attn_global(P(qkv_), P(vt), P(rel), dtype, 1, pitch, H_, W_, nh, d_, 0.1, P(out), None, None)

    assert call(W_=32) != 0                      # neither an image row of 64 nor a window of at most 16
    assert call(H_=3) != 0                       # 3 * 64 tokens is not a multiple of the 128-query tile
    assert call(d_=96) != 0                      # head widths 64 and 80 only
    assert call(pitch=100) != 0                  # rel_all rows shorter than 2H-1 + 2W-1
    assert call(dtype=_lib.F32) != 0
    assert lib.samq_attn_global(None, P(vt), P(rel), _lib.BF16, 1, 136, H, W, nh, d, 0.1, P(out), None, None) != 0
    assert b"" != lib.samq_last_error_string()
    assert lib.samq_attn_transpose_v(P(qkv), _lib.BF16, 1, H, 40, nh, d, P(vt), None) != 0   # W = 40: unsupported grid
    assert lib.samq_attn_global(P(qkv), P(vt), P(rel), _lib.BF16, 0, 136, H, W, nh, d, 0.1, P(out), None, None) == 0  # no units
    assert not ops.attn_global_supported(64, 64, 96, torch.bfloat16)
    assert ops.attn_global_supported(14, 14, 80, torch.float16)
    with pytest.raises(ValueError):
        ops.set_gemm_pair_mode(7)
    prev = ops.set_gemm_pair_mode(ops.GEMM_PAIR_AUTO)
    assert ops.set_gemm_pair_mode(prev) == ops.GEMM_PAIR_AUTO


# ---- packed checkpoints (quant/e2e_quant.py:10-14, RTN_quantization/Smooth_sam.py:126-142) -------

def test_packed_checkpoint_round_trip_w8a8(cuda_device, tmp_path):
    """save -> load into a float skeleton with other weights -> identical embeddings; the file
    holds int8 codes and scales for the linears, not float weights."""
    from sam_quantization_b200.RTN_quantization import (W8A8Linear, get_act_scales_sam,
                                                        replace_linear_with_target_and_quantize, smooth_sam)
    from sam_quantization_b200.checkpoint import load_quantized, save_quantized
    from sam_quantization_b200.sam_encoder import build_encoder
    dev = cuda_device
    mine, _ = _tiny_pair(dev, torch.float16, torch.bfloat16)
    scales = get_act_scales_sam(mine, [tiny_images(seed=200).to(dev, torch.float16)])
    smooth_sam(mine, scales, alpha=0.5)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, ["proj"], weight_quant="per_group", act_quant="per_token",
                                            quantize_output=True, group_size=32)
    img = tiny_images().to(dev, torch.float16)
    with torch.no_grad():
        want = mine(img)
    path = str(tmp_path / "w8a8.pt")
    save_quantized(mine, path)
    blob = torch.load(path, map_location="cpu")
    sd = blob["state_dict"]
    assert sd["image_encoder.blocks.0.attn.qkv.qweight"].dtype == torch.int8
    assert sd["image_encoder.blocks.0.attn.qkv.w_scale"].shape == (3 * 64, 2)          # [N, K / group]
    assert "image_encoder.blocks.0.attn.qkv.weight" not in sd
    assert "image_encoder.blocks.0.attn.proj.weight" in sd                             # excluded by name: still a Linear
    fresh = build_encoder(seed=99, dtype=torch.float16, attn_dtype=torch.bfloat16, device=dev, **TINY)
    load_quantized(fresh, path)
    lin = fresh.image_encoder.blocks[1].mlp.lin1
    assert isinstance(lin, W8A8Linear) and lin.weight_quant_name == "per_group" and lin.quantize_output and lin.group_size == 32
    assert isinstance(fresh.image_encoder.blocks[1].attn.proj, torch.nn.Linear)
    with torch.no_grad():
        assert torch.equal(fresh(img), want)


def test_packed_checkpoint_round_trip_quarot(cuda_device, tmp_path):
    """The rotation flags (which online transform, head width, the folded sign vector) travel with
    the checkpoint: a float skeleton loaded from it reproduces the rotated model bit for bit."""
    from sam_quantization_b200.checkpoint import load_quantized, save_quantized
    from sam_quantization_b200.quarot import rotate_sam, utils as qutils
    from sam_quantization_b200.sam_encoder import build_encoder
    dev = cuda_device
    mine, _ = _tiny_pair(dev, torch.float16, torch.bfloat16)
    args = types.SimpleNamespace(hidden_size_image_en=64, num_attention_head_image_en=4, hidden_size_mask_de=256,
                                 num_attention_head_mask_de=8, rotate_mode="hadamard", device=str(dev), seed=123, fp32_had=True)
    cfg = types.SimpleNamespace(n_bits=8, weight_quant="per_channel", act_quant="per_token", group_size=None,
                                quantize_output=False, quantize_input=True)
    rotate_sam(mine, args, cfg)
    img = tiny_images().to(dev, torch.float16)
    with torch.no_grad():
        want = mine(img)
    path = str(tmp_path / "quarot.pt")
    save_quantized(mine, path)
    fresh = build_encoder(seed=98, dtype=torch.float16, attn_dtype=torch.bfloat16, device=dev, **TINY)
    load_quantized(fresh, path)
    proj = fresh.image_encoder.blocks[0].attn.proj
    assert isinstance(proj, qutils.ActQuantWrapper) and proj.online_partial_had and proj.had_dim == 16 and proj.quantize_input
    assert fresh.image_encoder.blocks[0].mlp.lin2.online_full_had
    assert fresh.image_encoder.blocks[0].attn.qkv.pre_signs is not None
    with torch.no_grad():
        assert torch.equal(fresh(img), want)


def test_reference_format_state_dict_loads_into_w8a8linear(cuda_device):
    """A state dict written by the reference's class (a float ``weight`` [N, K] and a ``bias`` of
    shape [1, N], RTN_quantization/per_tensor_channel_group.py:111-128) loads: the weight is
    quantized on the way in, and assigning ``module.weight`` re-quantizes."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear
    g = torch.Generator().manual_seed(8)
    w = (torch.randn(72, 256, generator=g) * 0.02).half()
    b = (torch.randn(72, generator=g) * 0.01).half()
    x = torch.randn(50, 256, generator=g).half().to(cuda_device)
    lin = torch.nn.Linear(256, 72).half().to(cuda_device)
    lin.weight.data, lin.bias.data = w.clone().to(cuda_device), b.clone().to(cuda_device)
    want = W8A8Linear.from_float(lin, 8)(x)
    mod = W8A8Linear(256, 72).to(cuda_device)
    mod.load_state_dict({"weight": w.clone(), "bias": b.clone().view(1, -1)})
    assert torch.equal(mod(x), want)
    mod2 = W8A8Linear(256, 72).to(cuda_device)
    mod2.bias = b.clone().to(cuda_device)
    mod2.weight = w.clone().to(cuda_device)
    assert torch.equal(mod2(x), want)
    assert torch.equal(mod2.weight, mod.weight)


def test_encoder_runner_encode_overlaps_copies_and_matches_direct_calls(cuda_device):
    """``EncoderRunner.encode``: pinned host images in, host (or device) embeddings out, the copies of
    the neighbouring chunks overlapping the current forward; same embeddings as calling the model."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize
    from sam_quantization_b200.engine import EncoderRunner
    dev = cuda_device
    mine, _ = _tiny_pair(dev, torch.float16, torch.bfloat16)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    size = TINY["img_size"]
    imgs = torch.cat([tiny_images(seed=300 + i) for i in range(5)], 0)[:10].half()       # 10 images
    with torch.no_grad():
        want = torch.cat([mine(imgs[i:i + 2].to(dev)) for i in range(0, 10, 2)], 0)
    runner = EncoderRunner(mine, 2, img_size=size, device=dev, check_status=True)
    host_in = imgs.pin_memory()
    host_out = torch.empty(want.shape, dtype=want.dtype).pin_memory()
    for _ in range(2):                                           # the second call reuses the staging buffers
        host_out.zero_()
        runner.encode(host_in, host_out)
        torch.cuda.synchronize()
        assert torch.equal(host_out, want.cpu())
    dev_out = torch.empty_like(want)
    runner.encode(imgs.to(dev), dev_out)
    torch.cuda.synchronize()
    assert torch.equal(dev_out, want)
    runner.encode(host_in, dev_out.zero_())
    torch.cuda.synchronize()
    assert torch.equal(dev_out, want)
    # calls in a row without ordering the copies back on the current stream, one synchronize at the end
    for _ in range(3):
        host_out.zero_()
        runner.encode(host_in, host_out, wait=False)
    runner.synchronize()
    assert torch.equal(host_out, want.cpu())
    with pytest.raises(ValueError):
        runner.encode(host_in[:3], host_out[:3])


def test_runner_lanes_give_the_same_embeddings(cuda_device):
    """``EncoderRunner(lanes=2)`` records the forward of a batch as two sub-batches on concurrent
    streams inside one graph: image by image the embeddings equal the single-stream runner's and the
    eager model's, call after call."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize
    from sam_quantization_b200.engine import EncoderRunner
    dev = cuda_device
    mine, _ = _tiny_pair(dev, torch.float16, torch.bfloat16)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    size = TINY["img_size"]
    imgs = torch.cat([tiny_images(seed=400 + i) for i in range(4)], 0)[:8].half().to(dev)     # 8 images
    with torch.no_grad():
        want = torch.cat([mine(imgs[i:i + 2]) for i in range(0, 8, 2)], 0)
    one = EncoderRunner(mine, 4, img_size=size, device=dev)
    two = EncoderRunner(mine, 4, img_size=size, device=dev, lanes=2, check_status=True)
    assert two.lanes == 2
    for _ in range(3):
        for i in (0, 4):
            a = one(imgs[i:i + 4]).clone()
            b = two(imgs[i:i + 4]).clone()
            torch.cuda.synchronize()
            assert torch.equal(a, want[i:i + 4]) and torch.equal(b, want[i:i + 4])
    with pytest.raises(ValueError):
        EncoderRunner(mine, 3, img_size=size, device=dev, lanes=2)
    assert EncoderRunner(mine, 4, img_size=size, device=dev, lanes=2, use_graph=False).lanes == 1
