"""Encoder-level parity at the full architectures and 1024x1024 inputs of the benchmark configurations:
the CUDA engine against the float twin that runs the reference's fake-quant arithmetic on the
same random-init weights.  Final embeddings reach cosine >= 0.999 for the RTN and SmoothQuant
configurations (fp16 and fp32 tensors).  The QuaRot configuration does not (about 0.997 in both
dtypes) although each of its layers is bit-exact on identical inputs; its test shows that the
reference's own arithmetic disagrees with itself by the same amount under a change of summation
order, and asserts that the product is no further from the twin than that.

The twin shares nothing with the product but the float encoder itself: its quantizers, its
online transforms and its weight rotation are the restatements in oracle/torch_twin.py."""
import copy
import types

import numpy as np
import pytest
import torch

from oracle import oracle as O
from oracle.torch_twin import (RefActQuantWrapper, RefW8A8Linear, matmul_hadU, random_hadamard_Q, replace_linears,
                               rotate_encoder_weights)

pytestmark = pytest.mark.gpu


def cosine(a, b):
    a, b = a.double().flatten(), b.double().flatten()
    return float(a @ b / (a.norm() * b.norm()))


def images(n, seed, dtype=torch.float16):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(n, 3, 1024, 1024, generator=g)
    mean = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)
    return ((img - mean) / std).to(dtype)


def make_twin(model):
    twin = copy.deepcopy(model)
    for blk in twin.image_encoder.blocks:
        blk.attn.native_prep = False          # plain torch attention in the twin
    return twin


def run_batched(model, x, per_call):
    with torch.no_grad():
        return torch.cat([model(x[i:i + per_call]) for i in range(0, x.shape[0], per_call)], 0)


def test_config2_vit_b_rtn_w8a8(cuda_device):
    """SAM ViT-B, W8A8 on all linears (per-channel weights, per-token activations), fp16 with
    bf16 attention, the configuration's full batch of 8 images of 1024x1024."""
    from sam_quantization_b200.RTN_quantization import W8A8Linear, replace_linear_with_target_and_quantize
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder("vit_b", seed=2, device=cuda_device)
    twin = make_twin(mine)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    assert sum(isinstance(m, W8A8Linear) for m in mine.modules()) == 48
    x = images(8, 20).to(cuda_device)
    a, b = run_batched(mine, x, 8), run_batched(twin, x, 2)
    assert a.shape == (8, 256, 64, 64)
    assert cosine(a, b) >= 0.999
    assert min(cosine(a[i], b[i]) for i in range(8)) >= 0.999


# ---- configuration 3: ViT-L with QuaRot -----------------------------------------------------------

def build_quarot_pair(model_type, seed, dtype, device):
    """(product model after ``rotate_sam``, twin after the restated rotation, twin wrappers by name)."""
    from sam_quantization_b200.quarot import rotate_sam
    from sam_quantization_b200.sam_encoder import VIT_CONFIGS, build_encoder
    dim, _, heads, _ = VIT_CONFIGS[model_type]
    mine = build_encoder(model_type, seed=seed, dtype=dtype, device=device,
                         attn_dtype=torch.bfloat16 if dtype == torch.float16 else None)
    twin = make_twin(mine)
    signs, Q = random_hadamard_Q(dim, 123)
    rotate_encoder_weights(twin, Q.to(device), dim, heads)
    replace_linears(twin, lambda lin: RefActQuantWrapper(lin))
    wrappers = {}
    signs_dev = signs.to(device)
    for i, blk in enumerate(twin.image_encoder.blocks):
        for name, layer in (("attn.qkv", blk.attn.qkv), ("attn.proj", blk.attn.proj),
                            ("mlp.lin1", blk.mlp.lin1), ("mlp.lin2", blk.mlp.lin2)):
            layer.quantize_input = True
            wrappers[f"image_encoder.blocks.{i}.{name}"] = layer
        blk.attn.qkv.pre_signs = blk.mlp.lin1.pre_signs = signs_dev      # x @ Q == hadU(x * signs)
        blk.mlp.lin2.online_full_had = True
        blk.attn.proj.online_partial_had, blk.attn.proj.had_dim = True, dim // heads
    args = types.SimpleNamespace(hidden_size_image_en=dim, num_attention_head_image_en=heads, hidden_size_mask_de=256,
                                 num_attention_head_mask_de=8, rotate_mode="hadamard", device=str(device), seed=123,
                                 fp32_had=True)
    cfg = types.SimpleNamespace(n_bits=8, weight_quant="per_channel", act_quant="per_token", group_size=None,
                                quantize_output=False, quantize_input=True)
    qlayers = rotate_sam(mine, args, cfg)
    return mine, twin, wrappers, qlayers, signs


def test_config3_rotated_weights_equal_the_twins(cuda_device):
    """``rotate_sam``'s offline weight rotation against the independent restatement: the
    fake-quantized weights every wrapped Linear ends up with agree element for element except
    where a last-bit difference of the fp32 transform moved a value across a rounding boundary."""
    mine, twin, wrappers, qlayers, _ = build_quarot_pair("vit_l", 3, torch.float16, cuda_device)
    assert len(qlayers) == 96 and sorted(qlayers) == sorted(wrappers)
    for name, ref in wrappers.items():
        w_mine, w_ref = qlayers[name].module.weight.float(), ref.module.weight.float()
        step = w_ref.abs().amax(dim=1, keepdim=True) / 127
        moved = ((w_mine - w_ref).abs() > 0.25 * step).float().mean().item()
        assert (w_mine - w_ref).abs().max() <= 1.01 * step.max() and moved < 2e-3, (name, moved)


def test_config3_teacher_forced_all_96_layers(cuda_device):
    """Every one of the 96 wrapped linears of ViT-L QuaRot, fed the input its twin saw in a twin
    forward pass: int8 codes and scales equal the reference arithmetic bit for bit (the twin's
    torch ops over all rows, and the numpy oracle over a sample of rows), int32 accumulators are
    exact, and the layer output is within 1e-2 relative max-abs of the twin's layer output."""
    from sam_quantization_b200 import ops
    mine, twin, wrappers, qlayers, signs = build_quarot_pair("vit_l", 3, torch.float16, cuda_device)
    captured = {}
    hooks = [layer.register_forward_hook(lambda m, inp, out, name=name: captured.__setitem__(name, (inp[0].detach(), out.detach())))
             for name, layer in wrappers.items()]
    x = images(1, 30).to(cuda_device)
    with torch.no_grad():
        twin(x)
    for h in hooks:
        h.remove()
    assert len(captured) == 96
    signs_np = signs.numpy().astype(np.float32)
    worst = 0.0
    for name, (xin, yref) in captured.items():
        layer, ref = qlayers[name], wrappers[name]
        K = xin.shape[-1]
        x2 = xin.reshape(-1, K).contiguous()
        spec = layer._hadamard_spec(x2)
        got = ops.quantize(x2, ops.GRAN_ROW, hadamard=spec)
        # (1) the twin's own arithmetic over every row
        xt = x2
        if ref.pre_signs is not None:
            xt = matmul_hadU(x2.float() * ref.pre_signs.float()).half()
        elif ref.online_full_had:
            xt = matmul_hadU(x2.float()).half()
        elif ref.online_partial_had:
            v = x2.float().reshape(-1, K // ref.had_dim, ref.had_dim).transpose(1, 2).contiguous()
            xt = matmul_hadU(v).transpose(1, 2).reshape(-1, K).half()
        s = xt.abs().max(dim=-1, keepdim=True)[0].clamp_(min=1e-5).div_(127)
        q = xt.div(s).round()
        assert torch.equal(got["scale"], s.float().view(-1)), name
        assert torch.equal(got["q"], q.clamp(-127, 127).to(torch.int8)), name
        # (2) the numpy oracle over a sample of rows
        rows = torch.arange(0, x2.shape[0], 97, device=x2.device)
        xs = x2[rows].float().cpu().numpy()
        if ref.pre_signs is not None:
            ts = O.hadamard_full_online(xs, "f16", signs=signs_np)
        elif ref.online_full_had:
            ts = O.hadamard_full_online(xs, "f16")
        else:
            ts = O.hadamard_partial_online(xs, ref.had_dim, "f16")
        q_o, s_o, _ = O.quantize_rows(ts, "f16")
        assert np.array_equal(got["scale"][rows].cpu().numpy(), s_o[:, 0]), name
        assert np.array_equal(got["q"][rows].cpu().numpy(), O.saturate_codes(q_o)), name
        # (3) int32 accumulators, exact (fp64 product of integers below 2^53)
        acc = ops.gemm_i8(got["q"], layer.qweight, out_dtype=torch.int32)
        want = (got["q"].double() @ layer.qweight.double().t()).to(torch.int32)
        assert torch.equal(acc, want), name
        assert np.array_equal(acc[rows].cpu().numpy(), O.int32_accumulators(got["q"][rows].cpu().numpy(), layer.qweight.cpu().numpy())), name
        # (4) the whole layer
        y = layer(xin)
        err = float((y.float() - yref.float()).abs().max() / yref.float().abs().max())
        worst = max(worst, err)
        assert err <= 1e-2, (name, err)
    print(f"teacher-forced ViT-L QuaRot: 96 layers, worst layer-output rel max-abs error {worst:.2e}")


def _per_block_cosines(mine, twin, x):
    em, et = mine.image_encoder, twin.image_encoder
    with torch.no_grad():
        hm, ht = em.patch_embed(x) + em.pos_embed, et.patch_embed(x) + et.pos_embed
        out = []
        for bm, bt in zip(em.blocks, et.blocks):
            hm, ht = bm(hm), bt(ht)
            out.append(cosine(hm, ht))
    return out


@pytest.mark.parametrize("dtype,n_images", [(torch.float32, 2), (torch.float16, 16)])
def test_config3_vit_l_quarot_embeddings(cuda_device, dtype, n_images):
    """SAM ViT-L with QuaRot, W8A8: residual-stream rotation folded into the weights (Q from seed
    123), online 4096-point transform before lin2, transform across the 16 heads before proj; in
    fp32 tensors (the dtype the reference's evaluation runs in: it never casts the model to half)
    and in fp16 tensors with bf16 attention at the configuration's full batch of 16 images.

    COSINE >= 0.999 IS NOT REACHED on this configuration, in either dtype: the embeddings agree
    with the twin to about 0.997.  It is not a difference in the arithmetic of any layer: all 96
    layers reproduce the reference's codes bit for bit on identical inputs (teacher-forced test
    above).  A rotated, quantized, random-init network is chaotic in its roundings: a
    last-bit difference in one layer's float output (here: exact int32 dequantization against a
    float GEMM of fake-quantized values) is spread over the whole row by the next Hadamard, flips
    a few of the next quantizer's roundings, and each block amplifies the gap (1 - cos grows from
    1e-5 after one block to 3e-3 after 24, in fp32 as in fp16).  The reference's arithmetic
    disagrees with itself by the same amount when only the summation order of its float GEMM
    changes: ``alt`` below is the twin with every linear evaluated in fp64 and rounded once.  The
    assertions therefore are: the first block agrees to 1e-4; the product is as close to the twin
    as the twin is to its fp64-accumulating self; floors just under the measured values."""
    mine, twin, _, qlayers, _ = build_quarot_pair("vit_l", 3, dtype, cuda_device)
    assert len(qlayers) == 96
    alt = copy.deepcopy(twin)
    for m in alt.modules():
        if isinstance(m, RefActQuantWrapper):
            m.linear_dtype = torch.float64
    x = images(n_images, 30, dtype).to(cuda_device)
    per_block = _per_block_cosines(mine, twin, x[:1])
    per_block_alt = _per_block_cosines(alt, twin, x[:1])
    tag = str(dtype).split(".")[-1]
    print(f"{tag} per-block cosine, product vs twin:  ", " ".join(f"{c:.5f}" for c in per_block))
    print(f"{tag} per-block cosine, fp64 twin vs twin:", " ".join(f"{c:.5f}" for c in per_block_alt))
    assert per_block[0] >= 1 - 2e-4
    for k, c in enumerate(per_block):
        assert 1 - c <= 4e-4 * (k + 1) + 5e-4, (k, c)
    a, b, c = run_batched(mine, x, min(8, n_images)), run_batched(twin, x, 2), run_batched(alt, x, 2)
    c_mt, c_tt, c_ma = cosine(a, b), cosine(b, c), cosine(a, c)
    print(f"{tag} embeddings: product vs twin {c_mt:.5f}, twin vs fp64 twin {c_tt:.5f}, product vs fp64 twin {c_ma:.5f}")
    assert c_mt >= 0.995 and c_ma >= 0.995
    assert c_mt >= c_tt - 2e-3                    # as close to the reference as the reference is to itself
    if dtype == torch.float16:
        from sam_quantization_b200.sam_encoder import build_encoder
        y_float = run_batched(build_encoder("vit_l", seed=3, device=cuda_device), x[:2], 2)
        # both int8 paths track the float model equally well
        assert abs(cosine(a[:2], y_float) - cosine(b[:2], y_float)) < 0.01


# ---- configuration 4: ViT-H with SmoothQuant ---------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_config4_vit_h_smoothquant(cuda_device, dtype):
    """SAM ViT-H, SmoothQuant alpha 0.5 from the configuration's 8 calibration images through the
    float model, W8A8."""
    from sam_quantization_b200.RTN_quantization import (W8A8Linear, get_act_scales_sam,
                                                        replace_linear_with_target_and_quantize, smooth_sam)
    from sam_quantization_b200.sam_encoder import build_encoder
    mine = build_encoder("vit_h", seed=4, dtype=dtype, device=cuda_device,
                         attn_dtype=torch.bfloat16 if dtype == torch.float16 else None)
    twin = make_twin(mine)
    with torch.no_grad():
        scales = get_act_scales_sam(mine, (images(1, 200 + i, dtype).to(cuda_device) for i in range(8)), num_samples=8)
    smooth_sam(mine, scales, alpha=0.5)
    smooth_sam(twin, scales, alpha=0.5)
    replace_linear_with_target_and_quantize(mine, W8A8Linear, 8, [])
    replace_linears(twin, lambda lin: RefW8A8Linear.from_float(lin, 8))
    n = 2 if dtype == torch.float16 else 1
    x = images(n, 40, dtype).to(cuda_device)
    a, b = run_batched(mine, x, n), run_batched(twin, x, 1)
    print(f"ViT-H SmoothQuant {dtype}: cosine {cosine(a, b):.6f}")
    assert cosine(a, b) >= 0.999
    if dtype == torch.float16:
        # the CUDA-graph runner returns the same embeddings as the eager call
        from sam_quantization_b200.engine import EncoderRunner
        runner = EncoderRunner(mine, n, device=cuda_device)
        assert torch.equal(runner(x), a)
