"""Generates tests/golden/*.npz by running the reference's own Python functions on seeded inputs.

Run once where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/SAM_Quantization

The fixtures are committed; nothing at test time needs the reference.  fp16 / bf16 tensors are
stored widened to float32 (exact), integer tables as int8.
"""
from __future__ import annotations

import hashlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _import_reference(root):
    sys.path.insert(0, os.path.join(root, "RTN_quantization"))
    sys.path.insert(0, os.path.join(root, "quarot"))
    # the reference imports Dao-AILab's fast_hadamard_transform at module load; it is not part
    # of the checkout and only its CUDA entry is used, never by the functions called below
    sys.modules.setdefault("fast_hadamard_transform", types.ModuleType("fast_hadamard_transform"))
    import per_tensor_channel_group as ptcg
    import Smooth
    import hadamard_utils
    return ptcg, Smooth, hadamard_utils


def f32(t):
    return t.detach().to(torch.float32).cpu().clone().numpy()


def make_input(seed, shape, dtype, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape, generator=g)
    if outliers and shape[-1] >= 8:
        n_out = max(1, shape[-1] // 100)
        idx = torch.randperm(shape[-1], generator=g)[:n_out]
        x[..., idx] *= 20
    return x.to(dtype)


DT = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def quantizer_cases(ptcg):
    out = {}
    for dname, dt in DT.items():
        x = make_input(11, (24, 96), dt)
        x[3] = 0                                   # all-zero row -> clamp floor
        x[4] = x[4] * 1e-4                         # tiny row -> subnormal fp16 scale
        x[5, 0] = 30000.0 if dname != "f32" else 3e4
        out[f"{dname}/x"] = f32(x)
        out[f"{dname}/act_per_token"] = f32(ptcg.quantize_activation_per_token_absmax(x.clone()))
        out[f"{dname}/act_per_tensor"] = f32(ptcg.quantize_activation_per_tensor_absmax(x.clone()))
        out[f"{dname}/act_per_group32"] = f32(ptcg.quantize_activation_per_group_absmax_token_dim(x.clone(), 32))
        x3 = make_input(12, (2, 5, 64), dt)
        out[f"{dname}/x3"] = f32(x3)
        out[f"{dname}/act3_per_token"] = f32(ptcg.quantize_activation_per_token_absmax(x3.clone()))
        out[f"{dname}/act3_per_group16"] = f32(ptcg.quantize_activation_per_group_absmax_token_dim(x3.clone(), 16))
        w = (make_input(13, (40, 96), torch.float32, outliers=False) * 0.02).to(dt)
        out[f"{dname}/w"] = f32(w)
        out[f"{dname}/w_per_channel"] = f32(ptcg.quantize_weight_per_channel_absmax(w.clone()))
        out[f"{dname}/w_per_tensor"] = f32(ptcg.quantize_weight_per_tensor_absmax(w.clone()))
        out[f"{dname}/w_per_group32"] = f32(ptcg.quantize_weight_per_group_absmax_input_features(w.clone(), 32))
    return out


def linear_cases(ptcg):
    out = {}
    combos = [("per_channel", "per_token", None, False), ("per_tensor", "per_tensor", None, False),
              ("per_group", "per_group_token", 32, False), ("per_channel", "per_token", None, True),
              ("per_group", "per_token", 128, False)]
    for dname, dt in DT.items():
        x = make_input(21, (48, 256), dt)
        g = torch.Generator().manual_seed(22)
        w = (torch.randn(72, 256, generator=g) * 0.02).to(dt)
        b = (torch.randn(72, generator=g) * 0.01).to(dt)
        out[f"{dname}/x"], out[f"{dname}/w"], out[f"{dname}/b"] = f32(x), f32(w), f32(b)
        for wq, aq, gs, qo in combos:
            lin = torch.nn.Linear(256, 72, bias=True)
            lin.weight.data = w.clone()
            lin.bias.data = b.clone()
            m = ptcg.W8A8Linear.from_float(lin, 8, weight_quant=wq, act_quant=aq, quantize_output=qo, group_size=gs)
            y = m(x.clone())
            out[f"{dname}/y/{wq}/{aq}/{gs}/{int(qo)}"] = f32(y)
        out[f"{dname}/repr"] = np.array(repr(m))
    return out


def smooth_cases(Smooth):
    out = {}
    for dname, dt in (("f16", torch.float16), ("f32", torch.float32)):
        g = torch.Generator().manual_seed(31)
        C = 64
        ln = torch.nn.LayerNorm(C)
        ln.weight.data = (1 + 0.1 * torch.randn(C, generator=g)).to(dt)
        ln.bias.data = (0.1 * torch.randn(C, generator=g)).to(dt)
        fc1 = torch.nn.Linear(C, 96)
        fc2 = torch.nn.Linear(C, 32)
        fc1.weight.data = (0.02 * torch.randn(96, C, generator=g)).to(dt)
        fc2.weight.data = (0.02 * torch.randn(32, C, generator=g)).to(dt)
        act = torch.rand(C, generator=g) * 10 + 0.1
        act[5] = 200.0
        out[f"{dname}/ln_w"], out[f"{dname}/ln_b"] = f32(ln.weight), f32(ln.bias)
        out[f"{dname}/fc1_w"], out[f"{dname}/fc2_w"] = f32(fc1.weight), f32(fc2.weight)
        out[f"{dname}/act_scales"] = f32(act)
        Smooth.smooth_ln_fcs(ln, [fc1, fc2], act, alpha=0.5)
        out[f"{dname}/ln_w_s"], out[f"{dname}/ln_b_s"] = f32(ln.weight), f32(ln.bias)
        out[f"{dname}/fc1_w_s"], out[f"{dname}/fc2_w_s"] = f32(fc1.weight), f32(fc2.weight)
    return out


def hadamard_cases(H):
    out = {}
    for k in (12, 20, 28, 36, 40):
        out[f"had{k}"] = getattr(H, f"get_had{k}")().numpy().astype(np.int8)
    for n in (768, 1024, 1280, 3072, 4096, 5120, 12, 16, 64):
        _, k = H.get_hadK(n)
        out[f"hadK_of/{n}"] = np.array(k)
    for n in (16, 64, 256, 1024, 4096, 48, 768, 1280, 160):
        g = torch.Generator().manual_seed(40 + n)
        x = torch.randn(3, n, generator=g)
        out[f"hadU/{n}/x"] = f32(x)
        out[f"hadU/{n}/y"] = f32(H.matmul_hadU(x))
        xh = x.to(torch.float16)
        out[f"hadU/{n}/y_f16_via_f32"] = f32(H.matmul_hadU(xh.float()).to(torch.float16))
    for n in (64, 1024, 768):
        Q = H.random_hadamard_matrix(n, "cpu", 123)
        out[f"randhad/{n}/sha256"] = np.array(hashlib.sha256(Q.numpy().tobytes()).hexdigest())
        out[f"randhad/{n}/row0"] = Q[0].numpy()
        out[f"randhad/{n}/diag"] = torch.diagonal(Q).numpy()
        torch.manual_seed(123)
        s = torch.randint(low=0, high=2, size=(n,)).to(torch.float64) * 2 - 1
        out[f"randhad/{n}/signs"] = s.numpy().astype(np.int8)
    return out


def config1_case(ptcg, Smooth):
    """The single-linear benchmark configuration (one W8A8 linear, ViT-B fc1 of one image) run through the reference:
    inputs are regenerated from seeds at test time; outputs are kept as digests plus a strided
    sample so the fixture stays small."""
    out = {}
    g = torch.Generator().manual_seed(1)
    M, K, N = 4096, 768, 3072
    x = torch.randn(M, K, generator=g)
    idx = torch.randperm(K, generator=g)[:max(1, K // 100)]
    x[:, idx] *= 20
    w = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.01
    act = None
    for s in range(100, 108):
        gc = torch.Generator().manual_seed(s)
        xc = torch.randn(M, K, generator=gc)
        xc[:, idx] *= 20
        cur = xc.to(torch.float16).abs().max(dim=0)[0].float()
        act = cur if act is None else torch.max(act, cur)
    ln = torch.nn.LayerNorm(K)
    ln.weight.data = torch.ones(K, dtype=torch.float16)
    ln.bias.data = torch.zeros(K, dtype=torch.float16)
    lin = torch.nn.Linear(K, N)
    lin.weight.data = w.to(torch.float16)
    lin.bias.data = b.to(torch.float16)
    Smooth.smooth_ln_fcs(ln, [lin], act, alpha=0.5)
    s = 1.0 / ln.weight.data.float()          # ln.weight = 1 / s
    xs = (x.to(torch.float16) * ln.weight.data)   # LayerNorm's elementwise scale: x * (1/s)
    out["outlier_idx"] = idx.numpy()
    out["act_scales"] = f32(act)
    out["ln_weight_after"] = f32(ln.weight.data)
    out["w_smoothed_sha256"] = np.array(hashlib.sha256(lin.weight.data.numpy().tobytes()).hexdigest())
    fq_x = ptcg.quantize_activation_per_token_absmax(xs.clone())
    out["fq_x_sha256"] = np.array(hashlib.sha256(fq_x.numpy().tobytes()).hexdigest())
    m = ptcg.W8A8Linear.from_float(lin, 8, weight_quant="per_channel", act_quant="per_token")
    out["fq_w_sha256"] = np.array(hashlib.sha256(m.weight.data.numpy().tobytes()).hexdigest())
    y = m(xs.clone())
    out["y_sha256"] = np.array(hashlib.sha256(y.numpy().tobytes()).hexdigest())
    out["y_sample"] = f32(y[::97, ::53])
    out["fq_x_sample"] = f32(fq_x[::97, ::13])
    del s
    return out


TINY = dict(model_type="vit_b", img_size=224, window_size=4, embed_dim=64, depth=3, num_heads=4,
            global_attn_indexes=(2,), out_chans=32)


def tiny_images(seed=7, n=2, size=224):
    g = torch.Generator().manual_seed(seed)
    img = torch.rand(n, 3, size, size, generator=g)
    mean = torch.tensor([0.485, 0.456, 0.406]).view(1, 3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(1, 3, 1, 1)
    return (img - mean) / std


def encoder_case(ptcg):
    """A small encoder of this repository's architecture (14x14 tokens, window 4 -> padded to 16,
    one global block) whose Linears are replaced by the reference's own W8A8Linear, fp32 on CPU.
    Stores the embeddings for two quantization settings."""
    repo = os.path.dirname(os.path.dirname(HERE))
    sys.path.insert(0, repo)
    from sam_quantization_b200.sam_encoder import build_encoder
    from oracle.torch_twin import replace_linears
    out = {}
    for tag, kw in (("w8a8", dict(weight_quant="per_channel", act_quant="per_token", quantize_output=False)),
                    ("w8a8_qout", dict(weight_quant="per_channel", act_quant="per_token", quantize_output=True)),
                    ("w8a8_tensor", dict(weight_quant="per_tensor", act_quant="per_tensor", quantize_output=False))):
        model = build_encoder(seed=5, dtype=torch.float32, attn_dtype=None, **TINY)
        replace_linears(model, lambda lin: ptcg.W8A8Linear.from_float(lin, 8, **kw))
        with torch.no_grad():
            emb = model(tiny_images())
        out[f"{tag}/embedding"] = emb.numpy().astype(np.float32)
    model = build_encoder(seed=5, dtype=torch.float32, attn_dtype=None, **TINY)
    with torch.no_grad():
        out["float/embedding"] = model(tiny_images()).numpy().astype(np.float32)
    return out


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of hchautran/SAM_Quantization>")
    root = sys.argv[1]
    ptcg, Smooth, H = _import_reference(root)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    np.savez_compressed(os.path.join(HERE, "quantizers.npz"), **quantizer_cases(ptcg))
    np.savez_compressed(os.path.join(HERE, "w8a8_linear.npz"), **linear_cases(ptcg))
    np.savez_compressed(os.path.join(HERE, "smooth.npz"), **smooth_cases(Smooth))
    np.savez_compressed(os.path.join(HERE, "hadamard.npz"), **hadamard_cases(H))
    np.savez_compressed(os.path.join(HERE, "config1.npz"), **config1_case(ptcg, Smooth))
    np.savez_compressed(os.path.join(HERE, "encoder_tiny.npz"), **encoder_case(ptcg))
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
