"""Offline weight rotation of the SAM image encoder (quarot/rotation_utils.py:106-219,286-453).

``rotate_model`` swaps each block's attention and MLP for the online-rotating variants and then
``rotate_model_sam`` rotates the weights: qkv and lin1 take ``W Q`` (fp64), lin2 and proj take an
exact Hadamard on their input side, and the V slice of qkv takes a per-head Hadamard on its
output side (weight rows and bias) that the online partial Hadamard before proj undoes.  The
mask-decoder part of the reference's function (:165-167,204-219) needs the SAM decoder and is
outside this package.
"""
from __future__ import annotations

import torch

from . import model_utils
from .hadamard_utils import apply_exact_had_to_linear, random_hadamard_matrix


def random_orthogonal_matrix(size, device, seed):
    """QR of a Gaussian matrix with the signs of R's diagonal folded in (:106-126)."""
    if seed is not None:
        torch.manual_seed(seed)
        torch.cuda.manual_seed_all(seed)
    g = torch.randn(size, size, dtype=torch.float64).to(device)
    q, r = torch.linalg.qr(g)
    q *= torch.sign(torch.diag(r)).unsqueeze(0)
    return q


def get_orthogonal_matrix(size, mode, device, seed):
    if mode == "random":
        return random_orthogonal_matrix(size, device, seed)
    if mode == "hadamard":
        return random_hadamard_matrix(size, device, seed)
    raise ValueError(f"Unknown mode {mode}")


@torch.inference_mode()
def rotate_model_sam(model, Q_image_encoder, Q_mask_decoder, args):
    dev = args.device
    Q = Q_image_encoder.to(device=dev, dtype=torch.float64)
    for block in model.image_encoder.blocks:
        for lin in (block.attn.qkv, block.mlp.lin1):                     # :148-159
            dtype, home = lin.weight.dtype, lin.weight.device
            lin.weight.data = torch.matmul(lin.weight.data.to(device=dev, dtype=torch.float64), Q).to(device=home, dtype=dtype)
    for block in model.image_encoder.blocks:                             # :162-164
        apply_exact_had_to_linear(block.mlp.lin2, had_dim=-1, output=False)
    head_dim = args.hidden_size_image_en // args.num_attention_head_image_en
    C = args.hidden_size_image_en
    for block in model.image_encoder.blocks:                             # :173-194
        qkv = block.attn.qkv
        v = torch.nn.Linear(C, C, bias=True).to(device=qkv.weight.device, dtype=qkv.weight.dtype)
        v.weight.data = qkv.weight.data[2 * C:3 * C, :].clone()
        v.bias.data = qkv.bias.data[2 * C:3 * C].clone()
        apply_exact_had_to_linear(v, had_dim=head_dim, output=True)
        qkv.weight.data[2 * C:3 * C, :] = v.weight.data
        qkv.bias.data[2 * C:3 * C] = v.bias.data
        apply_exact_had_to_linear(block.attn.proj, had_dim=-1, output=False)


def rotate_model(model, Q_image_encoder, Q_mask_decoder, args):
    """:286-453 — install the online-rotating attention / MLP in every block (weights shared,
    not copied), hand them Q, then rotate the weights."""
    dev = torch.device(args.device)
    model.to(dev)
    Q_image_encoder = Q_image_encoder.to(dev)
    for block in model.image_encoder.blocks:
        old_attn, old_mlp = block.attn, block.mlp
        dim = old_attn.qkv.in_features
        input_size = None
        if getattr(old_attn, "use_rel_pos", False):
            input_size = ((old_attn.rel_pos_h.shape[0] + 1) // 2, (old_attn.rel_pos_w.shape[0] + 1) // 2)
        attn = model_utils.CustomAttention(dim=dim, num_heads=old_attn.num_heads, qkv_bias=old_attn.qkv.bias is not None,
                                           use_rel_pos=old_attn.use_rel_pos, input_size=input_size)
        attn.qkv, attn.proj = old_attn.qkv, old_attn.proj
        attn.attn_dtype = getattr(old_attn, "attn_dtype", None)
        if old_attn.use_rel_pos:
            attn.rel_pos_h, attn.rel_pos_w = old_attn.rel_pos_h, old_attn.rel_pos_w
        mlp = model_utils.custom_MLPBlock(embedding_dim=dim, mlp_dim=old_mlp.lin1.out_features)
        mlp.lin1, mlp.lin2, mlp.act = old_mlp.lin1, old_mlp.lin2, old_mlp.act
        attn._take_Q(Q_image_encoder)
        mlp._take_Q(Q_image_encoder)
        block.attn, block.mlp = attn.to(dev), mlp.to(dev)
    rotate_model_sam(model, Q_image_encoder, Q_mask_decoder, args)
