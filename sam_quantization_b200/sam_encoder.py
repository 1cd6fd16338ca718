"""SAM's ViT image encoder, the host of the four quantized linears per block.

The reference imports this model from the `segment_anything` package of its sam-hq submodule
(quarot/model_utils.py:3-5), which is not part of the reference checkout; the architecture is
written here from its description: 16x16 patch embedding of a 1024x1024 image to 64x64 tokens,
learned absolute position embedding, pre-norm blocks (LayerNorm eps 1e-6) with fused-qkv
multi-head attention using decomposed relative position bias, 14x14 windowed attention except
at the global-attention blocks, a 4x MLP with GELU, and a convolutional neck to 256 channels.
Module names (`blocks.{i}.attn.qkv`, `.attn.proj`, `.mlp.lin1`, `.mlp.lin2`, `.norm1`,
`.norm2`) are the ones the reference's recipes address (RTN_quantization/calibration.py:65,
RTN_quantization/utils.py:177-199, quarot/rotate_sam.py:76-94).

Block / Attention / MLP know about quantized linears that can fuse the GELU or the residual add
into their GEMM epilogue (`supports_fused_epilogue`) and use that when present; with plain
`nn.Linear` children they are an ordinary float ViT.
"""
from __future__ import annotations

from typing import Optional, Tuple, Type

import torch
import torch.nn as nn
import torch.nn.functional as F

VIT_CONFIGS = {
    # name: (embed_dim, depth, num_heads, global_attn_indexes)   quarot/rotation_utils.py:295-309
    "vit_b": (768, 12, 12, (2, 5, 8, 11)),
    "vit_l": (1024, 24, 16, (5, 11, 17, 23)),
    "vit_h": (1280, 32, 16, (7, 15, 23, 31)),
}


def window_partition(x: torch.Tensor, window_size: int) -> Tuple[torch.Tensor, Tuple[int, int]]:
    """[B, H, W, C] -> [B * nW, ws, ws, C], zero-padding H and W up to a multiple of the window
    (quarot/model_utils.py:15-36)."""
    B, H, W, C = x.shape
    pad_h = (-H) % window_size
    pad_w = (-W) % window_size
    if pad_h or pad_w:
        x = F.pad(x, (0, 0, 0, pad_w, 0, pad_h))
    Hp, Wp = H + pad_h, W + pad_w
    x = x.view(B, Hp // window_size, window_size, Wp // window_size, window_size, C)
    return x.permute(0, 1, 3, 2, 4, 5).reshape(-1, window_size, window_size, C), (Hp, Wp)


def window_unpartition(windows: torch.Tensor, window_size: int, pad_hw: Tuple[int, int],
                       hw: Tuple[int, int]) -> torch.Tensor:
    """Inverse of ``window_partition`` with the padding cut off (quarot/model_utils.py:39-59)."""
    Hp, Wp = pad_hw
    H, W = hw
    B = windows.shape[0] // ((Hp // window_size) * (Wp // window_size))
    x = windows.view(B, Hp // window_size, Wp // window_size, window_size, window_size, -1)
    x = x.permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, -1)
    if Hp > H or Wp > W:
        x = x[:, :H, :W, :].contiguous()
    return x


def _fusable(mod) -> bool:
    return bool(getattr(mod, "supports_fused_epilogue", False))


class MLPBlock(nn.Module):
    def __init__(self, embedding_dim: int, mlp_dim: int, act: Type[nn.Module] = nn.GELU):
        super().__init__()
        self.lin1 = nn.Linear(embedding_dim, mlp_dim)
        self.lin2 = nn.Linear(mlp_dim, embedding_dim)
        self.act = act()

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if _fusable(self.lin1) and isinstance(self.act, nn.GELU) and self.act.approximate == "none":
            h = self.lin1(x, activation="gelu")
        else:
            h = self.act(self.lin1(x))
        if residual is not None:
            if _fusable(self.lin2):
                return self.lin2(h, residual=residual)
            return residual + self.lin2(h)
        return self.lin2(h)


def get_rel_pos(q_size: int, k_size: int, rel_pos: torch.Tensor) -> torch.Tensor:
    """Rows of the relative-position table for every (query, key) coordinate pair."""
    max_rel_dist = int(2 * max(q_size, k_size) - 1)
    if rel_pos.shape[0] != max_rel_dist:
        r = F.interpolate(rel_pos.reshape(1, rel_pos.shape[0], -1).permute(0, 2, 1).float(), size=max_rel_dist, mode="linear")
        rel_pos = r.reshape(-1, max_rel_dist).permute(1, 0).to(rel_pos.dtype)
    q_coords = torch.arange(q_size, device=rel_pos.device)[:, None] * max(k_size / q_size, 1.0)
    k_coords = torch.arange(k_size, device=rel_pos.device)[None, :] * max(q_size / k_size, 1.0)
    rel = (q_coords - k_coords) + (k_size - 1) * max(q_size / k_size, 1.0)
    return rel_pos[rel.long()]


def decomposed_rel_pos_bias(q: torch.Tensor, rel_pos_h: torch.Tensor, rel_pos_w: torch.Tensor,
                            q_size: Tuple[int, int], k_size: Tuple[int, int]) -> torch.Tensor:
    """Additive attention bias [B*heads, q_h*q_w, k_h*k_w] from the decomposed relative position
    embeddings: bias[(qh,qw),(kh,kw)] = q . Rh[qh-kh] + q . Rw[qw-kw]."""
    q_h, q_w = q_size
    k_h, k_w = k_size
    Rh = get_rel_pos(q_h, k_h, rel_pos_h).to(q.dtype)
    Rw = get_rel_pos(q_w, k_w, rel_pos_w).to(q.dtype)
    B, _, dim = q.shape
    r_q = q.reshape(B, q_h, q_w, dim)
    rel_h = torch.einsum("bhwc,hkc->bhwk", r_q, Rh)
    rel_w = torch.einsum("bhwc,wkc->bhwk", r_q, Rw)
    bias = rel_h[:, :, :, :, None] + rel_w[:, :, :, None, :]
    return bias.reshape(B, q_h * q_w, k_h * k_w)


class Attention(nn.Module):
    """Multi-head attention with a fused qkv projection and decomposed relative position bias.
    ``attn_dtype`` is the type the softmax(QK^T)V math runs in (bf16 in the W8A8 configs)."""

    def __init__(self, dim: int, num_heads: int = 8, qkv_bias: bool = True, use_rel_pos: bool = False,
                 rel_pos_zero_init: bool = True, input_size: Optional[Tuple[int, int]] = None):
        super().__init__()
        self.num_heads = num_heads
        head_dim = dim // num_heads
        self.scale = head_dim ** -0.5
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim)
        self.use_rel_pos = use_rel_pos
        self.attn_dtype: Optional[torch.dtype] = None
        self.global_chunk = 4            # images per SDPA call when the bias is [heads, 4096, 4096]
        if use_rel_pos:
            assert input_size is not None
            self.rel_pos_h = nn.Parameter(torch.zeros(2 * input_size[0] - 1, head_dim))
            self.rel_pos_w = nn.Parameter(torch.zeros(2 * input_size[1] - 1, head_dim))

    def _sdpa(self, q, k, v, H, W):
        # q, k, v: [B, heads, HW, d]
        B, nh, L, d = q.shape
        bias = None
        if self.use_rel_pos:
            bias = decomposed_rel_pos_bias(q.reshape(B * nh, L, d), self.rel_pos_h, self.rel_pos_w, (H, W), (H, W))
            bias = bias.view(B, nh, L, L)
        return F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=self.scale)

    def attend(self, qkv: torch.Tensor, B: int, H: int, W: int) -> torch.Tensor:
        """qkv [B, H*W, 3*C] -> attention output [B, H, W, C]."""
        L = H * W
        qkv = qkv.reshape(B, L, 3, self.num_heads, -1).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        step = B if L <= 1024 else max(1, self.global_chunk)
        outs = [self._sdpa(q[i:i + step], k[i:i + step], v[i:i + step], H, W) for i in range(0, B, step)]
        x = outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        return x.permute(0, 2, 1, 3).reshape(B, H, W, -1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, H, W, _ = x.shape
        dt = x.dtype
        adt = self.attn_dtype or dt
        if _fusable(self.qkv):
            qkv = self.qkv(x, out_dtype=adt)                 # the GEMM epilogue stores bf16 directly
        else:
            qkv = self.qkv(x).to(adt)
        x = self.attend(qkv, B, H, W).to(dt)
        return self.proj(x)


class Block(nn.Module):
    def __init__(self, dim: int, num_heads: int, mlp_ratio: float = 4.0, qkv_bias: bool = True,
                 norm_layer: Type[nn.Module] = nn.LayerNorm, act_layer: Type[nn.Module] = nn.GELU,
                 use_rel_pos: bool = False, rel_pos_zero_init: bool = True, window_size: int = 0,
                 input_size: Optional[Tuple[int, int]] = None):
        super().__init__()
        self.norm1 = norm_layer(dim)
        self.attn = Attention(dim, num_heads=num_heads, qkv_bias=qkv_bias, use_rel_pos=use_rel_pos,
                              rel_pos_zero_init=rel_pos_zero_init,
                              input_size=input_size if window_size == 0 else (window_size, window_size))
        self.norm2 = norm_layer(dim)
        self.mlp = MLPBlock(embedding_dim=dim, mlp_dim=int(dim * mlp_ratio), act=act_layer)
        self.window_size = window_size

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shortcut = x
        x = self.norm1(x)
        if self.window_size > 0:
            H, W = x.shape[1], x.shape[2]
            x, pad_hw = window_partition(x, self.window_size)
        x = self.attn(x)
        if self.window_size > 0:
            x = window_unpartition(x, self.window_size, pad_hw, (H, W))
        x = shortcut + x
        return self.mlp(self.norm2(x), residual=x)


class PatchEmbed(nn.Module):
    def __init__(self, kernel_size=(16, 16), stride=(16, 16), padding=(0, 0), in_chans=3, embed_dim=768):
        super().__init__()
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=kernel_size, stride=stride, padding=padding)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x).permute(0, 2, 3, 1)


class LayerNorm2d(nn.Module):
    def __init__(self, num_channels: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(num_channels))
        self.bias = nn.Parameter(torch.zeros(num_channels))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        u = x.mean(1, keepdim=True)
        s = (x - u).pow(2).mean(1, keepdim=True)
        x = (x - u) / torch.sqrt(s + self.eps)
        return self.weight[:, None, None] * x + self.bias[:, None, None]


class ImageEncoderViT(nn.Module):
    def __init__(self, img_size: int = 1024, patch_size: int = 16, in_chans: int = 3, embed_dim: int = 768,
                 depth: int = 12, num_heads: int = 12, mlp_ratio: float = 4.0, out_chans: int = 256,
                 qkv_bias: bool = True, norm_layer: Type[nn.Module] = None, act_layer: Type[nn.Module] = nn.GELU,
                 use_abs_pos: bool = True, use_rel_pos: bool = True, rel_pos_zero_init: bool = True,
                 window_size: int = 14, global_attn_indexes: Tuple[int, ...] = ()):
        super().__init__()
        if norm_layer is None:
            norm_layer = lambda d: nn.LayerNorm(d, eps=1e-6)     # noqa: E731
        self.img_size = img_size
        self.patch_embed = PatchEmbed((patch_size, patch_size), (patch_size, patch_size), in_chans=in_chans, embed_dim=embed_dim)
        grid = img_size // patch_size
        self.pos_embed = nn.Parameter(torch.zeros(1, grid, grid, embed_dim)) if use_abs_pos else None
        self.blocks = nn.ModuleList([
            Block(embed_dim, num_heads, mlp_ratio, qkv_bias, norm_layer, act_layer, use_rel_pos, rel_pos_zero_init,
                  window_size if i not in global_attn_indexes else 0, (grid, grid))
            for i in range(depth)])
        self.neck = nn.Sequential(
            nn.Conv2d(embed_dim, out_chans, kernel_size=1, bias=False), LayerNorm2d(out_chans),
            nn.Conv2d(out_chans, out_chans, kernel_size=3, padding=1, bias=False), LayerNorm2d(out_chans))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(x)
        if self.pos_embed is not None:
            x = x + self.pos_embed
        for blk in self.blocks:
            x = blk(x)
        return self.neck(x.permute(0, 3, 1, 2))


class SamEncoderModel(nn.Module):
    """Container exposing ``image_encoder`` the way the reference's recipes expect a SAM model
    to (``model.image_encoder.blocks``); the prompt encoder and mask decoder are out of scope."""

    def __init__(self, image_encoder: ImageEncoderViT):
        super().__init__()
        self.image_encoder = image_encoder

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        return self.image_encoder(images)


def build_encoder(model_type: str = "vit_b", img_size: int = 1024, window_size: int = 14, seed: int = 0,
                  dtype: torch.dtype = torch.float16, device="cpu", attn_dtype: Optional[torch.dtype] = torch.bfloat16,
                  embed_dim: Optional[int] = None, depth: Optional[int] = None, num_heads: Optional[int] = None,
                  global_attn_indexes: Optional[Tuple[int, ...]] = None, out_chans: int = 256) -> SamEncoderModel:
    """Random-init encoder of the given family: all weights N(0, 0.02) (LayerNorm weight 1, bias
    0; the relative-position tables also N(0, 0.02) so that they matter), deterministic in
    ``seed``.  Explicit dims override the family's (for small test models)."""
    e, d, h, g = VIT_CONFIGS[model_type]
    embed_dim, depth, num_heads = embed_dim or e, depth or d, num_heads or h
    g = g if global_attn_indexes is None else global_attn_indexes
    enc = ImageEncoderViT(img_size=img_size, embed_dim=embed_dim, depth=depth, num_heads=num_heads,
                          window_size=window_size, global_attn_indexes=tuple(g), out_chans=out_chans)
    gen = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in enc.named_parameters():
            if "norm" in name or name.startswith("neck.1") or name.startswith("neck.3"):
                continue                                     # LayerNorms keep weight 1 / bias 0
            p.copy_(torch.randn(p.shape, generator=gen) * 0.02)
    for blk in enc.blocks:
        blk.attn.attn_dtype = attn_dtype
    return SamEncoderModel(enc).to(device=device, dtype=dtype).eval()
