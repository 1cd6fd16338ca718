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


_WINDOW_MAPS = {}


def window_row_maps(B: int, H: int, W: int, window_size: int, device) -> Tuple[torch.Tensor, torch.Tensor, Tuple[int, int]]:
    """Index form of ``window_partition`` / ``window_unpartition`` for token rows.

    ``part[r]``  : for row r of the window-ordered, zero-padded layout [B*nW*ws*ws], the row of the
                   [B*H*W] token layout it copies, or -1 for a padding row.
    ``unpart[t]``: for token row t, its row in the window-ordered layout.
    Both int32 on ``device``; cached per shape."""
    key = (B, H, W, window_size, str(device))
    if key not in _WINDOW_MAPS:
        tok = torch.arange(B * H * W, dtype=torch.float32).view(B, H, W, 1) + 1.0     # 0 marks padding
        win, (Hp, Wp) = window_partition(tok, window_size)
        part = (win.reshape(-1).to(torch.int64) - 1).to(torch.int32)
        pos = torch.arange(part.numel(), dtype=torch.float32).view(-1, window_size, window_size, 1)
        unpart = window_unpartition(pos, window_size, (Hp, Wp), (H, W)).reshape(-1).to(torch.int32)
        _WINDOW_MAPS[key] = (part.to(device), unpart.to(device), (Hp, Wp))
    return _WINDOW_MAPS[key]


class Attention(nn.Module):
    """Multi-head attention with a fused qkv projection and decomposed relative position bias.
    ``attn_dtype`` is the type the softmax(QK^T)V math runs in (bf16 in the W8A8 configs).

    The bias ``rel_h[q, kh] + rel_w[q, kw]`` is never materialised for windows: the query gets
    ``rel_h[q, :]`` and ``rel_w[q, :]`` appended to its features and the key gets one-hot codes of
    its row and column, so that ``q' . k' = scale * q . k + rel_h[q, kh] + rel_w[q, kw]`` and a
    stock fused attention kernel applies (head width d + H + W <= 128).  Global attention
    (64 x 64 keys) would need 128 extra features; it adds an explicit bias instead."""

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
        self.global_chunk = 4            # images per attention call when the bias is [heads, 4096, 4096]
        self.native_prep = True          # build the attention inputs with the library's CUDA kernels when possible
        # whole windowed attention in the library's own kernel (samq_attn_windowed).  Off by default: at
        # 0.43 ms for 200 windows x 16 heads it is still slower than augmented rows + the fused library
        # attention (0.31 ms); it needs K/V prefetch across windows to hide its load phase
        self.fused_window_kernel = False
        # attention of whole images (64 tokens wide) and of windows up to 16 x 16 in the library's tensor-core
        # kernel (samq_attn_global): scores and the relative-position bias stay on chip instead of going through
        # a [heads, L, L] bias tensor or augmented q / k rows
        self.fused_global_kernel = True
        # the same kernel for windows other than 14 x 14: correct, but one short-lived CTA per (window, head,
        # 128 queries) spends most of its ~10 us on set-up and pipeline fill; off by default
        self.tc_windows = False
        # 14 x 14 windows (every windowed block of SAM) in the persistent tensor-core kernel samq_attn_window14:
        # q, k, v read in place, the table products computed by the same MMA as the scores
        self.window14_kernel = True
        self._onehot = {}
        if use_rel_pos:
            assert input_size is not None
            self.rel_pos_h = nn.Parameter(torch.zeros(2 * input_size[0] - 1, head_dim))
            self.rel_pos_w = nn.Parameter(torch.zeros(2 * input_size[1] - 1, head_dim))

    # -- relative position terms -------------------------------------------------------------
    def _rel_terms(self, q: torch.Tensor, H: int, W: int):
        """q [B, H*W, nh, d] (any strides) -> rel_h [B, H, W, nh, H], rel_w [B, H, W, nh, W]."""
        B, L, nh, d = q.shape
        Rh = get_rel_pos(H, H, self.rel_pos_h).to(q.dtype)
        Rw = get_rel_pos(W, W, self.rel_pos_w).to(q.dtype)
        r_q = q.reshape(B, H, W, nh, d)
        rel_h = torch.einsum("bhwnc,hkc->bhwnk", r_q, Rh)
        rel_w = torch.einsum("bhwnc,wkc->bhwnk", r_q, Rw)
        return rel_h, rel_w

    def _key_codes(self, H: int, W: int, width: int, dtype, device) -> torch.Tensor:
        key = (H, W, width, dtype, str(device))
        if key not in self._onehot:
            kh = torch.arange(H).view(H, 1).expand(H, W).reshape(-1)
            kw = torch.arange(W).view(1, W).expand(H, W).reshape(-1)
            codes = torch.zeros(H * W, width)
            codes[torch.arange(H * W), kh] = 1.0
            codes[torch.arange(H * W), H + kw] = 1.0
            self._onehot[key] = codes.to(device=device, dtype=dtype)
        return self._onehot[key]

    def _rel_table(self, dtype, device) -> torch.Tensor:
        """Both relative-position tables as one matrix in the attention dtype, rebuilt only when
        a table changed (new storage or an in-place update)."""
        key = (self.rel_pos_h.data_ptr(), self.rel_pos_w.data_ptr(), self.rel_pos_h._version, self.rel_pos_w._version,
               dtype, str(device))
        cached = self.__dict__.get("_table_cache")
        if cached is None or cached[0] != key:
            from . import ops
            cached = (key, ops.rel_pos_table(self.rel_pos_h, self.rel_pos_w, dtype, device))
            self.__dict__["_table_cache"] = cached
        return cached[1]

    def _native(self, qkv: torch.Tensor, d: int, H: int, W: int) -> bool:
        if not (self.native_prep and qkv.is_cuda and qkv.dtype in (torch.float16, torch.bfloat16) and qkv.is_contiguous()):
            return False
        if d % 8 != 0:
            return False
        return d + H + W <= 128 or (H <= 64 and W % 8 == 0)

    def attend_flat(self, qkv: torch.Tensor, B: int, H: int, W: int) -> torch.Tensor:
        """qkv [B*H*W, 3C] -> attention output [B*H*W, C] (same dtype), heads side by side."""
        L, nh = H * W, self.num_heads
        qkv5 = qkv.view(B, L, 3, nh, -1)
        q, k, v = qkv5[:, :, 0], qkv5[:, :, 1], qkv5[:, :, 2]          # [B, L, nh, d] strided views
        d = q.shape[-1]
        if not self.use_rel_pos:
            out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=self.scale)
            return out.transpose(1, 2).reshape(B * L, nh * d)
        extra = H + W
        if self._native(qkv, d, H, W):
            from . import ops
            if self.window14_kernel and ops.attn_window14_supported(H, W, d, qkv.dtype):
                return ops.attn_window14(qkv, B, nh, self.rel_pos_h, self.rel_pos_w, self.scale,
                                         table=self._rel_table(qkv.dtype, qkv.device))
            if self.fused_window_kernel and ops.attn_windowed_supported(H, W, d):
                return ops.attn_windowed(qkv, B, H, W, nh, self.rel_pos_h, self.rel_pos_w, self.scale,
                                         table=self._rel_table(qkv.dtype, qkv.device))
            if self.fused_global_kernel and (W == 64 or self.tc_windows) and ops.attn_global_supported(H, W, d, qkv.dtype):
                return ops.attn_global(qkv, B, H, W, nh, self.rel_pos_h, self.rel_pos_w, self.scale,
                                       table=self._rel_table(qkv.dtype, qkv.device))
            if d + extra <= 128:
                width = (d + extra + 7) // 8 * 8
                qa, ka = ops.attn_window_prep(qkv, H, W, nh, self.rel_pos_h, self.rel_pos_w, self.scale, width,
                                              table=self._rel_table(qkv.dtype, qkv.device))
                out = F.scaled_dot_product_attention(qa.view(B, L, nh, width).transpose(1, 2), ka.view(B, L, nh, width).transpose(1, 2),
                                                     v.transpose(1, 2), scale=1.0)
                return out.transpose(1, 2).reshape(B * L, nh * d)
            outs = []
            step = max(1, self.global_chunk)
            for i in range(0, B, step):
                b = min(step, B - i)
                bias = ops.attn_rel_bias(qkv[i * L:(i + b) * L], b, H, W, nh, self.rel_pos_h, self.rel_pos_w,
                                         table=self._rel_table(qkv.dtype, qkv.device))
                o = F.scaled_dot_product_attention(q[i:i + b].transpose(1, 2), k[i:i + b].transpose(1, 2),
                                                   v[i:i + b].transpose(1, 2), attn_mask=bias, scale=self.scale)
                outs.append(o.transpose(1, 2).reshape(b * L, nh * d))
            return outs[0] if len(outs) == 1 else torch.cat(outs, 0)
        rel_h, rel_w = self._rel_terms(q, H, W)
        if d + extra <= 128:
            width = (d + extra + 7) // 8 * 8
            qa = q.new_zeros((B, L, nh, width)) if width > d + extra else q.new_empty((B, L, nh, width))
            qa[..., :d] = q * self.scale
            qa[..., d:d + H] = rel_h.reshape(B, L, nh, H)
            qa[..., d + H:d + extra] = rel_w.reshape(B, L, nh, W)
            ka = q.new_empty((B, L, nh, width))
            ka[..., :d] = k
            ka[..., d:] = self._key_codes(H, W, width - d, q.dtype, q.device).view(1, L, 1, width - d)
            out = F.scaled_dot_product_attention(qa.transpose(1, 2), ka.transpose(1, 2), v.transpose(1, 2), scale=1.0)
            return out.transpose(1, 2).reshape(B * L, nh * d)
        outs = []
        step = max(1, self.global_chunk)
        for i in range(0, B, step):
            rh, rw = rel_h[i:i + step], rel_w[i:i + step]                  # [b, H, W, nh, H|W]
            b = rh.shape[0]
            bias = rh.permute(0, 3, 1, 2, 4).reshape(b, nh, L, H, 1) + rw.permute(0, 3, 1, 2, 4).reshape(b, nh, L, 1, W)
            o = F.scaled_dot_product_attention(q[i:i + step].transpose(1, 2), k[i:i + step].transpose(1, 2),
                                               v[i:i + step].transpose(1, 2), attn_mask=bias.view(b, nh, L, L), scale=self.scale)
            outs.append(o.transpose(1, 2).reshape(b * L, nh * d))
        return outs[0] if len(outs) == 1 else torch.cat(outs, 0)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, H, W, C = x.shape
        dt = x.dtype
        adt = self.attn_dtype or dt
        if _fusable(self.qkv):
            qkv = self.qkv(x, out_dtype=adt)                 # the GEMM epilogue stores bf16 directly
        else:
            qkv = self.qkv(x).to(adt)
        o = self.attend_flat(qkv.reshape(B * H * W, 3 * C), B, H, W).to(dt)
        return self.proj(o.view(B, H, W, C))


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
        self.fuse = True                 # allow the fused quantized path when the linears support it

    # -- fused quantized path --------------------------------------------------------------------
    def _can_fuse(self, x: torch.Tensor) -> bool:
        if not (self.fuse and x.is_cuda and x.dim() == 4):
            return False
        lins = (self.attn.qkv, self.attn.proj, self.mlp.lin1, self.mlp.lin2)
        if not all(hasattr(m, "forward_fused") and m.can_fuse_prologue() for m in lins):
            return False
        if not (isinstance(self.norm1, nn.LayerNorm) and isinstance(self.norm2, nn.LayerNorm)):
            return False
        if not (isinstance(self.mlp.act, nn.GELU) and self.mlp.act.approximate == "none"):
            return False
        # an online dense rotation in front of qkv / lin1 must have been folded into the kernels
        for holder, lin in ((self.attn, self.attn.qkv), (self.mlp, self.mlp.lin1)):
            if getattr(holder, "Q", None) is not None and getattr(lin, "pre_signs", None) is None:
                return False
        return True

    def _forward_fused(self, x: torch.Tensor) -> torch.Tensor:
        """The block with LayerNorm, window partition / unpartition, GELU, both residual adds and
        the dtype casts around attention folded into the quantization and GEMM kernels:
        K1(norm1 + window gather) -> K2(qkv) -> attention -> K1(window scatter as a gather) ->
        K2(proj + residual) -> K1(norm2) -> K2(lin1 + GELU) -> K1 -> K2(lin2 + residual)."""
        B, H, W, C = x.shape
        x2 = x.reshape(B * H * W, C)
        adt = self.attn.attn_dtype or x.dtype
        ln1 = (self.norm1.weight, self.norm1.bias, self.norm1.eps)
        ln2 = (self.norm2.weight, self.norm2.bias, self.norm2.eps)
        if self.window_size > 0:
            part, unpart, (Hp, Wp) = window_row_maps(B, H, W, self.window_size, x.device)
            ws = self.window_size
            qkv = self.attn.qkv.forward_fused(x2, row_map=part, layer_norm=ln1, out_dtype=adt)
            o = self.attn.attend_flat(qkv, qkv.shape[0] // (ws * ws), ws, ws)
            y = self.attn.proj.forward_fused(o, row_map=unpart, as_dtype=x.dtype, residual=x2)
        else:
            qkv = self.attn.qkv.forward_fused(x2, layer_norm=ln1, out_dtype=adt)
            o = self.attn.attend_flat(qkv, B, H, W)
            y = self.attn.proj.forward_fused(o, as_dtype=x.dtype, residual=x2)
        h = self.mlp.lin1.forward_fused(y, layer_norm=ln2, activation="gelu")
        out = self.mlp.lin2.forward_fused(h, residual=y)
        return out.view(B, H, W, C)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._can_fuse(x):
            return self._forward_fused(x)
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
    """Non-overlapping patch projection.  The parameter lives in a Conv2d (``proj``) as in the
    original model; because kernel == stride it is evaluated as one matrix product over the
    unfolded patches, which is what a tensor-core GEMM wants."""

    def __init__(self, kernel_size=(16, 16), stride=(16, 16), padding=(0, 0), in_chans=3, embed_dim=768):
        super().__init__()
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=kernel_size, stride=stride, padding=padding)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        kh, kw = self.proj.kernel_size
        if tuple(self.proj.stride) != (kh, kw) or tuple(self.proj.padding) != (0, 0) or x.shape[2] % kh or x.shape[3] % kw:
            return self.proj(x).permute(0, 2, 3, 1)
        B, C, H, W = x.shape
        patches = x.view(B, C, H // kh, kh, W // kw, kw).permute(0, 2, 4, 1, 3, 5).reshape(B, H // kh, W // kw, C * kh * kw)
        return F.linear(patches, self.proj.weight.view(self.proj.out_channels, -1), self.proj.bias)


class LayerNorm2d(nn.Module):
    """LayerNorm over the channel axis of an NCHW tensor."""

    def __init__(self, num_channels: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(num_channels))
        self.bias = nn.Parameter(torch.zeros(num_channels))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        # per pixel over channels; done on the channels-last view so it is one fused kernel
        y = F.layer_norm(x.permute(0, 2, 3, 1), (x.shape[1],), self.weight, self.bias, self.eps)
        return y.permute(0, 3, 1, 2)


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

    def _neck(self, x: torch.Tensor) -> torch.Tensor:
        """x [B, H, W, C] -> [B, out, H, W].  The 1x1 convolution is a matrix product on the
        channels-last activations; the 3x3 convolution runs on the channels-last view."""
        c1, n1, c2, n2 = self.neck
        y = F.linear(x, c1.weight.view(c1.out_channels, -1), c1.bias)
        y = F.layer_norm(y, (c1.out_channels,), n1.weight, n1.bias, n1.eps)
        y = c2(y.permute(0, 3, 1, 2))
        return n2(y)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.patch_embed(x)
        if self.pos_embed is not None:
            x = x + self.pos_embed
        for blk in self.blocks:
            x = blk(x)
        return self._neck(x)


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
