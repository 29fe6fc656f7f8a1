"""Whole-model workloads for the drop-in hooks: a plain ViT and a Swin-v1 whose attention modules have the timm
attribute surface, so `patch_timm_attention(_train)` rewires them exactly as it would rewire a timm model (timm
itself need not be installed), plus the data-parallel gradient exchange for training them on several GPUs.

Reference: the hooks are exercised on timm `vit_tiny_patch16_*` / `swin_tiny_patch4_window7_*` models by
benchmarks/bench_timm_dropin.py and bench_timm_dropin_bwd.py, and recognised purely by attribute names
(src/elsa_twopass_clean/timm_dropin.py:153-172).  The models below follow the published architectures:
ViT-Tiny = patch 16, width 192, 12 blocks, 3 heads of 64, MLP 768, class token, learned positions;
Swin-T = patch 4, widths 96/192/384/768, depths 2/2/6/2, heads 3/6/12/24 of 32, 7x7 windows, every second block
shifted by 3, patch merging between stages, relative-position bias table per block.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F


# ---- attention modules with the timm attribute surface ------------------------------------------------
class VitAttention(nn.Module):
    """Multi-head self-attention as timm's ViT `Attention`: qkv, q_norm, k_norm, proj, num_heads, head_dim."""

    def __init__(self, dim: int, num_heads: int, qkv_bias: bool = True):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = dim // num_heads
        self.scale = self.head_dim ** -0.5
        self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
        self.q_norm = nn.Identity()
        self.k_norm = nn.Identity()
        self.attn_drop = nn.Dropout(0.0)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(0.0)

    def forward(self, x, attn_mask=None):
        b, n, c = x.shape
        qkv = self.qkv(x).reshape(b, n, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        q, k = self.q_norm(q), self.k_norm(k)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask)
        return self.proj_drop(self.proj(y.transpose(1, 2).reshape(b, n, c)))


def relative_position_index(win_h: int, win_w: int) -> torch.Tensor:
    coords = torch.stack(torch.meshgrid(torch.arange(win_h), torch.arange(win_w), indexing="ij")).flatten(1)
    rel = (coords[:, :, None] - coords[:, None, :]).permute(1, 2, 0).contiguous()
    rel[:, :, 0] += win_h - 1
    rel[:, :, 1] += win_w - 1
    rel[:, :, 0] *= 2 * win_w - 1
    return rel.sum(-1)


class SwinWindowAttention(nn.Module):
    """Window attention as timm's Swin-v1 `WindowAttention`: qkv, proj, relative_position_bias_table,
    relative_position_index, window_area, window_size, scale, num_heads, dim, softmax (and no logit_scale)."""

    def __init__(self, dim: int, num_heads: int, window_size):
        super().__init__()
        self.dim = dim
        self.window_size = tuple(window_size)
        self.window_area = self.window_size[0] * self.window_size[1]
        self.num_heads = num_heads
        self.scale = (dim // num_heads) ** -0.5
        self.relative_position_bias_table = nn.Parameter(
            torch.randn((2 * self.window_size[0] - 1) * (2 * self.window_size[1] - 1), num_heads) * 0.02)
        self.register_buffer("relative_position_index", relative_position_index(*self.window_size), persistent=False)
        self.qkv = nn.Linear(dim, dim * 3)
        self.attn_drop = nn.Dropout(0.0)
        self.proj = nn.Linear(dim, dim)
        self.proj_drop = nn.Dropout(0.0)
        self.softmax = nn.Softmax(dim=-1)

    def forward(self, x, mask=None):
        bw, n, c = x.shape
        qkv = self.qkv(x).reshape(bw, n, 3, self.num_heads, -1).permute(2, 0, 3, 1, 4)
        q, k, v = qkv.unbind(0)
        attn = (q * self.scale) @ k.transpose(-2, -1)
        bias = self.relative_position_bias_table[self.relative_position_index.view(-1)].view(n, n, -1)
        attn = attn + bias.permute(2, 0, 1).unsqueeze(0).to(attn.dtype)
        if mask is not None:
            nw = mask.shape[0]
            attn = attn.view(-1, nw, self.num_heads, n, n) + mask.unsqueeze(1).unsqueeze(0).to(attn.dtype)
            attn = attn.view(-1, self.num_heads, n, n)
        attn = self.softmax(attn)
        y = (attn @ v).transpose(1, 2).reshape(bw, n, c)
        return self.proj_drop(self.proj(y))


class _Mlp(nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden)
        self.fc2 = nn.Linear(hidden, dim)

    def forward(self, x):
        return self.fc2(F.gelu(self.fc1(x)))


def _init_weights(module: nn.Module) -> None:
    """trunc_normal(std 0.02) for linear / embedding weights, zeros for biases, ones / zeros for LayerNorm."""
    for m in module.modules():
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.LayerNorm):
            nn.init.ones_(m.weight)
            nn.init.zeros_(m.bias)


# ---- ViT ------------------------------------------------------------------------------------------------
class VitBlock(nn.Module):
    def __init__(self, dim: int, heads: int, mlp_hidden: int):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=1e-6)
        self.attn = VitAttention(dim, heads)
        self.norm2 = nn.LayerNorm(dim, eps=1e-6)
        self.mlp = _Mlp(dim, mlp_hidden)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class VisionTransformer(nn.Module):
    """Plain ViT classifier.  Defaults are ViT-Tiny; a 1024 x 1024 input gives 64*64 + 1 = 4097 tokens."""

    def __init__(self, *, img_size: int = 1024, patch: int = 16, dim: int = 192, depth: int = 12, heads: int = 3,
                 mlp_hidden: int = 768, num_classes: int = 1000, in_chans: int = 3):
        super().__init__()
        self.patch_embed = nn.Conv2d(in_chans, dim, kernel_size=patch, stride=patch)
        tokens = (img_size // patch) ** 2
        self.cls_token = nn.Parameter(torch.zeros(1, 1, dim))
        self.pos_embed = nn.Parameter(torch.zeros(1, tokens + 1, dim))
        self.blocks = nn.ModuleList([VitBlock(dim, heads, mlp_hidden) for _ in range(depth)])
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.head = nn.Linear(dim, num_classes)
        nn.init.trunc_normal_(self.pos_embed, std=0.02)
        nn.init.trunc_normal_(self.cls_token, std=0.02)
        _init_weights(self)

    def forward(self, img):
        x = self.patch_embed(img).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1) + self.pos_embed.to(x.dtype)
        for blk in self.blocks:
            x = blk(x)
        return self.head(self.norm(x)[:, 0])


def vit_tiny(img_size: int = 1024, num_classes: int = 1000) -> VisionTransformer:
    return VisionTransformer(img_size=img_size, patch=16, dim=192, depth=12, heads=3, mlp_hidden=768,
                             num_classes=num_classes)


# ---- Swin-v1 -----------------------------------------------------------------------------------------------
def _window_partition(x, w: int):
    b, hh, ww, c = x.shape
    x = x.view(b, hh // w, w, ww // w, w, c)
    return x.permute(0, 1, 3, 2, 4, 5).reshape(-1, w * w, c)


def _window_reverse(win, w: int, hh: int, ww: int):
    b = win.shape[0] // ((hh // w) * (ww // w))
    x = win.view(b, hh // w, ww // w, w, w, -1)
    return x.permute(0, 1, 3, 2, 4, 5).reshape(b, hh, ww, -1)


class SwinBlock(nn.Module):
    def __init__(self, dim: int, heads: int, resolution: int, window: int = 7, shift: int = 0, mlp_ratio: float = 4.0):
        super().__init__()
        self.resolution, self.window = resolution, min(window, resolution)
        self.shift = 0 if resolution <= window else shift
        self.norm1 = nn.LayerNorm(dim)
        self.attn = SwinWindowAttention(dim, heads, (self.window, self.window))
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = _Mlp(dim, int(dim * mlp_ratio))
        mask = None
        if self.shift > 0:
            img = torch.zeros(1, resolution, resolution, 1)
            cnt = 0
            for hs in (slice(0, -self.window), slice(-self.window, -self.shift), slice(-self.shift, None)):
                for ws in (slice(0, -self.window), slice(-self.window, -self.shift), slice(-self.shift, None)):
                    img[:, hs, ws, :] = cnt
                    cnt += 1
            mw = _window_partition(img, self.window).squeeze(-1)
            mask = mw[:, None, :] - mw[:, :, None]
            mask = mask.masked_fill(mask != 0, -100.0).masked_fill(mask == 0, 0.0)
        self.register_buffer("attn_mask", mask, persistent=False)

    def forward(self, x):
        b, length, c = x.shape
        r, w = self.resolution, self.window
        y = self.norm1(x).view(b, r, r, c)
        if self.shift:
            y = torch.roll(y, shifts=(-self.shift, -self.shift), dims=(1, 2))
        win = self.attn(_window_partition(y, w), mask=self.attn_mask)
        y = _window_reverse(win, w, r, r)
        if self.shift:
            y = torch.roll(y, shifts=(self.shift, self.shift), dims=(1, 2))
        x = x + y.reshape(b, length, c)
        return x + self.mlp(self.norm2(x))


class PatchMerging(nn.Module):
    def __init__(self, dim: int, resolution: int):
        super().__init__()
        self.resolution = resolution
        self.norm = nn.LayerNorm(4 * dim)
        self.reduction = nn.Linear(4 * dim, 2 * dim, bias=False)

    def forward(self, x):
        b, _, c = x.shape
        r = self.resolution
        x = x.view(b, r // 2, 2, r // 2, 2, c).permute(0, 1, 3, 4, 2, 5).reshape(b, (r // 2) ** 2, 4 * c)
        return self.reduction(self.norm(x))


class SwinTransformer(nn.Module):
    """Swin-v1 classifier; defaults are Swin-T at 224 x 224 (56 x 56 tokens in stage 1 = 64 windows per image)."""

    def __init__(self, *, img_size: int = 224, patch: int = 4, dim: int = 96, depths: Sequence[int] = (2, 2, 6, 2),
                 heads: Sequence[int] = (3, 6, 12, 24), window: int = 7, num_classes: int = 1000, in_chans: int = 3):
        super().__init__()
        self.patch_embed = nn.Conv2d(in_chans, dim, kernel_size=patch, stride=patch)
        self.embed_norm = nn.LayerNorm(dim)
        res = img_size // patch
        layers: List[nn.Module] = []
        for si, (depth, nh) in enumerate(zip(depths, heads)):
            if si > 0:
                layers.append(PatchMerging(dim, res))
                dim, res = dim * 2, res // 2
            for bi in range(depth):
                layers.append(SwinBlock(dim, nh, res, window=window, shift=0 if bi % 2 == 0 else window // 2))
        self.layers = nn.ModuleList(layers)
        self.norm = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, num_classes)
        _init_weights(self)

    def forward(self, img):
        x = self.embed_norm(self.patch_embed(img).flatten(2).transpose(1, 2))
        for layer in self.layers:
            x = layer(x)
        return self.head(self.norm(x).mean(dim=1))


def swin_tiny(img_size: int = 224, num_classes: int = 1000) -> SwinTransformer:
    return SwinTransformer(img_size=img_size, num_classes=num_classes)


# ---- data-parallel gradient exchange ----------------------------------------------------------------------
class BucketedGradientAllReduce:
    """Averages parameter gradients over the ranks of `group` in buckets, overlapped with the backward pass.

    Parameters are taken in reverse registration order (roughly the order in which their gradients become ready)
    and packed into buckets of about `bucket_bytes`; a hook on each parameter counts arrivals, and when a bucket is
    complete its gradients are flattened and an asynchronous all_reduce(SUM) is issued at once, while autograd goes
    on with earlier layers.  `finish()` waits for the outstanding collectives, divides by the world size and writes
    the averages back into `.grad`.  Works with any torch.distributed backend (NCCL on GPUs, gloo among CPU ranks).
    """

    def __init__(self, module: nn.Module, *, bucket_bytes: int = 4 << 20, group=None):
        import torch.distributed as dist
        self._dist, self.group = dist, group
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        params = [p for p in module.parameters() if p.requires_grad]
        self.buckets: List[List[torch.nn.Parameter]] = []
        cur, size = [], 0
        for p in reversed(params):
            cur.append(p)
            size += p.numel() * p.element_size()
            if size >= bucket_bytes:
                self.buckets.append(cur)
                cur, size = [], 0
        if cur:
            self.buckets.append(cur)
        self._bucket_of = {id(p): bi for bi, b in enumerate(self.buckets) for p in b}
        self._pending = [0] * len(self.buckets)
        self._inflight = []
        self._handles = [p.register_post_accumulate_grad_hook(self._on_grad) for p in params] if self.world > 1 else []
        self.reset()

    def reset(self) -> None:
        self._pending = [len(b) for b in self.buckets]
        self._inflight = []

    def _on_grad(self, p) -> None:
        bi = self._bucket_of[id(p)]
        self._pending[bi] -= 1
        if self._pending[bi] == 0:
            bucket = [q for q in self.buckets[bi] if q.grad is not None]
            flat = torch.cat([q.grad.reshape(-1).float() for q in bucket])
            work = self._dist.all_reduce(flat, op=self._dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._inflight.append((work, flat, bucket))

    def finish(self) -> None:
        """Call after backward(): completes the exchange; afterwards every rank holds the averaged gradients."""
        if self.world > 1:
            # parameters that received no gradient in this step leave their bucket incomplete: flush those now
            for bi, left in enumerate(self._pending):
                if left > 0:
                    bucket = [q for q in self.buckets[bi] if q.grad is not None]
                    if bucket:
                        flat = torch.cat([q.grad.reshape(-1).float() for q in bucket])
                        work = self._dist.all_reduce(flat, op=self._dist.ReduceOp.SUM, group=self.group, async_op=True)
                        self._inflight.append((work, flat, bucket))
            for work, flat, bucket in self._inflight:
                work.wait()
                flat.div_(self.world)
                off = 0
                for q in bucket:
                    n = q.numel()
                    q.grad.copy_(flat[off:off + n].view_as(q.grad))
                    off += n
        self.reset()

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []
