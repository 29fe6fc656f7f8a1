"""Drop-in replacements for timm ViT `Attention` and Swin-v1 `WindowAttention` modules.

Same contract as the reference hooks (src/elsa_twopass_clean/timm_dropin.py:13-194 for inference,
timm_dropin_bwd.py:13-216 for training): modules are recognised by their attribute names only, the
wrapper deep-copies the linear / norm layers so parameter names and checkpoints keep working, the
Swin relative-position bias (plus the shifted-window mask) is passed as an additive bias, and a
non-canonical Swin scale is folded into q because the operator's scale is fixed at 1/sqrt(d).

Both flavours share one implementation here; `training=True` routes through the autograd operator.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn as nn

from .attention import twopass_attention
from .attention_bwd import twopass_attention_qkvpacked, twopass_attention_train

_VIT_ATTRS = ("qkv", "q_norm", "k_norm", "proj", "num_heads", "head_dim")
_SWIN_ATTRS = ("qkv", "proj", "relative_position_bias_table", "relative_position_index", "window_area",
               "window_size", "scale", "num_heads", "dim")


@dataclass(frozen=True)
class PatchReport:
    vit_attention: int = 0
    swin_window_attention: int = 0

    @property
    def total(self) -> int:
        return self.vit_attention + self.swin_window_attention


def _is_vit_attention(module: nn.Module) -> bool:
    # `norm` and `attn_dim` only exist in newer timm releases; they are optional here
    return all(hasattr(module, a) for a in _VIT_ATTRS)


def _is_swin_v1_window_attention(module: nn.Module) -> bool:
    # Swin-v2 (cosine attention, has `logit_scale`) is a different operator: leave it alone
    return all(hasattr(module, a) for a in _SWIN_ATTRS) and not hasattr(module, "logit_scale")


def _split_heads(qkv: torch.Tensor, tokens_shape, heads: int, head_dim: int):
    """[B, N, 3*H*d] -> three [B, H, N, d] views of the projection output."""
    b, n = tokens_shape
    return qkv.reshape(b, n, 3, heads, head_dim).permute(2, 0, 3, 1, 4).unbind(0)


class _VitAttentionBase(nn.Module):
    _training_op = False

    def __init__(self, source: nn.Module, *, elsa_kwargs: Optional[dict] = None) -> None:
        super().__init__()
        self.num_heads = int(source.num_heads)
        self.head_dim = int(source.head_dim)
        self.attn_dim = int(getattr(source, "attn_dim", self.num_heads * self.head_dim))
        for name in ("qkv", "q_norm", "k_norm", "proj", "proj_drop"):
            setattr(self, name, copy.deepcopy(getattr(source, name)))
        self.norm = copy.deepcopy(source.norm) if hasattr(source, "norm") else nn.Identity()
        if self._training_op:
            self.attn_drop = copy.deepcopy(source.attn_drop) if hasattr(source, "attn_drop") else nn.Dropout(0.0)
        self.elsa_kwargs = dict(elsa_kwargs or {})

    def _op_kwargs(self, seq_len: int, dtype: torch.dtype) -> dict:
        return dict(self.elsa_kwargs)

    def forward(self, x: torch.Tensor, attn_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if attn_mask is not None:
            raise ValueError("ELSA ViT drop-in currently supports unmasked attention only")
        if self._training_op and self.training and getattr(self.attn_drop, "p", 0.0):
            raise ValueError("ELSA ViT bwd drop-in does not implement attention dropout")
        batch, seq_len, _ = x.shape
        qkv = self.qkv(x)
        if isinstance(self.q_norm, nn.Identity) and isinstance(self.k_norm, nn.Identity):
            # q, k, v are read in place from the projection output and the result comes back in [B, N, H, d] memory:
            # no per-layer copies on either side of the operator (the reference makes one, timm_dropin.py:46-51)
            y = twopass_attention_qkvpacked(qkv.view(batch, seq_len, 3, self.num_heads, self.head_dim),
                                            train=self._training_op, **self._op_kwargs(seq_len, qkv.dtype))
        else:
            q, k, v = _split_heads(qkv, (batch, seq_len), self.num_heads, self.head_dim)
            q, k = self.q_norm(q), self.k_norm(k)
            op: Callable = twopass_attention_train if self._training_op else twopass_attention
            y = op(q, k, v, **self._op_kwargs(seq_len, q.dtype))
        y = y.transpose(1, 2).reshape(batch, seq_len, self.attn_dim)
        return self.proj_drop(self.proj(self.norm(y)))


class _SwinWindowAttentionBase(nn.Module):
    _training_op = False

    def __init__(self, source: nn.Module, *, elsa_kwargs: Optional[dict] = None) -> None:
        super().__init__()
        self.dim = int(source.dim)
        self.window_size = tuple(int(s) for s in source.window_size)
        self.window_area = int(source.window_area)
        self.num_heads = int(source.num_heads)
        for name in ("qkv", "attn_drop", "proj", "proj_drop", "softmax"):
            setattr(self, name, copy.deepcopy(getattr(source, name)))
        self.scale = float(source.scale)
        self.head_dim = int(self.qkv.out_features // (3 * self.num_heads))
        self.attn_dim = self.head_dim * self.num_heads
        self.relative_position_bias_table = nn.Parameter(source.relative_position_bias_table.detach().clone())
        self.register_buffer("relative_position_index", source.relative_position_index.detach().clone(),
                             persistent=False)
        self.elsa_kwargs = dict(elsa_kwargs or {})

    def _get_rel_pos_bias(self) -> torch.Tensor:
        """[(2w-1)^2, H] table gathered into a [1, H, N, N] additive bias."""
        area = self.window_area
        table = self.relative_position_bias_table[self.relative_position_index.reshape(-1)]
        return table.view(area, area, self.num_heads).permute(2, 0, 1).contiguous().unsqueeze(0)

    def set_window_size(self, window_size) -> None:
        from timm.models.swin_transformer import (get_relative_position_index, resize_rel_pos_bias_table,
                                                  to_2tuple)
        window_size = tuple(int(s) for s in to_2tuple(window_size))
        if window_size == self.window_size:
            return
        self.window_size = window_size
        win_h, win_w = window_size
        self.window_area = win_h * win_w
        with torch.no_grad():
            table = resize_rel_pos_bias_table(self.relative_position_bias_table, new_window_size=window_size,
                                              new_bias_shape=((2 * win_h - 1) * (2 * win_w - 1), self.num_heads))
            self.relative_position_bias_table = nn.Parameter(table)
            self.register_buffer("relative_position_index",
                                 get_relative_position_index(win_h, win_w, device=table.device), persistent=False)

    def _elsa_kwargs_for_window(self, seq_len: int) -> dict:
        kwargs = dict(self.elsa_kwargs)
        kwargs["algorithm"] = "paper_scan"
        kwargs.setdefault("block_m", 64)
        kwargs.setdefault("block_n", 64)
        kwargs.setdefault("q_chunk_size", seq_len)
        return kwargs

    def forward(self, x: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.training and self.attn_drop.p:
            raise ValueError("ELSA Swin drop-in does not implement attention dropout"
                             if self._training_op else
                             "ELSA Swin drop-in forward is inference-only when attention dropout is nonzero")
        windows, seq_len, _ = x.shape
        qkv = self.qkv(x)
        canonical = self.head_dim ** -0.5
        packed = abs(self.scale - canonical) <= 1e-12
        if not packed:
            q, k, v = _split_heads(qkv, (windows, seq_len), self.num_heads, self.head_dim)
            q = q * (self.scale / canonical)
        bias = self._get_rel_pos_bias()
        if mask is not None:
            # shifted windows: the [nW, N, N] 0/-100 mask repeats over the images of the batch
            n_win = int(mask.shape[0])
            tiled = mask.view(1, n_win, 1, seq_len, seq_len).expand(windows // n_win, -1, self.num_heads, -1, -1)
            bias = bias + tiled.reshape(-1, self.num_heads, seq_len, seq_len)
        if packed:
            y = twopass_attention_qkvpacked(qkv.view(windows, seq_len, 3, self.num_heads, self.head_dim), bias=bias,
                                            train=self._training_op, **self._elsa_kwargs_for_window(seq_len))
        else:
            op: Callable = twopass_attention_train if self._training_op else twopass_attention
            y = op(q, k, v, bias=bias, **self._elsa_kwargs_for_window(seq_len))
        y = y.transpose(1, 2).reshape(windows, seq_len, self.attn_dim)
        return self.proj_drop(self.proj(y))


class ElsaTimmVitAttention(_VitAttentionBase):
    """Inference ViT attention: qkv -> [B,H,N,d] -> twopass_attention -> proj."""


class ElsaTimmSwinWindowAttention(_SwinWindowAttentionBase):
    """Inference Swin-v1 window attention with the relative-position bias as an additive bias."""


def _patch(model: nn.Module, vit_cls, swin_cls, elsa_kwargs):
    counts = {"vit": 0, "swin": 0}

    def visit(parent: nn.Module) -> None:
        for name, child in list(parent.named_children()):
            if _is_vit_attention(child):
                setattr(parent, name, vit_cls(child, elsa_kwargs=elsa_kwargs))
                counts["vit"] += 1
            elif _is_swin_v1_window_attention(child):
                setattr(parent, name, swin_cls(child, elsa_kwargs=elsa_kwargs))
                counts["swin"] += 1
            else:
                visit(child)

    visit(model)
    if counts["vit"] + counts["swin"] == 0:
        raise ValueError("no compatible timm ViT or Swin v1 attention modules were patched")
    return counts["vit"], counts["swin"]


def patch_timm_attention(model: nn.Module, *, elsa_kwargs: Optional[dict] = None) -> PatchReport:
    """Replace every compatible attention module of `model` in place (inference operator)."""
    vit, swin = _patch(model, ElsaTimmVitAttention, ElsaTimmSwinWindowAttention, elsa_kwargs)
    return PatchReport(vit_attention=vit, swin_window_attention=swin)
