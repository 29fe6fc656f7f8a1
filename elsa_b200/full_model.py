"""Toy pre-norm Transformer encoder with a switchable attention backend, for A/B studies of the operator inside a
whole model.  Mirrors the helper pair of the reference (src/elsa_twopass_clean/full_model.py:40-191 for inference,
full_model_bwd.py:48-205 for training): `make_model_pair` / `make_train_model_pair` return (baseline, elsa) encoders
with identical weights, the baseline running PyTorch SDPA, the other this package's `twopass_attention`
(`twopass_attention_train` in the trainable flavour).  One implementation serves both flavours here.
"""
from __future__ import annotations

from typing import Literal, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .attention import twopass_attention
from .attention_bwd import twopass_attention_train

AttentionBackend = Literal["elsa", "sdpa"]
SdpaKind = Literal["auto", "math", "flash", "mem_efficient"]


def _sdpa(q, k, v, *, is_causal: bool, kind: SdpaKind):
    """PyTorch scaled-dot-product attention, optionally pinned to one of its back-ends."""
    if kind == "auto":
        return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal)
    from torch.nn.attention import SDPBackend, sdpa_kernel
    backend = {"math": SDPBackend.MATH, "flash": SDPBackend.FLASH_ATTENTION,
               "mem_efficient": SDPBackend.EFFICIENT_ATTENTION}.get(kind)
    if backend is None:
        raise ValueError(f"unknown sdpa kind: {kind}")
    with sdpa_kernel(backend):
        return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal)


class SelfAttention(nn.Module):
    def __init__(self, dim: int, heads: int, *, backend: AttentionBackend, sdpa_kind: SdpaKind = "auto",
                 is_causal: bool = False, qkv_bias: bool = True, elsa_kwargs: Optional[dict] = None,
                 trainable: bool = False) -> None:
        super().__init__()
        if dim % heads != 0:
            raise ValueError("dim must be divisible by heads")
        self.dim, self.heads, self.head_dim = int(dim), int(heads), int(dim) // int(heads)
        self.backend, self.sdpa_kind, self.is_causal = backend, sdpa_kind, bool(is_causal)
        self.elsa_kwargs = dict(elsa_kwargs or {})
        self.trainable = bool(trainable)
        self.qkv = nn.Linear(dim, 3 * dim, bias=qkv_bias)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        batch, seq_len, channels = x.shape
        q, k, v = self.qkv(x).view(batch, seq_len, 3, self.heads, self.head_dim).permute(2, 0, 3, 1, 4).unbind(0)
        if self.backend == "elsa":
            op = twopass_attention_train if self.trainable else twopass_attention
            y = op(q, k, v, is_causal=self.is_causal, algorithm="paper_scan", **self.elsa_kwargs)
        elif self.backend == "sdpa":
            y = _sdpa(q, k, v, is_causal=self.is_causal, kind=self.sdpa_kind)
        else:
            raise ValueError(f"unknown attention backend: {self.backend}")
        return self.proj(y.transpose(1, 2).reshape(batch, seq_len, channels))


class MLP(nn.Module):
    def __init__(self, dim: int, hidden_dim: int) -> None:
        super().__init__()
        self.fc1 = nn.Linear(dim, hidden_dim)
        self.fc2 = nn.Linear(hidden_dim, dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(F.gelu(self.fc1(x)))


class TransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, *, mlp_ratio: float = 4.0, **attn_kwargs) -> None:
        super().__init__()
        self.norm1 = nn.LayerNorm(dim)
        self.attn = SelfAttention(dim, heads, **attn_kwargs)
        self.norm2 = nn.LayerNorm(dim)
        self.mlp = MLP(dim, int(dim * mlp_ratio))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


class TransformerEncoder(nn.Module):
    """Minimal encoder: `depth` pre-norm blocks and a final LayerNorm."""

    def __init__(self, *, dim: int = 192, depth: int = 1, heads: int = 3, mlp_ratio: float = 4.0,
                 backend: AttentionBackend, sdpa_kind: SdpaKind = "auto", is_causal: bool = False,
                 elsa_kwargs: Optional[dict] = None, trainable: bool = False) -> None:
        super().__init__()
        self.blocks = nn.ModuleList([
            TransformerBlock(dim, heads, mlp_ratio=mlp_ratio, backend=backend, sdpa_kind=sdpa_kind, is_causal=is_causal,
                             elsa_kwargs=elsa_kwargs, trainable=trainable) for _ in range(depth)])
        self.norm = nn.LayerNorm(dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for block in self.blocks:
            x = block(x)
        return self.norm(x)


def _pair(trainable: bool, *, dim, depth, heads, mlp_ratio, sdpa_kind, is_causal, elsa_kwargs):
    common = dict(dim=dim, depth=depth, heads=heads, mlp_ratio=mlp_ratio, is_causal=is_causal, trainable=trainable)
    baseline = TransformerEncoder(backend="sdpa", sdpa_kind=sdpa_kind, **common)
    elsa = TransformerEncoder(backend="elsa", elsa_kwargs=elsa_kwargs, **common)
    elsa.load_state_dict(baseline.state_dict())
    return baseline, elsa


def make_model_pair(*, dim: int = 192, depth: int = 1, heads: int = 3, mlp_ratio: float = 4.0,
                    sdpa_kind: SdpaKind = "auto", is_causal: bool = False, elsa_kwargs: Optional[dict] = None):
    """(baseline, elsa) inference encoders with the same weights (reference: full_model.py:162-191)."""
    return _pair(False, dim=dim, depth=depth, heads=heads, mlp_ratio=mlp_ratio, sdpa_kind=sdpa_kind,
                 is_causal=is_causal, elsa_kwargs=elsa_kwargs)


def make_train_model_pair(*, dim: int = 192, depth: int = 1, heads: int = 3, mlp_ratio: float = 4.0,
                          sdpa_kind: SdpaKind = "auto", is_causal: bool = False, elsa_kwargs: Optional[dict] = None):
    """(baseline, elsa) trainable encoders with the same weights (reference: full_model_bwd.py:176-205)."""
    return _pair(True, dim=dim, depth=depth, heads=heads, mlp_ratio=mlp_ratio, sdpa_kind=sdpa_kind,
                 is_causal=is_causal, elsa_kwargs=elsa_kwargs)
