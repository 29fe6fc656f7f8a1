"""Training flavour of the timm drop-ins (reference: src/elsa_twopass_clean/timm_dropin_bwd.py).

Same module surgery as `timm_dropin`, but attention goes through `twopass_attention_train`, so the
patched model can be trained; attention dropout is rejected in training mode.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .timm_dropin import _SwinWindowAttentionBase, _VitAttentionBase, _patch


@dataclass(frozen=True)
class TrainPatchReport:
    vit_attention: int = 0
    swin_window_attention: int = 0

    @property
    def total(self) -> int:
        return self.vit_attention + self.swin_window_attention


class ElsaTrainTimmVitAttention(_VitAttentionBase):
    _training_op = True

    def _elsa_kwargs_for_seq(self, seq_len: int, dtype: torch.dtype) -> dict:
        """Per-length tile hints (reference table timm_dropin_bwd.py:40-61); advisory for the
        B200 kernels except block_n (partition width) and q_chunk_size."""
        kwargs = dict(self.elsa_kwargs)
        kwargs["algorithm"] = "paper_scan"
        half = dtype != torch.float32
        if half and seq_len >= 4096:
            kwargs.setdefault("bwd_block_m", 32)
            kwargs.setdefault("bwd_block_n", 32)
        kwargs.setdefault("block_m", 64 if half else 32)
        kwargs.setdefault("q_chunk_size", seq_len)
        for name, val in (("phase1_warps", 4), ("phase2_warps", 4), ("phase1_stages", 2), ("phase2_stages", 1)):
            kwargs.setdefault(name, val)
        return kwargs

    def _op_kwargs(self, seq_len: int, dtype: torch.dtype) -> dict:
        return self._elsa_kwargs_for_seq(seq_len, dtype)


class ElsaTrainTimmSwinWindowAttention(_SwinWindowAttentionBase):
    _training_op = True

    def _elsa_kwargs_for_window(self, seq_len: int) -> dict:
        kwargs = super()._elsa_kwargs_for_window(seq_len)
        for name, val in (("phase1_warps", 4), ("phase2_warps", 4), ("phase1_stages", 2), ("phase2_stages", 1)):
            kwargs.setdefault(name, val)
        return kwargs


def patch_timm_attention_train(model: nn.Module, *, elsa_kwargs: Optional[dict] = None) -> TrainPatchReport:
    """Replace every compatible attention module of `model` in place (autograd operator)."""
    vit, swin = _patch(model, ElsaTrainTimmVitAttention, ElsaTrainTimmSwinWindowAttention, elsa_kwargs)
    return TrainPatchReport(vit_attention=vit, swin_window_attention=swin)
