"""elsa_b200: B200-native two-pass monoid attention behind the reference's PyTorch API.

Public names match `elsa_twopass_clean.__all__` of the reference for the attention operator and
its drop-in hooks (src/elsa_twopass_clean/__init__.py:8-21).
"""
from .attention import twopass_attention
from .attention_bwd import twopass_attention_backward, twopass_attention_train, twopass_attention_with_state
from .timm_dropin import PatchReport, patch_timm_attention
from .timm_dropin_bwd import TrainPatchReport, patch_timm_attention_train

__all__ = [
    "PatchReport",
    "TrainPatchReport",
    "patch_timm_attention",
    "patch_timm_attention_train",
    "twopass_attention",
    "twopass_attention_backward",
    "twopass_attention_train",
    "twopass_attention_with_state",
]
