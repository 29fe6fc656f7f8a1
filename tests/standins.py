"""Stand-ins for timm's ViT `Attention` and Swin-v1 `WindowAttention` (timm is not installed where these tests
run): the package's own timm-shaped attention modules, which expose exactly the attributes the drop-in detectors
look for (reference: src/elsa_twopass_clean/timm_dropin.py:153-172) and compute attention the plain way, so they
also serve as the numerical baseline of the drop-in tests."""
from elsa_b200.vision import SwinWindowAttention, VitAttention, relative_position_index  # noqa: F401
