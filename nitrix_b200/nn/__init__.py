"""``nitrix.nn``-shaped namespace: the attention entry point and its siblings, LayerNorm and the selective scan."""
from .attention import default_scale, qk_rms_norm, scaled_dot_product_attention
from .norm import layer_norm
from .ssm import selective_scan

__all__ = ["scaled_dot_product_attention", "default_scale", "qk_rms_norm", "layer_norm", "selective_scan"]
