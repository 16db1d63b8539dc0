"""``nitrix.nn``-shaped namespace: only the attention entry point is provided."""
from .attention import default_scale, qk_rms_norm, scaled_dot_product_attention

__all__ = ["scaled_dot_product_attention", "default_scale", "qk_rms_norm"]
