from .chunk import chunk_kda, check_status  # noqa: F401
from .decode import fused_sigmoid_gating_delta_rule_update, kda_decode  # noqa: F401
from .gate import fused_beta_sigmoid, fused_kda_gate  # noqa: F401
from .host import bind_host_to_gpu, chunk_kda_host  # noqa: F401
from .layer_ops import rms_norm_gated, short_conv  # noqa: F401

__all__ = ["chunk_kda", "chunk_kda_host", "check_status", "kda_decode", "fused_sigmoid_gating_delta_rule_update",
           "fused_kda_gate", "fused_beta_sigmoid", "bind_host_to_gpu", "short_conv", "rms_norm_gated"]
