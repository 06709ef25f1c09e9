from .chunk import chunk_gated_delta_rule  # noqa: F401

__all__ = ["chunk_gated_delta_rule"]
