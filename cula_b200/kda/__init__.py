from .chunk import chunk_kda, check_status  # noqa: F401

__all__ = ["chunk_kda", "check_status"]
