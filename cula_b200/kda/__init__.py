from .chunk import chunk_kda, check_status  # noqa: F401
from .host import chunk_kda_host  # noqa: F401

__all__ = ["chunk_kda", "chunk_kda_host", "check_status"]
