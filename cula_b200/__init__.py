"""B200-native Kimi Delta Attention (chunkwise) behind the ``chunk_kda`` interface of cuLA."""
__version__ = "0.1.0"
