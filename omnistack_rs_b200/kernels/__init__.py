from .hadamard import rotate_queries, rotate_kv_cache

__all__ = ["rotate_queries", "rotate_kv_cache"]
