from .reference import reference_attn, repeat_kv

__all__ = ["reference_attn", "repeat_kv"]
