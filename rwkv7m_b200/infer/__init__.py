from .generate import decode_one, generate, prefill, sample_next

__all__ = ["decode_one", "generate", "prefill", "sample_next"]
