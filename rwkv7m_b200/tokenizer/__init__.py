from .rwkv_tokenizer import RWKVTokenizer, default_vocab_path, tokenizer_metadata

__all__ = ["RWKVTokenizer", "default_vocab_path", "tokenizer_metadata"]
