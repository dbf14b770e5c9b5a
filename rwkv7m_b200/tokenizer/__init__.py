from .rwkv_tokenizer import RWKVTokenizer, Trie, default_vocab_path, tokenizer_metadata

__all__ = ["RWKVTokenizer", "Trie", "default_vocab_path", "tokenizer_metadata"]
