"""Native host runtime (C++ behind ctypes): the tokenizer's byte trie against the Python matcher, batch encoding, the data
loader's threaded gather against NumPy, and their use by the tokenizer, the batch dataset and the corpus converter."""

import json
import random

import numpy as np
import pytest
import torch

from rwkv7m_b200.tokenizer import RWKVTokenizer, Trie
from rwkv7m_b200.utils import host_runtime as H


@pytest.fixture(scope="module", autouse=True)
def _built():
    H.build_host_runtime()
    assert H.available()


def _texts(n=200, seed=0):
    rng = random.Random(seed)
    alphabet = ["hello", " world", "\n", "日本語", "の", "テキスト", " 1234567890", "ß", "🙂", "\t", "def f(x):", " return", "é", " "]
    return ["".join(rng.choice(alphabet) for _ in range(rng.randint(0, 40))) for _ in range(n)]


def test_native_trie_matches_the_python_matcher_on_the_shipped_vocabulary():
    native, plain = RWKVTokenizer(native=True), RWKVTokenizer(native=False)
    assert native._native is not None and plain._native is None
    assert native._native.max_token_len == max(len(t) for t in plain.token2idx) and native._native.node_count > 65536
    texts = _texts()
    for text in texts:
        ids = native.encode(text)
        assert ids == plain.encode(text)
        assert native.decode(ids) == text
    assert native.encode("", add_eos=True) == [0]
    batch = native.encode_batch(texts, add_eos=True, threads=3)
    assert batch == [plain.encode(t, add_eos=True) for t in texts]
    assert plain.encode_batch(texts[:5]) == [plain.encode(t) for t in texts[:5]]
    raw = bytes(range(256)) * 3                      # every byte value is a token of its own
    assert native.encode_bytes(raw) == plain.encode_bytes(raw) and native.decode_bytes(native.encode_bytes(raw)) == raw


def test_small_vocabulary_longest_match_and_uncovered_bytes(tmp_path):
    vocab = tmp_path / "vocab.txt"
    entries = [b"a", b"ab", b"abc", b"b", b"c", "あ".encode()]
    vocab.write_text("".join(f"{i + 1} {e!r} {len(e)}\n" for i, e in enumerate(entries)), encoding="utf-8")
    for native in (True, False):
        tok = RWKVTokenizer(vocab, native=native)
        assert tok.encode_bytes(b"abcabcb") == [3, 3, 4]
        assert tok.encode("cabあ") == [5, 2, 6]
        with pytest.raises(ValueError, match="offset 2"):
            tok.encode_bytes(b"abz")
    with pytest.raises(ValueError, match="not covered"):
        RWKVTokenizer(vocab, native=True).encode_batch([b"ab", b"zz"])
    trie = Trie()
    for i, e in enumerate(entries):
        trie.add(e, val=(e, i + 1))
    end, values = trie.find_longest(b"xabcab", 1)
    assert end == 4 and values == {(b"abc", 3)}
    assert trie.find_longest(b"ab", 1) == (2, {(b"b", 4)})
    with pytest.raises(ValueError):
        trie.find_longest(b"z", 0)


@pytest.mark.parametrize("dtype", [np.uint8, np.uint16, np.int32, np.uint32, np.int64])
def test_batch_gather_matches_numpy(dtype):
    rng = np.random.default_rng(1)
    hi = min(int(np.iinfo(dtype).max), 60000)
    stream = rng.integers(0, hi, size=5000).astype(dtype)
    window = 17
    offsets = rng.integers(0, stream.shape[0] - window, size=33)
    offsets[0], offsets[1] = 0, stream.shape[0] - window       # both ends of the stream
    for threads in (1, 4, 0):
        inputs = np.full((33, window - 1), -1, dtype=np.int32)
        targets = np.full((33, window - 1), -1, dtype=np.int32)
        H.gather_rows(stream, offsets, window, inputs, targets, threads=threads)
        rows = np.stack([stream[o:o + window] for o in offsets]).astype(np.int32)
        assert np.array_equal(inputs, rows[:, :-1]) and np.array_equal(targets, rows[:, 1:])
    with pytest.raises(IndexError):
        H.gather_rows(stream, np.array([stream.shape[0] - window + 1]), window, inputs[:1], targets[:1])
    with pytest.raises(IndexError):
        H.gather_rows(stream, np.array([-1]), window, inputs[:1], targets[:1])
    with pytest.raises(ValueError):
        H.gather_rows(stream, offsets, window, inputs.astype(np.int64), targets)
    with pytest.raises(ValueError):
        H.gather_rows(stream.astype(np.float32), offsets, window, inputs, targets)


def test_dataset_batches_are_the_same_with_and_without_the_native_gather(tiny_binidx, monkeypatch):
    from rwkv7m_b200.data import create_binidx_dataset

    for mode in ("magic", "sequential"):
        ds = create_binidx_dataset(tiny_binidx, ctx_len=4, batch_size=3, sampling_mode=mode)
        native = [ds.get_batch(s) for s in range(4)]
        monkeypatch.setattr(H, "available", lambda: False)
        plain = [ds.get_batch(s) for s in range(4)]
        monkeypatch.undo()
        for a, b in zip(native, plain):
            assert set(a) == set(b) == {"input_ids", "target_ids", "mask"}
            for key in a:
                assert a[key].dtype == b[key].dtype and torch.equal(a[key], b[key]), (mode, key)
        ds.close()


def test_corpus_converter_tokenises_once_and_keeps_the_document_order(tmp_path, monkeypatch):
    from rwkv7m_b200.cli import make_binidx
    from rwkv7m_b200.data import MMapIndexedDataset

    texts = [t for t in _texts(40, seed=3) if t]
    src = tmp_path / "rows.jsonl"
    src.write_text("".join(json.dumps({"text": t}, ensure_ascii=False) + "\n" for t in texts) + "\n", encoding="utf-8")
    stats = make_binidx.build_binidx(src, tmp_path / "native", epochs=2, seed=7, threads=2)
    assert stats["native_tokenizer"] and stats["items"] == 2 * len(texts)
    monkeypatch.setattr(H, "available", lambda: False)
    plain = make_binidx.build_binidx(src, tmp_path / "plain", epochs=2, seed=7)
    monkeypatch.undo()
    assert not plain["native_tokenizer"] and plain["tokens"] == stats["tokens"]
    a, b = MMapIndexedDataset(str(tmp_path / "native")), MMapIndexedDataset(str(tmp_path / "plain"))
    try:
        assert np.array_equal(a.get_global(0, a.data_size), b.get_global(0, b.data_size))
        # the order is that of shuffling the row list before every pass with the same generator
        tok = RWKVTokenizer(native=False)
        rows, rng, want = list(texts), random.Random(7), []
        for _ in range(2):
            rng.shuffle(rows)
            for t in rows:
                want += tok.encode(t, add_eos=True)
        assert a.get_global(0, a.data_size).tolist() == want
    finally:
        a.close()
        b.close()
    with pytest.raises(ValueError, match="does not fit"):
        make_binidx.build_binidx(src, tmp_path / "narrow", epochs=1, dtype="uint8")


def test_native_runtime_under_address_and_undefined_behaviour_sanitizers(tmp_path):
    """The C++ sources compiled with ``-fsanitize=address,undefined`` and driven by random inputs (tests/
    host_runtime_fuzz.cpp): no report, and the batch encoder agrees with the single-document one."""
    import shutil
    import subprocess
    from pathlib import Path

    compiler = shutil.which("g++") or shutil.which("c++")
    if compiler is None:
        pytest.skip("no C++ compiler")
    root = Path(__file__).resolve().parents[1]
    exe = tmp_path / "fuzz"
    build = subprocess.run([compiler, "-O1", "-g", "-std=c++17", "-fsanitize=address,undefined", "-fno-omit-frame-pointer",
                            "-pthread", str(root / "rwkv7m_b200" / "csrc" / "host_runtime.cpp"),
                            str(root / "tests" / "host_runtime_fuzz.cpp"), "-o", str(exe)], capture_output=True, text=True)
    if build.returncode != 0:
        pytest.skip("sanitizer runtime not available: " + build.stderr[-200:])
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0 and "fuzz ok" in run.stdout, (run.stdout + run.stderr)[-2000:]
    assert "runtime error" not in run.stderr and "AddressSanitizer" not in run.stderr
