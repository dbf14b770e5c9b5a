"""Property tests (hypothesis): tokenizer matchers agree on arbitrary input, the native gather equals slicing, the
magic-prime sampler is a permutation that ranks split without overlap, and the chunk planner of the batch layout."""

import numpy as np
import pytest
from hypothesis import assume, given, settings, strategies as st

from rwkv7m_b200.tokenizer import RWKVTokenizer
from rwkv7m_b200.utils import host_runtime as H


@pytest.fixture(scope="module")
def tokenizers():
    H.build_host_runtime()
    return RWKVTokenizer(native=True), RWKVTokenizer(native=False)


@settings(max_examples=60, deadline=None)
@given(data=st.binary(max_size=300))
def test_matchers_agree_on_arbitrary_bytes_and_round_trip(tokenizers, data):
    native, plain = tokenizers
    ids = native.encode_bytes(data)
    assert ids == plain.encode_bytes(data)
    assert native.decode_bytes(ids) == data                   # every byte value is in the vocabulary
    assert all(0 < i < native.vocab_size for i in ids)        # id 0 is reserved for the end-of-text marker


@settings(max_examples=40, deadline=None)
@given(texts=st.lists(st.text(max_size=80), max_size=12), threads=st.integers(0, 4))
def test_batch_encoding_equals_one_by_one(tokenizers, texts, threads):
    native, plain = tokenizers
    assert native.encode_batch(texts, add_eos=True, threads=threads) == [plain.encode(t, add_eos=True) for t in texts]


@settings(max_examples=40, deadline=None)
@given(n=st.integers(40, 400), window=st.integers(2, 33), rows=st.integers(0, 9), seed=st.integers(0, 2 ** 16),
       threads=st.integers(0, 3))
def test_native_gather_equals_slicing(n, window, rows, seed, threads):
    H.build_host_runtime()
    rng = np.random.default_rng(seed)
    stream = rng.integers(0, 60000, size=n).astype(np.uint16)
    offsets = rng.integers(0, n - window + 1, size=rows)
    inputs = np.empty((rows, window - 1), dtype=np.int32)
    targets = np.empty((rows, window - 1), dtype=np.int32)
    H.gather_rows(stream, offsets, window, inputs, targets, threads=threads)
    for r, o in enumerate(offsets):
        assert np.array_equal(inputs[r], stream[o:o + window - 1]) and np.array_equal(targets[r], stream[o + 1:o + window])


@settings(max_examples=25, deadline=None)
@given(ctx=st.integers(2, 9), slots=st.integers(12, 120), world=st.sampled_from([1, 2, 4]))
def test_magic_sampler_is_a_permutation_split_across_ranks(tmp_path_factory, ctx, slots, world):
    """Over one epoch of ``p`` samples the cubic-residue rule visits ``p`` distinct windows (cubing is a bijection modulo a
    prime that is 2 mod 3), every window lies inside the stream, and the ranks of a world take disjoint samples."""
    from rwkv7m_b200.data import MMapIndexedDatasetBuilder, create_binidx_dataset, find_magic_prime

    assume(find_magic_prime(slots * ctx + 1, ctx) / slots > 0.9)    # the sampler refuses a prime that skips a tenth of the data
    d = tmp_path_factory.mktemp("magic")
    prefix = str(d / "stream")
    builder = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=np.uint16)
    builder.add_item(np.arange(slots * ctx + 1, dtype=np.uint16) % 50000)
    builder.end_document()
    builder.finalize(prefix + ".idx")
    seen = []
    for rank in range(world):
        ds = create_binidx_dataset(prefix, ctx_len=ctx, batch_size=1, rank=rank, world_size=world)
        p = ds.magic_prime
        assert p % 3 == 2 and p <= slots
        per_rank = p // world
        offs = ds.offsets(np.arange(per_rank))
        assert offs.min() >= 0 and offs.max() + ctx + 1 <= ds.data_size and np.all(offs % ctx == 0)
        seen.append(offs // ctx)
        ds.close()
    windows = np.concatenate(seen)
    assert len(set(windows.tolist())) == len(windows)          # no window twice within the epoch, within or across ranks


@settings(max_examples=60, deadline=None)
@given(per_device=st.integers(1, 6), processes=st.sampled_from([1, 2, 4, 8]), devices=st.sampled_from([1, 2]))
def test_batch_layout_divides_the_global_batch(per_device, processes, devices):
    from rwkv7m_b200.parallel import compute_batch_layout

    global_batch = per_device * processes * devices
    layout = compute_batch_layout(global_batch, process_count=processes, local_device_count=devices)
    assert layout.process_batch_size * processes == global_batch
    assert layout.per_device_batch_size == per_device
    with pytest.raises(ValueError):
        compute_batch_layout(2 * global_batch + 1, process_count=2, local_device_count=devices)      # odd over two
