"""The runtime's choices of how to cut the work (K parts of a few-token product, key splits of decode
attention): what they may depend on, their bounds, and the cases that were measured."""
import pytest


def test_key_splits_depend_on_the_bucket_and_the_context_class_only():
    from odin_infer_b200.engine.runtime import context_class_of, decode_key_splits
    for n_seqs in (1, 2, 3, 4, 8, 12, 16, 24, 32, 64, 200, 256):
        for n_kv in (1, 2, 8):
            by_class = {}
            for longest in list(range(1, 1300, 37)) + [2048, 4000, 8192, 20000, 32768, 40000]:
                s = decode_key_splits(n_seqs, n_kv, longest)
                assert 1 <= s <= 16
                # never more CTAs than fit the GPU twice, unless one split already is
                assert s == 1 or n_seqs * n_kv * s <= 2 * 148
                cls = context_class_of(longest)
                assert by_class.setdefault(cls, s) == s, (n_seqs, n_kv, longest)


def test_key_splits_of_the_measured_cases():
    from odin_infer_b200.engine.runtime import decode_key_splits
    assert decode_key_splits(8, 8, 520) == 4       # 8 sequences of ~520 tokens: four splits were fastest
    assert decode_key_splits(4, 8, 520) == 4
    assert decode_key_splits(12, 8, 520) == 1      # from 12 sequences on: one
    assert decode_key_splits(16, 8, 520) == 1
    assert decode_key_splits(64, 8, 640) == 1
    assert decode_key_splits(4, 8, 32768) == 9     # long contexts: as many as fit the GPU twice
    assert decode_key_splits(1, 8, 32768) == 16
    assert decode_key_splits(3, 8, 100) == 1       # a page or two: nothing to split


def test_k_parts_fill_whole_rounds_and_never_depend_on_the_tokens():
    from odin_infer_b200.engine.runtime import choose_k_split
    # the 8B shape's decode products: q|k|v 48 tiles, o and down 32, gate|up 192; K blocks 64 or 192
    assert choose_k_split(48, 64, 8) == 3          # 144 CTAs
    assert choose_k_split(32, 64, 8) == 4          # 128
    assert choose_k_split(192, 64, 8) == 3         # 576 items, four rounds of 148
    assert choose_k_split(32, 192, 8) == 4
    for tiles in (1, 7, 32, 48, 100, 192, 1187):
        for kb in (1, 3, 16, 64, 192):
            for m in (1, 8, 16, 64, 128):
                s = choose_k_split(tiles, kb, m)
                assert 1 <= s <= 16 and s <= max(1, kb)
                per = (kb + s - 1) // s
                assert (kb + per - 1) // per == s, "an empty part"
