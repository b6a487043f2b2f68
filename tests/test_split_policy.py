"""The number of blocks that share a sequence in decode attention (a host decision, no device)."""
from bitnet_c_b200.csrc.ops import decode_splits


def test_bounds_hold_for_every_size():
    for pages in (1, 2, 3, 7, 8, 9, 16, 33, 64, 500):
        for blocks in (1, 3, 8, 32, 64, 96, 128, 255, 256, 257, 320, 4096):
            s = decode_splits(pages, blocks)
            assert 1 <= s <= min(32, pages)
            assert s == 1 or s * blocks <= 256


def test_few_sequences_split_and_many_do_not():
    kv_heads = 8
    assert decode_splits(16, 1 * kv_heads) in (6, 8)
    assert decode_splits(16, 4 * kv_heads) in (6, 8)
    assert decode_splits(16, 8 * kv_heads) == 4
    # the kernel shares a sequence's pages evenly, so two blocks pay at a thousand positions already
    assert decode_splits(16, 12 * kv_heads) == 2
    assert decode_splits(16, 16 * kv_heads) == 2
    # but never so many blocks that clusters come in two waves
    assert decode_splits(16, 24 * kv_heads) == 1
    assert decode_splits(32, 16 * kv_heads) == 2
    assert decode_splits(64, 8 * kv_heads) == 4
    assert decode_splits(64, 64 * kv_heads) == 1
    # one or two very long sequences: more blocks than a cluster holds
    assert decode_splits(1024, 1 * kv_heads) == 32
    assert decode_splits(1024, 2 * kv_heads) == 16
    assert decode_splits(128, 1 * kv_heads) == 8
    # a short bound never splits: the merge costs more than the walk
    assert decode_splits(4, 1) == 1
    assert decode_splits(8, 1) == 1
