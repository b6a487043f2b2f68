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


def _check_list(seq_pages, group, items):
    assert len(items) % group == 0
    seen = {}
    for c in range(0, len(items), group):
        run = items[c:c + group]
        splits = {(i >> 24) & 0x7F for i in run if i >= 0}
        if group in splits and group > 1:  # the splits of one sequence, in order, and nothing else
            assert splits == {group} and len({i & 0xFFFF for i in run}) == 1
            assert [(i >> 16) & 0xFF for i in run] == list(range(group))
        else:
            assert splits <= {1}
        for i in run:
            if i >= 0:
                seen.setdefault(i & 0xFFFF, []).append((i >> 16) & 0xFF)
    assert sorted(seen) == list(range(len(seq_pages)))  # every sequence, once or once per split
    assert all(z == [0] or z == list(range(group)) for z in seen.values())
    return seen


def test_work_lists_for_unequal_lengths():
    from bitnet_c_b200.csrc.ops import decode_items
    # even lengths, few blocks, or too many blocks: the plain grid
    assert decode_items([9] * 64, 8) is None
    assert decode_items([40, 3, 3], 8) is None
    assert decode_items(list(range(3, 67)), 8) is None
    # 8 sequences of 40 heads: the two long ones are split in two and come first
    pages = [9, 40, 16, 12, 10, 24, 9, 9]
    group, items = decode_items(pages, 40)
    seen = _check_list(pages, group, items)
    assert group == 2 and seen[1] == [0, 1] and seen[5] == [0, 1] and seen[0] == [0]
    assert [i & 0xFFFF for i in items[:4]] == [1, 1, 5, 5]
    # a recorded step keeps its grid: the list for a given group is padded to the capacity, and
    # splits nothing once the batch is even
    group, items = decode_items(pages, 40, group=2, capacity=16)
    assert len(items) == 16 and items.count(-1) == 6
    _check_list(pages, 2, items)
    group, items = decode_items([30] * 8, 40, group=2, capacity=16)
    assert all(z == [0] for z in _check_list([30] * 8, 2, items).values())
    for g in (1, 2, 3, 4):
        _check_list(pages, g, decode_items(pages, 40, group=g, capacity=g * 8)[1])
