"""Host-side bounds that size kernel launches: they must never be below what the kernels will need (no GPU)."""
import random

from sharpinference_b200.kernels import ops


def visible_lo(pos: int, kind: int, span: int) -> int:
    """First visible key of a row at ``pos``: the mask rule of csrc/common.cuh, restated."""
    if kind == ops.MASK_CHUNK:
        return pos // span * span
    if kind == ops.MASK_WINDOW:
        return max(0, pos - span + 1)
    return 0


def splits_of(pos: int, kind: int, span: int) -> int:
    """The 256-key splits (at absolute multiples of 256) that hold a visible key of the row."""
    return pos // ops.DECODE_SPLIT - visible_lo(pos, kind, span) // ops.DECODE_SPLIT + 1


def test_decode_split_bounds_hold_for_drawn_rows():
    r = random.Random(0)
    for _ in range(2000):
        kind = r.choice([ops.MASK_FULL, ops.MASK_CHUNK, ops.MASK_WINDOW])
        span = r.choice([1, 16, 100, 256, 257, 300, 512, 8192, 70000])
        rows = r.randint(1, 70)
        top = r.choice([1, 5, 255, 256, 257, 1000, 8192, 8193, 140000])
        positions = [r.randrange(top) for _ in range(rows)]
        max_context = max(positions) + 1
        per_row = ops.decode_splits(max_context, kind, span)
        need = [splits_of(p, kind, span) for p in positions]
        assert max(need) <= per_row, (kind, span, positions)
        # what attention_decode launches when it is told the rows' keys: never fewer CTAs than there are splits
        keys = sum(p + 1 for p in positions)
        items = min(rows * per_row, keys // ops.DECODE_SPLIT + rows)
        assert sum(need) <= items, (kind, span, positions)


def test_decode_split_bound_is_tight_for_whole_chunks():
    assert ops.decode_splits(8192, ops.MASK_FULL, 1) == 32
    assert ops.decode_splits(8193, ops.MASK_FULL, 1) == 33
    assert ops.decode_splits(1, ops.MASK_FULL, 1) == 1
    # a chunk of 8192 keys that starts on a split boundary never spans more than 33 splits, however long the row
    assert ops.decode_splits(10 ** 6, ops.MASK_CHUNK, 8192) == 33
    assert ops.decode_splits(100, ops.MASK_WINDOW, 700) == 1


def test_attention_planner_cuts_tiles_and_single_rows():
    """Portions become tiles of the planner's size, short entries single rows; the plan of a decode-only step
    has no arrays at all, so a replayed graph has nothing of it to refresh."""
    from sharpinference_b200.parts.attention import PagedAttentionPlanner
    p = PagedAttentionPlanner(64)
    d = p.plan([100, 7, 0, 33], [150, 1, 4, 5])
    assert d.arrays["tiles"].tolist() == [[0, 64, 100, 0], [64, 64, 164, 0], [128, 22, 228, 0], [155, 5, 33, 3]]
    assert d.arrays["decode_rows"].tolist() == [150, 151, 152, 153, 154]
    assert d.values == {"num_tiles": 4, "num_decode_rows": 5, "tile_rows": 64, "decode_keys": 8 + (1 + 2 + 3 + 4)}
    d = p.plan([10, 20, 30], [1, 1, 1], bucket=p.bucket([10, 20, 30], [1, 1, 1]))
    assert d.arrays["tiles"].shape == (0, 4) and d.arrays["decode_rows"].size == 0
    assert d.values["num_decode_rows"] == 3 and d.values["decode_keys"] == p.keys_bucket(63, 3) >= 63
    assert PagedAttentionPlanner(128).key != p.key


def test_keys_bucket_of_a_captured_decode_step():
    """A replayed graph's attention launch is sized by the bucket: never below the keys, at most an eighth (or
    256 keys a row) above; a batch that gains a key a row each step changes bucket every 256 steps at most."""
    from sharpinference_b200.parts.attention import PagedAttentionPlanner as StepRunner    # the bucket is the planner's
    for rows in (1, 3, 8, 64):
        for keys in list(range(rows, 3000, 7)) + [65080, 65536, 65537, 10 ** 6, 2 ** 31 - 5]:
            b = StepRunner.keys_bucket(keys, rows)
            assert b >= keys
            assert b - keys < max(512 * rows, keys // 8 + 1), (keys, rows)
            assert StepRunner.keys_bucket(b, rows) == b                       # a bucket is its own bucket
        start = 5 * rows
        buckets = [StepRunner.keys_bucket(start + rows * step, rows) for step in range(4096)]
        changes = sum(a != b for a, b in zip(buckets, buckets[1:]))
        assert changes <= 4096 // 256 + 1, (rows, changes)
    assert len({StepRunner.keys_bucket(8 * (8192 - 57 + i), 8) for i in range(58)}) == 1
