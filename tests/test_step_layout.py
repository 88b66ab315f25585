"""The step function's metadata buffer, laid out on the host (no GPU): segments, block tables, and the arrays
that a mixer's planner adds without the step function knowing what they mean."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from fakes import fake_blocks
from sharpinference_b200.cache import CacheManager
from sharpinference_b200.engine.step import StepEntry, StepError, StepRunner
from sharpinference_b200.models.model import ScheduleEntry
from sharpinference_b200.parts.attention import PagedAttentionPlanner
from sharpinference_b200.parts.base import CacheSpec, StepPlanData, StepPlanner


class ScanPlanner(StepPlanner):
    """A toy planner: per request (first row, rows), and the longest entry as a host value."""
    key = "scan"

    def plan(self, starts, lengths, bucket=None):
        first = np.cumsum([0] + list(lengths[:-1]))
        return StepPlanData(arrays={"segments": np.stack([first, lengths], axis=1)}, values={"longest": max(lengths)})


def runner_with(planners):
    specs = [CacheSpec("chunk", 8, 1, 8), CacheSpec("full", 0, 1, 8)]
    blocks = fake_blocks(specs)
    for b, p in zip(blocks, planners):
        b.mixer.step_planner = (lambda page_size, p=p: p)
    cache = CacheManager([ScheduleEntry(0), ScheduleEntry(1)], blocks, page_size=4, num_pages=16, max_requests=4,
                         dtype=torch.float32, device="cpu", allocate=False)
    model = SimpleNamespace(vocab_size=100, blocks=blocks)
    return StepRunner(model, cache), cache


def test_layout_holds_every_segment_on_16_bytes_and_the_planners_arrays():
    runner, cache = runner_with([PagedAttentionPlanner(8), ScanPlanner()])
    assert list(runner.planners) == [("paged_attention", 8), "scan"]
    for rid, n in (("a", 9), ("b", 0), ("c", 3)):
        cache.add_request(rid)
        if n:
            cache.reserve([(rid, n)])
            cache.commit(rid, n)
    entries = [StepEntry("a", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11], [0, 10]), StepEntry("b", [5], [0]), StepEntry("c", [7, 8], [])]
    cache.reserve([(e.request_id, len(e.tokens)) for e in entries])
    hs = runner.lay_out(entries)
    assert all(o % 4 == 0 for o, _ in hs.segments.values())

    def seg(name):
        o, shape = hs.segments[name]
        return hs.words[o:o + int(np.prod(shape))].reshape(shape)

    assert seg("token_ids").tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 5, 7, 8]
    assert seg("positions").tolist() == list(range(9, 20)) + [0] + [3, 4]
    assert seg("row_request").tolist() == [0] * 11 + [1] + [2, 2]
    assert seg("request_start").tolist() == [9, 0, 3] and seg("row_offsets").tolist() == [0, 11, 12, 14]
    assert seg("want_rows").tolist() == [0, 10, 11]
    for g in cache.groups:
        table = seg(("table", g.index))
        assert table.shape == (3, 5)
        for b, rid in enumerate("abc"):
            t = cache.requests[rid].tables[g.index]
            assert table[b].tolist() == t + [-1] * (5 - len(t))
    assert seg(("plan", ("paged_attention", 8), "tiles")).tolist() == [[0, 8, 9, 0], [8, 3, 17, 0]]
    assert seg(("plan", ("paged_attention", 8), "decode_rows")).tolist() == [11, 12, 13]
    assert seg(("plan", "scan", "segments")).tolist() == [[0, 11], [11, 1], [12, 2]]
    assert hs.plan_values["scan"] == {"longest": 11}
    ctx = runner.build_context(entries, host_step=hs)
    assert ctx.plans["scan"].segments.tolist() == [[0, 11], [11, 1], [12, 2]] and ctx.plans["scan"].longest == 11
    assert ctx.plans[("paged_attention", 8)].num_tiles == 2 and ctx.max_context == 20 and not ctx.decode_only
    assert ctx.block_tables[0].shape == (3, 5) and ctx.want_rows.tolist() == [0, 10, 11]


def test_a_fixed_width_narrower_than_the_tables_is_refused():
    runner, cache = runner_with([None, None])
    cache.add_request("a")
    cache.reserve([("a", 30)])
    with pytest.raises(StepError, match="columns"):
        runner.lay_out([StepEntry("a", list(range(30)), [])], width=4)
    assert runner.planners == {}
