"""Property tests (hypothesis) of host-side invariants: packing never loses or overlaps a token and the native code
agrees with its Python twin on arbitrary inputs; span sequentialisation and lane assignment never overlap; the two
loss reductions agree; the ATIF projection round-trips arbitrary steps."""
import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

from tunix_b200.experimental.trajectory import trajectory as T  # noqa: E402
from tunix_b200.perf.experimental import timeline, timeline_utils, trace_writer  # noqa: E402
from tunix_b200.rl import common, packing as P  # noqa: E402

_settings = settings(max_examples=40, deadline=None)


@st.composite
def _pack_items(draw):
    n = draw(st.integers(1, 24))
    items = []
    for i in range(n):
        p, c = draw(st.integers(1, 30)), draw(st.integers(1, 40))
        items.append(P.PackItem(prompt_ids=np.full(p, 1000 + i, np.int32), completion_ids=np.full(c, 2000 + i, np.int32),
                                completion_mask=np.ones(c, np.float32), advantages=np.full(c, float(i), np.float32)))
    return items


@_settings
@given(_pack_items(), st.integers(1, 5), st.sampled_from([1, 4, 8]), st.integers(1, 6))
def test_packing_places_every_token_once(items, rows, boundary, max_segments):
    budget = 96
    native = P.fill_one_chunk(items, rows, budget, max_segments, boundary)
    python = P.fill_one_chunk_py(items, rows, budget, max_segments, boundary)
    assert [sorted(b) for b in native[0]] == [sorted(b) for b in python[0]] and native[1] == python[1] and native[2] == python[2]
    bins, starts, leftover = native
    placed = [i for b in bins for i in b]
    assert sorted(placed + list(leftover)) == list(range(len(items)))             # every item is placed or left over, once
    assert all(len(b) <= max_segments for b in bins)
    if not placed:
        return
    bins = [b for b in bins if b]
    chunk = P.pack_chunk(items, bins, starts, budget, pad_id=-1)
    ref = P.pack_chunk_py(items, bins, starts, budget, pad_id=-1)
    for f in ("ids", "prompt_mask", "completion_mask", "advantages", "segment_ids", "segment_positions"):
        assert np.array_equal(getattr(chunk, f), getattr(ref, f)), f
    for r, members in enumerate(bins):
        row_ids, seg = chunk.ids[r], chunk.segment_ids[r]
        for k, i in enumerate(members):
            it = items[i]
            sel = seg == k + 1
            want = np.concatenate([it.prompt_ids, it.completion_ids])
            assert np.array_equal(row_ids[sel], want)                              # the segment is the item, contiguous and whole
            assert np.array_equal(chunk.segment_positions[r][sel], np.arange(len(want)))
            assert chunk.completion_mask[r][sel].sum() == len(it.completion_ids)
        assert (row_ids[seg == 0] == -1).all()                                     # everything else is padding


@st.composite
def _spans(draw):
    n = draw(st.integers(0, 20))
    out = {}
    for i in range(n):
        b = draw(st.floats(0, 100, allow_nan=False))
        d = draw(st.floats(0.001, 20, allow_nan=False))
        s = timeline.Span(name=f"s{i % 3}", begin=b, id=i)
        s.end = b + d
        out[i] = s
    return out


@_settings
@given(_spans())
def test_sequentialised_spans_never_overlap(spans):
    active, queue = timeline_utils.sequentialize_overlapping_spans(spans)
    for group in (active, queue):
        ordered = sorted(group.values(), key=lambda s: s.begin)
        assert all(a.end <= b.begin + 1e-9 for a, b in zip(ordered, ordered[1:]))
        assert all(s.begin < s.end for s in ordered)
    for sid, a in active.items():
        assert a.begin >= spans[sid].begin - 1e-9 and a.name == spans[sid].name       # work never starts before it was issued
        if sid in queue:
            assert abs(queue[sid].end - a.begin) < 1e-9                               # waiting ends where the work starts
    assert set(active) | set(queue) <= set(spans)            # a span that neither works nor waits on its own time is dropped
    if spans:
        first = min(spans.values(), key=lambda s: (s.begin, s.id))
        assert (active[first.id].begin, active[first.id].end) == (first.begin, first.end) and first.id not in queue
        assert max(a.end for a in active.values()) == pytest.approx(max(s.end for s in spans.values()))   # the timeline ends where it ended


@_settings
@given(_spans())
def test_lanes_hold_no_overlapping_spans(spans):
    lanes, n = trace_writer._assign_lanes(spans.values())
    assert set(lanes) == set(spans) and (n == 0) == (not spans)
    for lane in range(n):
        ordered = sorted((s for s in spans.values() if lanes[s.id] == lane), key=lambda s: s.begin)
        assert all(a.end <= b.begin for a, b in zip(ordered, ordered[1:]))
    if spans:                                                                          # greedy colouring of intervals is optimal
        events = sorted([(s.begin, 1) for s in spans.values()] + [(s.end, -1) for s in spans.values()], key=lambda e: (e[0], e[1]))
        depth = peak = 0
        for _, d in events:
            depth += d
            peak = max(peak, depth)
        assert n == peak


@_settings
@given(st.integers(1, 5), st.integers(1, 12), st.integers(0, 2 ** 16),
       st.sampled_from(["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale", "seq-mean-token-sum", "sequence-mean-token-sum-norm"]))
def test_the_two_loss_reductions_agree(B, Tn, seed, mode):
    g = torch.Generator().manual_seed(seed)
    L = torch.randn(B, Tn, generator=g)
    m = (torch.rand(B, Tn, generator=g) > 0.3).float()
    a = common.aggregate_loss(L, m, mode)
    got = a.sum / a.denominator.clamp(min=a.min_denominator or 1e-8)
    assert torch.allclose(got, common.reduced_loss_agg(L, m, mode).to(got.dtype), atol=1e-5, rtol=1e-5)


_text = st.text(st.characters(blacklist_categories=("Cs",)), max_size=20)


@_settings
@given(st.integers(0, 50), _text, st.lists(st.integers(0, 2 ** 31 - 1), max_size=12), st.one_of(st.none(), st.integers(0, 9)),
       st.one_of(st.none(), st.floats(-10, 10, allow_nan=False)), st.dictionaries(st.sampled_from(["a", "b", "c"]), st.integers(), max_size=3))
def test_atif_projection_round_trips_agent_steps(step_id, message, tokens, version, mc_return, extra):
    s = T.TunixAgentStep(step_id=step_id, source="agent", message=message, assistant_tokens=tokens, assistant_masks=[1] * len(tokens),
                         logprobs=[-0.5] * len(tokens), policy_version=version, mc_return=mc_return, extra=extra or None)
    atif = s.to_atif_step()
    assert type(atif) is T.Step and atif.step_id == step_id + 1 and atif.message == message
    assert atif.to_json() == s.to_atif_json()                                         # the writers' shortcut gives the same document
    back = T.TunixAgentStep.from_atif_step(T.Step.from_json(atif.to_json()))
    assert back.step_id == step_id and back.message == message and back.policy_version == version and back.mc_return == mc_return
    assert np.array_equal(back.assistant_tokens, np.asarray(tokens, np.int64)) and (back.extra or {}) == (extra or {})


@_settings
@given(st.integers(0, 3), st.integers(1, 4), st.lists(st.sampled_from(["dispatch", "consume", "filter"]), min_size=1, max_size=60))
def test_dispatch_window_never_runs_further_ahead_than_allowed(max_staleness, full, events):
    """Whatever the order of dispatches, consumed batches and filtered groups: a prompt of batch b is only let through
    while b <= next_batch + max_staleness, and a parked dispatcher is woken by the event that makes room."""
    import asyncio
    from tunix_b200.experimental.common.dispatch_window import DispatchWindow

    async def run():
        step = [0]
        w = DispatchWindow(max_staleness, lambda: step[0], full_batch_size=full, out_of_order_resume=True)
        dispatched = 0
        waiting = None
        for ev in events:
            if ev == "dispatch" and waiting is None:
                batch = dispatched // full
                waiting = asyncio.ensure_future(w.wait_for(batch))
                await asyncio.sleep(0)
            elif ev == "consume":
                step[0] += 1
                w.release()
            elif ev == "filter":
                w.on_group_filtered([{"prompt_id": f"f{dispatched}"}])
            await asyncio.sleep(0)
            await asyncio.sleep(0)
            if waiting is not None:
                batch = dispatched // full
                allowed = batch <= w.next_batch + max_staleness
                assert waiting.done() == allowed                  # through exactly when the window allows it
                if waiting.done():
                    dispatched += 1
                    waiting = None
        if waiting is not None:
            waiting.cancel()
    asyncio.run(run())
