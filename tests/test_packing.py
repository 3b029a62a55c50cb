"""Native (C++) packing against its Python twin."""
import numpy as np
import pytest

from tunix_b200.rl import packing as P


def _items(n, seed=0, routed=False, fields=()):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        p, c = int(rng.integers(1, 40)), int(rng.integers(1, 60))
        kw = {}
        if routed:
            kw["routed_experts"] = rng.integers(0, 8, (p + c - 1, 2, 2)).astype(np.int16)
        out.append(P.PackItem(prompt_ids=rng.integers(0, 100, p).astype(np.int32),
                              completion_ids=rng.integers(0, 100, c).astype(np.int32),
                              completion_mask=np.ones(c, np.float32), advantages=rng.normal(size=c).astype(np.float32),
                              per_token={f: rng.normal(size=c).astype(np.float32) for f in fields}, **kw))
    return out


@pytest.mark.parametrize("boundary,max_segments", [(1, 1000), (8, 1000), (1, 2), (16, 3)])
def test_ffd_native_matches_python(boundary, max_segments):
    items = _items(64, seed=boundary)
    a = P.fill_one_chunk(items, 4, 128, max_segments, boundary)
    b = P.fill_one_chunk_py(items, 4, 128, max_segments, boundary)
    assert [sorted(x) for x in a[0]] == [sorted(x) for x in b[0]]
    assert a[1] == b[1]
    assert a[2] == b[2]


@pytest.mark.parametrize("routed", [False, True])
def test_fill_native_matches_python(routed):
    items = _items(40, seed=3, routed=routed, fields=("old_per_token_logps",))
    bins, starts, left = P.fill_one_chunk(items, 6, 160, 1000, 4)
    a = P.pack_chunk(items, bins, starts, 160, pad_id=-7)
    b = P.pack_chunk_py(items, bins, starts, 160, pad_id=-7)
    for f in ("ids", "prompt_mask", "completion_mask", "advantages", "segment_ids", "segment_positions"):
        assert np.array_equal(getattr(a, f), getattr(b, f)), f
    assert np.array_equal(a.per_token["old_per_token_logps"], b.per_token["old_per_token_logps"])
    assert a.num_real_segments == b.num_real_segments
    if routed:
        assert np.array_equal(a.routed_experts, b.routed_experts)
    # invariants: positions restart per segment, prompt and completion masks are disjoint
    assert ((a.prompt_mask > 0) & (a.completion_mask > 0)).sum() == 0
    row = a[0]
    assert row.segment_positions[0] == 0 and row.segment_ids[0] == 1


def test_pack_core_places_everything():
    items = _items(100, seed=9)
    chunks, left = P.pack_core(items, 4, 128, pad_id=0)
    assert left == []
    seen = sorted(i for ch in chunks for b in ch.bin_indices for i in b)
    assert seen == list(range(100))
    total = sum(int((ch.segment_ids > 0).sum()) for ch in chunks)
    assert total == sum(it.num_tokens for it in items)


def test_invalid_boundary():
    with pytest.raises(ValueError):
        P.fill_one_chunk(_items(3), 2, 64, 10, 0)


def test_router_replay_census():
    routed = np.full((1, 4, 2, 2), -1, np.int16)
    routed[0, 0, 0] = [1, 2]
    routed[0, 1, 0] = [3, 3]
    seg = np.array([[1, 1, 1, 0]], np.int32)
    assert P.count_router_replay_forced_tokens(routed, seg) == (3, 1)


def test_native_packing_under_address_and_undefined_behaviour_sanitizers():
    """The C++ host library is rebuilt with -fsanitize=address,undefined and this file's tests, plus the batch
    assemblers', run against it in a child process with the sanitizer run-time preloaded: an out-of-bounds write,
    a use after free or signed overflow in the packing code aborts the child."""
    import os
    import subprocess
    import sys
    import pytest
    from tunix_b200 import _build
    try:
        _, asan = _build.sanitizer_toolchain()
        lib = _build.build_host_sanitized()
    except RuntimeError as e:
        pytest.skip(str(e))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1",
               TUNIX_B200_HOST_LIB=str(lib))
    who = subprocess.run([sys.executable, "-c", "from tunix_b200 import _lib; print(_lib.host()._name)"], env=env, cwd=root,
                         capture_output=True, text=True, timeout=300)
    assert who.returncode == 0 and who.stdout.strip().endswith("libtunix_b200_host_asan.so"), who.stderr[-2000:]
    run = subprocess.run([sys.executable, "-m", "pytest", "tests/test_packing.py", "tests/test_experimental_cpu.py", "-x", "-q",
                          "-p", "no:cacheprovider", "-k", "not sanitizers and (packing or pack or batch_assemblers or ffd or fill)"],
                         env=env, cwd=root, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert " passed" in run.stdout and "failed" not in run.stdout
