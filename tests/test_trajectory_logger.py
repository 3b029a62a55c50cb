"""Native trajectory serialiser against json.dumps / repr, and the async logger."""
import dataclasses
import json
import math

import numpy as np
import pytest

from tunix_b200.utils import trajectory_logger as T


@pytest.mark.parametrize("dtype", [np.int8, np.int32, np.int64, np.uint8, np.uint64, np.float32, np.float64, np.bool_])
def test_format_ndarray_matches_repr(dtype):
    rng = np.random.default_rng(0)
    a = (rng.normal(size=(3, 4, 2)) * 1000).astype(dtype)
    assert str(T.format_ndarray(a)) == repr(a.tolist())
    assert str(T.format_ndarray(a[:, ::2])) == repr(a[:, ::2].tolist())       # strided view
    assert str(T.format_ndarray(a[:0])) == repr(a[:0].tolist())                # zero extent


def test_float_repr_edge_cases():
    vals = np.array([0.0, -0.0, 1.0, 1e16, 1e15, 123456789012345678.0, 1e-4, 1e-5, 0.1, 1 / 3, 5e-324, 1.7976931348623157e308,
                     float("inf"), float("-inf"), float("nan"), 2.5e-7, 1e22, 1.5e300])
    assert str(T.format_ndarray(vals)) == repr(vals.tolist())


@dataclasses.dataclass
class Step:
    action: str
    reward: float
    tokens: np.ndarray


def test_dumps_json_matches_json_dumps():
    obj = {"s": "quote\" back\\ nl\n tab\t uni é \U0001F600 \x01", "i": 12345678901234567890, "f": [1.5, float("nan"), float("inf"), -1e-9],
           "n": None, "b": [True, False], 3: "intkey", "nested": {"t": (1, 2, (3,))}, "np": np.float32(0.25), "npi": np.int64(7)}
    assert T.dumps_json(obj) == json.dumps(T._to_jsonable(obj))
    st = Step("go", 1.5, np.arange(3, dtype=np.int32))
    assert json.loads(T.dumps_json(st)) == {"action": "go", "reward": 1.5, "tokens": [0, 1, 2]}
    assert T.dumps_json({"a": [1, {"b": 2}]}, indent=2) == json.dumps({"a": [1, {"b": 2}]}, indent=2)
    assert T.dumps_json({"arr": T.format_ndarray(np.array([1, 2]))}) == '{"arr": [1, 2]}'


def test_python_fallback_agrees():
    obj = {"a": np.arange(6).reshape(2, 3), "b": [1.0, 2.0]}
    assert json.loads(T.dumps_json(obj)) == json.loads(T.dumps_json_py(obj))


def test_async_logger_jsonl(tmp_path):
    with T.AsyncTrajectoryLogger(str(tmp_path), "jsonl") as lg:
        for i in range(50):
            lg.log({"i": i, "x": np.full(4, i, np.float32)})
        assert lg.flush(10)
    lines = open(tmp_path / "trajectories.jsonl").read().strip().split("\n")
    assert len(lines) == 50
    assert sorted(json.loads(l)["i"] for l in lines) == list(range(50))


def test_csv_logger(tmp_path):
    p = str(tmp_path / "t.csv")
    T.log_item(p, {"a": 1, "arr": np.array([1, 2])}, "csv")
    T.log_item(p, {"a": 2, "arr": np.array([3, 4])}, "csv")
    rows = open(p).read().strip().split("\n")
    assert rows[0] == "a,arr" and rows[1] == '1,"[1, 2]"'


def test_native_serializer_under_address_and_undefined_behaviour_sanitizers():
    """`_trajjson` rebuilt with -fsanitize=address,undefined; this file's tests run against it in a child process
    with the sanitizer run-time preloaded."""
    import os
    import subprocess
    import sys
    import pytest
    from tunix_b200 import _build
    try:
        _, asan = _build.sanitizer_toolchain()
        lib = _build.build_pyext_sanitized()
    except RuntimeError as e:
        pytest.skip(str(e))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1",
               TUNIX_B200_TRAJJSON_LIB=str(lib))
    who = subprocess.run([sys.executable, "-c", "from tunix_b200.utils import trajectory_logger as t; print(t._trajjson.__file__)"],
                         env=env, cwd=root, capture_output=True, text=True, timeout=300)
    assert who.returncode == 0 and who.stdout.strip() == str(lib), who.stdout + who.stderr[-2000:]
    run = subprocess.run([sys.executable, "-m", "pytest", "tests/test_trajectory_logger.py", "-x", "-q", "-p", "no:cacheprovider",
                          "-k", "not sanitizers"], env=env, cwd=root, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-3000:]
    assert " passed" in run.stdout and "failed" not in run.stdout
