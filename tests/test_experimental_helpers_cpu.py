"""Small helpers of the distributed stack: registries with discovery, prompt tagging, list summaries, wire checks,
unreduced metrics (test model: tunix/experimental/{rl/agentic/registry,common/*,metrics/*}_test.py)."""
import dataclasses
import sys
import textwrap

import numpy as np
import pytest
import torch

from tunix_b200.experimental.common import logging_utils, rpc_utils, tagging
from tunix_b200.experimental.metrics.metrics import MetricsBuffer, WeightedMetric
from tunix_b200.experimental.rl.agentic import registry as reg


def test_registry_decorator_forms():
    r = reg.Registry("T")

    @r.register("named")
    class A: ...

    @r.register()
    class B: ...

    @r.register
    class C: ...
    assert r.keys() == ["named", "B", "C"] and r.get("named") is A and "B" in r and not r.contains("A")
    with pytest.raises(KeyError, match="already registered in T for class 'B'"):
        r.register("B")(A)
    with pytest.raises(KeyError, match="Available keys"):
        r.get("missing")


def test_discovery_imports_only_decorated_modules(tmp_path):
    pkg = tmp_path / "userpkg_disc"
    pkg.mkdir()
    (pkg / "__init__.py").write_text("")
    (pkg / "agents.py").write_text(textwrap.dedent("""
        from tunix_b200.experimental.rl.agentic.registry import register_agent
        @register_agent("disc_agent")
        class MyAgent: ...
    """))
    (pkg / "envs.py").write_text(textwrap.dedent("""
        from tunix_b200.experimental.rl.agentic import registry as r
        @r.ENV_REGISTRY.register()
        class DiscEnv: ...
    """))
    (pkg / "heavy.py").write_text("raise RuntimeError('must not be imported')\n")
    (pkg / "own.py").write_text(textwrap.dedent("""
        from tunix_b200.experimental.rl.agentic.registry import Registry
        tools = Registry("tools")
        @tools.register
        class Tool: ...
    """))
    assert reg.has_registry_decorator(str(pkg / "agents.py")) and reg.has_registry_decorator(str(pkg / "envs.py"))
    assert reg.has_registry_decorator(str(pkg / "own.py")) and not reg.has_registry_decorator(str(pkg / "heavy.py"))
    assert not reg.has_registry_decorator(str(pkg / "missing.py"))
    got = reg.auto_discover_modules(str(pkg))
    assert sorted(got) == ["agents", "envs", "own"] and str(pkg) not in sys.path
    assert reg.AGENT_REGISTRY.get("disc_agent").__name__ == "MyAgent" and "DiscEnv" in reg.ENV_REGISTRY
    sys.path.insert(0, str(tmp_path))
    try:
        (pkg / "more.py").write_text("from tunix_b200.experimental.rl.agentic.registry import register_env\n@register_env('disc_env2')\nclass E: ...\n")
        assert "userpkg_disc.more" in reg.auto_discover_modules("userpkg_disc")
    finally:
        sys.path.remove(str(tmp_path))


def test_tagging_never_mutates():
    c = tagging.prompt_coordinates(5, 4)
    d = {"prompt_id": "a", "metadata": {"batch_idx": 99, "k": 1}}
    assert tagging.tag_prompt(d, c)["metadata"] == {"batch_idx": 1, "k": 1, "prompt_idx": 5, "intra_batch_idx": 1} and d["metadata"]["batch_idx"] == 99

    @dataclasses.dataclass(frozen=True)
    class Frozen:
        prompt_id: str
        metadata: dict = dataclasses.field(default_factory=dict)
    f = Frozen("x")
    assert tagging.tag_prompt(f, c).metadata == c and f.metadata == {}

    class Plain:
        metadata = None
    p = Plain()
    assert tagging.tag_prompt(p, c).metadata == c and p.metadata is None
    assert tagging.tag_prompt(7, c) == 7                               # cannot carry metadata: returned as it is


def test_summaries_and_wire_check():
    assert logging_utils.summarize_list([]) == "[]" and logging_utils.summarize_list(["a", None, "", "b"]) == "[a, b]"
    assert logging_utils.summarize_list(range(10)) == "[0, 1, ..., 8, 9]" and logging_utils.summarize_ids(range(10), 5) == "[0, 1, 2, ..., 8, 9]"
    with pytest.raises(ValueError):
        logging_utils.summarize_list(range(10), 1)

    @dataclasses.dataclass
    class Payload:
        arrays: dict
    shared = np.zeros(3)
    rpc_utils.validate_wire_safe(Payload({"a": shared, "b": [shared, (1, "x")], "c": {3: None}}))
    with pytest.raises(TypeError, match="non-numpy array of type torch.Tensor"):
        rpc_utils.validate_wire_safe(Payload({"a": [np.zeros(2), {"deep": torch.zeros(2)}]}))


def test_metrics_buffer_reduces_once():
    a, b = MetricsBuffer(3), MetricsBuffer(3)
    a.add_weighted("loss", WeightedMetric(torch.tensor(6.0), torch.tensor(3.0)))
    b.add_weighted("loss", WeightedMetric(torch.tensor(2.0), torch.tensor(1.0)))
    a.add_scalar("kl", torch.tensor(0.5)); b.add_scalar("kl", 1.5)
    a.add_scalar("max_len", 7, aggregation_fn=np.max); b.add_scalar("max_len", 9)
    a.merge(b)
    host = a.to_host()
    rpc_utils.validate_wire_safe(host.weighted_metrics)
    assert host.reduce() == {"loss": 2.0, "kl": 1.0, "max_len": 9.0} and host.mode == "train"
    assert float(WeightedMetric(np.float64(1.0), np.float64(0.0), eps=0.5).compute()) == 2.0
    assert float(WeightedMetric(torch.tensor(1.0), torch.tensor(0.1), min_denom=1.0).compute()) == 1.0
    assert float(WeightedMetric(1.0, 0.1, min_denom=1.0).compute()) == 1.0
