"""Worker factories for `runtime.launcher` (`--factory tunix_b200.experimental.worker.factories:<name>`): the process
that is started builds its own model and engine from plain arguments, since only strings cross the command line.

`make_rollout_worker` builds a decoder from a preset name (or a tiny built-in one), puts the dense sampler or, on a
GPU, the paged engine's server in front of it and installs weights that arrive with `sync_weights` as a
`{parameter name: array}` payload: the same payload `export_state` produces on the trainer's side."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch


class ByteTokenizer:
    """Bytes as tokens (ids 3..258), for self-contained demos; 0 pad, 1 bos, 2 eos."""

    def encode(self, s: str) -> list:
        return [3 + b for b in s.encode()]

    def decode(self, ids) -> str:
        return bytes(int(i) - 3 for i in ids if 3 <= int(i) < 259).decode(errors="replace")

    def bos_id(self) -> int:
        return 1

    def eos_id(self) -> int:
        return 2

    def pad_id(self) -> int:
        return 0


def toy_config(vocab_size: int = 320, dtype: torch.dtype = torch.float32):
    from ...models.config import ModelConfig
    return ModelConfig(family="llama3", num_layers=2, vocab_size=vocab_size, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16,
                       num_kv_heads=2, dtype=dtype, max_position=256)


def export_state(model: torch.nn.Module) -> dict:
    """Weights as host arrays keyed by parameter name (bf16 travels as its 16-bit pattern)."""
    out = {}
    for name, p in model.named_parameters():
        t = p.detach().cpu()
        out[name] = ("bf16", t.view(torch.int16).numpy()) if t.dtype == torch.bfloat16 else ("raw", t.numpy())
    return out


@torch.no_grad()
def install_state(model: torch.nn.Module, payload: dict) -> int:
    params = dict(model.named_parameters())
    missing = set(params) - set(payload)
    if missing:
        raise KeyError(f"payload lacks {sorted(missing)[:4]}")
    n = 0
    for name, (kind, arr) in payload.items():
        if name not in params:
            continue
        t = torch.from_numpy(np.ascontiguousarray(arr))
        if kind == "bf16":
            t = t.view(torch.bfloat16)
        params[name].copy_(t.to(params[name].device, params[name].dtype))
        n += 1
    return n


def make_rollout_worker(worker_id: str, role: str = "rollout", model: str = "toy", seed: int = 0, device: Optional[str] = None,
                        cache_size: int = 256, engine: str = "auto", max_new_tokens: int = 64, max_prompt_length: int = 128,
                        temperature: float = 1.0):
    from ...common.configs import CacheConfig
    from ...generate.sampler import Sampler
    from ...models.transformer import create_model
    from .rollout_worker import RolloutWorker
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    if model == "toy":
        cfg = toy_config(dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)
    else:
        from ...models.config import get_config
        cfg = get_config(model)
    net = create_model(cfg, device=dev, seed=seed)
    tok = ByteTokenizer()
    cc = CacheConfig(cache_size, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim)
    if engine == "paged" or (engine == "auto" and dev.type == "cuda"):
        from ...generate.engine import EngineServer, PagedEngine
        eng = EngineServer(PagedEngine(net, tok, cc), max_new_tokens=max_new_tokens, max_prompt_length=max_prompt_length,
                           temperature=temperature, seed=seed, eos_tokens=[tok.eos_id()])
    else:
        eng = Sampler(net, tok, cc)
    w = RolloutWorker(worker_id, eng, eos_tokens=[tok.eos_id()], apply_weights=lambda version, payload: install_state(net, payload))
    w.role = role
    w.model = net
    w.releases_bulk_payloads = True                     # install_state copies into the parameters and keeps nothing
    return w


def make_agentic_rollout_worker(worker_id: str, role: str = "rollout", model: str = "toy", seed: int = 0, device: Optional[str] = None,
                                cache_size: int = 2048, engine: str = "auto", max_new_tokens: int = 256, max_prompt_length: int = 1536,
                                temperature: float = 1.0, agent: str = "frozenlake", env: str = "frozenlake", chat_parser: str = "qwen",
                                discover: str = "", batch_window_s: float = 0.002):
    """An episode worker for launched processes: a model behind the asynchronous sampler protocol, agents and
    environments looked up by registry key. `discover`: comma-separated import paths or directories whose decorated
    agent / environment classes are registered before the first request (`registry.auto_discover_modules`); the
    FrozenLake pair is registered under "frozenlake"."""
    from ...common.configs import CacheConfig
    from ...generate.sampler import Sampler
    from ...models.transformer import create_model
    from ...rl.agentic.environments.frozenlake_environment import FrozenLakeAgent, FrozenLakeEnv
    from ...rl.agentic.parser.chat_template_parser import get_parser
    from ..rl.agentic import registry
    from ..rollout.sampler import EngineSamplerAdapter
    from .agentic_rollout_worker import AgenticRolloutWorker
    for reg, cls in ((registry.AGENT_REGISTRY, FrozenLakeAgent), (registry.ENV_REGISTRY, FrozenLakeEnv)):
        if "frozenlake" not in reg:
            reg.register("frozenlake")(cls)
    if discover:
        registry.auto_discover_modules(*[p for p in discover.split(",") if p])
    dev = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    if model == "toy":
        cfg = toy_config(dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32).replace(max_position=max(cache_size, 256))
    else:
        from ...models.config import get_config
        cfg = get_config(model)
    net = create_model(cfg, device=dev, seed=seed)
    tok = ByteTokenizer()
    cc = CacheConfig(cache_size, cfg.num_layers, cfg.num_kv_heads, cfg.head_dim)
    if engine == "paged" or (engine == "auto" and dev.type == "cuda"):
        from ...generate.engine import EngineServer, PagedEngine
        eng = EngineServer(PagedEngine(net, tok, cc), max_new_tokens=max_new_tokens, max_prompt_length=max_prompt_length,
                           temperature=temperature, seed=seed, eos_tokens=[tok.eos_id()])
        sampler = EngineSamplerAdapter(eng, tokenizer=tok, eos_tokens=[tok.eos_id()])
    else:
        sampler = EngineSamplerAdapter(Sampler(net, tok, cc), tokenizer=tok, eos_tokens=[tok.eos_id()], batch_window_s=batch_window_s)
    w = AgenticRolloutWorker(worker_id, sampler, tok, chat_parser=get_parser(chat_parser), eos_ids=[tok.eos_id()], default_agent=agent,
                             default_env=env, apply_weights=lambda version, payload: install_state(net, payload))
    w.role = role
    w.model = net
    w.releases_bulk_payloads = True
    return w
