"""Agentic RL: tools, parsers, environments, queue, sync lock, trajectory engine, end-to-end learner (CPU)."""
import asyncio
import threading
import time

import numpy as np
import pytest
import torch

from tunix_b200.rl.agentic.agents.agent_types import TrajectoryStatus
from tunix_b200.rl.agentic.agents.model_agent import ModelAgent
from tunix_b200.rl.agentic.agents.tool_agent import ToolAgent
from tunix_b200.rl.agentic.environments.task_environment import TaskEnvironment
from tunix_b200.rl.agentic.environments.tool_environment import ToolEnvironment
from tunix_b200.rl.agentic.parser.chat_template_parser import get_parser
from tunix_b200.rl.agentic.parser.tool_parser import GeminiToolParser, QwenToolParser
from tunix_b200.rl.agentic.queue_manager.group_queue_manager import GroupQueueManager
from tunix_b200.rl.agentic.tools.calculator_tool import CalculatorTool
from tunix_b200.rl.agentic.tools.tool_manager import ToolManager
from tunix_b200.rl.agentic.trajectory.trajectory_collect_engine import TrajectoryCollectEngine
from tunix_b200.rl.agentic.utils import RolloutSyncLock
from tests.test_sampler_cpu import CharTok


def test_tools_and_parsers():
    calc = CalculatorTool()
    assert calc.apply(expression="2*(3+4)").output == 14
    assert calc.apply(expression="__import__('os')").error
    tm = ToolManager([calc])
    out = tm.execute_calls([{"id": "a", "name": "calculator", "arguments": {"expression": "1+1"}},
                            {"id": "b", "name": "nope", "arguments": {}}])
    assert out["a"].output == 2 and out["b"].error
    q = QwenToolParser().parse('x <tool_call>{"name": "calculator", "arguments": {"expression": "3*3"}}</tool_call>')
    assert q == [{"name": "calculator", "arguments": {"expression": "3*3"}}]
    g = GeminiToolParser().parse('```tool_code\n{"name": "f", "args": {"a": 1}}\n```')
    assert g == [{"name": "f", "arguments": {"a": 1}}]
    msgs = [{"role": "user", "content": "hi"}]
    assert get_parser("qwen").parse(msgs, add_generation_prompt=True).endswith("<|im_start|>assistant\n")
    assert get_parser("gemma").parse(msgs).startswith("<bos><start_of_turn>user")
    assert "<|eot_id|>" in get_parser("llama").parse(msgs)
    g4 = get_parser("gemma4")
    assert g4.parse(msgs, add_generation_prompt=True) == "<bos><|turn>system\n<|think|><turn|>\n<|turn>user\nhi<turn|>\n<|turn>model\n"
    assert g4.parse([{"role": "assistant", "content": "ok<turn|>"}, {"role": "tool", "content": "42"}], is_first_msg=False) == \
        "<|turn>model\nok<turn|>\n<|tool_response>42<tool_response|>"
    from tunix_b200.rl.agentic.parser.chat_template_parser import Gemma4ChatTemplateParser
    quiet = Gemma4ChatTemplateParser(CharTok(), enable_thinking=False)
    assert quiet.parse(msgs, add_generation_prompt=True).endswith("<|turn>model\n<|channel>thought\n<channel|>")
    toks, n = quiet.update_assistant_end_tokens(np.asarray([5, 6]))
    assert n == 1 and len(toks) == 3


def test_group_queue_and_sync_lock():
    async def run():
        q = GroupQueueManager(group_size=2)
        await q.put("a0", "a")
        await q.put("b0", "b")
        await q.put("a1", "a")
        got = await q.get_batch(1)
        assert got == [["a0", "a1"]] and q.open_buckets == 1
        await q.put_exception(ValueError("boom"))
        with pytest.raises(ValueError):
            await q.get_batch(1)
    asyncio.run(run())
    lock, order = RolloutSyncLock(), []

    def rollout():
        with lock.acquire_rollout():
            order.append("r+")
            time.sleep(0.05)
            order.append("r-")
    t = threading.Thread(target=rollout)
    t.start()
    time.sleep(0.01)
    with lock.acquire_weight_sync():
        order.append("sync")
    t.join()
    assert order == ["r+", "r-", "sync"]


def test_multi_turn_tool_episode_records_tokens_and_masks():
    tok = CharTok()
    script = iter(['<tool_call>{"name": "calculator", "arguments": {"expression": "6*7"}}</tool_call>',
                   '<tool_call>{"name": "finish", "arguments": {"response": "42"}}</tool_call>'])

    async def model_call(chat_completions=None, prompt_token_ids=None, max_tokens=None):
        text = next(script)
        ids = tok.encode(text)
        return {"text": text, "tokens": ids, "logprobs": [-0.5] * len(ids)}
    env = ToolEnvironment(task={"question": "6*7?", "answer": "42"}, tools=[CalculatorTool()], reward_fn="exact_match", max_steps=4)
    eng = TrajectoryCollectEngine(ToolAgent(tools={"calculator": CalculatorTool()}), env, model_call=model_call, tokenizer=tok,
                                  chat_parser=get_parser("qwen"), max_steps=4)
    out = asyncio.run(eng.collect("Token"))
    assert out["status"] == TrajectoryStatus.SUCCEEDED and out["trajectory_reward"] == 1.0 and out["num_turns"] == 2
    m = out["conversation_masks"]
    assert m.sum() > 0 and (m == 0).sum() > 0                       # assistant and environment tokens both present
    assert np.all(out["old_logprobs"][m == 1] == -0.5) and np.all(out["old_logprobs"][m == 0] == 0)


def test_failed_episode_is_marked_not_raised():
    async def model_call(**kw):
        raise RuntimeError("engine down")
    eng = TrajectoryCollectEngine(ModelAgent(), TaskEnvironment(task={"question": "q"}), model_call=model_call, tokenizer=CharTok())
    traj = asyncio.run(eng.collect("Trajectory"))
    assert traj.status == TrajectoryStatus.FAILED


def test_agentic_grpo_learner_end_to_end():
    from tunix_b200 import optim
    from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
    from tunix_b200.rl.algorithm_config import GRPOConfig
    from tunix_b200.rl.rl_cluster import RLCluster
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)
    actor, ref = create_model(cfg, seed=0), create_model(cfg, seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1000, max_steps=3, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=2,
                          train_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=5, max_prompt_length=16, temperature=1.0, seed=1, kv_cache_size=64, eos_tokens=[63])
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(), cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    before = torch.cat([p.detach().reshape(-1).clone() for p in actor.parameters()])

    def length_reward(prompts, completions, completion_lengths=None, **kw):
        return [float(n % 3) for n in completion_lengths]
    learner = AgenticGRPOLearner(cl, [length_reward], GRPOConfig(num_generations=2, beta=0.04), max_concurrency=4,
                                 chat_parser=get_parser("raw"))
    learner.train([{"prompts": ["ab", "cd"]}, {"prompts": ["ef", "gh"]}])
    assert cl.global_steps == 2 and learner.policy_version == 2
    after = torch.cat([p.detach().reshape(-1) for p in actor.parameters()])
    assert cl.metrics_logger.metric_exists("", "trajectory/valid_frac", "train")
    # an external model client (e.g. the HTTP one) replaces the cluster's engine for the episodes' model calls
    calls = []

    async def client(chat_completions=None, prompt_token_ids=None, max_tokens=None):
        calls.append(len(prompt_token_ids))
        n = 2 + len(calls) % 3
        return {"text": "x" * n, "tokens": [5 + (len(calls) + k) % 50 for k in range(n)], "logprobs": [-1.0] * n}
    remote = AgenticGRPOLearner(cl, [length_reward], GRPOConfig(num_generations=2, beta=0.04), max_concurrency=4,
                                chat_parser=get_parser("raw"), model_client=client)
    remote.train([{"prompts": ["ab", "cd"]}, {"prompts": ["ef", "gh"]}, {"prompts": ["ij", "kl"]}])   # two consumed: resumed past
    assert len(calls) == 4 and cl.global_steps == 3


def test_frozenlake_environment_and_multi_turn_episode():
    from tunix_b200.rl.agentic.environments.frozenlake_environment import (FrozenLakeAgent, FrozenLakeEnv, generate_map,
                                                                            parse_move, shortest_path)
    assert parse_move("I think ```Left``` then ```Down```") == "down" and parse_move("go RIGHT now") == "right"
    assert parse_move("no idea") is None
    for seed in range(20):                                  # every generated map is solvable and reproducible
        g = generate_map(5, 0.6, seed)
        assert shortest_path(g) is not None and g == generate_map(5, 0.6, seed) and g[0][0] == "S" and g[-1][-1] == "G"
    env = FrozenLakeEnv({"map": ["S_O", "__O", "O_G"]}, max_steps=6)
    obs, _ = env.reset()
    assert "P _ O" in obs and "6 moves" in obs
    assert env.step("```Up```")[0].count("P") == 1 and env.pos == (0, 0)                   # walls clamp
    obs, r, done, info = env.step("banana")
    assert not done and info["valid"] is False and "not a move" in obs
    assert env.step("```Right```")[3]["moved"] == "right" and env.pos == (0, 1)
    obs, r, done, info = env.step("```Right```")
    assert done and r == 0.0 and "X" in obs and info["won"] is False                        # a hole ends the episode
    # a scripted model walks the shortest path through the collection engine: multi-turn, reward 1
    task = {"seed": 3, "size": 4, "p": 0.7, "max_steps": 10}
    env = FrozenLakeEnv(task)
    path = shortest_path(env.grid)
    tok = CharTok()
    script = iter([f"The goal is below and to the right. ```{m.capitalize()}```" for m in path])

    async def model_call(chat_completions=None, prompt_token_ids=None, max_tokens=None):
        text = next(script)
        ids = tok.encode(text)
        return {"text": text, "tokens": ids, "logprobs": [-0.1] * len(ids)}
    eng = TrajectoryCollectEngine(FrozenLakeAgent(), env, model_call=model_call, tokenizer=tok, chat_parser=get_parser("qwen"),
                                  max_steps=10)
    out = asyncio.run(eng.collect("Token"))
    assert out["status"] == TrajectoryStatus.SUCCEEDED and out["trajectory_reward"] == 1.0 and out["num_turns"] == len(path)
    assert (out["conversation_masks"] == 0).sum() > 0       # the maps the environment sent back are masked out of the loss
    # slippery episodes are reproducible from the task
    runs = []
    for _ in range(2):
        e = FrozenLakeEnv({"seed": 5, "size": 4, "is_slippery": True}, max_steps=5)
        e.reset()
        runs.append([e.step("```Down```")[3].get("moved") for _ in range(3) if e.step_count < 3])
    assert runs[0] == runs[1]


def test_episode_over_http_against_a_remote_engine_server():
    """A FrozenLake episode whose model calls go over HTTP to the OpenAI-style front end: prompts travel as token
    ids, sampled ids and log-probs come back and are what the trajectory records."""
    from tests.test_sampler_cpu import _FakeEngine
    from tunix_b200.generate.engine import EngineServer
    from tunix_b200.generate.openai_server import serve
    from tunix_b200.rl.agentic.environments.frozenlake_environment import FrozenLakeAgent, FrozenLakeEnv
    from tunix_b200.rl.agentic.http_model_client import HTTPModelClient, RemoteModelError
    tok = CharTok()
    fake = _FakeEngine(slots=4)
    fake.cache_size = 8192
    with EngineServer(fake, max_new_tokens=6, max_prompt_length=4096, eos_tokens=[2]) as eng, \
            serve(eng, tok, model_name="toy") as http:
        client = HTTPModelClient(http.url, route_key="episode-1")
        out = client.generate([1, 30, 31], max_tokens=3)
        assert out["tokens"] == [32, 33, 34] and out["logprobs"] == [0.0] * 3 and out["text"] == tok.decode([32, 33, 34])
        env = FrozenLakeEnv({"map": ["S_", "_G"]}, max_steps=3)
        engine = TrajectoryCollectEngine(FrozenLakeAgent(), env, model_call=client.with_route_key("episode-2"), tokenizer=tok,
                                         chat_parser=get_parser("qwen"), max_steps=3)
        res = asyncio.run(engine.collect("Token"))
        # the scripted engine continues from the prompt's last token, which is no move: the environment reminds, three turns pass
        assert res["num_turns"] == 3 and res["trajectory_reward"] == 0.0 and res["status"] != TrajectoryStatus.FAILED
        assert (res["conversation_masks"] == 1).sum() == 3 * 6 and client.calls == 1 + 3
        with pytest.raises(RemoteModelError, match="400"):
            client.generate([], 2)
        with pytest.raises(ValueError):
            asyncio.run(client(chat_completions=[{"role": "user", "content": "hi"}]))
        chat = HTTPModelClient(http.url, tokenizer=tok, chat_parser=get_parser("qwen"))
        assert len(asyncio.run(chat(chat_completions=[{"role": "user", "content": "hi"}], max_tokens=2))["tokens"]) == 2
    down = HTTPModelClient(http.url, retries=1, timeout=2.0)
    with pytest.raises(RemoteModelError, match="no answer"):
        down.generate([1, 2], 1)


def test_partial_rollout_resume_context_limit_and_routed_experts():
    tok = CharTok()
    calls = []

    async def model_call(chat_completions=None, prompt_token_ids=None, max_tokens=None):
        calls.append(len(prompt_token_ids))
        n = len(calls)
        text = '<tool_call>{"name": "calculator", "arguments": {"expression": "%d+1"}}</tool_call>' % n if n < 3 else \
            '<tool_call>{"name": "finish", "arguments": {"response": "3"}}</tool_call>'
        ids = tok.encode(text)
        return {"text": text, "tokens": ids, "logprobs": [-0.25] * len(ids), "policy_version": 7 + n // 2,
                "routed_experts": np.full((len(ids), 2, 2), n, np.int16)}

    def engine(**kw):
        env = ToolEnvironment(task={"question": "count", "answer": "3"}, tools=[CalculatorTool()], reward_fn="exact_match", max_steps=6)
        return TrajectoryCollectEngine(ToolAgent(tools={"calculator": CalculatorTool()}), env, model_call=model_call, tokenizer=tok,
                                       chat_parser=get_parser("qwen"), max_steps=6, **kw)
    eng = engine()
    part = asyncio.run(eng.collect("Token", max_new_steps=1))
    assert part["status"] == TrajectoryStatus.PARTIAL and part["num_turns"] == 1 and len(calls) == 1
    ctx_after_first = calls[0]
    out = asyncio.run(eng.resume("Token"))                                       # same agent, environment and token context
    assert out["status"] == TrajectoryStatus.SUCCEEDED and out["num_turns"] == 3 and out["trajectory_reward"] == 1.0
    assert calls[1] > ctx_after_first and calls[2] > calls[1]                    # every call sees the whole conversation so far
    assert out["policy_versions"] == [7, 8, 8] and out["policy_version"] == 7   # the oldest weights that contributed
    assert [int(r[0, 0, 0]) for r in out["routed_experts"]] == [1, 2, 3]
    with pytest.raises(RuntimeError):
        asyncio.run(eng.resume("Token"))                                         # a finished episode cannot be resumed
    # context window: the second call would start beyond the limit
    calls.clear()
    short = engine(max_context_tokens=ctx_after_first + 10)
    out = asyncio.run(short.collect("Token"))
    assert out["status"] == TrajectoryStatus.MAX_CONTEXT_LIMIT_REACHED and out["num_turns"] == 1


def test_agentic_learner_pack_first_scoring_eval_and_trajectory_log():
    from tunix_b200 import optim
    from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
    from tunix_b200.models.config import ModelConfig
    from tunix_b200.models.transformer import create_model
    from tunix_b200.rl.agentic.agentic_grpo_learner import AgenticGRPOLearner
    from tunix_b200.rl.algorithm_config import GRPOConfig
    from tunix_b200.rl.rl_cluster import RLCluster
    cfg = ModelConfig.tiny_llama().replace(num_layers=1, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2, head_dim=16, num_kv_heads=1)
    actor, ref = create_model(cfg, seed=0), create_model(cfg, seed=0)
    tc = RLTrainingConfig(eval_every_n_steps=1, max_steps=2, actor_optimizer=optim.AdamW(1e-3), mini_batch_size=2,
                          train_micro_batch_size=2)
    rc = RolloutConfig(max_tokens_to_generate=5, max_prompt_length=16, temperature=1.0, seed=1, kv_cache_size=64, eos_tokens=[63])
    cl = RLCluster(actor=actor, reference=ref, tokenizer=CharTok(), cluster_config=ClusterConfig(role_to_mesh={}, training_config=tc, rollout_config=rc))
    ref_calls, logged = [], []
    orig_ref = cl.get_ref_per_token_logps

    def spy_ref(p, c, *a, **kw):
        ref_calls.append((tuple(p.shape), tuple(c.shape), kw.get("segment_ids") is not None))
        return orig_ref(p, c, *a, **kw)
    cl.get_ref_per_token_logps = spy_ref

    def length_reward(prompts, completions, completion_lengths=None, **kw):
        return [float(n % 3) for n in completion_lengths]
    learner = AgenticGRPOLearner(cl, [length_reward], GRPOConfig(num_generations=2, beta=0.04), max_concurrency=4,
                                 chat_parser=get_parser("raw"), pack_first=True, pack_budget=48, trajectory_logger=logged.extend)
    before = torch.cat([p.detach().reshape(-1).clone() for p in actor.parameters()])
    learner.train([{"prompts": ["ab", "cd"]}, {"prompts": ["ef", "gh"]}], eval_ds=[{"prompts": ["xy"]}])
    assert cl.global_steps == 2 and not torch.equal(before, torch.cat([p.detach().reshape(-1) for p in actor.parameters()]))
    # the reference scored packed rows (no prompt side, segment ids given), not padded groups
    assert ref_calls and all(p[1] == 0 and seg for p, _, seg in ref_calls)
    assert len(logged) == 8 and {"conversation_tokens", "trajectory_reward", "policy_version"} <= set(logged[0])
    assert cl.metrics_logger.metric_exists("", "eval/rewards/mean", "eval")
    assert len(cl.metrics_logger.get_metric_history("", "eval/episodes", "eval")) == 2      # after each of the two steps


def test_collector_engine_pause_resume_versions_and_budget_facts():
    """The distributed rollout wrapper: sampler calls with derived seeds and per-call limits, a pause that holds the next
    turn until resume (which then runs under the newer policy version), request-scoped metadata on the item."""
    import dataclasses
    from tunix_b200.experimental.rollout import collector as col
    from tunix_b200.experimental.rollout.sampler import SamplingResponse
    tok = CharTok()
    texts = ['<tool_call>{"name": "calculator", "arguments": {"expression": "6*7"}}</tool_call>',
             '<tool_call>{"name": "finish", "arguments": {"response": "42"}}</tool_call>']
    seen = []

    class FakeSampler:
        async def sample(self, reqs):
            r = reqs[0]
            seen.append((r.sampling_params.seed, r.sampling_params.max_tokens, len(r.prompt_token_ids)))
            ids = tok.encode(texts[len(seen) - 1])
            return [SamplingResponse(request_id=r.request_id, token_ids=ids, logprobs=[-0.25] * len(ids), text=texts[len(seen) - 1])]

    @dataclasses.dataclass
    class Req:
        prompt_id: str = "p7"
        group_index: int = 2
        generation_kwargs: dict = dataclasses.field(default_factory=lambda: {"temperature": 1.0, "max_tokens": 400})
        max_turns: int = 4
        max_response_length: int = 1000
        target_policy_version: int = 3
        metadata: dict = dataclasses.field(default_factory=lambda: {"episode_timeout": 30.0, "tag": "x"})

    version = {"v": 3}
    env = ToolEnvironment(task={"question": "6*7?", "answer": "42"}, tools=[CalculatorTool()], reward_fn="exact_match", max_steps=4)
    eng = col.TrajectoryCollectorEngine("traj_p7_g2", Req(), FakeSampler(), env, ToolAgent(tools={"calculator": CalculatorTool()}),
                                        tok, get_parser("qwen"), eos_ids=[tok.encode(">")[0]], policy_version_fn=lambda: version["v"])

    async def run():
        task = asyncio.ensure_future(eng.run_episode())
        while len(seen) < 1:
            await asyncio.sleep(0.001)
        eng.pause()                       # weight sync begins after the first turn was requested
        await asyncio.sleep(0.05)
        n_paused = len(seen)
        version["v"] = 4
        eng.resume()
        return await task, n_paused
    item, n_paused = asyncio.run(run())
    assert n_paused <= 2 and len(seen) == 2
    seed = col.generate_vanilla_rollout_seed("p7", 2)
    assert seen[0][0] == seed and seen[1][0] == seed and seen[0][1] == 400       # per-call limit = the request's own
    assert seen[1][1] <= 400 and seen[1][2] > seen[0][2]                          # later turns see the longer context
    md = item.metadata
    assert item.group_id == "p7" and item.pair_index == 2 and md["tag"] == "x" and md["status"] == TrajectoryStatus.SUCCEEDED
    assert md["policy_versions"][0] == 3 and md["policy_versions"][-1] in (3, 4) and md["policy_version"] == 3
    assert item.traj["trajectory_reward"] == 1.0 and item.traj["policy_versions"] == md["policy_versions"]
    assert md["raw_length"] == len(item.traj["conversation_tokens"]) and md["clipped"] is False
    with pytest.raises(TypeError):
        col.TrajectoryCollectorEngine("t", dataclasses.replace(Req(), metadata={"overlong_filter": "yes"}), FakeSampler(), env,
                                      ToolAgent(tools={}), tok)
    with pytest.raises(ValueError):
        col.response_budget_facts([1], 0, {1})
