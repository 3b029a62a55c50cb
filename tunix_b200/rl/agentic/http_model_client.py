"""Model calls of agentic rollouts against a remote engine over HTTP.

`TrajectoryCollectEngine` only needs `await model_call(chat_completions=..., prompt_token_ids=..., max_tokens=...)`
returning `{"text", "tokens", "logprobs"}`. `HTTPModelClient` provides that against the OpenAI-style front end of
`generate/openai_server.py` (one or several engine servers in another process or on another host): the prompt goes
out as token ids, the sampled ids and their log-probs come back, so the trajectory that is trained on is exactly the
one that was sampled: no re-tokenisation on either side. `route_key` keeps the turns of one episode on the same
engine so that the conversation's prefix stays in its KV cache.

The reference reaches remote rollout engines through vLLM's server mode
(tunix/rl/agentic/agentic_rl_learner.py:293-301); this is the same role over plain HTTP."""
from __future__ import annotations

import asyncio
import json
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from typing import Optional, Sequence


class RemoteModelError(RuntimeError):
    pass


class HTTPModelClient:
    def __init__(self, base_url: str, *, route_key: Optional[str] = None, timeout: float = 600.0, max_connections: int = 64,
                 retries: int = 2, tokenizer=None, chat_parser=None):
        """`tokenizer` / `chat_parser` are only needed for calls that pass `chat_completions` without token ids."""
        self.base_url = base_url.rstrip("/")
        self.route_key, self.timeout, self.retries = route_key, timeout, retries
        self.tokenizer, self.chat_parser = tokenizer, chat_parser
        self._pool = ThreadPoolExecutor(max_connections, thread_name_prefix="http-model-client")
        self._stats = {"calls": 0}                          # shared with the views made by with_route_key

    @property
    def calls(self) -> int:
        return self._stats["calls"]

    def with_route_key(self, route_key: str) -> "HTTPModelClient":
        """A view of this client pinned to one conversation (shares the connection pool)."""
        twin = object.__new__(HTTPModelClient)
        twin.__dict__.update(self.__dict__)
        twin.route_key = route_key
        return twin

    def _post(self, body: dict) -> dict:
        data = json.dumps(body).encode()
        headers = {"Content-Type": "application/json"}
        if self.route_key:
            headers["x-route-key"] = self.route_key
        last: Optional[BaseException] = None
        for _ in range(self.retries + 1):
            try:
                req = urllib.request.Request(self.base_url + "/v1/completions", data=data, headers=headers)
                with urllib.request.urlopen(req, timeout=self.timeout) as r:
                    return json.loads(r.read())
            except urllib.error.HTTPError as e:
                detail = e.read().decode(errors="replace")[:500]
                if e.code in (400, 404):                    # the request is wrong: asking again will not help
                    raise RemoteModelError(f"{e.code} from {self.base_url}: {detail}") from e
                last = RemoteModelError(f"{e.code} from {self.base_url}: {detail}")
            except (urllib.error.URLError, ConnectionError, TimeoutError) as e:
                last = e
        raise RemoteModelError(f"no answer from {self.base_url} after {self.retries + 1} attempts") from last

    def generate(self, prompt_token_ids: Sequence[int], max_tokens: Optional[int] = None) -> dict:
        body = {"prompt": [int(t) for t in prompt_token_ids], "logprobs": True}
        if max_tokens is not None:
            body["max_tokens"] = int(max_tokens)
        ans = self._post(body)
        choice = ans["choices"][0]
        lp = choice.get("logprobs") or {}
        self._stats["calls"] += 1
        return {"text": choice["text"], "tokens": list(lp.get("tokens") or []), "logprobs": list(lp.get("token_logprobs") or []),
                "finish_reason": choice.get("finish_reason")}

    async def __call__(self, chat_completions=None, prompt_token_ids=None, max_tokens=None) -> dict:
        if prompt_token_ids is None:
            if self.tokenizer is None or self.chat_parser is None:
                raise ValueError("a call without prompt_token_ids needs the client's tokenizer and chat_parser")
            text = self.chat_parser.parse(list(chat_completions or []), add_generation_prompt=True, is_first_msg=True)
            prompt_token_ids = self.tokenizer.encode(text)
        return await asyncio.get_running_loop().run_in_executor(self._pool, self.generate, list(prompt_token_ids), max_tokens)

    def close(self) -> None:
        self._pool.shutdown(wait=False)
