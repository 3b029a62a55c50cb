"""OpenAI-style HTTP front end of the continuous-batching engine server
(the role of tunix/experimental/rollout/serve_vllm_sampler.py:54-360 in the reference, which puts FastAPI in front of
a vLLM sampler).

Routes:

    GET  /health, /v1/models        liveness and the served model's name
    GET  /metrics                   Prometheus text format: requests, errors by status, prompt / completion tokens,
                                    request latency histogram, requests in flight
    POST /v1/completions            {"prompt": str | [int] | [str | [int]], "max_tokens", "n", "stop", "logprobs", "stream"}
                                    (token ids as a prompt reach the engine untouched; with "logprobs" the answer
                                    carries the sampled token ids and their log-probs, which is what RL needs)
    POST /v1/chat/completions       {"messages": [{"role", "content"}], "max_tokens", "n", "stop", "stream"}

Every HTTP request becomes one `submit()` on the engine server and joins the running batch at its next check point;
one handler thread per connection waits for its own future, so concurrency on the wire turns directly into batch
width on the GPU. Sampling parameters are fixed per engine server (they shape its captured decode step): a request
whose `temperature` / `top_p` differ from the server's is answered with the server's values, reported back under
`"sampling"`. `stream: true` answers as server-sent events. A request for one completion (`n` = 1, one prompt) on a
back end that reports tokens while it generates (`EngineServer`, `PooledBackend`) is streamed as it is produced: a
chunk per check point of the engine's decode loop, the text cut at a stop string if one is given, then a finish chunk
and `[DONE]`. Other streamed requests carry one content chunk per choice, a finish chunk and `[DONE]`.

The back end is anything with `generate(prompt_token_ids, max_tokens) -> (tokens, logprobs)`, i.e.
`generate.engine.EngineServer`; chat prompts are rendered by a `ChatTemplateParser`. The server is the standard
library's threaded HTTP server: nothing here needs an event loop."""
from __future__ import annotations

import json
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Optional, Sequence


class _BadRequest(ValueError):
    pass


_LAT_BUCKETS = (0.05, 0.1, 0.25, 0.5, 1.0, 2.5, 5.0, 10.0, 30.0, 60.0, 120.0)


class _HTTPServer(ThreadingHTTPServer):
    request_queue_size = 1024                               # the listen backlog: hundreds of clients connect at once
    daemon_threads = True


class OpenAIServer:
    def __init__(self, backend, tokenizer, *, model_name: str = "tunix-b200", chat_parser=None,
                 host: str = "127.0.0.1", port: int = 0, request_timeout: Optional[float] = 600.0,
                 sampling: Optional[dict] = None):
        """`port=0` picks a free port (read it back from `.port`). `sampling` is echoed to clients."""
        if chat_parser is None:
            from ..rl.agentic.parser.chat_template_parser import get_parser
            chat_parser = get_parser("default", tokenizer)
        self.backend, self.tokenizer, self.chat_parser = backend, tokenizer, chat_parser
        self.model_name, self.request_timeout = model_name, request_timeout
        self.sampling = dict(sampling or {})
        self.requests_served = 0
        self._lock = threading.Lock()
        self._m = {"prompt_tokens": 0, "completion_tokens": 0, "inflight": 0, "errors": {}, "lat_sum": 0.0,
                   "lat_buckets": [0] * (len(_LAT_BUCKETS) + 1)}
        outer = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):                      # quiet: the engine's own metrics are the record
                pass

            def do_GET(self):
                if self.path in ("/health", "/v1/models"):
                    outer._send_json(self, 200, outer._models())
                elif self.path == "/metrics":
                    data = outer.metrics_text().encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    self.wfile.write(data)
                else:
                    outer._send_json(self, 404, {"error": {"message": f"no route {self.path}", "type": "not_found"}})

            def do_POST(self):
                try:
                    n = int(self.headers.get("Content-Length") or 0)
                    body = json.loads(self.rfile.read(n) or b"{}")
                    if not isinstance(body, dict):
                        raise _BadRequest("the request body must be a JSON object")
                    if body.get("route_key") is None and self.headers.get("x-route-key"):
                        body["route_key"] = self.headers.get("x-route-key")
                    if self.path == "/v1/completions":
                        outer._completions(self, body)
                    elif self.path == "/v1/chat/completions":
                        outer._chat(self, body)
                    else:
                        outer._send_json(self, 404, {"error": {"message": f"no route {self.path}", "type": "not_found"}})
                except (_BadRequest, json.JSONDecodeError) as e:
                    outer._send_json(self, 400, {"error": {"message": str(e), "type": "invalid_request_error"}})
                except TimeoutError as e:
                    outer._send_json(self, 504, {"error": {"message": f"generation timed out: {e}", "type": "timeout"}})
                except RuntimeError as e:                   # the engine server is closed or failed
                    outer._send_json(self, 503, {"error": {"message": str(e), "type": "unavailable"}})

        self._httpd = _HTTPServer((host, port), Handler)
        self.host, self.port = self._httpd.server_address[:2]
        self._thread = threading.Thread(target=self._httpd.serve_forever, name="tunix-b200-openai-server", daemon=True)
        self._thread.start()

    # ------------------------------------------------------------------ plumbing
    @property
    def url(self) -> str:
        return f"http://{self.host}:{self.port}"

    def close(self) -> None:
        self._httpd.shutdown()
        self._httpd.server_close()
        self._thread.join(5.0)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def metrics_text(self) -> str:
        with self._lock:
            m = {k: (dict(v) if isinstance(v, dict) else list(v) if isinstance(v, list) else v) for k, v in self._m.items()}
            served = self.requests_served
        p = "tunix_b200_http"
        lines = [f"# TYPE {p}_requests_total counter", f"{p}_requests_total {served}",
                 f"# TYPE {p}_errors_total counter"]
        lines += [f'{p}_errors_total{{status="{code}"}} {n}' for code, n in sorted(m["errors"].items())] or [f"{p}_errors_total 0"]
        lines += [f"# TYPE {p}_prompt_tokens_total counter", f"{p}_prompt_tokens_total {m['prompt_tokens']}",
                  f"# TYPE {p}_completion_tokens_total counter", f"{p}_completion_tokens_total {m['completion_tokens']}",
                  f"# TYPE {p}_requests_in_flight gauge", f"{p}_requests_in_flight {m['inflight']}",
                  f"# TYPE {p}_request_seconds histogram"]
        acc = 0
        for le, n in zip(_LAT_BUCKETS, m["lat_buckets"]):
            acc += n
            lines.append(f'{p}_request_seconds_bucket{{le="{le}"}} {acc}')
        acc += m["lat_buckets"][-1]
        lines += [f'{p}_request_seconds_bucket{{le="+Inf"}} {acc}', f"{p}_request_seconds_sum {m['lat_sum']:.6f}",
                  f"{p}_request_seconds_count {acc}"]
        return "\n".join(lines) + "\n"

    def _send_json(self, h, code: int, payload: dict) -> None:
        if code >= 400:
            with self._lock:
                self._m["errors"][code] = self._m["errors"].get(code, 0) + 1
        data = json.dumps(payload).encode()
        h.send_response(code)
        h.send_header("Content-Type", "application/json")
        h.send_header("Content-Length", str(len(data)))
        h.end_headers()
        h.wfile.write(data)

    @staticmethod
    def _send_sse(h, chunks: Sequence[dict]) -> None:
        data = b"".join(b"data: " + json.dumps(c).encode() + b"\n\n" for c in chunks) + b"data: [DONE]\n\n"
        h.send_response(200)
        h.send_header("Content-Type", "text/event-stream")
        h.send_header("Cache-Control", "no-cache")
        h.send_header("Content-Length", str(len(data)))
        h.end_headers()
        h.wfile.write(data)

    def _can_stream_live(self, n_prompts: int, n: int) -> bool:
        return n_prompts == 1 and n == 1 and bool(getattr(self.backend, "streams", False))

    def _stream_live(self, h, prompt, body: dict, make_chunk, finish_chunk) -> None:
        """Generate one completion and write it as server-sent events while the engine produces it.
        `make_chunk(text_piece, first)` / `finish_chunk(reason)` build the event payloads."""
        import queue as queue_lib
        ids = self.tokenizer.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        if not ids:
            raise _BadRequest("empty prompt")
        max_tokens = body.get("max_tokens")
        if max_tokens is not None and (not isinstance(max_tokens, int) or max_tokens < 1):
            raise _BadRequest("max_tokens must be a positive integer")
        stop = body.get("stop")
        stops = [stop] if isinstance(stop, str) else (stop or [])
        events: "queue_lib.Queue" = queue_lib.Queue()
        done = threading.Event()
        result: dict = {}

        def run():
            try:
                kw = {"route_key": body.get("route_key")} if getattr(self.backend, "routes", False) else {}
                result["out"] = self.backend.generate(ids, max_tokens, timeout=self.request_timeout,
                                                      on_tokens=lambda t, l: events.put([int(x) for x in t]), **kw)
            except BaseException as e:
                result["error"] = e
            finally:
                done.set()
                events.put(None)
        t0 = time.perf_counter()
        with self._lock:
            self._m["inflight"] += 1
        threading.Thread(target=run, daemon=True).start()
        head = events.get()                                 # the first piece, or the end: errors before any token keep their status code
        if head is None and "error" in result:
            with self._lock:
                self._m["inflight"] -= 1
            raise result["error"]
        events.put(head) if head is None else None
        pending_head = [head] if head is not None else []
        h.send_response(200)
        h.send_header("Content-Type", "text/event-stream")
        h.send_header("Cache-Control", "no-cache")
        h.send_header("Connection", "close")                # no length: the end of the connection ends the stream
        h.end_headers()

        def write(payload) -> None:
            h.wfile.write(b"data: " + (payload if isinstance(payload, bytes) else json.dumps(payload).encode()) + b"\n\n")
            h.wfile.flush()
        toks: list = []
        sent_text, held, stopped, first = "", "", False, True
        try:
            while True:
                piece = pending_head.pop() if pending_head else events.get()
                if piece is None:
                    break
                toks.extend(piece)
                if stopped:
                    continue                                # the engine runs on to its limit; nothing more is sent
                text = self.tokenizer.decode(toks)
                cut = min((i for i in (text.find(x) for x in stops) if i >= 0), default=-1)
                if cut >= 0:
                    text, stopped = text[:cut], True
                elif text.endswith("\ufffd"):
                    continue                                # half a multi-byte character: wait for the rest
                else:                                       # the tail may be the beginning of a stop string: keep it back
                    hold = max((k for x in stops for k in range(1, len(x)) if text.endswith(x[:k])), default=0)
                    held, text = text[len(text) - hold:] if hold else "", text[:len(text) - hold]
                if len(text) > len(sent_text):
                    write(make_chunk(text[len(sent_text):], first))
                    sent_text, first = text, False
            if "error" in result:
                write({"error": {"message": str(result["error"]), "type": "server_error"}})
            else:
                if not stopped and held:                    # what was kept back turned out not to be a stop string
                    write(make_chunk(held, first))
                limit = getattr(self.backend, "max_new_tokens", None)
                asked = min(max_tokens or limit or len(toks), limit or len(toks))
                write(finish_chunk("stop" if stopped or len(toks) < asked else "length"))
            write(b"[DONE]")
        finally:
            dt = time.perf_counter() - t0
            with self._lock:
                self._m["inflight"] -= 1
                self.requests_served += 1
                self._m["prompt_tokens"] += len(ids)
                self._m["completion_tokens"] += len(toks)
                self._m["lat_sum"] += dt
                self._m["lat_buckets"][next((i for i, le in enumerate(_LAT_BUCKETS) if dt <= le), len(_LAT_BUCKETS))] += 1

    def _models(self) -> dict:
        return {"status": "ok", "model": self.model_name, "object": "list",
                "data": [{"id": self.model_name, "object": "model"}]}

    # ------------------------------------------------------------------ generation
    def _generate(self, prompt, body: dict) -> dict:
        """`prompt`: text, or token ids (then nothing is tokenised here and the caller's ids reach the engine as is)."""
        ids = self.tokenizer.encode(prompt) if isinstance(prompt, str) else [int(t) for t in prompt]
        if not ids:
            raise _BadRequest("empty prompt")
        max_tokens = body.get("max_tokens")
        if max_tokens is not None and (not isinstance(max_tokens, int) or max_tokens < 1):
            raise _BadRequest("max_tokens must be a positive integer")
        limit = getattr(self.backend, "max_new_tokens", None)
        t0 = time.perf_counter()
        with self._lock:
            self._m["inflight"] += 1
        try:
            toks, lps = self._call_backend(ids, max_tokens, body)
        finally:
            with self._lock:
                self._m["inflight"] -= 1
        dt = time.perf_counter() - t0
        toks = [int(t) for t in toks]
        asked = min(max_tokens or limit or len(toks), limit or len(toks))
        with self._lock:
            self.requests_served += 1
            self._m["prompt_tokens"] += len(ids)
            self._m["completion_tokens"] += len(toks)
            self._m["lat_sum"] += dt
            self._m["lat_buckets"][next((i for i, le in enumerate(_LAT_BUCKETS) if dt <= le), len(_LAT_BUCKETS))] += 1
        return {"text": self.tokenizer.decode(toks), "tokens": toks, "prompt_tokens": len(ids),
                "logprobs": [float(x) for x in lps] if body.get("logprobs") and lps is not None else None,
                "finish_reason": "length" if len(toks) >= asked else "stop"}

    def _call_backend(self, ids, max_tokens, body):
        if getattr(self.backend, "routes", False):          # several engines: the key keeps a conversation on one of them
            return self.backend.generate(ids, max_tokens, timeout=self.request_timeout, route_key=body.get("route_key"))
        try:
            return self.backend.generate(ids, max_tokens, timeout=self.request_timeout)
        except TypeError:                                   # a back end without the timeout argument
            return self.backend.generate(ids, max_tokens)

    def _usage(self, results: Sequence[dict]) -> dict:
        p, c = sum(r["prompt_tokens"] for r in results), sum(len(r["tokens"]) for r in results)
        return {"prompt_tokens": p, "completion_tokens": c, "total_tokens": p + c}

    def _many(self, prompts: Sequence[str], body: dict) -> list:
        if len(prompts) == 1:
            return [self._generate(prompts[0], body)]
        out: list = [None] * len(prompts)                   # several prompts of one request run side by side
        errs: list = []

        def run(i):
            try:
                out[i] = self._generate(prompts[i], body)
            except BaseException as e:
                errs.append(e)
        threads = [threading.Thread(target=run, args=(i,)) for i in range(len(prompts))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errs:
            raise errs[0]
        return out

    @staticmethod
    def _n(body: dict) -> int:
        n = body.get("n", 1)
        if isinstance(n, bool) or not isinstance(n, int) or not 1 <= n <= 64:
            raise _BadRequest("n must be an integer between 1 and 64")
        return n

    @staticmethod
    def _apply_stop(result: dict, body: dict) -> dict:
        """Cut the text at the first stop string (the tokens and their count stay what the engine produced)."""
        stop = body.get("stop")
        if stop is None:
            return result
        stops = [stop] if isinstance(stop, str) else stop
        if not isinstance(stops, list) or not all(isinstance(x, str) and x for x in stops):
            raise _BadRequest("stop must be a non-empty string or a list of them")
        cut = min((i for i in (result["text"].find(x) for x in stops) if i >= 0), default=-1)
        if cut >= 0:
            result = dict(result, text=result["text"][:cut], finish_reason="stop")
        return result

    def _completions(self, h, body: dict) -> None:
        prompt = body.get("prompt")
        is_ids = lambda p: isinstance(p, list) and p and all(isinstance(t, int) and not isinstance(t, bool) for t in p)
        prompts = [prompt] if isinstance(prompt, str) or is_ids(prompt) else prompt
        if not isinstance(prompts, list) or not prompts or not all(isinstance(p, str) or is_ids(p) for p in prompts):
            raise _BadRequest("prompt must be a string, a list of token ids, or a list of either")
        n = self._n(body)
        self._apply_stop({"text": ""}, body)                # validate before generating
        rid, now = "cmpl-" + uuid.uuid4().hex, int(time.time())
        base = {"id": rid, "object": "text_completion", "created": now, "model": body.get("model") or self.model_name}
        if body.get("stream") and self._can_stream_live(len(prompts), n):
            self._stream_live(h, prompts[0], body,
                              lambda piece, first: dict(base, choices=[{"index": 0, "text": piece, "finish_reason": None}]),
                              lambda reason: dict(base, choices=[{"index": 0, "text": "", "finish_reason": reason}]))
            return
        results = [self._apply_stop(r, body) for r in self._many([p for p in prompts for _ in range(n)], body)]
        choices = [{"index": i, "text": r["text"], "finish_reason": r["finish_reason"],
                    "logprobs": {"token_logprobs": r["logprobs"], "tokens": r["tokens"]} if r["logprobs"] else None}
                   for i, r in enumerate(results)]
        if body.get("stream"):
            self._send_sse(h, [dict(base, choices=[c]) for c in choices])
        else:
            self._send_json(h, 200, dict(base, choices=choices, usage=self._usage(results), sampling=self.sampling))

    def _chat(self, h, body: dict) -> None:
        messages = body.get("messages")
        if not isinstance(messages, list) or not messages:
            raise _BadRequest("messages must be a non-empty list")
        msgs = []
        for m in messages:
            if not isinstance(m, dict) or "content" not in m:
                raise _BadRequest("every message needs a role and a content")
            msgs.append({"role": m.get("role", "user"), "content": m["content"]})
        prompt = self.chat_parser.parse(msgs, add_generation_prompt=True, is_first_msg=True)
        n = self._n(body)
        self._apply_stop({"text": ""}, body)
        rid, now = "chatcmpl-" + uuid.uuid4().hex, int(time.time())
        model = body.get("model") or self.model_name
        if body.get("stream") and self._can_stream_live(1, n):
            base = {"id": rid, "object": "chat.completion.chunk", "created": now, "model": model}
            self._stream_live(h, prompt, body,
                              lambda piece, first: dict(base, choices=[{"index": 0, "finish_reason": None, "delta": (
                                  {"role": "assistant", "content": piece} if first else {"content": piece})}]),
                              lambda reason: dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": reason}]))
            return
        results = [self._apply_stop(x, body) for x in self._many([prompt] * n, body)]
        r = results[0]
        if body.get("stream"):
            base = {"id": rid, "object": "chat.completion.chunk", "created": now, "model": model}
            self._send_sse(h, [
                dict(base, choices=[{"index": 0, "delta": {"role": "assistant", "content": r["text"]}, "finish_reason": None}]),
                dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": r["finish_reason"]}])])
            return
        self._send_json(h, 200, {
            "id": rid, "object": "chat.completion", "created": now, "model": model,
            "choices": [{"index": i, "message": {"role": "assistant", "content": x["text"]}, "finish_reason": x["finish_reason"]}
                        for i, x in enumerate(results)],
            "usage": self._usage(results), "sampling": self.sampling})


class PooledBackend:
    """Several engine servers (one per GPU or per replica) behind one front end. A request's `route_key` (JSON field
    or `x-route-key` header; the reference's server takes the same two, serve_vllm_sampler.py:229) pins it to one
    engine through `experimental.worker.routing.RoutingPool`; requests without a key go to the least loaded engine."""
    routes = True

    def __init__(self, engines: dict):
        from ..experimental.worker.routing import RoutingPool
        self.engines = dict(engines)
        self.pool = RoutingPool(self.engines, call=lambda e, r: e.generate(r["ids"], r["max_tokens"], timeout=r["timeout"],
                                                                           **({"on_tokens": r["on_tokens"]} if r.get("on_tokens") else {})))
        self.streams = all(getattr(e, "streams", False) for e in self.engines.values())
        limits = [getattr(e, "max_new_tokens", None) for e in self.engines.values()]
        self.max_new_tokens = min(x for x in limits if x is not None) if any(x is not None for x in limits) else None

    def generate(self, ids, max_tokens=None, timeout=None, route_key=None, on_tokens=None):
        try:
            return self.pool.submit({"ids": ids, "max_tokens": max_tokens, "timeout": timeout, "route_key": route_key,
                                     "on_tokens": on_tokens})
        except Exception as e:
            raise RuntimeError(str(e)) from e


def serve(engine_server, tokenizer, **kwargs: Any) -> OpenAIServer:
    """Put the HTTP front end on a running `EngineServer`; its sampling parameters are the ones echoed to clients."""
    t, p, k, seed = getattr(engine_server, "_sampling", (None, None, None, None))
    kwargs.setdefault("sampling", {"temperature": t, "top_p": p, "top_k": k, "seed": seed})
    return OpenAIServer(engine_server, tokenizer, **kwargs)
