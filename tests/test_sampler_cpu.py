"""Vanilla sampler behaviour on CPU with a tiny model and a character tokenizer."""
import numpy as np
import pytest
import torch

from tunix_b200.common.configs import CacheConfig
from tunix_b200.generate import sampling
from tunix_b200.generate.sampler import Sampler
from tunix_b200.models.config import ModelConfig
from tunix_b200.models.transformer import create_model


class CharTok:
    def encode(self, s):
        return [3 + (ord(c) % 60) for c in s]

    def decode(self, ids):
        return "".join(chr(97 + (int(i) % 26)) for i in ids)

    def bos_id(self):
        return 1

    def eos_id(self):
        return 2

    def pad_id(self):
        return 0


def _sampler():
    cfg = ModelConfig.tiny_llama().replace(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=2,
                                           head_dim=16, num_kv_heads=1)
    model = create_model(cfg, seed=0)
    return model, Sampler(model, CharTok(), CacheConfig(cache_size=64, num_layers=2, num_kv_heads=1, head_dim=16))


def test_greedy_matches_full_recompute_and_is_padding_invariant():
    model, s = _sampler()
    out = s(["hello", "hi"], max_generation_steps=6, return_logprobs=True, eos_tokens=[63])
    # recompute greedily without a cache, one prompt at a time (no padding)
    for i, prompt in enumerate(["hello", "hi"]):
        ids = s.tokenize(prompt).tolist()
        for step in range(6):
            logits, _ = model(torch.tensor([ids]))
            nxt = int(logits[0, -1].argmax())
            assert nxt == int(out.tokens[i][step]), (i, step)
            lp = torch.log_softmax(logits[0, -1].float(), -1)[nxt].item()
            assert abs(lp - out.logprobs[i][step]) < 1e-4
            ids.append(nxt)


def test_sampling_is_reproducible_per_seed_and_step():
    _, s = _sampler()
    a = s(["abc"], max_generation_steps=8, temperature=1.0, top_p=0.9, top_k=20, seed=7, eos_tokens=[63])
    b = s(["abc"], max_generation_steps=8, temperature=1.0, top_p=0.9, top_k=20, seed=7, eos_tokens=[63])
    c = s(["abc"], max_generation_steps=8, temperature=1.0, top_p=0.9, top_k=20, seed=8, eos_tokens=[63])
    assert np.array_equal(a.tokens[0], b.tokens[0])
    assert not np.array_equal(a.tokens[0], c.tokens[0])


def test_eos_stops_and_pad_output_and_echo():
    model, s = _sampler()
    first = int(s(["zz"], max_generation_steps=1, eos_tokens=[63]).tokens[0][0])
    out = s(["zz"], max_generation_steps=5, eos_tokens=[first], pad_output=True, echo=True)
    row = out.tokens[0]
    assert row.shape[0] == 5 + out.padded_prompt_tokens.shape[1]
    assert first in row.tolist()
    forb = s(["zz"], max_generation_steps=1, forbidden_tokens=[first], eos_tokens=[63])
    assert int(forb.tokens[0][0]) != first


def test_top_p_filter_keeps_minimal_prefix():
    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    z = sampling.filter_logits(logits, 1.0, 0.7, None)
    assert torch.isinf(z[0, 2]) and torch.isinf(z[0, 3]) and not torch.isinf(z[0, 1])
    z = sampling.filter_logits(logits, 1.0, None, 1)
    assert torch.isinf(z[0, 1:]).all()


def test_beam_search_finds_higher_score_than_greedy():
    model, s = _sampler()
    g = s(["hey"], max_generation_steps=5, eos_tokens=[63])
    b = s(["hey"], max_generation_steps=5, beam_size=4, eos_tokens=[63])

    def score(tokens):
        ids = s.tokenize("hey").tolist()
        tot = 0.0
        for t in tokens:
            logits, _ = model(torch.tensor([ids]))
            tot += torch.log_softmax(logits[0, -1].float(), -1)[int(t)].item()
            ids.append(int(t))
        return tot
    assert score(b.tokens[0]) >= score(g.tokens[0]) - 1e-5


def test_update_params_copies_lora_only():
    model, s = _sampler()
    name, p = next(iter(model.named_parameters()))
    s.update_params({name: torch.zeros_like(p)})
    assert float(dict(model.named_parameters())[name].abs().sum()) == 0.0


class _FakeEngine:
    """Stands in for PagedEngine under EngineServer: `_loop` serves the request source with a scripted model
    (token = last prompt token + step), one request per slot and step, so the server's queueing, token limits,
    pause / resume and failure hand-off run on the CPU."""

    def __init__(self, slots=2, fail_on=None):
        import torch
        self.cache_size, self.max_running, self.pack_weights, self._packed_on = 64, slots, False, False
        self.tokenizer, self.device = CharTok(), torch.device("cpu")
        self.refreshed, self.fail_on = 0, fail_on

    def _fuse_all(self):
        self.refreshed += 1

    def _pack_all(self):
        pass

    def _new_state(self, *a):
        return {}

    def _loop(self, st, B, max_steps, pad_id, source):
        import time
        running = {}
        while True:
            for rid, row, ln, lim in source.take(B - len(running)):
                if self.fail_on is not None and int(row[-1]) == self.fail_on:
                    raise RuntimeError("device fault")
                running[rid] = (int(row[-1]), lim, [])
            if not running:
                if source.idle():
                    continue
                return
            time.sleep(0.002)
            for rid in list(running):
                last, lim, out = running[rid]
                out.append(last + len(out) + 1)
                if getattr(source, "streaming", False) and len(out) < lim:
                    source.progress(rid, out, [0.0] * len(out))
                if len(out) >= lim:
                    source.deliver(rid, out, [0.0] * len(out))
                    del running[rid]


def test_engine_server_protocol_on_cpu():
    from concurrent.futures import ThreadPoolExecutor
    from tunix_b200.generate.engine import EngineServer
    eng = _FakeEngine(slots=2)
    with EngineServer(eng, max_new_tokens=5, max_prompt_length=8, eos_tokens=[2]) as srv:
        with ThreadPoolExecutor(6) as ex:
            outs = list(ex.map(lambda i: srv.generate([1, 10 * i], max_tokens=1 + i % 5, timeout=10), range(1, 9)))
        for i, (toks, lps) in zip(range(1, 9), outs):
            assert toks.tolist() == [10 * i + k + 1 for k in range(1 + i % 5)] and len(lps) == len(toks)
        assert srv.generate(list(range(100, 120)), 2, timeout=10)[0].tolist() == [120, 121]   # prompt cut to its tail
        assert srv.generate([1, 7], max_tokens=99, timeout=10)[0].shape == (5,)               # capped at the server's limit
        before = eng.refreshed
        assert srv.pause(timeout=5)
        fut = srv.submit([1, 3], 2)
        import time
        time.sleep(0.05)
        assert not fut.done()                       # queued, not admitted while paused
        srv.resume()
        assert fut.result(10)[0].tolist() == [4, 5] and eng.refreshed == before + 1          # weights re-read once
    with pytest.raises(RuntimeError):
        srv.submit([1])
    # a failure of the engine loop reaches every waiting client and closes the server
    bad = EngineServer(_FakeEngine(slots=1, fail_on=13), max_new_tokens=4, max_prompt_length=8, eos_tokens=[2])
    ok = bad.submit([1, 5], 2)
    assert ok.result(10)[0].tolist() == [6, 7]
    f1, f2 = bad.submit([1, 13], 2), bad.submit([1, 6], 2)
    with pytest.raises(RuntimeError, match="device fault"):
        f1.result(10)
    with pytest.raises(RuntimeError):
        f2.result(10)
    with pytest.raises(RuntimeError):
        bad.submit([1, 2])
    bad.close()


def test_engine_server_reports_tokens_while_a_request_runs():
    from tunix_b200.generate.engine import EngineServer
    with EngineServer(_FakeEngine(slots=2), max_new_tokens=6, max_prompt_length=8, eos_tokens=[2]) as srv:
        pieces, other = [], []
        fut = srv.submit([1, 20], 5, on_tokens=lambda t, l: pieces.append((t.tolist(), len(l))))
        quiet = srv.submit([1, 40], 3)                                   # a request without a listener beside it
        toks, _ = fut.result(10)
        assert quiet.result(10)[0].tolist() == [41, 42, 43]
        assert [t for p, _ in pieces for t in p] == toks.tolist() == [21, 22, 23, 24, 25]
        assert len(pieces) >= 3 and all(len(p) == n for p, n in pieces)      # arrived in several pieces, none repeated
        assert not srv.streaming                                             # the listener is gone with its request
        bad = srv.submit([1, 60], 3, on_tokens=lambda t, l: 1 / 0)           # a failing callback does not hurt the request
        assert bad.result(10)[0].tolist() == [61, 62, 63]


def _http(url, body=None):
    import json
    import urllib.error
    import urllib.request
    req = urllib.request.Request(url, data=None if body is None else json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=20) as r:
            return r.status, r.headers.get("Content-Type"), r.read()
    except urllib.error.HTTPError as e:
        return e.code, e.headers.get("Content-Type"), e.read()


def test_openai_style_http_front_end_over_the_engine_server():
    """Completions, chat, several prompts in one request, streaming and the error codes, over a real socket on the
    loop-back interface; the back end is the engine server driven by the scripted engine."""
    import json
    from concurrent.futures import ThreadPoolExecutor
    from tunix_b200.generate.engine import EngineServer
    from tunix_b200.generate.openai_server import serve
    tok = CharTok()
    with EngineServer(_FakeEngine(slots=4), max_new_tokens=6, max_prompt_length=32, eos_tokens=[2]) as eng:
        with serve(eng, tok, model_name="toy") as http:
            st, _, raw = _http(http.url + "/health")
            assert st == 200 and json.loads(raw)["data"][0]["id"] == "toy"
            last = tok.encode("hello")[-1]
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": "hello", "max_tokens": 3, "logprobs": True})
            out = json.loads(raw)
            want = [last + 1, last + 2, last + 3]
            assert st == 200 and out["object"] == "text_completion"
            assert out["choices"][0]["text"] == tok.decode(want) and out["choices"][0]["finish_reason"] == "length"
            assert out["choices"][0]["logprobs"]["tokens"] == want
            assert out["usage"] == {"prompt_tokens": 5, "completion_tokens": 3, "total_tokens": 8}
            assert out["sampling"]["temperature"] == 0.0
            # a list of prompts: one choice each, generated side by side
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": ["ab", "abc", "abcd"], "max_tokens": 2})
            ch = json.loads(raw)["choices"]
            assert [c["index"] for c in ch] == [0, 1, 2]
            assert [c["text"] for c in ch] == [tok.decode([tok.encode(p)[-1] + 1, tok.encode(p)[-1] + 2]) for p in ("ab", "abc", "abcd")]
            # chat: rendered by the template parser, answered as an assistant message
            msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
            st, _, raw = _http(http.url + "/v1/chat/completions", {"messages": msgs, "max_tokens": 4})
            out = json.loads(raw)
            prompt = http.chat_parser.parse(msgs, add_generation_prompt=True, is_first_msg=True)
            # the engine keeps the last 32 prompt tokens; the scripted model continues from the last one
            pl = tok.encode(prompt)[-1]
            assert st == 200 and out["choices"][0]["message"] == {"role": "assistant", "content": tok.decode([pl + k for k in range(1, 5)])}
            # streaming: server-sent events ending with [DONE]
            st, ctype, raw = _http(http.url + "/v1/chat/completions", {"messages": msgs, "max_tokens": 2, "stream": True})
            events = [e[len("data: "):] for e in raw.decode().strip().split("\n\n")]
            assert st == 200 and ctype == "text/event-stream" and events[-1] == "[DONE]"
            deltas = [json.loads(e)["choices"][0]["delta"] for e in events[:-2]]
            assert deltas[0]["role"] == "assistant" and all("role" not in d for d in deltas[1:])
            assert "".join(d["content"] for d in deltas) == tok.decode([pl + 1, pl + 2])
            assert json.loads(events[-2])["choices"][0] == {"index": 0, "delta": {}, "finish_reason": "length"}
            # a streamed completion arrives in pieces as the engine produces it; a stop string ends the stream early
            st, ctype, raw = _http(http.url + "/v1/completions", {"prompt": "hello", "max_tokens": 5, "stream": True})
            events = [e[len("data: "):] for e in raw.decode().strip().split("\n\n")]
            texts = [json.loads(e)["choices"][0]["text"] for e in events[:-2]]
            assert st == 200 and events[-1] == "[DONE]" and len(texts) >= 3
            assert "".join(texts) == tok.decode([last + k for k in range(1, 6)])
            assert json.loads(events[-2])["choices"][0] == {"index": 0, "text": "", "finish_reason": "length"}
            whole = "".join(texts)
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": "hello", "max_tokens": 5, "stream": True, "stop": whole[2:4]})
            events = [e[len("data: "):] for e in raw.decode().strip().split("\n\n")]
            assert "".join(json.loads(e)["choices"][0]["text"] for e in events[:-2]) == whole[:2]
            assert json.loads(events[-2])["choices"][0]["finish_reason"] == "stop"
            # text that only looks like the beginning of a stop string is delivered once it turns out not to be one
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": "hello", "max_tokens": 5, "stream": True, "stop": whole[-1] + "#"})
            events = [e[len("data: "):] for e in raw.decode().strip().split("\n\n")]
            assert "".join(json.loads(e)["choices"][0]["text"] for e in events[:-2]) == whole
            # concurrency on the wire becomes batch width in the engine
            with ThreadPoolExecutor(8) as ex:
                res = list(ex.map(lambda i: _http(http.url + "/v1/completions", {"prompt": "x" * (i + 1), "max_tokens": 2}), range(8)))
            assert all(r[0] == 200 for r in res) and http.requests_served >= 8
            with ThreadPoolExecutor(96) as ex:              # a burst of connections larger than a default listen backlog
                res = list(ex.map(lambda i: _http(http.url + "/v1/completions", {"prompt": "y" * (1 + i % 7), "max_tokens": 1}), range(192)))
            assert all(r[0] == 200 for r in res)
            # n samples per prompt (a GRPO group in one request) and stop strings
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": ["ab", "abc"], "max_tokens": 3, "n": 3})
            ch = json.loads(raw)["choices"]
            assert st == 200 and [c["index"] for c in ch] == list(range(6)) and ch[0]["text"] == ch[2]["text"] != ch[3]["text"]
            full = ch[0]["text"]
            st, _, raw = _http(http.url + "/v1/completions", {"prompt": "ab", "max_tokens": 3, "stop": [full[1:], "zzzz"]})
            c0 = json.loads(raw)["choices"][0]
            assert c0["text"] == full[:1] and c0["finish_reason"] == "stop" and json.loads(raw)["usage"]["completion_tokens"] == 3
            st, _, raw = _http(http.url + "/v1/chat/completions", {"messages": msgs, "max_tokens": 2, "n": 2})
            assert st == 200 and len(json.loads(raw)["choices"]) == 2 and json.loads(raw)["usage"]["completion_tokens"] == 4
            assert _http(http.url + "/v1/completions", {"prompt": "a", "n": 0})[0] == 400
            assert _http(http.url + "/v1/completions", {"prompt": "a", "stop": [""]})[0] == 400
            # errors
            assert _http(http.url + "/v1/completions", {"prompt": 5})[0] == 400
            assert _http(http.url + "/v1/completions", {"prompt": "a", "max_tokens": 0})[0] == 400
            assert _http(http.url + "/v1/chat/completions", {"messages": []})[0] == 400
            assert _http(http.url + "/v1/nothing", {})[0] == 404 and _http(http.url + "/nothing")[0] == 404
            eng.close()
            assert _http(http.url + "/v1/completions", {"prompt": "a"})[0] == 503    # engine gone: unavailable, not a hang
            st, ctype, raw = _http(http.url + "/metrics")
            text = raw.decode()
            assert st == 200 and ctype.startswith("text/plain")
            vals = {l.split(" ")[0]: float(l.split(" ")[1]) for l in text.splitlines() if l and not l.startswith("#")}
            assert vals["tunix_b200_http_requests_total"] == http.requests_served >= 14 + 192
            assert vals['tunix_b200_http_errors_total{status="400"}'] == 5 and vals['tunix_b200_http_errors_total{status="503"}'] == 1
            assert vals["tunix_b200_http_completion_tokens_total"] >= 3 + 6 + 4 + 2 + 16 and vals["tunix_b200_http_requests_in_flight"] == 0
            assert vals['tunix_b200_http_request_seconds_bucket{le="+Inf"}'] == vals["tunix_b200_http_request_seconds_count"] == http.requests_served


def test_openai_front_end_routes_conversations_over_several_engines():
    import json
    from tunix_b200.generate.engine import EngineServer
    from tunix_b200.generate.openai_server import OpenAIServer, PooledBackend
    tok = CharTok()
    engines = {f"gpu{i}": EngineServer(_FakeEngine(slots=2), max_new_tokens=4, max_prompt_length=16, eos_tokens=[2]) for i in range(3)}
    try:
        back = PooledBackend(engines)
        with OpenAIServer(back, tok, model_name="toy") as http:
            for conv in ("a", "b", "c", "d", "e"):
                owner = back.pool.owner(conv)
                before = engines[owner].admitted
                for turn in range(3):
                    st, _, raw = _http(http.url + "/v1/completions", {"prompt": "hi" * (turn + 1), "max_tokens": 2, "route_key": conv})
                    assert st == 200 and len(json.loads(raw)["choices"][0]["text"]) == 2
                assert engines[owner].admitted == before + 3                     # every turn reached the same engine
            for _ in range(6):                                                   # no key: spread over the engines
                assert _http(http.url + "/v1/completions", {"prompt": "x", "max_tokens": 1})[0] == 200
            assert all(s["served"] >= 2 for s in back.pool.stats().values())
            # streaming through the pool: pieces come from the engine the key belongs to
            owner = back.pool.owner("a")
            before = engines[owner].admitted
            st, ctype, raw = _http(http.url + "/v1/completions", {"prompt": "hi", "max_tokens": 4, "stream": True, "route_key": "a"})
            events = [e[len("data: "):] for e in raw.decode().strip().split("\n\n")]
            assert st == 200 and ctype == "text/event-stream" and len(events) >= 4 and events[-1] == "[DONE]"
            assert len("".join(json.loads(e)["choices"][0]["text"] for e in events[:-2])) == 4 and engines[owner].admitted == before + 1
            for e in engines.values():
                e.close()
            assert _http(http.url + "/v1/completions", {"prompt": "x"})[0] == 503
            assert _http(http.url + "/v1/completions", {"prompt": "x", "stream": True})[0] == 503     # also when a stream was asked for
    finally:
        for e in engines.values():
            e.close()
