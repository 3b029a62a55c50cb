"""More of the dense sampler's contract (test model: the behaviours covered by tests/generate/sampler_test.py):
argument checks, token-id prompts, prompt truncation bucket, top-k support, forbidden tokens over a whole sequence,
several stop tokens, returned logits, batch independence, cache bounds, beam bookkeeping."""
import numpy as np
import pytest
import torch

from tests.test_sampler_cpu import CharTok, _sampler


def test_argument_checks():
    _, s = _sampler()
    with pytest.raises(ValueError, match="exactly one"):
        s(max_generation_steps=2)
    with pytest.raises(ValueError, match="exactly one"):
        s(["a"], max_generation_steps=2, prompt_token_ids=[[5]])
    with pytest.raises(ValueError, match="exceeds cache size"):
        s(["a" * 10], max_generation_steps=60)
    out = s("single string", max_generation_steps=2, eos_tokens=[63])           # a bare string is one prompt
    assert len(out.tokens) == 1 and len(out.text) == 1


def test_token_id_prompts_equal_string_prompts():
    _, s = _sampler()
    a = s(["hello", "hi"], max_generation_steps=5, eos_tokens=[63], return_logprobs=True)
    ids = [s.tokenize("hello").tolist(), s.tokenize("hi").tolist()]
    b = s(prompt_token_ids=ids, max_generation_steps=5, eos_tokens=[63], return_logprobs=True)
    for x, y, lx, ly in zip(a.tokens, b.tokens, a.logprobs, b.logprobs):
        assert np.array_equal(x, y) and np.allclose(lx, ly, atol=1e-6)
    assert a.padded_prompt_tokens.shape[1] == 8                                 # next power of two of the longest prompt (+ bos)
    c = s(["hello", "hi"], max_generation_steps=5, eos_tokens=[63], max_prompt_length=16)
    assert c.padded_prompt_tokens.shape[1] == 16 and np.array_equal(c.tokens[0], a.tokens[0])    # the bucket does not change the result


def test_batch_rows_do_not_influence_each_other():
    _, s = _sampler()
    alone = s(["hello"], max_generation_steps=6, eos_tokens=[63], return_logprobs=True)
    batch = s(["x", "hello", "a much longer prompt"], max_generation_steps=6, eos_tokens=[63], return_logprobs=True)
    assert np.array_equal(alone.tokens[0], batch.tokens[1]) and np.allclose(alone.logprobs[0], batch.logprobs[1], atol=1e-4)


def test_top_k_restricts_the_support_and_k1_is_greedy():
    model, s = _sampler()
    greedy = s(["abc"], max_generation_steps=6, eos_tokens=[63])
    k1 = s(["abc"], max_generation_steps=6, temperature=1.5, top_k=1, seed=3, eos_tokens=[63])
    assert np.array_equal(greedy.tokens[0], k1.tokens[0])
    ids = s.tokenize("abc").tolist()
    with torch.no_grad():
        top3 = set(torch.topk(model(torch.tensor([ids]))[0][0, -1].float(), 3).indices.tolist())
    firsts = {int(s(["abc"], max_generation_steps=1, temperature=2.0, top_k=3, seed=i, eos_tokens=[63]).tokens[0][0]) for i in range(40)}
    assert firsts <= top3 and len(firsts) > 1


def test_temperature_sharpens_towards_greedy():
    _, s = _sampler()
    greedy = int(s(["abc"], max_generation_steps=1, eos_tokens=[63]).tokens[0][0])
    cold = [int(s(["abc"], max_generation_steps=1, temperature=0.01, seed=i, eos_tokens=[63]).tokens[0][0]) for i in range(10)]
    hot = {int(s(["abc"], max_generation_steps=1, temperature=5.0, seed=i, eos_tokens=[63]).tokens[0][0]) for i in range(30)}
    assert all(t == greedy for t in cold) and len(hot) > 5


def test_forbidden_tokens_never_appear_and_logprobs_stay_finite():
    _, s = _sampler()
    free = s(["zz"], max_generation_steps=10, temperature=1.0, seed=0, eos_tokens=[63])
    banned = sorted(set(int(t) for t in free.tokens[0]))[:3]
    out = s(["zz"], max_generation_steps=10, temperature=1.0, seed=0, eos_tokens=[63], forbidden_tokens=banned, return_logprobs=True)
    assert not set(int(t) for t in out.tokens[0]) & set(banned) and np.isfinite(out.logprobs[0]).all()


def test_any_of_several_stop_tokens_ends_a_row_and_rows_end_independently():
    _, s = _sampler()
    base = s(["aa", "bbbb"], max_generation_steps=8, eos_tokens=[63])
    stop0, stop1 = int(base.tokens[0][2]), int(base.tokens[1][4])
    out = s(["aa", "bbbb"], max_generation_steps=8, eos_tokens=[stop0, stop1, 63])
    for i, row in enumerate(out.tokens):
        hits = [k for k, t in enumerate(base.tokens[i]) if int(t) in (stop0, stop1)]
        assert len(row) == hits[0] + 1 and int(row[-1]) in (stop0, stop1)      # ends at its first stop token, which is kept
    padded = s(["aa", "bbbb"], max_generation_steps=8, eos_tokens=[stop0, stop1, 63], pad_output=True)
    assert all(len(r) == 8 for r in padded.tokens) and int(padded.tokens[0][-1]) == CharTok().pad_id()


def test_returned_logits_match_the_chosen_tokens():
    _, s = _sampler()
    out = s(["hello"], max_generation_steps=4, eos_tokens=[63], return_logits=True, return_logprobs=True)
    logits = np.asarray(out.logits[0])
    assert logits.shape == (4, 64)
    assert np.array_equal(logits.argmax(-1), out.tokens[0])                    # greedy: the arg-max of what was returned
    lp = torch.log_softmax(torch.from_numpy(logits).float(), -1).numpy()
    assert np.allclose(lp[np.arange(4), out.tokens[0]], out.logprobs[0], atol=1e-4)


def test_beam_search_returns_one_row_per_prompt_and_respects_the_limit():
    _, s = _sampler()
    out = s(["hello", "hi"], max_generation_steps=5, beam_size=3, eos_tokens=[63])
    assert len(out.tokens) == 2 and all(1 <= len(t) <= 5 for t in out.tokens)
    again = s(["hello", "hi"], max_generation_steps=5, beam_size=3, eos_tokens=[63])
    assert all(np.array_equal(a, b) for a, b in zip(out.tokens, again.tokens))  # deterministic
    one = s(["hello"], max_generation_steps=5, beam_size=1, eos_tokens=[63])
    greedy = s(["hello"], max_generation_steps=5, eos_tokens=[63])
    assert np.array_equal(one.tokens[0], greedy.tokens[0])                     # a beam of one is greedy decoding
