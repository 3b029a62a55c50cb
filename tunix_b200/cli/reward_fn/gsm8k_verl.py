"""GSM8K scoring in the style of the ReFT / verl recipes (tunix/cli/reward_fn/gsm8k_verl.py:17-120): the final answer is
the last `#### <number>` of the completion ("strict", which also checks the format) or its last number ("flexible");
only the last 300 characters are searched (regular expressions over very long completions are slow and the answer
sits at the end)."""
import re

_SOLUTION_CLIP_CHARS = 300
_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_FLEX = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(solution_str: str, method: str = "strict"):
    if method not in ("strict", "flexible"):
        raise ValueError("method must be 'strict' or 'flexible'")
    tail = solution_str[-_SOLUTION_CLIP_CHARS:]
    if method == "strict":
        found = _STRICT.findall(tail)
        return found[-1].replace(",", "").replace("$", "") if found else None
    for cand in reversed(_FLEX.findall(tail)):
        if cand not in ("", "."):
            return cand
    return None


def compute_score(solution_str: str, ground_truth: str, method: str = "strict", format_score: float = 0.0, score: float = 1.0):
    """`score` for the right answer, `format_score` for a well-formed wrong one, 0 without an answer."""
    answer = extract_solution(solution_str, method)
    if answer is None:
        return 0
    return score if answer == ground_truth else format_score


def reward_fn(prompts, completions, answer=None, method: str = "strict", format_score: float = 0.0, score: float = 1.0, **kwargs):
    """The same as a reward function over a batch (signature of the RL learners)."""
    golds = answer if answer is not None else [None] * len(completions)
    return [float(compute_score(c, str(g).replace(",", "").strip(), method, format_score, score)) if g is not None else 0.0
            for c, g in zip(completions, golds)]
