"""GSM8K-style rewards: format adherence and final-answer correctness (role of tunix/cli/reward_fn/gsm8k.py)."""
import re

_ANS = re.compile(r"<answer>\s*(.*?)\s*</answer>", re.S)
_NUM = re.compile(r"-?\d[\d,]*\.?\d*")


def _final_number(text: str):
    m = _ANS.search(text)
    src = m.group(1) if m else text
    nums = _NUM.findall(src.replace("$", ""))
    return nums[-1].replace(",", "").rstrip(".") if nums else None


def answer_reward(prompts, completions, answer=None, **kwargs):
    """1.0 for the right final number, 0.1 for a well-formed but wrong answer, else 0."""
    out = []
    for i, c in enumerate(completions):
        got = _final_number(c)
        gold = None if answer is None else str(answer[i]).replace(",", "").strip()
        if got is not None and gold is not None:
            try:
                out.append(1.0 if abs(float(got) - float(gold)) < 1e-6 else 0.1)
                continue
            except ValueError:
                pass
        out.append(0.1 if got is not None and _ANS.search(c) else 0.0)
    return out


def format_reward(prompts, completions, **kwargs):
    return [0.5 if re.search(r"<reasoning>.*?</reasoning>\s*<answer>.*?</answer>", c, re.S) else 0.0 for c in completions]
