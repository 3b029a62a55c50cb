"""The GSM8K "VTC" recipe in one place: prompt, graded reward, rollout metrics, raw-text prompting
(tunix/utils/gsm8k_vtc.py:17-253).

* `VTC_PROMPT_TEMPLATE` ends by OPENING `<reasoning>`; it is fed to the model verbatim (`VTCRawTextParser`), so the
  model continues the block. `is_vtc_format_correct` therefore asks the completion for exactly one `</reasoning>`
  followed by exactly one `<answer>…</answer>`, and does not ask for the opening tag.
* Reward: 1.0 format + right answer, 0.5 right answer without the format, 0.1 format only, 0.0 otherwise.
"""
from __future__ import annotations

import logging
import re
from typing import Any, Optional, Tuple

import numpy as np

from ..examples.data._records import normalize_record as normalize_single_example  # noqa: F401 (part of the recipe's API)
from ..examples.data._records import normalize_value as normalize_example_value
from ..rl.agentic.parser import chat_template_parser as _parsers

log = logging.getLogger(__name__)

VTC_PROMPT_TEMPLATE = """Solve the following math problem.
First, put your detailed step-by-step reasoning process inside <reasoning>...</reasoning> tags.
Then, put your final numerical answer inside <answer>\\boxed{{}}</answer> tags. Do not put anything else in the answer tags.

Problem: {}
<reasoning>
"""


def as_text(value: Any) -> str:
    v = normalize_example_value(value)
    return v if isinstance(v, str) else str(v)


def extract_hash_answer(text: str) -> Optional[str]:
    return text.split("####", 1)[1].strip() if "####" in text else None


def build_prompt(question: str) -> str:
    return VTC_PROMPT_TEMPLATE.format(question)


def extract_boxed_answer(text: str) -> Optional[str]:
    r"""The last `\boxed{…}` (braces may nest) of the last `<answer>` block, or of the whole text when there is no
    block; `\boxed 42` without braces is accepted as a fallback."""
    blocks = re.findall(r"<answer>(.*?)</answer>", text, re.DOTALL)
    content = blocks[-1] if blocks else text
    found, opens = [], []
    for i, ch in enumerate(content):
        if ch == "{":
            opens.append(i)
        elif ch == "}" and opens:
            j = opens.pop()
            if content[:j].endswith(r"\boxed"):
                found.append(content[j + 1:i].strip())
    if found:
        return found[-1]
    m = re.search(r"\\boxed\s*\{?\s*([a-zA-Z0-9\.,\-]+)\s*\}?", content)
    return m.group(1).strip() if m else None


def is_vtc_format_correct(text: str) -> bool:
    if text.count("</reasoning>") != 1 or text.count("<answer>") != 1 or text.count("</answer>") != 1:
        return False
    return text.find("</reasoning>") < text.find("<answer>") < text.find("</answer>")


def normalize_answer(text: Any) -> Optional[str]:
    return None if text is None else str(text).replace(",", "").strip()


def vtc_completion_outcome(completion: str, gold: Any) -> Tuple[float, bool, bool, bool]:
    """(score, format_ok, answer_ok, extracted_ok)."""
    format_ok = is_vtc_format_correct(completion)
    pred, true = normalize_answer(extract_boxed_answer(completion)), normalize_answer(normalize_example_value(gold))
    answer_ok = pred is not None and true is not None and pred == true
    score = {(True, True): 1.0, (True, False): 0.1, (False, True): 0.5, (False, False): 0.0}[(format_ok, answer_ok)]
    return score, format_ok, answer_ok, pred is not None


def vtc_env_reward(task: dict, action: Any) -> float:
    """Environment reward: the action's text against the task's `answer` (or `gold_answer`)."""
    gold = task.get("answer", task.get("gold_answer"))
    return vtc_completion_outcome(str(getattr(action, "action", action)), gold)[0]


def vtc_reward_fn(prompts, completions, answer, **kwargs) -> list:
    """The same grading in the batched reward-function signature of the GRPO learners."""
    return [vtc_completion_outcome(str(c), a)[0] for c, a in zip(completions, answer)]


def vtc_metric_fn(prompts, completions, rewards, advantages, answer=None, **kwargs) -> dict:
    """Per-group rollout metrics, `{name: (value, aggregation)}`; "solved" = reward above the format-only tier."""
    r = np.asarray(rewards, np.float32)
    solve_all, solve_none = bool(np.all(r > 0.1)), bool(np.all(np.isclose(r, 0.0)))
    ratio = float(np.mean(r > 0.1))
    log.info("[rollout-metric] n=%d solve_ratio=%.3f reward_mean=%.3f reward_max=%.3f", len(r), ratio, float(r.mean()), float(r.max()))
    return {"rewards/solve_all": (int(solve_all), np.mean), "rewards/solve_none": (int(solve_none), np.mean),
            "rewards/solve_partial": (int(not solve_all and not solve_none), np.mean), "rewards/solve_ratio": (ratio, np.mean)}


VTCRawTextParser = _parsers.RawTextParser
