"""Binary format and answer rewards for `<reasoning>…</reasoning><answer>…</answer>` completions
(tunix/cli/reward_fn/simple_math.py:24-76): `check_format` pays `r` for a completion of exactly that shape,
`check_answer` pays `r` when the first number after `<answer>` equals the reference answer as a float."""
import re

reasoning_start, reasoning_end = "<reasoning>", "</reasoning>"
solution_start, solution_end = "<answer>", "</answer>"

match_format = re.compile(rf"^\s*{reasoning_start}.+?{reasoning_end}.*?{solution_start}(.+?){solution_end}\s*$",
                          flags=re.MULTILINE | re.DOTALL)
_first_number = re.compile(rf"{solution_start}.*?([\d\.]+)", flags=re.MULTILINE | re.DOTALL)


def check_format(prompts, completions, r=0.1, **kwargs):
    return [0 if match_format.search(c) is None else r for c in completions]


def check_answer(prompts, completions, answer, r=1, **kwargs):
    out = []
    for c, gold in zip(completions, answer):
        m = _first_number.search(c)
        if m is None:
            out.append(0)
            continue
        try:
            out.append(r if float(m.group(1).strip()) == float(str(gold).strip()) else 0.0)
        except ValueError:
            out.append(0)
    return out
