"""English → French translation as supervised fine-tuning data (tunix/examples/data/translation_dataset.py:24-209).

Each record becomes `prefix + source + suffix` (no loss) followed by the target with EOS (loss), padded to
`max_target_length`; records that do not fit are dropped, batches are full (the remainder is dropped). Records are
either MTNT-style `{"src": ..., "dst": ...}` or OPUS-100-style `{"translation": {"en": ..., "fr": ...}}`."""
from __future__ import annotations

from typing import Iterable, Iterator, Optional, Tuple

import numpy as np

from ...sft.peft_trainer import TrainingInput
from . import _records

INPUT_TEMPLATE = {"prefix": "Translate this into French:\n", "suffix": "\n"}
INPUT_TEMPLATE_IT = {"prefix": "<start_of_turn>user\nTranslate this into French:\n",
                     "suffix": "\n<end_of_turn>\n<start_of_turn>model\n"}


def _pair(rec: dict) -> Tuple[str, str]:
    if "src" in rec:
        return str(rec["src"]), str(rec["dst"])
    if "translation" in rec:
        return str(rec["translation"]["en"]), str(rec["translation"]["fr"])
    raise KeyError(f"translation record needs 'src'/'dst' or 'translation': {sorted(rec)}")


def build_train_input(src_tokens, dst_tokens, max_seq_len: int, pad_id: int) -> Optional[TrainingInput]:
    """One unbatched example, or None when source + target exceed `max_seq_len`."""
    src, dst = np.asarray(src_tokens, np.int32), np.asarray(dst_tokens, np.int32)
    n = len(src) + len(dst)
    if n > max_seq_len:
        return None
    tokens = np.full(max_seq_len, pad_id, np.int32)
    tokens[:n] = np.concatenate([src, dst])
    mask = np.zeros(max_seq_len, bool)
    mask[len(src):n] = True                                   # the loss sees the translation only
    return TrainingInput(input_tokens=tokens, input_mask=mask)


class _Loader:
    """Re-iterable: every `iter()` walks the epochs again (`num_epochs=None` repeats for ever)."""

    def __init__(self, records, batch_size, num_epochs, max_seq_len, tokenizer, template):
        self.records, self.batch_size, self.num_epochs = records, batch_size, num_epochs
        self.max_seq_len, self.tokenizer, self.template = max_seq_len, tokenizer, template

    def _examples(self) -> Iterator[TrainingInput]:
        epoch = 0
        while self.num_epochs is None or epoch < self.num_epochs:
            for rec in self.records:
                src, dst = _pair(rec)
                ex = build_train_input(
                    self.tokenizer.tokenize(src, prefix=self.template["prefix"], suffix=self.template["suffix"], add_eos=False),
                    self.tokenizer.tokenize(dst, add_eos=True), self.max_seq_len, self.tokenizer.pad_id())
                if ex is not None:
                    yield ex
            epoch += 1

    def __iter__(self) -> Iterator[TrainingInput]:
        rows = []
        for ex in self._examples():
            rows.append(ex)
            if len(rows) == self.batch_size:
                yield TrainingInput(input_tokens=np.stack([r.input_tokens for r in rows]),
                                    input_mask=np.stack([r.input_mask for r in rows]))
                rows = []


def create_datasets(dataset_name, global_batch_size: int, max_target_length: int, num_train_epochs: Optional[int], tokenizer,
                    instruct_tuned: bool = False, input_template: Optional[dict] = None,
                    eval_dataset=None) -> Tuple[Iterable[TrainingInput], Iterable[TrainingInput]]:
    """(train, eval) iterables of `TrainingInput` batches. `dataset_name`: a directory with `train*` / `valid*` files,
    a file (then `eval_dataset` names the evaluation file, or the last 10 % are held out), or a hub name."""
    template = input_template or (INPUT_TEMPLATE_IT if instruct_tuned else INPUT_TEMPLATE)
    train = _records.load_records(dataset_name, "train")
    if eval_dataset is not None:
        evals = _records.load_records(eval_dataset, "valid")
    else:
        try:
            evals = _records.load_records(dataset_name, "valid")
        except Exception:
            evals = None
        if evals is None or evals == train:
            cut = max(1, int(len(train) * 0.9))
            train, evals = train[:cut], train[cut:]
    mk = lambda recs, epochs: _Loader(recs, global_batch_size, epochs, max_target_length, tokenizer, template)
    return mk(train, num_train_epochs), mk(evals, 1)
