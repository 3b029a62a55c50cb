"""Regex key mapping between checkpoint naming schemes (tunix/utils/torch_utils.py:5-27)."""
from __future__ import annotations

import re


def map_key(mapping: dict, source_key: str):
    """mapping: {regex: target} or {regex: (target, transform)}. Exactly one pattern must match the whole key;
    returns (target key with groups substituted, transform or None)."""
    hits = []
    for pat, tgt in mapping.items():
        m = re.fullmatch(pat, source_key)
        if m:
            transform = None
            if isinstance(tgt, tuple):
                tgt, transform = tgt
            hits.append((m.expand(tgt) if "\\" in tgt else tgt, transform))
    if len(hits) != 1:
        raise ValueError(f"{source_key!r} matched {len(hits)} patterns; exactly one is required")
    return hits[0]
