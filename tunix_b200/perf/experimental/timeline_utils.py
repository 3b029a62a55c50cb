"""Timeline ids and span post-processing (tunix/perf/experimental/timeline_utils.py:28-223).

Ids: `host-<thread id>` for host threads, `cuda<k>` for GPUs, `<id>_queue` for the lane that shows how long work
waited behind other work of its timeline."""
from __future__ import annotations

import logging
import threading
from typing import Mapping, Optional, Sequence

import numpy as np

from . import constants
from .timeline import Span, Timeline

log = logging.getLogger(__name__)


def generate_host_timeline_id() -> str:
    return f"host-{threading.get_ident()}"


def is_host_timeline(tl_id: str) -> bool:
    return tl_id.startswith("host-")


def generate_queued_timeline_id(tl_id: str) -> str:
    return f"{tl_id}_queue"


def is_queued_timeline(tl_id: str) -> bool:
    return tl_id.endswith("_queue")


def generate_device_timeline_id(device) -> str:
    """A string stays as it is; a rank or CUDA index becomes `cuda<k>`; a `torch.device` `cuda:<k>` likewise."""
    if isinstance(device, str):
        return device
    if isinstance(device, (int, np.integer)):
        return f"cuda{int(device)}"
    if hasattr(device, "type") and hasattr(device, "index"):
        return f"{device.type}{device.index if device.index is not None else 0}"
    if hasattr(device, "platform") and hasattr(device, "id"):
        return f"{device.platform}{device.id}"
    raise ValueError(f"Unsupported id type: {type(device)}")


def generate_device_timeline_ids(devices) -> list:
    if devices is None:
        return []
    if isinstance(devices, np.ndarray):
        devices = devices.flatten().tolist()
    return [generate_device_timeline_id(d) for d in devices]


def is_timeline_only_of_allowed_type(tl: Timeline, allowed_span_names: Sequence[str], include_cur_step: bool = False) -> bool:
    """True when the timeline has spans and every one of them carries an allowed name."""
    seen = False
    for step in (tl.all_steps if include_cur_step else tl.committed_steps):
        for s in step.values():
            seen = True
            if s.name not in allowed_span_names:
                return False
    return seen


def _copy(s: Span, name: str, begin: float, end: float, tags: Optional[Mapping]) -> Span:
    out = Span(name=name, begin=begin, id=s.id, parent_id=s.parent_id, tags=tags)
    out.end = end
    return out


def sequentialize_overlapping_spans(spans: Mapping[int, Span]):
    """(active, queue): spans of one timeline that overlap ran one after the other. The first keeps its times; one
    that began while its predecessor was active becomes active when the predecessor ended, and the wait before that is
    a `queue` span tagged with its name (queue spans do not overlap each other either). A span that lies entirely
    inside its predecessor's active time has no active time left and appears as a queue span only."""
    active: dict = {}
    queue: dict = {}
    cur_end = last_queue_end = float("-inf")
    for s in sorted(spans.values(), key=lambda x: (x.begin, x.id)):
        if s.begin < cur_end:
            a_begin, a_end = cur_end, max(cur_end, s.end)
            q_begin = max(s.begin, last_queue_end)
            if q_begin < a_begin:
                queue[s.id] = _copy(s, constants.QUEUE, q_begin, a_begin, {constants.NAME: s.name})
                last_queue_end = a_begin
        else:
            a_begin, a_end = s.begin, s.end
        if a_begin < a_end:
            active[s.id] = _copy(s, s.name, a_begin, a_end, dict(s.tags) if s.tags else None)
            cur_end = a_end
        else:
            log.warning("span %r lies inside another span's active time and is dropped from the active spans", s.name)
    return active, queue
