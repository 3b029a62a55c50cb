"""Spans as a tree (tunix/perf/span.py:28-320): `SpanGroup`s (a training step, a mini-batch, ...) hold spans and
further groups in order of time. The module gives the tree queries the exporters use (first / last / n-th / all
inner groups of a name, over one group or a batch of groups, e.g. one per rank), deep copies, and `merge_span_group_trees`,
which folds the trees of two observers of the same run into one: identical nodes are unified, anything else that
overlaps at one level is an error. `tree_from_tracer` builds the tree from the flat, parent-linked spans that
`perf.trace.PerfTracer` records."""
from __future__ import annotations

import math
from typing import Iterable, List, Optional, Union

_INF = float("inf")


class Span:
    def __init__(self, name: str, begin: float):
        self.name, self.begin, self.end = name, begin, _INF

    def __repr__(self) -> str:
        return f"{self.name}: {self.begin:.6f}, {self.end:.6f}"

    @property
    def ended(self) -> bool:
        return self.end != _INF

    @property
    def duration(self) -> float:
        return self.end - self.begin


class SpanGroup:
    def __init__(self, name: str, outer: Optional["SpanGroup"] = None):
        self.name, self.begin, self.end = name, 0.0, _INF
        self.inner: List[Union[Span, "SpanGroup"]] = []
        if outer is not None:
            self.outer = outer
            outer.inner.append(self)
        else:
            self.outer = self                       # the root is its own parent

    def __repr__(self) -> str:
        return f"{self.name}: {self.begin:.6f}, {self.end:.6f}"

    @property
    def duration(self) -> float:
        return self.end - self.begin

    def _groups(self, name: str) -> list:
        return [x for x in self.inner if isinstance(x, SpanGroup) and x.name == name]

    def _spans(self, name: str) -> list:
        return [x for x in self.inner if isinstance(x, Span) and x.name == name]

    def find_first_inner_group(self, name: str) -> Optional["SpanGroup"]:
        return next(iter(self._groups(name)), None)

    def find_last_inner_group(self, name: str) -> Optional["SpanGroup"]:
        g = self._groups(name)
        return g[-1] if g else None

    def find_all_inner_groups(self, name: str) -> list:
        return self._groups(name)

    def find_last_inner_span(self, name: str) -> Optional[Span]:
        s = self._spans(name)
        return s[-1] if s else None

    def find_all_inner_spans(self, name: str) -> list:
        return self._spans(name)


def span_group_tostring(group: SpanGroup, born: float = 0.0) -> str:
    lines: list = []

    def walk(node, depth: int) -> None:
        lines.append(f"{'  ' * depth}- {node.name} ({node.begin - born:.6f}, {node.end - born:.6f})\n")
        for child in getattr(node, "inner", ()):
            walk(child, depth + 1)
    walk(group, 0)
    return "".join(lines)


def span_group_print(group: SpanGroup, born: float = 0.0) -> None:
    print(span_group_tostring(group, born))


def span_group_stack_clone(stack: List[SpanGroup]) -> List[SpanGroup]:
    """A copy of a chain of open groups (outermost first) without their contents: what a new observer starts from."""
    out: list = []
    for g in stack:
        c = SpanGroup(g.name, out[-1] if out else None)
        c.begin, c.end = g.begin, g.end
        out.append(c)
    return out


def span_group_batch_query_first(batch: Iterable[SpanGroup], name: str) -> list:
    return [g for g in (b.find_first_inner_group(name) for b in batch) if g is not None]


def span_group_batch_query_last(batch: Iterable[SpanGroup], name: str) -> list:
    return [g for g in (b.find_last_inner_group(name) for b in batch) if g is not None]


def span_group_batch_query_nth(batch: Iterable[SpanGroup], name: str, index: int) -> list:
    out = []
    for b in batch:
        inner = b.find_all_inner_groups(name)
        if 0 <= index < len(inner):
            out.append(inner[index])
    return out


def span_group_batch_query_all(batch: Iterable[SpanGroup], name: str) -> list:
    return [g for b in batch for g in b.find_all_inner_groups(name)]


def clone_span_or_group(node, outer: Optional[SpanGroup] = None):
    if isinstance(node, SpanGroup):
        g = SpanGroup(node.name, outer)
        g.begin, g.end = node.begin, node.end
        for child in node.inner:
            clone_span_or_group(child, g)
        return g
    s = Span(node.name, node.begin)
    s.end = node.end
    if outer is not None:
        outer.inner.append(s)
    return s


def _same_node(a, b) -> bool:
    """Same kind, name and times (the tree below is not compared)."""
    close = lambda x, y: x == y or math.isclose(x, y, rel_tol=1e-15, abs_tol=1e-9)
    return isinstance(b, type(a)) and isinstance(a, type(b)) and a.name == b.name and close(a.begin, b.begin) and close(a.end, b.end)


def _merge_inplace(target: SpanGroup, source: SpanGroup) -> None:
    for child in source.inner:
        target.inner.append(child)
        if isinstance(child, SpanGroup):
            child.outer = target
    target.inner.sort(key=lambda x: x.begin)
    merged: list = []
    cur = None
    for node in target.inner:
        if cur is None:
            cur = node
        elif cur.end > node.begin:
            if not _same_node(cur, node):
                raise ValueError(f"Merge is not possible: Overlap detected between {cur!r} and {node!r}")
            if isinstance(cur, SpanGroup):
                _merge_inplace(cur, node)                   # a duplicate span is simply dropped
        else:
            merged.append(cur)
            cur = node
    if cur is not None:
        merged.append(cur)
    target.inner = merged


def merge_span_group_trees(tree1, tree2):
    """A new tree holding both; the inputs are left as they are. The roots must be the same node."""
    if not _same_node(tree1, tree2):
        raise ValueError(f"Roots are not identical: {tree1!r} vs {tree2!r}. Merge expected identical roots.")
    target, source = clone_span_or_group(tree1), clone_span_or_group(tree2)
    if isinstance(target, SpanGroup):
        _merge_inplace(target, source)
    return target


def tree_from_tracer(spans, root_name: str = "root", timeline: Optional[str] = None) -> SpanGroup:
    """The tree of the spans a `PerfTracer` recorded (optionally of one timeline): a recorded span that has children, or
    that was opened as a group, becomes a `SpanGroup`; the root spans first begin to last end."""
    spans = [s for s in spans if timeline is None or s.timeline == timeline]
    has_child = {id(s.parent) for s in spans if s.parent is not None}
    root = SpanGroup(root_name)
    made: dict = {}

    def node_of(s):
        if id(s) in made:
            return made[id(s)]
        outer = node_of(s.parent) if s.parent is not None and any(s.parent is x for x in spans) else root
        if not isinstance(outer, SpanGroup):
            raise ValueError(f"span {s.name!r} is nested in {outer.name!r}, which is not a group")
        if id(s) in has_child or s.tags.get("group"):
            n = SpanGroup(s.name, outer)
            n.begin = s.begin
        else:
            n = Span(s.name, s.begin)
            outer.inner.append(n)
        n.end = s.end if s.end is not None else _INF
        made[id(s)] = n
        return n
    for s in sorted(spans, key=lambda x: x.begin):
        node_of(s)

    def order(g: SpanGroup) -> None:
        g.inner.sort(key=lambda x: x.begin)
        for c in g.inner:
            if isinstance(c, SpanGroup):
                order(c)
    order(root)
    if root.inner:
        root.begin, root.end = root.inner[0].begin, max(c.end for c in root.inner)
    return root
