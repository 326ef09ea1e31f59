"""Matching of FX nodes against policy rules, and the graph partitioning built on it.

Behaviour follows the reference's ``dynaflow/matching.py``:

* ``Op`` matches one ``call_function`` node whose target's ``__name__`` fully
  matches a regular expression (``matching.py:8-15``).
* ``Mod`` matches the longest leading run of nodes that belong to one instance
  of a module class, judged by the innermost ``nn_module_stack`` entry
  (``matching.py:18-49``).
* ``MatchingRule`` matches a sequence of those, skipping ``getitem`` nodes, with
  an optional veto hook (``matching.py:52-90``).
* ``split_graph`` gives every match a subgraph of its own (``matching.py:93-126``);
  ``tag_graph`` labels top-level subgraphs (``matching.py:129-158``).

All three rule types are frozen dataclasses and therefore usable as dict keys.
"""
from __future__ import annotations

import dataclasses
import functools
import re
from collections.abc import Callable, Sequence

import torch
import torch.fx
from torch.fx.passes.split_module import split_module


@functools.lru_cache(maxsize=256)
def _compiled(pattern: str) -> re.Pattern:
    return re.compile(pattern)


def _is_getitem(node: torch.fx.Node) -> bool:
    return node.op == "call_function" and getattr(node.target, "__name__", None) == "getitem"


@dataclasses.dataclass(frozen=True)
class Op:
    """A function call whose name fully matches ``pattern``."""

    pattern: str

    def matches(self, node: torch.fx.Node) -> bool:
        target = node.target
        if node.op != "call_function" or not callable(target):
            return False
        return _compiled(self.pattern).fullmatch(target.__name__) is not None


@dataclasses.dataclass(frozen=True)
class Mod:
    """A run of nodes traced from one instance of ``target_cls``."""

    target_cls: type[torch.nn.Module]

    @classmethod
    def get_module_info(cls, node: torch.fx.Node) -> tuple[str, type[torch.nn.Module]] | None:
        """(qualified name, class) of the innermost module the node was traced in:
        the ``nn_module_stack`` entry whose name sorts last."""
        stack = node.meta.get("nn_module_stack")
        if stack is None:
            return None
        name, klass = max(stack.values(), key=lambda entry: entry[0])
        return name, klass

    def matches(self, node_list: Sequence[torch.fx.Node]) -> int:
        """Length of the leading run of ``node_list`` inside one ``target_cls`` instance."""
        owner: str | None = None
        count = 0
        for node in node_list:
            info = self.get_module_info(node)
            if info is None or info[1] is not self.target_cls:
                break
            if owner is None:
                owner = info[0]
            elif info[0] != owner:
                break
            count += 1
        return count


@dataclasses.dataclass(frozen=True)
class MatchingRule:
    """``condition`` is one ``Op``/``Mod`` or a tuple of them matched in sequence;
    ``hook(node_list, start_idx)`` may veto a match."""

    condition: Op | Mod | tuple[Op | Mod, ...]
    hook: Callable[[list[torch.fx.Node], int], bool] | None = None

    def matches(self, node_list: list[torch.fx.Node], start_idx: int) -> int:
        """Number of nodes matched from ``start_idx`` (0 = no match). ``getitem``
        nodes met while conditions remain are consumed without using one up."""
        conditions = self.condition if isinstance(self.condition, tuple) else (self.condition,)
        pos = start_idx
        remaining = list(conditions)
        total = len(node_list)
        while remaining and pos < total:
            node = node_list[pos]
            if _is_getitem(node):
                pos += 1
                continue
            cond = remaining[0]
            if isinstance(cond, Op):
                if not cond.matches(node):
                    return 0
                pos += 1
            else:
                run = cond.matches(node_list[pos:])
                if run == 0:
                    return 0
                pos += run
            remaining.pop(0)
        length = pos - start_idx
        if length > 0 and self.hook is not None and not self.hook(node_list, start_idx):
            return 0
        return length


def assign_subgraph_ids(nodes: list[torch.fx.Node], split_rules: list[MatchingRule]) -> dict[torch.fx.Node, int]:
    """Node -> subgraph id. Ids grow along the node list; each match takes a
    fresh id and the nodes after it another fresh one, so matched operators end
    up alone in their subgraph."""
    ids: dict[torch.fx.Node, int] = {}
    current = 0
    pos = 0
    while pos < len(nodes):
        length = 0
        for rule in split_rules:
            length = rule.matches(nodes, pos)
            if length > 0:
                break
        if length > 0:
            current += 1
            for node in nodes[pos:pos + length]:
                ids[node] = current
            current += 1
            pos += length
        else:
            ids[nodes[pos]] = current
            pos += 1
    return ids


def split_graph(graph: torch.fx.GraphModule, split_rules: list[MatchingRule]) -> torch.fx.GraphModule:
    """Cuts the traced forward into ``submod_<id>`` subgraphs around the rule matches,
    keeping the original node order."""
    ids = assign_subgraph_ids(list(graph.graph.nodes), split_rules)
    return split_module(graph, None, lambda node: ids.get(node, 0), keep_original_order=True)


def tag_graph(gm: torch.fx.GraphModule, tag_rules: dict[MatchingRule, set[str]]) -> None:
    """Sets ``.tag`` (a set of strings) on every top-level subgraph: the union of
    the tags of all rules that match somewhere inside it. At each position the
    first matching rule (dict order) wins and its match is skipped over."""
    for name, module in gm.named_children():
        if not hasattr(module, "graph"):
            continue
        tags: set[str] = set()
        nodes = list(module.graph.nodes)
        pos = 0
        while pos < len(nodes):
            step = 1
            for rule, rule_tags in tag_rules.items():
                length = rule.matches(nodes, pos)
                if length > 0:
                    tags.update(rule_tags)
                    step = length
                    break
            pos += step
        module.tag = tags
