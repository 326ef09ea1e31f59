"""Subgraph back-ends (``dynaflow/executor/__init__.py:1-2`` exports the same two names)."""
from .compiler import SubgraphBackend as SubgraphBackend
from .compiler import SubgraphCompiler as SubgraphCompiler
