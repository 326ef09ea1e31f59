"""Run-time half of the scheduling layer: per-nano-batch environments and the engine."""
