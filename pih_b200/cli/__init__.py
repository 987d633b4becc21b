"""Command lines: the worker-style generator and the trace replay."""
