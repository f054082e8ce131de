"""Helpers shared by the test-suite: multi-process worker bodies (importable from spawned children)."""
