"""Operators backed by the hand-written sm_100a kernels (and their autograd wrappers)."""
