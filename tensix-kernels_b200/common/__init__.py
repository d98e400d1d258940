"""Helpers shared by the dense_reader path: the ttnn-like tensor surface, device queries, test checks."""
