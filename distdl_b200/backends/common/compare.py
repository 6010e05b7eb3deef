"""Predicates on teams (``src/distdl/backends/common/compare.py:4-25``); with
rank-tuple partitions they reduce to tuple comparisons."""
from .world import PROC_NULL


def check_identical_comm(c1, c2):
    return tuple(c1) == tuple(c2)


def check_identical_group(g1, g2):
    return tuple(g1) == tuple(g2)


def check_null_comm(c):
    return c is None or len(c) == 0


def check_null_group(g):
    return g is None or len(g) == 0


def check_null_rank(r):
    return r is None or r == PROC_NULL
