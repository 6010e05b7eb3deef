"""Rank-ordered printing for debugging distributed programs."""
from __future__ import annotations

import sys


def print_sequential(P, val, file=None):
    """Every active worker of partition ``P`` prints ``val`` in rank order
    (one barrier per rank, so output is not interleaved)."""
    file = file or sys.stdout
    if not getattr(P, "active", False):
        return
    for r in range(P.size):
        if r == P.rank:
            print(f"[{P.rank}/{P.size}] {val}", file=file, flush=True)
        P.barrier()
