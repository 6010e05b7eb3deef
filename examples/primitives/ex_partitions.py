"""Partitions: teams of workers and Cartesian grids derived from them (4 workers)."""
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2])
say(P_world, "index", P.index, "neighbours", P.neighbor_ranks(P.rank))
row = P.create_allreduction_partition((1,))          # my row of the grid
say(P_world, "row team", row.ranks)
P_src = cart(P_world, [0, 1], [1, 2])
P_send, P_recv = P_src.create_broadcast_partition_to(P)
say(P_world, "broadcast: send team", P_send.ranks, "recv team", P_recv.ranks)
