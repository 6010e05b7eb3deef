"""Embedding tables: columns split over the model-parallel workers (DistributedEmbedding, broadcast
over the data-parallel ones) and additionally rows split over the data-parallel workers
(DistributedEmbeddingZero, gathered on use).  The initial values do not depend on the grid: the
table is drawn on worker 0 and scattered."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 1, 2])                        # [data, sequence, model]
from distdl_b200.nn import DistributedEmbedding, DistributedEmbeddingZero  # noqa: E402

torch.manual_seed(0)
ids = torch.randint(0, 50, (3, 7))                                # this worker's [batch / 2, sequence] token ids
emb = DistributedEmbedding(P, 50, 16, collect_state=True)
y = emb(ids)
say(P_world, "DistributedEmbedding: table shard", tuple(emb.weight.shape), "-> y", tuple(y.shape))
zero = DistributedEmbeddingZero(P, 50, 16, collect_state=True)
y = zero(ids)
y.sum().backward()
say(P_world, "DistributedEmbeddingZero: table shard", tuple(zero.weight.shape), "-> y", tuple(y.shape),
    "grad", tuple(zero.weight.grad.shape))
sd = zero.state_dict()
if rank == 0:
    print("whole table on worker 0:", tuple(sd["weight"].shape))
