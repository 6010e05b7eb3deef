"""Self-attention over a sequence that is split across workers ("context parallelism" by
head <-> sequence all-to-all).

New relative to the reference, which has no attention code; its long-context story is
sequence parallelism of the linear and norm layers only.  The layer is built from existing
parts: two :class:`~distdl_b200.nn.Repartition` pairs move ``q``, ``k``, ``v`` from the
sequence-split layout ``[batch, seq / S, heads, head_dim]`` to the head-split layout
``[batch, seq, heads / S, head_dim]`` (one all-to-all each), the local attention kernel
(:func:`distdl_b200.ops.attention`, flash attention on tcgen05 for bf16 CUDA tensors) then
sees whole sequences of its own heads, and one more Repartition brings the output back.
Backward is the adjoint chain (Repartition is its own adjoint pair), so nothing but the
partitions has to be specified.
"""

from .. import ops
from .module import Module
from .repartition import Repartition


class DistributedSelfAttention(Module):
    r"""``forward(q, k, v) -> out`` with ``q [b, s_local, Hq, D]``, ``k, v [b, s_local, Hkv, D]``
    on ``P_seq = [B, S, H, 1]`` (batch x sequence split; ``H`` > 1 when the heads are already
    split over tensor-parallel workers); the local head counts must divide by ``S`` (``Hkv``
    too).  ``causal`` masks with GLOBAL positions, which the head-split layout gives for free
    because every worker then holds complete sequences."""

    def __init__(self, P_seq, causal=True, scale=None):
        super().__init__()
        self.P_seq = P_seq
        self.causal, self.scale = causal, scale
        if not P_seq.active:
            return
        if P_seq.dim != 4 or int(P_seq.shape[3]) != 1:
            raise ValueError("DistributedSelfAttention expects a partition of shape [B, S, H, 1]")
        B, S, H = int(P_seq.shape[0]), int(P_seq.shape[1]), int(P_seq.shape[2])
        self.S = S
        base = P_seq.create_partition_inclusive(range(P_seq.size))
        # worker (b, c, t) of the input grid becomes head shard c * H + t of batch shard b
        self.P_head = base.create_cartesian_topology_partition([B, 1, S * H, 1])
        self.to_heads_q = Repartition(P_seq, self.P_head)
        self.to_heads_k = Repartition(P_seq, self.P_head)
        self.to_heads_v = Repartition(P_seq, self.P_head)
        self.to_seq = Repartition(self.P_head, P_seq)

    def forward(self, q, k, v):
        if not self.P_seq.active:
            return q
        if self.S == 1:
            qh, kh, vh = q, k, v
        else:
            if q.shape[2] % self.S or k.shape[2] % self.S:
                raise ValueError(f"query / key heads ({q.shape[2]}, {k.shape[2]}) must divide by the "
                                 f"sequence-parallel size {self.S}")
            qh, kh, vh = self.to_heads_q(q), self.to_heads_k(k), self.to_heads_v(v)
        b, s, hq, d = qh.shape
        hkv = kh.shape[2]
        o = ops.attention(qh.reshape(b * s, hq, d), kh.reshape(b * s, hkv, d), vh.reshape(b * s, hkv, d), b, s,
                          causal=self.causal, scale=self.scale)
        o = o.reshape(b, s, hq, d)
        return o if self.S == 1 else self.to_seq(o)
