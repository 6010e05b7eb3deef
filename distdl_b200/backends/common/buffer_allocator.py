"""Assigns staging buffers to the messages of Repartition and HaloExchange
(``src/distdl/backends/common/buffer_allocator.py:7-94``)."""
from __future__ import annotations

import numpy as np


def allocate_repartition_buffers(buffer_manager, P_x_to_y_overlaps, P_y_to_x_overlaps, dtype, device=None):
    """One buffer per message that leaves or enters this worker (overlaps with
    ``"self"`` or ``None`` need none).  Returns ``(send_views, recv_views)``
    aligned with the two overlap lists; sends take the first buffers."""
    def need(overlaps):
        return [i for i, (sl, sh, partner) in enumerate(overlaps) if sl is not None and partner != "self"]
    s_idx, r_idx = need(P_x_to_y_overlaps), need(P_y_to_x_overlaps)
    bufs = buffer_manager.request_buffers(len(s_idx) + len(r_idx), dtype=dtype, device=device)
    send = [None] * len(P_x_to_y_overlaps)
    recv = [None] * len(P_y_to_x_overlaps)
    k = 0
    for i in s_idx:
        send[i] = bufs[k].get_view(tuple(P_x_to_y_overlaps[i][1]))
        k += 1
    for i in r_idx:
        recv[i] = bufs[k].get_view(tuple(P_y_to_x_overlaps[i][1]))
        k += 1
    return send, recv


def allocate_halo_exchange_buffers(buffer_manager, slices, recv_buffer_shape, send_buffer_shape, dtype, device=None):
    """Four buffers (left/right x send/recv) re-viewed per dimension, since the
    dimensions are exchanged one after another.  Returns a list with one
    ``[left_send, left_recv, right_send, right_recv]`` entry per dimension
    (``None`` where nothing moves)."""
    bufs = buffer_manager.request_buffers(4, dtype=dtype, device=device)
    out = []
    for d, (lb, lg, rb, rg) in enumerate(slices):
        def view(buf, sl, width):
            if width <= 0:
                return None
            shape = tuple(int(s.stop - s.start) for s in sl)
            return buf.get_view(shape) if int(np.prod(shape)) > 0 else None
        out.append([view(bufs[0], lb, send_buffer_shape[d][0]), view(bufs[1], lg, recv_buffer_shape[d][0]),
                    view(bufs[2], rb, send_buffer_shape[d][1]), view(bufs[3], rg, recv_buffer_shape[d][1])])
    return out
