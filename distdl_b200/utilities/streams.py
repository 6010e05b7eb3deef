"""The side stream of a device, used for data movement that needs no handshake with other
GPUs (in-place gathers of parameter shards).

Kernels that wait for other GPUs (staged collectives, the fused GEMM + collective kernels)
all run on the stream the caller is on: two such kernels must never be resident at the same
time on one GPU, because each may need the SMs the other holds while their peers wait for
both.  Wait-free copies have no such problem, so they may overlap the compute stream.

``deferred()`` marks a region (a weight prefetch) in which the consumer promises to call
``join()`` before it touches the results; outside such a region every side-stream operation
is joined immediately."""
import contextlib
import threading

import torch

_side = {}
_state = threading.local()


def side_stream(device=None) -> "torch.cuda.Stream | None":
    if not torch.cuda.is_available():
        return None
    if device is not None and torch.device(device).type != "cuda":
        return None
    idx = torch.cuda.current_device() if device is None or torch.device(device).index is None \
        else torch.device(device).index
    s = _side.get(idx)
    if s is None:
        s = torch.cuda.Stream(device=idx)
        _side[idx] = s
    return s


def is_deferred() -> bool:
    return getattr(_state, "deferred", 0) > 0


@contextlib.contextmanager
def deferred():
    _state.deferred = getattr(_state, "deferred", 0) + 1
    try:
        yield
    finally:
        _state.deferred -= 1


def join():
    """The current stream waits for everything queued on the side stream of its device."""
    if not _side:
        return
    idx = torch.cuda.current_device()
    s = _side.get(idx)
    if s is not None:
        cur = torch.cuda.current_stream(idx)
        if cur.cuda_stream != s.cuda_stream:
            cur.wait_stream(s)
