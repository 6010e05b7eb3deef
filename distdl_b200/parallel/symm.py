"""Symmetric (peer-mapped) memory of the native backend.

Every process allocates one staging buffer and one signal pad on its GPU,
exports them as CUDA IPC handles, and maps the buffers of every other process
of the node; after that a kernel on any GPU can load from / store to any
peer's buffer over NVLink / NVSwitch.  Handles are exchanged once through
``torch.distributed`` (plumbing only).  The reference bootstraps one NCCL
communicator per rank set instead (``src/distdl/backends/nccl_cupy/nccl_comm.py:132-144``).

Flag protocol bookkeeping lives here as well: flags are counters that only
grow, and the host keeps, per peer, how many barrier steps have been consumed,
so each launch knows the value its first barrier has to wait for.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native

c_void_p, c_int, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
_PP = ctypes.POINTER(c_void_p)
_IP = ctypes.POINTER(c_int)
_UP = ctypes.POINTER(ctypes.c_uint)

_native.declare("dd_symm_alloc", [c_size_t, _PP])
_native.declare("dd_symm_free", [c_void_p])
_native.declare("dd_ipc_get_handle", [c_void_p, ctypes.c_char_p])
_native.declare("dd_ipc_open_handle", [ctypes.c_char_p, _PP])
_native.declare("dd_ipc_close_handle", [c_void_p])
_native.declare("dd_collective_ctas", [])
_native.declare("dd_collective_max_peers", [])
_TEAM = [c_int, c_int, c_int, _PP, _PP, _IP, _UP]
_native.declare("dd_allreduce", _TEAM + [c_void_p, c_size_t, c_int, c_int, _IP, c_void_p])
_native.declare("dd_allgather", _TEAM + [c_void_p, c_size_t, _IP, c_void_p])
_native.declare("dd_reducescatter", _TEAM + [c_void_p, c_size_t, c_int, _IP, c_void_p])
_native.declare("dd_reducescatter_push", _TEAM + [_PP, c_void_p, c_size_t, c_int, _IP, c_void_p])
_native.declare("dd_reducescatter_acc", _TEAM + [c_void_p, c_size_t, ctypes.c_float, _IP, c_void_p])
_native.declare("dd_exchange", _TEAM + [_PP, ctypes.POINTER(ctypes.c_ulonglong), ctypes.c_ulonglong, _IP, c_void_p])
_native.declare("dd_alltoall", _TEAM + [c_void_p, c_size_t, _IP, c_void_p])
_native.declare("dd_team_barrier", _TEAM + [_IP, c_void_p])

SIGNAL_PAD_BYTES = 64 * 1024
GUARD_BYTES = 4096            # guard zone after every region of the staging buffer
GUARD_PATTERN = 0xA5
MB = 1 << 20
# Regions of the staging buffer (same layout on every process).
REGION_SIZES = (("coll", None), ("ag_shard", 128 * MB), ("rs0", 224 * MB), ("rs1", 224 * MB), ("misc", 4 * MB),
                ("inbox", 64 * MB))      # inbox: chunk buffers of the box exchange, one slot per source GPU


class SymmetricHeap:
    """One staging buffer + signal pad per process, mapped into every process."""

    def __init__(self, staging_bytes: int):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("torch.distributed must be initialised before the symmetric heap")
        lib = _native.lib()
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.max_peers = lib.dd_collective_max_peers()
        if self.world > self.max_peers:
            raise RuntimeError(f"the native transport handles up to {self.max_peers} GPUs of one node")
        self.staging_bytes = int(staging_bytes)
        self._team_cache = {}          # rank tuple -> the arguments of a team that never change
        self.regions = {}
        # every region is followed by a guard zone that holds a fixed pattern: a kernel that runs past
        # the end of its region (on this GPU or, through the peer mapping, on another one) leaves a
        # trace that check_canaries() finds
        off = 0
        for name, size in REGION_SIZES:
            size = self.staging_bytes if size is None else size
            self.regions[name] = (off, size)
            off += size + GUARD_BYTES
        self.total_bytes = off
        self.device = torch.device("cuda", torch.cuda.current_device())
        self._local_buf, self._local_pad = c_void_p(), c_void_p()
        _native.check(lib.dd_symm_alloc(self.total_bytes, ctypes.byref(self._local_buf)), "dd_symm_alloc")
        _native.check(lib.dd_symm_alloc(SIGNAL_PAD_BYTES, ctypes.byref(self._local_pad)), "dd_symm_alloc")
        hb, hp = ctypes.create_string_buffer(64), ctypes.create_string_buffer(64)
        _native.check(lib.dd_ipc_get_handle(self._local_buf, hb), "dd_ipc_get_handle")
        _native.check(lib.dd_ipc_get_handle(self._local_pad, hp), "dd_ipc_get_handle")
        mine = (bytes(hb.raw), bytes(hp.raw), os.getpid())
        gathered = [None] * self.world
        dist.all_gather_object(gathered, mine)
        self.buf_ptrs, self.pad_ptrs = [], []
        for r, (b, p, _pid) in enumerate(gathered):
            if r == self.rank:
                self.buf_ptrs.append(self._local_buf.value)
                self.pad_ptrs.append(self._local_pad.value)
                continue
            pb, pp = c_void_p(), c_void_p()
            _native.check(lib.dd_ipc_open_handle(b, ctypes.byref(pb)), "dd_ipc_open_handle")
            _native.check(lib.dd_ipc_open_handle(p, ctypes.byref(pp)), "dd_ipc_open_handle")
            self.buf_ptrs.append(pb.value)
            self.pad_ptrs.append(pp.value)
        # barrier steps consumed so far with every peer (flags are counters)
        self.steps_done = [0] * self.world
        self.poisoned = False
        for name, (roff, size) in self.regions.items():
            _wrap_device_pointer(self._local_buf.value + roff + size, GUARD_BYTES, torch.uint8,
                                 self.device).fill_(GUARD_PATTERN)
        torch.cuda.synchronize()
        dist.barrier()

    def check_canaries(self):
        """Names of the regions whose guard zone no longer holds its pattern (empty list = intact).
        Synchronises the device."""
        bad = []
        for name, (roff, size) in self.regions.items():
            guard = _wrap_device_pointer(self._local_buf.value + roff + size, GUARD_BYTES, torch.uint8, self.device)
            if not bool((guard == GUARD_PATTERN).all().item()):
                bad.append(name)
        return bad

    def staging_tensor(self, nbytes: int, dtype=torch.uint8) -> torch.Tensor:
        """A tensor view of the head of the local staging buffer (no copy, no ownership)."""
        if nbytes > self.staging_bytes:
            raise ValueError(f"{nbytes} bytes exceed the staging buffer ({self.staging_bytes})")
        n = nbytes // torch.empty((), dtype=dtype).element_size()
        return _wrap_device_pointer(self._local_buf.value, n, dtype, self.device)

    def region_ptr(self, name, rank=None, offset=0):
        """Address of a region in the staging buffer of ``rank`` (default: mine), as mapped here."""
        base = self.buf_ptrs[self.rank if rank is None else rank]
        return base + self.regions[name][0] + offset

    def region_tensor(self, name, nbytes, dtype=torch.uint8, offset=0):
        """Tensor view of (the head of) one of my regions."""
        off, size = self.regions[name]
        if offset + nbytes > size:
            raise ValueError(f"{nbytes} bytes do not fit region {name!r} ({size} bytes)")
        n = nbytes // torch.empty((), dtype=dtype).element_size()
        return _wrap_device_pointer(self._local_buf.value + off + offset, n, dtype, self.device)

    def team_args(self, ranks):
        """ctypes arguments describing a team (ordered world ranks containing this rank)."""
        key = tuple(ranks)
        fixed = self._team_cache.get(key)
        if fixed is None:
            n = len(key)
            fixed = self._team_cache[key] = (n, key.index(self.rank), self.rank,
                                             (c_void_p * n)(*[self.buf_ptrs[r] for r in key]),
                                             (c_void_p * n)(*[self.pad_ptrs[r] for r in key]),
                                             (c_int * n)(*[int(r) for r in key]))
        expect = (ctypes.c_uint * fixed[0])(*[(self.steps_done[r] + 1) & 0xFFFFFFFF for r in key])
        return fixed + (expect,)

    def advance(self, ranks, steps: int):
        for r in ranks:
            if r != self.rank:
                self.steps_done[r] += steps


class SymmetricRegion:
    """A separately allocated buffer of the same size on every process, mapped into all
    of them (``ptrs[rank]`` = address of that rank's copy as seen from here)."""

    def __init__(self, heap: "SymmetricHeap", nbytes: int):
        lib = _native.lib()
        sizes = [None] * heap.world
        dist.all_gather_object(sizes, int(nbytes))
        self.nbytes = (max(sizes) + 255) // 256 * 256
        self.heap = heap
        self._local = c_void_p()
        _native.check(lib.dd_symm_alloc(self.nbytes, ctypes.byref(self._local)), "dd_symm_alloc")
        hb = ctypes.create_string_buffer(64)
        _native.check(lib.dd_ipc_get_handle(self._local, hb), "dd_ipc_get_handle")
        handles = [None] * heap.world
        dist.all_gather_object(handles, bytes(hb.raw))
        self.ptrs = []
        for r, hnd in enumerate(handles):
            if r == heap.rank:
                self.ptrs.append(self._local.value)
                continue
            p = c_void_p()
            _native.check(lib.dd_ipc_open_handle(hnd, ctypes.byref(p)), "dd_ipc_open_handle")
            self.ptrs.append(p.value)
        self.local_ptr = self._local.value
        dist.barrier()

    def tensor(self, numel: int, dtype) -> torch.Tensor:
        """Tensor view of the head of the local copy."""
        return _wrap_device_pointer(self.local_ptr, numel, dtype, self.heap.device)

    def contains(self, ptr: int, nbytes: int) -> bool:
        return self.local_ptr <= ptr and ptr + nbytes <= self.local_ptr + self.nbytes


_param_regions = []


def register_param_region(region: SymmetricRegion):
    """Declares ``region`` to hold parameters at the same offsets on every process: the
    native transport then gathers such a parameter by reading the peers' copies in place."""
    _param_regions.append(region)


def find_param_region(ptr: int, nbytes: int):
    for reg in _param_regions:
        if reg.contains(ptr, nbytes):
            return reg
    return None


class _DevicePointer:
    """Minimal object exposing ``__cuda_array_interface__`` for a raw pointer."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                         "strides": None}


_TYPESTR = {torch.uint8: "|u1", torch.float32: "<f4", torch.int32: "<i4", torch.int16: "<i2", torch.int64: "<i8"}


def _wrap_device_pointer(ptr, n, dtype, device):
    if dtype in _TYPESTR:
        return torch.as_tensor(_DevicePointer(ptr, n, _TYPESTR[dtype]), device=device)
    # bf16 / fp16 have no typestr torch accepts here: wrap as int16 and reinterpret
    t = torch.as_tensor(_DevicePointer(ptr, n, "<i2"), device=device)
    return t.view(dtype)


_heap = None


def heap(staging_bytes: int = None) -> SymmetricHeap:
    """The process-wide heap (created on first use; every process must call)."""
    global _heap
    if _heap is None:
        size = staging_bytes or int(os.environ.get("DISTDL_SYMM_BYTES", str(512 * MB)))
        _heap = SymmetricHeap(size)
    return _heap


def heap_ready() -> bool:
    return _heap is not None


# ----------------------------------------------------------------- NVLink multicast region
_native.declare("dd_mc_supported", [])
_native.declare("dd_mc_round_size", [c_int, c_size_t, ctypes.POINTER(c_size_t)])
_native.declare("dd_mc_create", [c_int, c_size_t, _IP])
_native.declare("dd_mc_import", [c_int, c_size_t, c_int])
_native.declare("dd_mc_add_device", [])
_native.declare("dd_mc_bind_and_map", [_PP, _PP])
_native.declare("dd_mc_teardown", [])
_native.declare("dd_close_fd", [c_int])
_native.declare("dd_mc_max_ctas", [])
_native.declare("dd_mc_allreduce", [c_int, c_int, _PP, ctypes.c_uint, c_size_t, c_size_t, c_void_p, c_size_t, c_int,
                                    c_int, c_int, _IP, c_void_p])


class MulticastRegion:
    """One buffer per GPU of the job, all bound to one NVLink multicast object: a kernel reads the
    sum over all GPUs of a word with one ``multimem.ld_reduce`` and writes a word into all copies
    with one ``multimem.st`` (the reduction runs inside NVSwitch).  Used by the all-reduce of the
    job-wide team (:func:`distdl_b200.parallel.collectives.all_reduce`).

    Creating it is collective over all processes.  The multicast object is created by rank 0 and
    reaches the other processes as a file descriptor over a unix socket.  OFF unless asked for
    (``DISTDL_MULTIMEM=1`` or :func:`enable_multicast`): a process that ends while its memory is
    still bound disturbs the GPUs of the others, so only jobs whose processes leave together
    (after :func:`disable_multicast`) should turn it on; tests that end a rank on purpose must not."""

    def __init__(self, heap: "SymmetricHeap", nbytes: int):
        import socket
        import tempfile
        lib = _native.lib()
        self.heap = heap
        W, rank = heap.world, heap.rank
        size = ctypes.c_size_t(0)
        _native.check(lib.dd_mc_round_size(W, int(nbytes), ctypes.byref(size)), "dd_mc_round_size")
        self.nbytes = int(size.value)
        # rank 0 creates the object and hands its descriptor to every other process
        path = [None]
        if rank == 0:
            fd = c_int(-1)
            _native.check(lib.dd_mc_create(W, self.nbytes, ctypes.byref(fd)), "dd_mc_create")
            srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            path[0] = os.path.join(tempfile.gettempdir(), f"distdl_b200_mc_{os.getpid()}.sock")
            if os.path.exists(path[0]):
                os.unlink(path[0])
            srv.bind(path[0])
            srv.listen(W)
        dist.broadcast_object_list(path, src=0)
        if rank == 0:
            srv.settimeout(60.0)
            for _ in range(W - 1):
                conn, _addr = srv.accept()
                socket.send_fds(conn, [b"mc"], [fd.value])
                conn.recv(1)                       # the peer has imported the object
                conn.close()
            srv.close()
            os.unlink(path[0])
            lib.dd_close_fd(fd.value)
        else:
            cli = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            cli.settimeout(60.0)
            cli.connect(path[0])
            _msg, fds, _flags, _addr = socket.recv_fds(cli, 16, 1)
            _native.check(lib.dd_mc_import(W, self.nbytes, fds[0]), "dd_mc_import")
            cli.send(b"k")
            cli.close()
            lib.dd_close_fd(fds[0])
        dist.barrier()
        _native.check(lib.dd_mc_add_device(), "dd_mc_add_device")
        dist.barrier()                                 # every device is part of the object
        local, mc = c_void_p(), c_void_p()
        _native.check(lib.dd_mc_bind_and_map(ctypes.byref(local), ctypes.byref(mc)), "dd_mc_bind_and_map")
        self.local_ptr, self.mc_ptr = local.value, mc.value
        self.steps_done = 0                            # barrier steps consumed by the multicast kernels
        # the grid of every multicast kernel of this process (the per-CTA counters have to advance in step)
        self.ctas = max(1, min(lib.dd_mc_max_ctas(), int(os.environ.get("DISTDL_MC_CTAS", "96"))))
        dist.barrier()

    def local_tensor(self, nbytes, dtype=torch.uint8, offset=0):
        n = nbytes // torch.empty((), dtype=dtype).element_size()
        return _wrap_device_pointer(self.local_ptr + offset, n, dtype, self.heap.device)

    def close(self):
        """Collective: every process calls it when no kernel using the region is in flight."""
        torch.cuda.synchronize()
        dist.barrier()
        _native.lib().dd_mc_teardown()
        dist.barrier()


_multicast = None


def multicast_supported() -> bool:
    return bool(_native.lib().dd_mc_supported())


def enable_multicast(nbytes: int = 128 * MB):
    """Creates the job-wide multicast region (collective over all processes; a no-op where the
    GPUs do not support multicast objects or the job spans more than 8 GPUs).  Returns the region
    or None."""
    global _multicast
    if _multicast is None:
        h = heap()
        ok = [None] * h.world
        dist.all_gather_object(ok, bool(h.world > 1 and h.world <= 8 and multicast_supported()))
        if all(ok):
            _multicast = MulticastRegion(h, nbytes)
    return _multicast


def multicast_region():
    """The region if it exists; created on first use when ``DISTDL_MULTIMEM=1``."""
    if _multicast is None and os.environ.get("DISTDL_MULTIMEM", "0") == "1" and heap_ready():
        return enable_multicast()
    return _multicast


def disable_multicast():
    """Collective tear-down of the multicast region (call before the processes exit)."""
    global _multicast
    if _multicast is not None:
        _multicast.close()
        _multicast = None


class DeviceTimeout(RuntimeError):
    """A kernel gave up a bounded wait for another GPU."""


def require_healthy():
    """Called by every host wrapper that launches a kernel using the flag counters (the staged
    collectives, the exchange, the barriers, the fused GEMM + collective kernels, the MoE
    routing kernels): refuses the launch once a bounded wait has run out.  After a time-out the
    counters of this process are out of step with its peers, so every further such kernel would
    only spin for the full wait limit."""
    if _heap is not None and _heap.poisoned:
        raise DeviceTimeout("the symmetric heap is poisoned by an earlier device time-out; restart the job "
                            "from its last checkpoint")
    _one_waiting_stream()


_last_waiting = [None]             # stream of the last peer-waiting launch


def _one_waiting_stream():
    """Kernels that wait for other GPUs must not be resident on one GPU from two streams at once: each
    could hold the SMs that the other needs while their peers wait for both.  Every such launch passes
    through here; a launch on another stream than the previous one is refused unless everything
    queued on that stream (the previous such kernel included) has finished."""
    if not torch.cuda.is_available() or os.environ.get("DISTDL_STREAM_GUARD", "1") == "0":
        return
    cur = torch.cuda.current_stream()
    last = _last_waiting[0]
    if last is not None and last.cuda_stream != cur.cuda_stream and last.device == cur.device and not last.query():
        raise RuntimeError("a kernel that waits for other GPUs is still running on another stream of this GPU: "
                           "launch the collectives, exchanges and fused GEMMs of one GPU on one stream "
                           "(or synchronise the streams first)")
    _last_waiting[0] = cur


def check_health():
    """Reads the device status record (synchronises the device).  If a kernel gave up a
    bounded wait since the last check, the symmetric heap is marked poisoned (its flag
    counters are out of step with the peers, so every later collective would time out as
    well) and :class:`DeviceTimeout` is raised with the recorded place and counter values.
    Recovery: restart the job from the last checkpoint."""
    code, where, expected, seen = _native.read_status()
    if _heap is not None and os.environ.get("DISTDL_CHECK_CANARIES", "1") != "0":
        bad = _heap.check_canaries()
        if bad:
            _heap.poisoned = True
            raise DeviceTimeout(f"the guard zones after the staging regions {bad} were overwritten: a kernel wrote "
                                f"past the end of its region")
    if code == 0:
        return
    if _heap is not None:
        _heap.poisoned = True
    raise DeviceTimeout(f"device status {code}: a bounded wait ran out at site {where} "
                        f"(waited for {expected & 0xFFFFFFFF}, saw {seen & 0xFFFFFFFF})")
