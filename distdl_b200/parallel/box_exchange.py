"""Host side of the box-exchange kernel (``csrc/box_exchange.cu``): strided boxes of local
tensors travel between GPUs in one launch, packed and unpacked by the kernel itself.

A :class:`BoxPlan` describes the exchange of one primitive once -- which box of which tensor
goes to (comes from) which worker, in which phase -- in terms of named tensor *slots* and
nd-slices.  :meth:`BoxPlan.run` binds the slots to this call's tensors, fills in addresses
and the running chunk numbers of the pair-wise flag protocol and launches the kernel.  The
geometry (collapsed extents, byte strides, copy unit) is computed once per tensor layout and
cached, so a repeated exchange costs the host little more than the launch.

Used by HaloExchange (one phase per dimension; the adjoint sends the ghost regions back,
adds them into the bulk and clears them) and by Repartition (one phase).  Stands where the
reference packs and unpacks with array slicing around grouped sends and receives
(``src/distdl/backends/nccl_cupy/functional/halo_exchange.py:49-80``,
``src/distdl/backends/nccl_cupy/functional/repartition.py:142-205``).

Flag bookkeeping: chunks on an ordered pair of GPUs are numbered over the life of the process
(``sent[peer]`` / ``received[peer]``); both ends count alike because both know every message's
size.  Messages of one ordered pair are matched in the order in which they are listed.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native
from ..ops._util import stream_ptr
from . import symm

_v, _i, _u, _ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong
_native.declare("dd_box_exchange", [_v, _i, _i, ctypes.POINTER(_u), ctypes.POINTER(_v), ctypes.POINTER(_v), _i, _ull,
                                    _ull, _v])
_native.declare("dd_box_max_items", [])
_native.declare("dd_box_bufs", [])
_native.declare("dd_box_item_bytes", [])
_native.declare("dd_box_copy_host", [_v, _v])
_native.declare("dd_box_progress", [ctypes.POINTER(_u)])
_native.declare("dd_box_piece_bytes", [_i])

SEND, RECV, LOCAL = 0, 1, 2
_ADD = {torch.float32: 1, torch.bfloat16: 2, torch.float16: 3, torch.float64: 4}
MAX_PEERS = 8


class _Box(ctypes.Structure):
    _fields_ = [("base", _v), ("s", ctypes.c_longlong * 3), ("n", _i * 4), ("lo", _v), ("hi", _v)]


def _storage_bounds(t):
    """[lo, hi) of the tensor's storage: what the bounds-checking build of the library verifies
    every address against."""
    st = t.untyped_storage()
    return st.data_ptr(), st.data_ptr() + st.nbytes()


class BoxItem(ctypes.Structure):
    _fields_ = [("a", _Box), ("b", _Box), ("bytes", _ull), ("first_seq", _u), ("unit", _i), ("unit_b", _i),
                ("kind", _i), ("peer", _i), ("phase", _i), ("clear_source", _i), ("add", _i)]


def collapse(shape, strides, itemsize, aligned16):
    """A strided nd box as ``(n[4], s[3] in bytes, unit)`` or None when it needs more than three
    outer directions.  ``shape`` / ``strides`` in elements; ``aligned16``: the box's first byte
    is 16-byte aligned.  Dimensions of extent 1 are dropped and dimensions that are contiguous
    with each other are merged; the innermost run is copied in 16-byte units when run length,
    start and every outer stride allow it, else element by element."""
    dims = [(int(n), int(s)) for n, s in zip(shape, strides) if int(n) != 1]
    merged = []
    for n, s in dims:
        if merged and merged[-1][1] == s * n:
            merged[-1] = (merged[-1][0] * n, s)
        else:
            merged.append((n, s))
    if merged and merged[-1][1] == 1:
        run, outer = merged[-1][0], merged[:-1]
    else:
        run, outer = 1, merged
    if len(outer) > 3:
        return None
    unit = itemsize
    n3 = run
    if (run * itemsize) % 16 == 0 and aligned16 and all((s * itemsize) % 16 == 0 for _, s in outer):
        unit, n3 = 16, run * itemsize // 16
    outer = [(1, 0)] * (3 - len(outer)) + outer
    return [n for n, _ in outer] + [n3], [s * itemsize for _, s in outer], unit


def _slices_of(view_shape, slices):
    """(offset in elements given strides later, shape) of an nd-slice; ``slices`` None = everything."""
    if slices is None:
        return [0] * len(view_shape), [int(n) for n in view_shape]
    starts = [int(sl.start or 0) for sl in slices]
    shape = [max(0, int(sl.stop if sl.stop is not None else n) - st) for sl, st, n in zip(slices, starts, view_shape)]
    return starts, shape


class _State:
    """Per-process bookkeeping of the pair-wise protocol."""

    def __init__(self):
        self.h = symm.heap()
        self.sent = [0] * MAX_PEERS          # chunks sent so far to world rank r
        self.received = [0] * MAX_PEERS
        self.progress = 0                    # pieces completed so far by this GPU's kernels
        lib = _native.lib()
        self.max_items = lib.dd_box_max_items()
        self.bufs = lib.dd_box_bufs()
        self.piece = {u: int(lib.dd_box_piece_bytes(u)) for u in (1, 2, 4, 8, 16)}
        assert lib.dd_box_item_bytes() == ctypes.sizeof(BoxItem), "BoxItem layout differs from the library's"
        off, size = self.h.regions["inbox"]
        self.slot = (size // MAX_PEERS) // 256 * 256
        self.chunk = (self.slot // self.bufs) // 256 * 256
        W = self.h.world
        self.inbox = (_v * MAX_PEERS)(*[self.h.region_ptr("inbox", r) if r < W else None for r in range(MAX_PEERS)])
        self.pads = (_v * MAX_PEERS)(*[self.h.pad_ptrs[r] if r < W else None for r in range(MAX_PEERS)])


_state = None


def state() -> _State:
    global _state
    if _state is None:
        _state = _State()
    return _state


def _limits():
    """(most items per launch, chunk bytes, piece bytes): from the heap when there is one, else the
    library's constants with the default inbox size (plans can then be compiled without a GPU)."""
    if symm.heap_ready():
        st = state()
        return st.max_items, st.chunk, st.piece
    lib = _native.lib()
    slot = (dict(symm.REGION_SIZES)["inbox"] // MAX_PEERS) // 256 * 256
    return (lib.dd_box_max_items(), (slot // lib.dd_box_bufs()) // 256 * 256,
            {u: int(lib.dd_box_piece_bytes(u)) for u in (1, 2, 4, 8, 16)})


def pieces_of(nbytes: int, chunk: int, piece: int, local: bool = False) -> int:
    """Pieces the kernel cuts a message into (what its progress counter advances by)."""
    if local:
        return -(-nbytes // piece)
    full, rest = divmod(nbytes, chunk)
    return full * (-(-chunk // piece)) + (-(-rest // piece) if rest else 0)


class BoxPlan:
    """``phases``: a list of phases, each a list of operations

    * ``("send", world_rank, slot, slices, clear)``: the box ``slices`` of the tensor bound to
      ``slot`` goes to ``world_rank``; with ``clear`` it is zeroed after it was read;
    * ``("recv", world_rank, slot, slices, add)``: the message from ``world_rank`` lands in
      that box, added to what is there with ``add``;
    * ``("copy", src_slot, src_slices, dst_slot, dst_slices)``: a local box-to-box copy.

    A phase starts when everything of the phase before it is complete on this GPU."""

    def __init__(self, phases):
        self.phases = [list(p) for p in phases]
        self._compiled = {}

    # ------------------------------------------------------------------ geometry
    @staticmethod
    def _meta(t):
        return (tuple(t.shape), tuple(t.stride()), t.dtype, t.data_ptr() % 16)

    def _geometry(self, meta, slices):
        shape, strides, dtype, mis = meta
        es = torch.empty((), dtype=dtype).element_size()
        starts, bshape = _slices_of(shape, slices)
        off = sum(a * s for a, s in zip(starts, strides)) * es
        vol = 1
        for n in bshape:
            vol *= n
        geo = collapse(bshape, strides, es, (mis + off) % 16 == 0) if vol else ([1, 1, 1, 0], [0, 0, 0], es)
        return off, vol * es, geo, bshape

    def _compile(self, metas):
        """Items (with byte offsets in place of addresses), per-phase piece counts and the ops that
        need a contiguous temporary because their box does not collapse or their dtype cannot be
        added by the kernel."""
        max_items, chunk, piece = _limits()
        launches = []                  # one entry per kernel launch: (items, pieces per phase, pre ops, post ops)
        items, phase_pieces, pre, post = [], [], [], []
        phase_in_launch = 0

        def flush():
            nonlocal items, phase_pieces, pre, post, phase_in_launch
            if items or pre or post:
                launches.append((items, phase_pieces, pre, post))
            items, phase_pieces, pre, post, phase_in_launch = [], [], [], [], 0

        for ops in self.phases:
            recs, pieces, needs_tmp = [], 0, False
            for op in ops:
                if op[0] == "copy":
                    _, s_slot, s_sl, d_slot, d_sl = op
                    so, sb, sg, _ = self._geometry(metas[s_slot], s_sl)
                    do, db, dg, _ = self._geometry(metas[d_slot], d_sl)
                    assert sb == db, "local copy between boxes of different size"
                    if sb == 0:
                        continue
                    if sg is None or dg is None:
                        recs.append(("torch_copy", s_slot, s_sl, d_slot, d_sl))
                        needs_tmp = True
                        continue
                    recs.append((LOCAL, -1, s_slot, so, sg, sb, 0, 0, d_slot, do, dg))
                    pieces += pieces_of(sb, chunk, piece[min(sg[2], dg[2])], local=True)
                    continue
                kind, peer, slot, sl, flag = op
                off, nbytes, geo, bshape = self._geometry(metas[slot], sl)
                if nbytes == 0:
                    continue
                dtype = metas[slot][2]
                add_code = _ADD.get(dtype, -1) if (kind == "recv" and flag) else 0
                if geo is None or add_code < 0:
                    recs.append(("tmp", kind, int(peer), slot, sl, bool(flag), bshape, dtype, nbytes))
                    needs_tmp = True
                else:
                    recs.append((SEND if kind == "send" else RECV, int(peer), slot, off, geo, nbytes,
                                 int(bool(flag)) if kind == "send" else 0, add_code, None, 0, None))
                # (an op that goes through a contiguous temporary moves it in 16-byte units where the size allows)
                eff_unit = geo[2] if (geo is not None and add_code >= 0) else \
                    (16 if nbytes % 16 == 0 else torch.empty((), dtype=dtype).element_size())
                pieces += pieces_of(nbytes, chunk, piece[eff_unit])
            n_new = sum(1 for r in recs if r[0] != "torch_copy")
            if needs_tmp or len(items) + n_new > max_items or phase_in_launch >= 8:
                flush()
            if needs_tmp:
                # a phase with temporaries is a launch of its own: gather into contiguous buffers
                # before it, scatter / add after it
                for r in recs:
                    if r[0] == "torch_copy":
                        pre.append(r)
                    elif r[0] == "tmp":
                        _, kind, peer, slot, sl, flag, bshape, dtype, nbytes = r
                        tmp_slot = ("tmp", len(pre) + len(post) + len(items))
                        (pre if kind == "send" else post).append(("tmp_" + kind, slot, sl, flag, tmp_slot, bshape, dtype))
                        geo = ([1, 1, 1, nbytes // 16], [0, 0, 0], 16) if nbytes % 16 == 0 else \
                            ([1, 1, 1, nbytes // torch.empty((), dtype=dtype).element_size()], [0, 0, 0],
                             torch.empty((), dtype=dtype).element_size())
                        items.append((SEND if kind == "send" else RECV, peer, tmp_slot, 0, geo, nbytes, 0, 0, None, 0,
                                      None, 0))
                    else:
                        items.append(r + (0,))
                phase_pieces.append(pieces)
                flush()
                continue
            for r in recs:
                items.append(r + (phase_in_launch,))
            phase_pieces.append(pieces)
            phase_in_launch += 1
        flush()
        return launches

    # ----------------------------------------------------------------------- run
    def run(self, **tensors):
        """Runs the exchange on the tensors bound to the slots (in place on their storage)."""
        symm.require_healthy()
        st = state()
        key = tuple((k, self._meta(t)) for k, t in sorted(tensors.items()))
        launches = self._compiled.get(key)
        if launches is None:
            launches = self._compile({k: self._meta(t) for k, t in tensors.items()})
            self._compiled[key] = launches
        lib = _native.lib()
        for items, phase_pieces, pre, post in launches:
            bound = dict(tensors)
            for op in pre:
                if op[0] == "torch_copy":
                    _, s_slot, s_sl, d_slot, d_sl = op
                    _view(bound[d_slot], d_sl).copy_(_view(bound[s_slot], s_sl))
                else:
                    _, slot, sl, clear, tmp_slot, bshape, dtype = op
                    src = _view(bound[slot], sl)
                    bound[tmp_slot] = src.contiguous()
                    if clear:
                        src.zero_()
            for op in post:
                _, slot, sl, add, tmp_slot, bshape, dtype = op
                bound[tmp_slot] = torch.empty(bshape, dtype=dtype, device=bound[slot].device)
            if items:
                arr = (BoxItem * len(items))()
                for rec, it in zip(items, arr):
                    kind, peer, slot, off, geo, nbytes, clear, add, d_slot, d_off, d_geo, phase = rec
                    n, s, unit = geo
                    it.a.base = bound[slot].data_ptr() + off
                    it.a.n[:] = n
                    it.a.s[:] = s
                    it.a.lo, it.a.hi = _storage_bounds(bound[slot])
                    it.unit = unit
                    it.bytes, it.kind, it.peer, it.phase, it.clear_source, it.add = nbytes, kind, peer, phase, clear, add
                    if kind == LOCAL:
                        n2, s2, unit2 = d_geo
                        it.b.base = bound[d_slot].data_ptr() + d_off
                        it.b.n[:] = n2
                        it.b.s[:] = s2
                        it.b.lo, it.b.hi = _storage_bounds(bound[d_slot])
                        it.unit_b = unit2
                    elif kind == SEND:
                        it.first_seq = st.sent[peer] & 0xFFFFFFFF
                        st.sent[peer] += -(-nbytes // st.chunk)
                    else:
                        it.first_seq = st.received[peer] & 0xFFFFFFFF
                        st.received[peer] += -(-nbytes // st.chunk)
                targets = (_u * 8)()
                for p, n in enumerate(phase_pieces):
                    st.progress += n
                    targets[p] = st.progress & 0xFFFFFFFF
                _native.launch_count += 1
                _native.check(lib.dd_box_exchange(arr, len(items), max(1, len(phase_pieces)), targets, st.inbox, st.pads,
                                                  st.h.rank, st.slot, st.chunk, stream_ptr()), "dd_box_exchange")
            for op in post:
                _, slot, sl, add, tmp_slot, bshape, dtype = op
                dst = _view(bound[slot], sl)
                if add:
                    dst.add_(bound[tmp_slot])
                else:
                    dst.copy_(bound[tmp_slot])


    # ------------------------------------------------------------ host execution
    def run_on_host(self, transport, team, **tensors):
        """The plan executed with the kernel's own index arithmetic on the host and the messages
        carried by ``transport.exchange`` (CPU tensors).  This is the definition of what
        :meth:`run` does, in a form that runs on CPU ranks; the tests compare it with the
        slicing formulation of the primitives."""
        for ops in self.phases:
            sends, recvs, targets = [], [], []
            for op in ops:
                if op[0] == "copy":
                    _, s_slot, s_sl, d_slot, d_sl = op
                    src = _view(tensors[s_slot], s_sl)
                    if src.numel():
                        flat = torch.empty(src.numel() * src.element_size(), dtype=torch.uint8)
                        if not host_copy("send", tensors[s_slot], s_sl, flat):
                            flat = src.contiguous().view(-1).view(torch.uint8)
                        if not host_copy("recv", tensors[d_slot], d_sl, flat):
                            _view(tensors[d_slot], d_sl).copy_(flat.view(src.dtype).view(src.shape))
                    continue
                kind, peer, slot, sl, flag = op
                box = _view(tensors[slot], sl)
                if box.numel() == 0:
                    continue
                nbytes = box.numel() * box.element_size()
                if kind == "send":
                    flat = torch.empty(nbytes, dtype=torch.uint8)
                    if not host_copy("send", tensors[slot], sl, flat, clear=bool(flag)):
                        flat = box.contiguous().view(-1).view(torch.uint8)
                        if flag:
                            box.zero_()
                    sends.append((int(peer), flat))
                else:
                    recvs.append((int(peer), (nbytes,), torch.uint8))
                    targets.append((slot, sl, bool(flag)))
            got = transport.exchange(sends, recvs, list(team))
            for (slot, sl, add), flat in zip(targets, got):
                flat = flat.contiguous()
                box = _view(tensors[slot], sl)
                if not host_copy("recv", tensors[slot], sl, flat, add=add):
                    val = flat.view(box.dtype).view(box.shape)
                    box.add_(val) if add else box.copy_(val)


def _view(t, slices):
    return t if slices is None else t[tuple(slices)]


def host_copy(kind, tensor, slices, contiguous, add=False, clear=False):
    """The kernel's index arithmetic on the host (CPU tensors), for tests without a GPU: packs the
    box ``slices`` of ``tensor`` into the flat buffer ``contiguous`` (``kind="send"``) or unpacks
    the buffer into the box (``kind="recv"``).  Returns False when the box does not collapse or the host cannot add
    its dtype."""
    plan = BoxPlan([])
    off, nbytes, geo, _ = plan._geometry(BoxPlan._meta(tensor), slices)
    if geo is None or (add and tensor.dtype not in (torch.float32, torch.float64)):
        return False
    n, s, unit = geo
    it = BoxItem()
    it.a.base = tensor.data_ptr() + off
    it.a.n[:] = n
    it.a.s[:] = s
    it.unit, it.bytes, it.kind = unit, nbytes, SEND if kind == "send" else RECV
    it.clear_source = int(clear)
    it.add = _ADD.get(tensor.dtype, 0) if add else 0
    _native.check(_native.lib().dd_box_copy_host(ctypes.byref(it), contiguous.data_ptr()), "dd_box_copy_host")
    return True
