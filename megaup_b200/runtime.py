"""Symmetric-memory runtime under the two fused Ulysses exchange GEMMs.

Same public surface as the reference's ``mega_up/runtime.py`` (names,
arguments, errors), different machinery: each rank's arena is a device-local
``cuMemCreate`` allocation exported as a POSIX file descriptor, handed to the
other ranks of the node over AF_UNIX sockets and mapped by them with
``cuMemMap`` (libmegaup.so, ``mup_arena_*``). Slot hand-off uses
system-scope release/acquire flags in a control page behind each arena
(``mup_flag_barrier``) with bounded waits; there is no NCCL call on the data
path - the process group only carries host-side metadata.

A second, single-process transport emulates a UP group on one GPU with ``up``
ordinary device buffers (the way the reference's
``tests/run_pull_gemm_contention.py:191-199`` emulates peers); its barrier is
the stream order itself.
"""

from __future__ import annotations

import ctypes
import operator
import os
import socket
import threading
import uuid
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Iterator, Sequence

import torch
import torch.distributed as dist
from torch import Tensor

from . import _native

SUPPORTED_UP_DEGREES = (2, 4, 8)
# Default arena capacity in rows (B*S) per rank; pass ``max_rows`` to match the
# largest local token count.
DEFAULT_MAX_ROWS = 131_072
# Both GEMMs tile the non-exchanged output width with 256-column tiles and the
# peer-write routes 64-column sub-tiles, so the exchanged width must be a
# multiple of 256 and every rank's shard a multiple of 128.
HIDDEN_MULTIPLE = 256
SHARD_MULTIPLE = 128

_CONTROL_BYTES = 4096
_FLAG_TIMEOUT_NS = int(float(os.environ.get("MEGA_UP_FLAG_TIMEOUT_S", "30")) * 1e9)
_KERNEL_TIMEOUT_NS = int(float(os.environ.get("MEGA_UP_KERNEL_TIMEOUT_S", "5")) * 1e9)
# How the two slot hand-offs of an operation ("the slots are written" /
# "the slots may be reused") are carried out, MEGA_UP_HANDOFF:
#   lazy      (default) a peer-write keeps its two stand-alone barrier kernels; a
#             pull has one (the peers have staged), and its second hand-off
#             ("I will not read a peer arena again") is only signalled, by the
#             last pull warp to run out of tickets, long before the GEMM ends;
#             the next operation waits for it where it first touches the slots:
#             a peer-write deep inside its GEMM (before its first peer store), a
#             pull in its staging copy;
#   folded    both hand-offs ride inside the kernels (no barrier launches);
#   barriers  two stand-alone barrier kernels per operation (the reference's
#             protocol, runtime.py:264, :281, :415, :421 there).
# Measured on B200s, Wan2.1-14B projection, us per call (peer-write / pull):
# two GPUs lazy 172.3 / 191.3, barriers 172.6 / 191.9; four GPUs lazy 179.4 /
# 195.4, barriers 179.0 / 196.9. With an earlier kernel revision on two GPUs:
# barriers 182.8 / 206.2, folded 192.0 / 198.1, and with the peer-write's second
# hand-off signalled from the tail of its copy-out as well 189.1 / 196.8 (a
# copy kernel that collects arrivals and raises flags is slower than the plain
# copy plus a barrier kernel).
_HANDOFF = os.environ.get("MEGA_UP_HANDOFF") or {"1": "folded", "0": "barriers"}.get(
    os.environ.get("MEGA_UP_FUSED_SYNC", ""), "lazy"
)
if _HANDOFF not in ("lazy", "folded", "barriers"):
    raise ValueError(f"MEGA_UP_HANDOFF must be lazy, folded or barriers, got {_HANDOFF!r}")
_FUSED_SYNC = _HANDOFF == "folded"


def _wire_epoch(count: int) -> int:
    """The 32-bit value a sync point travels as. 0 means "no wait / no signal"
    in the kernels' hand-off description, so the sequence skips it when it
    wraps; waits compare by signed distance, which the gap of one does not
    disturb."""

    return (count - 1) % 0xFFFFFFFF + 1 if count > 0 else 0


def unsupported_shape_reason(width: int, up: int) -> str | None:
    """Return why ``width`` columns cannot be exchanged across ``up`` ranks,
    else ``None`` (reference: mega_up/runtime.py:32-57).

    The exchanged width is the output width of a peer-write projection and the
    input width of a pull projection.
    """

    if up not in SUPPORTED_UP_DEGREES:
        return f"UP must be one of {SUPPORTED_UP_DEGREES}, got {up}"
    if width <= 0 or width % up:
        return f"width={width} must be positive and divisible by UP={up}"
    if width % HIDDEN_MULTIPLE:
        return f"width={width} must be a multiple of {HIDDEN_MULTIPLE}"
    shard = width // up
    if shard % SHARD_MULTIPLE:
        return f"the head shard width/UP={shard} must be a multiple of {SHARD_MULTIPLE}"
    return None


def supports_shape(width: int, up: int) -> bool:
    """Whether ``width`` columns can be exchanged across ``up`` ranks."""

    return unsupported_shape_reason(width, up) is None


# --------------------------------------------------------------------------- raw memory


class _DeviceSpan:
    """A span of device memory exposed to torch through the CUDA array
    interface; keeps ``owner`` (the native arena wrapper) alive."""

    def __init__(self, address: int, nbytes: int, owner: object) -> None:
        self.address = address
        self.nbytes = nbytes
        self.owner = owner

    @property
    def __cuda_array_interface__(self) -> dict[str, object]:
        return {
            "shape": (self.nbytes // 2,),
            "typestr": "<i2",
            "data": (self.address, False),
            "version": 3,
            "strides": None,
        }

    def as_bf16(self, device: torch.device) -> Tensor:
        return torch.as_tensor(self, device=device).view(torch.bfloat16)


class _NativeArena:
    """Owns one ``mup_arena`` (a local allocation or a mapped peer)."""

    def __init__(self, handle: ctypes.c_void_p) -> None:
        self._handle = handle
        address = ctypes.c_void_p()
        nbytes = ctypes.c_uint64()
        fd = ctypes.c_int()
        _native.call(
            "mup_arena_info", handle, ctypes.byref(address), ctypes.byref(nbytes), ctypes.byref(fd)
        )
        self.address = int(address.value)
        self.nbytes = int(nbytes.value)
        self.fd = int(fd.value)

    @classmethod
    def create(cls, device_index: int, nbytes: int) -> "_NativeArena":
        handle = ctypes.c_void_p()
        _native.call("mup_arena_create", device_index, nbytes, ctypes.byref(handle))
        return cls(handle)

    @classmethod
    def import_fd(cls, device_index: int, fd: int, nbytes: int) -> "_NativeArena":
        handle = ctypes.c_void_p()
        _native.call("mup_arena_import", device_index, fd, nbytes, ctypes.byref(handle))
        return cls(handle)

    def __del__(self) -> None:
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            try:
                _native.lib().mup_arena_destroy(handle)
            except Exception:
                pass


class _StatusWord:
    """Pinned host word the kernels write an error code into."""

    def __init__(self) -> None:
        self._host = ctypes.POINTER(ctypes.c_uint32)()
        device = ctypes.c_void_p()
        _native.call("mup_status_create", ctypes.byref(self._host), ctypes.byref(device))
        self.device_address = int(device.value)

    def read(self) -> int:
        return int(self._host[0])

    def clear(self) -> None:
        self._host[0] = 0

    def __del__(self) -> None:
        host, self._host = getattr(self, "_host", None), None
        if host:
            try:
                _native.lib().mup_status_destroy(host)
            except Exception:
                pass


# --------------------------------------------------------------------------- FD exchange


def exchange_fds(group: dist.ProcessGroup | None, fd: int) -> list[int]:
    """All-gather one file descriptor per rank across the processes of a node.

    Every rank listens on an abstract AF_UNIX socket whose name is shared with
    ``all_gather_object``; each rank then connects to every peer and receives
    that peer's descriptor as SCM_RIGHTS ancillary data. Returns the list of
    descriptors indexed by rank (entry ``rank`` is ``fd`` itself); received
    descriptors belong to the caller.
    """

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    name = f"\0megaup-{os.getpid()}-{uuid.uuid4().hex}"
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(name)
    server.listen(world)
    server.settimeout(120.0)

    def serve() -> None:
        for _ in range(world - 1):
            connection, _ = server.accept()
            with connection:
                connection.recv(16)
                socket.send_fds(connection, [b"fd"], [fd])

    thread = threading.Thread(target=serve, daemon=True)
    thread.start()
    names: list[object] = [None] * world
    dist.all_gather_object(names, (rank, name), group=group)
    received = [-1] * world
    received[rank] = fd
    try:
        for entry in names:
            peer, peer_name = entry  # type: ignore[misc]
            if peer == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                client.settimeout(120.0)
                client.connect(peer_name)
                client.sendall(str(rank).encode().ljust(16))
                _, fds, _, _ = socket.recv_fds(client, 16, 1)
                if len(fds) != 1:
                    raise RuntimeError(f"rank {peer} did not send a file descriptor")
                received[peer] = fds[0]
        thread.join(timeout=120.0)
    finally:
        server.close()
    return received


# --------------------------------------------------------------------------- runtime


def _group_key(group: object) -> str:
    name = getattr(group, "group_name", None)
    return str(name) if name is not None else f"process-group-{id(group)}"


@dataclass
class MegaUPRuntime:
    """One reusable BF16 symmetric arena for an explicit UP process group.

    The arena holds ``max_rows * hidden`` elements per rank. An operation
    exchanging ``rows`` rows of ``width`` elements fits when
    ``rows * width <= max_rows * hidden`` (reference: runtime.py:115-225).
    """

    group: object
    arena: Tensor
    handle: object
    peer_buffers: tuple[Tensor, ...]
    peer_address_table: Tensor
    max_rows: int
    hidden: int
    local_rank: int
    up: int
    emulated: bool = False
    _flag_addresses: tuple[int, ...] = field(default=(), repr=False)
    _status: _StatusWord | None = field(default=None, repr=False)
    _epoch: int = field(default=0, init=False, repr=False)
    _done_counter: Tensor | None = field(default=None, init=False, repr=False)
    _flag_array: object = field(default=None, init=False, repr=False)
    _done_value: int = field(default=0, init=False, repr=False)
    _leased: bool = field(default=False, init=False, repr=False)
    _leased_stream: int | None = field(default=None, init=False, repr=False)
    _lease_lock: threading.Lock = field(default_factory=threading.Lock, init=False, repr=False)
    _completion_event: torch.cuda.Event | None = field(default=None, init=False, repr=False)
    _completion_stream: int | None = field(default=None, init=False, repr=False)
    _spare_event: torch.cuda.Event | None = field(default=None, init=False, repr=False)
    # device-side failures observed so far; pull executables compare it with the
    # count they last saw and zero their counters after a failure
    failure_count: int = field(default=0, init=False, repr=False)
    # kind of the operation that last used the arena ("peer_write" / "pull"): a
    # lazily handed-off operation leaves its second sync point to its successor
    _last_operation: str | None = field(default=None, init=False, repr=False)

    @property
    def shard_hidden(self) -> int:
        return self.hidden // self.up

    @property
    def device(self) -> torch.device:
        return self.arena.device

    @property
    def arena_nbytes(self) -> int:
        return self.arena.numel() * self.arena.element_size()

    @property
    def status_address(self) -> int:
        return 0 if self._status is None else self._status.device_address

    @property
    def kernel_timeout_ns(self) -> int:
        return _KERNEL_TIMEOUT_NS

    def _stream(self) -> int:
        # inside a lease the operation's stream was looked up once, on entry
        handle = self._leased_stream
        return handle if handle is not None else torch.cuda.current_stream(self.device).cuda_stream

    @property
    def handoff(self) -> str:
        """``"lazy"``, ``"folded"`` or ``"barriers"`` (see ``MEGA_UP_HANDOFF``); an
        emulated single-process group needs none: its stream order is the hand-off."""

        return "none" if self.emulated else _HANDOFF

    @property
    def fused_sync(self) -> bool:
        """Whether both slot hand-offs ride inside the kernels (multi-process runtimes)."""

        return self.handoff == "folded"

    def _sync(self, *, wait: bool, signal: bool) -> "_native.MupSync":
        """Hand-off description for one kernel: ``wait`` for the sync point reached
        so far before its first access to the slots, ``signal`` the next sync
        point from its last CTA. Sync points are numbered alike on every rank
        (every rank issues the same operations in the same order)."""

        if self._done_counter is None:
            self._done_counter = torch.zeros(1, dtype=torch.int64, device=self.device)
        self._peer_flag_array()
        sync = _native.MupSync(
            peer_flags=self._flag_array,
            up=self.up,
            rank=self.local_rank,
            wait_epoch=_wire_epoch(self._epoch) if wait else 0,
            signal_epoch=_wire_epoch(self._epoch + 1) if signal else 0,
            done_counter=self._done_counter.data_ptr(),
            done_before=self._done_value,
            done_after=0,
            status_device_ptr=self.status_address or None,
            timeout_ns=_FLAG_TIMEOUT_NS,
        )
        if signal:
            self._epoch += 1
        return sync

    def _peer_flag_array(self) -> object:
        """The peers' flag addresses as a C array, built once."""

        if self._flag_array is None:
            self._flag_array = _native.pointer_array(self._flag_addresses)
        return self._flag_array

    def _next_handoff(self) -> "_native.MupSync":
        """Folded protocol: the next kernel of an operation waits for the sync point
        reached so far and signals the next one. Every operation launches two
        such kernels (peer-write: GEMM, copy-out; pull: staging copy, GEMM), so
        an operation still spans two sync points, as with explicit barriers."""

        return self._sync(wait=True, signal=True)

    def _copy(self, name: str, *args: object, sync: "_native.MupSync | None" = None) -> None:
        """Launch a layout copy, with a hand-off folded in when ``sync`` is given."""

        if sync is None:
            _native.call(name, *args, self._stream())
            return
        _native.call(name + "_synced", *args, self._stream(), ctypes.byref(sync))
        self._done_value = int(sync.done_after)

    def _copy_out_sync(self) -> "_native.MupSync | None":
        """Hand-off folded into a copy-out of peer-written slots (folded protocol
        only; otherwise barrier kernels stand before and behind the copy)."""

        if self.handoff == "folded":
            return self._sync(wait=True, signal=True)
        return None

    def _stage_sync(self) -> "_native.MupSync | None":
        """Hand-off of a staging copy into this rank's own slots. Lazy: the peers
        must have finished pulling the previous contents, which only a previous
        PULL leaves open (after a peer-write this rank read the slots itself,
        earlier on this stream)."""

        if self.handoff == "folded":
            return self._sync(wait=True, signal=True)
        if self.handoff == "lazy" and self._last_operation == "pull":
            return self._sync(wait=True, signal=False)
        return None

    def check_status(self) -> None:
        """Raise if a kernel of an earlier operation gave up on a bounded wait.

        The status word is written by the device; call after the stream has
        been synchronised to observe the outcome of the latest operation.
        """

        if self._status is None:
            return
        word = self._status.read()
        if word:
            self._status.clear()
            self.failure_count += 1
            raise RuntimeError(
                f"Mega-UP device-side failure: {_native.decode_status(word)}; the results of the "
                "operations enqueued since the last check are invalid (the next operation resets "
                "the pull counters)"
            )

    @contextmanager
    def lease(self) -> Iterator["MegaUPRuntime"]:
        """Non-re-entrant use of the arena; consecutive operations may run on
        different streams (reference: runtime.py:151-171).

        The status word the kernels write when a bounded wait runs out is read
        on entry and after the operation has been enqueued (a plain host load of
        pinned memory, no synchronisation): a failure of an EARLIER operation
        raises ``RuntimeError`` here, at the next operation, so that a caller who
        never calls ``check_status()`` still hears of it."""

        self.check_status()
        stream = torch.cuda.current_stream(self.device)
        handle = stream.cuda_stream
        with self._lease_lock:
            if self._leased:
                raise RuntimeError(
                    "Mega-UP arena was re-entered before the previous operation completed"
                )
            self._leased = True
            previous, previous_stream = self._completion_event, self._completion_stream
        # the same stream orders the operations by itself
        if previous is not None and previous_stream != handle:
            stream.wait_event(previous)
        self._leased_stream = handle
        try:
            yield self
            self.check_status()
        finally:
            self._leased_stream = None
            # Two event objects take turns: a wait enqueued on the one recorded by
            # the previous operation keeps referring to that record, so the other
            # one can be recorded again now.
            done = self._spare_event or torch.cuda.Event()
            done.record(stream)
            with self._lease_lock:
                self._spare_event = self._completion_event
                self._completion_event = done
                self._completion_stream = handle
                self._leased = False

    def barrier(self, *, timeout_s: float | None = None) -> None:
        """All-peer slot hand-off on the current stream (reference: runtime.py:108-112).

        The device-side wait is bounded (``MEGA_UP_FLAG_TIMEOUT_S``, 30 s, or
        ``timeout_s``): a peer that never arrives makes the kernel end with a
        status code that ``check_status()`` raises, instead of hanging the GPU.
        """

        if self.emulated:
            return  # one process drives every emulated rank on one stream
        self._epoch += 1
        _native.call(
            "mup_flag_barrier",
            self._peer_flag_array(),
            self.up,
            self.local_rank,
            _wire_epoch(self._epoch),
            self.status_address,
            _FLAG_TIMEOUT_NS if timeout_s is None else int(timeout_s * 1e9),
            self._stream(),
        )

    def check_capacity(self, rows: int, width: int) -> None:
        """Check that ``rows`` rows of ``width`` elements fit the arena."""

        if rows <= 0 or width <= 0 or width % self.up:
            raise ValueError(
                "rows and width must be positive and width divisible by "
                f"UP={self.up}, got rows={rows}, width={width}"
            )
        if rows * width > self.max_rows * self.hidden:
            raise ValueError(
                f"{rows} rows of {width} elements exceed the arena of "
                f"max_rows*hidden={self.max_rows}*{self.hidden} elements per rank"
            )

    def _packed(self, buffer: Tensor, rows: int, width: int) -> Tensor:
        shard = width // self.up
        return buffer.view(-1).narrow(0, 0, self.up * rows * shard).view(self.up, rows, shard)

    def slots(self, rows: int, width: int | None = None) -> Tensor:
        """``[UP, rows, width/UP]`` view of the densely packed arena slots: slot
        ``p`` starts at element ``p * rows * width/UP`` whatever the arena's
        nominal shape (reference: runtime.py:190-205)."""

        width = self.hidden if width is None else int(width)
        self.check_capacity(rows, width)
        return self._packed(self.arena, rows, width)

    def remote_write_views(self, rows: int, width: int | None = None) -> tuple[Tensor, ...]:
        """This source rank's ``[rows, width/UP]`` slot in every peer arena
        (reference: runtime.py:207-225)."""

        width = self.hidden if width is None else int(width)
        self.check_capacity(rows, width)
        return tuple(self._packed(peer, rows, width)[self.local_rank] for peer in self.peer_buffers)

    # ----- slot <-> user layout copies (libmegaup.so, HBM-bound) -----

    def _regroup(
        self, dst: Tensor, src: Tensor, batch: int, sequence: int, shard: int, to_batch_major: bool,
        sync: "_native.MupSync | None" = None,
    ) -> None:
        if batch == 1:
            # source-major and batch-major coincide: one straight copy
            self._copy(
                "mup_gather_rows", dst.data_ptr(), src.data_ptr(), None, self.up * sequence, shard,
                sync=sync,
            )
        else:
            self._copy(
                "mup_regroup_rows", dst.data_ptr(), src.data_ptr(), self.up, batch, sequence, shard,
                1 if to_batch_major else 0, sync=sync,
            )

    def copy_peer_written(
        self,
        *,
        batch: int,
        sequence: int,
        shard_heads: int,
        head_dim: int,
        out: Tensor | None = None,
        _managed: bool = False,
    ) -> Tensor:
        """Materialize compact peer writes as ``[B,UP*S,H/UP,D]``: barrier,
        copy, barrier (reference: runtime.py:227-282). ``_managed`` (used by the
        prepared executables) follows the runtime's hand-off protocol instead:
        the copy kernel then hands the slots back from its last block."""

        rows = int(batch) * int(sequence)
        shard = int(shard_heads) * int(head_dim)
        width = self.up * shard
        self.check_capacity(rows, width)
        expected = (batch, self.up * sequence, shard_heads, head_dim)
        if out is None:
            out = torch.empty(expected, dtype=self.arena.dtype, device=self.arena.device)
        elif (
            tuple(out.shape) != expected
            or out.dtype != self.arena.dtype
            or out.device != self.arena.device
            or not out.is_contiguous()
        ):
            raise ValueError(
                f"out must be a contiguous BF16 tensor on the runtime device with shape {expected}"
            )
        if _managed and self.handoff == "folded":
            self._regroup(out, self.slots(rows, width), batch, sequence, shard, True, sync=self._copy_out_sync())
            return out
        self.barrier()
        self._regroup(out, self.slots(rows, width), batch, sequence, shard, True)
        self.barrier()
        return out

    def _check_row_index(self, index: Tensor, rows: int) -> None:
        total = self.up * rows
        if (
            not isinstance(index, Tensor)
            or index.ndim != 1
            or index.numel() != total
            or index.dtype != torch.int64
            or index.device != self.device
            or not index.is_contiguous()
        ):
            raise ValueError(
                f"index must be a 1-D int64 tensor with UP*rows={total} entries on the runtime device"
            )

    def copy_peer_written_indexed(
        self, *, rows: int, index: Tensor, out: Tensor, _managed: bool = False
    ) -> Tensor:
        """Output row ``i`` receives source-major arena row ``index[i]``
        (reference: runtime.py:298-337)."""

        self._check_row_index(index, rows)
        total = self.up * rows
        if (
            out.dtype != self.arena.dtype
            or out.device != self.arena.device
            or not out.is_contiguous()
            or out.numel() == 0
            or out.numel() % total
        ):
            raise ValueError(
                "out must be a contiguous BF16 tensor on the runtime device "
                f"with a multiple of UP*rows={total} elements"
            )
        shard = out.numel() // total
        self.check_capacity(rows, self.up * shard)
        args = (out.data_ptr(), self.slots(rows, self.up * shard).data_ptr(), index.data_ptr(), total, shard)
        if _managed and self.handoff == "folded":
            self._copy("mup_gather_rows", *args, sync=self._copy_out_sync())
            return out
        self.barrier()
        self._copy("mup_gather_rows", *args)
        self.barrier()
        return out

    def stage_rows_indexed(
        self, *, rows: int, source: Tensor, index: Tensor, _managed: bool = False
    ) -> None:
        """Slot row ``(d, j)`` receives ``source[index[d*rows + j]]``, then
        barrier (reference: runtime.py:339-373)."""

        self._check_row_index(index, rows)
        total = self.up * rows
        if (
            source.ndim != 2
            or int(source.shape[0]) != total
            or source.dtype != self.arena.dtype
            or source.device != self.arena.device
            or not source.is_contiguous()
        ):
            raise ValueError(
                "source must be a contiguous 2-D BF16 tensor on the runtime "
                f"device with UP*rows={total} rows"
            )
        shard = int(source.shape[1])
        self._copy(
            "mup_gather_rows", self.slots(rows, self.up * shard).data_ptr(), source.data_ptr(),
            index.data_ptr(), total, shard, sync=self._stage_sync() if _managed else None,
        )
        if not (_managed and self.handoff == "folded"):
            self.barrier()

    def stage_head_parallel(self, tensor: Tensor, _managed: bool = False) -> tuple[int, int, int, int]:
        """Stage ``[B,UP*S,H/UP,D]`` as ``[destination, B*S, H/UP*D]`` slots,
        then barrier (reference: runtime.py:375-416)."""

        if tensor.ndim != 4:
            raise ValueError(
                f"head-parallel input must be [B,UP*S,H/UP,D], got {tuple(tensor.shape)}"
            )
        batch, global_sequence, shard_heads, head_dim = map(int, tensor.shape)
        if global_sequence % self.up:
            raise ValueError(
                f"sequence dimension {global_sequence} is not divisible by UP={self.up}"
            )
        sequence = global_sequence // self.up
        shard = shard_heads * head_dim
        rows = batch * sequence
        self._regroup(
            self.slots(rows, self.up * shard), tensor, batch, sequence, shard, False,
            sync=self._stage_sync() if _managed else None,
        )
        if not (_managed and self.handoff == "folded"):
            self.barrier()
        return batch, sequence, shard_heads, head_dim

    def finish_pull(self) -> None:
        """Keep the arena from being reused until every peer pull has completed."""

        self.barrier()


# One runtime per process group and ``hidden``.
_RUNTIMES: dict[tuple[str, int], MegaUPRuntime] = {}


def _gather_phase_errors(group, up: int, device: torch.device, phase: str, local_error: str | None) -> None:
    records: list[object] = [None] * up
    with torch.cuda.device(device):
        dist.all_gather_object(records, (phase, local_error), group=group)
    errors = tuple(
        (rank, record[1]) for rank, record in enumerate(records)
        if isinstance(record, tuple) and record[1] is not None
    )
    if errors:
        raise RuntimeError(f"Mega-UP {phase} failed: {errors}")


def _arena_bytes(max_rows: int, hidden: int) -> int:
    data = max_rows * hidden * 2
    return (data + _CONTROL_BYTES - 1) // _CONTROL_BYTES * _CONTROL_BYTES


def initialize_runtime(
    group: dist.ProcessGroup,
    *,
    hidden: int,
    max_rows: int = DEFAULT_MAX_ROWS,
    device: torch.device | str | None = None,
) -> MegaUPRuntime:
    """Collectively allocate the runtime for ``group`` (reference:
    runtime.py:452-654): same arguments on every rank, one runtime per
    ``(group, hidden)``; a repeated call returns the existing runtime and must
    repeat its ``max_rows`` and device. A rank-local bad argument raises
    ``ValueError`` on every rank before anything is allocated.
    """

    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized")
    up = dist.get_world_size(group)
    local_rank = dist.get_rank(group)
    current = torch.device("cuda", torch.cuda.current_device())
    key_group = _group_key(group)
    normalized: torch.device | None = None
    local_error: str | None = None
    try:
        hidden = operator.index(hidden)
        reason = unsupported_shape_reason(hidden, up)
        if reason is not None:
            raise ValueError(f"hidden: {reason}")
        if max_rows <= 0:
            raise ValueError(f"max_rows must be positive, got {max_rows}")
        normalized = current if device is None else torch.device(device)
        if normalized.type != "cuda":
            raise ValueError(f"Mega-UP requires a CUDA device, got {normalized}")
        ordinal = current.index if normalized.index is None else normalized.index
        if ordinal is None or not 0 <= ordinal < torch.cuda.device_count():
            raise ValueError(f"invalid CUDA device ordinal {ordinal}")
        normalized = torch.device("cuda", ordinal)
        if normalized != current:
            raise ValueError(
                "runtime device must be the process's current CUDA device: "
                f"requested {normalized}, current {current}"
            )
    except (RuntimeError, TypeError, ValueError) as error:
        local_error = f"{type(error).__name__}: {error}"
    existing = _RUNTIMES.get((key_group, hidden)) if local_error is None else None
    compatible = local_error is None and (
        existing is None
        or (existing.max_rows == max_rows and existing.up == up and existing.device == normalized)
    )
    record = (
        repr(hidden),
        repr(max_rows),
        up,
        None if normalized is None else normalized.type,
        existing is not None,
        compatible,
        local_error,
    )
    records: list[object] = [None] * up
    with torch.cuda.device(current):
        dist.all_gather_object(records, record, group=group)
    errors = tuple(
        (rank, item[6]) for rank, item in enumerate(records) if item is not None and item[6] is not None
    )
    if errors:
        raise ValueError(f"Mega-UP runtime collective validation failed: {errors}")
    if any(item is None or item[:4] != record[:4] for item in records):
        raise ValueError(
            "all UP ranks must initialize Mega-UP with identical hidden, "
            "max_rows, degree, and device type"
        )
    if len({bool(item[4]) for item in records}) != 1:
        raise RuntimeError("Mega-UP runtime cache state differs across ranks")
    if any(not item[5] for item in records):
        raise RuntimeError(
            f"the group already has a Mega-UP runtime for hidden={hidden} "
            "with a different max_rows or device"
        )
    if existing is not None:
        return existing

    assert normalized is not None
    device = normalized
    data_bytes = max_rows * hidden * 2
    control_offset = _arena_bytes(max_rows, hidden)
    local: _NativeArena | None = None
    error: str | None = None
    try:
        local = _NativeArena.create(device.index, control_offset + _CONTROL_BYTES)
    except Exception as exc:  # noqa: BLE001 - reported collectively
        error = f"{type(exc).__name__}: {exc}"
    _gather_phase_errors(group, up, current, "symmetric allocation", error)
    assert local is not None

    mapped: list[_NativeArena | None] = [None] * up
    error = None
    try:
        # every rank maps the same number of bytes: sizes agree because the
        # arguments agree (checked above)
        fds = exchange_fds(group, local.fd)
        for peer in range(up):
            if peer == local_rank:
                mapped[peer] = local
            else:
                mapped[peer] = _NativeArena.import_fd(device.index, fds[peer], local.nbytes)
                os.close(fds[peer])
    except Exception as exc:  # noqa: BLE001
        error = f"{type(exc).__name__}: {exc}"
    _gather_phase_errors(group, up, current, "symmetric rendezvous", error)

    error = None
    runtime: MegaUPRuntime | None = None
    try:
        shape = (up, max_rows, hidden // up)
        peer_buffers = tuple(
            _DeviceSpan(m.address, data_bytes, m).as_bf16(device).view(shape) for m in mapped  # type: ignore[union-attr]
        )
        table = torch.tensor(
            [m.address for m in mapped], dtype=torch.int64, device=device  # type: ignore[union-attr]
        ).view(torch.uint64)
        runtime = MegaUPRuntime(
            group=group,
            arena=peer_buffers[local_rank],
            handle=tuple(mapped),
            peer_buffers=peer_buffers,
            peer_address_table=table,
            max_rows=max_rows,
            hidden=hidden,
            local_rank=local_rank,
            up=up,
            _flag_addresses=tuple(m.address + control_offset for m in mapped),  # type: ignore[union-attr]
            _status=_StatusWord(),
        )
        runtime.barrier()
        torch.cuda.synchronize(device)
        runtime.check_status()
    except Exception as exc:  # noqa: BLE001
        error = f"{type(exc).__name__}: {exc}"
    _gather_phase_errors(group, up, current, "peer buffer binding", error)
    assert runtime is not None
    _RUNTIMES[(key_group, hidden)] = runtime
    return runtime


def initialize_emulated_group(
    up: int,
    *,
    hidden: int,
    max_rows: int = DEFAULT_MAX_ROWS,
    device: torch.device | str | None = None,
) -> tuple[MegaUPRuntime, ...]:
    """``up`` runtimes in ONE process on ONE GPU, sharing ``up`` ordinary
    device arenas: rank ``r``'s kernels store into / load from the other
    runtimes' arenas through plain device pointers. For single-GPU tests and
    measurements; drive the ranks phase by phase (see ``ops.emulated_*``)."""

    reason = unsupported_shape_reason(operator.index(hidden), up)
    if reason is not None:
        raise ValueError(f"hidden: {reason}")
    if max_rows <= 0:
        raise ValueError(f"max_rows must be positive, got {max_rows}")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    arenas = tuple(
        torch.zeros((up, max_rows, hidden // up), dtype=torch.bfloat16, device=device)
        for _ in range(up)
    )
    table = torch.tensor([a.data_ptr() for a in arenas], dtype=torch.int64, device=device).view(
        torch.uint64
    )
    status = _StatusWord()
    return tuple(
        MegaUPRuntime(
            group=None,
            arena=arenas[rank],
            handle=None,
            peer_buffers=arenas,
            peer_address_table=table,
            max_rows=max_rows,
            hidden=hidden,
            local_rank=rank,
            up=up,
            emulated=True,
            _status=status,
        )
        for rank in range(up)
    )


__all__ = [
    "DEFAULT_MAX_ROWS",
    "HIDDEN_MULTIPLE",
    "SHARD_MULTIPLE",
    "SUPPORTED_UP_DEGREES",
    "MegaUPRuntime",
    "initialize_emulated_group",
    "initialize_runtime",
    "supports_shape",
    "unsupported_shape_reason",
]
