"""BSHD, SBHD and packed-THD host APIs of the two fused Ulysses exchange GEMMs.

Drop-in for the reference's ``mega_up/ops.py``: the same public functions,
``Prepared*`` classes, ``THDLayout``, argument meaning and error behaviour
(local contract failure -> ``ValueError``; with ``validate_group=True`` the
error is gathered and raised on every rank before any device barrier; set-up
failure -> ``RuntimeError``; wrong layout type -> ``TypeError``). The three
layouts differ only in how rows are counted and how the slots are copied to or
from the user tensor, so they share one implementation here.

Every operation has two phases separated by the slot hand-off barrier:
peer-write = launch, then materialise; pull = stage, then launch. A
multi-process runtime runs both inside ``__call__``; a single-process emulated
group (``runtime.initialize_emulated_group``) runs phase 1 for every rank
before phase 2 (``emulated_peer_write`` / ``emulated_pull``).
"""

from __future__ import annotations

import hashlib
import struct
from collections.abc import Sequence
from dataclasses import dataclass

import torch
import torch.distributed as dist
from torch import Tensor

from .runtime import HIDDEN_MULTIPLE, MegaUPRuntime, unsupported_shape_reason

# --------------------------------------------------------------------------- layout contract


def _source_major_to_bshd(
    source_major: Tensor, *, batch: int, sequence: int, shard_heads: int, head_dim: int
) -> Tensor:
    """``[source, B*S, H/UP*D]`` -> ``[B, UP*S, H/UP, D]`` (reference: ops.py:23-53)."""

    if source_major.ndim != 3:
        raise ValueError("source_major must be a 3-D tensor")
    up = int(source_major.shape[0])
    expected = (up, batch * sequence, shard_heads * head_dim)
    if tuple(source_major.shape) != expected:
        raise ValueError(f"source_major must have shape {expected}, got {tuple(source_major.shape)}")
    grouped = source_major.view(up, batch, sequence, shard_heads, head_dim).transpose(0, 1)
    return grouped.reshape(batch, up * sequence, shard_heads, head_dim).contiguous()


def _bshd_to_destination_major(head_parallel: Tensor, *, up: int, sequence: int) -> Tensor:
    """``[B, UP*S, H/UP, D]`` -> ``[destination, B*S, H/UP*D]`` (reference: ops.py:56-89)."""

    if head_parallel.ndim != 4:
        raise ValueError("head_parallel must be a 4-D tensor")
    batch, global_sequence, shard_heads, head_dim = map(int, head_parallel.shape)
    if global_sequence != up * sequence:
        raise ValueError(f"sequence dimension must be UP*S={up * sequence}, got {global_sequence}")
    grouped = head_parallel.view(batch, up, sequence, shard_heads, head_dim).transpose(0, 1)
    return grouped.reshape(up, batch * sequence, shard_heads * head_dim).contiguous()


def _normalize_cu_seqlens(cu_seqlens: Tensor | Sequence[int]) -> tuple[int, ...]:
    """Validate rank-local packed boundaries; return host ints (reference: ops.py:97-119)."""

    if isinstance(cu_seqlens, Tensor):
        if cu_seqlens.ndim != 1:
            raise ValueError("cu_seqlens must be a 1-D tensor")
        if cu_seqlens.dtype not in (torch.int32, torch.int64):
            raise ValueError("cu_seqlens must be an int32 or int64 tensor")
        values = tuple(int(v) for v in cu_seqlens.tolist())
    else:
        values = tuple(int(v) for v in cu_seqlens)
    if len(values) < 2:
        raise ValueError("cu_seqlens needs at least one sample, e.g. [0, T]")
    if values[0] != 0:
        raise ValueError(f"cu_seqlens[0] must be 0, got {values[0]}")
    if any(b < a for a, b in zip(values, values[1:])):
        raise ValueError("cu_seqlens must be non-decreasing")
    if values[-1] <= 0:
        raise ValueError("cu_seqlens[-1], the local token count, must be positive")
    return values


@dataclass(frozen=True)
class THDLayout:
    """Per-sample regroup for the split-sample packing scheme (reference: ops.py:122-153).

    The default THD contract needs no layout: every rank holds a contiguous
    slab of the global packed stream and the head-parallel tensor is already
    in global order. Use a layout when every sample is instead split evenly
    across the UP group, so that all ranks share the same rank-local
    ``cu_seqlens``. Arena order is source-major (row ``r*T + j`` = local row
    ``j`` of source rank ``r``); regrouped order keeps each sample contiguous
    with its UP chunks in rank order, so the public boundaries are
    ``cu_seqlens_out = UP * cu_seqlens``.
    """

    up: int
    tokens: int
    cu_seqlens: tuple[int, ...]
    to_thd_index: Tensor
    to_source_major_index: Tensor
    fingerprint: str

    @property
    def num_samples(self) -> int:
        return len(self.cu_seqlens) - 1

    @property
    def cu_seqlens_out(self) -> tuple[int, ...]:
        return tuple(self.up * v for v in self.cu_seqlens)

    @property
    def device(self) -> torch.device:
        return self.to_thd_index.device


def _build_thd_layout(
    cu_seqlens: Tensor | Sequence[int], *, up: int, device: torch.device | str | None
) -> THDLayout:
    """Source-major row ``r*T + j`` (sample ``s`` spanning local ``[a, b)``) lives at
    regrouped row ``UP*a + r*(b - a) + (j - a)``; ``to_thd_index`` is the
    inverse permutation (reference: ops.py:156-200)."""

    if up <= 0:
        raise ValueError(f"up must be positive, got {up}")
    cu = _normalize_cu_seqlens(cu_seqlens)
    tokens = cu[-1]
    bounds = torch.tensor(cu, dtype=torch.int64, device=device)
    starts, lengths = bounds[:-1], bounds[1:] - bounds[:-1]
    row = torch.arange(tokens, dtype=torch.int64, device=device)
    sample = torch.searchsorted(bounds[1:].contiguous(), row, right=True)
    start, length = starts[sample], lengths[sample]
    ranks = torch.arange(up, dtype=torch.int64, device=device).unsqueeze(1)
    to_source_major = (up * start + (row - start) + ranks * length).reshape(-1)
    to_thd = torch.empty_like(to_source_major)
    to_thd[to_source_major] = torch.arange(up * tokens, dtype=torch.int64, device=device)
    fingerprint = hashlib.sha1(struct.pack(f"<{len(cu)}q", *cu)).hexdigest()
    return THDLayout(
        up=up,
        tokens=tokens,
        cu_seqlens=cu,
        to_thd_index=to_thd,
        to_source_major_index=to_source_major,
        fingerprint=fingerprint,
    )


def prepare_thd_layout(cu_seqlens: Tensor | Sequence[int], runtime: MegaUPRuntime) -> THDLayout:
    """Build the split-sample regroup permutations for ``runtime`` (reference: ops.py:203-219).

    ``cu_seqlens`` are rank-local boundaries in tokens, identical on every UP
    rank. Build once per step and reuse for every layer; a CUDA ``cu_seqlens``
    is synchronised to the host here.
    """

    return _build_thd_layout(cu_seqlens, up=runtime.up, device=runtime.device)


def _source_major_to_thd(
    source_major: Tensor, layout: THDLayout, *, shard_heads: int, head_dim: int
) -> Tensor:
    """``[source, T, H/UP*D]`` -> packed ``[UP*T, H/UP, D]`` (reference: ops.py:222-242)."""

    expected = (layout.up, layout.tokens, shard_heads * head_dim)
    if tuple(source_major.shape) != expected:
        raise ValueError(f"source_major must have shape {expected}, got {tuple(source_major.shape)}")
    total = layout.up * layout.tokens
    flat = source_major.reshape(total, shard_heads * head_dim)
    return flat.index_select(0, layout.to_thd_index).view(total, shard_heads, head_dim)


def _thd_to_destination_major(head_parallel: Tensor, layout: THDLayout) -> Tensor:
    """Packed ``[UP*T, H/UP, D]`` -> ``[destination, T, H/UP*D]`` (reference: ops.py:245-264)."""

    if head_parallel.ndim != 3:
        raise ValueError("head_parallel must be a 3-D THD tensor")
    total = layout.up * layout.tokens
    if int(head_parallel.shape[0]) != total:
        raise ValueError(
            f"head_parallel must have UP*T={total} rows, got {int(head_parallel.shape[0])}"
        )
    shard = int(head_parallel.shape[1]) * int(head_parallel.shape[2])
    flat = head_parallel.reshape(total, shard)
    return flat.index_select(0, layout.to_source_major_index).view(layout.up, layout.tokens, shard)


# --------------------------------------------------------------------------- validation


def _tensor_signature(tensor: object) -> tuple[object, ...]:
    if not isinstance(tensor, Tensor):
        return ("not-a-tensor", type(tensor).__name__)
    return (
        tuple(int(v) for v in tensor.shape),
        str(tensor.dtype),
        tensor.device.type,
        bool(tensor.is_contiguous()),
    )


def _optional_signature(tensor: Tensor | None) -> tuple[object, ...] | None:
    return None if tensor is None else _tensor_signature(tensor)


def _layout_fingerprint(layout: object) -> str | None:
    return layout.fingerprint if isinstance(layout, THDLayout) else None


def _check_runtime_device(runtime: MegaUPRuntime) -> None:
    capability = torch.cuda.get_device_capability(runtime.device)
    if capability[0] != 10:
        raise ValueError(
            f"Mega-UP kernels do not support this GPU (compute capability {capability})"
        )


def _check_weight(weight: object, runtime: MegaUPRuntime) -> tuple[int, int]:
    if not isinstance(weight, Tensor) or weight.ndim != 2 or min(weight.shape) <= 0:
        raise ValueError(
            "weight must be a non-empty [out_features, in_features] tensor, "
            f"got {_tensor_signature(weight)}"
        )
    if weight.dtype != torch.bfloat16 or weight.device != runtime.device or not weight.is_contiguous():
        raise ValueError("weight must be contiguous BF16 on the runtime device")
    return int(weight.shape[0]), int(weight.shape[1])


def _check_exchanged_width(width: int, runtime: MegaUPRuntime, name: str) -> None:
    reason = unsupported_shape_reason(width, runtime.up)
    if reason is not None:
        raise ValueError(f"{name}: {reason}")


def _check_peer_weight(weight: object, runtime: MegaUPRuntime, head_dim: int) -> tuple[int, int]:
    """The output width N is exchanged: every rank receives N/UP columns holding
    whole ``head_dim``-wide heads; K only needs 16-byte rows for TMA."""

    n, k = _check_weight(weight, runtime)
    _check_exchanged_width(n, runtime, "peer-write out_features")
    if n % (runtime.up * head_dim):
        raise ValueError(
            f"out_features={n} must be a multiple of UP*head_dim={runtime.up * head_dim}"
        )
    if k % 8:
        raise ValueError(f"in_features={k} must be a multiple of 8")
    return n, k


def _check_pull_weight(weight: object, runtime: MegaUPRuntime, head_dim: int) -> tuple[int, int]:
    """The input width K is exchanged; N is tiled by 256 and returned as N/head_dim heads."""

    n, k = _check_weight(weight, runtime)
    _check_exchanged_width(k, runtime, "pull in_features")
    if n % HIDDEN_MULTIPLE or n % head_dim:
        raise ValueError(
            f"out_features={n} must be a multiple of {HIDDEN_MULTIPLE} and of head_dim={head_dim}"
        )
    return n, k


def _check_bias(bias: object, runtime: MegaUPRuntime, out_features: int) -> None:
    if bias is None:
        return
    if not isinstance(bias, Tensor) or tuple(bias.shape) != (out_features,):
        raise ValueError(f"bias must have shape ({out_features},), got {_tensor_signature(bias)}")
    if bias.dtype != torch.bfloat16 or bias.device != runtime.device or not bias.is_contiguous():
        raise ValueError("bias must be contiguous BF16 on the runtime device")
    if bias.data_ptr() % 16:
        raise ValueError("bias must be 16-byte aligned")


def _check_layout(layout: object, runtime: MegaUPRuntime) -> None:
    if not isinstance(layout, THDLayout):
        raise TypeError("layout must be a THDLayout from prepare_thd_layout")
    if layout.up != runtime.up:
        raise ValueError(f"THD layout was built for UP={layout.up}, runtime has UP={runtime.up}")
    if layout.device != runtime.device:
        raise ValueError(f"THD layout lives on {layout.device}, runtime on {runtime.device}")


def _check_activation(tensor: Tensor, runtime: MegaUPRuntime, name: str) -> None:
    if tensor.dtype != torch.bfloat16 or tensor.device != runtime.device or not tensor.is_contiguous():
        raise ValueError(f"{name} must be contiguous BF16 on the runtime device")


def _check_out(out: Tensor | None, expected: tuple[int, ...], runtime: MegaUPRuntime) -> None:
    if out is not None and (
        tuple(out.shape) != expected
        or out.dtype != torch.bfloat16
        or out.device != runtime.device
        or not out.is_contiguous()
    ):
        raise ValueError(
            "out must be contiguous BF16 on the runtime device with "
            f"shape {expected}, got {_tensor_signature(out)}"
        )


def _weight_widths(weight: object) -> tuple[int, int]:
    if not isinstance(weight, Tensor) or weight.ndim != 2:
        raise ValueError(
            "weight must be a 2-D [out_features, in_features] tensor, got "
            f"{_tensor_signature(weight)}"
        )
    return int(weight.shape[0]), int(weight.shape[1])


def _check_input_heads(heads: int, head_dim: int, in_features: int) -> None:
    if heads * head_dim != in_features:
        raise ValueError(
            f"heads*head_dim={heads}*{head_dim} must equal the weight's in_features={in_features}"
        )


def _check_positive(shape: tuple[int, ...]) -> None:
    if min(shape) <= 0:
        raise ValueError(f"all dimensions must be positive, got {shape}")


def _collective_validate(
    runtime: MegaUPRuntime, operation: str, metadata: object, local_error: str | None
) -> None:
    """Make a rank-local contract failure raise on every rank before any kernel
    or barrier (reference: ops.py:623-655). A single-process emulated group has
    nobody to tell."""

    if runtime.group is None:
        return
    record = (operation, metadata, local_error)
    records: list[object] = [None] * runtime.up
    if runtime.device.type == "cuda":
        with torch.cuda.device(runtime.device):
            dist.all_gather_object(records, record, group=runtime.group)
    else:
        dist.all_gather_object(records, record, group=runtime.group)
    errors = tuple(
        (rank, item[2]) for rank, item in enumerate(records)
        if isinstance(item, tuple) and item[2] is not None
    )
    if errors:
        raise ValueError(f"Mega-UP collective validation failed: {errors}")
    if any(not isinstance(item, tuple) or item[:2] != record[:2] for item in records):
        raise ValueError(
            "all UP ranks must enter the same operation with identical "
            "metadata and runtime configuration"
        )


def _runtime_tag(runtime: MegaUPRuntime) -> tuple[int, int, int]:
    return (runtime.hidden, runtime.max_rows, runtime.up)


def _guarded(function, *args, **kwargs):
    """Run a validation step; return ``(result, error string or None)``."""

    try:
        return function(*args, **kwargs), None
    except Exception as error:  # noqa: BLE001 - reported to the caller / the group
        return None, f"{type(error).__name__}: {error}"


# --------------------------------------------------------------------------- logical shapes

# A layout names its dimensions in user order; ``rows`` is their product without
# heads/head_dim, and the exchanged tensor has UP times the sequence-like one.
_DIMS = {
    "bshd": ("batch", "sequence", "heads", "head_dim"),
    "sbhd": ("sequence", "batch", "heads", "head_dim"),
    "thd": ("tokens", "heads", "head_dim"),
}
_LABEL = {"bshd": "BSHD", "sbhd": "(S,B,H,D)", "thd": "(T,H,D)"}
_INPUT_LABEL = {"bshd": "[B,S,H,D]", "sbhd": "[S,B,H,D]", "thd": "[T,H,D]"}
_PULL_LABEL = {"bshd": "[B,UP*S,H/UP,D]", "sbhd": "[UP*S,B,H/UP,D]", "thd": "[UP*T,H/UP,D]"}
_SUFFIX = {"bshd": "", "sbhd": " SBHD", "thd": " THD"}
# index of the sequence-like dimension that the exchange multiplies by UP
_SEQ_AXIS = {"bshd": 1, "sbhd": 0, "thd": 0}


def _rows(kind: str, shape: tuple[int, ...]) -> int:
    rows = 1
    for v in shape[:-2]:
        rows *= v
    return rows


def _exchanged_shape(kind: str, shape: tuple[int, ...], up: int, shard_heads: int) -> tuple[int, ...]:
    """User shape of the head-parallel tensor: sequence-like axis times UP, heads -> shard heads."""

    dims = list(shape)
    dims[_SEQ_AXIS[kind]] *= up
    dims[-2] = shard_heads
    return tuple(dims)


def _peer_input_shape(
    kind: str, x: Tensor, runtime: MegaUPRuntime, layout: THDLayout | None, *, n: int, k: int
) -> tuple[int, ...]:
    """Validate a peer-write activation; return its logical shape (reference: ops.py:440-485, :555-574)."""

    ndim = len(_DIMS[kind])
    if not isinstance(x, Tensor) or x.ndim != ndim:
        got = tuple(x.shape) if isinstance(x, Tensor) else type(x).__name__
        raise ValueError(f"peer-write{_SUFFIX[kind]} input must be {_INPUT_LABEL[kind]}, got {got}")
    shape = tuple(int(v) for v in x.shape)
    if min(shape) <= 0:
        raise ValueError(f"all {_LABEL[kind]} dimensions must be positive, got {tuple(x.shape)}")
    if kind == "thd" and layout is not None:
        _check_layout(layout, runtime)
        if shape[0] != layout.tokens:
            raise ValueError(
                f"input has {shape[0]} rows but the THD layout describes {layout.tokens} local tokens"
            )
    _check_input_heads(shape[-2], shape[-1], k)
    runtime.check_capacity(_rows(kind, shape), n)
    _check_activation(x, runtime, "input")
    return shape


def _pull_input_shape(
    kind: str, head_x: Tensor, runtime: MegaUPRuntime, layout: THDLayout | None, *, k: int
) -> tuple[int, ...]:
    """Validate a head-parallel pull input; return the LOGICAL (per-rank, all heads)
    shape (reference: ops.py:488-552, :577-605)."""

    ndim = len(_DIMS[kind])
    if not isinstance(head_x, Tensor) or head_x.ndim != ndim:
        got = tuple(head_x.shape) if isinstance(head_x, Tensor) else type(head_x).__name__
        raise ValueError(f"pull{_SUFFIX[kind]} input must be {_PULL_LABEL[kind]}, got {got}")
    shape = [int(v) for v in head_x.shape]
    if min(shape) <= 0:
        raise ValueError(f"all head-parallel dimensions must be positive, got {tuple(head_x.shape)}")
    axis = _SEQ_AXIS[kind]
    if shape[axis] % runtime.up:
        what = "pull THD input rows" if kind == "thd" else "sequence dimension"
        raise ValueError(f"{what} {shape[axis]} must be divisible by UP={runtime.up}")
    shape[axis] //= runtime.up
    if kind == "thd" and layout is not None:
        _check_layout(layout, runtime)
        if shape[0] != layout.tokens:
            raise ValueError(
                f"pull THD input must have UP*T={runtime.up * layout.tokens} rows, got {head_x.shape[0]}"
            )
    shape[-2] *= runtime.up
    logical = tuple(shape)
    _check_input_heads(logical[-2], logical[-1], k)
    runtime.check_capacity(_rows(kind, logical), k)
    _check_activation(head_x, runtime, "head-parallel input")
    return logical


# --------------------------------------------------------------------------- peer-write GEMM


def _bind_peer_write(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None,
    rows: int,
    operation: str,
    metadata: object,
    validate_group: bool,
) -> object:
    """Bind the kernel to this rank's slot in every peer arena, reporting a
    set-up failure on every rank (reference: ops.py:677-714)."""

    def bind():
        from .kernels.peer_write_gemm import make_peer_write_launch

        n, k = int(weight.shape[0]), int(weight.shape[1])
        return make_peer_write_launch(
            weight,
            None,
            runtime.remote_write_views(rows, n),
            a_shape=(rows, k),
            bias=bias,
            local_rank=runtime.local_rank,
            status_address=runtime.status_address,
            timeout_ns=runtime.kernel_timeout_ns,
        )

    launch, error = _guarded(bind)
    if validate_group:
        _collective_validate(runtime, f"{operation}_setup", metadata, error)
    if error is not None:
        raise RuntimeError(error)
    return launch


class _PeerWriteBase:
    """Shared behaviour of the three prepared peer-write executables."""

    _kind = "bshd"
    runtime: MegaUPRuntime
    weight: Tensor
    bias: Tensor | None
    launch: object
    head_dim: int

    @property
    def in_features(self) -> int:
        return int(self.weight.shape[1])

    @property
    def out_features(self) -> int:
        return int(self.weight.shape[0])

    def _logical_shape(self) -> tuple[int, ...]:
        return tuple(getattr(self, name) for name in _DIMS[self._kind])

    def _layout(self) -> THDLayout | None:
        return getattr(self, "layout", None)

    @property
    def _shard_heads(self) -> int:
        return self.out_features // (self.runtime.up * self.head_dim)

    @property
    def output_shape(self) -> tuple[int, ...]:
        return _exchanged_shape(self._kind, self._logical_shape(), self.runtime.up, self._shard_heads)

    def _validate_call(self, x: Tensor, out: Tensor | None, validate_group: bool) -> None:
        expected = self._logical_shape()

        def check():
            shape = _peer_input_shape(
                self._kind, x, self.runtime, self._layout(), n=self.out_features, k=self.in_features
            )
            if shape != expected:
                raise ValueError(
                    f"prepared{_SUFFIX[self._kind]} peer-write GEMM expects "
                    f"{_LABEL[self._kind]} {expected}, got {shape}"
                )
            _check_out(out, self.output_shape, self.runtime)
            return shape

        shape, error = _guarded(check)
        if validate_group:
            metadata = [shape]
            if self._kind == "thd":
                metadata.append(_layout_fingerprint(self._layout()))
            metadata += [
                _tensor_signature(self.weight),
                _optional_signature(self.bias),
                _optional_signature(out),
                *_runtime_tag(self.runtime),
            ]
            _collective_validate(self.runtime, f"peer_write_gemm_{self._kind}", tuple(metadata), error)
        if error is not None:
            raise ValueError(error)

    # phase 1: the GEMM whose epilogue stores into the peers' slots
    def _launch(self, x: Tensor) -> None:
        rows = _rows(self._kind, self._logical_shape())
        runtime = self.runtime
        if runtime.handoff in ("folded", "lazy"):
            # the kernel waits for the slots' owners before its first store (they may
            # still be copying the previous result out); folded: its last CTA also
            # raises the "written" flag, lazy: a barrier kernel follows instead
            sync = runtime._sync(wait=True, signal=runtime.handoff == "folded")
            self.launch(x.view(rows, self.in_features), sync=sync, stream_handle=runtime._stream())
            runtime._done_value = int(sync.done_after)
        else:
            self.launch(x.view(rows, self.in_features), stream_handle=runtime._stream())
        runtime._last_operation = "peer_write"

    # phase 2: barrier, slots -> ordinary memory, barrier
    def _materialize(self, out: Tensor) -> None:
        runtime, up = self.runtime, self.runtime.up
        shape = self._logical_shape()
        layout = self._layout()
        if layout is not None:
            runtime.copy_peer_written_indexed(
                rows=shape[0], index=layout.to_thd_index, out=out, _managed=True
            )
            return
        # SBHD rows are sequence-major and a THD slab is already in global
        # order, so both materialise like BSHD with B = 1.
        batch, sequence = (shape[0], shape[1]) if self._kind == "bshd" else (1, _rows(self._kind, shape))
        runtime.copy_peer_written(
            batch=batch,
            sequence=sequence,
            shard_heads=self._shard_heads,
            head_dim=self.head_dim,
            out=out.view(batch, up * sequence, self._shard_heads, self.head_dim),
            _managed=True,
        )

    def __call__(self, x: Tensor, *, out: Tensor | None = None, validate_group: bool = True) -> Tensor:
        self._validate_call(x, out, validate_group)
        if out is None:
            out = torch.empty(self.output_shape, dtype=torch.bfloat16, device=self.runtime.device)
        with torch.no_grad(), self.runtime.lease():
            self._launch(x)
            self._materialize(out)
        return out


@dataclass
class PreparedPeerWriteGemm(_PeerWriteBase):
    """Reusable peer-write executable for a fixed ``[B,S,H,D]`` input shape."""

    runtime: MegaUPRuntime
    weight: Tensor
    batch: int
    sequence: int
    heads: int
    head_dim: int
    launch: object
    bias: Tensor | None = None
    _kind = "bshd"


@dataclass
class PreparedPeerWriteGemmSBHD(_PeerWriteBase):
    """Reusable peer-write executable for a fixed sequence-first ``[S,B,H,D]`` input shape."""

    runtime: MegaUPRuntime
    weight: Tensor
    sequence: int
    batch: int
    heads: int
    head_dim: int
    launch: object
    bias: Tensor | None = None
    _kind = "sbhd"


@dataclass
class PreparedPeerWriteGemmTHD(_PeerWriteBase):
    """Reusable packed-THD peer-write executable for a fixed token count.

    ``layout`` is ``None`` for the contiguous-slab contract (output rows in
    source-rank order) or a ``THDLayout`` that regroups every sample to be
    contiguous.
    """

    runtime: MegaUPRuntime
    weight: Tensor
    tokens: int
    heads: int
    head_dim: int
    launch: object
    layout: THDLayout | None = None
    bias: Tensor | None = None
    _kind = "thd"


_PEER_CLASSES = {
    "bshd": PreparedPeerWriteGemm,
    "sbhd": PreparedPeerWriteGemmSBHD,
    "thd": PreparedPeerWriteGemmTHD,
}


def _resolve_thd_tokens(tokens: int | None, layout: THDLayout | None, runtime: MegaUPRuntime) -> int:
    if layout is not None:
        _check_layout(layout, runtime)
        if tokens is None:
            tokens = layout.tokens
        elif tokens != layout.tokens:
            raise ValueError(f"tokens={tokens} disagrees with layout.tokens={layout.tokens}")
    if tokens is None:
        raise ValueError("tokens is required when no THD layout is given")
    return tokens


def _prepare_peer_write(
    kind: str,
    weight: Tensor,
    runtime: MegaUPRuntime,
    dims: dict[str, int | None],
    *,
    layout: THDLayout | None,
    bias: Tensor | None,
    validate_group: bool,
):
    operation = f"prepare_peer_write_gemm_{kind}"
    heads, head_dim = dims["heads"], dims["head_dim"]

    def check():
        _check_runtime_device(runtime)
        _check_positive((heads, head_dim))
        n, k = _check_peer_weight(weight, runtime, head_dim)
        _check_bias(bias, runtime, n)
        if kind == "thd":
            dims["tokens"] = _resolve_thd_tokens(dims["tokens"], layout, runtime)
        shape = tuple(dims[name] for name in _DIMS[kind])
        _check_positive(shape)
        _check_input_heads(heads, head_dim, k)
        runtime.check_capacity(_rows(kind, shape), n)
        return shape

    shape, error = _guarded(check)
    if kind == "thd":
        metadata: tuple[object, ...] = (
            shape, _layout_fingerprint(layout), _tensor_signature(weight), _optional_signature(bias)
        )
    else:
        shape_for_metadata = tuple(dims[name] for name in _DIMS[kind])
        metadata = (shape_for_metadata, _tensor_signature(weight), _optional_signature(bias))
    if validate_group:
        _collective_validate(runtime, operation, (*metadata, *_runtime_tag(runtime)), error)
    if error is not None:
        raise ValueError(error)
    launch = _bind_peer_write(
        weight, runtime, bias=bias, rows=_rows(kind, shape), operation=operation,
        metadata=metadata, validate_group=validate_group,
    )
    fields = dict(zip(_DIMS[kind], shape))
    if kind == "thd":
        fields["layout"] = layout
    return _PEER_CLASSES[kind](runtime=runtime, weight=weight, launch=launch, bias=bias, **fields)


def prepare_peer_write_gemm_bshd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    batch: int,
    sequence: int,
    heads: int,
    head_dim: int,
    bias: Tensor | None = None,
    validate_group: bool = True,
) -> PreparedPeerWriteGemm:
    """Prepare a reusable ``linear(weight, bias) + all-to-all`` replacement:
    ``[B,S,H,D]`` to ``[B,UP*S,N/(UP*D),D]`` for ``weight [N, K]`` with
    ``K = heads * head_dim``. Weight, bias, arena slots and the tile order are
    validated and bound once; a call checks the input, launches the kernel and
    copies the received rows into the output."""

    dims = dict(batch=batch, sequence=sequence, heads=heads, head_dim=head_dim)
    return _prepare_peer_write(
        "bshd", weight, runtime, dims, layout=None, bias=bias, validate_group=validate_group
    )


def prepare_peer_write_gemm_sbhd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    sequence: int,
    batch: int,
    heads: int,
    head_dim: int,
    bias: Tensor | None = None,
    validate_group: bool = True,
) -> PreparedPeerWriteGemmSBHD:
    """Sequence-first variant: ``[S,B,H,D]`` to ``[UP*S,B,N/(UP*D),D]``."""

    dims = dict(sequence=sequence, batch=batch, heads=heads, head_dim=head_dim)
    return _prepare_peer_write(
        "sbhd", weight, runtime, dims, layout=None, bias=bias, validate_group=validate_group
    )


def prepare_peer_write_gemm_thd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    heads: int,
    head_dim: int,
    tokens: int | None = None,
    layout: THDLayout | None = None,
    bias: Tensor | None = None,
    validate_group: bool = True,
) -> PreparedPeerWriteGemmTHD:
    """Packed-THD variant: ``[T,H,D]`` to ``[UP*T,N/(UP*D),D]``; ``tokens`` may be
    omitted when ``layout`` is given."""

    dims = dict(tokens=tokens, heads=heads, head_dim=head_dim)
    return _prepare_peer_write(
        "thd", weight, runtime, dims, layout=layout, bias=bias, validate_group=validate_group
    )


def _peer_write_one_shot(
    kind: str,
    x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None,
    layout: THDLayout | None,
    out: Tensor | None,
    validate_group: bool,
) -> Tensor:
    def check():
        n, k = _weight_widths(weight)
        return _peer_input_shape(kind, x, runtime, layout, n=n, k=k)

    shape, error = _guarded(check)
    if validate_group:
        metadata = [shape]
        if kind == "thd":
            metadata.append(_layout_fingerprint(layout))
        metadata += [
            _tensor_signature(weight), _optional_signature(bias), _optional_signature(out),
            *_runtime_tag(runtime),
        ]
        _collective_validate(runtime, f"peer_write_gemm_{kind}_input", tuple(metadata), error)
    if error is not None:
        raise ValueError(error)
    dims = dict(zip(_DIMS[kind], shape))
    prepared = _prepare_peer_write(
        kind, weight, runtime, dims, layout=layout, bias=bias, validate_group=validate_group
    )
    return prepared(x, out=out, validate_group=validate_group)


def peer_write_gemm_bshd(
    x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    out: Tensor | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Fuse ``linear([B,S,H,D], weight, bias)`` with the Ulysses head all-to-all.

    ``weight [N, K]`` and ``bias [N]`` follow ``torch.nn.functional.linear``
    with ``K = H*D``. Returns ``[B,UP*S,N/(UP*D),D]`` in ordinary CUDA memory.
    Repeated calls with one shape should use ``prepare_peer_write_gemm_bshd``.
    """

    return _peer_write_one_shot(
        "bshd", x, weight, runtime, bias=bias, layout=None, out=out, validate_group=validate_group
    )


def peer_write_gemm_thd(
    x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    layout: THDLayout | None = None,
    out: Tensor | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Packed variant: ``x [T,H,D]`` -> ``[UP*T,N/(UP*D),D]``. Without ``layout`` the
    rows are in source-rank order (the global packed order when every rank
    holds a contiguous slab); with a ``layout`` every sample is regrouped to
    be contiguous with boundaries ``layout.cu_seqlens_out``."""

    return _peer_write_one_shot(
        "thd", x, weight, runtime, bias=bias, layout=layout, out=out, validate_group=validate_group
    )


def peer_write_gemm_sbhd(
    x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    out: Tensor | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Sequence-first variant: ``x [S,B,H,D]`` -> ``[UP*S,B,N/(UP*D),D]``, the UP
    sequence chunks in rank order."""

    return _peer_write_one_shot(
        "sbhd", x, weight, runtime, bias=bias, layout=None, out=out, validate_group=validate_group
    )


# --------------------------------------------------------------------------- head-shard pull GEMM


def _compile_pull(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None,
    rows: int,
    workspace_epochs: int,
    operation: str,
    metadata: object,
    validate_group: bool,
) -> tuple[Tensor, Tensor, object]:
    """Allocate the dense input / output buffers and bind the kernel, reporting a
    set-up failure on every rank (reference: ops.py:1383-1443)."""

    def bind():
        from .kernels.headshard_pull_gemm import compile_headshard_pull_gemm

        n, k = int(weight.shape[0]), int(weight.shape[1])
        dy = torch.empty((rows, k), dtype=torch.bfloat16, device=runtime.device)
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=runtime.device)
        compiled = compile_headshard_pull_gemm(
            tuple(peer.data_ptr() for peer in runtime.peer_buffers),
            weight,
            out,
            dy,
            logical_m=rows,
            rank=runtime.local_rank,
            up=runtime.up,
            bias=bias,
            workspace_epochs=workspace_epochs,
            peer_rows=rows,
            status_address=runtime.status_address,
            timeout_ns=runtime.kernel_timeout_ns,
        )
        return dy, out, compiled

    result, error = _guarded(bind)
    if validate_group:
        _collective_validate(runtime, f"{operation}_setup", metadata, error)
    if error is not None:
        raise RuntimeError(error)
    return result


class _PullBase:
    """Shared behaviour of the three prepared pull executables."""

    _kind = "bshd"
    runtime: MegaUPRuntime
    weight: Tensor
    bias: Tensor | None
    heads: int
    head_dim: int
    materialized_input: Tensor
    output_2d: Tensor
    compiled: object

    @property
    def in_features(self) -> int:
        return int(self.weight.shape[1])

    @property
    def out_features(self) -> int:
        return int(self.weight.shape[0])

    def _logical_shape(self) -> tuple[int, ...]:
        return tuple(getattr(self, name) for name in _DIMS[self._kind])

    def _layout(self) -> THDLayout | None:
        return getattr(self, "layout", None)

    @property
    def input_shape(self) -> tuple[int, ...]:
        up = self.runtime.up
        return _exchanged_shape(self._kind, self._logical_shape(), up, self.heads // up)

    @property
    def output(self) -> Tensor:
        lead = self._logical_shape()[:-2]
        return self.output_2d.view(*lead, self.out_features // self.head_dim, self.head_dim)

    def _validate_call(self, head_x: Tensor, validate_group: bool) -> None:
        expected = self._logical_shape()

        def check():
            shape = _pull_input_shape(
                self._kind, head_x, self.runtime, self._layout(), k=self.in_features
            )
            if shape != expected:
                raise ValueError(
                    f"prepared{_SUFFIX[self._kind]} pull-GEMM expects logical "
                    f"{_LABEL[self._kind]} {expected}, got {shape}"
                )
            return shape

        shape, error = _guarded(check)
        if validate_group:
            metadata = [shape]
            if self._kind == "thd":
                metadata.append(_layout_fingerprint(self._layout()))
            metadata += [
                _tensor_signature(self.weight),
                _optional_signature(self.bias),
                int(self.compiled.epoch),
                int(self.compiled.workspace_epochs),
                *_runtime_tag(self.runtime),
            ]
            _collective_validate(
                self.runtime, f"headshard_pull_gemm_{self._kind}", tuple(metadata), error
            )
        if error is not None:
            raise ValueError(error)

    # phase 1: head-parallel tensor -> destination-major slots, then barrier
    def _stage(self, head_x: Tensor) -> None:
        runtime, up = self.runtime, self.runtime.up
        shape = self._logical_shape()
        shard_heads = self.heads // up
        layout = self._layout()
        if layout is not None:
            runtime.stage_rows_indexed(
                rows=shape[0],
                source=head_x.view(up * shape[0], self.in_features // up),
                index=layout.to_source_major_index,
                _managed=True,
            )
            return
        # Rank chunks follow each other along the leading axis for SBHD and a
        # THD slab, so both stage like BSHD with B = 1.
        batch, sequence = (shape[0], shape[1]) if self._kind == "bshd" else (1, _rows(self._kind, shape))
        runtime.stage_head_parallel(
            head_x.view(batch, up * sequence, shard_heads, self.head_dim), _managed=True
        )

    # phase 2: pull + GEMM, then barrier so no peer's slot is reused too early
    def _launch(self) -> None:
        runtime = self.runtime
        handle = runtime._stream()
        if runtime.handoff in ("folded", "lazy"):
            # the last pull worker to finish hands every arena back, long before the
            # GEMM ends; folded: the pull workers also wait for the peers' staging
            # copies themselves, lazy: a barrier kernel has done that already
            sync = runtime._sync(wait=runtime.handoff == "folded", signal=True)
            self.compiled(sync=sync, stream_handle=handle)
            runtime._done_value = int(sync.done_after)
        else:
            self.compiled(stream_handle=handle)
            runtime.finish_pull()
        runtime._last_operation = "pull"

    def __call__(self, head_x: Tensor, *, validate_group: bool = True) -> Tensor:
        self._validate_call(head_x, validate_group)
        with torch.no_grad(), self.runtime.lease():
            self._refresh_workspace()
            self._stage(head_x)
            self._launch()
        return self.output

    def _refresh_workspace(self) -> None:
        """Zero the pull counters when they are used up, and after any device-side
        failure the runtime has reported (an aborted launch leaves the ticket
        cursor and the ready counts out of step with the launch ordinal)."""

        runtime = self.runtime
        seen = getattr(self, "_failures_seen", 0)
        if self.compiled.epoch >= self.compiled.workspace_epochs or seen != runtime.failure_count:
            self.compiled.reset_workspace(torch.cuda.current_stream(runtime.device))
            self._failures_seen = runtime.failure_count


@dataclass
class PreparedHeadShardPullGemm(_PullBase):
    """Reusable pull-GEMM executable with stable input/output buffers."""

    runtime: MegaUPRuntime
    weight: Tensor
    batch: int
    sequence: int
    heads: int
    head_dim: int
    materialized_input: Tensor
    output_2d: Tensor
    compiled: object
    bias: Tensor | None = None
    _kind = "bshd"


@dataclass
class PreparedHeadShardPullGemmSBHD(_PullBase):
    """Reusable sequence-first pull-GEMM executable with stable buffers."""

    runtime: MegaUPRuntime
    weight: Tensor
    sequence: int
    batch: int
    heads: int
    head_dim: int
    materialized_input: Tensor
    output_2d: Tensor
    compiled: object
    bias: Tensor | None = None
    _kind = "sbhd"


@dataclass
class PreparedHeadShardPullGemmTHD(_PullBase):
    """Reusable packed-THD pull-GEMM executable for a fixed token count; ``layout``
    is ``None`` for the contiguous-slab contract or a ``THDLayout`` for
    split-sample regrouped input."""

    runtime: MegaUPRuntime
    weight: Tensor
    tokens: int
    heads: int
    head_dim: int
    materialized_input: Tensor
    output_2d: Tensor
    compiled: object
    layout: THDLayout | None = None
    bias: Tensor | None = None
    _kind = "thd"


_PULL_CLASSES = {
    "bshd": PreparedHeadShardPullGemm,
    "sbhd": PreparedHeadShardPullGemmSBHD,
    "thd": PreparedHeadShardPullGemmTHD,
}


def _prepare_pull(
    kind: str,
    weight: Tensor,
    runtime: MegaUPRuntime,
    dims: dict[str, int | None],
    *,
    layout: THDLayout | None,
    bias: Tensor | None,
    workspace_epochs: int,
    validate_group: bool,
):
    operation = f"prepare_headshard_pull_gemm_{kind}"
    heads, head_dim = dims["heads"], dims["head_dim"]

    def check():
        _check_runtime_device(runtime)
        _check_positive((heads, head_dim))
        n, k = _check_pull_weight(weight, runtime, head_dim)
        _check_bias(bias, runtime, n)
        if kind == "thd":
            dims["tokens"] = _resolve_thd_tokens(dims["tokens"], layout, runtime)
        shape = tuple(dims[name] for name in _DIMS[kind])
        _check_positive(shape)
        if heads % runtime.up:
            raise ValueError(f"heads={heads} must be divisible by UP={runtime.up}")
        _check_input_heads(heads, head_dim, k)
        runtime.check_capacity(_rows(kind, shape), k)
        if workspace_epochs <= 0:
            raise ValueError(f"workspace_epochs must be positive, got {workspace_epochs}")
        return shape

    shape, error = _guarded(check)
    if kind == "thd":
        metadata: tuple[object, ...] = (
            shape, _layout_fingerprint(layout), _tensor_signature(weight),
            _optional_signature(bias), repr(workspace_epochs),
        )
    else:
        metadata = (
            tuple(dims[name] for name in _DIMS[kind]), _tensor_signature(weight),
            _optional_signature(bias), repr(workspace_epochs),
        )
    if validate_group:
        _collective_validate(runtime, operation, (*metadata, *_runtime_tag(runtime)), error)
    if error is not None:
        raise ValueError(error)
    dy, out, compiled = _compile_pull(
        weight, runtime, bias=bias, rows=_rows(kind, shape), workspace_epochs=workspace_epochs,
        operation=operation, metadata=metadata, validate_group=validate_group,
    )
    fields = dict(zip(_DIMS[kind], shape))
    if kind == "thd":
        fields["layout"] = layout
    return _PULL_CLASSES[kind](
        runtime=runtime, weight=weight, materialized_input=dy, output_2d=out, compiled=compiled,
        bias=bias, **fields,
    )


def prepare_headshard_pull_gemm_bshd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    batch: int,
    sequence: int,
    heads: int,
    head_dim: int,
    bias: Tensor | None = None,
    workspace_epochs: int = 4096,
    validate_group: bool = True,
) -> PreparedHeadShardPullGemm:
    """Prepare a reusable ``all-to-all + linear(weight, bias)`` replacement:
    ``[B,UP*S,H/UP,D]`` to ``[B,S,N/D,D]`` for ``weight [N, K]`` with
    ``K = heads * head_dim``. The returned output aliases a reusable buffer
    that the next call overwrites; ``clone()`` it to keep it."""

    dims = dict(batch=batch, sequence=sequence, heads=heads, head_dim=head_dim)
    return _prepare_pull(
        "bshd", weight, runtime, dims, layout=None, bias=bias,
        workspace_epochs=workspace_epochs, validate_group=validate_group,
    )


def prepare_headshard_pull_gemm_sbhd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    sequence: int,
    batch: int,
    heads: int,
    head_dim: int,
    bias: Tensor | None = None,
    workspace_epochs: int = 4096,
    validate_group: bool = True,
) -> PreparedHeadShardPullGemmSBHD:
    """Sequence-first variant: ``[UP*S,B,H/UP,D]`` to ``[S,B,N/D,D]``."""

    dims = dict(sequence=sequence, batch=batch, heads=heads, head_dim=head_dim)
    return _prepare_pull(
        "sbhd", weight, runtime, dims, layout=None, bias=bias,
        workspace_epochs=workspace_epochs, validate_group=validate_group,
    )


def prepare_headshard_pull_gemm_thd(
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    heads: int,
    head_dim: int,
    tokens: int | None = None,
    layout: THDLayout | None = None,
    bias: Tensor | None = None,
    workspace_epochs: int = 4096,
    validate_group: bool = True,
) -> PreparedHeadShardPullGemmTHD:
    """Packed-THD variant: ``[UP*T,H/UP,D]`` to ``[T,N/D,D]``; ``tokens`` may be
    omitted when ``layout`` is given."""

    dims = dict(tokens=tokens, heads=heads, head_dim=head_dim)
    return _prepare_pull(
        "thd", weight, runtime, dims, layout=layout, bias=bias,
        workspace_epochs=workspace_epochs, validate_group=validate_group,
    )


def _pull_one_shot(
    kind: str,
    head_x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None,
    layout: THDLayout | None,
    validate_group: bool,
) -> Tensor:
    def check():
        _, k = _weight_widths(weight)
        return _pull_input_shape(kind, head_x, runtime, layout, k=k)

    shape, error = _guarded(check)
    if validate_group:
        metadata = [shape]
        if kind == "thd":
            metadata.append(_layout_fingerprint(layout))
        metadata += [_tensor_signature(weight), _optional_signature(bias), *_runtime_tag(runtime)]
        _collective_validate(runtime, f"headshard_pull_gemm_{kind}_input", tuple(metadata), error)
    if error is not None:
        raise ValueError(error)
    dims = dict(zip(_DIMS[kind], shape))
    prepared = _prepare_pull(
        kind, weight, runtime, dims, layout=layout, bias=bias, workspace_epochs=1,
        validate_group=validate_group,
    )
    return prepared(head_x, validate_group=validate_group)


def headshard_pull_gemm_bshd(
    head_x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Fuse the Ulysses sequence all-to-all with ``linear(., weight, bias)``:
    ``head_x [B,UP*S,H/UP,D]`` -> ``[B,S,N/D,D]``. Repeated calls with one
    shape should use ``prepare_headshard_pull_gemm_bshd``."""

    return _pull_one_shot(
        "bshd", head_x, weight, runtime, bias=bias, layout=None, validate_group=validate_group
    )


def headshard_pull_gemm_sbhd(
    head_x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Sequence-first variant: ``head_x [UP*S,B,H/UP,D]`` -> ``[S,B,N/D,D]``."""

    return _pull_one_shot(
        "sbhd", head_x, weight, runtime, bias=bias, layout=None, validate_group=validate_group
    )


def headshard_pull_gemm_thd(
    head_x: Tensor,
    weight: Tensor,
    runtime: MegaUPRuntime,
    *,
    bias: Tensor | None = None,
    layout: THDLayout | None = None,
    validate_group: bool = True,
) -> Tensor:
    """Packed variant: ``head_x [UP*T,H/UP,D]`` -> ``[T,N/D,D]``; with a ``layout`` the
    input rows are in regrouped (sample-contiguous) order."""

    return _pull_one_shot(
        "thd", head_x, weight, runtime, bias=bias, layout=layout, validate_group=validate_group
    )


# --------------------------------------------------------------------------- single-process emulation


def emulated_peer_write(
    prepared: Sequence[_PeerWriteBase], xs: Sequence[Tensor], outs: Sequence[Tensor] | None = None
) -> list[Tensor]:
    """Run one peer-write operation on every rank of an emulated group: all
    launches first (they fill every rank's slots), then every rank's copy-out."""

    results: list[Tensor] = []
    for rank, (op, x) in enumerate(zip(prepared, xs)):
        op._validate_call(x, None if outs is None else outs[rank], False)
    with torch.no_grad():
        for op, x in zip(prepared, xs):
            op._launch(x)
        for rank, op in enumerate(prepared):
            out = (
                torch.empty(op.output_shape, dtype=torch.bfloat16, device=op.runtime.device)
                if outs is None
                else outs[rank]
            )
            op._materialize(out)
            results.append(out)
    return results


def emulated_pull(prepared: Sequence[_PullBase], head_xs: Sequence[Tensor]) -> list[Tensor]:
    """Run one pull operation on every rank of an emulated group: all staging
    copies first, then every rank's pull + GEMM."""

    for op, head_x in zip(prepared, head_xs):
        op._validate_call(head_x, False)
    with torch.no_grad():
        for op, head_x in zip(prepared, head_xs):
            op._refresh_workspace()
            op._stage(head_x)
        for op in prepared:
            op._launch()
    return [op.output for op in prepared]


__all__ = [
    "PreparedHeadShardPullGemm",
    "PreparedHeadShardPullGemmSBHD",
    "PreparedHeadShardPullGemmTHD",
    "PreparedPeerWriteGemm",
    "PreparedPeerWriteGemmSBHD",
    "PreparedPeerWriteGemmTHD",
    "THDLayout",
    "emulated_peer_write",
    "emulated_pull",
    "headshard_pull_gemm_bshd",
    "headshard_pull_gemm_sbhd",
    "headshard_pull_gemm_thd",
    "peer_write_gemm_bshd",
    "peer_write_gemm_sbhd",
    "peer_write_gemm_thd",
    "prepare_headshard_pull_gemm_bshd",
    "prepare_headshard_pull_gemm_sbhd",
    "prepare_headshard_pull_gemm_thd",
    "prepare_peer_write_gemm_bshd",
    "prepare_peer_write_gemm_sbhd",
    "prepare_peer_write_gemm_thd",
    "prepare_thd_layout",
]
