"""``brute.Tensor``: a ``torch.Tensor`` subclass with a 1-bit ``bit1`` dtype.

Same surface and laziness contract as the reference's ``brute/tensor.py``:

* a bit1 tensor IS a ``torch.bool`` tensor (so every torch op has a meaning) that
  carries an int64-packed side buffer, 64 bits per word along the last axis,
  pad bits 0 (``_packed_buf``);
* results of packed-domain ops are built from the packed buffer only (``_bool_dirty``); their
  bool tensor has the logical sizes and contiguous strides over an EMPTY storage until something
  reads it (``_ensure_bool_valid``; the reference, brute/tensor.py:288-352, allocates the full
  bool tensor up front). Reading fills that same storage object, so views and plain aliases
  taken before or after share it, as they do in the reference;
* in-place writes to the bool storage are noticed through torch's version
  counter (``_packed_ver``) and re-pack lazily (brute/tensor.py:362-388);
* a transpose of the last two dimensions remembers its source (``_t_source``) so that
  ``a @ b.t()`` feeds the (N, K) packed buffer to the xnor GEMM
  (brute/tensor.py:1210-1266), and so that its own packed words come from a bit-matrix
  transpose of the source's instead of a pack of the bool view.

The dispatch is organised differently from the reference: ``__torch_function__``
looks the function up in a handler table (``_FAST``) instead of walking one long
chain of tests; a handler returns ``NotImplemented`` to fall through to the
generic bool path. On CUDA the packed-domain handlers call this package's own
kernels (fused xnor / masked not / select / reductions over any axis / float->bit pack /
flip, roll and index_select along the packed axis) where the reference composes several
ATen launches or goes through bool.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

try:
    from . import _cbrute
except ImportError as exc:          # pragma: no cover
    raise ImportError("brute_b200/_cbrute.so is missing: the host helper module has not been built. "
                      "Run `python brute_b200/build.py` (needs g++ and the installed torch's headers).") from exc
from . import streams as _streams
from .dtype import _PACK_STORAGE_DTYPE, _PACK_WIDTH, _Bit1DType, bit1

_ops = torch.ops.brute

# op codes of torch.ops.brute.bitwise_packed (include/brute_b200.h)
_OP_AND, _OP_OR, _OP_XOR, _OP_XNOR = 0, 1, 2, 3
_SIGN_GT0, _SIGN_GE0 = 0, 1


# The base class's as_subclass, which Tensor overrides (a dirty lazy tensor is materialised before a
# caller gets a plain alias of it). Internal code reads shapes and versions through this one.
_AS = torch.Tensor.as_subclass


def _plain(t: torch.Tensor) -> torch.Tensor:
    return _AS(t, torch.Tensor) if isinstance(t, Tensor) else t


def _join_streams() -> None:
    """Inside a ``parallel_streams`` block the package's ops run on pool streams while plain torch ops
    run on the caller's stream. Every front-end entry point that is about to hand packed or bool data
    to a plain torch op calls this first: the caller's stream then waits for the pool work queued so
    far. Entry points that only launch this package's kernels skip it (those are ordered by the
    block's own events), which is what lets independent ops overlap."""
    if _streams._ACTIVE is not None:
        _streams._ACTIVE.join()


def _is_b1(x) -> bool:
    return isinstance(x, Tensor) and x.__dict__.get("_is_bit1", False)


def _words(n_bits: int) -> int:
    return (n_bits + _PACK_WIDTH - 1) // _PACK_WIDTH


def _to_bool(t: torch.Tensor) -> torch.Tensor:
    """Any tensor -> bool; floats threshold at x > 0 (brute/tensor.py:163-169)."""
    if t.dtype == torch.bool:
        return t
    if t.is_floating_point():
        return t > 0
    return t.bool()


def _pack_bool(bool_t: torch.Tensor) -> torch.Tensor:
    if bool_t.dtype != torch.bool:
        bool_t = bool_t.bool()
    if bool_t.dim() == 0:
        bool_t = bool_t.unsqueeze(0)
    return _ops.pack_bool(bool_t.contiguous())


def _unpack_pm1(packed: torch.Tensor, logical_shape: list) -> torch.Tensor:
    if len(logical_shape) == 0:
        return _ops.unpack_bits(packed, [1]).squeeze(0)
    return _ops.unpack_bits(packed, logical_shape)


def _packed_bin(code: int, pa: torch.Tensor, pb: torch.Tensor, last_bits: int) -> torch.Tensor:
    """Word-wise op on two packed buffers: one fused kernel on CUDA, ATen elsewhere."""
    if pa.is_cuda and pa.shape == pb.shape and pb.device == pa.device:
        return _ops.bitwise_packed(pa, pb, code, last_bits)
    if code == _OP_AND:
        return torch.bitwise_and(pa, pb)
    if code == _OP_OR:
        return torch.bitwise_or(pa, pb)
    if code == _OP_XOR:
        return torch.bitwise_xor(pa, pb)
    return _ops.bit1_not_packed(torch.bitwise_xor(pa, pb), last_bits)


def _arg_leaves(args, kwargs) -> list:
    """Leaves of a call's arguments. Nearly every call has tensors and scalars at the top level or
    one list deep; walking those by hand costs a microsecond where the general tree flattener
    costs twenty. Anything nested deeper (or a dict) goes to the general one."""
    out = []
    for a in args if not kwargs else (*args, *kwargs.values()):
        if isinstance(a, (list, tuple)):
            for b in a:
                if isinstance(b, (list, tuple, dict)):
                    out.extend(torch.utils._pytree.tree_leaves(b))
                else:
                    out.append(b)
        elif isinstance(a, dict):
            out.extend(torch.utils._pytree.tree_leaves(a))
        else:
            out.append(a)
    return out


def _rebuild_brute_tensor(plain_tensor: torch.Tensor, is_bit1: bool = False):
    """Pickle hook: rebuild from the (bool or plain) base tensor."""
    t = plain_tensor.as_subclass(Tensor)
    t._is_bit1 = is_bit1
    t._packed_buf = None
    return t


if hasattr(torch.serialization, "add_safe_globals"):
    torch.serialization.add_safe_globals([_rebuild_brute_tensor])


class Tensor(torch.Tensor):
    """torch.Tensor subclass; ``dtype=brute.bit1`` gives packed 1-bit storage."""

    # ------------------------------------------------------------------ build
    @staticmethod
    def __new__(cls, data, *, dtype=None, device=None):
        raw = _plain(data) if isinstance(data, torch.Tensor) else data
        if isinstance(dtype, _Bit1DType):
            if isinstance(raw, torch.Tensor):
                if device is not None:
                    raw = raw.to(device=device)
                if raw.is_cuda and raw.dtype in (torch.float32, torch.bfloat16, torch.float16) and raw.dim() >= 1:
                    # one fused pass float -> bits; the bool view stays lazy
                    return cls._make_bit1_from_packed(_ops.pack_sign(raw, _SIGN_GT0), list(raw.shape))
                bool_t = _to_bool(raw)
            else:
                bool_t = torch.as_tensor(raw, dtype=torch.bool)
                if device is not None:
                    bool_t = bool_t.to(device=device)
            return cls._make_bit1(bool_t)
        if isinstance(raw, torch.Tensor):
            t = raw.to(dtype=dtype, device=device) if (dtype is not None or device is not None) else raw
        elif isinstance(raw, (list, tuple)):
            t = torch.tensor(raw, dtype=dtype, device=device)
        else:
            t = torch.as_tensor(raw, dtype=dtype, device=device)
        return cls._make_plain(t)

    def __init__(self, data, *, dtype=None, device=None):
        pass

    @classmethod
    def _make_bit1(cls, bool_t: torch.Tensor, lazy_pack: bool = False) -> "Tensor":
        """Wrap a valid bool tensor; pack now, or on first use of ``_packed_buf``."""
        inst = _plain(bool_t).as_subclass(cls)
        d = inst.__dict__
        d["_is_bit1"] = True
        d["_bool_dirty"] = False
        if lazy_pack:
            d["_packed_buf_cache"] = None
            d.pop("_packed_ver", None)
        else:
            inst._packed_buf = _pack_bool(_plain(bool_t))
        return inst

    @classmethod
    def _make_plain(cls, t: torch.Tensor) -> "Tensor":
        inst = _plain(t).as_subclass(cls)
        d = inst.__dict__
        d["_is_bit1"] = False
        d["_packed_buf_cache"] = None
        return inst

    @classmethod
    def _make_bit1_from_packed(cls, packed: torch.Tensor, logical_shape: list,
                               bool_view: Optional[torch.Tensor] = None) -> "Tensor":
        """bit1 tensor whose source of truth is ``packed``. Without ``bool_view`` the
        bool storage is allocated uninitialised and marked dirty."""
        dirty = bool_view is None
        if dirty:
            # Logical sizes, contiguous strides, 0 bytes of storage: a lazy result that is never
            # read as bool costs no memory (the reference allocates a full bool tensor here,
            # brute/tensor.py:316, 1 GiB at 2^30 bits). _ensure_bool_valid fills the storage in place.
            bool_t = _cbrute.lazy_bool(tuple(logical_shape), packed.device)
        else:
            assert bool_view.dtype == torch.bool, "bool_view must be torch.bool"
            bool_t = _plain(bool_view)
        inst = bool_t.as_subclass(cls)
        d = inst.__dict__
        d["_is_bit1"] = True
        d["_packed_buf_cache"] = packed
        d["_packed_ver"] = bool_t._version
        d["_bool_dirty"] = dirty
        return inst

    def _ensure_bool_valid(self) -> None:
        """Fill the bool storage from the packed buffer if it is stale."""
        d = self.__dict__
        if not d.get("_bool_dirty", False):
            return
        packed = d.get("_packed_buf_cache")
        if packed is None:
            d["_bool_dirty"] = False
            return
        base = _plain(self)
        with torch._C.DisableTorchFunctionSubclass():
            shape = list(base.shape)
            src = packed if packed.is_contiguous() else packed.contiguous()
            if len(shape) == 0:
                unpacked = _ops.unpack_bool(src, [1]).reshape(())
            else:
                unpacked = _ops.unpack_bool(src, shape)
            _join_streams()          # bool storage is read by plain torch ops on the caller's stream
            if base.numel() and base.untyped_storage().nbytes() == 0:
                # still the empty placeholder: move the unpacked allocation into ITS storage object
                # (no copy), so that every alias of this tensor sees the data
                if len(shape) == 0:
                    base.untyped_storage().resize_(1)
                    base.copy_(unpacked)
                else:
                    _cbrute.adopt_storage(base, unpacked)
            else:
                base.copy_(unpacked)
            ver = base._version
        d["_bool_dirty"] = False
        d["_packed_ver"] = ver          # the copy_ bumped the version: re-pin

    def _mark_packed_only(self, packed: torch.Tensor) -> None:
        """The packed buffer was updated in place of the bool storage."""
        d = self.__dict__
        d["_packed_buf_cache"] = packed
        d["_bool_dirty"] = True
        d["_packed_ver"] = _plain(self)._version

    def as_subclass(self, cls):
        """A plain alias exposes the bool storage to the caller: fill it first if it is stale (the
        reference hands out uninitialised memory here; an unread lazy result here owns none)."""
        if self.__dict__.get("_bool_dirty", False):
            self._ensure_bool_valid()
        return _AS(self, cls)

    # ------------------------------------------------------------- properties
    @property
    def dtype(self):
        if self.__dict__.get("_is_bit1", False):
            return bit1
        return super().dtype

    @property
    def _packed_buf(self) -> Optional[torch.Tensor]:
        d = self.__dict__
        cache = d.get("_packed_buf_cache")
        if not d.get("_is_bit1", False) or d.get("_bool_dirty", False):
            return cache
        ver = _plain(self)._version
        if cache is None or d.get("_packed_ver") != ver:
            cache = self._packed_from_transposed_source()
            if cache is None:
                cache = _pack_bool(_plain(self))
            d["_packed_buf_cache"] = cache
            d["_packed_ver"] = ver
        return cache

    def _packed_from_transposed_source(self) -> Optional[torch.Tensor]:
        """A transpose of the last two dimensions whose source still has (or can make) its packed
        words: transpose the bit matrices in the packed domain instead of packing the bool view."""
        src = self.__dict__.get("_t_source")
        if src is None or not _is_b1(src) or src.dim() < 2 or src.dim() != self.dim():
            return None
        if tuple(src.shape[:-2]) != tuple(self.shape[:-2]) or src.shape[-1] != self.shape[-2] or src.shape[-2] != self.shape[-1]:
            return None
        sp = src._packed_buf_contig()
        if sp is None:
            return None
        return _ops.transpose_packed(sp, int(src.shape[-2]), int(src.shape[-1]))

    @_packed_buf.setter
    def _packed_buf(self, val: Optional[torch.Tensor]) -> None:
        d = self.__dict__
        d["_packed_buf_cache"] = val
        if val is not None:
            d["_packed_ver"] = _plain(self)._version
        else:
            d.pop("_packed_ver", None)

    def _packed_buf_contig(self) -> Optional[torch.Tensor]:
        pb = self._packed_buf
        if pb is None or pb.is_contiguous():
            return pb
        _join_streams()
        return pb.contiguous()

    def element_size(self) -> int:
        if _is_b1(self):
            raise TypeError(
                "element_size() is not defined for bit1 tensors: a logical element occupies less "
                "than one byte. Use tensor._packed_buf.nbytes for the packed footprint.")
        return super().element_size()

    @property
    def nbytes(self) -> int:
        if _is_b1(self):
            pb = self._packed_buf
            return pb.nbytes if pb is not None else 0
        return super().nbytes

    @property
    def itemsize(self) -> int:
        if _is_b1(self):
            raise TypeError("itemsize is not defined for bit1 tensors: an element is smaller than a byte.")
        return super().itemsize

    def type(self, dtype=None, non_blocking: bool = False, **kwargs):
        if dtype is None:
            return "brute.Bit1Tensor" if _is_b1(self) else super().type()
        if _is_b1(self):
            self._ensure_bool_valid()
        return Tensor._make_plain(_plain(self).type(dtype, non_blocking=non_blocking, **kwargs))

    # ---------------------------------------------------------------- new_*
    def _new(self, maker: str, dtype, device, bit1_args, plain_args, kwargs) -> "Tensor":
        eff = dtype if dtype is not None else self.dtype
        base = _plain(self)
        if isinstance(eff, _Bit1DType):
            return Tensor._make_bit1(getattr(base, maker)(*bit1_args, dtype=torch.bool, device=device))
        return Tensor._make_plain(getattr(base, maker)(*plain_args, dtype=dtype, device=device, **kwargs))

    def new_tensor(self, data, *, dtype=None, device=None, **kwargs) -> "Tensor":
        return self._new("new_tensor", dtype, device, (data,), (data,), kwargs)

    def new_empty(self, size, *, dtype=None, device=None, **kwargs) -> "Tensor":
        return self._new("new_empty", dtype, device, (size,), (size,), kwargs)

    def new_full(self, size, fill_value, *, dtype=None, device=None, **kwargs) -> "Tensor":
        return self._new("new_full", dtype, device, (size, bool(fill_value)), (size, fill_value), kwargs)

    def new_ones(self, size, *, dtype=None, device=None, **kwargs) -> "Tensor":
        return self._new("new_ones", dtype, device, (size,), (size,), kwargs)

    def new_zeros(self, size, *, dtype=None, device=None, **kwargs) -> "Tensor":
        return self._new("new_zeros", dtype, device, (size,), (size,), kwargs)

    # ------------------------------------------------------------ conversion
    def bool(self) -> "Tensor":
        if _is_b1(self):
            self._ensure_bool_valid()
            return Tensor._make_plain(_plain(self))
        return Tensor._make_plain(_plain(self).bool())

    def to(self, *args, **kwargs) -> "Tensor":
        kwargs = dict(kwargs)
        want = kwargs.get("dtype")
        if want is None:
            want = next((a for a in args if isinstance(a, _Bit1DType)), None)
        if isinstance(want, _Bit1DType):
            dev = kwargs.get("device")
            if _is_b1(self):
                self._ensure_bool_valid()
                base = _plain(self)
            else:
                base = _plain(self)
                if dev:
                    base = base.to(device=dev)
                if base.is_cuda and base.dtype in (torch.float32, torch.bfloat16, torch.float16) and base.dim() >= 1:
                    return Tensor._make_bit1_from_packed(_ops.pack_sign(base, _SIGN_GT0), list(base.shape))
                base = _to_bool(base)
            if dev:
                base = base.to(device=dev)
            return Tensor._make_bit1(base)
        if _is_b1(self):
            explicit = kwargs.get("dtype")
            if explicit is None:
                explicit = next((a for a in args if isinstance(a, torch.dtype)), None)
            if explicit is None:
                # a move between devices: carry the packed words (1/8 of the bytes) when they are
                # current, and leave the bool view of the result lazy
                d = self.__dict__
                pb = d.get("_packed_buf_cache")
                plain = _plain(self)
                if (pb is not None and plain.dim() >= 1
                        and (d.get("_bool_dirty", False) or d.get("_packed_ver") == plain._version)):
                    try:
                        probe = torch.empty(0, dtype=torch.bool, device=pb.device).to(*args, **kwargs)
                    except Exception:                    # not a device-only request: the bool path decides
                        probe = None
                    if probe is not None and probe.dtype == torch.bool and probe.device != pb.device:
                        _join_streams()
                        return Tensor._make_bit1_from_packed(pb.contiguous().to(probe.device), list(plain.shape))
                    # same device: the reference's path below (it also validates the bool view,
                    # which its tests rely on: tests/unit/test_lazy_bool.py:85-90)
            self._ensure_bool_valid()
            moved = _plain(self).to(*args, **kwargs)
            if explicit is None and moved.dtype == torch.bool:
                return Tensor._make_bit1(moved)
            return Tensor._make_plain(moved)
        return Tensor._make_plain(_plain(self).to(*args, **kwargs))

    def unpack_pm1(self) -> torch.Tensor:
        """Packed storage -> float32, +1.0 for True and -1.0 for False."""
        if not _is_b1(self):
            raise TypeError("unpack_pm1() is only valid for bit1 tensors")
        return _unpack_pm1(self._packed_buf_contig(), list(self.shape))

    # ----------------------------------------------- packed binary operators
    # The operators are the per-op hot path of the front end (a few microseconds of kernel): they
    # read shapes and versions from the plain alias (one as_subclass) instead of through
    # __torch_function__, which costs a round trip per attribute.
    def _packed_fast(self, plain: torch.Tensor) -> torch.Tensor:
        """``self._packed_buf`` given the plain alias of ``self``."""
        d = self.__dict__
        cache = d.get("_packed_buf_cache")
        if cache is not None and (d.get("_bool_dirty", False) or d.get("_packed_ver") == plain._version):
            return cache
        return self._packed_buf

    def _bin_operands(self, other):
        """(packed self, packed other, shape) when both are bit1 of one shape with >= 1 dim, else None."""
        if not (self.__dict__.get("_is_bit1", False) and isinstance(other, Tensor)
                and other.__dict__.get("_is_bit1", False)):
            return None
        ps, po = _AS(self, torch.Tensor), _AS(other, torch.Tensor)
        shape = ps.shape
        if len(shape) == 0 or shape != po.shape:
            return None
        return self._packed_fast(ps), other._packed_fast(po), shape

    def _same_shape_b1(self, other) -> bool:
        return self._bin_operands(other) is not None

    def _bin_new(self, other, code: int) -> "Tensor":
        pa, pb, shape = self._bin_operands(other)
        return Tensor._make_bit1_from_packed(_packed_bin(code, pa, pb, shape[-1]), shape)

    def _bin_inplace(self, other, code: int) -> "Tensor":
        pa, pb, shape = self._bin_operands(other)
        self._mark_packed_only(_packed_bin(code, pa, pb, shape[-1]))
        return self

    def __and__(self, other):
        ops = self._bin_operands(other)
        if ops is None:
            return super().__and__(other)
        return Tensor._make_bit1_from_packed(_packed_bin(_OP_AND, ops[0], ops[1], ops[2][-1]), ops[2])

    def __or__(self, other):
        ops = self._bin_operands(other)
        if ops is None:
            return super().__or__(other)
        return Tensor._make_bit1_from_packed(_packed_bin(_OP_OR, ops[0], ops[1], ops[2][-1]), ops[2])

    def __xor__(self, other):
        ops = self._bin_operands(other)
        if ops is None:
            return super().__xor__(other)
        return Tensor._make_bit1_from_packed(_packed_bin(_OP_XOR, ops[0], ops[1], ops[2][-1]), ops[2])

    def __eq__(self, other):
        ops = self._bin_operands(other) if isinstance(other, Tensor) else None
        if ops is None:
            return super().__eq__(other)
        return Tensor._make_bit1_from_packed(_packed_bin(_OP_XNOR, ops[0], ops[1], ops[2][-1]), ops[2])

    def __ne__(self, other):
        ops = self._bin_operands(other) if isinstance(other, Tensor) else None
        if ops is None:
            return super().__ne__(other)
        return Tensor._make_bit1_from_packed(_packed_bin(_OP_XOR, ops[0], ops[1], ops[2][-1]), ops[2])

    __hash__ = torch.Tensor.__hash__

    def __iand__(self, other):
        return self._bin_inplace(other, _OP_AND) if self._same_shape_b1(other) else super().__iand__(other)

    def __ior__(self, other):
        return self._bin_inplace(other, _OP_OR) if self._same_shape_b1(other) else super().__ior__(other)

    def __ixor__(self, other):
        return self._bin_inplace(other, _OP_XOR) if self._same_shape_b1(other) else super().__ixor__(other)

    def __invert__(self):
        if self.__dict__.get("_is_bit1", False):
            plain = _AS(self, torch.Tensor)
            shape = plain.shape
            if len(shape) >= 1:
                return Tensor._make_bit1_from_packed(
                    _ops.bit1_not_packed(self._packed_fast(plain), shape[-1]), shape)
        return super().__invert__()

    # -------------------------------------------------------------- indexing
    def _leading_axis_fast(self, idx) -> bool:
        """The index touches only axis 0, so packed rows can be sliced directly."""
        if not _is_b1(self) or self.dim() < 2:
            return False
        if isinstance(idx, bool):
            return False
        if isinstance(idx, int):
            return True
        if isinstance(idx, slice):
            return idx.step is None or idx.step == 1
        if isinstance(idx, torch.Tensor) and idx.dim() == 1 and idx.dtype in (torch.int64, torch.int32):
            return True
        return False

    def _last_axis_int_index(self, idx) -> Optional[int]:
        """``x[..., j]`` or ``x[:, ..., :, j]``: the integer j on the packed axis."""
        if not (_is_b1(self) and self.dim() >= 1) or not isinstance(idx, tuple):
            return None
        if len(idx) == 2 and idx[0] is Ellipsis and isinstance(idx[1], int) and not isinstance(idx[1], bool):
            return idx[1]
        if len(idx) == self.dim() and isinstance(idx[-1], int) and not isinstance(idx[-1], bool):
            if all(isinstance(s, slice) and s == slice(None) for s in idx[:-1]):
                return idx[-1]
        return None

    def _norm_col(self, j: int) -> int:
        K = int(self.shape[-1])
        jj = j + K if j < 0 else j
        if not 0 <= jj < K:
            raise IndexError(f"index {j} is out of bounds for axis {self.dim() - 1} with size {K}")
        return jj

    def _column_gather(self, j: int) -> "Tensor":
        """Column j along the packed axis, as a bit1 tensor of shape ``shape[:-1]``."""
        j = self._norm_col(j)
        word = self._packed_buf.select(-1, j // _PACK_WIDTH)
        return Tensor._make_bit1(((word >> (j % _PACK_WIDTH)) & 1).bool().contiguous())

    def _column_scatter(self, j: int, value: bool) -> None:
        """``x[..., j] = value`` touching one packed word column (and the bool
        column too when the bool storage is valid, for aliasing views)."""
        j = self._norm_col(j)
        d = self.__dict__
        pb = d.get("_packed_buf_cache")
        if pb is None:
            return super().__setitem__((slice(None),) * (self.dim() - 1) + (j,), bool(value))
        mask = torch.ones((), dtype=pb.dtype, device=pb.device) << (j % _PACK_WIDTH)
        col = pb.select(-1, j // _PACK_WIDTH)
        if value:
            col.bitwise_or_(mask)
        else:
            col.bitwise_and_(mask.bitwise_not())
        if not d.get("_bool_dirty", False):
            plain = _plain(self)
            view = plain.select(-1, j)
            view.copy_(torch.tensor(bool(value), dtype=torch.bool, device=plain.device).expand_as(view))
        d["_packed_ver"] = _plain(self)._version

    def _last_axis_tensor_index(self, idx) -> Optional[torch.Tensor]:
        """``x[..., t]`` / ``x[:, ..., :, t]`` with t a 1-D integer tensor on the packed axis: t, else None."""
        if not (_is_b1(self) and self.dim() >= 1) or not isinstance(idx, tuple) or not idx:
            return None
        t = idx[-1]
        if not (isinstance(t, torch.Tensor) and t.dim() == 1 and t.dtype in (torch.int64, torch.int32)):
            return None
        lead = idx[:-1]
        if lead == (Ellipsis,) or (len(lead) == self.dim() - 1
                                   and all(isinstance(x, slice) and x == slice(None) for x in lead)):
            return _plain(t)
        return None

    def _scatter_last_axis(self, index: torch.Tensor, src, value: bool, bool_write: Callable,
                           negative_ok: bool = True) -> None:
        """Write through a tensor index on the packed axis without leaving the packed domain
        (the reference re-packs the whole tensor after the bool write, brute/tensor.py:362-388).
        ``src``: None (every indexed position takes ``value``), or a tensor of shape
        ``shape[:-1] + [len(index)]``. ``bool_write(plain)`` applies the same write to the bool
        storage; it runs only when that storage is live, so that aliasing views see the write."""
        plain = _plain(self)
        n = int(plain.shape[-1])
        ix = index.to(device=plain.device, dtype=torch.int64)
        if ix.numel():
            lo, hi = int(ix.min()), int(ix.max())       # torch raises on an index out of range; so does this
            if lo < (-n if negative_ok else 0) or hi >= n:
                raise IndexError(f"index {hi if hi >= n else lo} is out of bounds for dimension {plain.dim() - 1} with size {n}")
            if lo < 0:
                ix = torch.where(ix < 0, ix + n, ix)
        d = self.__dict__
        pb = self._packed_buf_contig()
        if pb._base is not None:
            pb = pb.clone()                  # a view into another tensor's words: never written in place
        sp = None
        if src is not None:
            sp = src._packed_buf_contig() if _is_b1(src) else _pack_bool(_to_bool(_plain(src)))
        if not d.get("_bool_dirty", False):
            bool_write(plain)
        _ops.scatter_packed_(pb, ix, sp, bool(value), n)
        d["_packed_buf_cache"] = pb
        d["_packed_ver"] = plain._version

    def __getitem__(self, idx):
        _join_streams()
        if self._leading_axis_fast(idx):
            packed = self._packed_buf
            if isinstance(idx, torch.Tensor):
                sub = packed.index_select(0, _plain(idx).to(torch.int64))
                shape = [int(idx.numel())] + list(self.shape[1:])
            else:
                sub = packed[idx]
                shape = list(self.shape[1:]) if isinstance(idx, int) else [sub.shape[0]] + list(self.shape[1:])
            if sub.numel() != 0:
                return Tensor._make_bit1_from_packed(sub, shape)
        # x[..., a:b:s] is a view in torch (writes through it reach the base), so it takes the bool
        # path like in the reference; index_select along the packed axis, which copies, stays packed
        return super().__getitem__(idx)

    def _row_pattern(self, value: bool) -> torch.Tensor:
        """One packed row of all-`value` bits with zero pad bits."""
        K = int(self.shape[-1])
        ref = self._packed_buf
        row = torch.zeros(_words(K), dtype=ref.dtype, device=ref.device)
        if value:
            row.bitwise_not_()
            if K % _PACK_WIDTH:
                row[-1] = (1 << (K % _PACK_WIDTH)) - 1
        return row

    def __setitem__(self, idx, value):
        _join_streams()
        scalar = isinstance(value, (bool, int))
        if scalar and self._leading_axis_fast(idx) and not isinstance(idx, torch.Tensor):
            pb = self._packed_buf
            row = self._row_pattern(bool(value))
            if isinstance(idx, int):
                pb[idx].copy_(row.expand_as(pb[idx]))
            else:
                tgt = pb[idx]
                tgt.copy_(row.expand_as(tgt))
            self._mark_packed_only(pb)
            return
        j = self._last_axis_int_index(idx)
        if scalar and j is not None:
            self._column_scatter(j, bool(value))
            return
        t = self._last_axis_tensor_index(idx)
        if t is not None and self.numel():
            if scalar:
                def write(plain, t=t, v=bool(value)):
                    plain[..., t.to(plain.device)] = v
                self._scatter_last_axis(t, None, bool(value), write)
                return
            if (isinstance(value, torch.Tensor) and _plain(value).dtype == torch.bool
                    and tuple(value.shape) == tuple(self.shape[:-1]) + (int(t.numel()),)):
                if _is_b1(value):
                    value._ensure_bool_valid()

                def write(plain, t=t, v=_plain(value)):
                    plain[..., t.to(plain.device)] = v
                self._scatter_last_axis(t, value, False, write)
                return
        return super().__setitem__(idx, value)

    # -------------------------------------------------------- bit1 methods
    def popcount(self) -> "Tensor":
        """Number of True elements, 0-dim int64."""
        if _is_b1(self):
            return Tensor._make_plain(_ops.packed_popcount(self._packed_buf_contig()))
        base = _plain(self)
        if base.dtype == torch.bool:
            return Tensor._make_plain(base.long().sum())
        raise TypeError(f"popcount() is only defined for bit1 and bool tensors; got dtype={self.dtype}")

    def hamming(self, other: "Tensor") -> "Tensor":
        """Number of positions where self and other differ, 0-dim int64."""
        if not (_is_b1(self) and _is_b1(other)):
            raise TypeError("hamming() is only defined for bit1 tensors")
        sa, sb = _AS(self, torch.Tensor).shape, _AS(other, torch.Tensor).shape
        if sa != sb:
            raise ValueError(f"hamming() requires matching shapes; got {tuple(sa)} vs {tuple(sb)}")
        return Tensor._make_plain(_ops.bit1_hamming_total(self._packed_buf_contig(), other._packed_buf_contig()))

    def word_popcount(self) -> "Tensor":
        """int32 popcount of every packed word (same shape as the packed buffer)."""
        if not _is_b1(self):
            raise TypeError("word_popcount() is only defined for bit1 tensors")
        return Tensor._make_plain(_ops.popcount(self._packed_buf_contig()))

    def randomize_(self) -> "Tensor":
        """Uniformly random bits in place; pad bits of every row stay 0."""
        if not _is_b1(self):
            raise TypeError("randomize_() is only defined for bit1 tensors")
        _join_streams()
        pb = self._packed_buf.clone()
        _ops.randomize_bits(pb)
        K = int(self.shape[-1]) if self.dim() >= 1 else 0
        if K % _PACK_WIDTH and pb.numel() > 0:
            pb.select(-1, pb.size(-1) - 1).bitwise_and_(
                torch.tensor((1 << (K % _PACK_WIDTH)) - 1, dtype=pb.dtype, device=pb.device))
        self._mark_packed_only(pb)
        return self

    # ------------------------------------------------- shape ops (methods)
    def _reshape_packed(self, new_shape: list) -> Optional["Tensor"]:
        """Reshape through the packed buffer when the last axis allows it."""
        _join_streams()              # reshape of a strided packed view copies with a plain torch op
        total = self.numel()
        new_shape = [int(d) for d in new_shape]
        if new_shape.count(-1) == 1:
            known = 1
            for d in new_shape:
                if d != -1:
                    known *= d
            if known > 0 and total % known == 0:
                new_shape = [(total // known) if d == -1 else d for d in new_shape]
        if not new_shape or any(d < 0 for d in new_shape):
            return None
        prod = 1
        for d in new_shape:
            prod *= d
        if prod != total:
            return None
        old_last = int(self.shape[-1]) if self.dim() >= 1 else 0
        new_last = new_shape[-1]
        packed = self._packed_buf
        if old_last == new_last and self.dim() >= 1:
            return Tensor._make_bit1_from_packed(packed.reshape(new_shape[:-1] + [packed.shape[-1]]), new_shape)
        if old_last % _PACK_WIDTH == 0 and new_last % _PACK_WIDTH == 0:
            return Tensor._make_bit1_from_packed(packed.reshape(new_shape[:-1] + [new_last // _PACK_WIDTH]), new_shape)
        return None

    @staticmethod
    def _size_args(size) -> list:
        if len(size) == 1 and isinstance(size[0], (list, tuple, torch.Size)):
            return list(size[0])
        return list(size)

    def view(self, *size):
        if _is_b1(self) and self.dim() >= 1 and not (len(size) == 1 and isinstance(size[0], torch.dtype)):
            r = self._reshape_packed(self._size_args(size))
            if r is not None:
                return r
        return super().view(*size)

    def reshape(self, *size):
        if _is_b1(self) and self.dim() >= 1:
            r = self._reshape_packed(self._size_args(size))
            if r is not None:
                return r
        return super().reshape(*size)

    def _flat_packed(self) -> Optional["Tensor"]:
        last = int(self.shape[-1]) if self.dim() >= 1 else 0
        if last > 0 and last % _PACK_WIDTH == 0:
            return Tensor._make_bit1_from_packed(self._packed_buf.reshape(-1), [self.numel()])
        return None

    def flatten(self, start_dim: int = 0, end_dim: int = -1):
        if _is_b1(self) and self.dim() >= 1:
            nd = self.dim()
            sd = start_dim if start_dim >= 0 else nd + start_dim
            ed = end_dim if end_dim >= 0 else nd + end_dim
            if sd == 0 and ed == nd - 1:
                r = self._flat_packed()
                if r is not None:
                    return r
        return super().flatten(start_dim, end_dim)

    def ravel(self):
        if _is_b1(self) and self.dim() >= 1:
            r = self._flat_packed()
            if r is not None:
                return r
        return super().ravel()

    def contiguous(self, memory_format=torch.contiguous_format):
        if _is_b1(self) and _plain(self).is_contiguous(memory_format=memory_format):
            return self
        return super().contiguous(memory_format=memory_format)

    def _bool_view_if_valid(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> Optional[torch.Tensor]:
        if self.__dict__.get("_bool_dirty", False):
            return None
        return fn(_plain(self))

    def _permute_packed(self, dims) -> Optional["Tensor"]:
        """permute that keeps the packed axis last: permute the packed buffer too."""
        if not _is_b1(self) or self.dim() < 1:
            return None
        nd = self.dim()
        try:
            norm = tuple(int(d) if int(d) >= 0 else nd + int(d) for d in dims)
        except (TypeError, ValueError):
            return None
        if len(norm) != nd or sorted(norm) != list(range(nd)) or norm[-1] != nd - 1:
            return None
        return Tensor._make_bit1_from_packed(self._packed_buf.permute(*norm), [int(self.shape[d]) for d in norm])

    def _lazy_from_bool(self, fn: Callable[[torch.Tensor], torch.Tensor]) -> "Tensor":
        self._ensure_bool_valid()
        return Tensor._make_bit1(fn(_plain(self)), lazy_pack=True)

    def permute(self, *dims):
        if _is_b1(self) and self.dim() >= 1:
            if len(dims) == 1 and isinstance(dims[0], (list, tuple)):
                dims = tuple(dims[0])
            r = self._permute_packed(dims)
            return r if r is not None else self._lazy_from_bool(lambda b: b.permute(*dims))
        return super().permute(*dims)

    def movedim(self, source, destination):
        if _is_b1(self) and self.dim() >= 1 and isinstance(source, int) and isinstance(destination, int):
            nd = self.dim()
            s = source if source >= 0 else nd + source
            dst = destination if destination >= 0 else nd + destination
            order = [i for i in range(nd) if i != s]
            order.insert(dst, s)
            r = self._permute_packed(order)
            return r if r is not None else self._lazy_from_bool(lambda b: b.movedim(source, destination))
        return super().movedim(source, destination)

    moveaxis = movedim

    def swapaxes(self, axis0: int, axis1: int):
        if _is_b1(self) and self.dim() >= 2 and isinstance(axis0, int) and isinstance(axis1, int):
            return self.transpose(axis0, axis1)
        return super().swapaxes(axis0, axis1)

    swapdims = swapaxes

    def reshape_as(self, other):
        if _is_b1(self) and self.dim() >= 1 and isinstance(other, torch.Tensor):
            r = self._reshape_packed(list(other.shape))
            if r is not None:
                return r
        return super().reshape_as(other)

    def view_as(self, other):
        if _is_b1(self) and self.dim() >= 1 and isinstance(other, torch.Tensor):
            r = self._reshape_packed(list(other.shape))
            if r is not None:
                return r
        return super().view_as(other)

    def _transposed_with_source(self, d0: int, d1: int) -> "Tensor":
        """Transpose that moves the packed axis: a bool view, packed lazily; a 2-D
        one remembers its source for the matmul fast path."""
        self._ensure_bool_valid()
        plain = _AS(self, torch.Tensor)
        inst = Tensor._make_bit1(plain.transpose(d0, d1), lazy_pack=True)
        nd = plain.dim()
        if {d0, d1} == {nd - 2, nd - 1}:
            inst.__dict__["_t_source"] = self
        return inst

    def transpose(self, dim0: int, dim1: int):
        if _is_b1(self) and self.dim() >= 2:
            nd = self.dim()
            d0 = dim0 if dim0 >= 0 else nd + dim0
            d1 = dim1 if dim1 >= 0 else nd + dim1
            if d0 == d1:
                return self
            if d0 != nd - 1 and d1 != nd - 1:
                shape = list(self.shape)
                shape[d0], shape[d1] = shape[d1], shape[d0]
                return Tensor._make_bit1_from_packed(
                    self._packed_buf.transpose(d0, d1), shape,
                    bool_view=self._bool_view_if_valid(lambda b: b.transpose(d0, d1)))
            return self._transposed_with_source(d0, d1)
        return super().transpose(dim0, dim1)

    def t(self) -> "Tensor":
        plain = _AS(self, torch.Tensor)
        if not self.__dict__.get("_is_bit1", False):
            return Tensor._make_plain(plain.t())
        if plain.dim() < 2:
            return self
        return self._transposed_with_source(0, 1)

    def unsqueeze(self, dim: int):
        if _is_b1(self) and self.dim() >= 1 and isinstance(dim, int):
            nd = self.dim()
            d = dim if dim >= 0 else nd + 1 + dim
            if 0 <= d <= nd - 1:
                shape = list(self.shape)
                shape.insert(d, 1)
                return Tensor._make_bit1_from_packed(
                    self._packed_buf.unsqueeze(d), shape,
                    bool_view=self._bool_view_if_valid(lambda b: b.unsqueeze(d)))
            if d == nd:
                return self._lazy_from_bool(lambda b: b.unsqueeze(nd))
        return super().unsqueeze(dim)

    def squeeze(self, *args, **kwargs):
        if _is_b1(self) and self.dim() >= 1:
            dim = args[0] if args else kwargs.get("dim")
            if dim is None:
                axes = [i for i, s in enumerate(self.shape[:-1]) if s == 1]
            elif isinstance(dim, int):
                nd = self.dim()
                d = dim if dim >= 0 else nd + dim
                if not (0 <= d < nd - 1 and self.shape[d] == 1):
                    return super().squeeze(*args, **kwargs)
                axes = [d]
            else:
                return super().squeeze(*args, **kwargs)
            if not axes:
                return self        # the packed axis itself is never squeezed away
            shape = [s for i, s in enumerate(self.shape) if i not in axes]
            if not shape:
                return super().squeeze(*args, **kwargs)
            packed = self._packed_buf
            for i in sorted(axes, reverse=True):
                packed = packed.squeeze(i)

            def squeeze_bool(b):
                for i in sorted(axes, reverse=True):
                    b = b.squeeze(i)
                return b
            return Tensor._make_bit1_from_packed(packed, shape, bool_view=self._bool_view_if_valid(squeeze_bool))
        return super().squeeze(*args, **kwargs)

    def clone(self, *, memory_format=torch.preserve_format):
        _join_streams()
        if _is_b1(self) and self.dim() >= 1:
            return Tensor._make_bit1_from_packed(self._packed_buf.clone(), list(self.shape))
        return super().clone(memory_format=memory_format)

    def detach(self):
        if _is_b1(self) and self.dim() >= 1:
            pb = self.__dict__.get("_packed_buf_cache")
            if pb is not None and (self.__dict__.get("_bool_dirty", False)
                                   or self.__dict__.get("_packed_ver") == _plain(self)._version):
                return Tensor._make_bit1_from_packed(pb.detach(), list(self.shape))
        return super().detach()

    # ----------------------------------------------------------------- matmul
    @staticmethod
    def _matmul_bit1(a: "Tensor", b: "Tensor"):
        """A (M,K) @ B with B stored (N,K), or B = src.t() with src stored (N,K)."""
        sa, sb = _AS(a, torch.Tensor).shape, _AS(b, torch.Tensor).shape
        if not (len(sa) == 2 and len(sb) == 2):
            return NotImplemented
        K = sa[-1]
        if sb[-1] == K:
            pa, pb = a._packed_buf_contig(), b._packed_buf_contig()
            if pa.shape[-1] == pb.shape[-1]:
                return _ops.xnor_popcount_matmul(pa, pb, K)
        src = b.__dict__.get("_t_source")
        if _is_b1(src) and _AS(src, torch.Tensor).shape[-1] == K:
            pa, ps = a._packed_buf_contig(), src._packed_buf_contig()
            if pa.shape[-1] == ps.shape[-1]:
                return _ops.xnor_popcount_matmul(pa, ps, K)
        return NotImplemented

    def __matmul__(self, other):
        if _is_b1(self) and _is_b1(other):
            r = Tensor._matmul_bit1(self, other)
            if r is not NotImplemented:
                return r
        return super().__matmul__(other)

    # ---------------------------------------------------------------- dispatch
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in _METADATA_FUNCS:
            if args and isinstance(args[0], Tensor):
                with torch._C.DisableTorchFunctionSubclass():
                    return func(*args, **kwargs)
        if func in _BASE_FUNCS:
            # hand back the plain base so that view-chain walkers terminate
            with torch._C.DisableTorchFunctionSubclass():
                return args[0]._base

        flat = _arg_leaves(args, kwargs)
        bit1_ins = [x for x in flat if _is_b1(x)]
        if not bit1_ins:
            with torch._C.DisableTorchFunctionSubclass():
                out = func(*args, **kwargs)
            return _wrap_plain(out)

        other_bools = [x for x in flat
                       if isinstance(x, torch.Tensor) and not _is_b1(x) and _plain(x).dtype == torch.bool]

        # packed-domain fast paths: only when no plain bool tensor is mixed in
        handler = _FAST.get(func)
        if _streams._ACTIVE is not None and handler not in _KERNEL_ONLY_HANDLERS:
            _streams._ACTIVE.join()
        if handler is not None and (not other_bools or func in _MATMUL_FUNCS):
            out = handler(func, args, kwargs, bit1_ins)
            if out is not NotImplemented:
                return out

        # generic path: expose the bool storage to torch
        for t in bit1_ins:
            t._ensure_bool_valid()
        u_args = torch.utils._pytree.tree_map(_plain_leaf, args)
        u_kwargs = torch.utils._pytree.tree_map(_plain_leaf, kwargs)
        if func in _ARG_FUNCS:
            # argmax / argmin are not implemented for bool
            u_args = (u_args[0].to(torch.uint8),) + tuple(u_args[1:])
            return Tensor._make_plain(func(*u_args, **u_kwargs))
        out = func(*u_args, **u_kwargs)

        promote = bool(bit1_ins) if func in _MASK_USING_FUNCS else not other_bools
        lazy = func in _LAZY_VIEW_FUNCS
        scalar_reduce = func in _ALL_FUNCS or func in _ANY_FUNCS

        def rewrap(r):
            if not isinstance(r, torch.Tensor):
                return r
            if promote and r.dtype == torch.bool:
                if r.dim() == 0 and scalar_reduce:
                    return Tensor._make_plain(r)
                return Tensor._make_bit1(r, lazy_pack=lazy)
            return r if isinstance(r, cls) else Tensor._make_plain(r)

        if isinstance(out, torch.Tensor):
            return rewrap(out)
        if isinstance(out, (tuple, list)):
            return type(out)(rewrap(r) for r in out)
        return out

    # ------------------------------------------------------------ persistence
    def __deepcopy__(self, memo):
        if _is_b1(self):
            self._ensure_bool_valid()
        new_t = super().__deepcopy__(memo)
        new_t.__dict__["_is_bit1"] = self.__dict__.get("_is_bit1", False)
        new_t.__dict__["_packed_buf_cache"] = None
        new_t.__dict__.pop("_packed_ver", None)
        new_t.__dict__["_bool_dirty"] = False
        new_t.__dict__.pop("_t_source", None)
        return new_t

    def __reduce_ex__(self, _proto):
        if _is_b1(self):
            self._ensure_bool_valid()
        return (_rebuild_brute_tensor, (_plain(self), self.__dict__.get("_is_bit1", False)))

    def __array__(self, dtype=None, copy=None):
        if _is_b1(self):
            self._ensure_bool_valid()
        arr = _plain(self).numpy(force=True)
        if dtype is not None:
            return arr.astype(dtype, copy=copy if copy is not None else False)
        return arr.copy() if copy else arr

    def __repr__(self):
        if _is_b1(self):
            self._ensure_bool_valid()
        with torch._C.DisableTorchFunctionSubclass():
            base = _plain(self).__repr__()
        if _is_b1(self):
            if "dtype=torch.bool" in base:
                base = base.replace("dtype=torch.bool", "dtype=brute.bit1")
            else:
                base = base[:-1] + ", dtype=brute.bit1)"
        return base.replace("tensor(", "brute.Tensor(")


# =============================================================================
# dispatch tables
# =============================================================================
def _getter(name: str):
    prop = getattr(torch.Tensor, name, None)
    return getattr(prop, "__get__", prop) if prop is not None else None


_METADATA_FUNCS = frozenset(f for f in [
    _getter("shape"), _getter("ndim"), _getter("dtype"), _getter("device"), _getter("layout"),
    _getter("requires_grad"), _getter("_version"), _getter("is_cuda"), _getter("is_mps"),
    _getter("is_cpu"), _getter("is_leaf"),
    torch.Tensor.dim, torch.Tensor.numel, torch.Tensor.size, torch.Tensor.stride,
    torch.Tensor.storage_offset, torch.Tensor.is_contiguous, torch.Tensor.__len__, torch.numel,
] if f is not None)
_BASE_FUNCS = frozenset(f for f in [_getter("_base")] if f is not None)

_MATMUL_FUNCS = frozenset([torch.matmul, torch.mm, torch.bmm, torch.Tensor.matmul, torch.Tensor.mm,
                           torch.Tensor.bmm, torch.Tensor.__matmul__])
_ALL_FUNCS = frozenset([torch.all, torch.Tensor.all])
_ANY_FUNCS = frozenset([torch.any, torch.Tensor.any])
_ARG_FUNCS = frozenset([torch.argmax, torch.Tensor.argmax, torch.argmin, torch.Tensor.argmin])
_MASK_USING_FUNCS = frozenset([torch.where, torch.masked_select, torch.Tensor.masked_select,
                               torch.masked_fill, torch.Tensor.masked_fill, torch.Tensor.__getitem__])
# pure layout ops: when they reach the generic path the result is a strided bool
# view, which is packed only if somebody asks for the packed buffer
_LAZY_VIEW_FUNCS = frozenset([
    torch.permute, torch.Tensor.permute, torch.movedim, torch.moveaxis, torch.Tensor.movedim,
    torch.Tensor.moveaxis, torch.swapaxes, torch.swapdims, torch.Tensor.swapaxes, torch.Tensor.swapdims,
    torch.t, torch.unsqueeze, torch.Tensor.unsqueeze, torch.squeeze, torch.Tensor.squeeze,
    torch.ravel, torch.Tensor.ravel, torch.Tensor.reshape_as, torch.Tensor.view_as,
    torch.Tensor.view, torch.Tensor.reshape, torch.reshape, torch.Tensor.flatten, torch.flatten,
    torch.Tensor.transpose, torch.transpose,
])


def _plain_leaf(x):
    return _AS(x, torch.Tensor) if isinstance(x, Tensor) else x


def _wrap_plain(out):
    if isinstance(out, torch.Tensor):
        return Tensor._make_plain(out)
    if isinstance(out, (tuple, list)):
        return type(out)(Tensor._make_plain(r) if isinstance(r, torch.Tensor) else r for r in out)
    return out


_FAST: Dict[Callable, Callable] = {}


def _fast(*funcs):
    def deco(fn):
        for f in funcs:
            _FAST[f] = fn
        return fn
    return deco


def _arg(args, kwargs, pos: int, name: str, default=None):
    if len(args) > pos:
        return args[pos]
    return kwargs.get(name, default)


@_fast(*_MATMUL_FUNCS)
def _h_matmul(func, args, kwargs, b1: List[Tensor]):
    if len(b1) >= 2:
        return Tensor._matmul_bit1(b1[0], b1[1])
    return NotImplemented


@_fast(torch.sum, torch.Tensor.sum, torch.count_nonzero, torch.Tensor.count_nonzero)
def _h_sum(func, args, kwargs, b1):
    if len(b1) == 1 and len(args) <= 1 and "dim" not in kwargs and "dtype" not in kwargs:
        return Tensor._make_plain(_ops.packed_popcount(b1[0]._packed_buf_contig()))
    return NotImplemented


def _reduce_leading(packed: torch.Tensor, dim: int, use_or: bool) -> torch.Tensor:
    """OR / AND over a non-packed, non-empty axis of the packed words in one fused pass
    (the reference halves the axis log2(n) times with ATen launches, brute/tensor.py:1440-1457)."""
    return _ops.reduce_rows_packed(packed, dim, use_or)


@_fast(*_ALL_FUNCS, *_ANY_FUNCS)
def _h_all_any(func, args, kwargs, b1):
    if len(b1) != 1:
        return NotImplemented
    a = b1[0]
    is_any = func in _ANY_FUNCS
    if len(args) <= 1 and "dim" not in kwargs:
        # full reduction: a plain 0-dim bool on the tensor's own device, no host sync
        total = _ops.packed_popcount(a._packed_buf_contig())
        return Tensor._make_plain((total != 0) if is_any else (total == a.numel()))
    dim = _arg(args, kwargs, 1, "dim")
    keepdim = _arg(args, kwargs, 2, "keepdim", False)
    if a.dim() < 1 or not isinstance(dim, int) or isinstance(dim, bool) or not isinstance(keepdim, bool):
        return NotImplemented
    nd = a.dim()
    d = dim if dim >= 0 else nd + dim
    if d == nd - 1:
        packed = a._packed_buf_contig()
        if packed.is_cuda:
            res = _ops.row_any(packed) if is_any else _ops.row_all(packed, int(a.shape[-1]))
        elif is_any:
            res = (packed != 0).any(dim=-1)
        else:
            res = _ops.popcount(packed).to(torch.int64).sum(dim=-1) == int(a.shape[-1])
        if keepdim:
            res = res.unsqueeze(-1)
        return Tensor._make_plain(res) if res.dim() == 0 else Tensor._make_bit1(res)
    if 0 <= d < nd - 1:
        if a.shape[d] == 0:
            return NotImplemented       # identity of an empty axis: leave it to the bool path
        out = _reduce_leading(a._packed_buf_contig(), d, is_any)
        shape = list(a.shape)
        if keepdim:
            shape[d] = 1
            out = out.unsqueeze(d)
        else:
            shape.pop(d)
        return Tensor._make_bit1_from_packed(out.contiguous(), shape)
    return NotImplemented


@_fast(torch.equal)
def _h_equal(func, args, kwargs, b1):
    if len(b1) >= 2 and b1[0].shape == b1[1].shape:
        pa, pb = b1[0]._packed_buf, b1[1]._packed_buf
        if pa.shape == pb.shape:
            return torch.equal(pa, pb)       # pad bits are 0 in both
    return NotImplemented


_BIN_CODES = {
    torch.bitwise_and: _OP_AND, torch.logical_and: _OP_AND, torch.Tensor.bitwise_and: _OP_AND,
    torch.Tensor.logical_and: _OP_AND, torch.Tensor.__and__: _OP_AND,
    torch.bitwise_or: _OP_OR, torch.logical_or: _OP_OR, torch.Tensor.bitwise_or: _OP_OR,
    torch.Tensor.logical_or: _OP_OR, torch.Tensor.__or__: _OP_OR,
    torch.bitwise_xor: _OP_XOR, torch.logical_xor: _OP_XOR, torch.Tensor.bitwise_xor: _OP_XOR,
    torch.Tensor.logical_xor: _OP_XOR, torch.Tensor.__xor__: _OP_XOR,
    torch.ne: _OP_XOR, torch.Tensor.ne: _OP_XOR, torch.Tensor.__ne__: _OP_XOR,
    torch.eq: _OP_XNOR, torch.Tensor.eq: _OP_XNOR, torch.Tensor.__eq__: _OP_XNOR,
}


@_fast(*_BIN_CODES.keys())
def _h_binary(func, args, kwargs, b1):
    if len(b1) >= 2 and len(args) >= 2 and not kwargs and isinstance(args[0], Tensor):
        ops = args[0]._bin_operands(args[1])
        if ops is not None:
            return Tensor._make_bit1_from_packed(_packed_bin(_BIN_CODES[func], ops[0], ops[1], ops[2][-1]), ops[2])
    return NotImplemented


@_fast(torch.bitwise_not, torch.logical_not, torch.Tensor.bitwise_not, torch.Tensor.logical_not,
       torch.Tensor.__invert__)
def _h_not(func, args, kwargs, b1):
    if len(b1) == 1 and not kwargs and _AS(b1[0], torch.Tensor).dim() >= 1:
        return b1[0].__invert__()
    return NotImplemented


@_fast(torch.Tensor.contiguous)
def _h_contiguous(func, args, kwargs, b1):
    if len(b1) == 1 and _plain(b1[0]).is_contiguous():
        return b1[0]
    return NotImplemented


@_fast(torch.Tensor.view, torch.Tensor.reshape, torch.reshape)
def _h_reshape(func, args, kwargs, b1):
    if len(b1) != 1 or b1[0].dim() < 1:
        return NotImplemented
    if "shape" in kwargs:
        raw = kwargs["shape"]
        shape = list(raw) if isinstance(raw, (list, tuple, torch.Size)) else [raw]
    elif len(args) == 2 and isinstance(args[1], (list, tuple, torch.Size)):
        shape = list(args[1])
    else:
        shape = list(args[1:])
    if not shape or not all(isinstance(s, int) and not isinstance(s, bool) for s in shape):
        return NotImplemented
    r = b1[0]._reshape_packed(shape)
    return r if r is not None else NotImplemented


@_fast(torch.Tensor.flatten, torch.flatten)
def _h_flatten(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        a = b1[0]
        start = _arg(args, kwargs, 1, "start_dim", 0)
        end = _arg(args, kwargs, 2, "end_dim", -1)
        if start == 0 and end in (-1, a.dim() - 1):
            r = a._flat_packed()
            if r is not None:
                return r
    return NotImplemented


@_fast(torch.ravel, torch.Tensor.ravel)
def _h_ravel(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        r = b1[0]._flat_packed()
        if r is not None:
            return r
    return NotImplemented


@_fast(torch.Tensor.transpose, torch.transpose, torch.swapaxes, torch.swapdims,
       torch.Tensor.swapaxes, torch.Tensor.swapdims)
def _h_transpose(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 2:
        d0 = _arg(args, kwargs, 1, "dim0", kwargs.get("axis0"))
        d1 = _arg(args, kwargs, 2, "dim1", kwargs.get("axis1"))
        if isinstance(d0, int) and isinstance(d1, int):
            return b1[0].transpose(d0, d1)
    return NotImplemented


@_fast(torch.t)
def _h_t(func, args, kwargs, b1):
    return b1[0].t() if len(b1) == 1 and b1[0].dim() <= 2 else NotImplemented


@_fast(torch.clone, torch.Tensor.clone)
def _h_clone(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        return Tensor._make_bit1_from_packed(b1[0]._packed_buf.clone(), list(b1[0].shape))
    return NotImplemented


@_fast(torch.detach, torch.Tensor.detach)
def _h_detach(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        a = b1[0]
        pb = a.__dict__.get("_packed_buf_cache")
        if pb is not None and (a.__dict__.get("_bool_dirty", False)
                               or a.__dict__.get("_packed_ver") == _plain(a)._version):
            return Tensor._make_bit1_from_packed(pb.detach(), list(a.shape))
    return NotImplemented


@_fast(torch.permute, torch.Tensor.permute)
def _h_permute(func, args, kwargs, b1):
    if len(b1) != 1 or b1[0].dim() < 1:
        return NotImplemented
    if "dims" in kwargs:
        dims = kwargs["dims"]
    elif len(args) == 2 and isinstance(args[1], (list, tuple)):
        dims = args[1]
    elif len(args) > 2:
        dims = tuple(args[1:])
    else:
        return NotImplemented
    r = b1[0]._permute_packed(dims)
    return r if r is not None else NotImplemented


@_fast(torch.movedim, torch.moveaxis, torch.Tensor.movedim, torch.Tensor.moveaxis)
def _h_movedim(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        a = b1[0]
        src = _arg(args, kwargs, 1, "source")
        dst = _arg(args, kwargs, 2, "destination")
        if isinstance(src, int) and isinstance(dst, int):
            nd = a.dim()
            s = src if src >= 0 else nd + src
            d = dst if dst >= 0 else nd + dst
            order = [i for i in range(nd) if i != s]
            order.insert(d, s)
            r = a._permute_packed(order)
            if r is not None:
                return r
    return NotImplemented


@_fast(torch.unsqueeze, torch.Tensor.unsqueeze)
def _h_unsqueeze(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        d = _arg(args, kwargs, 1, "dim")
        if isinstance(d, int):
            return b1[0].unsqueeze(d)
    return NotImplemented


@_fast(torch.squeeze, torch.Tensor.squeeze)
def _h_squeeze(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        if len(args) == 1 and "dim" not in kwargs:
            return b1[0].squeeze()
        d = _arg(args, kwargs, 1, "dim")
        if isinstance(d, int):
            return b1[0].squeeze(d)
    return NotImplemented


@_fast(torch.Tensor.reshape_as, torch.Tensor.view_as)
def _h_reshape_as(func, args, kwargs, b1):
    target = _arg(args, kwargs, 1, "other")
    if _is_b1(args[0]) and args[0].dim() >= 1 and isinstance(target, torch.Tensor):
        r = args[0]._reshape_packed(list(target.shape))
        if r is not None:
            return r
    return NotImplemented


@_fast(torch.index_select, torch.Tensor.index_select)
def _h_index_select(func, args, kwargs, b1):
    if len(b1) == 1 and _is_b1(args[0]):
        a = args[0]
        dim = _arg(args, kwargs, 1, "dim")
        idx = _arg(args, kwargs, 2, "index")
        if a.dim() >= 2 and dim == 0 and isinstance(idx, torch.Tensor) and idx.dim() == 1:
            return Tensor._make_bit1_from_packed(a._packed_buf.index_select(0, _plain(idx)),
                                                 [int(idx.numel())] + list(a.shape[1:]))
        if (a.dim() >= 1 and isinstance(dim, int) and dim in (-1, a.dim() - 1) and isinstance(idx, torch.Tensor)
                and idx.dim() == 1 and idx.dtype in (torch.int64, torch.int32) and not _is_b1(idx)):
            # the packed axis: gather bits in the packed domain. torch raises on an index out of
            # range; so does this (one small reduction on the index vector, no pass over the data)
            n = int(a.shape[-1])
            ix = _plain(idx).to(torch.int64)
            if ix.numel() and (int(ix.min()) < 0 or int(ix.max()) >= n):
                raise IndexError("index out of range in self")
            out = _ops.gather_packed(a._packed_buf_contig(), ix.to(a.device), n)
            return Tensor._make_bit1_from_packed(out, list(a.shape[:-1]) + [int(ix.numel())])
    return NotImplemented


@_fast(torch.Tensor.fill_, torch.Tensor.zero_)
def _h_fill(func, args, kwargs, b1):
    if len(b1) != 1 or not _is_b1(args[0]) or args[0].dim() < 1:
        return NotImplemented
    a = args[0]
    value = False if func is torch.Tensor.zero_ else _arg(args, kwargs, 1, "value")
    if not isinstance(value, (bool, int)):
        return NotImplemented
    plain = _plain(a)
    d = a.__dict__
    dirty = d.get("_bool_dirty", False)
    if not dirty:
        # the bool storage is live (maybe a strided view of another tensor): write it, so that
        # aliases see the fill; the version bump tells their owners to re-pack
        plain.fill_(bool(value))
    K = int(a.shape[-1])
    # always a fresh buffer: the old one may be shared with packed-domain views of this tensor
    pb = torch.full(list(a.shape[:-1]) + [_words(K)], -1 if value else 0, dtype=_PACK_STORAGE_DTYPE,
                    device=plain.device)
    if value and K > 0 and K % _PACK_WIDTH:
        pb[..., -1] = (1 << (K % _PACK_WIDTH)) - 1
    # a packed-only tensor stays packed-only: nothing is allocated for a fill
    d["_packed_buf_cache"] = pb
    d["_packed_ver"] = plain._version
    return a


@_fast(torch.Tensor.index_fill_)
def _h_index_fill_(func, args, kwargs, b1):
    a = args[0] if args else None
    dim, index, value = _arg(args, kwargs, 1, "dim"), _arg(args, kwargs, 2, "index"), _arg(args, kwargs, 3, "value")
    if (_is_b1(a) and a.dim() >= 1 and a.numel() and isinstance(dim, int) and dim in (-1, a.dim() - 1)
            and isinstance(index, torch.Tensor) and not _is_b1(index) and index.dim() == 1
            and index.dtype in (torch.int64, torch.int32) and isinstance(value, (bool, int))):
        a._scatter_last_axis(_plain(index), None, bool(value),
                             lambda plain: plain.index_fill_(-1, _plain(index).to(plain.device), bool(value)))
        return a
    return NotImplemented


@_fast(torch.Tensor.index_copy_)
def _h_index_copy_(func, args, kwargs, b1):
    a = args[0] if args else None
    dim, index, src = _arg(args, kwargs, 1, "dim"), _arg(args, kwargs, 2, "index"), _arg(args, kwargs, 3, "source")
    if (_is_b1(a) and a.dim() >= 1 and a.numel() and isinstance(dim, int) and dim in (-1, a.dim() - 1)
            and isinstance(index, torch.Tensor) and not _is_b1(index) and index.dim() == 1
            and index.dtype in (torch.int64, torch.int32) and isinstance(src, torch.Tensor)
            and _plain(src).dtype == torch.bool
            and tuple(src.shape) == tuple(a.shape[:-1]) + (int(index.numel()),)):
        if _is_b1(src):
            src._ensure_bool_valid()
        a._scatter_last_axis(_plain(index), src, False,
                             lambda plain: plain.index_copy_(-1, _plain(index).to(plain.device), _plain(src)),
                             negative_ok=False)          # torch's index_copy_ takes no negative index
        return a
    return NotImplemented


@_fast(torch.where, torch.Tensor.where)
def _h_where(func, args, kwargs, b1):
    if len(b1) == 3 and len(args) >= 3 and all(_is_b1(x) for x in args[:3]):
        cond, a, b = args[0], args[1], args[2]
        if cond.dim() >= 1 and tuple(cond.shape) == tuple(a.shape) == tuple(b.shape):
            pc, pa, pb = cond._packed_buf_contig(), a._packed_buf_contig(), b._packed_buf_contig()
            if pa.is_cuda:
                out = _ops.select_packed(pc, pa, pb)
            else:
                out = torch.bitwise_or(torch.bitwise_and(pa, pc), torch.bitwise_and(pb, torch.bitwise_not(pc)))
            return Tensor._make_bit1_from_packed(out, list(a.shape))
    return NotImplemented


@_fast(torch.flipud)
def _h_flipud(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 2:
        return Tensor._make_bit1_from_packed(b1[0]._packed_buf.flip(0), list(b1[0].shape))
    return NotImplemented


@_fast(torch.fliplr)
def _h_fliplr(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 3:
        return Tensor._make_bit1_from_packed(b1[0]._packed_buf.flip(1), list(b1[0].shape))
    return NotImplemented


@_fast(torch.flip, torch.Tensor.flip)
def _h_flip(func, args, kwargs, b1):
    if len(b1) == 1 and b1[0].dim() >= 1:
        a = b1[0]
        dims = _arg(args, kwargs, 1, "dims")
        if isinstance(dims, int) and all(isinstance(x, int) for x in args[1:]):
            dims = tuple(args[1:])          # Tensor.flip(0, 2): the dims as separate arguments
        if isinstance(dims, (list, tuple)) and dims and all(isinstance(x, int) for x in dims):
            nd = a.dim()
            norm = [x if x >= 0 else nd + x for x in dims]
            if (nd - 1) not in norm:
                return Tensor._make_bit1_from_packed(a._packed_buf.flip(norm), list(a.shape))
            if len(set(norm)) == len(norm) and all(0 <= x < nd for x in norm):
                # the packed axis: reverse the bits of every row in the packed domain; the other
                # axes are word-wise flips of the packed buffer
                others = [x for x in norm if x != nd - 1]
                packed = a._packed_buf_contig()
                if others:
                    packed = packed.flip(others)
                return Tensor._make_bit1_from_packed(_ops.flip_packed(packed, int(a.shape[-1])), list(a.shape))
    return NotImplemented


@_fast(torch.roll, torch.Tensor.roll)
def _h_roll(func, args, kwargs, b1):
    if len(b1) != 1 or not _is_b1(args[0]) or args[0].dim() < 1:
        return NotImplemented
    a = args[0]
    shifts = _arg(args, kwargs, 1, "shifts")
    dims = _arg(args, kwargs, 2, "dims", None)
    if isinstance(shifts, int) and isinstance(dims, int):
        shifts, dims = (shifts,), (dims,)
    if dims is None or not isinstance(shifts, (list, tuple)) or not isinstance(dims, (list, tuple)):
        return NotImplemented          # dims=None rolls the flattened tensor: leave it to the bool path
    if len(shifts) != len(dims) or not all(isinstance(x, int) for x in list(shifts) + list(dims)):
        return NotImplemented
    nd = a.dim()
    norm = [x if x >= 0 else nd + x for x in dims]
    if not all(0 <= x < nd for x in norm):
        return NotImplemented
    packed = a._packed_buf_contig()
    lead = [(s_, d_) for s_, d_ in zip(shifts, norm) if d_ != nd - 1]
    if lead:
        packed = torch.roll(packed, [s_ for s_, _ in lead], [d_ for _, d_ in lead])
    last = sum(s_ for s_, d_ in zip(shifts, norm) if d_ == nd - 1)
    if any(d_ == nd - 1 for d_ in norm) and int(a.shape[-1]) > 0:
        packed = _ops.roll_packed(packed.contiguous(), int(a.shape[-1]), int(last))
    return Tensor._make_bit1_from_packed(packed, list(a.shape))


@_fast(torch.Tensor.repeat)
def _h_repeat(func, args, kwargs, b1):
    if len(b1) == 1 and _is_b1(args[0]):
        a = args[0]
        reps = args[1:]
        if len(reps) == 1 and isinstance(reps[0], (list, tuple, torch.Size)):
            reps = tuple(reps[0])
        if a.dim() >= 1 and len(reps) == a.dim() and all(isinstance(r, int) and r >= 0 for r in reps):
            last = int(a.shape[-1])
            shape = [int(a.shape[i]) * int(reps[i]) for i in range(a.dim())]
            if reps[-1] == 1 or (last > 0 and last % _PACK_WIDTH == 0):
                return Tensor._make_bit1_from_packed(a._packed_buf.repeat(*reps), shape)
            if last > 0 and reps[-1] > 1 and all(x > 0 for x in shape):
                # ragged last dim: repeat the other axes word-wise, then lay the row's bits end to end
                packed = a._packed_buf_contig().repeat(*reps[:-1], 1)
                pos = torch.arange(last * reps[-1], dtype=torch.int64, device=a.device) % last
                return Tensor._make_bit1_from_packed(_ops.gather_packed(packed.contiguous(), pos, last), shape)
    return NotImplemented


@_fast(torch.repeat_interleave, torch.Tensor.repeat_interleave)
def _h_repeat_interleave(func, args, kwargs, b1):
    if len(b1) == 1 and len(args) >= 2 and _is_b1(args[0]):
        a = args[0]
        repeats = args[1]
        dim = kwargs.get("dim", args[2] if len(args) > 2 else None)
        if a.dim() >= 1 and dim is not None and isinstance(repeats, int):
            d = int(dim) if int(dim) >= 0 else a.dim() + int(dim)
            if 0 <= d < a.dim() - 1:
                shape = list(a.shape)
                shape[d] = int(shape[d]) * repeats
                return Tensor._make_bit1_from_packed(a._packed_buf.repeat_interleave(repeats, dim=d), shape)
    return NotImplemented


# handlers that do nothing but launch this package's kernels on packed buffers (see _join_streams)
_KERNEL_ONLY_HANDLERS = frozenset([_h_matmul, _h_sum, _h_binary, _h_not])

__all__ = ["Tensor", "bit1"]
