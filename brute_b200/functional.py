"""bit1-aware factory functions (surface of the reference's ``brute/functional.py``).

For ``dtype=brute.bit1`` constant factories write the packed words directly and
leave the bool view lazy; random factories threshold as the reference does
(``rand`` at >= 0.5, ``randn`` at >= 0, brute/functional.py:123-133) — on CUDA
``randn`` goes through the fused float->bit pack. Every other dtype is a thin
wrapper that keeps results inside ``brute.Tensor``.
"""
from __future__ import annotations

import torch

from .dtype import _PACK_STORAGE_DTYPE, _PACK_WIDTH, _Bit1DType
from .tensor import Tensor, _plain

_SIGN_GE0 = 1


def _norm_size(size) -> tuple:
    if len(size) == 1 and isinstance(size[0], (list, tuple, torch.Size)):
        return tuple(size[0])
    return tuple(size)


def _packed_shape(size: tuple) -> tuple:
    """Packed-buffer shape of a logical shape; a 0-dim tensor packs to one word."""
    if len(size) == 0:
        return (1,)
    last = int(size[-1])
    return tuple(size[:-1]) + ((last + _PACK_WIDTH - 1) // _PACK_WIDTH if last > 0 else 0,)


def _make_bit1_eager(packed: torch.Tensor, size: tuple, device) -> Tensor:
    """Wrap a freshly built packed buffer; the bool view is filled on first read."""
    return Tensor._make_bit1_from_packed(packed, list(size))


def _tail_mask(size: tuple):
    if size and size[-1] > 0 and size[-1] % _PACK_WIDTH:
        return (1 << (size[-1] % _PACK_WIDTH)) - 1
    return None


def zeros(*size, dtype=None, device=None, **kwargs) -> Tensor:
    size = _norm_size(size)
    if isinstance(dtype, _Bit1DType):
        return _make_bit1_eager(torch.zeros(_packed_shape(size), dtype=_PACK_STORAGE_DTYPE, device=device), size, device)
    return Tensor._make_plain(torch.zeros(size, dtype=dtype, device=device, **kwargs))


def ones(*size, dtype=None, device=None, **kwargs) -> Tensor:
    size = _norm_size(size)
    if isinstance(dtype, _Bit1DType):
        packed = torch.full(_packed_shape(size), -1, dtype=_PACK_STORAGE_DTYPE, device=device)
        mask = _tail_mask(size)
        if len(size) == 0:
            packed.fill_(1)
        elif mask is not None and packed.numel() > 0:
            packed[..., -1] = mask
        return _make_bit1_eager(packed, size, device)
    return Tensor._make_plain(torch.ones(size, dtype=dtype, device=device, **kwargs))


def empty(*size, dtype=None, device=None, **kwargs) -> Tensor:
    size = _norm_size(size)
    if isinstance(dtype, _Bit1DType):
        packed = torch.empty(_packed_shape(size), dtype=_PACK_STORAGE_DTYPE, device=device)
        if len(size) == 0:
            packed.bitwise_and_(1)
        elif _tail_mask(size) is not None and packed.numel() > 0:
            packed[..., -1] = 0          # pad bits must be 0 even in "empty" storage
        return _make_bit1_eager(packed, size, device)
    return Tensor._make_plain(torch.empty(size, dtype=dtype, device=device, **kwargs))


def full(size, fill_value, *, dtype=None, device=None, **kwargs) -> Tensor:
    if isinstance(size, int):
        size = (size,)
    if isinstance(dtype, _Bit1DType):
        maker = ones if bool(fill_value) else zeros
        return maker(*size, dtype=dtype, device=device)
    return Tensor._make_plain(torch.full(size, fill_value, dtype=dtype, device=device, **kwargs))


def tensor(data, *, dtype=None, device=None, **kwargs) -> Tensor:
    if isinstance(dtype, _Bit1DType):
        return Tensor._make_bit1(torch.tensor(data, dtype=torch.bool, device=device))
    return Tensor._make_plain(torch.tensor(data, dtype=dtype, device=device, **kwargs))


def as_tensor(data, *, dtype=None, device=None) -> Tensor:
    if isinstance(dtype, _Bit1DType):
        if isinstance(data, torch.Tensor):
            bool_t = _plain(data)
            bool_t = bool_t if bool_t.dtype == torch.bool else bool_t.bool()
        else:
            bool_t = torch.as_tensor(data, dtype=torch.bool, device=device)
        if device is not None:
            bool_t = bool_t.to(device=device)
        return Tensor._make_bit1(bool_t)
    return Tensor._make_plain(torch.as_tensor(data, dtype=dtype, device=device))


def from_numpy(ndarray) -> Tensor:
    return Tensor._make_plain(torch.from_numpy(ndarray))


def _gen_kw(generator):
    return {"generator": generator} if generator is not None else {}


def rand(*size, dtype=None, device=None, generator=None, **kwargs) -> Tensor:
    size = _norm_size(size)
    if isinstance(dtype, _Bit1DType):
        return Tensor._make_bit1(torch.rand(size, device=device, **_gen_kw(generator)) >= 0.5)
    return Tensor._make_plain(torch.rand(size, dtype=dtype, device=device, **_gen_kw(generator), **kwargs))


def randn(*size, dtype=None, device=None, generator=None, **kwargs) -> Tensor:
    size = _norm_size(size)
    if isinstance(dtype, _Bit1DType):
        x = torch.randn(size, device=device, **_gen_kw(generator))
        if x.is_cuda and x.dim() >= 1:
            return Tensor._make_bit1_from_packed(torch.ops.brute.pack_sign(x, _SIGN_GE0), list(size))
        return Tensor._make_bit1(x >= 0)
    return Tensor._make_plain(torch.randn(size, dtype=dtype, device=device, **_gen_kw(generator), **kwargs))


def randint(low_or_high, high=None, size=None, *, dtype=None, device=None, generator=None, **kwargs) -> Tensor:
    if isinstance(dtype, _Bit1DType):
        s = size if size is not None else (low_or_high,)
        return Tensor._make_bit1(torch.randint(0, 2, s, device=device, **_gen_kw(generator)).bool())
    if high is None:
        return Tensor._make_plain(torch.randint(low_or_high, size, dtype=dtype, device=device,
                                                **_gen_kw(generator), **kwargs))
    return Tensor._make_plain(torch.randint(low_or_high, high, size, dtype=dtype, device=device,
                                            **_gen_kw(generator), **kwargs))


def _like(input, dtype, device, bit1_maker, plain_maker):
    eff = dtype if dtype is not None else input.dtype
    base = _plain(input) if isinstance(input, torch.Tensor) else input
    if isinstance(eff, _Bit1DType):
        return Tensor._make_bit1(bit1_maker(base))
    return Tensor._make_plain(plain_maker(base))


def rand_like(input: Tensor, *, dtype=None, device=None) -> Tensor:
    dev = device or input.device
    return _like(input, dtype, device,
                 lambda b: (torch.rand_like(b.float()) >= 0.5).to(device=dev),
                 lambda b: torch.rand_like(b, dtype=dtype, device=device))


def randn_like(input: Tensor, *, dtype=None, device=None) -> Tensor:
    dev = device or input.device
    return _like(input, dtype, device,
                 lambda b: (torch.randn_like(b.float()) >= 0).to(device=dev),
                 lambda b: torch.randn_like(b, dtype=dtype, device=device))


def zeros_like(input: Tensor, *, dtype=None, device=None) -> Tensor:
    return _like(input, dtype, device,
                 lambda b: torch.zeros_like(b, dtype=torch.bool, device=device),
                 lambda b: torch.zeros_like(b, dtype=dtype, device=device))


def ones_like(input: Tensor, *, dtype=None, device=None) -> Tensor:
    return _like(input, dtype, device,
                 lambda b: torch.ones_like(b, dtype=torch.bool, device=device),
                 lambda b: torch.ones_like(b, dtype=dtype, device=device))


def full_like(input: Tensor, fill_value, *, dtype=None, device=None, **kwargs) -> Tensor:
    return _like(input, dtype, device,
                 lambda b: torch.full_like(b, bool(fill_value), dtype=torch.bool, device=device),
                 lambda b: torch.full_like(b, fill_value, dtype=dtype, device=device, **kwargs))


def empty_like(input: Tensor, *, dtype=None, device=None, **kwargs) -> Tensor:
    return _like(input, dtype, device,
                 lambda b: torch.empty_like(b, dtype=torch.bool, device=device),
                 lambda b: torch.empty_like(b, dtype=dtype, device=device, **kwargs))


def arange(start, end=None, step=1, *, dtype=None, device=None, **kwargs) -> Tensor:
    if end is None:
        return Tensor._make_plain(torch.arange(start, dtype=dtype, device=device, **kwargs))
    return Tensor._make_plain(torch.arange(start, end, step, dtype=dtype, device=device, **kwargs))


def linspace(start, end, steps, *, dtype=None, device=None, **kwargs) -> Tensor:
    return Tensor._make_plain(torch.linspace(start, end, steps, dtype=dtype, device=device, **kwargs))


def eye(n, m=None, *, dtype=None, device=None, **kwargs) -> Tensor:
    if m is None:
        return Tensor._make_plain(torch.eye(n, dtype=dtype, device=device, **kwargs))
    return Tensor._make_plain(torch.eye(n, m, dtype=dtype, device=device, **kwargs))
