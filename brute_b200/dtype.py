"""The ``bit1`` pseudo-dtype and the packing constants.

Mirrors the surface of the reference's ``brute/dtype.py`` (sentinel class with
``repr`` "brute.bit1" and ``str`` "bit1", equality by type, constant hash; torch
dtype aliases; pack width 64 bits in int64 storage, brute/dtype.py:5-34).
"""
import torch

_bool = bool


class _Bit1DType:
    """Sentinel for 1-bit elements packed 64 per int64 word."""

    __slots__ = ()

    def __repr__(self) -> str:
        return "brute.bit1"

    def __str__(self) -> str:
        return "bit1"

    def __eq__(self, other) -> _bool:
        return isinstance(other, _Bit1DType)

    def __ne__(self, other) -> _bool:
        return not isinstance(other, _Bit1DType)

    def __hash__(self) -> int:
        return hash("brute._Bit1DType_singleton")


bit1 = _Bit1DType()

# torch dtype aliases, so that `brute.float32` etc. resolve
bool = torch.bool
float32 = torch.float32
float64 = torch.float64
float16 = torch.float16
bfloat16 = torch.bfloat16
int8 = torch.int8
int16 = torch.int16
int32 = torch.int32
int64 = torch.int64
uint8 = torch.uint8
uint16 = torch.uint16
uint32 = torch.uint32
uint64 = torch.uint64
complex64 = torch.complex64
complex128 = torch.complex128
float8_e4m3fn = torch.float8_e4m3fn
float8_e5m2 = torch.float8_e5m2

_PACK_WIDTH: int = 64
_PACK_STORAGE_DTYPE: torch.dtype = torch.int64
