"""Entry points for the parts of the path that the reference composes by hand.

* ``pack_sign``       float -> bit1 in one pass (threshold x > 0 or x >= 0);
* ``binary_linear``   one binarised-MLP layer: xnor GEMM, per-channel fp32
                      scale, re-binarisation, re-pack, fused in the GEMM epilogue;
* ``binary_attention`` sign-binarised Q.K^T scored by popcount, fp32 softmax, @ V;
* ``sharded_matmul``  the xnor GEMM with B's rows (output features) split across
                      the ranks of a ``torch.distributed`` group, optional all-gather.
"""
from __future__ import annotations

from typing import Optional

import torch

from .tensor import Tensor, _is_b1

_ops = torch.ops.brute
SIGN_GT0, SIGN_GE0 = 0, 1


def pack_sign(x: torch.Tensor, ge0: bool = False) -> Tensor:
    """Binarise a float tensor into a bit1 tensor: bit = x > 0, or x >= 0 with ``ge0``."""
    base = x.as_subclass(torch.Tensor)
    packed = _ops.pack_sign(base, SIGN_GE0 if ge0 else SIGN_GT0)
    return Tensor._make_bit1_from_packed(packed, list(base.shape))


def binary_linear(x: Tensor, weight: Tensor, scale: torch.Tensor, ge0: bool = True) -> Tensor:
    """bit1 [M, K] x bit1 weight [N, K] -> bit1 [M, N] = sign(scale[n] * (K - 2H))."""
    K = int(x.shape[-1])
    out = _ops.xnor_matmul_scale_sign_pack(x._packed_buf_contig(), weight._packed_buf_contig(),
                                           scale.as_subclass(torch.Tensor), K, SIGN_GE0 if ge0 else SIGN_GT0)
    return Tensor._make_bit1_from_packed(out, [int(x.shape[0]), int(weight.shape[0])])


def binary_attention(q: Tensor, k: Tensor, v: torch.Tensor, causal: bool = True,
                     scale: Optional[float] = None) -> torch.Tensor:
    """q, k bit1 [B, H, S, D]; v bf16 [B, H, S, D] -> bf16 [B, H, S, D]."""
    if not (_is_b1(q) and _is_b1(k)):
        raise TypeError("binary_attention: q and k must be bit1 tensors")
    D = int(q.shape[-1])
    if scale is None:
        scale = D ** -0.5
    return _ops.binary_attention(q._packed_buf_contig(), k._packed_buf_contig(),
                                 v.as_subclass(torch.Tensor), bool(causal), float(scale))


def shard_bounds(n: int, world_size: int, rank: int) -> tuple:
    """Rows [lo, hi) of an n-row operand owned by `rank`: equal blocks, the last
    ranks one row shorter when world_size does not divide n."""
    base, extra = divmod(n, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sharded_matmul(a_packed: torch.Tensor, b_packed: torch.Tensor, K: int, group=None,
                   gather: bool = False) -> torch.Tensor:
    """Column-sharded xnor GEMM: this rank computes C[:, lo:hi] for its block of
    B's rows. With ``gather`` the blocks are all-gathered (NCCL on GPUs) and
    concatenated so every rank returns the full [M, N] matrix; the collective is
    queued on the same stream right behind the GEMM, with no host sync between."""
    import torch.distributed as dist

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    N = b_packed.shape[0]
    lo, hi = shard_bounds(N, world, rank)
    c_local = _ops.xnor_popcount_matmul(a_packed, b_packed[lo:hi], K)
    if not gather or world == 1:
        return c_local
    M = a_packed.shape[0]
    if N % world == 0:
        # rank blocks arrive stacked along dim 0: [world * M, N / world]
        stacked = torch.empty((world * M, N // world), dtype=c_local.dtype, device=c_local.device)
        dist.all_gather_into_tensor(stacked, c_local.contiguous(), group=group)
        return stacked.view(world, M, N // world).permute(1, 0, 2).reshape(M, N)
    # uneven blocks: pad every block to the widest one, gather, drop the padding
    widths = [shard_bounds(N, world, r)[1] - shard_bounds(N, world, r)[0] for r in range(world)]
    wmax = max(widths)
    padded = torch.zeros((M, wmax), dtype=c_local.dtype, device=c_local.device)
    padded[:, :hi - lo] = c_local
    stacked = torch.empty((world * M, wmax), dtype=c_local.dtype, device=c_local.device)
    dist.all_gather_into_tensor(stacked, padded, group=group)
    blocks = stacked.view(world, M, wmax)
    return torch.cat([blocks[r, :, :widths[r]] for r in range(world)], dim=1)
