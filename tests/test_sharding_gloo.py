"""The multi-rank layout of the column-sharded GEMM and of the head-sharded attention on two CPU ranks (gloo).

Checks the partition of B's rows, the local GEMM per rank and the layout of the
optional all-gather against the unsharded result. The CPU ranks use the oracle
for the local contraction (see tests/conftest.py); the collective and the layout
logic are the product's (brute_b200/kernels.py)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, n_rows, result_dir):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import conftest
    conftest.install_oracle_cpu_ops()
    from brute_b200.kernels import shard_bounds, sharded_matmul
    g = torch.Generator().manual_seed(1234)                 # same operands on every rank
    K = 200
    a = torch.randint(0, 2, (9, K), generator=g).bool()
    b = torch.randint(0, 2, (n_rows, K), generator=g).bool()
    ap, bp = torch.ops.brute.pack_bool(a), torch.ops.brute.pack_bool(b)
    full = torch.ops.brute.xnor_popcount_matmul(ap, bp, K)
    lo, hi = shard_bounds(n_rows, world, rank)
    local = sharded_matmul(ap, bp, K, gather=False)
    assert torch.equal(local, full[:, lo:hi])
    gathered = sharded_matmul(ap, bp, K, gather=True)
    assert torch.equal(gathered, full)
    # the pipelined gather: several row blocks, int16 transport (K <= 32767) and int32 transport
    for blocks in (1, 2, 4, 9):
        assert torch.equal(sharded_matmul(ap, bp, K, gather=True, row_blocks=blocks), full), blocks
    import brute_b200.kernels as kernels
    full_wide = torch.ops.brute.xnor_popcount_matmul(ap, bp, K)
    wide = kernels._gather_row_blocks(ap, bp[lo:hi], 40000, world, None, 3) if n_rows % world == 0 else None
    if wide is not None:          # K > 32767 keeps int32 on the wire; the integers differ only by the K offset
        assert torch.equal(wide - (40000 - K), full_wide)
    np.save(os.path.join(result_dir, f"ok{rank}.npy"), np.array([lo, hi]))
    dist.barrier()
    dist.destroy_process_group()


def _attention_worker(rank, world, port, heads, result_dir):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import conftest
    conftest.install_oracle_cpu_ops()
    import brute_b200 as brute
    from brute_b200.kernels import shard_bounds, sharded_attention
    g = torch.Generator().manual_seed(99)                   # same operands on every rank
    B, H, S, D = 1, heads, 40, 64
    q = brute.pack_sign(torch.randn((B, H, S, D), generator=g), ge0=True)
    k = brute.pack_sign(torch.randn((B, H, S, D), generator=g), ge0=True)
    v = torch.randn((B, H, S, D), generator=g).to(torch.bfloat16)
    full = brute.binary_attention(q, k, v, causal=True)
    lo, hi = shard_bounds(B * H, world, rank)
    local = sharded_attention(q, k, v, causal=True)
    assert local.shape == (hi - lo, S, D)
    assert torch.equal(local, full.reshape(B * H, S, D)[lo:hi])
    gathered = sharded_attention(q, k, v, causal=True, gather=True)
    assert torch.equal(gathered, full)
    np.save(os.path.join(result_dir, f"att{rank}.npy"), np.array([lo, hi]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 3])
def test_two_rank_sharded_attention(tmp_path, lib_built, heads):
    port = 30500 + (os.getpid() % 1000) + heads
    mp.spawn(_attention_worker, args=(2, port, heads, str(tmp_path)), nprocs=2, join=True)
    spans = [np.load(tmp_path / f"att{r}.npy") for r in range(2)]
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == heads


@pytest.mark.parametrize("n_rows", [16, 13])
def test_two_rank_sharded_gemm(tmp_path, lib_built, n_rows):
    port = 29500 + (os.getpid() % 1000) + n_rows
    mp.spawn(_worker, args=(2, port, n_rows, str(tmp_path)), nprocs=2, join=True)
    spans = [np.load(tmp_path / f"ok{r}.npy") for r in range(2)]
    assert spans[0][0] == 0 and spans[0][1] == spans[1][0] and spans[1][1] == n_rows


def test_four_rank_sharded_gemm(tmp_path, lib_built):
    """The same checks with four ranks: the replicated result is assembled from four rank blocks
    (int16 transport, row blocks) and must equal the local GEMM on every rank."""
    port = 29500 + (os.getpid() % 1000) + 77
    mp.spawn(_worker, args=(4, port, 16, str(tmp_path)), nprocs=4, join=True)
    spans = [np.load(tmp_path / f"ok{r}.npy") for r in range(4)]
    assert spans[0][0] == 0 and spans[-1][1] == 16
    assert all(spans[i][1] == spans[i + 1][0] for i in range(3))


def test_shard_bounds_cover_everything():
    from brute_b200.kernels import shard_bounds
    for n in (0, 1, 7, 16, 16384):
        for w in (1, 2, 4, 8):
            spans = [shard_bounds(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(w - 1))
            assert max(h - l for l, h in spans) - min(h - l for l, h in spans) <= 1
