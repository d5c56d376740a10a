"""Drives tests/op_catalog.py: every operation of the table on torch.bool and on bit1.

Three drivers, as in the reference's suite (tests/unit/test_parity_catalog.py:64-80,
test_edge_cases_catalog.py:36-68, test_fuzz_catalog.py:56-113 there): small fixed shapes, the edge
cases each operation declares (empty, 0-dim, non-contiguous, broadcasting, a ragged last dimension,
several packed words per row), and seeded random shapes. Runs on CPU tensors (the CPU dispatch key of
torch.ops.brute.* is bound to the oracle by tests/conftest.py, so the subclass state machine runs
without a GPU) and, marked gpu, on CUDA tensors with the product's kernels.
"""
import os

import pytest
import torch

import op_catalog as cat

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]
EDGES = ("empty", "0-dim", "non-contig", "broadcast", "tail", "wide")


@pytest.fixture(scope="module")
def brute(lib_built):
    import conftest
    conftest.install_oracle_cpu_ops()
    import brute_b200
    return brute_b200


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("op", cat.OPS, ids=lambda o: o.name)
def test_parity(op, device, brute):
    cat.run_case(op, cat.edge_inputs(op, "base", device), brute)


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("op", cat.OPS, ids=lambda o: o.name)
def test_edges(op, device, brute):
    ran = 0
    for edge in EDGES:
        if edge not in op.edges:
            continue
        bools = cat.edge_inputs(op, edge, device)
        if bools is None:
            continue
        cat.run_case(op, bools, brute)
        ran += 1
    if not ran:
        pytest.skip("no edge case applies")


def _fuzz_shapes(op, rng):
    if op.kind in ("vector", "diagvec"):
        n = int(rng.integers(1, 131 if op.kind == "vector" else 20))
        return [(n,)] * op.arity
    if op.kind == "matrix":
        r, c = int(rng.integers(1, 9)), int(rng.integers(1, 140))
        return [(r, c)] * op.arity
    m, n = int(rng.integers(1, 9)), int(rng.integers(1, 9))
    k = int(rng.choice([1, 13, 64, 65, 128, 192, 200]))
    return [(m, k), (n, k)][:op.arity]


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("op", cat.OPS, ids=lambda o: o.name)
def test_fuzz(op, device, brute):
    import numpy as np
    examples = int(os.environ.get("BRUTE_FUZZ_EXAMPLES", "6"))
    seed = int(os.environ.get("BRUTE_TEST_SEED", "1234"))
    rng = np.random.default_rng([seed, abs(hash(op.name)) % (2 ** 31)] if False else [seed, len(op.name), sum(map(ord, op.name))])
    for i in range(examples):
        shapes = _fuzz_shapes(op, rng)
        bools = [cat.rand_bool(s, device, 1000 * i + j + sum(map(ord, op.name))) for j, s in enumerate(shapes)]
        cat.run_case(op, bools, brute)
