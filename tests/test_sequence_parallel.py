"""Host logic of the sequence-parallel path on CPU with a world_size-2 gloo group: the
all-gather around the rectangular attention and the 2-FWL ring, each against the unsharded
computation (the CUDA kernels are replaced by their einsum twins here; their parity is in
tests/test_rect_attention_gpu.py)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hamiltonzero_b200 import sequence_parallel as SP
from oracle import attention as A


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _twin(q, k, v, bias, mask):
    return torch.from_numpy(A.rectangular_edge_attention(q.numpy(), k.numpy(), v.numpy(), bias.numpy(),
                                                         mask.numpy()))


def _worker(rank, world, port, data, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, bias, mask, a, b = (torch.from_numpy(x) for x in data)
        n = q.shape[0] // world
        rows = slice(rank * n, (rank + 1) * n)
        att = SP.sequence_parallel_edge_attention(q[rows], k[rows], v[rows], bias[rows], mask[rows],
                                                  attention=_twin)
        fwl = SP.ring_learned_fwl2_local(a[rows].contiguous(), b[rows].contiguous())
        out[rank] = (att.numpy(), fwl.numpy())
    finally:
        dist.destroy_process_group()


def test_gather_and_ring_match_the_unsharded_computation_gloo():
    rng = np.random.default_rng(0)
    n, h, d, c = 12, 4, 8, 5
    q, k, v = (rng.standard_normal((n, h, d)).astype(np.float32) for _ in range(3))
    bias = rng.standard_normal((n, n, h)).astype(np.float32)
    mask = (rng.random(n) > 0.3).astype(np.uint8)
    a = rng.standard_normal((n, n, c)).astype(np.float32)
    b = rng.standard_normal((n, n, c)).astype(np.float32)
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, _free_port(), (q, k, v, bias, mask, a, b), out), nprocs=2, join=True)
    att = np.concatenate([out[0][0], out[1][0]])
    fwl = np.concatenate([out[0][1], out[1][1]])
    np.testing.assert_allclose(att, A.rectangular_edge_attention(q, k, v, bias, mask), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(fwl, np.einsum("ikc,kjc->ijc", a, b), rtol=1e-5, atol=1e-5)


def test_single_process_ring_is_the_plain_product_and_checks_shapes():
    import pytest
    rng = np.random.default_rng(1)
    a = torch.from_numpy(rng.standard_normal((6, 6, 3)).astype(np.float32))
    b = torch.from_numpy(rng.standard_normal((6, 4, 3)).astype(np.float32))
    got = SP.ring_learned_fwl2_columns_local(a, b)
    np.testing.assert_allclose(got.numpy(), np.einsum("ikc,kjc->ijc", a.numpy(), b.numpy()), rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        SP.ring_learned_fwl2_columns_local(a, b[:5])
    with pytest.raises(ValueError):
        SP.ring_learned_fwl2_local(a, b)
    with pytest.raises(TypeError):
        SP.ring_learned_fwl2_columns_local(a, b.double())


def test_rectangular_oracle_reduces_to_the_square_twin():
    """With Lq = Lk and the keys-only mask the rectangular restatement equals the einsum twin
    of the square op (both follow the same softmax; -1e30 against -1e9 on masked keys)."""
    rng = np.random.default_rng(2)
    n, h, d = 10, 4, 8
    q, k, v = (rng.standard_normal((n, h, d)) for _ in range(3))
    bias = rng.standard_normal((n, n, h))
    mask = np.array([1, 1, 0, 1, 1, 1, 0, 1, 1, 1])
    np.testing.assert_allclose(A.rectangular_edge_attention(q, k, v, bias, mask),
                               A.reference_edge_attention(q, k, v, bias, mask), rtol=1e-12, atol=1e-12)
