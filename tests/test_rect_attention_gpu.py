"""GPU parity of the rectangular flash attention (hz_mha_rect_fwd) and the 2-FWL panel product
(hz_fwl2_panel) against the float64 oracle. Tolerance: 1e-5 of the output scale (three-term TF32
contractions, base-2 online softmax in fp32)."""
import numpy as np
import pytest
import torch

from hamiltonzero_b200 import sequence_parallel as SP
from oracle import attention as A

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("lq,lk,h,d,masked", [
    (16, 32, 4, 8, 0.0),          # one block
    (128, 1024, 8, 32, 0.2),      # a rank's rows against 1024 gathered keys
    (100, 200, 8, 16, 0.3),       # ragged rows and keys
    (37, 77, 4, 64, 0.1),
    (64, 96, 16, 32, 0.5),        # sixteen heads (one stage of shared memory)
    (33, 64, 8, 32, 0.97),        # almost everything masked
])
def test_rectangular_attention_matches_oracle(hz_lib, lq, lk, h, d, masked):
    rng = np.random.default_rng(lq + lk)
    q, = (rng.standard_normal((lq, h, d)).astype(np.float32),)
    k, v = (rng.standard_normal((lk, h, d)).astype(np.float32) for _ in range(2))
    bias = (2.0 * rng.standard_normal((lq, lk, h))).astype(np.float32)
    mask = (rng.random(lk) >= masked).astype(np.uint8)
    mask[rng.integers(lk)] = 1
    got = SP.rectangular_edge_attention(q, k, v, bias, mask)
    want = A.rectangular_edge_attention(q, k, v, bias, mask)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


def test_fully_masked_keys_give_the_mean_of_v_like_the_reference(hz_lib):
    """Every key masked: all scores are -1e30 + O(1), which fp32 rounds to the same number, so
    the softmax is uniform - the reference's kernel returns the mean of v, and so does this one
    when the key count is a multiple of the key block."""
    rng = np.random.default_rng(3)
    lq, lk, h, d = 16, 64, 4, 16
    q, k, v = (rng.standard_normal((n, h, d)).astype(np.float32) for n in (lq, lk, lk))
    bias = rng.standard_normal((lq, lk, h)).astype(np.float32)
    got = SP.rectangular_edge_attention(q, k, v, bias, np.zeros(lk, np.uint8))
    np.testing.assert_allclose(got, np.broadcast_to(v.mean(0), got.shape), rtol=1e-5, atol=1e-6)


def test_batched_call_and_argument_checks(hz_lib):
    rng = np.random.default_rng(4)
    b, lq, lk, h, d = 3, 48, 80, 8, 32
    q = rng.standard_normal((b, lq, h, d)).astype(np.float32)
    k, v = (rng.standard_normal((b, lk, h, d)).astype(np.float32) for _ in range(2))
    bias = rng.standard_normal((b, lq, lk, h)).astype(np.float32)
    got = SP.noncausal_bias_mha(q, k, v, bias)
    for i in range(b):
        want = A.rectangular_edge_attention(q[i], k[i], v[i], bias[i], np.ones(lk))
        assert np.abs(got[i] - want).max() <= 1e-5 * np.abs(want).max()
    with pytest.raises(ValueError):
        SP.noncausal_bias_mha(q, k, v, bias[:, :, :, :4])
    with pytest.raises(ValueError):
        SP.rectangular_edge_attention(q[0], k[0], v[0], bias[0], np.ones(lk + 1))
    from hamiltonzero_b200._lib import HzError
    with pytest.raises(HzError):
        SP.noncausal_bias_mha(q[..., :12].copy(), k[..., :12].copy(), v[..., :12].copy(), bias)   # D = 12


def test_fwl2_panel_and_single_rank_ring(hz_lib):
    rng = np.random.default_rng(5)
    rows, world, cols, c = 24, 3, 40, 12
    a = torch.from_numpy(rng.standard_normal((rows, rows * world, c)).astype(np.float32)).cuda()
    panels = [torch.from_numpy(rng.standard_normal((rows, cols, c)).astype(np.float32)).cuda()
              for _ in range(world)]
    out = torch.empty(rows, cols, c, device="cuda")
    for origin, p in enumerate(panels):
        SP.fwl2_panel(a, p, out, origin, origin > 0)
    want = np.einsum("ikc,kjc->ijc", a.cpu().numpy().astype(np.float64),
                     torch.cat(panels).cpu().numpy().astype(np.float64))
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    sq = torch.from_numpy(rng.standard_normal((16, 16, 8)).astype(np.float32)).cuda()
    got = SP.ring_learned_fwl2_local(sq, sq)
    want = np.einsum("ikc,kjc->ijc", sq.cpu().numpy().astype(np.float64), sq.cpu().numpy().astype(np.float64))
    assert np.abs(got.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()


def _sp_worker(rank, world, port, data, out):
    import os
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        q, k, v, bias, mask, a, b = (torch.from_numpy(x).cuda() for x in data)
        n = q.shape[0] // world
        rows = slice(rank * n, (rank + 1) * n)
        att = SP.sequence_parallel_edge_attention(q[rows], k[rows].contiguous(), v[rows].contiguous(),
                                                  bias[rows].contiguous(), mask[rows].contiguous())
        fwl = SP.ring_learned_fwl2_local(a[rows].contiguous(), b[rows].contiguous())
        torch.cuda.synchronize()
        out[rank] = (att.cpu().numpy(), fwl.cpu().numpy())
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_on_two_gpus(hz_lib):
    """All-gather of keys/values + the rectangular kernel, and the 2-FWL ring (paired
    send/receive + the panel kernel), one process per GPU over NCCL, against the unsharded oracle.
    Skipped on a box with one GPU; the same logic runs on gloo in tests/test_sequence_parallel.py."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    import torch.multiprocessing as mp
    rng = np.random.default_rng(6)
    n, h, d, c = 256, 8, 32, 16
    q, k, v = (rng.standard_normal((n, h, d)).astype(np.float32) for _ in range(3))
    bias = rng.standard_normal((n, n, h)).astype(np.float32)
    mask = (rng.random(n) > 0.2).astype(np.uint8)
    a = rng.standard_normal((n, n, c)).astype(np.float32)
    b = rng.standard_normal((n, n, c)).astype(np.float32)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_sp_worker, args=(2, port, (q, k, v, bias, mask, a, b), out), nprocs=2, join=True)
    att = np.concatenate([out[0][0], out[1][0]])
    fwl = np.concatenate([out[0][1], out[1][1]])
    want = A.rectangular_edge_attention(q, k, v, bias, mask)
    assert np.abs(att - want).max() <= 1e-5 * np.abs(want).max()
    want = np.einsum("ikc,kjc->ijc", a.astype(np.float64), b.astype(np.float64))
    assert np.abs(fwl - want).max() <= 1e-5 * np.abs(want).max()
