"""Multi-rank host logic on CPU: world_size 2 over gloo, the device kernels replaced by the CPU
oracle as the local compute.  Checks the row partition, the gathered layout and the int64-key MAX
reduction of the vocabulary-sharded lm_head (tie rule: highest value, lowest index)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cogni_ml_b200 import QuantWeight, synth
from cogni_ml_b200.sharded import (ShardedLmHead, ShardedQuantWeight, pack_top1_key, shard_bytes,
                                   shard_rows, unpack_top1_key)


class OracleShard:
    """CPU stand-in for DeviceQuantWeight over rows [r0, r1): same method names, oracle inside."""

    def __init__(self, qw, r0, r1, device):
        from cogni_ml_b200.quant_matmul import row_bytes
        rb = row_bytes(qw.type, qw.in_dim)
        self.raw, self.type, self.in_dim = qw.raw[r0 * rb:r1 * rb], qw.type, qw.in_dim
        self.out_dim, self.row_begin = r1 - r0, r0

    def _logits(self, x):
        from oracle import loader
        b = x.numel() // self.in_dim
        y = loader.matmul_add(x.numpy(), b, self.in_dim, self.raw, self.type, self.out_dim,
                              np.zeros(self.out_dim, np.float32))
        return y.reshape(b, self.out_dim)

    def gemv(self, x, out=None):
        out.copy_(torch.from_numpy(self._logits(x)))
        return out

    def gemv_top2(self, x, want_keys=False):
        y = self._logits(x)
        order = np.argsort(-y, axis=1, kind="stable")[:, :2]
        val = np.take_along_axis(y, order, axis=1)
        key = pack_top1_key(val, order + self.row_begin)
        return (torch.from_numpy((order + self.row_begin).astype(np.int32)), torch.from_numpy(val),
                torch.from_numpy(key))

    def gemv_top1(self, x, want_keys=False):
        y = self._logits(x)
        idx = y.argmax(axis=1)                       # first maximum, as the CPU reference
        val = y[np.arange(y.shape[0]), idx]
        key = pack_top1_key(val, idx + self.row_begin)
        return (torch.from_numpy((idx + self.row_begin).astype(np.int32)), torch.from_numpy(val),
                torch.from_numpy(key))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dim, in_dim, batch, tie):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import loader
        raw = synth.make_weight(synth.Q6_K, out_dim, in_dim, seed=13)
        if tie:  # identical rows in different shards: equal logits, the lower index must win
            rb = raw.size // out_dim
            raw = raw.copy()
            raw[(out_dim - 3) * rb:(out_dim - 2) * rb] = raw[5 * rb:6 * rb]
        qw = QuantWeight(raw, synth.Q6_K, out_dim, in_dim)
        x = torch.from_numpy(synth.make_activation(batch, in_dim, seed=13))
        full = loader.matmul_add(x.numpy(), batch, in_dim, raw, synth.Q6_K, out_dim,
                                 np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
        y = ShardedQuantWeight(qw, "cpu", local_factory=OracleShard).gemv(x)
        assert y.shape == (batch, out_dim)
        assert np.array_equal(y.numpy(), full), "gathered layout differs from the unsharded result"
        idx, val = ShardedLmHead(qw, "cpu", local_factory=OracleShard).top1(x)
        for b in range(batch):
            ri, rv = loader.top1(full[b])
            assert int(idx[b]) == ri and float(val[b]) == float(rv)
        idx2, val2 = ShardedLmHead(qw, "cpu", local_factory=OracleShard).top2(x)
        for b in range(batch):
            order = np.argsort(-full[b], kind="stable")[:2]
            assert idx2[b].tolist() == order.tolist() and val2[b].tolist() == full[b][order].tolist()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tie", [False, True])
def test_world_size_2_gather_and_argmax_reduce(tie):
    mp.spawn(_worker, args=(2, _free_port(), 64, 512, 3, tie), nprocs=2, join=True)


def test_shard_rows_partition():
    for n, g in [(12288, 8), (151936, 8), (4096, 2), (10, 4), (7, 8)]:
        spans = [shard_rows(n, r, g) for r in range(g)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    assert shard_rows(151936, 3, 8) == (3 * 18992, 4 * 18992)
    with pytest.raises(ValueError):
        shard_rows(10, 4, 4)


def test_shard_bytes_is_a_contiguous_slice():
    raw = synth.make_weight(synth.Q4_K, 16, 512, seed=1)
    qw = QuantWeight(raw, synth.Q4_K, 16, 512)
    parts = [shard_bytes(qw, r, 4) for r in range(4)]
    assert np.array_equal(np.concatenate(parts), raw)
    assert parts[1].base is not None          # a view of the original bytes, not a repack


def test_top1_key_order_and_round_trip():
    vals = np.array([-np.inf, -3.5, -0.0, 0.0, 1e-30, 2.0, 2.0, np.inf], np.float32)
    idx = np.array([9, 8, 7, 6, 5, 4, 3, 2], np.int64)
    keys = pack_top1_key(vals, idx)
    order = np.argsort(keys, kind="stable")
    # keys sort like (value ascending, index descending): the maximum is value 2.0 at index 3
    # once +inf is removed
    assert list(vals[order][:2]) == [-np.inf, -3.5]
    assert keys[6] > keys[5]                   # equal values: lower index has the larger key
    assert keys[3] > keys[2]                   # -0.0 == +0.0 as values: index 6 beats index 7
    i2, v2 = unpack_top1_key(keys)
    assert np.array_equal(i2, idx.astype(np.int32))
    assert np.array_equal(v2, vals)
