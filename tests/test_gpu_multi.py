"""Row / vocabulary sharding on real GPUs: two ranks over NCCL (skipped on a one-GPU box).

Each rank uploads its contiguous row shard, runs the device GEMV / fused lm_head, and the
exchange step (all-gather of shard outputs, MAX all-reduce of top-1 keys) must reproduce the CPU
oracle's unsharded result on every rank."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    import torch.distributed as dist

    from cogni_ml_b200 import QuantWeight, synth
    from cogni_ml_b200.sharded import ShardedLmHead, ShardedQuantWeight
    from oracle import loader

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        for qtype, out_dim, in_dim, batch in [(synth.Q4_K, 2048, 1024, 1), (synth.Q6_K, 1024, 2560, 4)]:
            raw = synth.make_weight(qtype, out_dim, in_dim, seed=17, tensor_id=qtype)
            qw = QuantWeight(raw, qtype, out_dim, in_dim)
            x = synth.make_activation(batch, in_dim, seed=17)
            ref = loader.matmul_add(x, batch, in_dim, raw, qtype, out_dim,
                                    np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
            xd = torch.from_numpy(x).to(dev)
            y = ShardedQuantWeight(qw, dev).gemv(xd).cpu().numpy()
            assert np.abs(y - ref).max() <= 1e-3 * np.abs(ref).max()
            idx, val = ShardedLmHead(qw, dev).top1(xd)
            for b in range(batch):
                ri, rv = loader.top1(ref[b])
                assert int(idx[b]) == ri
                assert abs(float(val[b]) - float(rv)) <= 1e-3 * np.abs(ref[b]).max()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


def test_two_rank_row_sharded_gemv_and_vocab_sharded_top1(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
