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


def _exchange_worker(rank, world, port):
    """The exchange fused into the GEMV launch: launch A leaves y1 = W1 x on every GPU as
    (value, epoch) words (8-byte peer stores), launch B computes W2 y1 straight from those words,
    polling each for A's epoch, and exchanges again; repeated so that epochs and buffers are reused
    many times.  Then two matrices at batch 4 in one launch."""
    import torch.distributed as dist

    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, lib, synth
    from cogni_ml_b200.sharded import ExchangingGemv, PeerExchange, shard_rows
    from oracle import loader

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        n1, k1, n2 = 2048, 1024, 1024
        raw1 = synth.make_weight(synth.Q4_K, n1, k1, seed=27, tensor_id=1)
        raw2 = synth.make_weight(synth.Q6_K, n2, n1, seed=27, tensor_id=2)
        x = synth.make_activation(1, k1, seed=27)
        zero = lambda n: np.zeros(n, np.float32)
        # the chain y1 = W1 x, y2 = W2 y1, y1' = W1 y2, ... : every launch reads the gathered words of
        # the launch before it, so no rank can run ahead of a reader; six GEMVs keep the values
        # (which grow by two orders of magnitude per step) inside the f32 range
        steps = 3
        ref, refs = x, []
        for it in range(steps):
            y1_ref = loader.matmul_add(ref, 1, k1, raw1, synth.Q4_K, n1, zero(n1))
            y2_ref = loader.matmul_add(y1_ref, 1, n1, raw2, synth.Q6_K, n2, zero(n2))
            ref = y2_ref
        ex = PeerExchange(1 << 20, dev)
        r0, r1 = shard_rows(n1, rank, world)
        w1 = DeviceQuantWeight.upload(QuantWeight(raw1, synth.Q4_K, n1, k1), dev, r0, r1)
        r0, r1 = shard_rows(n2, rank, world)
        w2 = DeviceQuantWeight.upload(QuantWeight(raw2, synth.Q6_K, n2, n1), dev, r0, r1)
        buf1 = ex.buffer("y1", 1, n1)
        buf2 = ex.buffer("y2", 1, n2)
        xd = torch.from_numpy(x).to(dev)
        first = ExchangingGemv(ex, [w1], xd, [buf1], wait_previous=False)
        a = ExchangingGemv(ex, [w1], buf2, [buf1], wait_previous=True)     # k1 == n2
        b = ExchangingGemv(ex, [w2], buf1, [buf2], wait_previous=True)
        for rounds in range(12):         # the same three-step chain again and again: epochs 1 .. 72
            for it in range(steps):
                (first if it == 0 else a).run()
                b.run()
            y2 = ex.unpack(buf2).cpu().numpy().reshape(-1)   # waits for the words of the last exchange
            torch.cuda.synchronize()
            dist.barrier()                                    # every rank's launches have completed
            assert np.abs(y2 - y2_ref).max() <= 5e-3 * np.abs(y2_ref).max(), rounds   # six chained GEMVs
        assert ex.epoch() == 72
        y1 = buf1[..., 0].cpu().numpy().reshape(-1)
        assert np.abs(y1 - y1_ref).max() <= 5e-3 * np.abs(y1_ref).max()
        assert lib.cogni_qmm_wait_timeouts() == 0
        # batch 4, two matrices in one launch (the ffn_gate + ffn_up way of use), then a consumer
        # of batch 4 reading the gathered words
        xb = synth.make_activation(4, k1, seed=28)
        rawu = synth.make_weight(synth.Q4_K, n1, k1, seed=28, tensor_id=3)
        r0, r1 = shard_rows(n1, rank, world)
        wu = DeviceQuantWeight.upload(QuantWeight(rawu, synth.Q4_K, n1, k1), dev, r0, r1)
        g_buf = ex.buffer("g4", 4, n1)
        u_buf = ex.buffer("u4", 4, n1)
        d_buf = ex.buffer("d4", 4, n2)
        ExchangingGemv(ex, [w1, wu], torch.from_numpy(xb).to(dev), [g_buf, u_buf], wait_previous=False).run()
        ExchangingGemv(ex, [w2], g_buf, [d_buf], wait_previous=True).run()
        d4 = ex.unpack(d_buf).cpu().numpy()
        torch.cuda.synchronize()
        dist.barrier()
        g_ref = loader.matmul_add(xb, 4, k1, raw1, synth.Q4_K, n1, zero(n1)).reshape(4, n1)
        u_ref = loader.matmul_add(xb, 4, k1, rawu, synth.Q4_K, n1, zero(n1)).reshape(4, n1)
        for ref, buf in ((g_ref, g_buf), (u_ref, u_buf)):
            got = buf[..., 0].cpu().numpy()
            assert np.abs(got - ref).max() <= 1e-3 * np.abs(ref).max()
        d_ref = loader.matmul_add(g_ref, 4, n1, raw2, synth.Q6_K, n2, zero(n2)).reshape(4, n2)
        assert np.abs(d4 - d_ref).max() <= 2e-3 * np.abs(d_ref).max()
        assert lib.cogni_qmm_wait_timeouts() == 0
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _nccl_capi_worker(rank, world, port):
    """The C-ABI entries that take the host's ncclComm_t: the communicator is made here the way a
    host binding would (ncclGetUniqueId on rank 0, ncclCommInitRank everywhere, through ctypes on
    libnccl), the sharded GEMV + all-gather and the sharded fused top-1 + MAX all-reduce run inside
    libcogni_qmm, and every rank must hold the CPU oracle's unsharded answer."""
    import ctypes as C

    import torch.distributed as dist

    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, lib, synth
    from cogni_ml_b200._lib import check
    from cogni_ml_b200.sharded import shard_rows
    from oracle import loader

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nccl = C.CDLL("libnccl.so.2")

    class UniqueId(C.Structure):
        _fields_ = [("internal", C.c_byte * 128)]

    uid = UniqueId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(C.byref(uid)) == 0
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0)
    C.memmove(C.byref(uid), box[0], 128)
    comm = C.c_void_p()
    nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
    assert nccl.ncclCommInitRank(C.byref(comm), world, uid, rank) == 0
    try:
        stream = torch.cuda.current_stream().cuda_stream
        for qtype, out_dim, in_dim, batch in [(synth.Q4_K, 2048, 1024, 1), (synth.Q6_K, 4096, 2560, 8)]:
            raw = synth.make_weight(qtype, out_dim, in_dim, seed=19, tensor_id=qtype)
            x = synth.make_activation(batch, in_dim, seed=19)
            ref = loader.matmul_add(x, batch, in_dim, raw, qtype, out_dim,
                                    np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
            r0, r1 = shard_rows(out_dim, rank, world)
            rows = r1 - r0
            dw = DeviceQuantWeight.upload(QuantWeight(raw, qtype, out_dim, in_dim), dev, r0, r1)
            xd = torch.from_numpy(x).to(dev)
            gather = torch.full((world, batch, rows), float("nan"), dtype=torch.float32, device=dev)
            check(lib.cogni_qmm_sharded_gemv_nccl(comm, world, rank, qtype, dw.raw.data_ptr(), xd.data_ptr(),
                                                  gather.data_ptr(), in_dim, rows, batch, 1, stream),
                  "cogni_qmm_sharded_gemv_nccl")
            y = gather.permute(1, 0, 2).reshape(batch, out_dim).cpu().numpy()
            assert np.abs(y - ref).max() <= 1e-3 * np.abs(ref).max()
            scratch = dw.top1_scratch(batch)
            keys = torch.zeros(batch, dtype=torch.int64, device=dev)
            idx = torch.zeros(batch, dtype=torch.int32, device=dev)
            val = torch.zeros(batch, dtype=torch.float32, device=dev)
            check(lib.cogni_qmm_sharded_top1_nccl(comm, world, qtype, dw.raw.data_ptr(), xd.data_ptr(), in_dim,
                                                  rows, batch, r0, scratch.data_ptr(), scratch.numel(),
                                                  keys.data_ptr(), idx.data_ptr(), val.data_ptr(), stream),
                  "cogni_qmm_sharded_top1_nccl")
            torch.cuda.synchronize()
            for b in range(batch):
                assert int(idx[b]) == loader.top1(ref[b])[0]
        dist.barrier()
    finally:
        nccl.ncclCommDestroy.argtypes = [C.c_void_p]
        nccl.ncclCommDestroy(comm)
        dist.destroy_process_group()


def test_two_rank_sharded_entries_on_the_hosts_nccl_communicator(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_nccl_capi_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_two_rank_exchange_fused_into_the_gemv(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_exchange_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_two_rank_row_sharded_gemv_and_vocab_sharded_top1(cuda):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
