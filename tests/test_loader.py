"""Streaming weight upload: chunk planning on the CPU; on a GPU the uploaded bytes are the verbatim
GGUF bytes of the requested rows, for whole tensors and for row shards, read from a memory-mapped
file as the reference's tensors are (src/ml/gguf/reader.cr:183-215)."""
import numpy as np
import pytest

from cogni_ml_b200 import QuantWeight, plan_chunks, synth


def test_plan_chunks_covers_the_range_in_order():
    assert plan_chunks(0, 8) == []
    assert plan_chunks(5, 8) == [(0, 5)]
    assert plan_chunks(16, 8) == [(0, 8), (8, 8)]
    pieces = plan_chunks(1000, 96)
    assert pieces[0] == (0, 96) and pieces[-1] == (960, 40)
    assert sum(s for _, s in pieces) == 1000 and all(pieces[i][0] + pieces[i][1] == pieces[i + 1][0]
                                                     for i in range(len(pieces) - 1))
    with pytest.raises(ValueError):
        plan_chunks(10, 0)


@pytest.mark.gpu
def test_uploader_copies_verbatim_bytes_from_an_mmap(cuda, tmp_path):
    import torch

    from cogni_ml_b200 import WeightUploader
    out_dim, in_dim = 777, 1024
    tensors = []
    path = tmp_path / "weights.bin"
    with open(path, "wb") as f:
        for i, qt in enumerate((synth.Q4_K, synth.Q6_K, synth.Q8_0)):
            raw = synth.make_weight(qt, out_dim, in_dim, seed=i)
            tensors.append((qt, f.tell(), raw.size))
            f.write(raw.tobytes())
    mm = np.memmap(path, dtype=np.uint8, mode="r")
    up = WeightUploader(cuda, chunk_bytes=100_000, n_buffers=2)   # several chunks per tensor
    qws = [QuantWeight(mm[o:o + n], qt, out_dim, in_dim) for qt, o, n in tensors]
    whole = [up.upload(q) for q in qws]
    shards = [up.upload_shard(qws[0], r, 4) for r in range(4)]
    up.finish(whole + shards)
    for q, d in zip(qws, whole):
        assert d.resident and np.array_equal(d.raw.cpu().numpy(), np.asarray(q.raw))
    assert np.array_equal(np.concatenate([s.raw.cpu().numpy() for s in shards]), np.asarray(qws[0].raw))
    assert [s.row_begin for s in shards] == [0, 195, 389, 583] and sum(s.out_dim for s in shards) == out_dim
    assert up.bytes_uploaded == sum(n for _, _, n in tensors) + tensors[0][2]
    # an uploaded weight computes like one uploaded the plain way
    x = torch.from_numpy(synth.make_activation(1, in_dim)).to(cuda)
    from cogni_ml_b200 import DeviceQuantWeight
    ref = DeviceQuantWeight.upload(qws[1], cuda).gemv(x)
    assert torch.equal(whole[1].gemv(x), ref)
