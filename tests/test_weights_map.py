"""The name -> weight map and the recurrent layer's validation, on CPU (device upload replaced by a
recorder), in the manner of spec/qwen35_weights_spec.cr and spec/qwen35_weights_lifecycle_spec.cr."""
import threading

import numpy as np
import pytest

from cogni_ml_b200 import synth
from cogni_ml_b200.weights import GGUFTensor, Qwen35DeviceWeights, RecurrentLayerWeights, load_qw

Q4_K, Q5_K, Q6_K = synth.Q4_K, synth.Q5_K, synth.Q6_K


def tiny_tensor(name, qtype, in_dim, out_dim):
    # bytes are never read by these tests: a zero view of the right size is enough
    return GGUFTensor(name, qtype, [in_dim, out_dim], np.zeros(synth.tensor_bytes(qtype, out_dim, in_dim), np.uint8))


def recurrent_layer(layer=0, hidden=256, ffn=512, down_type=Q6_K, qkv_type=Q5_K):
    p = f"blk.{layer}"
    t = [tiny_tensor(f"{p}.attn_qkv.weight", qkv_type, hidden, 8192),
         tiny_tensor(f"{p}.attn_gate.weight", Q4_K, hidden, 4096),
         tiny_tensor(f"{p}.ssm_alpha.weight", Q4_K, hidden, 32),
         tiny_tensor(f"{p}.ssm_beta.weight", Q4_K, hidden, 32),
         GGUFTensor(f"{p}.ssm_out.weight", Q4_K, [4096, hidden], np.zeros(synth.tensor_bytes(Q4_K, hidden, 4096), np.uint8)),
         tiny_tensor(f"{p}.ffn_gate.weight", Q4_K, hidden, ffn),
         tiny_tensor(f"{p}.ffn_up.weight", Q4_K, hidden, ffn),
         tiny_tensor(f"{p}.ffn_down.weight", down_type, ffn, hidden)]
    return {x.name: x for x in t}


def test_load_qw_follows_the_gguf_convention():
    t = recurrent_layer()
    qw = load_qw(t, "blk.0.ffn_gate.weight")
    assert (qw.in_dim, qw.out_dim, qw.type, qw.route_tag) == (256, 512, Q4_K, "qwen35:blk.0.ffn_gate.weight")
    with pytest.raises(KeyError, match="missing tensor 'blk.9.ffn_gate.weight'"):
        load_qw(t, "blk.9.ffn_gate.weight")


def test_recurrent_layer_validation_matches_the_runner():
    w = RecurrentLayerWeights.load(recurrent_layer(), 0)
    assert (w.hidden, w.ffn_dim, w.out_dim, w.qkv_dim, w.ffn_down_type) == (256, 512, 256, 8192, Q6_K)
    assert set(w.weights) == {"attn_qkv", "attn_gate", "ssm_alpha", "ssm_beta", "ssm_out", "ffn_gate",
                              "ffn_up", "ffn_down"}
    assert RecurrentLayerWeights.load(recurrent_layer(down_type=Q4_K), 0).ffn_down_type == Q4_K
    with pytest.raises(ValueError, match="expected Q5_K attn_qkv"):
        RecurrentLayerWeights.load(recurrent_layer(qkv_type=Q4_K), 0)
    with pytest.raises(ValueError, match="expected Q4_K ffn gate/up and Q4_K/Q6_K ffn down"):
        RecurrentLayerWeights.load(recurrent_layer(down_type=Q5_K), 0)
    with pytest.raises(ValueError, match="missing blk.3.attn_qkv.weight"):
        RecurrentLayerWeights.load(recurrent_layer(), 3)
    bad = recurrent_layer()
    bad["blk.0.ffn_up.weight"] = tiny_tensor("blk.0.ffn_up.weight", Q4_K, 256, 768)
    with pytest.raises(ValueError, match="ffn shape mismatch"):
        RecurrentLayerWeights.load(bad, 0)


class Backing:
    def __init__(self):
        self.closes = 0

    def close(self):
        self.closes += 1


def test_device_map_shards_rows_and_closes_once_from_many_threads():
    tensors = recurrent_layer()
    uploads = []

    def upload(qw, r0, r1):
        uploads.append((qw.route_tag, r0, r1))
        return (qw, r0, r1)

    backing = Backing()
    w = Qwen35DeviceWeights(tensors, "cpu", backing=backing, rank=1, world=4, upload=upload)
    assert ("qwen35:blk.0.ffn_gate.weight", 128, 256) in uploads
    assert w["blk.0.ffn_down.weight"][1:] == (64, 128)
    assert set(w.layer(0)) == {"attn_qkv", "attn_gate", "ssm_alpha", "ssm_beta", "ssm_out", "ffn_gate",
                               "ffn_up", "ffn_down"}
    with pytest.raises(KeyError, match="missing tensor"):
        w["blk.1.ffn_down.weight"]
    threads = [threading.Thread(target=w.close) for _ in range(4)]   # as the lifecycle spec: 4 closers
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    w.close()
    assert w.closed and backing.closes == 1
    with pytest.raises(RuntimeError, match="closed"):
        w["blk.0.ffn_gate.weight"]
