"""The seeded synthetic tensors: determinism, layouts and the value ranges the configs specify."""
import numpy as np

from cogni_ml_b200 import synth


def test_same_seed_same_bytes_and_chunking_does_not_matter_for_size():
    a = synth.make_weight(synth.Q6_K, 33, 512, seed=3, tensor_id=7)
    b = synth.make_weight(synth.Q6_K, 33, 512, seed=3, tensor_id=7)
    c = synth.make_weight(synth.Q6_K, 33, 512, seed=4, tensor_id=7)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert a.size == 33 * 2 * 210
    assert synth.tensor_bytes(synth.Q4_K, 12288, 4096) == 28_311_552


def test_value_ranges_follow_the_benchmark_configs(oracle):
    n = 64
    w8 = synth.make_weight(synth.Q8_0, n, 1024, seed=1).reshape(-1, 34)
    d8 = w8[:, :2].copy().view(np.float16).astype(np.float32).ravel()
    q8 = w8[:, 2:].view(np.int8)
    assert (d8 >= 0).all() and d8.max() < 0.02 * 6 / 127 and q8.min() >= -127
    w4 = synth.make_weight(synth.Q4_K, n, 1024, seed=1).reshape(-1, 144)
    d4 = w4[:, :4].copy().view(np.float16).astype(np.float32)
    assert (d4 >= 0).all() and d4.max() < 0.07
    for j in range(8):
        sc, m = zip(*(oracle.get_scale_min_k4(j, blk[4:16]) for blk in w4[:50]))
        assert 0 <= min(sc) and max(sc) <= 63 and 0 <= min(m) and max(m) <= 63
    w6 = synth.make_weight(synth.Q6_K, n, 1024, seed=1).reshape(-1, 210)
    sc6 = w6[:, 192:208].view(np.int8)
    assert sc6.min() >= -64 and sc6.max() <= 63
    d6 = w6[:, 208:210].copy().view(np.float16).astype(np.float32)
    assert (d6 >= 0).all() and d6.max() < 0.007
    # many Q6_K / Q8_0 scales are subnormal halves, as the real distributions produce
    assert (w6[:, 209] < 0x04).mean() > 0.01


def test_activations_are_standard_normal():
    x = synth.make_activation(16, 4096, seed=0)
    assert x.dtype == np.float32 and x.shape == (16, 4096)
    assert abs(float(x.mean())) < 0.02 and abs(float(x.std()) - 1.0) < 0.02
