"""The allocation-free lm_head entry point against the ordinary one.

Some callers of this library cannot allocate device memory when they need the lm_head (all of HBM
already belongs to their own arena, or their host only lends them input and output buffers), so
cogni_qmm_gemv_top1_noalloc keeps its scratch in a fixed array inside the library.  It must give
the same (index, value, key) as cogni_qmm_gemv_top1 with a caller-provided scratch buffer, on
every call: the array is shared and keeps the previous call's contents, so two calls in a row
with different inputs are checked.  This file is named to be collected last.
"""
import numpy as np
import pytest
import torch

from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth
from cogni_ml_b200._lib import check, lib

pytestmark = pytest.mark.gpu


def _noalloc_top1(dw, x):
    batch = x.shape[0]
    idx = torch.full((batch,), -1, dtype=torch.int32, device=x.device)
    val = torch.full((batch,), float("nan"), dtype=torch.float32, device=x.device)
    key = torch.zeros(batch, dtype=torch.int64, device=x.device)
    check(lib.cogni_qmm_gemv_top1_noalloc(dw.type, dw.raw.data_ptr(), x.data_ptr(), dw.in_dim,
                                          dw.out_dim, batch, dw.row_begin, idx.data_ptr(),
                                          val.data_ptr(), key.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream),
          "cogni_qmm_gemv_top1_noalloc")
    return idx, val, key


def test_noalloc_top1_matches_scratch_entry_point_twice(cuda, oracle):
    out_dim, in_dim = 9000, 1024
    w = synth.make_weight(synth.Q6_K, out_dim, in_dim, seed=91)
    dw = DeviceQuantWeight.upload(QuantWeight(w, synth.Q6_K, out_dim, in_dim), cuda)
    dw.row_begin = 123
    for call, batch in enumerate([4, 2]):   # second call: other inputs, smaller batch, same array
        x = torch.from_numpy(synth.make_activation(batch, in_dim, seed=91 + call)).to(cuda)
        ref_idx, ref_val, ref_key = dw.gemv_top1(x, want_keys=True)
        idx, val, key = _noalloc_top1(dw, x)
        torch.cuda.synchronize()
        assert torch.equal(idx, ref_idx), f"call {call}"
        assert torch.equal(key, ref_key), f"call {call}"
        # same kernel, same reduction order: the values agree to the last bit, well inside the
        # 1e-3 * |y|inf tolerance the parity tests allow
        assert torch.equal(val, ref_val), f"call {call}"
        # and against the CPU oracle: QuantMatmul, then the first maximum (shard offset added)
        xh = x.cpu().numpy()
        logits = oracle.matmul_add(xh, batch, in_dim, w, synth.Q6_K, out_dim,
                                   np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
        for b in range(batch):
            oi, ov = oracle.top1(logits[b])
            assert int(idx[b]) == oi + 123, f"call {call} row {b}"
            assert abs(float(val[b]) - float(ov)) <= 1e-3 * abs(float(ov))


def test_noalloc_top1_rejects_shapes_beyond_the_fixed_array(cuda):
    limit = lib.cogni_qmm_gemv_top1_noalloc_max_scratch()
    assert limit == 1 << 20
    out_dim, batch = 1 << 22, 16
    assert lib.cogni_qmm_gemv_top1_scratch_bytes(out_dim, batch) > limit
    x = torch.zeros(batch, 256, dtype=torch.float32, device=cuda)
    w = torch.zeros(256, dtype=torch.uint8, device=cuda)   # never read: the size check comes first
    out = torch.zeros(batch, dtype=torch.int32, device=cuda)
    val = torch.zeros(batch, dtype=torch.float32, device=cuda)
    st = lib.cogni_qmm_gemv_top1_noalloc(synth.Q6_K, w.data_ptr(), x.data_ptr(), 256, out_dim,
                                         batch, 0, out.data_ptr(), val.data_ptr(), None, None)
    assert st == 1006
    assert b"maximum" in lib.cogni_qmm_status_string(st)
