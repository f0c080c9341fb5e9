"""The CPU oracle pinned to reference-authored code, on the GPU.

The reference holds no golden vectors for Q8_0 / Q4_K / Q5_K / Q6_K, but it ships an independent
implementation of exactly this arithmetic that runs on the device: its hand-written PTX GEMV kernels
(src/ml/cuda/kernels/q4k_gemv_probe.ptx, q5k_gemv_probe.ptx, q6k_gemv_probe.ptx,
q4k_dual_gemv_probe.ptx, the heredocs in bin/cuda_q8_gemv_probe.cr:39-227 and
src/ml/cuda/qwen_output_head_runner.cr:14-625).  oracle/make_ref.py assembles them, unmodified, into
cubins; here they are loaded with cuModuleLoadData and launched exactly as the reference's probes
launch them (bin/cuda_q4k_gemv_probe.cr:158-266), and three things are compared on the same seeded
tensors:
    oracle (the C restatement of QuantMatmul.matmul_add)   vs   the reference's kernels   (the pin)
    this engine's kernels                                   vs   the reference's kernels
The thresholds are the reference probes' own: cos >= 0.99999 and max_diff <= 1e-3
(bin/cuda_q4k_gemv_probe.cr:289, cuda_q5k:216, cuda_q6k:601); Q8_0 cos >= 0.999999 and
max_diff <= 1e-4 (bin/cuda_q8_gemv_probe.cr:390).  The probes apply max_diff as an absolute bound to
model tensors whose outputs are of order 1; the benchmark's synthetic distributions give outputs of
order 100, so the same bound is applied relative to |y|inf there, and literally (absolute) on the
`unit` variants, whose activations are N(0,1) * 2**-12 so that |y|inf <= 1.
"""
import numpy as np
import pytest
import torch

from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth

pytestmark = pytest.mark.gpu

Q8_0, Q4_K, Q5_K, Q6_K = synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K
K_TYPES = [Q4_K, Q5_K, Q6_K]


@pytest.fixture(scope="module")
def ref(cuda):
    from oracle import ref_kernels
    if not ref_kernels.available():
        pytest.fail("oracle/_ref/*.cubin missing: run `python oracle/make_ref.py` where the reference "
                    "checkout is available (the built cubins travel with the repository snapshot)")
    torch.zeros(1, device=cuda)  # torch's primary context is current on this thread from here on
    return ref_kernels


def cosine(a, b):
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def thresholds(qtype):
    return (0.999999, 1e-4) if qtype == Q8_0 else (0.99999, 1e-3)


def assert_probe_ok(got, want, qtype, what, absolute=False):
    cos_min, diff_max = thresholds(qtype)
    scale = 1.0 if absolute else max(1.0, float(np.abs(want).max()))
    diff = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max())
    cos = cosine(got, want)
    print(f"{what} cos={cos:.9f} max_diff={diff:.3e} ymax={float(np.abs(want).max()):.3e} "
          f"ok={cos >= cos_min and diff <= diff_max * scale}")
    assert cos >= cos_min, f"{what}: cos {cos}"
    assert diff <= diff_max * scale, f"{what}: max_diff {diff:.3e} > {diff_max} * {scale:.3e}"


def upload(cuda, w, x):
    return torch.from_numpy(w).to(cuda), torch.from_numpy(x).to(cuda)


SHAPES = {  # small first; then the benchmark configurations' own shapes
    Q8_0: [(64, 1024), (3584, 1024)],
    Q4_K: [(64, 1024), (12288, 4096), (1024, 4096)],
    Q5_K: [(64, 1024), (4096, 4096)],
    Q6_K: [(64, 1024), (4096, 12288), (256, 5120)],
}


@pytest.mark.parametrize("qtype", [Q8_0] + K_TYPES)
@pytest.mark.parametrize("variant", ["baseline", "unit"])
def test_oracle_and_engine_against_reference_warp4(cuda, oracle, ref, qtype, variant):
    for out_dim, in_dim in SHAPES[qtype]:
        w = synth.make_weight(qtype, out_dim, in_dim, seed=31, tensor_id=qtype)
        x = synth.make_activation(1, in_dim, seed=31)
        if variant == "unit":
            x = x * np.float32(2.0 ** -12)  # exact: every product and sum scales with it
        dw, dx = upload(cuda, w, x)
        out = torch.full((out_dim,), float("nan"), dtype=torch.float32, device=cuda)
        torch.cuda.synchronize()
        ref.gemv_warp4(qtype, dw.data_ptr(), dx.data_ptr(), out.data_ptr(), in_dim, out_dim)
        ref.synchronize()
        y_ref = out.cpu().numpy()
        assert np.isfinite(y_ref).all(), "the reference kernel left rows unwritten"
        y_cpu = oracle.matmul_add(x, 1, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                                  threads=oracle.max_threads())
        absolute = variant == "unit"
        if absolute:
            assert np.abs(y_cpu).max() <= 1.0
        tag = f"type={qtype} {out_dim}x{in_dim} {variant}"
        assert_probe_ok(y_cpu, y_ref, qtype, f"oracle_vs_reference_ptx {tag}", absolute)
        eng = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
        y_eng = eng.gemv(dx).cpu().numpy().ravel()
        assert_probe_ok(y_eng, y_ref, qtype, f"engine_vs_reference_ptx {tag}", absolute)


@pytest.mark.parametrize("qtype", K_TYPES)
def test_oracle_against_reference_tbatch4_and_batched(cuda, oracle, ref, qtype):
    """The weight-stationary four-token kernels and the row-batched ones (x [tokens][in_dim], out
    [tokens][out_dim]; q4k_gemv_probe.ptx:437,1584; q5k:237,589; q6k:977,1582)."""
    out_dim, in_dim = {Q4_K: (4096, 4096), Q5_K: (4096, 4096), Q6_K: (4096, 12288)}[qtype]
    w = synth.make_weight(qtype, out_dim, in_dim, seed=32, tensor_id=qtype)
    x = synth.make_activation(4, in_dim, seed=32)
    dw, dx = upload(cuda, w, x)
    y_cpu = oracle.matmul_add(x, 4, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                              threads=oracle.max_threads())
    for name in ("tbatch4", "batched"):
        out = torch.full((4, out_dim), float("nan"), dtype=torch.float32, device=cuda)
        torch.cuda.synchronize()
        if name == "tbatch4":
            ref.gemv_tbatch4(qtype, dw.data_ptr(), dx.data_ptr(), out.data_ptr(), in_dim, out_dim)
        else:
            ref.gemv_batched(qtype, dw.data_ptr(), dx.data_ptr(), out.data_ptr(), in_dim, out_dim, 4)
        ref.synchronize()
        y_ref = out.cpu().numpy().ravel()
        assert np.isfinite(y_ref).all()
        assert_probe_ok(y_cpu, y_ref, qtype, f"oracle_vs_reference_ptx {name} type={qtype}")
    eng = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    assert_probe_ok(eng.gemv(dx).cpu().numpy().ravel(), y_ref, qtype, f"engine_vs_reference_ptx batch4 type={qtype}")


@pytest.mark.parametrize("qtype", [Q4_K, Q6_K])
def test_oracle_against_reference_gemv_add(cuda, oracle, ref, qtype):
    """y = residual + W x (q4k_gemv_probe.ptx:1362, q6k_gemv_probe.ptx:398): the oracle passes the
    residual as matmul_add's bias, the accumulator start (bin/cuda_ffn_sequence_probe.cr:266)."""
    out_dim, in_dim = (4096, 4096) if qtype == Q4_K else (4096, 12288)
    w = synth.make_weight(qtype, out_dim, in_dim, seed=33, tensor_id=qtype)
    x = synth.make_activation(1, in_dim, seed=33)
    res = synth.make_activation(1, out_dim, seed=33, tensor_id=5).ravel()
    dw, dx = upload(cuda, w, x)
    dres = torch.from_numpy(res).to(cuda)
    out = torch.full((out_dim,), float("nan"), dtype=torch.float32, device=cuda)
    torch.cuda.synchronize()
    ref.gemv_add_warp4(qtype, dw.data_ptr(), dx.data_ptr(), dres.data_ptr(), out.data_ptr(), in_dim, out_dim)
    ref.synchronize()
    y_cpu = oracle.matmul_add(x, 1, in_dim, w, qtype, out_dim, res, threads=oracle.max_threads())
    assert_probe_ok(y_cpu, out.cpu().numpy(), qtype, f"oracle_vs_reference_ptx add type={qtype}")


def test_oracle_against_reference_dual_gemv(cuda, oracle, ref):
    """q4_k_dual_gemv_warp4_f32 (q4k_dual_gemv_probe.ptx:5): ssm_alpha + ssm_beta from one x, the
    shape the reference uses it on (4096 -> 32 twice) and the engine's gemv_many beside it."""
    out_dim, in_dim = 32, 4096
    wa = synth.make_weight(Q4_K, out_dim, in_dim, seed=34, tensor_id=1)
    wb = synth.make_weight(Q4_K, out_dim, in_dim, seed=34, tensor_id=2)
    x = synth.make_activation(1, in_dim, seed=34)
    dwa, dx = upload(cuda, wa, x)
    dwb = torch.from_numpy(wb).to(cuda)
    oa = torch.full((out_dim,), float("nan"), dtype=torch.float32, device=cuda)
    ob = torch.full((out_dim,), float("nan"), dtype=torch.float32, device=cuda)
    torch.cuda.synchronize()
    ref.q4k_dual_gemv(dwa.data_ptr(), dwb.data_ptr(), dx.data_ptr(), oa.data_ptr(), ob.data_ptr(), in_dim, out_dim)
    ref.synchronize()
    zero = np.zeros(out_dim, np.float32)
    assert_probe_ok(oracle.matmul_add(x, 1, in_dim, wa, Q4_K, out_dim, zero), oa.cpu().numpy(), Q4_K, "oracle_vs_reference_ptx dual a")
    assert_probe_ok(oracle.matmul_add(x, 1, in_dim, wb, Q4_K, out_dim, zero), ob.cpu().numpy(), Q4_K, "oracle_vs_reference_ptx dual b")


@pytest.mark.parametrize("out_dim,in_dim", [(4096, 1024), (32768, 2560)])
def test_oracle_against_reference_fused_top1(cuda, oracle, ref, out_dim, in_dim):
    """q6_k_gemv_top1_partial_f32 + output_top1_values_reduce_probe (q6k_gemv_probe.ptx:1331;
    src/ml/cuda/qwen_output_head_runner.cr:530-624, 940-942): the reference's fused lm_head top-1
    against the oracle's QuantMatmul + first-maximum scan, and this engine's fused top-1."""
    w = synth.make_weight(Q6_K, out_dim, in_dim, seed=35, tensor_id=Q6_K)
    x = synth.make_activation(1, in_dim, seed=35)
    dw, dx = upload(cuda, w, x)
    width = (out_dim + 3) // 4
    pid = torch.zeros(width, dtype=torch.int32, device=cuda)
    pval = torch.zeros(width, dtype=torch.float32, device=cuda)
    tid = torch.full((1,), -1, dtype=torch.int32, device=cuda)
    tval = torch.full((1,), float("nan"), dtype=torch.float32, device=cuda)
    torch.cuda.synchronize()
    ref.q6k_top1(dw.data_ptr(), dx.data_ptr(), pid.data_ptr(), pval.data_ptr(), tid.data_ptr(),
                 tval.data_ptr(), in_dim, out_dim)
    ref.synchronize()
    logits = oracle.matmul_add(x, 1, in_dim, w, Q6_K, out_dim, np.zeros(out_dim, np.float32),
                               threads=oracle.max_threads())
    idx, val = oracle.top1(logits)
    top2 = np.partition(logits, -2)[-2]
    print(f"top1 vocab={out_dim} oracle_id={idx} reference_id={int(tid)} margin={float(val - top2):.3e}")
    assert int(tid) == idx
    assert abs(float(tval) - float(val)) <= 1e-3 * max(1.0, abs(float(val)))
    eng = DeviceQuantWeight.upload(QuantWeight(w, Q6_K, out_dim, in_dim), cuda)
    eidx, _ = eng.gemv_top1(dx)
    assert int(eidx[0]) == int(tid)
