"""Host-side lifecycle logic, no GPU: the mirror of spec/cuda_resident_sequence_runner_spec.cr."""
import numpy as np
import pytest

from cogni_ml_b200 import ResidentSequenceRunner, QuantWeight, synth


def test_runs_only_the_active_token_prefix_on_the_token_local_path():
    seen = []
    runner = ResidentSequenceRunner(4, lambda: None, lambda: None, lambda tok: seen.append(tok))
    runner.active_tokens = 2
    runner.run_sequence()
    assert seen == [0, 1]
    assert runner.run_repeated(3) == 6


def test_passes_active_token_count_to_sequence_overrides():
    seen = []
    runner = ResidentSequenceRunner(8, lambda: None, lambda: None, lambda _tok: None, None,
                                    lambda active: seen.append(active))
    runner.active_tokens = 4
    runner.run_sequence()
    assert seen == [4]


def test_rejects_invalid_active_token_counts():
    runner = ResidentSequenceRunner(4, lambda: None, lambda: None, lambda _tok: None)
    with pytest.raises(ValueError, match="active_tokens must be positive"):
        runner.active_tokens = 0
    with pytest.raises(ValueError, match="active_tokens must be <= tokens"):
        runner.active_tokens = 5
    with pytest.raises(ValueError, match="tokens must be positive"):
        ResidentSequenceRunner(0, lambda: None, lambda: None, lambda _tok: None)
    with pytest.raises(ValueError, match="reps must be positive"):
        runner.run_repeated(0)


def test_reset_active_tokens_and_optional_read_outputs():
    calls = []
    runner = ResidentSequenceRunner(3, lambda: calls.append("up"), lambda: calls.append("reset"),
                                    lambda _tok: None, lambda: calls.append("read"))
    runner.active_tokens = 1
    runner.reset_active_tokens()
    assert runner.active_tokens == 3
    runner.upload_weights()
    runner.reset_sequence()
    runner.read_outputs()
    assert calls == ["up", "reset", "read"]
    ResidentSequenceRunner(1, lambda: None, lambda: None, lambda _t: None).read_outputs()  # no-op


def test_quant_weight_checks_its_byte_count():
    raw = synth.make_weight(synth.Q4_K, 4, 512, seed=1)
    qw = QuantWeight(raw, synth.Q4_K, 4, 512)
    assert qw.raw.size == 4 * 2 * 144
    with pytest.raises(ValueError, match="bytes"):
        QuantWeight(raw[:-1], synth.Q4_K, 4, 512)
    with pytest.raises(ValueError):
        QuantWeight(raw, synth.Q4_K, 4, 500)
