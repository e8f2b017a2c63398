"""The metric test harness against two metrics, in unfused and fused modes."""
import pytest
import torch

from torchrec_b200.metrics.metrics_config import RecComputeMode
from torchrec_b200.metrics.test_utils import TestMetric, gen_test_batch, gen_test_tasks, gen_test_timestamps, rec_metric_value_test_launcher
from torchrec_b200.metrics.test_utils.mock_metrics import assert_tensor_dict_equals, create_metric_states_dict, create_tensor_list_states, create_tensor_states


class _RefMSE(TestMetric):
    @staticmethod
    def _get_states(labels, predictions, weights, required_inputs_tensor=None):
        return {"err": (weights * (labels - predictions) ** 2).sum(), "n": weights.sum()}

    @staticmethod
    def _compute(states):
        return states["err"] / states["n"]


class _RefCTR(TestMetric):
    @staticmethod
    def _get_states(labels, predictions, weights, required_inputs_tensor=None):
        return {"pos": (weights * labels).sum(), "n": weights.sum()}

    @staticmethod
    def _compute(states):
        return states["pos"] / states["n"]


@pytest.mark.parametrize("mode", [RecComputeMode.UNFUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_COMPUTATION])
def test_launcher_checks_mse_and_ctr(mode):
    from torchrec_b200.metrics.ctr import CTRMetric
    from torchrec_b200.metrics.mse import MSEMetric

    rec_metric_value_test_launcher(MSEMetric, mode, _RefMSE, "mse", ["t1", "t2"])
    rec_metric_value_test_launcher(CTRMetric, mode, _RefCTR, "ctr", ["only"], nsteps=5, batch_window_size=2)


def test_launcher_detects_a_wrong_reference():
    from torchrec_b200.metrics.mse import MSEMetric

    with pytest.raises(AssertionError):
        rec_metric_value_test_launcher(MSEMetric, RecComputeMode.UNFUSED_TASKS_COMPUTATION, _RefCTR, "mse", ["t1"])


def test_generators_and_state_helpers():
    b = gen_test_batch(8, seed=3, mask_tensor_name="mask")
    assert set(b) == {"label", "prediction", "weight", "tensor", "mask"} and b["prediction"].dtype == torch.double
    assert torch.equal(gen_test_batch(8, seed=3)["label"], b["label"])
    assert gen_test_batch(4, n_classes=5)["prediction"].shape == (4, 5)
    assert [t.label_name for t in gen_test_tasks(["a", "b"])] == ["a-label", "b-label"]
    ts = gen_test_timestamps(4)
    assert ts[0] == 0.0 and all(y > x for x, y in zip(ts, ts[1:]))
    s = create_metric_states_dict("ne", "NEMetricComputation", {**create_tensor_states(["x"], 2), **create_tensor_list_states(["y"])})
    assert_tensor_dict_equals(s, {k: v for k, v in s.items()})
    with pytest.raises(AssertionError):
        assert_tensor_dict_equals(s, {**s, "ne.NEMetricComputation.x": s["ne.NEMetricComputation.x"] + 1})
