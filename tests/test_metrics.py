"""Metrics against direct formulas on the concatenated data: lifetime vs window, fused vs unfused task modes,
fused updates, cross-rank sync on gloo, state snapshot (cf. ``torchrec/metrics/tests`` and its ``test_utils`` harness)."""
import math

import pytest
import torch

from torchrec_b200.metrics.metrics_config import DefaultTaskInfo, MetricsConfig, RecComputeMode, RecMetricDef, RecMetricEnum, RecTaskInfo, ThroughputDef
from torchrec_b200.test_utils.multi_process import MultiProcessContext, run_multi_process


def _data(n_batches=5, B=32, seed=0, n_tasks=1):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n_batches):
        p = torch.rand(n_tasks, B, generator=g)
        l = (torch.rand(n_tasks, B, generator=g) < p).float()
        w = torch.rand(n_tasks, B, generator=g)
        out.append((p, l, w))
    return out


def _ref(name, p, l, w):
    p, l, w = p.double(), l.double(), w.double()
    eta = 1e-12
    if name == "ne":
        pc = p.clamp(eta, 1 - eta)
        ce = -(w * (l * torch.log2(pc) + (1 - l) * torch.log2(1 - pc))).sum()
        pos, neg, n = (w * l).sum(), (w * (1 - l)).sum(), w.sum()
        m = (pos / n).clamp(eta, 1 - eta)
        return float(ce / (-pos * torch.log2(m) - neg * torch.log2(1 - m)))
    if name == "calibration":
        return float((w * p).sum() / (w * l).sum())
    if name == "ctr":
        return float((w * l).sum() / w.sum())
    if name == "mse":
        return float((w * (l - p) ** 2).sum() / w.sum())
    if name == "mae":
        return float((w * (l - p).abs()).sum() / w.sum())
    if name == "accuracy":
        return float((w * ((p >= 0.5) == (l >= 0.5)).double()).sum() / w.sum())
    if name == "precision":
        tp = (w * (p >= 0.5) * l).sum(); fp = (w * (p >= 0.5) * (1 - l)).sum()
        return float(tp / (tp + fp))
    if name == "recall":
        tp = (w * (p >= 0.5) * l).sum(); fn = (w * (p < 0.5) * l).sum()
        return float(tp / (tp + fn))
    if name == "weighted_avg":
        return float((w * p).sum() / w.sum())
    raise KeyError(name)


_SIMPLE = {
    "ne": ("torchrec_b200.metrics.ne", "NEMetric"), "calibration": ("torchrec_b200.metrics.calibration", "CalibrationMetric"),
    "ctr": ("torchrec_b200.metrics.ctr", "CTRMetric"), "mse": ("torchrec_b200.metrics.mse", "MSEMetric"), "mae": ("torchrec_b200.metrics.mae", "MAEMetric"),
    "accuracy": ("torchrec_b200.metrics.accuracy", "AccuracyMetric"), "precision": ("torchrec_b200.metrics.precision", "PrecisionMetric"),
    "recall": ("torchrec_b200.metrics.recall", "RecallMetric"), "weighted_avg": ("torchrec_b200.metrics.weighted_avg", "WeightedAvgMetric"),
}


def _cls(name):
    import importlib

    mod, cls = _SIMPLE[name]
    return getattr(importlib.import_module(mod), cls)


@pytest.mark.parametrize("name", sorted(_SIMPLE))
def test_lifetime_and_window_values(name):
    B, window = 32, 64  # window = last 2 batches
    m = _cls(name)(world_size=1, my_rank=0, batch_size=B, tasks=[DefaultTaskInfo], window_size=window)
    data = _data()
    for p, l, w in data:
        m.update(predictions={"DefaultTask": p[0]}, labels={"DefaultTask": l[0]}, weights={"DefaultTask": w[0]})
    res = m.compute()
    cat = lambda i, d: torch.cat([x[i][0] for x in d])
    life = _ref(name, cat(0, data), cat(1, data), cat(2, data))
    win = _ref(name, cat(0, data[-2:]), cat(1, data[-2:]), cat(2, data[-2:]))
    ns = str(m._namespace)
    assert math.isclose(float(res[f"{ns}-DefaultTask|lifetime_{name}"]), life, rel_tol=1e-9)
    assert math.isclose(float(res[f"{ns}-DefaultTask|window_{name}"]), win, rel_tol=1e-9)


@pytest.mark.parametrize("mode", [RecComputeMode.FUSED_TASKS_COMPUTATION, RecComputeMode.FUSED_TASKS_AND_STATES_COMPUTATION])
def test_fused_tasks_equal_unfused(mode):
    from torchrec_b200.metrics.ne import NEMetric

    tasks = [RecTaskInfo(name=f"t{i}", label_name=f"l{i}", prediction_name=f"p{i}", weight_name=f"w{i}") for i in range(3)]
    a = NEMetric(world_size=1, my_rank=0, batch_size=32, tasks=tasks, window_size=64)
    b = NEMetric(world_size=1, my_rank=0, batch_size=32, tasks=tasks, window_size=64, compute_mode=mode)
    for p, l, w in _data(n_tasks=3):
        d = lambda x: {t.name: x[i] for i, t in enumerate(tasks)}
        a.update(predictions=d(p), labels=d(l), weights=d(w))
        b.update(predictions=p, labels=l, weights=w)  # fused modes also take stacked tensors
    ra, rb = a.compute(), b.compute()
    assert ra.keys() == rb.keys()
    for k in ra:
        assert math.isclose(float(ra[k]), float(rb[k]), rel_tol=1e-9), k


def test_fused_update_limit_matches_plain():
    from torchrec_b200.metrics.calibration import CalibrationMetric

    a = CalibrationMetric(world_size=1, my_rank=0, batch_size=32, tasks=[DefaultTaskInfo], window_size=10_000)
    b = CalibrationMetric(world_size=1, my_rank=0, batch_size=32, tasks=[DefaultTaskInfo], window_size=10_000, fused_update_limit=3)
    for p, l, w in _data():
        for m in (a, b):
            m.update(predictions={"DefaultTask": p[0]}, labels={"DefaultTask": l[0]}, weights={"DefaultTask": w[0]})
    ra, rb = a.compute(), b.compute()
    for k in ra:
        assert math.isclose(float(ra[k]), float(rb[k]), rel_tol=1e-9)


def test_auc_family_against_sklearn():
    from sklearn.metrics import average_precision_score, roc_auc_score

    from torchrec_b200.metrics.auc import AUCMetric
    from torchrec_b200.metrics.auprc import AUPRCMetric

    data = _data(B=64)
    auc = AUCMetric(world_size=1, my_rank=0, batch_size=64, tasks=[DefaultTaskInfo], window_size=10_000)
    pr = AUPRCMetric(world_size=1, my_rank=0, batch_size=64, tasks=[DefaultTaskInfo], window_size=10_000)
    for p, l, w in data:
        p = p.round(decimals=1)  # ties
        for m in (auc, pr):
            m.update(predictions={"DefaultTask": p[0]}, labels={"DefaultTask": l[0]}, weights={"DefaultTask": w[0]})
    P = torch.cat([x[0][0].round(decimals=1) for x in data]).numpy(); L = torch.cat([x[1][0] for x in data]).numpy(); W = torch.cat([x[2][0] for x in data]).numpy()
    assert math.isclose(float(auc.compute()["auc-DefaultTask|window_auc"]), roc_auc_score(L, P, sample_weight=W), rel_tol=1e-9)
    assert math.isclose(float(pr.compute()["auprc-DefaultTask|window_auprc"]), average_precision_score(L, P, sample_weight=W), rel_tol=1e-9)


def _sync_worker(rank, world_size):
    from torchrec_b200.metrics.auc import AUCMetric
    from torchrec_b200.metrics.ne import NEMetric

    with MultiProcessContext(rank, world_size, "gloo"):
        all_data = [_data(seed=10 + r) for r in range(world_size)]
        ne = NEMetric(world_size=world_size, my_rank=rank, batch_size=32, tasks=[DefaultTaskInfo], window_size=10_000, compute_on_all_ranks=True)
        auc = AUCMetric(world_size=world_size, my_rank=rank, batch_size=32, tasks=[DefaultTaskInfo], window_size=10_000, compute_on_all_ranks=True)
        for p, l, w in all_data[rank]:
            for m in (ne, auc):
                m.update(predictions={"DefaultTask": p[0]}, labels={"DefaultTask": l[0]}, weights={"DefaultTask": w[0]})
        cat = lambda i: torch.cat([x[i][0] for d in all_data for x in d])
        assert math.isclose(float(ne.compute()["ne-DefaultTask|lifetime_ne"]), _ref("ne", cat(0), cat(1), cat(2)), rel_tol=1e-9)
        from sklearn.metrics import roc_auc_score
        assert math.isclose(float(auc.compute()["auc-DefaultTask|window_auc"]), roc_auc_score(cat(1).numpy(), cat(0).numpy(), sample_weight=cat(2).numpy()), rel_tol=1e-9)
        # local states are untouched by the global compute
        own = lambda i: torch.cat([x[i][0] for x in all_data[rank]])
        assert math.isclose(float(ne.local_compute()["ne-DefaultTask|local_lifetime_ne"]), _ref("ne", own(0), own(1), own(2)), rel_tol=1e-9)


def test_cross_rank_sync_gloo():
    run_multi_process(_sync_worker, world_size=2)


def test_metric_module_snapshot_and_throughput():
    from torchrec_b200.metrics.metric_module import RecMetricModule, generate_metric_module
    from torchrec_b200.metrics.metric_state_snapshot import MetricStateSnapshot

    cfg = MetricsConfig(rec_tasks=[DefaultTaskInfo], rec_metrics={e: RecMetricDef(rec_tasks=[DefaultTaskInfo], window_size=1000) for e in
                                                                 (RecMetricEnum.NE, RecMetricEnum.AUC, RecMetricEnum.MSE)},
                        throughput_metric=ThroughputDef(warmup_steps=1), compute_interval_steps=2)
    m = generate_metric_module(RecMetricModule, cfg, batch_size=32, world_size=1, my_rank=0, state_metrics_mapping={}, device=torch.device("cpu"))
    data = _data()
    for p, l, w in data[:3]:
        m.update({"prediction": p[0], "label": l[0], "weight": w[0]})
    assert not m.should_compute()
    snap = MetricStateSnapshot.from_metrics(m)
    before = m.compute()
    for p, l, w in data[3:]:
        m.update({"prediction": p[0], "label": l[0], "weight": w[0]})
    assert float(m.compute()["ne-DefaultTask|lifetime_ne"]) != float(before["ne-DefaultTask|lifetime_ne"])
    snap.restore(m)
    after = m.compute()
    for k in ("ne-DefaultTask|lifetime_ne", "auc-DefaultTask|window_auc", "mse-DefaultTask|lifetime_mse"):
        assert math.isclose(float(after[k]), float(before[k]), rel_tol=1e-12)
    assert int(after["throughput-throughput|total_examples"]) == 5 * 32
    sd = m.state_dict()
    m2 = generate_metric_module(RecMetricModule, cfg, batch_size=32, world_size=1, my_rank=0, state_metrics_mapping={}, device=torch.device("cpu"))
    m2.load_state_dict(sd)
    assert math.isclose(float(m2.compute()["ne-DefaultTask|lifetime_ne"]), float(after["ne-DefaultTask|lifetime_ne"]), rel_tol=1e-12)


def test_every_registered_metric_constructs_and_reports():
    """All entries of the registry build with default arguments (plus the few required ones) and report finite values."""
    from torchrec_b200.metrics.metric_module import REC_METRICS_MAPPING
    from torchrec_b200.metrics.metrics_config import SessionMetricDef

    extra = {
        RecMetricEnum.SEGMENTED_NE: {"num_groups": 2}, RecMetricEnum.MULTICLASS_RECALL: {"number_of_classes": 3},
        RecMetricEnum.TOWER_QPS: {"warmup_steps": 0},
    }
    for enum, cls in REC_METRICS_MAPPING.items():
        task = DefaultTaskInfo
        if enum in (RecMetricEnum.RECALL_SESSION_LEVEL, RecMetricEnum.PRECISION_SESSION_LEVEL):
            task = RecTaskInfo(name="DefaultTask", session_metric_def=SessionMetricDef(session_var_name="session", top_threshold=2))
        if enum == RecMetricEnum.TENSOR_WEIGHTED_AVG:
            task = RecTaskInfo(name="DefaultTask", tensor_name="x")
        m = cls(world_size=1, my_rank=0, batch_size=16, tasks=[task], window_size=64, **extra.get(enum, {}))
        g = torch.Generator().manual_seed(3)
        p = torch.rand(16, generator=g)
        l = (torch.rand(16, generator=g) < p).float()
        req = {"session": torch.arange(16) // 4, "session_id": torch.arange(16) // 4, "grouping_keys": torch.arange(16) % 2, "x": torch.rand(16, generator=g),
               "num_candidates": torch.tensor([4, 4, 4, 4])}
        if enum == RecMetricEnum.MULTICLASS_RECALL:
            p = torch.rand(16, 3, generator=g); l = torch.randint(0, 3, (16,), generator=g).float()
        m.update(predictions={"DefaultTask": p}, labels={"DefaultTask": l}, weights={"DefaultTask": torch.ones(16)}, required_inputs=req)
        res = m.compute()
        assert res, enum
        for k, v in res.items():
            assert torch.isfinite(torch.as_tensor(v, dtype=torch.double)).all() or "recall" in k or "precision" in k, (enum, k, v)
