"""The state / compute helper functions that the metric modules expose, against brute-force oracles
(cf. ``torchrec/metrics/tests/test_precision.py``, ``test_recall.py``, ``test_gauc.py``, ``test_xauc.py``, ``test_rauc.py``)."""
import torch

from torchrec_b200.metrics import auprc, cali_free_ne, gauc, hindsight_target_pr, model_utils, multiclass_recall, ne, ne_positive, precision
from torchrec_b200.metrics import rauc, recall, segmented_ne, unweighted_ne, xauc


def _data(n=64, tasks=2, seed=0):
    g = torch.Generator().manual_seed(seed)
    p = torch.rand(tasks, n, generator=g, dtype=torch.double)
    l = (torch.rand(tasks, n, generator=g) < 0.4).double()
    w = torch.rand(tasks, n, generator=g, dtype=torch.double) + 0.1
    return l, p, w


def test_confusion_sums_at_a_threshold():
    l, p, w = _data()
    p[0, 0] = 0.5  # a prediction equal to the threshold is a predicted positive, and also counted by the at-or-below side
    for t in range(2):
        tp = sum(float(w[t, i]) for i in range(64) if p[t, i] >= 0.5 and l[t, i] == 1)
        fp = sum(float(w[t, i]) for i in range(64) if p[t, i] >= 0.5 and l[t, i] == 0)
        fn = sum(float(w[t, i]) for i in range(64) if p[t, i] <= 0.5 and l[t, i] == 1)
        assert abs(float(precision.compute_true_pos_sum(l, p, w)[t]) - tp) < 1e-9
        assert abs(float(precision.compute_false_pos_sum(l, p, w)[t]) - fp) < 1e-9
        assert abs(float(recall.compute_true_pos_sum(l, p, w)[t]) - tp) < 1e-9
        assert abs(float(recall.compute_false_neg_sum(l, p, w)[t]) - fn) < 1e-9
    states = precision.get_precision_states(l, p, None)
    assert torch.allclose(states["true_pos_sum"], precision.compute_true_pos_sum(l, p, torch.ones_like(p)))


def test_threshold_sweep_sums():
    l, p, w = _data(n=32, tasks=1)
    l, p, w = l[0], p[0], w[0]
    tp = hindsight_target_pr.compute_true_pos_sum(l, p, w)
    fp = hindsight_target_pr.compute_false_pos_sum(l, p, w)
    fn = hindsight_target_pr.compute_false_neg_sum(l, p, w)
    assert tp.shape == (hindsight_target_pr.THRESHOLD_GRANULARITY,)
    thr = torch.linspace(0, 1, hindsight_target_pr.THRESHOLD_GRANULARITY, dtype=torch.double)
    for i in (0, 137, 500, 999):
        assert abs(float(tp[i]) - float((w * l * (p >= thr[i])).sum())) < 1e-9
        assert abs(float(fp[i]) - float((w * (1 - l) * (p >= thr[i])).sum())) < 1e-9
        assert abs(float(fn[i]) - float((w * l * (p <= thr[i])).sum())) < 1e-9
    states = hindsight_target_pr.get_pr_states(l, p, w)
    assert torch.equal(states["true_pos_sum"], tp)


def test_ne_family_states_and_values():
    l, p, w = _data()
    eta = 1e-12
    base = ne.get_ne_states(l, p, w, eta)
    un = unweighted_ne.get_unweighted_ne_states(l, p, w, eta)
    assert torch.allclose(un["weighted_num_samples"], torch.full((2,), 64.0, dtype=torch.double))
    cf = cali_free_ne.get_cali_free_ne_states(l, p, w, eta)
    assert torch.allclose(cf["weighted_sum_predictions"], (w * p).sum(-1)) and torch.allclose(cf["cross_entropy_sum"], base["cross_entropy_sum"])
    pos = ne_positive.get_ne_positive_states(l, p, w, eta)
    value = ne_positive.compute_ne_positive(pos["cross_entropy_positive_sum"], pos["weighted_num_samples"], pos["pos_labels"], pos["neg_labels"], eta)
    mean = pos["pos_labels"] / pos["weighted_num_samples"]
    norm = -(pos["pos_labels"] * torch.log2(mean) + pos["neg_labels"] * torch.log2(1 - mean))
    assert torch.allclose(value, -(w * l * torch.log2(p)).sum(-1) / norm)
    zero = torch.zeros(2, dtype=torch.double)
    assert torch.equal(ne_positive.compute_ne_positive(zero, zero, zero, zero, eta, True), torch.full((2,), eta, dtype=torch.double))


def test_segmented_states_match_a_mask_per_group():
    l, p, w = _data()
    keys = torch.randint(0, 3, (64,), generator=torch.Generator().manual_seed(1))
    s = segmented_ne.get_segemented_ne_states(l, p, w, keys, 1e-12, 3)
    for g in range(3):
        m = keys == g
        assert torch.allclose(s["weighted_num_samples"][:, g], w[:, m].sum(-1))
        assert torch.allclose(s["pos_labels"][:, g], (w * l)[:, m].sum(-1))
        assert torch.allclose(s["cross_entropy_sum"][:, g], ne.compute_cross_entropy(l[:, m], p[:, m], w[:, m], 1e-12).sum(-1))
    value = segmented_ne.compute_ne_helper(s["cross_entropy_sum"], s["weighted_num_samples"], s["pos_labels"], s["neg_labels"], 1e-12)
    assert value.shape == (2, 3) and bool(torch.isfinite(value).all())


def test_multiclass_states():
    g = torch.Generator().manual_seed(2)
    scores = torch.rand(1, 40, 5, generator=g, dtype=torch.double)
    labels = torch.randint(0, 5, (1, 40), generator=g)
    weights = torch.rand(1, 40, generator=g, dtype=torch.double)
    s = multiclass_recall.get_multiclass_recall_states(scores, labels, weights, 5)
    top1 = (scores.argmax(-1) == labels).double()
    assert abs(float(s["tp_at_k"][0, 0]) - float((top1 * weights).sum())) < 1e-9
    assert abs(float(s["tp_at_k"][0, 4]) - float(weights.sum())) < 1e-9 and abs(float(s["total_weights"][0]) - float(weights.sum())) < 1e-9


def test_xauc_states_against_all_pairs():
    l, p, w = _data(n=24)
    l = torch.rand(2, 24, generator=torch.Generator().manual_seed(3), dtype=torch.double)
    s = xauc.get_xauc_states(l, p, w)
    for t in range(2):
        agree = total = 0.0
        for i in range(24):
            for j in range(i + 1, 24):
                total += float(w[t, i] * w[t, j])
                if (p[t, i] > p[t, j]) == (l[t, i] > l[t, j]):
                    agree += float(w[t, i] * w[t, j])
        assert abs(float(s["weighted_num_pairs"][t]) - total) < 1e-9 and abs(float(s["error_sum"][t]) - agree) < 1e-9
    assert torch.allclose(xauc.compute_xauc(s["error_sum"], s["weighted_num_pairs"]), s["error_sum"] / s["weighted_num_pairs"])
    assert float(xauc.compute_xauc(torch.zeros(1, dtype=torch.double), torch.zeros(1, dtype=torch.double))) == 0.0


def test_gauc_dense_and_jagged_forms_agree():
    gen = torch.Generator().manual_seed(4)
    lengths = torch.tensor([5, 1, 7, 3, 4])
    n = int(lengths.sum())
    p = torch.rand(2, n, generator=gen, dtype=torch.double) + 0.01
    l = (torch.rand(2, n, generator=gen) < 0.5).double()
    w = torch.rand(2, n, generator=gen, dtype=torch.double) + 0.1
    jag = gauc.get_auc_states(l, p, w, lengths)
    as3d = lambda x: gauc.to_3d(x.t().contiguous(), lengths, 7).permute(2, 0, 1)
    dense = gauc.compute_gauc_3d(as3d(p), as3d(l), as3d(w))
    assert as3d(p).shape == (2, 5, 7) and float(as3d(p)[0, 1, 1:].abs().sum()) == 0.0
    assert torch.allclose(jag["auc_sum"], dense["auc_sum"], atol=1e-8) and torch.equal(jag["num_samples"].long(), dense["num_samples"].long())
    win = gauc.compute_window_auc(jag["auc_sum"], jag["num_samples"])
    assert torch.allclose(win["gauc"], jag["auc_sum"] / jag["num_samples"], atol=1e-6)
    assert abs(float(gauc.compute_window_auc(torch.zeros(1), torch.zeros(1))["gauc"]) - 0.5) < 1e-6


def test_per_group_curves_and_inversions():
    l, p, w = _data(n=30)
    keys = torch.arange(30) % 3
    got = auprc.compute_auprc_per_group(2, p, l, w, keys)
    for t in range(2):
        want = torch.stack([auprc.compute_auprc(1, p[t:t + 1, keys == g], l[t:t + 1, keys == g], w[t:t + 1, keys == g])[0] for g in range(3)]).mean()
        assert abs(float(got[t]) - float(want)) < 1e-12
    # the leading placeholder example (key -1) is dropped
    pad = lambda x: torch.cat([torch.zeros(2, 1, dtype=x.dtype), x], dim=1)
    assert torch.allclose(auprc.compute_auprc_per_group(2, pad(p), pad(l), pad(w), torch.cat([torch.tensor([-1]), keys])), got)
    reg = torch.rand(2, 30, generator=torch.Generator().manual_seed(5), dtype=torch.double)
    got = rauc.compute_rauc_per_group(2, [p[:, :10], p[:, 10:]], [reg[:, :10], reg[:, 10:]], [w[:, :10], w[:, 10:]], keys)
    for t in range(2):
        want = torch.stack([rauc.compute_rauc(1, p[t:t + 1, keys == g], reg[t:t + 1, keys == g], w[t:t + 1, keys == g])[0] for g in range(3)]).mean()
        assert abs(float(got[t]) - float(want)) < 1e-12
    seq = [3.0, 1.0, 2.0, 5.0, 4.0]
    brute = sum(1 for i in range(5) for j in range(i + 1, 5) if seq[i] > seq[j])
    assert abs(rauc.count_reverse_pairs_divide_and_conquer(seq) - brute / 10) < 1e-12


def test_session_names_to_run_numbers():
    assert model_utils.session_ids_to_tensor(["a", "a", "b", "a", "a", "c"]).tolist() == [1, 1, 2, 3, 3, 4]
    out = model_utils.parse_required_inputs({"session": ["x", "x", "y"]}, ["session"], ndcg_transform_input=True)
    assert out["session"].tolist() == [1, 1, 2]
