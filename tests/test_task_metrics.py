"""Classification, correlation and retrieval metrics against scikit-learn / scipy / by hand."""

import numpy as np
import pytest
import torch

from axlearn_b200.common import metrics_classification as mc
from axlearn_b200.common import metrics_correlation as mcorr
from axlearn_b200.common import metrics_retrieval as mr

sk = pytest.importorskip("sklearn.metrics")
stats = pytest.importorskip("scipy.stats")


def test_classification_metrics_match_sklearn():
    rng = np.random.default_rng(0)
    y = rng.integers(0, 2, 200)
    score = np.round(rng.random(200) * 0.6 + y * 0.25, 2)      # ties on purpose
    pred = (score > 0.5).astype(int)
    yt, st, pt = torch.tensor(y), torch.tensor(score), torch.tensor(pred)
    out = mc.precision_recall_f_score(yt, pt, beta=2.0)
    assert out["precision"].item() == pytest.approx(sk.precision_score(y, pred), abs=1e-5)
    assert out["recall"].item() == pytest.approx(sk.recall_score(y, pred), abs=1e-5)
    assert out["f_score"].item() == pytest.approx(sk.fbeta_score(y, pred, beta=2.0), abs=1e-5)
    assert mc.binary_classification_roc_auc_score(yt, st).item() == pytest.approx(sk.roc_auc_score(y, score), abs=1e-5)
    cm = mc.confusion_matrix(yt, pt, num_classes=2)
    assert np.array_equal(cm.numpy(), sk.confusion_matrix(y, pred))
    prc = mc.precision_recall_curve(yt, st)
    p_ref, r_ref, _ = sk.precision_recall_curve(y, score)
    # sklearn lists thresholds ascending and appends (1, 0).
    np.testing.assert_allclose(prc["precisions"].numpy()[::-1], p_ref[-len(prc["precisions"]) - 1:-1], atol=1e-6)
    np.testing.assert_allclose(prc["recalls"].numpy()[::-1], r_ref[-len(prc["recalls"]) - 1:-1], atol=1e-6)
    # Masked examples do not count.
    w = torch.ones(200)
    w[:50] = 0
    assert mc.binary_classification_roc_auc_score(yt, st, weight=w).item() == pytest.approx(
        sk.roc_auc_score(y[50:], score[50:]), abs=1e-5)
    assert mc.binary_classification_roc_auc_score(torch.ones(5), torch.rand(5)).item() == 0.0
    logits = torch.tensor([2.0, -1.0, 0.0])
    assert mc.brier_score(torch.tensor([1, 0, 1]), logits).item() == pytest.approx(
        sk.brier_score_loss([1, 0, 1], torch.sigmoid(logits).numpy()), abs=1e-6)


def test_correlation_metrics():
    rng = np.random.default_rng(1)
    x = np.round(rng.normal(size=60), 1)                       # ties
    y = 0.5 * x + rng.normal(size=60) * 0.5
    xt, yt = torch.tensor(x), torch.tensor(y)
    assert mcorr.pearson_corrcoef(xt, yt).item() == pytest.approx(stats.pearsonr(x, y)[0], abs=1e-5)
    assert mcorr.spearman_corrcoef(xt, yt).item() == pytest.approx(stats.spearmanr(x, y)[0], abs=1e-5)
    mask = torch.ones(60)
    mask[40:] = 0
    assert mcorr.spearman_corrcoef(xt, yt, mask=mask).item() == pytest.approx(stats.spearmanr(x[:40], y[:40])[0], abs=1e-5)
    a, b = rng.integers(0, 2, 100), rng.integers(0, 2, 100)
    assert mcorr.matthews_corrcoef(torch.tensor(a), torch.tensor(b)).item() == pytest.approx(
        sk.matthews_corrcoef(b, a), abs=1e-5)


def test_retrieval_metrics_by_hand():
    sim = torch.tensor([[0.9, 0.1, 0.5, 0.3],      # ranking: 0, 2, 3, 1
                        [0.2, 0.8, 0.4, 0.6]])     # ranking: 1, 3, 2, 0
    rel = torch.tensor([[0, 0, 1, 1], [1, 0, 0, 0]])
    acc = mr.top_k_accuracy(sim, relevance_labels=rel, top_ks=(1, 2, 4))
    assert [a.item() for a in acc] == [0.0, 0.5, 1.0]
    assert mr.top_k_accuracy(sim, gt_targets=torch.tensor([0, 3]), top_ks=(1,))[0].item() == 0.5
    rec = mr.top_k_recall(sim, relevance_labels=rel, top_ks=(2, 3))
    assert [r.item() for r in rec] == [0.25, 0.5]
    assert mr.mean_reciprocal_rank(sim, relevance_labels=rel).item() == pytest.approx((1 / 2 + 1 / 4) / 2)
    assert mr.average_rank(sim, relevance_labels=rel).item() == pytest.approx((2 + 3 + 4) / 3)
    ap = mr.average_precision_at_k(sim, relevance_labels=rel, top_ks=(3,))[3]
    assert ap[0].item() == pytest.approx((1 / 2 + 2 / 3) / 2) and ap[1].item() == 0.0
    ndcg = mr.ndcg_at_k(sim, relevance_labels=rel, top_ks=(4,))[4]
    ref = np.mean([sk.ndcg_score(rel[i:i + 1].numpy(), sim[i:i + 1].numpy(), k=4) for i in range(2)])
    assert ndcg.item() == pytest.approx(ref, abs=1e-5)
    # Padding: the second query is dropped, item 0 of the first is hidden.
    qp = torch.tensor([False, True])
    ip = torch.tensor([[True, False, False, False], [False] * 4])
    assert mr.top_k_accuracy(sim, relevance_labels=rel, top_ks=(1,), query_padding=qp, item_paddings=ip)[0].item() == 1.0
    assert mr.metric_at_k_name("recall", 5) == "recall@5"
