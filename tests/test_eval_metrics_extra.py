"""GLUE metrics, precision / recall levels, CLIP and embedding retrieval evaluation."""
import pytest
import torch

from axlearn_b200.common.eval_classification import precision_at_recall, recall_at_precision
from axlearn_b200.common.eval_retrieval import (
    EmbeddingRetrievalMetricCalculator,
    KnnMetricCalculator,
    calculate_clip_retrieval_metrics,
)
from axlearn_b200.common.evaler import PredictionOutputs
from axlearn_b200.common.metrics_glue import glue_metrics


def test_glue_metrics_against_scipy_and_sklearn():
    sk = pytest.importorskip("sklearn.metrics")
    stats = pytest.importorskip("scipy.stats")
    g = torch.Generator().manual_seed(0)
    y = torch.randint(0, 2, (50,), generator=g)
    p = torch.where(torch.rand(50, generator=g) < 0.7, y, 1 - y)
    mask = torch.rand(50, generator=g) < 0.8
    m = glue_metrics(task="cola", target_labels=y, preds=p, mask=mask)
    assert float(m["accuracy"].mean) == pytest.approx(sk.accuracy_score(y[mask], p[mask]))
    assert float(m["matthews_corr"].mean) == pytest.approx(sk.matthews_corrcoef(y[mask], p[mask]), abs=1e-5)
    p_bad = p.clone()
    p_bad[0] = 7                                                      # out of range = wrong
    wrong = p.clone()
    wrong[0] = 1 - y[0]
    mask[0] = True
    m = glue_metrics(task="mrpc", target_labels=y, preds=p_bad, mask=mask)
    assert float(m["f1"].mean) == pytest.approx(sk.f1_score(y[mask], wrong[mask]), abs=1e-5)
    a, b = torch.randn(40, generator=g), torch.randn(40, generator=g)
    m = glue_metrics(task="stsb", target_labels=a, preds=a + 0.5 * b, mask=torch.ones(40))
    assert float(m["pearson_corr"].mean) == pytest.approx(stats.pearsonr(a, a + 0.5 * b)[0], abs=1e-5)
    assert float(m["spearman_corr"].mean) == pytest.approx(stats.spearmanr(a, a + 0.5 * b)[0], abs=1e-5)
    assert "accuracy" not in m


def test_precision_recall_levels():
    y = torch.tensor([1, 1, 0, 1, 0, 0])
    s = torch.tensor([0.9, 0.8, 0.7, 0.6, 0.2, 0.1])
    assert float(precision_at_recall(y, s, 0.6)) == pytest.approx(1.0)     # top two are positive
    assert float(precision_at_recall(y, s, 1.0)) == pytest.approx(0.75)
    assert float(recall_at_precision(y, s, 0.99)) == pytest.approx(2 / 3)


def test_clip_retrieval_metrics():
    img = torch.eye(3)
    txt = torch.stack([torch.eye(3), 0.5 * torch.eye(3).roll(1, 0)], dim=1)       # second caption of each image is wrong
    m = calculate_clip_retrieval_metrics(image_embeddings=img, text_embeddings=txt,
                                         text_paddings=torch.zeros(3, 2, dtype=torch.bool), top_ks=(1,))
    assert float(m["text_to_image@1"]) == pytest.approx(0.5) and float(m["image_to_text@1"]) == pytest.approx(1.0)
    m = calculate_clip_retrieval_metrics(image_embeddings=img, text_embeddings=txt,
                                         text_paddings=torch.tensor([[False, True]] * 3), top_ks=(1,))
    assert float(m["text_to_image@1"]) == pytest.approx(1.0)


def test_embedding_retrieval_and_knn():
    emb = torch.tensor([[1.0, 0], [0.9, 0.1], [0, 1.0], [0.1, 0.9], [1.0, 0.05]])
    labels = torch.tensor([0, 0, 1, 1, 1])                                   # the last one sits in the wrong cluster
    outs = [PredictionOutputs({"label": labels[:3]}, {"embedding": emb[:3]}),
            PredictionOutputs({"label": labels[3:]}, {"embedding": emb[3:]})]
    calc = EmbeddingRetrievalMetricCalculator.default_config().set(name="r", top_ks=(1,), query_chunk_size=2).instantiate(
        parent=None, model=None, model_param_partition_specs=None)
    s = calc.get_summaries(model_params=None, state=None, all_forward_outputs=outs)
    assert float(s["accuracy@1"].mean) == pytest.approx(2 / 5)      # the stray point also misleads its two neighbours
    knn = KnnMetricCalculator.default_config().set(name="k", top_ks=(1, 3)).instantiate(
        parent=None, model=None, model_param_partition_specs=None)
    s = knn.get_summaries(model_params=None, state=None, all_forward_outputs=outs)
    assert float(s["knn_accuracy@1"].mean) == pytest.approx(2 / 5)
