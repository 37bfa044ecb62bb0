"""Multi-stream models, text dual encoders, SPLADE pooling, DPR configs and their metrics."""
import math

import torch

from axlearn_b200.common import neural_retrieval as nr
from axlearn_b200.common import prng, schedule
from axlearn_b200.common import text_dual_encoder as tde
from axlearn_b200.common.config import config_for_function
from axlearn_b200.common.loss import flops_loss, ranking_pairwise_loss
from axlearn_b200.common.metrics_text_dual_encoder import (
    calculate_retrieval_metrics_from_embeddings,
    calculate_retrieval_metrics_from_similarity_matrix,
)
from axlearn_b200.common.module import functional
from axlearn_b200.common.layers import Linear
from axlearn_b200.common.splade import SpladePooling
from axlearn_b200.common.utils import flatten_items


def _tower(dim=16):
    return nr.set_bert_dpr_encoder_config(vocab_size=50, num_layers=1, model_dim=dim, num_heads=2, max_seq_len=12)


def _batch(b=4, negs=2, t=8):
    g = torch.Generator().manual_seed(0)
    ids = lambda n: torch.randint(1, 50, (b, n, t), generator=g)
    return {
        nr.QUERY_ENCODER_NAME: {tde.POSITIVE_INPUT_IDS: ids(1), tde.POSITIVE_PADDINGS: torch.zeros(b, 1)},
        nr.PASSAGE_ENCODER_NAME: {tde.POSITIVE_INPUT_IDS: ids(1), tde.POSITIVE_PADDINGS: torch.zeros(b, 1),
                                  tde.NEGATIVE_INPUT_IDS: ids(negs),
                                  tde.NEGATIVE_PADDINGS: torch.tensor([[0, 1]] * b, dtype=torch.float32)},
    }


def test_dpr_two_towers_loss_is_in_batch_cross_entropy_over_live_keys():
    cfg = nr.set_dpr_model_config(query_encoder_cfg=_tower(), passage_encoder_cfg=_tower(),
                                  contrastive_loss_scale_factor=2.0)
    model = cfg.set(name="dpr").instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert set(params) == {nr.QUERY_ENCODER_NAME, nr.PASSAGE_ENCODER_NAME, "contrastive_fusion_network"} or \
        set(params) == {nr.QUERY_ENCODER_NAME, nr.PASSAGE_ENCODER_NAME}
    batch = _batch()
    (loss, _), col = functional(model, prng.PRNGKey(1), params, [batch], is_training=False,
                                drop_output_collections=())
    pred, _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=False, method="predict")
    q = pred[nr.QUERY_ENCODER_NAME][tde.POSITIVE_EMBEDDINGS]
    p = pred[nr.PASSAGE_ENCODER_NAME]
    assert q.shape == (4, 1, 16) and p[tde.NEGATIVE_EMBEDDINGS].shape == (4, 2, 16)
    keys = torch.cat([p[tde.POSITIVE_EMBEDDINGS].reshape(4, 16), p[tde.NEGATIVE_EMBEDDINGS].reshape(8, 16)])
    logits = (q.reshape(4, 16) @ keys.t()) * 2.0
    logits[:, 4:][:, 1::2] = -1e9                                   # padded negatives
    expected = torch.nn.functional.cross_entropy(logits, torch.arange(4))
    torch.testing.assert_close(loss, expected, rtol=1e-4, atol=1e-5)
    assert any(k.endswith("loss_contrastive_fusion_network") for k, _ in flatten_items(col.summaries))


def test_siamese_dpr_has_one_set_of_tower_weights():
    cfg = nr.set_siamese_dpr_model_config(shared_encoder_cfg=_tower())
    model = cfg.set(name="dpr").instantiate(parent=None)
    params = model.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert not params.get(nr.PASSAGE_ENCODER_NAME)
    batch = _batch()
    batch[nr.PASSAGE_ENCODER_NAME][tde.POSITIVE_INPUT_IDS] = batch[nr.QUERY_ENCODER_NAME][tde.POSITIVE_INPUT_IDS]
    pred, _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=False, method="predict")
    torch.testing.assert_close(pred[nr.QUERY_ENCODER_NAME][tde.POSITIVE_EMBEDDINGS],
                               pred[nr.PASSAGE_ENCODER_NAME][tde.POSITIVE_EMBEDDINGS])
    (loss, _), _ = functional(model, prng.PRNGKey(1), params, [batch], is_training=False)
    assert torch.isfinite(loss)


def test_ranking_pairwise_loss_counts_only_graded_pairs():
    logits = torch.tensor([[2.0, 1.0, 0.0, 5.0]])
    ranks = torch.tensor([[1, 2, 3, 0]])                            # last doc is ungraded
    loss, pairs = ranking_pairwise_loss(logits=logits, ranks=ranks, loss_scale=torch.ones(1))
    assert pairs == 3
    want = (2 * math.log1p(math.exp(-1.0)) + math.log1p(math.exp(-2.0))) / 3
    torch.testing.assert_close(loss, torch.tensor(want), rtol=1e-5, atol=1e-6)
    layer = tde.RankingPairwiseLossLayer.default_config().set(
        name="r", left_encoder_name="q", right_encoder_name="d").instantiate(parent=None)
    batch = {"q": {tde.POSITIVE_EMBEDDINGS: torch.tensor([[[1.0, 0.0]]])},
             "d": {tde.PAIRWISE_LOSS_EMBEDDINGS: torch.tensor([[[2.0, 0], [1.0, 0], [0.0, 0], [5.0, 0]]]),
                   tde.PAIRWISE_LOSS_PADDINGS: torch.tensor([[0, 0, 0, 1]]), tde.RANKS: torch.tensor([[1, 2, 3, 4]])}}
    (l2, aux), _ = functional(layer, None, {}, [batch], is_training=False)
    torch.testing.assert_close(l2, loss)
    assert aux[tde.NUM_VALID_RANKING_PAIRS] == 3


def test_flops_loss_layer_follows_its_schedule_and_advances_the_step():
    emb = torch.tensor([[1.0, 0.0, -2.0], [3.0, 0.0, 0.0]])
    loss, count = flops_loss(embeddings=emb)
    torch.testing.assert_close(loss, torch.tensor(2.0 ** 2 + 1.0 ** 2))
    torch.testing.assert_close(count, torch.tensor(1.5))
    loss_p, count_p = flops_loss(embeddings=emb, paddings=torch.tensor([0.0, 1.0]))
    torch.testing.assert_close(loss_p, torch.tensor(5.0))
    torch.testing.assert_close(count_p, torch.tensor(1.0))
    cfg = tde.FLOPsLossLayer.default_config().set(
        name="f", left_encoder_name="q", right_encoder_name="d",
        flops_weight_schedule=config_for_function(schedule.polynomial).set(begin_step=0, begin_value=0.0, end_step=10, end_value=1.0))
    layer = cfg.instantiate(parent=None)
    params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
    assert params["step"].dtype == torch.int32
    batch = {"q": {tde.POSITIVE_EMBEDDINGS: emb[:, None]},
             "d": {tde.POSITIVE_EMBEDDINGS: emb[:, None], tde.POSITIVE_PADDINGS: torch.zeros(2, 1)}}
    params["step"] = torch.tensor(5, dtype=torch.int32)
    (l, _), col = functional(layer, None, params, [batch], is_training=True, drop_output_collections=())
    torch.testing.assert_close(l, torch.tensor(0.5 * 2 * 5.0))
    assert int(col.state_updates["step"]) == 6


def test_splade_pooling_max_and_sum_modes():
    x = torch.randn(2, 5, 8)
    pad = torch.tensor([[0, 0, 0, 1, 1], [0, 0, 0, 0, 0]]).bool()
    for mode in ("max", "sum"):
        cfg = SpladePooling.default_config().set(name="s", input_dim=8, output_dim=20, splade_mode=mode)
        cfg.vocab_mapping.inner_head = Linear.default_config().set(bias=False)
        layer = cfg.instantiate(parent=None)
        params = layer.initialize_parameters_recursively(prng.PRNGKey(0), device="cpu")
        y, _ = functional(layer, None, params, dict(tokens=x, paddings=pad), is_training=False)
        assert y.shape == (2, 1, 20) and (y >= 0).all()
        x2 = x.clone()
        x2[0, 3:] = 100.0                                          # padded positions do not matter
        y2, _ = functional(layer, None, params, dict(tokens=x2, paddings=pad), is_training=False)
        torch.testing.assert_close(y, y2)


def test_retrieval_metrics_from_embeddings():
    q = torch.eye(4)[:, None, :]                                    # query i matches key i
    pos = torch.eye(4)[:, None, :].clone()
    pos[3, 0] = torch.tensor([1.0, 0, 0, 0.5])                      # query 3's positive ranks below key 0's... for q3: own=0.5, key0=0
    neg = torch.zeros(4, 1, 4)
    neg[2, 0] = torch.tensor([0, 0, 2.0, 0])                        # a hard negative for query 2 (score 2 > 1)
    m = calculate_retrieval_metrics_from_embeddings(
        top_ks_for_accuracy=[1, 2], query_embeddings=q, query_paddings=torch.zeros(4, 1),
        text_positive_embeddings=pos, text_positive_paddings=torch.zeros(4, 1),
        text_negative_embeddings=neg, text_negative_paddings=torch.zeros(4, 1), top_ks_for_ndcg=[1, 2])
    torch.testing.assert_close(m["retrieval_accuracy@1"], torch.tensor(0.75))
    torch.testing.assert_close(m["retrieval_accuracy@2"], torch.tensor(1.0))
    torch.testing.assert_close(m["avg_rank"], torch.tensor((1 + 1 + 2 + 1) / 4))
    torch.testing.assert_close(m["ndcg@1"], torch.tensor(0.75))
    torch.testing.assert_close(m["ndcg@2"], torch.tensor((3 + 1 / math.log2(3)) / 4))
    # Masking the hard negative and padding query 3 restores a perfect score over 3 queries.
    m2 = calculate_retrieval_metrics_from_embeddings(
        top_ks_for_accuracy=[1], query_embeddings=q, query_paddings=torch.tensor([[0.0], [0], [0], [1]]),
        text_positive_embeddings=pos, text_positive_paddings=torch.zeros(4, 1),
        text_negative_embeddings=neg, text_negative_paddings=torch.tensor([[0.0], [0], [1], [0]]))
    torch.testing.assert_close(m2["retrieval_accuracy@1"], torch.tensor(1.0))
    sim = torch.tensor([[0.9, 0.1], [0.8, 0.2]])
    m3 = calculate_retrieval_metrics_from_similarity_matrix(
        sim=sim, text_positive_paddings=torch.zeros(2, 1), query_paddings=torch.zeros(2, 1),
        text_paddings=torch.zeros(2), top_ks_for_accuracy=[1])
    torch.testing.assert_close(m3["retrieval_accuracy@1"], torch.tensor(0.5))
