"""Batched padded NMS against a sequential greedy reference."""

import torch

from axlearn_b200.vision import nms, similarity_ops


def _greedy(boxes, thr):
    keep = []
    for j in range(boxes.shape[0]):
        ok = True
        for i in keep:
            if similarity_ops.pairwise_iou(boxes_a=boxes[i][None], boxes_b=boxes[j][None]).item() > thr:
                ok = False
                break
        if ok:
            keep.append(j)
    return keep


def _random_boxes(b, n, gen):
    yx = torch.rand(b, n, 2, generator=gen) * 0.7
    hw = torch.rand(b, n, 2, generator=gen) * 0.3 + 0.02
    return torch.cat([yx, yx + hw], dim=-1)


def test_keep_mask_equals_sequential_greedy():
    gen = torch.Generator().manual_seed(0)
    boxes = _random_boxes(3, 120, gen)
    for thr in (0.1, 0.3, 0.6):
        keep = nms.nms_keep_mask(boxes, iou_threshold=thr)
        for b in range(3):
            assert keep[b].nonzero().flatten().tolist() == _greedy(boxes[b], thr)


def test_suppression_chain():
    # a suppresses b; b would have suppressed c, but b is gone, so c stays.
    boxes = torch.tensor([[[0.0, 0.0, 1.0, 1.0], [0.0, 0.3, 1.0, 1.3], [0.0, 0.6, 1.0, 1.6]]])
    assert nms.nms_keep_mask(boxes, iou_threshold=0.5).tolist() == [[True, False, True]]


def test_padded_outputs():
    gen = torch.Generator().manual_seed(1)
    boxes = _random_boxes(2, 50, gen)
    scores = torch.rand(2, 50, generator=gen).sort(dim=-1, descending=True).values
    boxes[1, 30:] = 0.0                                   # padding boxes at the tail
    scores[1, 30:] = 0.0
    out_s, out_b = nms.non_max_suppression_padded(scores, boxes, 40, 0.3)
    assert out_s.shape == (2, 40) and out_b.shape == (2, 40, 4)
    for b in range(2):
        kept = [j for j in _greedy(boxes[b], 0.3) if similarity_ops.areas(boxes[b][j]) > 0][:40]
        torch.testing.assert_close(out_s[b, :len(kept)], scores[b, kept])
        torch.testing.assert_close(out_b[b, :len(kept)], boxes[b, kept])
        assert not out_s[b, len(kept):].any() and not out_b[b, len(kept):].any()
    small_s, small_b = nms.non_max_suppression_padded(scores[:, :5], boxes[:, :5], 8, 0.3)
    assert small_s.shape == (2, 8) and small_b.shape == (2, 8, 4)


def test_multiclass():
    gen = torch.Generator().manual_seed(2)
    boxes = _random_boxes(2, 40, gen)
    scores = torch.rand(2, 40, 3, generator=gen)
    out = nms.multiclass_nms_padded(scores, boxes, max_output_size_per_class=10, max_total_size=15, iou_threshold=0.4,
                                    score_threshold=0.2)
    assert out["detection_boxes"].shape == (2, 15, 4) and out["detection_classes"].shape == (2, 15)
    for b in range(2):
        n = int(out["num_detections"][b])
        s = out["detection_scores"][b]
        assert (s[:n] > 0.2).all() and (s[n:] == 0).all() and (s[:-1] >= s[1:]).all()
        for cls in range(3):
            order = scores[b, :, cls].argsort(descending=True, stable=True)
            order = order[scores[b, order, cls] > 0.2]
            want = [order[j].item() for j in _greedy(boxes[b, order], 0.4)][:10]
            got_scores = sorted(s[:n][out["detection_classes"][b, :n] == cls].tolist(), reverse=True)
            want_scores = sorted(scores[b, want, cls].tolist(), reverse=True)
            # Whatever of this class made the global cut is a prefix of the class's kept list.
            assert got_scores == [round(x, 10) for x in want_scores[:len(got_scores)]] or \
                torch.allclose(torch.tensor(got_scores), torch.tensor(want_scores[:len(got_scores)]))
    # Per-class boxes.
    per_class = boxes[:, :, None, :].expand(2, 40, 3, 4).contiguous()
    out2 = nms.multiclass_nms_padded(scores, per_class, max_output_size_per_class=10, max_total_size=15,
                                     iou_threshold=0.4, score_threshold=0.2)
    torch.testing.assert_close(out2["detection_scores"], out["detection_scores"])
