import numpy as np
import torch

from idrak_b200.vision import detection as D


def test_boxes_and_nms():
    a = torch.tensor([[0.0, 0, 10, 10], [5, 5, 15, 15], [20, 20, 30, 30]])
    iou = D.box_iou(a, a)
    assert torch.allclose(iou.diag(), torch.ones(3)) and abs(iou[0, 1].item() - 25 / 175) < 1e-6 and iou[0, 2] == 0
    assert torch.equal(D.xywh_to_xyxy(torch.tensor([[1.0, 2, 3, 4]])), torch.tensor([[1.0, 2, 4, 6]]))
    assert torch.equal(D.cxcywh_to_xyxy(torch.tensor([[5.0, 5, 4, 2]])), torch.tensor([[3.0, 4, 7, 6]]))
    boxes = torch.tensor([[0.0, 0, 10, 10], [1, 1, 11, 11], [0, 0, 9, 9], [50, 50, 60, 60]])
    scores = torch.tensor([0.9, 0.8, 0.95, 0.5])
    assert D.nms(boxes, scores, 0.5).tolist() == [2, 3]
    assert D.nms(boxes, scores, 0.5, classes=torch.tensor([0, 1, 0, 0])).tolist() == [2, 1, 3]
    assert D.nms(boxes, scores, 0.5, top_k=1).tolist() == [2]
    assert D.nms(boxes[:0], scores[:0]).numel() == 0
    try:
        import torchvision
        big = torch.rand(200, 4) * 50
        big[:, 2:] += big[:, :2]
        sc = torch.rand(200)
        assert D.nms(big, sc, 0.4).tolist() == torchvision.ops.nms(big, sc, 0.4).tolist()
    except ImportError:
        pass


def test_augmentations_carry_boxes():
    img = torch.arange(20 * 30 * 3, dtype=torch.float32).reshape(20, 30, 3)
    boxes = torch.tensor([[2.0, 3, 10, 12], [20, 5, 29, 15]])
    f, fb = D.flip_horizontal(img, boxes)
    assert torch.equal(f[:, 0], img[:, -1]) and fb.tolist() == [[20.0, 3, 28, 12], [1, 5, 10, 15]]
    c, cb, keep = D.crop(img, boxes, (0, 0, 15, 15))
    assert c.shape == (15, 15, 3) and keep.tolist() == [0] and cb.tolist() == [[2.0, 3, 10, 12]]
    c, cb, keep = D.crop(img, boxes, (5, 0, 25, 20), min_visible=0.5)
    assert keep.tolist() == [0, 1] and cb.tolist() == [[0.0, 3, 5, 12], [15, 5, 20, 15]]
    rng = np.random.default_rng(0)
    c, cb, keep = D.random_crop(img, boxes, rng)
    assert c.shape[0] <= 20 and (cb[:, 2] <= c.shape[1]).all()
    assert D.resize_boxes(boxes, (20, 30), (40, 15))[0].tolist() == [1.0, 6, 5, 24]
    j = D.color_jitter(torch.full((4, 4, 3), 100, dtype=torch.uint8), rng)
    assert j.dtype == torch.uint8 and j.shape == (4, 4, 3)


def test_average_precision_by_hand():
    gt = [D.GroundTruth(torch.tensor([[0.0, 0, 10, 10], [20, 20, 30, 30]]), torch.tensor([1, 1])),
          D.GroundTruth(torch.tensor([[5.0, 5, 15, 15]]), torch.tensor([1]))]
    det = [D.Detections(torch.tensor([[0.0, 0, 10, 10], [40, 40, 50, 50], [20, 20, 30, 29]]), torch.tensor([0.9, 0.8, 0.7]), torch.tensor([1, 1, 1])),
           D.Detections(torch.tensor([[5.0, 5, 15, 15]]), torch.tensor([0.6]), torch.tensor([1]))]
    # ranked: TP(.9) FP(.8) TP(.7) TP(.6) over 3 truths -> precision at recalls 1/3, 2/3, 1 = 1, 2/3, 3/4
    ap_all = D.average_precision(det, gt, 1, 0.5, style="voc")
    assert abs(ap_all - (1 / 3 * 1 + 1 / 3 * 0.75 + 1 / 3 * 0.75)) < 1e-9
    ap_coco = D.average_precision(det, gt, 1, 0.5, style="coco")
    assert abs(ap_coco - (34 * 1.0 + 67 * 0.75) / 101) < 1e-9
    assert D.average_precision(det, gt, 7, 0.5) is None
    # a second detection of the same object is a false positive; a match to a crowd region is ignored
    dup = [D.Detections(torch.tensor([[0.0, 0, 10, 10], [0, 0, 10, 9]]), torch.tensor([0.9, 0.8]), torch.tensor([1, 1]))]
    one = [D.GroundTruth(torch.tensor([[0.0, 0, 10, 10]]), torch.tensor([1]))]
    assert abs(D.average_precision(dup, one, 1, 0.5, "voc") - 1.0) < 1e-9          # recall 1 reached at precision 1
    crowd = [D.GroundTruth(torch.tensor([[0.0, 0, 10, 10], [50, 50, 90, 90]]), torch.tensor([1, 1]), torch.tensor([False, True]))]
    det2 = [D.Detections(torch.tensor([[52.0, 52, 88, 88], [0, 0, 10, 10]]), torch.tensor([0.95, 0.9]), torch.tensor([1, 1]))]
    assert abs(D.average_precision(det2, crowd, 1, 0.5, "voc") - 1.0) < 1e-9
    summary = D.mean_average_precision(det, gt)
    assert 0 < summary["map"] < summary["map50"] and abs(summary["map50"] - ap_coco) < 1e-9 and "ap_class_1" in summary
