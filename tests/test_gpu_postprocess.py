"""GPU parity: anchor decode and score filter entry points against the oracle.

Indices, counts and the direction class are exact; floating-point columns within 1e-5 relative (the GPU's
expf and the host's differ in the last place; everything else is computed in the same order).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _head_outputs(gpu, seed, frames, height, width, dirs, logit_mean=-4.0):
    """Seeded stand-ins for the 2D head's four outputs, [frames, N, *]."""
    rs = np.random.RandomState(seed)
    n = height * width * dirs
    box = (rs.randn(frames, n, 7) * 0.3).astype(np.float32)
    cls = (logit_mean + 1.5 * rs.randn(frames, n, 1)).astype(np.float32)
    iou = rs.uniform(-1, 1, (frames, n, 1)).astype(np.float32)
    dr = rs.randn(frames, n, 2).astype(np.float32)
    dr[:, ::7, 1] = dr[:, ::7, 0]          # ties: the later direction must win
    # keep every score clear of the threshold so that a last-place difference of expf cannot flip a decision
    thr = gpu.schedule.SCORE_THRESHOLD
    score = 1.0 / (1.0 + np.exp(-cls.astype(np.float64)))
    cls[np.abs(score - thr) < 1e-4] = -10.0
    return box, cls, iou, dr


def _close(got, want):
    np.testing.assert_allclose(got, want, rtol=TOL, atol=1e-6)


def _to_gpu(*arrays):
    import torch

    return [torch.from_numpy(a).cuda() for a in arrays]


def test_anchor_decode_full_size(gpu, oracle):
    S = gpu.schedule
    box, _, _, _ = _head_outputs(gpu, 1, 2, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, 2)
    ap = gpu.anchor_params()
    got = gpu.anchor_decode(_to_gpu(box)[0], ap).cpu().numpy()
    oparams = oracle.anchor_params(gpu.synth.POINT_RANGE, S.CAR_SIZE, S.DIRECTION_ANGLES)
    for b in range(2):
        want = oracle.anchor_decode(box[b], oparams, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, 2)
        _close(got[b], want)
        # columns without exp are computed in the same order: identical
        np.testing.assert_array_equal(got[b][:, [0, 1, 2, 6]], want[:, [0, 1, 2, 6]])


def _check_filter(gpu, oracle, frames, height, width, max_box, logit_mean, fused, seed):
    S = gpu.schedule
    box, cls, iou, dr = _head_outputs(gpu, seed, frames, height, width, 2, logit_mean)
    ap = gpu.anchor_params(height=height, width=width)
    fp = gpu.filter_params(height=height, width=width, max_box_num=max_box)
    oparams = oracle.anchor_params(gpu.synth.POINT_RANGE, S.CAR_SIZE, S.DIRECTION_ANGLES)
    decoded = np.stack([oracle.anchor_decode(box[b], oparams, height, width, 2) for b in range(frames)])
    tb, tc, ti, td = _to_gpu(box if fused else decoded, cls, iou, dr)
    r = gpu.filter_boxes(tb, tc, ti, td, fp, anchors=ap if fused else None)
    overflow = False
    for b in range(frames):
        ob, oc, oi, od, valid, passed = oracle.filter_boxes(decoded[b], cls[b], iou[b], dr[b], 2, max_box,
                                                            S.SCORE_THRESHOLD, S.DIRECTION_OFFSET)
        overflow |= passed > max_box
        assert int(r["valid"][b]) == valid
        np.testing.assert_array_equal(r["direction"][b].cpu().numpy(), od)
        _close(r["box"][b].cpu().numpy(), ob)
        _close(r["score"][b].cpu().numpy(), oc)
        _close(r["iou"][b].cpu().numpy(), oi)
        assert not r["box"][b, valid:].any() and not r["score"][b, valid:].any()
    assert bool(r["status"] & gpu.STATUS_BOX_OVERFLOW) == overflow
    return overflow


@pytest.mark.parametrize("fused", [False, True])
def test_filter_full_size(gpu, oracle, fused):
    S = gpu.schedule
    assert not _check_filter(gpu, oracle, 3, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, S.MAX_BOX_NUM, -4.0, fused, 2)


@pytest.mark.parametrize("fused", [False, True])
def test_filter_clamps_at_max_box_and_reports(gpu, oracle, fused):
    assert _check_filter(gpu, oracle, 2, 40, 36, 50, -1.0, fused, 3)


def test_filter_nothing_passes_and_ragged_last_chunk(gpu, oracle):
    # 7 x 9 x 2 = 126 anchors: less than one chunk; all scores far below the threshold
    assert not _check_filter(gpu, oracle, 1, 7, 9, 10, -30.0, True, 4)
    # 13 x 21 x 2 = 546 anchors: two full chunks and a ragged one
    _check_filter(gpu, oracle, 2, 13, 21, 500, 0.0, False, 5)


def test_filter_rejects_bad_arguments(gpu):
    import torch

    fp = gpu.filter_params(max_box_num=0)
    x = torch.zeros((1, 70400, 7), device="cuda")
    with pytest.raises(gpu.SessdError):
        gpu.filter_boxes(x, x, x, x, fp)
    with pytest.raises(gpu.SessdError):   # the two parameter blocks disagree on the feature map
        gpu.filter_boxes(x, x, x, x, gpu.filter_params(), anchors=gpu.anchor_params(height=100))


# ---- rotated NMS ---------------------------------------------------------------------------------------

def _random_boxes(rs, n, spread):
    """Car-sized boxes scattered over `spread` metres, with clusters so that suppression happens."""
    centres = rs.uniform(0, spread, (max(n // 4, 1), 2))
    pick = rs.randint(0, len(centres), n)
    b = np.zeros((n, 9), np.float32)
    b[:, 0:2] = centres[pick] + rs.randn(n, 2) * 0.6
    b[:, 2] = rs.uniform(-1.5, -0.5, n)
    b[:, 3] = rs.uniform(1.4, 1.9, n)
    b[:, 4] = rs.uniform(3.4, 4.5, n)
    b[:, 5] = rs.uniform(1.4, 1.7, n)
    b[:, 6] = rs.uniform(-3.2, 3.2, n)
    b[:, 8] = np.round(rs.uniform(0.05, 1.0, n), 2)      # two decimals: plenty of equal scores
    return b


def _clear_of_threshold(oracle, boxes, thresh, eps=1e-4):
    """True when no pair's IoU lies within eps of the threshold (then a last-place difference of the
    device's trigonometric functions cannot flip a decision)."""
    n = len(boxes)
    for i in range(n):
        for j in range(i + 1, n):
            if abs(boxes[i, 0] - boxes[j, 0]) + abs(boxes[i, 1] - boxes[j, 1]) < 12:
                if abs(oracle.bev_iou(boxes[i], boxes[j]) - thresh) < eps:
                    return False
    return True


@pytest.mark.parametrize("thresh", [0.01, 0.3])
def test_rotated_nms_matches_oracle(gpu, oracle, thresh):
    import torch

    rs = np.random.RandomState(31)
    M = 500
    counts = [500, 137, 0, 64]
    boxes = np.zeros((len(counts), M, 9), np.float32)
    for b, n in enumerate(counts):
        for attempt in range(20):
            cand = _random_boxes(rs, n, 60.0)
            if _clear_of_threshold(oracle, cand, thresh):
                break
        else:
            pytest.fail("could not draw boxes clear of the threshold")
        boxes[b, :n] = cand
        boxes[b, n:] = 7.0    # rows past the count must be ignored
    valid = np.array(counts, np.int32)
    kept, kept_num = gpu.rotated_nms(torch.from_numpy(boxes).cuda(), torch.from_numpy(valid).cuda(), thresh)
    kept, kept_num = kept.cpu().numpy(), kept_num.cpu().numpy()
    for b, n in enumerate(counts):
        want, order = oracle.rotated_nms(boxes[b, :n], thresh)
        assert int(kept_num[b]) == len(want)
        np.testing.assert_array_equal(kept[b, :len(want)], want)     # same boxes, same order, copied bit for bit
        assert not kept[b, len(want):].any()
        if n > 100:
            assert 0 < len(want) < n                                    # the case does suppress something


def test_rotated_nms_with_non_finite_scores(gpu, oracle):
    """A NaN or infinite score (a non-finite fp16 head output makes one) must not break the ranking: NaN ranks as
    minus infinity, +inf first, every box still gets a rank of its own and the kept list equals the oracle's."""
    import torch

    rs = np.random.RandomState(77)
    n, M = 200, 256
    for attempt in range(20):
        cand = _random_boxes(rs, n, 60.0)
        if _clear_of_threshold(oracle, cand, 0.1):
            break
    else:
        pytest.fail("could not draw boxes clear of the threshold")
    cand[[3, 50, 51, 120], 8] = np.nan
    cand[[7, 90], 8] = np.inf
    cand[[11, 140], 8] = -np.inf
    boxes = np.zeros((1, M, 9), np.float32)
    boxes[0, :n] = cand
    kept, kept_num = gpu.rotated_nms(torch.from_numpy(boxes).cuda(), torch.tensor([n], dtype=torch.int32, device="cuda"), 0.1)
    kept, kept_num = kept.cpu().numpy(), kept_num.cpu().numpy()
    want, order = oracle.rotated_nms(cand, 0.1)
    assert int(kept_num[0]) == len(want)
    np.testing.assert_array_equal(kept[0, :len(want)].view(np.uint32), want.view(np.uint32))   # bit patterns: NaN == NaN
    assert not kept[0, len(want):].any()
    assert order[0] == 7 and order[1] == 90    # +inf first, lower row first among equals


def test_rotated_nms_table_larger_than_the_staged_copy(gpu, oracle):
    """A 1,200-row box table: its suppression mask (1,200 x 19 words) does not fit the block's staging buffer,
    so the greedy pass reads the mask in place; same answer as the oracle."""
    import torch

    rs = np.random.RandomState(77)
    M, counts = 1200, [700, 1200]
    boxes = np.zeros((len(counts), M, 9), np.float32)
    for b, n in enumerate(counts):
        for attempt in range(20):
            cand = _random_boxes(rs, n, 150.0)
            if _clear_of_threshold(oracle, cand, 0.1):
                break
        else:
            pytest.fail("could not draw boxes clear of the threshold")
        boxes[b, :n] = cand
    valid = np.array(counts, np.int32)
    kept, kept_num = gpu.rotated_nms(torch.from_numpy(boxes).cuda(), torch.from_numpy(valid).cuda(), 0.1)
    kept, kept_num = kept.cpu().numpy(), kept_num.cpu().numpy()
    for b, n in enumerate(counts):
        want, _ = oracle.rotated_nms(boxes[b, :n], 0.1)
        assert int(kept_num[b]) == len(want) and 0 < len(want) < n
        np.testing.assert_array_equal(kept[b, :len(want)], want)
        assert not kept[b, len(want):].any()


def test_rotated_nms_after_score_filter(gpu, oracle):
    """Score filter -> NMS on the device, the reference's post-processing chain (se-ssd-ai-trt.cpp:1868-1892)."""
    S = gpu.schedule
    box, cls, iou, dr = _head_outputs(gpu, 9, 2, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, 2, logit_mean=-4.5)
    r = gpu.filter_boxes(*_to_gpu(box, cls, iou, dr), gpu.filter_params(), anchors=gpu.anchor_params())
    kept, kept_num = gpu.rotated_nms(r["box"], r["valid"], S.NMS_THRESH)
    for b in range(2):
        n = int(r["valid"][b])
        src = r["box"][b, :n].cpu().numpy()
        if not _clear_of_threshold(oracle, src, S.NMS_THRESH, 1e-5):
            pytest.skip("a pair sits on the threshold for this seed")
        want, _ = oracle.rotated_nms(src, S.NMS_THRESH)
        assert int(kept_num[b]) == len(want) and len(want) > 0
        np.testing.assert_array_equal(kept[b, :len(want)].cpu().numpy(), want)
