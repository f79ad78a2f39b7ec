"""GPU: the whole frame -> boxes chain (the reference's end-to-end configuration, random-init weights).

The sparse front end and the post-processing kernels have their own parity tests; this file checks the glue:
the fp16 neck and head against the fp32 CPU restatement of the reference's layer graph on the same BEV map
(tolerance 2e-2 of the output's largest magnitude: fourteen fp16 layers), the head-output layout against the
post-processing oracle (exact decisions, 1e-5 on values), and the chained NMS against the oracle's greedy NMS.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NECK_TOL = 2e-2


def _norm_err(got, want):
    return float(np.abs(got.astype(np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.fixture(scope="module")
def chain(gpu, oracle):
    """One 20,000-point synthetic frame through the detector, with the classification bias set so that a few
    hundred anchors pass the score threshold (random heads would pass half of them)."""
    import torch
    from oracle import neck as oracle_neck

    D, S = gpu.detector, gpu.synth
    w, sc, sh = gpu.random_weights()
    bb = gpu.Backbone(60000, w, sc, sh, dtype=1)
    blobs = D.random_neck_weights()
    frame = S.single_frame()
    pts = torch.from_numpy(frame).cuda()[None]
    sizes = torch.tensor([len(frame)], dtype=torch.int32, device="cuda")
    det = D.Detector(bb, D.Neck2D(blobs))
    logits = det(pts, sizes)["heads"]["cls"][0, :, 0].float().cpu().numpy()
    thr_logit = float(np.log(gpu.schedule.SCORE_THRESHOLD / (1 - gpu.schedule.SCORE_THRESHOLD)))
    shift = thr_logit - float(np.sort(logits)[-300])            # about 300 of 70,400 anchors pass
    blobs["bbox_head.tasks.0.conv_cls.bias"] = blobs["bbox_head.tasks.0.conv_cls.bias"] + np.float32(shift)
    det = D.Detector(bb, D.Neck2D(blobs))
    out = det(pts, sizes)
    torch.cuda.synchronize()
    bev, _ = bb.run(pts, sizes)
    want = oracle_neck.neck_and_head(bev.float().cpu().numpy(), blobs)
    yield dict(out=out, want=want, det=det, bev=bev, blobs=blobs)
    bb.close()


def test_neck_and_head_match_fp32_restatement(gpu, chain):
    out, want = chain["out"], chain["want"]
    assert out["status"] == 0
    feat = chain["det"].neck.features(chain["bev"]).float().cpu().numpy()
    assert feat.shape == (1, 128, 200, 176) and np.abs(want["features"]).max() > 1e-3
    assert _norm_err(feat, want["features"]) <= NECK_TOL
    for name, width in (("box", 7), ("cls", 1), ("iou", 1), ("dir", 2)):
        got = out["heads"][name].cpu().numpy()
        assert got.shape == (1, 70400, width) == want[name].shape
        assert _norm_err(got, want[name]) <= NECK_TOL, name


def test_post_processing_of_the_head_outputs_matches_oracle(gpu, oracle, chain):
    S = gpu.schedule
    out = chain["out"]
    heads = {k: v[0].cpu().numpy() for k, v in out["heads"].items()}
    score = 1.0 / (1.0 + np.exp(-heads["cls"][:, 0].astype(np.float64)))
    if (np.abs(score - S.SCORE_THRESHOLD) < 1e-6).any():
        pytest.skip("a score sits on the threshold for this seed")
    oparams = oracle.anchor_params(gpu.synth.POINT_RANGE, S.CAR_SIZE, S.DIRECTION_ANGLES)
    decoded = oracle.anchor_decode(heads["box"], oparams, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, 2)
    ob, oc, oi, od, valid, passed = oracle.filter_boxes(decoded, heads["cls"], heads["iou"], heads["dir"], 2,
                                                        S.MAX_BOX_NUM, S.SCORE_THRESHOLD, S.DIRECTION_OFFSET)
    f = out["filtered"]
    assert 100 <= passed <= S.MAX_BOX_NUM and int(f["valid"][0]) == valid
    np.testing.assert_array_equal(f["direction"][0].cpu().numpy(), od)
    np.testing.assert_allclose(f["box"][0].cpu().numpy(), ob, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(f["score"][0].cpu().numpy(), oc, rtol=1e-5, atol=1e-6)
    src = f["box"][0, :valid].cpu().numpy()
    want, _ = oracle.rotated_nms(src, S.NMS_THRESH)
    ious = [oracle.bev_iou(src[i], src[j]) for i in range(min(valid, 60)) for j in range(i)]
    if any(abs(v - S.NMS_THRESH) < 1e-5 for v in ious):
        pytest.skip("a pair sits on the NMS threshold for this seed")
    n = int(out["num"][0])
    assert n == len(want) and 0 < n <= valid
    np.testing.assert_array_equal(out["boxes"][0, :n].cpu().numpy(), want)


def test_end_to_end_boxes_against_the_fp32_chain(gpu, oracle, chain):
    """Boxes from the fp32 CPU neck, pushed through the oracle's post-processing, are found by the GPU chain
    wherever the score is clear of the threshold (fp16 can flip a decision that sits on it)."""
    S = gpu.schedule
    want = {k: v[0] for k, v in chain["want"].items() if k != "features"}
    oparams = oracle.anchor_params(gpu.synth.POINT_RANGE, S.CAR_SIZE, S.DIRECTION_ANGLES)
    decoded = oracle.anchor_decode(want["box"], oparams, S.FEATURE_MAP_HEIGHT, S.FEATURE_MAP_WIDTH, 2)
    ob, oc, _, _, valid, _ = oracle.filter_boxes(decoded, want["cls"], want["iou"], want["dir"], 2, S.MAX_BOX_NUM,
                                                 S.SCORE_THRESHOLD, S.DIRECTION_OFFSET)
    f = chain["out"]["filtered"]
    got = f["box"][0, :int(f["valid"][0])].cpu().numpy()
    logit = want["cls"][:, 0]
    thr_logit = np.log(S.SCORE_THRESHOLD / (1 - S.SCORE_THRESHOLD))
    spread = np.abs(chain["want"]["cls"]).max()
    clear = np.flatnonzero(logit - thr_logit > 4 * NECK_TOL * spread)      # passes by more than the neck's error bar
    assert len(clear) > 10
    for a in clear[:50]:
        d = np.abs(got[:, :3] - decoded[a, :3]).max(axis=1)
        assert d.min() <= 0.05 * max(1.0, np.abs(decoded[a, :3]).max()), f"anchor {a} has no box on the GPU"


def test_captured_chain_replays_on_new_frames(gpu, chain):
    """The whole chain recorded into one CUDA graph gives, on replay with other frames in its input buffers,
    the boxes of the plain call on those frames, bit for bit."""
    import torch

    det = chain["det"]
    S = gpu.synth
    P = 20000
    det.capture(P)
    for seed in (3, 4):
        frame = S.lidar_frame(gpu.sharding.frame_seed(seed), n_points=P, n_boxes=15)
        n = P if seed == 3 else P - 3000
        pts = torch.zeros((1, P, 4), device="cuda")
        pts[0, :n] = torch.from_numpy(frame[:n]).cuda()
        sizes = torch.tensor([n], dtype=torch.int32, device="cuda")
        want = det(pts, sizes)
        got = det.replay(pts, sizes)
        assert got["status"] == 0 and want["status"] == 0
        k = int(want["num"][0])
        assert int(got["num"][0]) == k and k > 0
        assert torch.equal(got["boxes"][0, :k], want["boxes"][0, :k])
        assert torch.equal(got["filtered"]["valid"], want["filtered"]["valid"])
