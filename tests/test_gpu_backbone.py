"""GPU parity of the fused front end (voxelise -> 14 conv layers -> dense BEV) and of Sparse2Dense."""
import os

import numpy as np
import pytest

import make_golden_inputs as mk
from conftest import match_rows, rel_err

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _oracle_layer(oracle, case, l, W, sc, sh, c, n, f, fp16, pair_log=None):
    """One conv layer + folded BatchNorm + ReLU on the oracle: (coors, n, features) -> the same for the output.
    pair_log (a list) receives the layer's number of rulebook pairs."""
    maxV = case["max_voxels"]
    if l.subm:
        pairs, pnum, st = oracle.subm_rulebook(c, n, l.out_shape, maxV)
        oc, on = c, n
    else:
        oc, on, pairs, pnum, st = oracle.spconv_rulebook(c, n, l.ksize, l.stride, l.padding, l.out_shape, maxV)
        oc = oc[:on].copy()
    assert st == 0
    if pair_log is not None:
        pair_log.append(int(pnum.astype(np.int64).sum()))
    y = oracle.conv_apply(f, pairs, pnum, W, on, half_inputs=fp16)
    return oc, on, oracle.scale_shift_relu(y, sc, sh, True, half_out=fp16)


def _oracle_layers(oracle, case, fp16, pair_log=None):
    """Runs the oracle layer by layer, returning (coors, n, features) after every layer."""
    vox, coors, npv, n, st = oracle.voxelize(case["points"], case["range"], case["voxel"], case["max_voxels"])
    feat = vox[:n]
    if fp16:
        feat = feat.astype(np.float16).astype(np.float32)
    outs = [(coors[:n].copy(), n, feat)]
    for l, W, sc, sh in zip(case["layers"], case["weights"], case["scale"], case["shift"]):
        c, n, f = outs[-1]
        outs.append(_oracle_layer(oracle, case, l, W, sc, sh, c, n, f, fp16, pair_log))
    return outs


def _check_fp32_layers(want, views, tol=1e-5):
    """Rows are matched by coordinate: the library numbers the outputs of strided layers in (z, y, x) order, the
    oracle in first-seen order; a row's value does not depend on its number."""
    for i, ((wc, wn, wf), (gf, gc, gn)) in enumerate(zip(want, views)):
        assert int(gn[0]) == wn, f"layer {i - 1}"
        perm = match_rows(gc[0, :wn], wc)
        assert rel_err(gf[0, :wn][perm], wf) <= tol, f"layer {i - 1}"
        np.testing.assert_array_equal(gf[0, :wn][perm], wf)   # same summation order as the oracle


def _max_norm_err(a, b):
    b = np.asarray(b, np.float64)
    return float(np.abs(np.asarray(a, np.float64) - b).max() / max(np.abs(b).max(), 1e-30)) if b.size else 0.0


def _check_fp16_layers(oracle, case, want, views, tol=1e-2, drift_tol=2e-2):
    """fp16 parity: every layer is within `tol` (element-wise relative) of the oracle applied to the SAME
    input (the library's own previous layer), which is what a per-layer tolerance means. Against the
    oracle's own chain, one-ulp differences of earlier layers are inherited and values next to the ReLU
    threshold flip between 0 and tiny, so that comparison is normalised by the layer's largest magnitude
    (`drift_tol`). The coordinate sets must be identical; rows are matched by coordinate (the library numbers
    the outputs of strided layers in (z, y, x) order, the oracle in first-seen order)."""
    params = list(zip(case["layers"], case["weights"], case["scale"], case["shift"]))
    for i, ((wc, wn, wf), (gf, gc, gn)) in enumerate(zip(want, views)):
        assert int(gn[0]) == wn, f"layer {i - 1}"
        perm = match_rows(gc[0, :wn], wc)
        drift = _max_norm_err(gf[0, :wn][perm], wf)
        assert drift <= drift_tol, f"layer {i - 1}: drift {drift}"
        if i == 0:
            np.testing.assert_array_equal(gf[0, :wn][perm], wf)   # voxel means are exact
            continue
        l, W, sc, sh = params[i - 1]
        pf, pc, pn = views[i - 1]
        m = int(pn[0])
        oc, on, y = _oracle_layer(oracle, case, l, W, sc, sh, pc[0, :m], m, pf[0, :m], True)
        assert on == wn
        err = rel_err(gf[0, :wn][match_rows(gc[0, :wn], oc[:on])], y)
        assert err <= tol, f"layer {i - 1}: rel err {err}"


def _gpu_run(gpu, case, dtype, frames=None):
    import torch

    frames = frames or [case["points"]]
    P = max(len(f) for f in frames)
    pts = np.zeros((len(frames), P, 4), np.float32)
    sizes = np.zeros(len(frames), np.int32)
    for b, f in enumerate(frames):
        pts[b, :len(f)], sizes[b] = f, len(f)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=dtype,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    dense, ws = bb.run(torch.from_numpy(pts).cuda(), torch.from_numpy(sizes).cuda())
    torch.cuda.synchronize()
    assert gpu.read_status(ws) == 0
    views = [bb.layer_view(ws, len(frames), P, i) for i in range(-1, len(case["layers"]))]
    views = [(f.float().cpu().numpy(), c.cpu().numpy(), n.cpu().numpy()) for f, c, n in views]
    d = dense.float().cpu().numpy()
    bb.close()
    return d, views


@pytest.mark.parametrize("dtype,tol", [(0, 1e-5), (1, 1e-2)])
def test_small_backbone_every_layer(gpu, oracle, dtype, tol):
    case = mk.small_case(gpu)
    want = _oracle_layers(oracle, case, fp16=bool(dtype))
    dense, views = _gpu_run(gpu, case, dtype)
    if dtype == 1:
        _check_fp16_layers(oracle, case, want, views, tol)
    else:
        _check_fp32_layers(want, views, tol)
    c, n, f = want[-1]
    Cc, D, H, W = case["bev"]
    gf, gc, gn = views[-1]
    # the BEV map is exactly the scatter of the library's own last layer ...
    np.testing.assert_array_equal(dense, oracle.sparse2dense(gf[0, :n], gc[0, :n], n, Cc, D, H, W))
    # ... and stays within the chain tolerance of the oracle's map
    want_dense = oracle.sparse2dense(f, c, n, Cc, D, H, W)
    assert (rel_err(dense, want_dense) <= tol) if dtype == 0 else (_max_norm_err(dense, want_dense) <= 2e-2)


def test_small_backbone_matches_committed_golden(gpu):
    g = np.load(os.path.join(GOLDEN, "front_end_small.npz"))
    case = mk.small_case(gpu)
    dense, views = _gpu_run(gpu, case, 0)
    gf, gc, gn = views[-1]
    n = int(gn[0])
    np.testing.assert_array_equal([int(v[2][0]) for v in views[1:]], g["layer_rows"])
    perm = match_rows(gc[0, :n], g["coors"])
    np.testing.assert_allclose(gf[0, :n][perm], g["feat"], rtol=1e-5, atol=1e-7)
    nz = np.flatnonzero(dense)
    np.testing.assert_array_equal(nz, g["dense_nz"])
    np.testing.assert_allclose(dense.ravel()[nz], g["dense_val"], rtol=1e-5, atol=1e-7)


def test_batched_frames_equal_single_frame_runs(gpu):
    """Frames in one batch must not influence each other (they are sharded across GPUs as units)."""
    case = mk.small_case(gpu)
    other = mk.small_case(gpu, n_points=900, seed=123)["points"]
    d_b, v_b = _gpu_run(gpu, case, 1, frames=[other, case["points"], np.zeros((0, 4), np.float32)])
    d_1, v_1 = _gpu_run(gpu, case, 1)
    np.testing.assert_array_equal(d_b[1], d_1[0])
    assert not d_b[2].any()
    for (fb, cb, nb), (f1, c1, n1) in zip(v_b, v_1):
        n = int(n1[0])
        assert int(nb[1]) == n and int(nb[2]) == 0
        np.testing.assert_array_equal(fb[1, :n], f1[0, :n])
        c1 = c1[0, :n].copy()
        c1[:, 0] = 1
        np.testing.assert_array_equal(cb[1, :n], c1)


def test_full_size_backbone_fp16_20k_points(gpu, oracle):
    """The single-frame backbone case at the reference's full grid, fp16, per-layer 1e-2."""
    S = gpu.synth
    w, sc, sh = gpu.random_weights()
    case = dict(points=S.single_frame(), range=S.POINT_RANGE, voxel=S.VOXEL_SIZE, max_voxels=60000,
                layers=gpu.schedule.LAYERS, weights=w, scale=sc, shift=sh, bev=(64, 2, 200, 176))
    want = _oracle_layers(oracle, case, fp16=True)
    dense, views = _gpu_run(gpu, case, 1)
    _check_fp16_layers(oracle, case, want, views)
    c, n, f = want[-1]
    gf, gc, gn = views[-1]
    np.testing.assert_array_equal(dense, oracle.sparse2dense(gf[0, :n], gc[0, :n], n, 64, 2, 200, 176))


def test_sweep_frame_every_layer_against_the_oracle(gpu, oracle):
    """The configuration the throughput figure is quoted on: one 120,000-point sweep frame, max_voxels 200,000,
    fp16, through sessd_backbone_enqueue. Row counts, coordinate sets and per-layer rulebook pair counts are exact;
    every layer's features are within 1e-2 (relative) of the oracle applied to the same input; the BEV map is the
    scatter of the last layer."""
    import torch

    S = gpu.synth
    w, sc, sh = gpu.random_weights()
    case = dict(points=S.sweep_frame(0), range=S.POINT_RANGE, voxel=S.VOXEL_SIZE, max_voxels=200000,
                layers=gpu.schedule.LAYERS, weights=w, scale=sc, shift=sh, bev=(64, 2, 200, 176))
    want_pairs = []
    want = _oracle_layers(oracle, case, fp16=True, pair_log=want_pairs)
    dense, views = _gpu_run(gpu, case, 1)
    _check_fp16_layers(oracle, case, want, views)
    c, n, f = want[-1]
    gf, gc, gn = views[-1]
    np.testing.assert_array_equal(dense, oracle.sparse2dense(gf[0, :n], gc[0, :n], n, 64, 2, 200, 176))
    want_dense = oracle.sparse2dense(f, c, n, 64, 2, 200, 176)
    assert _max_norm_err(dense, want_dense) <= 2e-2
    # the P of the flop count 2 * P * Cin * Cout, layer by layer (indice_num of the reference, submConv3dlayer.cu:413)
    bb = gpu.Backbone(200000, w, sc, sh, dtype=1)
    pts = torch.from_numpy(case["points"][None]).cuda()
    sizes = torch.tensor([len(case["points"])], dtype=torch.int32, device="cuda")
    d, ws = bb.run(pts, sizes)
    got_pairs = gpu.pair_counts(bb, pts, sizes, ws, d)
    bb.close()
    assert got_pairs == want_pairs


def test_round_trip_dense_to_sparse_at_sweep_size(gpu):
    """Size-independent property at the 120k-point size: every active output row reappears in the BEV map
    at channel c*D+z, pixel (y,x), and nothing else is non-zero."""
    import torch

    S = gpu.synth
    w, sc, sh = gpu.random_weights()
    bb = gpu.Backbone(200000, w, sc, sh, dtype=1)
    f = S.sweep_frame(3)
    pts = torch.from_numpy(f[None]).cuda()
    sizes = torch.tensor([len(f)], dtype=torch.int32, device="cuda")
    dense, ws = bb.run(pts, sizes)
    torch.cuda.synchronize()
    assert gpu.read_status(ws) == 0
    feat, coors, num = bb.layer_view(ws, 1, len(f), len(bb.layers) - 1)
    n = int(num[0])
    c = coors[0, :n].long()
    d = dense[0].reshape(64, 2, 200, 176)
    got = d[:, c[:, 1], c[:, 2], c[:, 3]].T
    assert torch.equal(got, feat[0, :n])
    assert int((dense != 0).sum()) == int((feat[0, :n] != 0).sum())
    # the rows are unique cells
    key = (c[:, 1] * 200 + c[:, 2]) * 176 + c[:, 3]
    assert key.unique().numel() == n
    bb.close()


def test_sweep_size_batch_equals_single_frame_runs(gpu):
    """Four 120k-point frames in one call: blocks of the tensor-core kernel then walk several row groups
    across frame boundaries. Every frame's BEV map and final rows must be bit-identical to the frame run
    alone, with a clean status word (a bounded wait that gives up shows there)."""
    import torch

    S = gpu.synth
    w, sc, sh = gpu.random_weights()
    bb = gpu.Backbone(200000, w, sc, sh, dtype=1)
    frames = np.stack([S.sweep_frame(i) for i in range(4)])
    pts = torch.from_numpy(frames).cuda()
    sizes = torch.full((4,), frames.shape[1], dtype=torch.int32, device="cuda")
    last = len(bb.layers) - 1
    for rep in range(2):   # the second pass reuses the workspace the first one left behind
        dense, ws = bb.run(pts, sizes)
        torch.cuda.synchronize()
        assert gpu.read_status(ws) == 0
    feat, coors, num = [t.clone() for t in bb.layer_view(ws, 4, frames.shape[1], last)]
    dense = dense.clone()
    for b in (0, 3):
        d1, ws1 = bb.run(pts[b:b + 1], sizes[b:b + 1])
        torch.cuda.synchronize()
        assert gpu.read_status(ws1) == 0
        f1, c1, n1 = bb.layer_view(ws1, 1, frames.shape[1], last)
        n = int(n1[0])
        assert int(num[b]) == n and torch.equal(dense[b], d1[0])
        assert torch.equal(feat[b, :n], f1[0, :n]) and torch.equal(coors[b, :n, 1:], c1[0, :n, 1:])
    bb.close()


def test_backbone_enqueue_can_be_captured_in_a_cuda_graph(gpu):
    """The enqueue call allocates nothing, synchronises nothing and reads its row counts on the device, so a
    host can capture it once and replay it (the first call, which configures the kernels, stays outside)."""
    import torch

    case = mk.small_case(gpu)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=1,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    P = len(case["points"])
    pts = torch.zeros((1, P, 4), device="cuda")
    sizes = torch.zeros((1,), dtype=torch.int32, device="cuda")
    pts[0] = torch.from_numpy(case["points"]).cuda()
    sizes[0] = P
    want, ws = bb.run(pts, sizes)          # plain call; also the warm-up
    want = want.clone()
    dense = torch.empty_like(want)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            bb.run(pts, sizes, workspace=ws, dense=dense)
    for half in (False, True):             # replay on new inputs written into the captured buffers
        if half:
            sizes[0] = P // 2
        dense.fill_(7)
        graph.replay()
        torch.cuda.synchronize()
        assert gpu.read_status(ws) == 0
        if not half:
            assert torch.equal(dense, want)
        else:
            ref, _ = bb.run(pts, sizes)
            torch.cuda.synchronize()
            assert torch.equal(dense, ref) and not torch.equal(dense, want)
    bb.close()


def test_backbone_from_weight_file_equals_backbone_from_arrays(gpu, tmp_path):
    """A weight file in the exporter's format, with the state-dict names the reference's builder looks up
    (conv `backbone.middle_conv.<i>.weight`, batch norm at <i+1>), gives the same BEV map as a backbone
    created from the arrays with the batch norm folded by the oracle's restatement."""
    import torch
    from oracle import formats as oracle_formats

    case = mk.small_case(gpu)
    rng = np.random.default_rng(21)
    blobs, scale, shift = [], [], []
    for layer, w in zip(case["layers"], case["weights"]):
        i = int("".join(ch for ch in layer.name if ch.isdigit()))
        bn = [rng.uniform(0.5, 1.5, layer.cout), rng.standard_normal(layer.cout) * 0.1,
              rng.standard_normal(layer.cout) * 0.1, rng.uniform(0.5, 2.0, layer.cout)]
        bn = [a.astype(np.float32) for a in bn]
        blobs.append((f"backbone.middle_conv.{i}.weight", w))
        for suffix, a in zip(("weight", "bias", "running_mean", "running_var"), bn):
            blobs.append((f"backbone.middle_conv.{i + 1}.{suffix}", a))
        blobs.append((f"backbone.middle_conv.{i + 1}.num_batches_tracked", np.array([100.0], np.float32)))
        sc, sh = oracle_formats.fold_batchnorm(*bn, 1e-5)
        scale.append(sc)
        shift.append(sh)
    path = tmp_path / "model.wts"
    oracle_formats.write_wts(path, blobs)
    wts = gpu.formats.Wts(path)
    kw = dict(dtype=1, layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    from_file = gpu.Backbone.from_wts(wts, case["max_voxels"], **kw)
    from_arrays = gpu.Backbone(case["max_voxels"], case["weights"], scale, shift, **kw)
    pts = torch.from_numpy(case["points"]).cuda()[None]
    sizes = torch.tensor([pts.shape[1]], dtype=torch.int32, device="cuda")
    a, wsa = from_file.run(pts, sizes)
    b, wsb = from_arrays.run(pts, sizes)
    torch.cuda.synchronize()
    assert gpu.read_status(wsa) == 0 and gpu.read_status(wsb) == 0
    assert float(a.float().abs().sum()) > 0
    # the folded scale may differ from the oracle's in the square root's last bit: 1e-2 relative is the fp16
    # bar of the whole stack; in practice the maps are equal
    assert rel_err(a.float().cpu().numpy(), b.float().cpu().numpy()) <= 1e-2
    short = gpu.formats.Wts(path)
    with pytest.raises(gpu.SessdError):              # a module index the file does not hold
        gpu.Backbone.from_wts(short, case["max_voxels"], module_index=[100 + 3 * i for i in range(len(case["layers"]))], **kw)
    from_file.close()
    from_arrays.close()


@pytest.mark.parametrize("graphs", [False, True])
def test_pipeline_groups_equal_direct_backbone_runs(gpu, graphs):
    """Seven frames through a pipeline of groups of two on two stream slots (three full groups and a partial
    one), from host buffers and from device buffers, with plain launches and with graph replay: voxel counts,
    status words and the BEV maps left in the slots must equal direct backbone runs of the same frames, on
    every pass (a replayed graph reads the new contents of the slot's staging buffers)."""
    import torch

    case = mk.small_case(gpu)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=1,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    P, F, B = len(case["points"]), 7, 2
    rng = np.random.default_rng(5)
    host_pts = torch.zeros((F, P, 4), dtype=torch.float32).pin_memory()
    host_sizes = torch.zeros((F,), dtype=torch.int32).pin_memory()
    vnum = torch.zeros((F,), dtype=torch.int32).pin_memory()
    status = torch.zeros((F,), dtype=torch.int32).pin_memory()
    pipe = gpu.Pipeline(bb, B, P, nstreams=2)
    if graphs:
        pipe.use_graphs(True)
    last = len(bb.layers) - 1
    launches = []
    for rep in range(3):                   # pass 0 warms the slots, pass 1 captures, pass 2 replays
        for f in range(F):
            n = int(rng.integers(P // 3, P + 1))
            host_pts[f, :n] = torch.from_numpy(case["points"][rng.permutation(P)[:n]])
            host_sizes[f] = n
        want_dense, want_num = [], []
        for f in range(F):
            d, ws = bb.run(host_pts[f:f + 1].cuda(), host_sizes[f:f + 1].cuda())
            torch.cuda.synchronize()
            assert gpu.read_status(ws) == 0
            want_dense.append(d[0].clone())
            want_num.append(int(bb.layer_view(ws, 1, P, last)[2][0]))
        for from_host in (True, False):
            vnum.fill_(-1)
            status.fill_(-1)
            l0 = gpu.launch_count()
            if from_host:
                pipe.run_host(host_pts, host_sizes, vnum, status)
                assert vnum.tolist() == want_num and status.tolist() == [0] * F
            else:
                pipe.run_device(host_pts.cuda(), host_sizes.cuda())
            launches.append(gpu.launch_count() - l0)
            assert pipe.status_bits() == 0
            # groups 0..3 ran on slots 0,1,0,1: slot 0 holds frames 4,5 and slot 1 the partial group (frame 6)
            assert torch.equal(pipe.dense(0)[0], want_dense[4]) and torch.equal(pipe.dense(0)[1], want_dense[5])
            assert torch.equal(pipe.dense(1)[0], want_dense[6])
    assert len(set(launches)) == 1 and launches[0] > 0      # replayed kernels are counted like launched ones
    # the variant that also brings the BEV maps to the host: one region per stream slot, holding its last group
    host_dense = torch.zeros((2, B) + tuple(want_dense[0].shape), dtype=torch.float16).pin_memory()
    pipe.run_host_bev(host_pts, host_sizes, vnum, status, host_dense)
    assert vnum.tolist() == want_num and status.tolist() == [0] * F
    assert torch.equal(host_dense[0, 0], want_dense[4].cpu()) and torch.equal(host_dense[0, 1], want_dense[5].cpu())
    assert torch.equal(host_dense[1, 0], want_dense[6].cpu())
    pipe.close()
    bb.close()


def test_pipeline_host_runs_reuse_both_input_and_bev_buffers(gpu):
    """Eleven frames in groups of two on two stream slots: every slot takes three groups, so that the copy-in
    of a group waits for the group that used the same input buffer two turns earlier and the BEV buffer of a
    group waits for the copy-out of its previous contents. Two runs in a row (the second starts with the
    events the first one left); voxel counts of every frame and the BEV maps of the last group of each slot
    must equal direct backbone runs."""
    import torch

    case = mk.small_case(gpu)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=1,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    P, F, B = len(case["points"]), 11, 2
    rng = np.random.default_rng(11)
    host_pts = torch.zeros((F, P, 4), dtype=torch.float32).pin_memory()
    host_sizes = torch.zeros((F,), dtype=torch.int32).pin_memory()
    vnum = torch.zeros((F,), dtype=torch.int32).pin_memory()
    status = torch.zeros((F,), dtype=torch.int32).pin_memory()
    pipe = gpu.Pipeline(bb, B, P, nstreams=2)
    last = len(bb.layers) - 1
    for rep in range(2):
        for f in range(F):
            n = int(rng.integers(P // 3, P + 1))
            host_pts[f].zero_()
            host_pts[f, :n] = torch.from_numpy(case["points"][rng.permutation(P)[:n]])
            host_sizes[f] = n
        want_dense, want_num = [], []
        for f in range(F):
            d, ws = bb.run(host_pts[f:f + 1].cuda(), host_sizes[f:f + 1].cuda())
            torch.cuda.synchronize()
            want_dense.append(d[0].clone())
            want_num.append(int(bb.layer_view(ws, 1, P, last)[2][0]))
        host_dense = torch.zeros((2, B) + tuple(want_dense[0].shape), dtype=torch.float16).pin_memory()
        vnum.fill_(-1)
        status.fill_(-1)
        pipe.run_host_bev(host_pts, host_sizes, vnum, status, host_dense)
        assert vnum.tolist() == want_num and status.tolist() == [0] * F
        # groups 0..5 ran on slots 0,1,0,1,0,1: slot 0 ends with frames 8,9 and slot 1 with the partial group (frame 10)
        assert torch.equal(host_dense[0, 0], want_dense[8].cpu()) and torch.equal(host_dense[0, 1], want_dense[9].cpu())
        assert torch.equal(host_dense[1, 0], want_dense[10].cpu())
        assert torch.equal(pipe.dense(0)[0], want_dense[8]) and torch.equal(pipe.dense(1)[0], want_dense[10])
        vnum.fill_(-1)
        pipe.run_host(host_pts, host_sizes, vnum, status)
        assert vnum.tolist() == want_num and status.tolist() == [0] * F
        assert torch.equal(pipe.dense(0)[1], want_dense[9]) and torch.equal(pipe.dense(1)[0], want_dense[10])
    pipe.close()
    bb.close()


@pytest.mark.parametrize("dtype", [0, 1])
def test_sparse2dense_plugin_entry(gpu, oracle, dtype):
    import torch

    rs = np.random.RandomState(4)
    B, V, Cc, D, H, W = 2, 512, 64, 2, 20, 16
    feat = np.zeros((B, V, Cc), np.float32)
    coors = np.zeros((B, V, 4), np.int32)
    num = np.array([300, 0], np.int32)
    cells = rs.permutation(D * H * W)[:300]
    coors[0, :300, 1], coors[0, :300, 2], coors[0, :300, 3] = cells // (H * W), (cells // W) % H, cells % W
    feat[0, :300] = rs.randn(300, Cc)
    tdt = torch.float32 if dtype == 0 else torch.float16
    p = gpu.S2DParams(W, H, D, Cc)
    dense = gpu.sparse2dense(torch.from_numpy(feat).cuda().to(tdt), torch.from_numpy(coors).cuda(),
                             torch.from_numpy(num).cuda(), p, dtype)
    src = feat[0, :300].astype(np.float16).astype(np.float32) if dtype else feat[0, :300]
    want = oracle.sparse2dense(src, coors[0], 300, Cc, D, H, W, batch=1)
    np.testing.assert_array_equal(dense[0].float().cpu().numpy(), want[0])
    assert not dense[1].any()


def test_misaligned_workspace_is_refused(gpu):
    """A workspace that does not start on a 256-byte boundary is refused before any kernel runs (the kernels
    use 16- and 32-byte vector accesses relative to it)."""
    import torch

    case = mk.small_case(gpu)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=1,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    pts = torch.from_numpy(case["points"]).cuda()[None]
    sizes = torch.tensor([pts.shape[1]], dtype=torch.int32, device="cuda")
    nbytes = bb.workspace_bytes(1, pts.shape[1])
    raw = torch.empty(nbytes + 512, dtype=torch.uint8, device="cuda")
    launches = gpu.launch_count()
    with pytest.raises(gpu.SessdError):
        bb.run(pts, sizes, workspace=raw[16:16 + nbytes])
    assert gpu.launch_count() == launches
    dense, ws = bb.run(pts, sizes, workspace=raw[256:256 + nbytes])
    torch.cuda.synchronize()
    assert gpu.read_status(ws) == 0
    bb.close()


def test_empty_and_out_of_range_frames_inside_a_batch(gpu):
    """Frames with no points, and with points that all lie outside the range, between ordinary frames: they
    come out with zero rows at every layer and an all-zero BEV map, the ordinary frames exactly as when run
    alone, and nothing is reported in the status word."""
    import torch

    case = mk.small_case(gpu)
    bb = gpu.Backbone(case["max_voxels"], case["weights"], case["scale"], case["shift"], dtype=1,
                      layers=case["layers"], point_range=case["range"], voxel_size=case["voxel"])
    P = len(case["points"])
    pts = np.zeros((4, P, 4), np.float32)
    pts[0] = case["points"]
    pts[2] = case["points"] + np.array([1000.0, 0, 0, 0], np.float32)      # every point beyond x_max
    pts[3] = case["points"][::-1]
    sizes = np.array([P, 0, P, P], np.int32)
    dense, ws = bb.run(torch.from_numpy(pts).cuda(), torch.from_numpy(sizes).cuda())
    torch.cuda.synchronize()
    assert gpu.read_status(ws) == 0
    for layer in range(-1, len(bb.layers)):
        num = bb.layer_view(ws, 4, P, layer)[2].cpu().numpy()
        assert num[1] == 0 and num[2] == 0 and num[0] > 0 and num[3] == num[0]
    assert not dense[1].any() and not dense[2].any()
    alone, ws1 = bb.run(torch.from_numpy(pts[:1]).cuda(), torch.from_numpy(sizes[:1]).cuda())
    torch.cuda.synchronize()
    assert torch.equal(dense[0], alone[0])
    # frame 3 holds the same points in reverse order: the same cells at every layer (checked above through the
    # row counts), numbered differently
    assert dense[3].any()
    bb.close()
