"""GPU parity: sparse conv plugins' entry points against the oracle.

Rulebooks must be bit-exact after canonical sorting; fp32 features within 1e-5 relative (the kernel
repeats the oracle's summation order, so they are in fact identical); fp16 within 1e-2 relative.
"""
import numpy as np
import pytest

from conftest import canonical_rulebook, match_rows, rel_err

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
FP16_TOL = 1e-2


def _layer(pkg, subm, cin, cout, K, S, P, in_shape):
    out_shape = in_shape if subm else tuple((in_shape[j] + 2 * P[j] - K[j]) // S[j] + 1 for j in range(3))
    return pkg.schedule.ConvLayer("t", subm, cin, cout, tuple(K), tuple(S), tuple(P), tuple(in_shape), out_shape)


def _random_coords(rs, n, shape):
    vol = int(np.prod(shape))
    cells = rs.permutation(vol)[:n] if vol < 5_000_000 else np.unique(rs.randint(0, vol, int(n * 1.2)))[:n]
    cells = rs.permutation(cells)
    c = np.zeros((len(cells), 4), np.int32)
    c[:, 1], c[:, 2], c[:, 3] = cells // (shape[1] * shape[2]), (cells // shape[2]) % shape[1], cells % shape[2]
    return c


def _run_layer(gpu, layer, frames, W, scale=None, shift=None, relu=False, dtype=0, maxV=None):
    """frames: list of (coors [n,4], feat [n,Cin]). Returns per-frame dicts of numpy arrays."""
    import torch

    maxV = maxV or max(max(len(c) for c, _ in frames) * 3, 64)
    B = len(frames)
    tdt = np.float32 if dtype == gpu.F32 else np.float16
    feat = np.zeros((B, maxV, layer.cin), tdt)
    coors = np.zeros((B, maxV, 4), np.int32)
    num = np.zeros(B, np.int32)
    for b, (c, f) in enumerate(frames):
        c = c.copy()
        c[:, 0] = b
        coors[b, :len(c)], feat[b, :len(c)], num[b] = c, f.astype(tdt), len(c)
    p = gpu.conv_params(layer, maxV)
    w = gpu.ConvWeights(p, W, scale, shift, relu, dtype)
    fn = gpu.subm_conv if layer.subm else gpu.sparse_conv
    tf, tc, tn = torch.from_numpy(feat).cuda(), torch.from_numpy(coors).cuda(), torch.from_numpy(num).cuda()
    r = fn(tf, tc, tn, p, w, keep_workspace=True)
    out_num = r["voxel_num"] if not layer.subm else tn
    res = []
    for b in range(B):
        pairs, pnum = gpu.rulebook_export(p, B, b, r["workspace"], out_num)
        d = dict(features=r["features"][b].float().cpu().numpy(), pairs=pairs.cpu().numpy(),
                 pair_num=pnum.cpu().numpy().astype(np.uint32), status=r["status"])
        if layer.subm:
            d["coors"], d["num"] = coors[b], int(num[b])
        else:
            d["coors"], d["num"] = r["coors"][b].cpu().numpy(), int(r["voxel_num"][b])
        res.append(d)
    w.close()
    return res, maxV


def _check_layer(gpu, oracle, layer, frames, W, scale=None, shift=None, relu=False, dtype=0, maxV=None, tol=None):
    res, maxV = _run_layer(gpu, layer, frames, W, scale, shift, relu, dtype, maxV)
    half = dtype == gpu.F16
    tol = tol if tol is not None else (FP16_TOL if half else FP32_TOL)
    for b, ((c, f), g) in enumerate(zip(frames, res)):
        c = c.copy()
        c[:, 0] = b
        n = len(c)
        assert g["status"] == 0
        if layer.subm:
            pairs, pnum, st = oracle.subm_rulebook(c, n, layer.out_shape, maxV, ksize=layer.ksize[0],
                                                   padding=layer.padding[0])
            oc, on = c, n
        else:
            oc, on, pairs, pnum, st = oracle.spconv_rulebook(c, n, layer.ksize, layer.stride, layer.padding,
                                                             layer.out_shape, maxV)
        assert st == 0 and g["num"] == on
        # the same set of output coordinates (a submanifold layer keeps the caller's rows; a strided layer numbers
        # its outputs in (z, y, x) order, the oracle in first-seen order) ...
        perm = match_rows(g["coors"][:on], oc[:on])
        if layer.subm:
            np.testing.assert_array_equal(perm, np.arange(on))
        else:
            gk = g["coors"][:on].astype(np.int64)
            lin = (gk[:, 1] * layer.out_shape[1] + gk[:, 2]) * layer.out_shape[2] + gk[:, 3]
            assert (np.diff(lin) > 0).all()
        assert not g["coors"][on:].any()
        # ... and the rulebook is identical after canonical sorting, with identical per-offset counts
        np.testing.assert_array_equal(g["pair_num"], pnum)
        np.testing.assert_array_equal(
            canonical_rulebook(g["pairs"], g["pair_num"], c, g["coors"][:on], layer.in_shape, layer.out_shape),
            canonical_rulebook(pairs, pnum, c, oc[:on], layer.in_shape, layer.out_shape))
        fin = f.astype(np.float16).astype(np.float32) if half else f
        want = oracle.conv_apply(fin, pairs, pnum, W, on, half_inputs=half)
        if scale is not None or relu:
            want = oracle.scale_shift_relu(want, scale, shift, relu, half_out=half)
        elif half:
            want = want.astype(np.float16).astype(np.float32)
        got = g["features"][:on][perm]
        assert rel_err(got, want) <= tol, rel_err(got, want)
        if not half:
            np.testing.assert_array_equal(got, want)   # same summation order as the oracle
        assert not g["features"][on:].any()


def test_subm_16_16_fp32_on_16000_active_voxels(gpu, oracle):
    """The single-layer case: 16,000 unique voxels in [41,1600,1408], N(0,1) features, N(0,1/sqrt(27*16)) weights."""
    S = gpu.synth
    coors = S.active_voxels()
    feat = S.normal_f32(S.SEED_BASE + 11, (16000, 16))
    W = S.normal_f32(S.SEED_BASE + 12, (27, 16, 16), 1.0 / np.sqrt(27 * 16))
    layer = _layer(gpu, True, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), (41, 1600, 1408))
    _check_layer(gpu, oracle, layer, [(coors, feat)], W, maxV=20000)


@pytest.mark.parametrize("cin,cout", [(4, 16), (16, 16), (16, 32), (32, 32), (32, 64), (64, 64)])
@pytest.mark.parametrize("dtype", [0, 1])
def test_subm_all_channel_pairs(gpu, oracle, cin, cout, dtype):
    rs = np.random.RandomState(cin * 100 + cout)
    shape = (6, 20, 24)
    frames = [(_random_coords(rs, n, shape), None) for n in (700, 150)]
    frames = [(c, rs.randn(len(c), cin).astype(np.float32)) for c, _ in frames]
    W = (rs.randn(27, cin, cout) / np.sqrt(9 * cin)).astype(np.float32)
    sc = (1 + 0.1 * rs.randn(cout)).astype(np.float32)
    sh = (0.1 * rs.randn(cout)).astype(np.float32)
    layer = _layer(gpu, True, cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape)
    _check_layer(gpu, oracle, layer, frames, W, dtype=dtype)
    _check_layer(gpu, oracle, layer, frames, W, sc, sh, True, dtype=dtype)


@pytest.mark.parametrize("ksize,pad,cin,cout,dtype", [(1, 0, 16, 16, 0), (1, 0, 32, 32, 1), (3, 0, 16, 16, 0),
                                                      (2, 0, 16, 32, 1)])
def test_subm_other_kernel_sizes_take_the_generic_map_path(gpu, oracle, ksize, pad, cin, cout, dtype):
    """Submanifold layers whose kernel is not 3x3x3 / padding 1 build their neighbour map from a flat coordinate
    table (one look-up per offset and output row) and their tile masks in a pass of their own; the reference's
    plugin accepts any cubic kernel (submConv3dlayer.cu:271-358 takes ksize and padding as run-time values)."""
    rs = np.random.RandomState(40 + ksize * 7 + cin)
    shape = (6, 20, 24)
    frames = [(_random_coords(rs, n, shape), None) for n in (800, 130)]
    frames = [(c, rs.randn(len(c), cin).astype(np.float32)) for c, _ in frames]
    W = (rs.randn(ksize ** 3, cin, cout) / np.sqrt(2 * cin)).astype(np.float32)
    layer = _layer(gpu, True, cin, cout, (ksize,) * 3, (1, 1, 1), (pad,) * 3, shape)
    _check_layer(gpu, oracle, layer, frames, W, dtype=dtype)


@pytest.mark.parametrize("cin,cout,dtype", [(3, 5, 0), (8, 24, 0), (24, 8, 1), (5, 40, 1), (128, 16, 0)])
def test_channel_counts_outside_the_schedule(gpu, oracle, cin, cout, dtype):
    """The reference's plugins take any in_channel / out_channel (submConv3dlayer.cu:479-518 loops over run-time
    counts); pairs that have no specialised kernel run on the run-time-shaped CUDA-core kernel, with the same
    parity bar: rulebook exact, fp32 bit-equal to the oracle's order of additions, fp16 within 1e-2."""
    rs = np.random.RandomState(cin * 131 + cout)
    shape = (6, 20, 24)
    frames = [(_random_coords(rs, n, shape), None) for n in (500, 90)]
    frames = [(c, rs.randn(len(c), cin).astype(np.float32)) for c, _ in frames]
    W = (rs.randn(27, cin, cout) / np.sqrt(9 * cin)).astype(np.float32)
    sc = (1 + 0.1 * rs.randn(cout)).astype(np.float32)
    sh = (0.1 * rs.randn(cout)).astype(np.float32)
    _check_layer(gpu, oracle, _layer(gpu, True, cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape), frames, W, sc, sh,
                 True, dtype=dtype)
    Ws = (rs.randn(27, cin, cout) / np.sqrt(4 * cin)).astype(np.float32)
    _check_layer(gpu, oracle, _layer(gpu, False, cin, cout, (3, 3, 3), (2, 2, 2), (1, 1, 1), shape), frames, Ws,
                 dtype=dtype, maxV=2048)


STRIDED = [
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (9, 22, 26), 16, 32),
    ((3, 3, 3), (2, 2, 2), (1, 1, 1), (7, 20, 24), 32, 64),
    ((3, 3, 3), (2, 2, 2), (0, 1, 1), (11, 20, 16), 64, 64),
    ((3, 1, 1), (2, 1, 1), (0, 0, 0), (5, 20, 16), 64, 64),
]


@pytest.mark.parametrize("K,S,P,shape,cin,cout", STRIDED)
@pytest.mark.parametrize("dtype", [0, 1])
def test_strided_layers_of_the_schedule(gpu, oracle, K, S, P, shape, cin, cout, dtype):
    rs = np.random.RandomState(sum(shape) + cin)
    frames = []
    for n in (900, 0, 37):
        c = _random_coords(rs, n, shape) if n else np.zeros((0, 4), np.int32)
        frames.append((c, rs.randn(len(c), cin).astype(np.float32)))
    W = (rs.randn(int(np.prod(K)), cin, cout) / np.sqrt(4 * cin)).astype(np.float32)
    layer = _layer(gpu, False, cin, cout, K, S, P, shape)
    _check_layer(gpu, oracle, layer, frames, W, dtype=dtype, maxV=4096)


def test_strided_full_resolution_shapes(gpu, oracle):
    """Layer 6 geometry at full size: [41,1600,1408] -> [21,800,704] on voxelised synthetic points."""
    S = gpu.synth
    _, coors, _, n, _ = oracle.voxelize(S.single_frame(), S.POINT_RANGE, S.VOXEL_SIZE, 20000)
    rs = np.random.RandomState(5)
    feat = rs.randn(n, 16).astype(np.float32)
    W = (rs.randn(27, 16, 32) * 0.05).astype(np.float32)
    layer = gpu.schedule.LAYERS[2]
    _check_layer(gpu, oracle, layer, [(coors[:n], feat)], W, maxV=60000)


def test_every_cell_active_tiny_grid(gpu, oracle):
    """Exhaustive neighbourhoods: all 4x6x5 cells active, borders included."""
    shape = (4, 6, 5)
    cells = np.arange(int(np.prod(shape)))
    c = np.zeros((len(cells), 4), np.int32)
    c[:, 1], c[:, 2], c[:, 3] = cells // 30, (cells // 5) % 6, cells % 5
    rs = np.random.RandomState(1)
    f = rs.randn(len(c), 16).astype(np.float32)
    W = rs.randn(27, 16, 16).astype(np.float32)
    _check_layer(gpu, oracle, _layer(gpu, True, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape), [(c, f)], W)
    _check_layer(gpu, oracle, _layer(gpu, False, 16, 32, (3, 3, 3), (2, 2, 2), (1, 1, 1), shape), [(c, f)],
                 rs.randn(27, 16, 32).astype(np.float32))


def test_output_overflow_sets_status_and_truncates(gpu, oracle):
    """More active outputs than max_voxels: the status bit is set, exactly max_voxels rows come back, they are the
    first max_voxels of the full output set in (z, y, x) order, and their features are those of the untruncated
    layer (the reference writes past its buffers in this situation)."""
    rs = np.random.RandomState(9)
    shape = (9, 22, 26)
    c = _random_coords(rs, 600, shape)
    f = rs.randn(len(c), 16).astype(np.float32)
    W = rs.randn(27, 16, 32).astype(np.float32)
    layer = _layer(gpu, False, 16, 32, (3, 3, 3), (2, 2, 2), (1, 1, 1), shape)
    res, maxV = _run_layer(gpu, layer, [(c, f)], W, maxV=640)
    oc, on, pairs, pnum, st = oracle.spconv_rulebook(c, len(c), layer.ksize, layer.stride, layer.padding,
                                                     layer.out_shape, 640)
    assert st & oracle.VOXEL_OVERFLOW and res[0]["status"] & gpu.STATUS_VOXEL_OVERFLOW
    assert res[0]["num"] == on == 640
    fc, fn, fpairs, fpnum, fst = oracle.spconv_rulebook(c, len(c), layer.ksize, layer.stride, layer.padding,
                                                        layer.out_shape, 8192)
    assert fst == 0 and fn > 640
    full = oracle.conv_apply(f, fpairs, fpnum, W, fn)
    lin = (fc[:fn, 1].astype(np.int64) * layer.out_shape[1] + fc[:fn, 2]) * layer.out_shape[2] + fc[:fn, 3]
    first = np.argsort(lin)[:640]
    np.testing.assert_array_equal(res[0]["coors"][:640], fc[first])
    np.testing.assert_array_equal(res[0]["features"][:640], full[first])


def test_bad_coordinate_is_reported_not_dereferenced(gpu):
    rs = np.random.RandomState(2)
    shape = (4, 6, 5)
    c = _random_coords(rs, 20, shape)
    c[3, 2] = 77   # y outside the grid
    f = rs.randn(len(c), 16).astype(np.float32)
    res, _ = _run_layer(gpu, _layer(gpu, True, 16, 16, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape), [(c, f)],
                        rs.randn(27, 16, 16).astype(np.float32))
    assert res[0]["status"] & gpu.STATUS_BAD_COORD


@pytest.mark.parametrize("cin,cout", [(32, 32), (64, 64)])
def test_more_row_groups_than_resident_blocks_fp16(gpu, oracle, cin, cout):
    """4 frames x 45,000 rows: 352 groups of 512 rows, more than a persistent grid holds at once, so blocks
    walk through several groups and their staging rings wrap many times."""
    rs = np.random.RandomState(77 + cin)
    shape = (10, 200, 176)
    frames = []
    for n in (45000, 44000, 45000, 30001):
        c = _random_coords(rs, n, shape)
        frames.append((c, rs.randn(len(c), cin).astype(np.float32)))
    W = (rs.randn(27, cin, cout) / np.sqrt(5 * cin)).astype(np.float32)
    layer = _layer(gpu, True, cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape)
    _check_layer(gpu, oracle, layer, frames, W, dtype=gpu.F16, maxV=45056)


def test_bounded_waits_run_out_report_and_leave_the_context_usable(gpu):
    """Time-out path of the tensor-core kernel, made on the host: with the library's test hook on, the kernel's
    weight streamer stays silent, the MMA issuers' bounded wait for the first weight block runs out, every block
    leaves through its abort path and the call reports SESSD_STATUS_TIMEOUT with the code of that wait. Nothing
    faults; the same call with the hook off then gives the result it gave before."""
    import torch

    rs = np.random.RandomState(5)
    shape, cin, cout, n, maxV = (10, 60, 60), 32, 32, 3000, 4096
    c = _random_coords(rs, n, shape)
    layer = _layer(gpu, True, cin, cout, (3, 3, 3), (1, 1, 1), (1, 1, 1), shape)
    feat = np.zeros((1, maxV, cin), np.float16)
    coors = np.zeros((1, maxV, 4), np.int32)
    feat[0, :len(c)] = rs.randn(len(c), cin).astype(np.float16)
    coors[0, :len(c)] = c
    coors[0, :, 0] = 0
    W = (rs.randn(27, cin, cout) / np.sqrt(5 * cin)).astype(np.float32)
    p = gpu.conv_params(layer, maxV)
    w = gpu.ConvWeights(p, W, None, None, False, gpu.F16)
    tf, tc = torch.from_numpy(feat).cuda(), torch.from_numpy(coors).cuda()
    tn = torch.tensor([len(c)], dtype=torch.int32, device="cuda")
    good = gpu.subm_conv(tf, tc, tn, p, w)
    assert good["status"] == 0
    want = good["features"].clone()
    assert gpu.lib().sessd_conv_weights_debug_withhold(w.handle, 1) == 0
    try:
        r = gpu.subm_conv(tf, tc, tn, p, w, keep_workspace=True)
    finally:
        gpu.lib().sessd_conv_weights_debug_withhold(w.handle, 0)
    assert r["status"] & gpu.STATUS_TIMEOUT
    where = int(r["workspace"][4:8].view(torch.int32)[0])
    assert where & 15 == 5                    # an MMA issuer waiting for a weight block
    again = gpu.subm_conv(tf, tc, tn, p, w)
    assert again["status"] == 0 and torch.equal(again["features"], want)
    w.close()
