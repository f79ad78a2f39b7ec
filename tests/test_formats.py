"""Host-side readers and writers of the reference's on-disk formats (weight files, batch-norm folding, point
cloud files) against the pure-Python restatement in oracle/formats.py. No GPU needed."""
import numpy as np
import pytest

from oracle import formats as oracle_formats


def _bits(a):
    return np.asarray(a, np.float32).view(np.uint32)


def _blobs(seed=3):
    rng = np.random.default_rng(seed)
    special = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, 1e-45, -1e-45, 3.4028235e38, 1.17549435e-38], np.float32)
    payload = np.array([0x7FC00001, 0xFFC12345, 0x7F800001, 0x00000001, 0x80000000], np.uint32).view(np.float32)
    return [
        ("backbone.middle_conv.0.weight", rng.standard_normal((27, 4, 16)).astype(np.float32)),
        ("backbone.middle_conv.1.weight", rng.uniform(0.5, 1.5, 16).astype(np.float32)),
        ("backbone.middle_conv.1.num_batches_tracked", np.array([12345.0], np.float32)),
        ("special.values", special),
        ("nan.payloads", payload),
        ("empty.blob", np.zeros((0,), np.float32)),
        ("random.bits", rng.integers(0, 2 ** 32, 4099, dtype=np.uint64).astype(np.uint32).view(np.float32)),
    ]


def test_exporter_format_file_loads_bit_exact(pkg, tmp_path):
    blobs = _blobs()
    path = tmp_path / "model.wts"
    oracle_formats.write_wts(path, blobs)
    w = pkg.formats.Wts(path)
    assert len(w) == len(blobs)
    for i, (name, want) in enumerate(blobs):
        got_name, got = w.entry(i)
        assert got_name == name and got.dtype == np.float32
        assert np.array_equal(_bits(got), _bits(want.reshape(-1)))
        assert np.array_equal(_bits(w.find(name)), _bits(want.reshape(-1)))
    assert w.find("not.there") is None
    with pytest.raises(pkg.SessdError):
        w.entry(len(blobs))
    w.close()


def test_saved_file_is_the_exporters_bytes_and_reads_back(pkg, tmp_path):
    blobs = _blobs(seed=4)
    ours, theirs = tmp_path / "ours.wts", tmp_path / "theirs.wts"
    pkg.formats.save_wts(ours, blobs)
    oracle_formats.write_wts(theirs, blobs)
    assert ours.read_bytes() == theirs.read_bytes()
    back = oracle_formats.read_wts(ours)              # the reference's reader, restated
    assert list(back) == [k for k, _ in blobs]
    for name, want in blobs:
        assert np.array_equal(_bits(back[name]), _bits(want.reshape(-1)))


def test_repeated_name_keeps_the_last_blob(pkg, tmp_path):
    path = tmp_path / "dup.wts"
    oracle_formats.write_wts(path, [("a", [1.0, 2.0]), ("b", [3.0]), ("a", [4.0, 5.0, 6.0])])
    w = pkg.formats.Wts(path)
    assert len(w) == 3 and w.entry(0)[1].tolist() == [1.0, 2.0]
    assert w.find("a").tolist() == [4.0, 5.0, 6.0] == oracle_formats.read_wts(path)["a"].tolist()


def test_white_space_and_hex_forms_the_stream_reader_accepts(pkg, tmp_path):
    path = tmp_path / "loose.wts"
    path.write_text("  2\r\n\tx   3\n3F800000\n 0x40000000 c0400000 \n\ny 1 0\n")
    w = pkg.formats.Wts(path)
    assert w.find("x").tolist() == [1.0, 2.0, -3.0] and w.find("y").tolist() == [0.0]


@pytest.mark.parametrize("text", ["", "0\n", "x\n", "1\nname\n", "1\nname 3 3f800000 3f800000\n", "1\nname 1 3g800000\n",
                                  "1\nname 1 13f800000\n", "2\nname 1 3f800000\n", "1\nname -1\n",
                                  "1\nname 4000000000 0\n"])
def test_malformed_files_are_refused(pkg, tmp_path, text):
    path = tmp_path / "bad.wts"
    path.write_text(text)
    with pytest.raises(pkg.SessdError):
        pkg.formats.Wts(path)


def test_missing_file_and_bad_names(pkg, tmp_path):
    with pytest.raises(pkg.SessdError):
        pkg.formats.Wts(tmp_path / "absent.wts")
    with pytest.raises(pkg.SessdError):
        pkg.formats.save_wts(tmp_path / "x.wts", [("has space", [1.0])])
    with pytest.raises(pkg.SessdError):
        pkg.formats.save_wts(tmp_path / "x.wts", [])
    with pytest.raises(pkg.SessdError):
        pkg.formats.save_wts(tmp_path / "no_such_dir" / "x.wts", [("a", [1.0])])


def test_fold_batchnorm_matches_the_builders_arithmetic(pkg):
    rng = np.random.default_rng(9)
    for n in (1, 16, 64, 257):
        g = rng.uniform(0.2, 2.0, n).astype(np.float32)
        b = rng.standard_normal(n).astype(np.float32)
        m = rng.standard_normal(n).astype(np.float32)
        v = rng.uniform(1e-4, 4.0, n).astype(np.float32)
        v[0] = 0.0                                   # a dead channel: only eps under the root
        sc, sh = pkg.formats.fold_batchnorm(g, b, m, v, 1e-5)
        want_sc, want_sh = oracle_formats.fold_batchnorm(g, b, m, v, 1e-5)
        # fp32 throughout on both sides; 1e-6 relative leaves room for the square root's last bit only
        assert np.allclose(sc, want_sc, rtol=1e-6, atol=0) and np.allclose(sh, want_sh, rtol=1e-6, atol=1e-6)


def test_point_cloud_file(pkg, tmp_path):
    rng = np.random.default_rng(11)
    pts = rng.standard_normal((1000, 4)).astype(np.float32)
    path = tmp_path / "000000.bin"
    pts.tofile(path)
    for cap in (1000, 1500):
        got, n = pkg.formats.load_points(path, cap)
        want, want_n = oracle_formats.read_points(path, cap)
        assert n == want_n == 1000 and np.array_equal(_bits(got), _bits(want))
    with pytest.raises(pkg.SessdError):              # does not fit: the reference exits
        pkg.formats.load_points(path, 999)
    assert oracle_formats.read_points(path, 999) is None
    ragged = tmp_path / "ragged.bin"                 # a trailing partial record is copied but not counted
    ragged.write_bytes(pts[:10].tobytes() + b"\x01\x02\x03\x04\x05")
    got, n = pkg.formats.load_points(ragged, 16)
    want, want_n = oracle_formats.read_points(ragged, 16)
    assert n == want_n == 10 and np.array_equal(_bits(got), _bits(want))
    empty = tmp_path / "empty.bin"
    empty.write_bytes(b"")
    got, n = pkg.formats.load_points(empty, 4)
    assert n == 0 and not got.any()
    with pytest.raises(pkg.SessdError):
        pkg.formats.load_points(tmp_path / "absent.bin", 4)


def test_neck_blobs_survive_a_weight_file_and_drive_the_fp32_restatement(pkg, tmp_path):
    """Random-init neck/head blobs under the reference's state-dict names: written and read back bit for bit,
    and accepted by the CPU restatement of the layer graph, whose outputs have the plugin input layout."""
    from oracle import neck as oracle_neck

    blobs = pkg.detector.random_neck_weights()
    assert len(blobs) == 14 * 5 + 4 * 2
    path = tmp_path / "neck.wts"
    pkg.formats.save_wts(path, blobs)
    w = pkg.formats.Wts(path)
    back = {}
    for name, want in blobs.items():
        got = w.find(name)
        assert np.array_equal(_bits(got), _bits(want.reshape(-1)))
        back[name] = got
    rng = np.random.default_rng(2)
    bev = np.zeros((1, 128, 202, 178), np.float32)
    bev[:, :, 61:101, 41:91] = rng.random((1, 128, 40, 50), dtype=np.float32) * (rng.random((1, 1, 40, 50)) < 0.2)
    out = oracle_neck.neck_and_head(bev, back)
    assert out["features"].shape == (1, 128, 200, 176)
    assert [out[k].shape for k in ("box", "cls", "iou", "dir")] == [(1, 70400, 7), (1, 70400, 1), (1, 70400, 1), (1, 70400, 2)]
    # far from the occupied patch every pixel of the same parity (the stride-2 transposed convolutions) sees
    # the same empty neighbourhood and gets the same numbers, which pins the (pixel, anchor) order of the reshape
    box = out["box"].reshape(200, 176, 2, 7)
    assert np.allclose(box[150, 150], box[150, 152], atol=1e-6) and np.allclose(box[150, 150], box[152, 150], atol=1e-6)
    assert not np.allclose(box[150, 150, 0], box[150, 150, 1])
    assert not np.allclose(box[80, 60], box[150, 150])


def test_committed_weight_file_fixture(pkg):
    """tests/golden/tiny.wts was written by the restated exporter loop (tests/golden/make_golden.py); the
    library's reader must return the bit patterns the generator put in, and re-saving must give the file back."""
    import os
    import sys

    golden = os.path.join(os.path.dirname(__file__), "golden")
    sys.path.insert(0, golden)
    import make_golden

    path = os.path.join(golden, "tiny.wts")
    w = pkg.formats.Wts(path)
    blobs = make_golden.tiny_wts_blobs()
    assert len(w) == len(blobs)
    for i, (name, want) in enumerate(blobs):
        got_name, got = w.entry(i)
        assert got_name == name and np.array_equal(_bits(got), _bits(want.reshape(-1)))
    assert open(path, "rb").read().startswith(b"4\nbackbone.middle_conv.0.weight 24  ")
