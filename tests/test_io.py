"""DAPHNE's binary matrix format (.dbdf): the device-direct reader/writer against the reference's own serializer.

CPU: the committed fixtures (written by the reference, tests/golden/make_dbdf_fixtures.py) have the documented layout
(doc/BinaryFormat.md) and the reference reads them back.  GPU: files written by the reference are read by
db2_readDaphne bit for bit, files written by db2_writeDaphne are byte-identical to the reference's and read back by the
reference; a file larger than the two staging buffers takes the pipelined path; malformed files are refused."""
import struct
from pathlib import Path

import numpy as np
import pytest

from tests.golden.make_dbdf_fixtures import fixtures

GOLD = Path(__file__).parent / "golden"
VT_CODE = {np.dtype(np.float64): 7, np.dtype(np.float32): 6, np.dtype(np.int64): 2}


def _parse(path):
    b = Path(path).read_bytes()
    ver, dt, rows, cols, vt = struct.unpack_from("<BBQQB", b, 0)
    rx, cx, brows, bcols, bt, bvt = struct.unpack_from("<QQIIBB", b, 19)
    return dict(ver=ver, dt=dt, rows=rows, cols=cols, vt=vt, rx=rx, cx=cx, brows=brows, bcols=bcols, bt=bt, bvt=bvt,
                payload=b[45:])


def test_fixtures_have_the_documented_layout():
    for name, arr in fixtures().items():
        h = _parse(GOLD / name)
        assert (h["ver"], h["dt"], h["rows"], h["cols"]) == (1, 1, arr.shape[0], arr.shape[1])
        assert h["vt"] == h["bvt"] == VT_CODE[arr.dtype] and (h["rx"], h["cx"], h["bt"]) == (0, 0, 1)
        assert (h["brows"], h["bcols"]) == arr.shape and h["payload"] == arr.tobytes()


def test_reference_reads_its_fixtures_back():
    from oracle import refkernels as ref
    if not ref.available():
        pytest.skip("oracle/_ref not built")
    for name, arr in fixtures().items():
        got = ref.readDaphne(GOLD / name, arr.dtype)
        assert got.dtype == arr.dtype and np.array_equal(got, arr)


@pytest.mark.gpu
def test_read_the_references_files(ctx, tmp_path):
    import daphne_b200.kernels as k
    for name, arr in fixtures().items():
        got = k.readDaphne(ctx, GOLD / name).to_numpy()
        assert got.dtype == arr.dtype and np.array_equal(got, arr), name
    from oracle import refkernels as ref
    if ref.available():
        rng = np.random.default_rng(41)
        for shape, dt in [((1, 1), np.float64), ((1000, 37), np.float64), ((513, 129), np.float32), ((77, 5), np.int64)]:
            a = (rng.standard_normal(shape) * 1e3).astype(dt)
            ref.writeDaphne(a, tmp_path / "a.dbdf")
            got = k.readDaphne(ctx, tmp_path / "a.dbdf").to_numpy()
            assert got.dtype == a.dtype and np.array_equal(got, a), (shape, dt)


@pytest.mark.gpu
def test_write_is_byte_identical_and_read_back_by_the_reference(ctx, tmp_path):
    import daphne_b200.kernels as k
    from oracle import refkernels as ref
    rng = np.random.default_rng(42)
    for shape, dt in [((3, 4), np.float64), ((2000, 33), np.float64), ((100, 7), np.float32), ((9, 9), np.int64)]:
        a = (rng.standard_normal(shape) * 100).astype(dt)
        k.writeDaphne(k.DenseMatrix.from_numpy(ctx, a), tmp_path / "ours.dbdf")
        h = _parse(tmp_path / "ours.dbdf")
        assert (h["rows"], h["cols"], h["vt"]) == (shape[0], shape[1], VT_CODE[np.dtype(dt)]) and h["payload"] == a.tobytes()
        if ref.available():
            ref.writeDaphne(a, tmp_path / "ref.dbdf")
            assert (tmp_path / "ours.dbdf").read_bytes() == (tmp_path / "ref.dbdf").read_bytes()
            assert np.array_equal(ref.readDaphne(tmp_path / "ours.dbdf", dt), a)
    # a row view (leading dimension > columns) is written densely
    big = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((500, 16)))
    k.writeDaphne(big.slice_rows(100, 300), tmp_path / "view.dbdf")
    assert np.array_equal(k.readDaphne(ctx, tmp_path / "view.dbdf").to_numpy(), big.to_numpy()[100:300])


@pytest.mark.gpu
def test_large_file_goes_through_both_staging_buffers(ctx, tmp_path):
    import daphne_b200.kernels as k
    a = np.random.default_rng(43).standard_normal((2_500_000, 8))  # 160 MB: three pieces of 64 MiB
    A = k.DenseMatrix.from_numpy(ctx, a)
    k.writeDaphne(A, tmp_path / "big.dbdf")
    B = k.readDaphne(ctx, tmp_path / "big.dbdf")
    assert np.array_equal(B.to_numpy(), a)
    assert abs(k.aggAll(k.AggOpCode.SUM, B) - a.sum()) <= 1e-9 * np.abs(a).sum()


@pytest.mark.gpu
def test_malformed_files_are_refused(ctx, tmp_path):
    import daphne_b200.kernels as k
    good = (GOLD / "ref_dense_3x4_f64.dbdf").read_bytes()
    cases = {"version": bytes([2]) + good[1:], "frame": good[:1] + bytes([3]) + good[2:],
             "value type": good[:18] + bytes([0]) + good[19:], "truncated": good[:-8], "header only": good[:20],
             "sparse block": good[:43] + bytes([2]) + good[44:]}
    for what, data in cases.items():
        p = tmp_path / "bad.dbdf"
        p.write_bytes(data)
        with pytest.raises(k.Db2Error):
            k.readDaphne(ctx, p)
    with pytest.raises(k.Db2Error):
        k.readDaphne(ctx, tmp_path / "does_not_exist.dbdf")
