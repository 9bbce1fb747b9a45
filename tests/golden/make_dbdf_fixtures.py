"""Writes the .dbdf fixtures with the REFERENCE's own serializer (oracle/_ref, built from a DAPHNE source tree):

    python tests/golden/make_dbdf_fixtures.py

ref_dense_3x4_f64.dbdf   3 x 4 double   values i + 0.5
ref_dense_5x3_f32.dbdf   5 x 3 float    values 0.25 * i - 1
ref_dense_4x2_i64.dbdf   4 x 2 int64    values (i - 3) * 10**12
The files are committed (< 200 bytes each) so that the reader is checked against the reference's bytes on machines
without a DAPHNE checkout."""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parents[1]))


def fixtures():
    return {"ref_dense_3x4_f64.dbdf": (np.arange(12, dtype=np.float64) + 0.5).reshape(3, 4),
            "ref_dense_5x3_f32.dbdf": (0.25 * np.arange(15, dtype=np.float32) - 1).reshape(5, 3),
            "ref_dense_4x2_i64.dbdf": ((np.arange(8, dtype=np.int64) - 3) * 10 ** 12).reshape(4, 2)}


if __name__ == "__main__":
    from oracle import refkernels as ref
    assert ref.available(), "oracle/_ref is not built (make -C oracle ref)"
    for name, arr in fixtures().items():
        ref.writeDaphne(arr, HERE / name)
        print(name, (HERE / name).stat().st_size, "bytes")
