"""Regenerates the golden fixtures in this directory.

Run from the repository root on a machine where the reference sources are mounted and
`make -C oracle ref` has built the harness around the reference's own converter:

    python tests/golden/make_golden.py

format_ref_{fp16,tf32}.npz hold inputs and the output of the reference's CSR2BTCFNOBITMAP
(src/utils/convert.h:146-225, 8x16 / 8x8 windows) for a hand-written 20x40 matrix and two
random matrices.  format_ref_bitmap_{fp16,tf32}.npz hold the output of the reference's CSR2BTCF
(convert.h:22-139) and BTCF2GBTCF (convert.h:232-276) for the same matrices plus one with windows
long enough to be split into groups.  sample.mtx / short.mtx are small MatrixMarket files written
here, mtx_ref_{fp16,tf32}.npz what the reference's load_matrix (src/utils/load.h:152-322) reads
from them.  synth_checksums.json pins the synthetic-input generators.
"""
import hashlib
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import oracle  # noqa: E402
from cases import random_csr  # noqa: E402
from hopper_spmm_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def hand_example():
    ent = [(1, 1), (1, 33), (2, 5), (3, 17), (9, 2), (9, 40), (10, 2), (20, 7), (20, 8)]  # 1-based
    rows, cols = 20, 40
    rp = np.zeros(rows + 1, np.uint32)
    for r, _ in ent:
        rp[r] += 1
    rp = np.cumsum(rp).astype(np.uint32)
    ci = np.array([c - 1 for _, c in ent], np.uint32)
    vals = np.arange(1, len(ent) + 1, dtype=np.float32)
    return rows, cols, rp, ci, vals


SAMPLE_MTX = """%%MatrixMarket matrix coordinate real general
% a 9 x 12 matrix; entries in no particular order
%
9 12 14
3 4 0.5
1 1 -1.25
9 12 3.0e-2
3 1 7
this line is not an entry
1 12 0.333333

5 6 65504
5 2 1e-8
2 7 -0.1
   4   4   2.5
9 1 1
7 7 -3
3 9 0.0009765625
6 3 100.1
8 8 4
1 2 99
"""

SHORT_MTX = """%%MatrixMarket matrix coordinate real general
4 5 6
2 3 1.5
1 5 -2
4 1 0.25
"""


def main():
    with open(os.path.join(HERE, "sample.mtx"), "w") as fh:
        fh.write(SAMPLE_MTX)
    with open(os.path.join(HERE, "short.mtx"), "w") as fh:
        fh.write(SHORT_MTX)
    for flavour, dt in (("fp16", np.float16), ("tf32", np.float32)):
        out = {}
        cases = {"hand": hand_example(),
                 "rand_a": random_csr(203, 517, 0.03, 1, dt, empty_rows=[(40, 60)]),
                 "rand_b": random_csr(64, 33, 0.2, 2, dt, dense_rows=[5])}
        for name, (rows, cols, rp, ci, v) in cases.items():
            v = v.astype(dt)
            f = oracle.ref_convert(flavour, rows, cols, rp, ci, v)
            out.update({f"{name}_shape": np.array([rows, cols]), f"{name}_row_ptr": rp, f"{name}_col_idx": ci,
                        f"{name}_values": v, f"{name}_rowOffset": f.rowOffset, f"{name}_tcA2B": f.tcA2B,
                        f"{name}_data": f.data, f"{name}_rowIdx": f.rowIdx,
                        f"{name}_window": np.array([f.row_window, f.col_window])})
        np.savez_compressed(os.path.join(HERE, f"format_ref_{flavour}.npz"), **out)

        out = {}
        cases["wide"] = random_csr(40, 3000, 0.3, 3, dt, empty_rows=[(8, 16)])
        for name, (rows, cols, rp, ci, v) in cases.items():
            v = v.astype(dt)
            f, (go, gr, at) = oracle.ref_convert_bitmap(flavour, rows, cols, rp, ci, v)
            out.update({f"{name}_shape": np.array([rows, cols]), f"{name}_row_ptr": rp, f"{name}_col_idx": ci,
                        f"{name}_values": v, f"{name}_rowOffset": f.rowOffset, f"{name}_nnzOffset": f.nnzOffset,
                        f"{name}_tcA2B": f.tcA2B, f"{name}_tcBit": f.tcBit, f"{name}_data": f.data,
                        f"{name}_rowIdx": f.rowIdx, f"{name}_window": np.array([f.row_window, f.col_window]),
                        f"{name}_groupOffset": go, f"{name}_group_rowIdx": gr, f"{name}_atomic": at})
        np.savez_compressed(os.path.join(HERE, f"format_ref_bitmap_{flavour}.npz"), **out)

        out = {}
        for name in ("sample", "short"):
            rows, cols, rp, ci, v = oracle.ref_load_matrix(flavour, os.path.join(HERE, f"{name}.mtx"))
            out.update({f"{name}_shape": np.array([rows, cols]), f"{name}_row_ptr": rp, f"{name}_col_idx": ci,
                        f"{name}_values": v})
        np.savez_compressed(os.path.join(HERE, f"mtx_ref_{flavour}.npz"), **out)

    sums = {}
    for name, k in (("uniform_4096_fp16", 0), ("blocks_16384_tf32", 2), ("rmat20_gnn_fp16", 6),
                    ("pruned_llm_fp16", 4), ("rmat24_sharded_fp16", 10)):
        csr, B = synth.make_config(name, 0, "cpu", k)
        rp, ci, v = csr.numpy()
        h = hashlib.sha256()
        for a in (rp, ci):
            h.update(np.ascontiguousarray(a).tobytes())
        sums[f"{name}/{k}"] = {"rows": csr.rows, "cols": csr.cols, "nnz": csr.nnz, "structure_sha256": h.hexdigest(),
                               "values_sum": float(np.asarray(v, np.float64).sum()),
                               "B_sum": float(B.double().sum())}
    with open(os.path.join(HERE, "synth_checksums.json"), "w") as fh:
        json.dump(sums, fh, indent=1, sort_keys=True)


if __name__ == "__main__":
    main()
