"""Tolerance rules of the end-to-end parity tests.

The stated tolerances are rel <= 1e-2 for fp16 inputs with fp32 accumulation and rel <= 5e-3
for tf32.  Two measurements are applied to every result:

  * the reference's own pass/fail rule (verify_result, src/tf32.cu:38-71: relative to |ref|
    above 1e-6, absolute 1e-5 below) against an oracle that sees the inputs as the tensor core
    sees them (fp16 exactly; tf32 = fp32 with the low 13 mantissa bits dropped).  Cancellation
    can push single elements past a relative bound, so at most 1e-3 of the elements may fail it;
  * the error relative to the magnitude sum  sum_k |a_k| |b_kj|  against the plain fp32 oracle,
    which must stay below the stated tolerance for EVERY element.
"""
import numpy as np

import oracle

TOL = {np.dtype(np.float16): 1e-2, np.dtype(np.float32): 5e-3}


def check(got, rows, rp, ci, v, B, tf32_mode=1, threads=0):
    tol = TOL[np.dtype(B.dtype)]
    got = np.asarray(got, np.float32)
    assert np.isfinite(got).all(), "non-finite values in C"
    ref = oracle.spmm_csr(rows, rp, ci, v, B, n_threads=threads)
    mag = oracle.spmm_csr(rows, rp, ci, np.abs(v), np.abs(B), n_threads=threads)
    err = np.abs(got - ref)
    scaled = float((err / np.maximum(mag, 1e-30))[mag > 0].max()) if (mag > 0).any() else 0.0
    assert float(err[mag == 0].max()) == 0.0 if (mag == 0).any() else True, "rows without entries must be zero"
    assert scaled <= tol, f"error relative to the magnitude sum {scaled:.3e} > {tol}"
    tight = ref if B.dtype == np.float16 else oracle.spmm_csr(rows, rp, ci, v, B, n_threads=threads, tf32_mode=tf32_mode)
    bad, max_rel, max_abs = oracle.compare(got, tight, tol)
    # (a result of fewer than a thousand elements may hold one such element)
    assert bad <= max(1.0, 1e-3 * got.size), f"{bad} of {got.size} elements fail the reference's rule (max rel {max_rel:.3e})"
    return {"scaled_err": scaled, "rule_failures": bad, "max_rel": max_rel, "max_abs": max_abs}


def rows_subset(rp, ci, v, ranges):
    """CSR (row_ptr rebased to zero) of the rows in `ranges`, a list of [begin, end) pairs, stacked in order."""
    rp = np.asarray(rp)
    counts, cols, vals = [], [], []
    for a, b in ranges:
        lo, hi = int(rp[a]), int(rp[b])
        counts.append(np.diff(rp[a:b + 1].astype(np.int64)))
        cols.append(ci[lo:hi])
        vals.append(v[lo:hi])
    sub_rp = np.concatenate([[0], np.cumsum(np.concatenate(counts))]).astype(np.uint32)
    return sub_rp, np.concatenate(cols), np.concatenate(vals)


def check_rows(got_rows, rp, ci, v, B, ranges, threads=0):
    """The same two measurements on a sample of rows: `got_rows` holds C's rows of `ranges`, stacked in
    order.  For results too large to recompute whole on the host; the sample should hold the heaviest
    rows, the first window and the last one."""
    sub_rp, sub_ci, sub_v = rows_subset(rp, ci, v, ranges)
    stats = check(got_rows, len(sub_rp) - 1, sub_rp, sub_ci, sub_v, B, threads=threads)
    stats["checked_rows"] = len(sub_rp) - 1
    return stats
