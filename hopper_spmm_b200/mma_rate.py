"""Prints what one tcgen05.mma of the SpMM's shape costs on this GPU (SM clocks per MMA).

    python -m hopper_spmm_b200.mma_rate

One condensed tile is one MMA per 128-feature chunk, so these figures are the tensor-pipe floor of
the format: time per tile and SM cannot fall below the two-issuer figure whatever the tile's fill.
"""
import ctypes as C

from . import _capi


def measure(tf32: bool, m: int, n: int, issuers: int, count: int = 512, device: int = 0):
    out = (C.c_double * 2)()
    st = _capi.lib().b200spmm_kat_umma_rate(int(tf32), m, n, count, issuers, out, device)
    if st != 0:
        raise RuntimeError(_capi.lib().b200spmm_status_string(st).decode())
    return out[0], out[1]


def main() -> None:
    print("dtype  M    N  issuers  clocks/MMA (issue)  clocks/MMA (issue + drain)  per MMA and SM")
    for tf32 in (False, True):
        for m in (128, 64):
            for n in (16, 64, 256):
                for issuers in (1, 2):
                    a, b = measure(tf32, m, n, issuers)
                    print(f"{'tf32' if tf32 else 'fp16'}  {m:3d}  {n:3d}  {issuers:7d}  {a:18.1f}  {b:26.1f}  {b / issuers:14.1f}")


if __name__ == "__main__":
    main()
