"""CPU restatement of the reference's NVFP4 (E2M1 codes + one E4M3 scale per 16) quantiser.

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``; never by the product.

What it restates (paths inside the reference project):

* CUDA kernels ``sageattention3_blackwell/sageattn4/quantization/fp4_quantization_4d.cu``
  ``scaled_fp4_quant_kernel`` (:164-284) and ``scaled_fp4_quant_trans_kernel`` (:286-412):
  per 16 consecutive elements ``absmax`` (taken in bf16), ``SF = e4m3(absmax / 6)``,
  ``inv = (SF == 0) ? 0 : 1 / SF``, ``code = e2m1_rn(x * inv)``; element 0 of a pair goes to
  the low nibble (``fp32_vec_to_e2m1`` :77-99); scale bytes land in a 64-row swizzled atom
  (:268-275, :393-403); the K variant permutes rows inside each 32-row group
  (``permute_token_within_block`` :146-162).
* Python emulation ``sageattention3_blackwell/sageattn4/api.py:77-110``
  (``round_to_blockscaled_fp4`` / ``round_to_token_blockscaled_fp4``), whose tie handling
  (:100-103) documents the intended round-half-to-even on the E2M1 grid.

Pinning: ``tests/test_oracle_golden.py`` checks this file against vectors produced by the
reference's own Python emulation (``tests/golden/make_golden.py``), and the ``-m gpu`` tests
check it against the reference's own CUDA kernels compiled for sm_100a (``oracle/build_ref.py``).

Two arithmetic modes:

``exact``   IEEE fp32 ``absmax / 6`` and ``1 / SF`` - what the Python emulation does.
``device``  the reference CUDA build uses ``--use_fast_math``, so both divisions are the
            GPU's approximate ``div.approx.ftz`` / ``rcp.approx.ftz``.  Both are functions of
            very few input bits (absmax is a bf16; SF is one of 127 E4M3 values), so their
            results are tabulated once on a B200 (``tests/golden/device_tables.npz``, produced
            by ``tests/golden/make_device_tables.py``) and looked up here.  With the tables the
            CPU result is bit-identical to the reference CUDA kernel.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
_E2M1_MID = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)

_TABLES = Path(__file__).resolve().parent.parent / "tests" / "golden" / "device_tables.npz"


def _e4m3_table() -> np.ndarray:
    """Value of every non-negative finite E4M3 (fn) code 0..126 (code 127 is NaN)."""
    codes = np.arange(127)
    e = codes >> 3
    m = codes & 7
    sub = (m / 8.0) * 2.0 ** -6
    nor = (1.0 + m / 8.0) * 2.0 ** (e.astype(np.float64) - 7)
    return np.where(e == 0, sub, nor).astype(np.float64)


E4M3_VALUES = _e4m3_table()                       # float64, exact
_E4M3_MID = (E4M3_VALUES[:-1] + E4M3_VALUES[1:]) / 2.0


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """``cvt.rn.satfinite.e4m3x2.f32`` for non-negative inputs: nearest, ties to even code,
    saturating at 448 (code 126).  Returns uint8 codes."""
    x64 = np.asarray(x, dtype=np.float64)
    idx = np.searchsorted(_E4M3_MID, x64, side="left")          # midpoints strictly below x
    idx = np.minimum(idx, 126)
    tie = (idx < 126) & (x64 == _E4M3_MID[np.minimum(idx, 125)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    return idx.astype(np.uint8)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    return E4M3_VALUES[np.asarray(code, dtype=np.int64) & 0x7F].astype(np.float32)


def e2m1_encode(y: np.ndarray) -> np.ndarray:
    """``cvt.rn.satfinite.e2m1x2.f32`` for one value: 4-bit code, bit 3 = sign (kept for
    zero results too), magnitude rounded to nearest with ties to the even code, saturating at 6."""
    y = np.asarray(y, dtype=np.float32)
    a = np.abs(y)
    idx = np.searchsorted(_E2M1_MID, a, side="left")
    idx = np.minimum(idx, 7)
    tie = (idx < 7) & (a == _E2M1_MID[np.minimum(idx, 6)])
    idx = np.where(tie & (idx % 2 == 1), idx + 1, idx)
    return (idx | (np.signbit(y).astype(np.int64) << 3)).astype(np.uint8)


def e2m1_decode(nib: np.ndarray) -> np.ndarray:
    nib = np.asarray(nib, dtype=np.int64)
    mag = E2M1_VALUES[nib & 7]
    return np.where(nib & 8, -mag, mag).astype(np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bit pattern (round to nearest even), as uint16."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


_device_tables = None


def device_tables():
    """(sf_of_absmax[32768] uint8, inv_of_sf[128] float32) measured on a B200, or None."""
    global _device_tables
    if _device_tables is None and _TABLES.exists():
        z = np.load(_TABLES)
        _device_tables = (z["sf_of_absmax"].astype(np.uint8), z["inv_of_sf"].astype(np.float32))
    return _device_tables


def quantize_nvfp4(x: np.ndarray, mode: str = "exact"):
    """Quantise along the last axis (length multiple of 16).

    ``x`` holds bf16-representable fp32 values.  Returns ``(codes, sf)`` with ``codes`` uint8
    ``[..., n/2]`` (element 2i in the low nibble of byte i) and ``sf`` uint8 E4M3 ``[..., n/16]``.
    Follows fp4_quantization_4d.cu:211-251.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    assert n % 16 == 0
    blk = x.reshape(*x.shape[:-1], n // 16, 16)
    amax = np.abs(blk).max(axis=-1)                                   # bf16-representable
    if mode == "device":
        tabs = device_tables()
        if tabs is None:
            raise FileNotFoundError(f"device tables missing: {_TABLES}")
        sf = tabs[0][to_bf16_bits(amax) & 0x7FFF]
        inv = tabs[1][sf]
    elif mode == "exact":
        sf = e4m3_encode(amax / np.float32(6.0))
        sfv = e4m3_decode(sf)
        with np.errstate(divide="ignore"):
            inv = np.where(sfv == 0, np.float32(0), np.float32(1.0) / sfv).astype(np.float32)
    else:
        raise ValueError(mode)
    y = blk * inv[..., None]                                          # fp32 multiply
    nib = e2m1_encode(y).reshape(*x.shape[:-1], n // 2, 2)
    codes = (nib[..., 0] | (nib[..., 1] << 4)).astype(np.uint8)
    return codes, sf


def dequantize_nvfp4(codes: np.ndarray, sf: np.ndarray) -> np.ndarray:
    codes = np.asarray(codes, dtype=np.uint8)
    lo = e2m1_decode(codes & 0xF)
    hi = e2m1_decode(codes >> 4)
    v = np.stack([lo, hi], axis=-1).reshape(*codes.shape[:-1], codes.shape[-1] * 2)
    s = np.repeat(e4m3_decode(sf), 16, axis=-1)
    return (v * s).astype(np.float32)


def fake_quant(x: np.ndarray, mode: str = "exact") -> np.ndarray:
    """quantise + dequantise; equals api.py:77-106 ``round_to_blockscaled_fp4`` in fp32."""
    return dequantize_nvfp4(*quantize_nvfp4(x, mode))


# ---------------------------------------------------------------------------------------------
# Storage layouts of the reference kernels (needed to compare with their raw output buffers)
# ---------------------------------------------------------------------------------------------

def ref_k_row_permutation() -> np.ndarray:
    """perm[p] = input token (within a 128-row block) that the reference K kernel writes to output
    row p (fp4_quantization_4d.cu:146-162)."""
    p = np.arange(128)
    r = p % 32
    return (p // 32) * 32 + (r // 8) * 2 + ((r % 8) // 2) * 8 + (r % 8) % 2


def ref_sf_offset(row: np.ndarray, col: np.ndarray, row_stride: int) -> np.ndarray:
    """Byte offset, inside one (batch, head) slab, of the scale for (row, 16-block col) in the
    reference's 64-row scale atom (fp4_quantization_4d.cu:268-275).  ``row_stride`` is the
    number of scale bytes per row (= blocks per row)."""
    row = np.asarray(row)
    col = np.asarray(col)
    base = (row // 64) * 64 * row_stride
    r = row % 64
    return base + (col // 4) * 256 + (col % 4) + (r // 16) * 4 + (r % 16) * 16


def ref_sf_unswizzle(raw: np.ndarray) -> np.ndarray:
    """raw: uint8 [..., rows, cols] buffer as written by the reference kernels -> logical
    [..., rows, cols] scale bytes.  rows must be a multiple of 64 and cols of 4."""
    rows, cols = raw.shape[-2:]
    flat = raw.reshape(*raw.shape[:-2], rows * cols)
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    return flat[..., ref_sf_offset(r, c, cols)]
