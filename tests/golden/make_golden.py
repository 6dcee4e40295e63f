"""Generates tests/golden/q4k_ref_vectors.npz by running the reference engine's OWN host code
(oracle/_ref/libqw38_ref.so, built by oracle/Makefile from the reference checkout).

Run where the reference checkout is present:  python tests/golden/make_golden.py
The fixture is committed; the tests that consume it run anywhere."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as orc  # noqa: E402


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def main() -> None:
    orc.build_ref()
    ref = orc.ref()
    if ref is None:
        raise SystemExit("reference host library was not built (no reference checkout?)")
    out = {}

    # --- A. The fixture of tests/q4k_q8_test.cpp:36-66: n=137, k=259 (padded 512). ----------
    n, k, pk = 137, 259, 512
    codes = np.zeros((n, pk), dtype=np.int8)
    meta = np.zeros((n, 2, 16), dtype=np.uint8)
    r = np.arange(n)[:, None]
    c = np.arange(k)[None, :]
    codes[:, :k] = (r * 7 + c * 11) % 16
    for row in range(n):
        for b in range(2):
            dh = 1 if row == 0 else [0x1400, 0x1800, 0x1A00][row % 3]
            mh = 2 if row == 0 else (0x1000 if b == 0 else 0x1400)
            m = meta[row, b]
            m[0], m[1], m[2], m[3] = dh & 255, dh >> 8, mh & 255, mh >> 8
            for g in range(8):
                s, mm = (row * 13 + g * 17 + 3) % 64, (row * 11 + g * 7 + 5) % 64
                if g < 4:
                    m[4 + g] |= s
                    m[4 + g + 4] |= mm
                else:
                    m[4 + g + 4] |= (s & 15) | ((mm & 15) << 4)
                    m[4 + g - 4] |= (s >> 4) << 6
                    m[4 + g] |= (mm >> 4) << 6
    pn = 144
    pc = np.zeros(pn * pk // 2, dtype=np.uint8)
    ps = np.zeros(pn * 2 * 16, dtype=np.uint8)
    st = ref.ref_pack_q4k(p(codes), p(meta), C.c_uint64(n), C.c_uint64(pk), p(pc), C.c_uint64(pc.size), p(ps),
                          C.c_uint64(ps.size))
    assert st == 0, st
    assert ref.ref_validate_q4k(C.c_uint64(n), C.c_uint64(pk), p(pc), C.c_uint64(pc.size), p(ps), C.c_uint64(ps.size)) == 0
    uc = np.zeros((n, pk), dtype=np.int8)
    um = np.zeros((n, 2, 16), dtype=np.uint8)
    assert ref.ref_unpack_q4k(C.c_uint64(n), C.c_uint64(pk), p(pc), C.c_uint64(pc.size), p(ps), C.c_uint64(ps.size), p(uc), p(um)) == 0
    assert (uc == codes).all() and (um == meta).all()
    out.update(a_codes=codes, a_meta=meta, a_packed_codes=pc, a_packed_scales=ps)
    # bf16-operand GEMV of the older decode policy on the same matrix (reference_gemv_packed).
    xb = np.array([orc.lib().orc_fp32_to_bf16(C.c_float(((i * 19) % 67 - 44) * 0.125)) for i in range(pk)], dtype=np.uint16)
    y = np.zeros(n, dtype=np.float32)
    assert ref.ref_gemv_packed_q4k(C.c_uint64(n), C.c_uint64(pk), p(pc), C.c_uint64(pc.size), p(ps), C.c_uint64(ps.size), p(xb), p(y)) == 0
    dq = np.zeros((n, pk), dtype=np.uint16)
    assert ref.ref_dequantize_bf16(p(codes), p(meta), C.c_uint64(n), C.c_uint64(pk), p(dq)) == 0
    out.update(a_x_bf16=xb, a_gemv_bf16_policy=y, a_dequant_bf16=dq)

    # --- B. Fitter and pinned upstream bodies on seeded float rows. --------------------------
    rng = np.random.default_rng(20240611)
    rows, kk = 6, 1024
    w = (rng.standard_normal((rows, kk)) * np.array([0.02, 0.5, 1.0, 3.0, 1e-3, 10.0])[:, None]).astype(np.float32)
    w[1, :32] = 0.0  # a constant sub-block
    fit_codes = np.zeros((rows, kk), dtype=np.int8)
    fit_meta = np.zeros((rows, kk // 256, 16), dtype=np.uint8)
    for i in range(rows):
        for b in range(kk // 256):
            blk = np.ascontiguousarray(w[i, b * 256:(b + 1) * 256])
            cc = np.zeros(256, dtype=np.int8)
            mm = np.zeros(16, dtype=np.uint8)
            assert ref.ref_quantize_q4k_block(p(blk), p(cc), p(mm)) == 0
            fit_codes[i, b * 256:(b + 1) * 256] = cc
            fit_meta[i, b] = mm
    blocks = np.zeros((rows, kk // 256, 144), dtype=np.uint8)
    deq = np.zeros((rows, kk), dtype=np.float32)
    for i in range(rows):
        ref.ref_llama_quantize_row_q4k(p(np.ascontiguousarray(w[i])), p(blocks[i]), C.c_int64(kk))
        ref.ref_llama_dequantize_row_q4k(p(blocks[i]), p(deq[i]), C.c_int64(kk))
    out.update(b_weights=w, b_fit_codes=fit_codes, b_fit_meta=fit_meta, b_blocks144=blocks, b_dequant_f32=deq)

    # --- C. Exhaustive fp16 decode (src/format/floatcvt.hpp), non-NaN patterns. ------------------
    halves = np.arange(65536, dtype=np.uint32)
    f = np.array([ref.ref_fp16_to_fp32(C.c_uint16(int(h))) for h in halves], dtype=np.float32)
    out.update(c_fp16_as_f32_bits=f.view(np.uint32))

    # --- D. get_scale_min_k4 on seeded 12-byte groups. --------------------------------------------
    q12 = rng.integers(0, 256, size=(64, 12), dtype=np.uint8)
    sc = np.zeros((64, 8), dtype=np.uint8)
    mn = np.zeros((64, 8), dtype=np.uint8)
    for i in range(64):
        for j in range(8):
            a, b = C.c_uint8(0), C.c_uint8(0)
            ref.ref_llama_scale_min(j, p(q12[i]), C.byref(a), C.byref(b))
            sc[i, j], mn[i, j] = a.value, b.value
    out.update(d_q12=q12, d_sc=sc, d_mn=mn)

    # --- E. Fitter corner cases and refusals (quantize_q4k_block, every block attempted). -------
    from tests.helpers import fitter_cases
    cases = np.ascontiguousarray(fitter_cases(20240612, 98))
    nb = cases.shape[0]
    e_codes = np.zeros((nb, 256), dtype=np.int8)
    e_meta = np.zeros((nb, 16), dtype=np.uint8)
    e_status = np.zeros(nb, dtype=np.uint8)
    ref.ref_quantize_q4k_blocks.restype = C.c_uint64
    refused = ref.ref_quantize_q4k_blocks(p(cases), C.c_uint64(nb), p(e_codes), p(e_meta), p(e_status))
    assert refused == int((e_status != 0).sum()) and 9 not in e_status
    print("fitter cases:", nb, "refused by kind:", np.bincount(e_status, minlength=6)[1:])
    out.update(e_weights=cases, e_fit_codes=e_codes, e_fit_meta=e_meta, e_fit_status=e_status)

    path = Path(__file__).with_name("q4k_ref_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
