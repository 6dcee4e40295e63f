"""Pins the CPU oracle (oracle/q4k_oracle.c) before anything trusts it:
against golden vectors produced by the reference's own host code (tests/golden/make_golden.py),
against the literals of the reference's tests, against an independent numpy restatement, and --
when the reference host library is present on this machine -- against that library live."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from qw38_b200 import synth


def test_fp16_decode_exhaustive(golden):
    want = golden["c_fp16_as_f32_bits"]
    lib = orc.lib()
    got = np.array([lib.orc_fp16_to_fp32(C.c_uint16(h)) for h in range(65536)], dtype=np.float32).view(np.uint32)
    nan = (want & 0x7FFFFFFF) > 0x7F800000
    assert (got[~nan] == want[~nan]).all()
    assert ((got[nan] & 0x7FFFFFFF) > 0x7F800000).all()
    # numpy's own fp16 agrees, including subnormals (decode_mmv_unit_test.cpp:417-447 pins those)
    np_bits = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32).view(np.uint32)
    assert (np_bits[~nan] == want[~nan]).all()


def test_fp32_to_fp16_roundtrip_and_rne():
    lib = orc.lib()
    for h in list(range(0, 0x7C00, 7)) + [0x0001, 0x03FF, 0x0400, 0x7BFF]:
        f = np.uint16(h).view(np.float16).astype(np.float32)
        assert lib.orc_fp32_to_fp16(C.c_float(float(f))) == h
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(20000) * 10 ** rng.uniform(-7, 4, 20000)).astype(np.float32)
    got = np.array([lib.orc_fp32_to_fp16(C.c_float(float(v))) for v in x], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert (got == want).all()


def test_bf16_rne_matches_reference_conversion():
    r = orc.ref()
    lib = orc.lib()
    rng = np.random.default_rng(4)
    x = (rng.standard_normal(5000) * 10 ** rng.uniform(-10, 10, 5000)).astype(np.float32)
    got = np.array([lib.orc_fp32_to_bf16(C.c_float(float(v))) for v in x], dtype=np.uint16)
    assert (got == synth.f32_to_bf16_bits(x)).all()
    if r is not None:
        want = np.array([r.ref_fp32_to_bf16(C.c_float(float(v))) for v in x], dtype=np.uint16)
        assert (got == want).all()


def test_scale_min_decode_matches_pinned_upstream(golden):
    q12, sc, mn = golden["d_q12"], golden["d_sc"], golden["d_mn"]
    lib = orc.lib()
    for i in range(q12.shape[0]):
        s8 = np.zeros(8, dtype=np.uint8)
        m8 = np.zeros(8, dtype=np.uint8)
        lib.orc_scale_min(q12[i].ctypes.data_as(C.c_void_p), s8.ctypes.data_as(C.c_void_p), m8.ctypes.data_as(C.c_void_p))
        assert (s8 == sc[i]).all() and (m8 == mn[i]).all()
        back = np.zeros(12, dtype=np.uint8)
        lib.orc_pack_scale_min(s8.ctypes.data_as(C.c_void_p), m8.ctypes.data_as(C.c_void_p), back.ctypes.data_as(C.c_void_p))
        assert (back == q12[i]).all()
    assert (synth.pack_scale_min(sc, mn) == q12).all()


def test_split_tile_layout_matches_reference_packer(golden):
    codes, meta = golden["a_codes"], golden["a_meta"]
    oc, om = orc.pack_split(codes, meta)
    assert (oc == golden["a_packed_codes"]).all()
    assert (om == golden["a_packed_scales"]).all()
    sc, sm = synth.split_tiles(codes.astype(np.uint8), meta)
    assert (sc == oc).all() and (sm == om).all()
    # tile coordinates pinned by tests/pack_layout_test.cpp:197-260
    tiles_k = 2
    for row, kb in [(0, 0), (7, 1), (8, 0), (136, 1)]:
        tr = ((row // 8) * tiles_k + kb) * 8 + row % 8
        want = codes[row, kb * 256:(kb + 1) * 256].astype(np.uint8)
        assert (oc[tr * 128:(tr + 1) * 128] == (want[0::2] | (want[1::2] << 4))).all()
        assert (om[tr * 16:(tr + 1) * 16] == meta[row, kb]).all()
    # padded rows 137..143 hold zero codes and zero metadata
    for row in range(137, 144):
        tr = ((row // 8) * tiles_k) * 8 + row % 8
        assert not oc[tr * 128:(tr + 1) * 128].any() and not om[tr * 16:(tr + 1) * 16].any()


def test_blocks144_equal_the_fitters_logical_codes(golden):
    """The reference proves code-for-code equality of its fitter and the upstream 144-byte
    blocks (tests/q4k_reference_test.cpp:46-58); the oracle's converters must agree."""
    blocks, fc, fm = golden["b_blocks144"], golden["b_fit_codes"], golden["b_fit_meta"]
    rows, kk = fc.shape
    codes, meta = orc.blocks144_to_logical(blocks, rows, kk)
    assert (codes == fc).all() and (meta == fm).all()
    assert (orc.logical_to_blocks144(fc, fm) == blocks).all()
    assert (synth.blocks144(fc.astype(np.uint8), fm) == blocks).all()
    a = orc.blocks144_to_split(blocks, rows, kk)
    b = orc.pack_split(fc, fm)
    assert (a[0] == b[0]).all() and (a[1] == b[1]).all()


def test_dequant_and_bf16_policy_gemv_match_reference(golden):
    codes, meta = golden["a_codes"], golden["a_meta"]
    oc, om = golden["a_packed_codes"], golden["a_packed_scales"]
    y = orc.bf16_gemv(oc, om, 137, 512, 512, golden["a_x_bf16"])
    assert (y.view(np.uint32) == golden["a_gemv_bf16_policy"].view(np.uint32)).all()
    # weight values: (d*sc)*q - dmin*m in fp32, as dequantize_row_q4_K
    blocks, deq = golden["b_blocks144"], golden["b_dequant_f32"]
    rows, kk = deq.shape
    c, m = orc.blocks144_to_logical(blocks, rows, kk)
    d = m[..., 0:2].copy().view(np.float16).astype(np.float32)[..., 0]
    dm = m[..., 2:4].copy().view(np.float16).astype(np.float32)[..., 0]
    lib = orc.lib()
    for i in range(rows):
        for b in range(kk // 256):
            s8 = np.zeros(8, dtype=np.uint8)
            m8 = np.zeros(8, dtype=np.uint8)
            lib.orc_scale_min(m[i, b, 4:].copy().ctypes.data_as(C.c_void_p), s8.ctypes.data_as(C.c_void_p), m8.ctypes.data_as(C.c_void_p))
            for g in range(8):
                q = c[i, b * 256 + g * 32:b * 256 + (g + 1) * 32].astype(np.float32)
                want = (d[i, b] * np.float32(s8[g])) * q - dm[i, b] * np.float32(m8[g])
                assert (want.astype(np.float32).view(np.uint32) == deq[i, b * 256 + g * 32:b * 256 + (g + 1) * 32].view(np.uint32)).all()


def test_bf16_dequantiser_matches_reference(golden):
    got = orc.dequantize_bf16(golden["a_codes"], golden["a_meta"])
    assert (got == golden["a_dequant_bf16"]).all()


def reference_test_input(m: int, k: int) -> np.ndarray:
    """bf16 activations of tests/q4k_q8_test.cpp:69-77."""
    r = np.arange(m)[:, None]
    c = np.arange(k)[None, :]
    v = (((r * 23 + c * 19) % 67).astype(np.int64) - 44) * 0.125 * (1 + r % 5)
    v = v.astype(np.float32)
    v[:, 32:64] = 0
    lit = np.array([127.0, 0.5, 1.5, -0.5, -1.5], dtype=np.float32)
    v[:, :5] = lit
    if m > 2:
        v[2, :] = 0
    return synth.f32_to_bf16_bits(v)


def test_q8_quantiser_literals_and_independent_restatement():
    m, k, pk = 33, 259, 512
    xb = reference_test_input(m, k)
    z, a, s, fail = orc.q8_quantize(xb, bf16_bits=True)
    assert fail == 0
    assert list(z[0, :5]) == [127, 0, 2, 0, -2]          # ties to even, saturation (q4k_q8_test.cpp:93)
    assert s[0, 2] < 0                                   # negative-sum fixture (:94)
    assert (z[2] == 0).all() and (a[2] == 1).all()       # whole zero token, zero-group scale 1
    assert (z[:, k:] == 0).all()                         # K tail padding
    assert np.abs(s).max() <= 32 * 127
    # independent numpy statement of tests/q4k_q8_test.cpp:83-92
    x = orc.bf16_bits_to_f32(xb)
    xp = np.zeros((m, pk), dtype=np.float32)
    xp[:, :k] = x
    g = xp.reshape(m, pk // 32, 32)
    peak = np.abs(g).max(axis=2)
    ra = np.where(peak == 0, np.float32(1), peak / np.float32(127)).astype(np.float32)
    rz = np.clip(np.rint(g / ra[..., None]), -127, 127).astype(np.int8)
    assert (rz.reshape(m, pk) == z).all()
    assert (ra.view(np.uint32) == a.view(np.uint32)).all()
    assert (rz.astype(np.int32).sum(axis=2) == s).all()


@pytest.mark.parametrize("bits", [0x7F80, 0xFF80, 0x7FC0])
def test_q8_quantiser_nonfinite_sets_flag_and_nan_scale(bits):
    xb = reference_test_input(3, 259)
    xb[0, 0] = bits
    z, a, s, fail = orc.q8_quantize(xb, bf16_bits=True)
    assert fail == 1 and np.isnan(a[0, 0]) and (z[0, :32] == 0).all() and s[0, 0] == 0
    assert np.isfinite(a[0, 1:]).all()


def test_contraction_matches_independent_restatement(golden):
    """orc_q4k_q8_project / orc_q4k_q8_dots vs a numpy restatement of
    tests/q4k_q8_test.cpp:121-131 built from the LOGICAL scalars, not the packed bytes."""
    codes, meta = golden["a_codes"], golden["a_meta"]
    n, k, pk, G = 137, 259, 512, 16
    oc, om = golden["a_packed_codes"], golden["a_packed_scales"]
    m = 5
    z, a, s, _ = orc.q8_quantize(reference_test_input(m, k), bf16_bits=True)
    dots = orc.dots(oc, n, pk, z)
    want_dots = np.einsum("ngi,tgi->tng", codes.reshape(n, G, 32).astype(np.int64), z.reshape(m, G, 32).astype(np.int64))
    assert (dots == want_dots).all()
    assert np.abs(dots).max() <= 32 * 15 * 127
    r = np.arange(n)[:, None]
    g = np.arange(8)[None, :]
    sc = np.tile(((r * 13 + g * 17 + 3) % 64), (1, 2)).astype(np.float32)   # same per block
    mn = np.tile(((r * 11 + g * 7 + 5) % 64), (1, 2)).astype(np.float32)
    d = np.repeat(meta[..., 0:2].copy().view(np.float16).astype(np.float32)[..., 0], 8, axis=1)
    dm = np.repeat(meta[..., 2:4].copy().view(np.float16).astype(np.float32)[..., 0], 8, axis=1)
    D = (d * sc).astype(np.float32)
    Mn = (dm * mn).astype(np.float32)
    t1 = (D[None] * want_dots.astype(np.float32)).astype(np.float32)
    t2 = (Mn[None] * s[:, None, :].astype(np.float32)).astype(np.float32)
    term = (a[:, None, :] * (t1 - t2).astype(np.float32)).astype(np.float32)
    want = term.astype(np.float64).sum(axis=2)
    out, out64 = orc.project(oc, om, n, pk, z, a, s, want64=True)
    assert np.allclose(out64, want, rtol=1e-12, atol=1e-9)
    assert (out == want.astype(np.float32)).all() or np.abs(out - want).max() < 1e-4
    res = np.linspace(-1, 1, m * n, dtype=np.float32).reshape(m, n)
    out_r = orc.project(oc, om, n, pk, z, a, s, residual=res)
    assert (out_r == (out64.astype(np.float32) + res)).all()
    rows = orc.project_rows(oc, om, n, pk, z, a, s, 40, 17)
    assert (rows == out[:, 40:57]).all()


def test_q8_1_export_definition():
    x = synth.activations(2, 512, seed=5)
    z, a, s, _ = orc.q8_quantize(x)
    rec = orc.q8_1_export(z, a, s).reshape(-1, 36)
    d = rec[:, 0:2].copy().view(np.float16)[:, 0]
    ss = rec[:, 2:4].copy().view(np.float16)[:, 0]
    assert (d == a.reshape(-1).astype(np.float16)).all()
    assert (ss == (a.reshape(-1) * s.reshape(-1).astype(np.float32)).astype(np.float16)).all()
    assert (rec[:, 4:].view(np.int8) == z.reshape(-1, 32)).all()


def test_live_reference_library_agrees_when_present(golden):
    r = orc.ref()
    if r is None:
        pytest.skip("reference host library not built on this machine")
    codes, meta = synth.logical_q4k(24, 768, seed=11)
    oc, om = orc.pack_split(codes.astype(np.int8), meta)
    pc = np.zeros_like(oc)
    ps = np.zeros_like(om)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    cs = np.ascontiguousarray(codes, dtype=np.int8)
    assert r.ref_pack_q4k(p(cs), p(meta), C.c_uint64(24), C.c_uint64(768), p(pc), C.c_uint64(pc.size), p(ps), C.c_uint64(ps.size)) == 0
    assert (pc == oc).all() and (ps == om).all()
    assert r.ref_validate_q4k(C.c_uint64(24), C.c_uint64(768), p(oc), C.c_uint64(oc.size), p(om), C.c_uint64(om.size)) == 0
    xb = synth.f32_to_bf16_bits(synth.activations(1, 768, seed=2)[0])
    y = np.zeros(24, dtype=np.float32)
    assert r.ref_gemv_packed_q4k(C.c_uint64(24), C.c_uint64(768), p(oc), C.c_uint64(oc.size), p(om), C.c_uint64(om.size), p(xb), p(y)) == 0
    assert (orc.bf16_gemv(oc, om, 24, 768, 768, xb).view(np.uint32) == y.view(np.uint32)).all()
