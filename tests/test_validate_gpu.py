"""GPU tests of q4k_validate_weight: the Q4_K rows of format::validate_cuda_v0
(src/format/unpack.cpp:156-226) on a resident weight.  Offences are planted at known bytes; the
verdict must name the first one in the reference's scan order (tile rows ascending, codes before
metadata, d before dmin) -- checked analytically and, where the reference's host code was built
on this machine, against it."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import synth
from qw38_b200.q4k_q8 import PrefillWeight, VALIDATE_ERRORS, quantize_q4k_weight, validate_weight

pytestmark = pytest.mark.gpu


def host_weight(n, k, seed):
    codes, meta = synth.logical_q4k(n, k, seed=seed)
    return synth.split_tiles(codes, meta)


def reference_verdict(n, k, hc, hs):
    ref = orc.ref()
    if ref is None or not hasattr(ref, "ref_validate_q4k_where"):
        return None
    off = C.c_uint64(0)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    kind = ref.ref_validate_q4k_where(C.c_uint64(n), C.c_uint64(k), vp(hc), C.c_uint64(hc.size), vp(hs), C.c_uint64(hs.size),
                                      C.byref(off))
    return kind, off.value


def check(n, k, hc, hs, want):
    got = validate_weight(PrefillWeight.from_host(hc, hs, n, k))
    assert got == want
    ref = reference_verdict(n, k, hc, hs)
    if ref is not None:
        assert ref == want


def tile_row(row, kb, tiles_k):
    return ((row // 8) * tiles_k + kb) * 8 + row % 8


@pytest.mark.parametrize("n,k", [(137, 512), (64, 1024), (5, 256)])
def test_packed_weights_are_admissible(n, k):
    hc, hs = host_weight(n, k, 3)
    check(n, k, hc, hs, (0, 0))
    assert sorted(VALIDATE_ERRORS) == [1, 2, 3]


def test_fitted_weights_are_admissible():
    w = torch.randn(37, 768, device="cuda") * 0.1
    assert validate_weight(quantize_q4k_weight(w)) == (0, 0)


def test_each_rule_and_its_offset():
    n, k, tiles_k = 137, 512, 2
    hc, hs = host_weight(n, k, 4)
    # a code nibble in a padded row
    c = hc.copy(); tr = tile_row(140, 1, tiles_k); c[tr * 128 + 77] = 0x30
    check(n, k, c, hs, (1, tr * 128 + 77))
    # a metadata byte in a padded row
    s = hs.copy(); tr = tile_row(143, 0, tiles_k); s[tr * 16 + 9] = 1
    check(n, k, hc, s, (2, tr * 16 + 9))
    # negative d, infinite dmin, NaN d on live rows
    s = hs.copy(); tr = tile_row(20, 1, tiles_k); s[tr * 16 + 1] |= 0x80
    check(n, k, hc, s, (3, tr * 16))
    s = hs.copy(); tr = tile_row(136, 0, tiles_k); s[tr * 16 + 2] = 0x00; s[tr * 16 + 3] = 0x7C
    check(n, k, hc, s, (3, tr * 16 + 2))
    s = hs.copy(); tr = tile_row(0, 0, tiles_k); s[tr * 16 + 0] = 0x01; s[tr * 16 + 1] = 0x7E
    check(n, k, hc, s, (3, tr * 16))
    # fp16 subnormal and zero scales are admissible
    s = hs.copy(); tr = tile_row(9, 1, tiles_k); s[tr * 16: tr * 16 + 4] = [1, 0, 0, 0]
    check(n, k, hc, s, (0, 0))


def test_first_offence_in_scan_order_wins():
    n, k, tiles_k = 137, 512, 2
    hc, hs = host_weight(n, k, 5)
    c, s = hc.copy(), hs.copy()
    late = tile_row(142, 1, tiles_k)
    c[late * 128 + 3] = 0x01                      # padded code, late tile row
    early = tile_row(139, 1, tiles_k)
    s[early * 16 + 15] = 0xFF                     # padded metadata, earlier tile row
    check(n, k, c, s, (2, early * 16 + 15))
    c[early * 128 + 127] = 0xF0                   # same tile row: codes are scanned before metadata
    check(n, k, c, s, (1, early * 128 + 127))
    c[early * 128 + 5] = 0x0A                     # lower byte of the same row
    check(n, k, c, s, (1, early * 128 + 5))
    live = tile_row(77, 0, tiles_k)
    s[live * 16 + 3] |= 0x80                      # dmin negative in a far earlier tile row
    check(n, k, c, s, (3, live * 16 + 2))
    s[live * 16 + 1] |= 0x80                      # d of the same block is read first
    check(n, k, c, s, (3, live * 16))


def test_large_weight_with_one_planted_offence():
    n, k = 5120, 5120
    hc, hs = host_weight(n, k, 6)
    check(n, k, hc, hs, (0, 0))
    s = hs.copy(); tr = tile_row(4097, 13, 20); s[tr * 16 + 3] = 0xFC
    got = validate_weight(PrefillWeight.from_host(hc, s, n, k))
    assert got == (3, tr * 16 + 2)


# ---- q4k_dequantize_bf16: compiler::dequantize_to_bf16 from the resident weight ---------------------

def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def test_dequantise_matches_reference_vectors(golden):
    from qw38_b200.q4k_q8 import dequantize_bf16
    w = PrefillWeight.from_host(golden["a_packed_codes"], golden["a_packed_scales"], 137, 512)
    assert np.array_equal(bf16_bits(dequantize_bf16(w)), golden["a_dequant_bf16"])


@pytest.mark.parametrize("n,k", [(300, 1280), (8, 256), (1021, 5120)])
def test_dequantise_matches_cpu_statement(n, k):
    from qw38_b200.q4k_q8 import dequantize_bf16
    codes, meta = synth.logical_q4k(n, k, seed=n)
    hc, hs = synth.split_tiles(codes, meta)
    got = bf16_bits(dequantize_bf16(PrefillWeight.from_host(hc, hs, n, k)))
    assert np.array_equal(got, orc.dequantize_bf16(codes[:, :k], meta))


def test_fit_then_dequantise_stays_close_to_the_weights():
    from qw38_b200.q4k_q8 import dequantize_bf16
    torch.manual_seed(3)
    w = torch.randn(64, 2048, device="cuda") * 0.05
    back = dequantize_bf16(quantize_q4k_weight(w)).float()
    err = (back - w).abs().reshape(64, -1, 32)
    span = (w.reshape(64, -1, 32).amax(dim=2) - w.reshape(64, -1, 32).amin(dim=2).clamp(max=0)).unsqueeze(2)
    # in units of a group's step (range / 15): the weighted fit may clip an outlier by most of a step,
    # the typical error is a quarter of one (the reference's host fitter gives 0.83 and 0.26 here)
    ratio = err / (span / 15)
    assert float(ratio.max()) < 1.25 and float((ratio ** 2).mean().sqrt()) < 0.35


def test_dequantise_rejects_wrong_output_length():
    import ctypes
    from qw38_b200 import _lib as L
    codes, meta = synth.logical_q4k(16, 256, seed=1)
    w = PrefillWeight.from_host(*synth.split_tiles(codes, meta), 16, 256)
    out = torch.zeros(16 * 256 + 8, dtype=torch.bfloat16, device="cuda")
    st = L.load().q4k_dequantize_bf16(ctypes.byref(w.c_struct()), ctypes.c_void_p(out.data_ptr()), out.numel(), None)
    assert st == L.ERR_INVALID_ARGUMENT and not out.any()


# ---- q4k_unpack_logical: format::unpack_cuda_v0 from the resident weight ------------------------------

def test_unpack_matches_reference_vectors(golden):
    from qw38_b200.q4k_q8 import unpack_logical
    w = PrefillWeight.from_host(golden["a_packed_codes"], golden["a_packed_scales"], 137, 512)
    codes, meta = unpack_logical(w)
    assert np.array_equal(codes.cpu().numpy(), golden["a_codes"])
    assert np.array_equal(meta.cpu().numpy(), golden["a_meta"])


@pytest.mark.parametrize("n,k", [(21, 768), (1021, 5120), (64, 17408)])
def test_fit_pack_unpack_round_trip(n, k):
    from qw38_b200.q4k_q8 import quantize_q4k_blocks, unpack_logical
    torch.manual_seed(n)
    w = torch.randn(n, k, device="cuda") * 0.03
    codes, meta, status = quantize_q4k_blocks(w)
    ucodes, umeta = unpack_logical(quantize_q4k_weight(w))
    assert torch.equal(ucodes.reshape(-1, 256), codes) and torch.equal(umeta.reshape(-1, 16), meta)


def test_bf16_operand_for_a_library_gemm_follows_the_unpacked_weights():
    """The operand of the reference's BF16 prefill route (unpack -> library GEMM): the bit-exact bf16 weights from
    q4k_dequantize_bf16, multiplied here by torch with fp32 accumulation, reproduce the exact product within bf16
    rounding (2^-8) plus accumulation noise.  (The library GEMM itself is not part of this package.)"""
    from qw38_b200.q4k_q8 import dequantize_bf16
    n, k, m = 256, 1024, 33
    codes, meta = synth.logical_q4k(n, k, seed=9)
    w = PrefillWeight.from_host(*synth.split_tiles(codes, meta), n, k)
    torch.manual_seed(1)
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    wb = dequantize_bf16(w)
    y = torch.matmul(x, wb.t()).float().cpu().numpy()
    ref = x.double().cpu().numpy() @ wb.double().cpu().numpy().T
    rms = np.sqrt((ref ** 2).mean())
    assert np.abs(y - ref).max() <= 2.0 ** -8 * np.abs(ref).max() + 1e-3 * rms
