"""GPU tests of the device-side Q4_K fitter (compiler::quantize_q4k_block,
src/compiler/quantization/q4k.cpp:186-278): codes, the 16 metadata bytes and the refusal of every
block must equal the reference's host fitter bit for bit -- against the committed vectors that
the reference's own code produced, and, where that code was built on this machine, against it
directly on a larger seeded set."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import _lib as L
from qw38_b200.q4k_q8 import FIT_ERRORS, Q4KError, q4k_q8_project, pack_q8, quantize_q4k_blocks, quantize_q4k_weight
from tests.helpers import fitter_cases

pytestmark = pytest.mark.gpu
DEV = "cuda"


def fit(weights: np.ndarray):
    t = torch.from_numpy(np.ascontiguousarray(weights)).to(DEV)
    codes, meta, status = quantize_q4k_blocks(t, check=False)
    return codes.cpu().numpy(), meta.cpu().numpy(), status.cpu().numpy()


def test_fitter_matches_reference_vectors(golden):
    g = golden
    codes, meta, status = fit(g["b_weights"].reshape(-1, 256))
    assert (status == 0).all()
    assert np.array_equal(codes, g["b_fit_codes"].reshape(-1, 256))
    assert np.array_equal(meta, g["b_fit_meta"].reshape(-1, 16))


def test_fitter_corner_cases_and_refusals_match_reference_vectors(golden):
    g = golden
    codes, meta, status = fit(g["e_weights"])
    assert np.array_equal(status, g["e_fit_status"])
    assert set(status.tolist()) == {0, 1, 2, 3, 4, 5}  # every refusal of the reference is exercised
    assert np.array_equal(meta, g["e_fit_meta"])
    assert np.array_equal(codes, g["e_fit_codes"])
    assert not codes[status != 0].any() and not meta[status != 0].any()


def test_fitter_check_raises_the_first_refusal_in_block_order(golden):
    g = golden
    first = int(np.nonzero(g["e_fit_status"])[0][0])
    t = torch.from_numpy(g["e_weights"]).to(DEV)
    with pytest.raises(Q4KError) as err:
        quantize_q4k_blocks(t)
    assert f"block {first}: {FIT_ERRORS[int(g['e_fit_status'][first])]}" in str(err.value)
    ok = torch.from_numpy(g["e_weights"][:first]).to(DEV)
    quantize_q4k_blocks(ok)  # no refusal before that block


def test_fitter_bf16_input_equals_widened_fp32_input():
    w = fitter_cases(77, 400)
    w = w[np.isfinite(w).all(axis=1)]
    bits = (w.view(np.uint32) >> 16).astype(np.uint16)  # truncation: any bf16 pattern will do
    wide = (bits.astype(np.uint32) << 16).view(np.float32)
    t16 = torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)
    c16, m16, s16 = quantize_q4k_blocks(t16, check=False)
    c32, m32, s32 = fit(wide)
    assert np.array_equal(c16.cpu().numpy(), c32) and np.array_equal(m16.cpu().numpy(), m32)
    assert np.array_equal(s16.cpu().numpy(), s32)


@pytest.mark.parametrize("n,k", [(21, 768), (8, 256), (130, 1280)])
def test_fit_weight_is_fit_then_pack(n, k):
    rng = np.random.default_rng(n * 1000 + k)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    w[3, 256:288] = 0.0
    codes, meta, status = fit(w.reshape(-1, 256))
    assert (status == 0).all()
    want_codes, want_scales = orc.pack_split(codes.reshape(n, k), meta.reshape(n, k // 256, 16))
    pw = quantize_q4k_weight(torch.from_numpy(w).to(DEV))
    assert np.array_equal(pw.codes.cpu().numpy(), want_codes)
    assert np.array_equal(pw.scales.cpu().numpy(), want_scales)
    # bf16 weights, as a checkpoint holds them
    wb = torch.from_numpy(w).to(DEV).to(torch.bfloat16)
    pb = quantize_q4k_weight(wb)
    cb, mb, sb = fit(wb.float().cpu().numpy().reshape(-1, 256))
    wc, ws = orc.pack_split(cb.reshape(n, k), mb.reshape(n, k // 256, 16))
    assert np.array_equal(pb.codes.cpu().numpy(), wc) and np.array_equal(pb.scales.cpu().numpy(), ws)


def test_fitted_weight_feeds_the_projection():
    """Fit on the device, project on the device: the result follows the float matmul within the
    quantisation noise of 4-bit weights and 8-bit activations."""
    n, k, m = 64, 1024, 3
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    pw = quantize_q4k_weight(torch.from_numpy(w).to(DEV))
    xq = pack_q8(torch.from_numpy(x).to(DEV).to(torch.bfloat16), torch.zeros(1, dtype=torch.int32, device=DEV))
    y = q4k_q8_project(pw, xq).cpu().numpy()
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    err = np.abs(y - ref)
    assert err.max() < 0.08 * np.sqrt((ref ** 2).mean()) * 4, err.max()


def test_fit_rejects_bad_geometry_before_any_launch():
    lib = L.load()
    w = torch.zeros(2, 300, device=DEV)
    buf = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = lambda t: C.c_void_p(t.data_ptr())
    assert lib.q4k_fit_weight(p(w), 0, 2, 300, p(buf), 8 * 256, p(buf[2048:]), 8 * 32, None, p(flag), None) == L.ERR_INVALID_ARGUMENT
    assert lib.q4k_fit_weight(p(w), 7, 2, 256, p(buf), 8 * 128, p(buf[2048:]), 8 * 16, None, p(flag), None) == L.ERR_INVALID_ARGUMENT
    assert lib.q4k_fit_blocks(p(w), 0, 0, p(buf), p(buf[2048:]), None, p(flag), None) == L.ERR_INVALID_ARGUMENT
    # overlapping outputs
    assert lib.q4k_fit_blocks(p(w), 0, 2, p(buf), p(buf[256:]), None, p(flag), None) == L.ERR_INVALID_ARGUMENT
    assert int(flag.item()) == 0


def test_fitter_matches_reference_host_code_at_scale():
    ref = orc.ref()
    if ref is None or not hasattr(ref, "ref_quantize_q4k_blocks"):
        pytest.skip("the reference's host code was not built on this machine; the committed vectors cover it")
    w = np.ascontiguousarray(fitter_cases(424242, 30000))
    nb = w.shape[0]
    rc = np.zeros((nb, 256), dtype=np.int8)
    rm = np.zeros((nb, 16), dtype=np.uint8)
    rs = np.zeros(nb, dtype=np.uint8)
    ref.ref_quantize_q4k_blocks.restype = C.c_uint64
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    ref.ref_quantize_q4k_blocks(vp(w), C.c_uint64(nb), vp(rc), vp(rm), vp(rs))
    codes, meta, status = fit(w)
    assert np.array_equal(status, rs)
    bad_meta = np.nonzero((meta != rm).any(axis=1))[0]
    assert bad_meta.size == 0, f"{bad_meta.size} blocks differ in metadata, first {bad_meta[:5]}"
    bad = np.nonzero((codes != rc).any(axis=1))[0]
    assert bad.size == 0, f"{bad.size} blocks differ in codes, first {bad[:5]}"
