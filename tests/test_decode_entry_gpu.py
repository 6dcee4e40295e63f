"""GPU tests of the decode entry points (launch_decode_mmv, _paired, _ranges of cuda/decode_mmv.hpp) under the
Q8-K32 activation policy: quantise + project + DecodeEpilogue in one call, validated like
cuda/decode_mmv.cu:440-540, results against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import _lib as L
from qw38_b200 import synth
from qw38_b200.q4k_q8 import (DecodeMmvDesc, Q4KError, decode_workspace, launch_decode_mmv, launch_decode_mmv_paired,
                              launch_decode_mmv_ranges, prefill_paired_swiglu, prefill_project)
from tests.helpers import assert_close_contract

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def setup(n, k, m, seed):
    codes, meta = synth.logical_q4k(n, k, seed=seed)
    hc, hs = synth.split_tiles(codes, meta)
    from qw38_b200.q4k_q8 import PrefillWeight
    w = PrefillWeight.from_host(hc, hs, n, k)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=seed + 1))
    x = torch.from_numpy(xb.view(np.int16)).to(DEV).view(torch.bfloat16)
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    ref = orc.project(hc, hs, n, k, rz, ra, rs)
    return w, x, ref


@pytest.mark.parametrize("m", [1, 5, 16])
def test_decode_mmv_epilogues(m):
    n, k = 520, 1280
    w, x, ref = setup(n, k, m, seed=3)
    ws = decode_workspace(m, n, k)
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    out32 = torch.empty((m, n), dtype=torch.float32, device=DEV)
    launch_decode_mmv(DecodeMmvDesc(w, x, out32, L.EPILOGUE_STORE_FP32), ws, f)
    assert_close_contract(out32.cpu().numpy(), ref)
    out16 = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    launch_decode_mmv(DecodeMmvDesc(w, x, out16, L.EPILOGUE_STORE_BF16), ws, f)
    want16 = synth.f32_to_bf16_bits(out32.cpu().numpy())
    assert (bf16_bits(out16) == want16).all(), "StoreBf16 is the RNE rounding of the fp32 result"
    res = torch.from_numpy(synth.activations(m, n, seed=8)).to(DEV)
    sep = torch.empty((m, n), dtype=torch.float32, device=DEV)
    launch_decode_mmv(DecodeMmvDesc(w, x, sep, L.EPILOGUE_RESIDUAL_ADD_FP32, residual=res), ws, f)
    assert torch.equal(sep, out32 + res), "residual is the last fp32 add"
    inplace = res.clone()
    launch_decode_mmv(DecodeMmvDesc(w, x, None, L.EPILOGUE_RESIDUAL_ADD_FP32, residual=inplace), ws, f)
    assert torch.equal(inplace, sep), "an empty output updates the residual in place"
    assert f.item() == 0
    # contract violations are rejected before anything is launched
    canary = torch.full((m, n), 7.0, dtype=torch.float32, device=DEV)
    with pytest.raises(Q4KError, match="must not supply residual"):
        launch_decode_mmv(DecodeMmvDesc(w, x, canary, L.EPILOGUE_STORE_FP32, residual=res), ws, f)
    with pytest.raises(Q4KError, match="requires paired"):
        launch_decode_mmv(DecodeMmvDesc(w, x, out16, L.EPILOGUE_SWIGLU_STORE_BF16), ws, f)
    with pytest.raises(Q4KError, match="activation policy"):
        launch_decode_mmv(DecodeMmvDesc(w, x, canary, L.EPILOGUE_STORE_FP32, activation_policy=7), ws, f)
    with pytest.raises(Q4KError, match="workspace"):
        launch_decode_mmv(DecodeMmvDesc(w, x, canary, L.EPILOGUE_STORE_FP32), ws[:1024], f)
    torch.cuda.synchronize()
    assert (canary == 7.0).all()


@pytest.mark.parametrize("m,n,k", [(1, 1000, 2048), (8, 1000, 2048), (16, 640, 17408), (3, 136, 17408), (9, 34816 // 8, 5120)])
def test_decode_mmv_paired_swiglu_and_ranges(m, n, k):
    """One launch per call: the gate / up pair's tiles alternate through the blocks and the reducer writes
    bf16(SiLU(gate) * up); ranges and plain pairs walk their weights' tiles one after the other.  K = 17408 runs with
    K slices through the global scratch (the epilogue is then applied by the last block of a row range)."""
    wa, x, ref_a = setup(n, k, m, seed=11)
    codes, meta = synth.logical_q4k(n, k, seed=12)
    hc, hs = synth.split_tiles(codes, meta)
    from qw38_b200.q4k_q8 import PrefillWeight
    wb = PrefillWeight.from_host(hc, hs, n, k)
    xb = bf16_bits(x)
    rz, ra, rs, _ = orc.q8_quantize(xb.reshape(m, k), bf16_bits=True)
    ref_b = orc.project(hc, hs, n, k, rz, ra, rs)
    ws = decode_workspace(m, 2 * n, k)
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    launch_decode_mmv_paired(DecodeMmvDesc(wa, x, y, L.EPILOGUE_SWIGLU_STORE_BF16),
                             DecodeMmvDesc(wb, x, None, L.EPILOGUE_SWIGLU_STORE_BF16), ws, f)
    g, u = ref_a.astype(np.float64), ref_b.astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    got = bf16_to_f32(bf16_bits(y)).astype(np.float64)
    tol = 2.0 ** -7 * np.abs(want) + 2e-3 * np.sqrt((want ** 2).mean())     # bf16 rounding + the fp32 contract of both inputs
    assert (np.abs(got - want) <= tol).all()
    # paired, plain stores: two outputs from one quantisation
    oa = torch.empty((m, n), dtype=torch.float32, device=DEV)
    ob = torch.empty((m, n), dtype=torch.float32, device=DEV)
    launch_decode_mmv_paired(DecodeMmvDesc(wa, x, oa, L.EPILOGUE_STORE_FP32), DecodeMmvDesc(wb, x, ob, L.EPILOGUE_STORE_FP32), ws, f)
    assert_close_contract(oa.cpu().numpy(), ref_a)
    assert_close_contract(ob.cpu().numpy(), ref_b)
    # ranges: same results as the paired stores
    ra_, rb_ = torch.empty_like(oa), torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    launch_decode_mmv_ranges([DecodeMmvDesc(wa, x, ra_, L.EPILOGUE_STORE_FP32), DecodeMmvDesc(wb, x, rb_, L.EPILOGUE_STORE_BF16)], ws, f)
    assert torch.equal(ra_, oa)
    assert (bf16_bits(rb_) == synth.f32_to_bf16_bits(ob.cpu().numpy())).all()
    with pytest.raises(Q4KError, match="must not declare"):
        launch_decode_mmv_paired(DecodeMmvDesc(wa, x, y, L.EPILOGUE_SWIGLU_STORE_BF16),
                                 DecodeMmvDesc(wb, x, y, L.EPILOGUE_SWIGLU_STORE_BF16), ws, f)
    with pytest.raises(Q4KError, match="must match"):
        launch_decode_mmv_paired(DecodeMmvDesc(wa, x, oa, L.EPILOGUE_STORE_FP32),
                                 DecodeMmvDesc(wb, x.clone(), ob, L.EPILOGUE_STORE_FP32), ws, f)
    with pytest.raises(Q4KError, match="two or three"):
        launch_decode_mmv_ranges([DecodeMmvDesc(wa, x, ra_, L.EPILOGUE_STORE_FP32)], ws, f)
    assert f.item() == 0


def test_prefill_project_and_paired_swiglu():
    """PrefillEngine::project / paired_swiglu over the same composition, beyond sixteen rows (tcgen05 path)."""
    m, n, k = 130, 1000, 2048
    wa, x, ref_a = setup(n, k, m, seed=21)
    codes, meta = synth.logical_q4k(n, k, seed=22)
    hc, hs = synth.split_tiles(codes, meta)
    from qw38_b200.q4k_q8 import PrefillWeight
    wb = PrefillWeight.from_host(hc, hs, n, k)
    rz, ra, rs, _ = orc.q8_quantize(bf16_bits(x).reshape(m, k), bf16_bits=True)
    ref_b = orc.project(hc, hs, n, k, rz, ra, rs)
    ws = decode_workspace(m, n, k)
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    res = torch.from_numpy(synth.activations(m, n, seed=5)).to(DEV)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    prefill_project(DecodeMmvDesc(wa, x, out, L.EPILOGUE_RESIDUAL_ADD_FP32, residual=res), ws, f)
    assert_close_contract(out.cpu().numpy() - res.cpu().numpy(), ref_a)
    with pytest.raises(Q4KError):
        launch_decode_mmv(DecodeMmvDesc(wa, x, out, L.EPILOGUE_STORE_FP32), ws, f)      # decode entry stops at 16 rows
    y = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    prefill_paired_swiglu(wa, wb, x, y, ws, f)
    g, u = ref_a.astype(np.float64), ref_b.astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    got = bf16_to_f32(bf16_bits(y)).astype(np.float64)
    tol = 2.0 ** -7 * np.abs(want) + 2e-3 * np.sqrt((want ** 2).mean())
    assert (np.abs(got - want) <= tol).all()
    assert f.item() == 0


@pytest.mark.parametrize("m,n,k", [(1, 520, 1280), (3, 137, 259), (1, 1000, 5120)])
def test_decode_mmv_bf16_policy(m, n, k):
    """The reference's own activation policy (bf16-rounded weights x bf16 activations): compared with the CPU
    statement of src/compiler/quantization/reference.cpp at the reference's decode_mmv_tol budget
    (cuda/decode_mmv.hpp: 1e-3 + 1e-4|ref| for fp32, 8e-3 for the bf16 store), K tail and ragged rows included."""
    codes, meta = synth.logical_q4k(n, k, seed=31)
    hc, hs = synth.split_tiles(codes, meta)
    from qw38_b200.q4k_q8 import PrefillWeight, pad_k
    w = PrefillWeight.from_host(hc, hs, n, k)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=32))
    x = torch.from_numpy(xb.view(np.int16)).to(DEV).view(torch.bfloat16)
    ref = np.stack([orc.bf16_gemv(hc, hs, n, k, pad_k(k), xb[t]) for t in range(m)])
    ws = decode_workspace(m, 2 * n, k)
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty((m, n), dtype=torch.float32, device=DEV)
    launch_decode_mmv(DecodeMmvDesc(w, x, out, L.EPILOGUE_STORE_FP32, activation_policy=L.ACTIVATION_BF16), ws, f)
    got = out.cpu().numpy()
    scale = np.abs(ref).max()
    assert (np.abs(got - ref) <= 1e-3 + 1e-4 * np.abs(ref) + 2e-6 * scale * np.sqrt(k)).all()
    res = torch.from_numpy(synth.activations(m, n, seed=33)).to(DEV)
    inplace = res.clone()
    launch_decode_mmv(DecodeMmvDesc(w, x, None, L.EPILOGUE_RESIDUAL_ADD_FP32, residual=inplace, activation_policy=L.ACTIVATION_BF16), ws, f)
    assert torch.equal(inplace, res + out)
    y = torch.empty((m, n), dtype=torch.bfloat16, device=DEV)
    launch_decode_mmv(DecodeMmvDesc(w, x, y, L.EPILOGUE_STORE_BF16, activation_policy=L.ACTIVATION_BF16), ws, f)
    assert (bf16_bits(y) == synth.f32_to_bf16_bits(got)).all()
    # paired SwiGLU under the same policy
    codes2, meta2 = synth.logical_q4k(n, k, seed=34)
    hc2, hs2 = synth.split_tiles(codes2, meta2)
    w2 = PrefillWeight.from_host(hc2, hs2, n, k)
    ref2 = np.stack([orc.bf16_gemv(hc2, hs2, n, k, pad_k(k), xb[t]) for t in range(m)])
    launch_decode_mmv_paired(DecodeMmvDesc(w, x, y, L.EPILOGUE_SWIGLU_STORE_BF16, activation_policy=L.ACTIVATION_BF16),
                             DecodeMmvDesc(w2, x, None, L.EPILOGUE_SWIGLU_STORE_BF16, activation_policy=L.ACTIVATION_BF16), ws, f)
    g, u = ref.astype(np.float64), ref2.astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    got_y = bf16_to_f32(bf16_bits(y)).astype(np.float64)
    assert (np.abs(got_y - want) <= 2.0 ** -7 * np.abs(want) + 8e-3 + 1e-3 * np.abs(u)).all()
    with pytest.raises(Q4KError, match="must match"):       # policies of a pair must agree
        launch_decode_mmv_paired(DecodeMmvDesc(w, x, out, L.EPILOGUE_STORE_FP32, activation_policy=L.ACTIVATION_BF16),
                                 DecodeMmvDesc(w2, x, torch.empty_like(out), L.EPILOGUE_STORE_FP32), ws, f)
    assert f.item() == 0
