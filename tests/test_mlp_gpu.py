"""The fused MLP chain behind q4k_q8_mlp (cuda/q4k_q8.hpp:44-49): RMS norm + Q8 pack -> gate ->
up -> SwiGLU + Q8 pack -> down + residual, and its failure-flag protocol.  The CPU chain is
the oracle's; like the reference's own integration test (tests/q8_mlp_integration_test.cpp:21-47)
the comparison is 0.02 + 0.002|ref| because a bf16 rounding that lands on the other side of a
tie moves one activation code."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import _lib as L
from qw38_b200 import synth
from qw38_b200.q4k_q8 import (PrefillWeight, Q4KError, hidden_rms_q8, q4k_q8_mlp, q8_mlp_workspace_bytes,
                              swiglu_pack_q8)
from tests.helpers import assert_close_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"
HIDDEN, FFN = 512, 1024


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def make_weight(n, k, seed):
    codes, meta = synth.logical_q4k(n, k, seed=seed)
    hc, hs = synth.split_tiles(codes, meta)
    return PrefillWeight.from_host(hc, hs, n, k), hc, hs


@pytest.fixture(scope="module")
def mlp():
    return make_weight(FFN, HIDDEN, 1), make_weight(FFN, HIDDEN, 2), make_weight(HIDDEN, FFN, 3)


def cpu_chain(mlp, h, gamma_bits, eps):
    (_, gc, gs), (_, uc, us), (_, dc, ds) = mlp
    xb = orc.hidden_rms_bf16(h, gamma_bits, eps)
    z, a, s, f1 = orc.q8_quantize(xb, bf16_bits=True)
    g = orc.project(gc, gs, FFN, HIDDEN, z, a, s)
    u = orc.project(uc, us, FFN, HIDDEN, z, a, s)
    vb = orc.swiglu_bf16(g, u)
    z2, a2, s2, f2 = orc.q8_quantize(vb, bf16_bits=True)
    return orc.project(dc, ds, HIDDEN, FFN, z2, a2, s2, residual=h), (f1 | f2)


def inputs(m, seed=0):
    h = synth.activations(m, HIDDEN, seed=seed, scale=2.0)
    gamma = synth.f32_to_bf16_bits((np.random.default_rng(seed).standard_normal(HIDDEN) * 0.1).astype(np.float32))
    return h, gamma


@pytest.mark.parametrize("m", [1, 3, 40, 130])
def test_mlp_chain_matches_cpu_chain(mlp, m):
    h, gamma = inputs(m, seed=m)
    ref, bad = cpu_chain(mlp, h, gamma, 1e-6)
    assert not bad
    ws = torch.empty(q8_mlp_workspace_bytes(m, HIDDEN, FFN), dtype=torch.uint8, device=DEV)
    out = torch.empty((m, HIDDEN), dtype=torch.float32, device=DEV)
    hd, gd = dev(h), dev(gamma.view(np.int16)).view(torch.bfloat16)
    assert q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], hd, gd, 1e-6, out, m, ws) is True
    assert_close_reference(out.cpu().numpy(), ref)
    # enqueue-only form with a caller-owned sticky flag: same numbers, flag stays clear
    pending = torch.zeros(1, dtype=torch.int32, device=DEV)
    out2 = torch.empty_like(out)
    q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], hd, gd, 1e-6, out2, m, ws, pending_failure=pending)
    assert torch.equal(out2, out) and pending.item() == 0


def test_rms_and_swiglu_producers(mlp):
    m = 9
    h, gamma = inputs(m, seed=3)
    h[1] = 0.0                                  # zero row: scale floor of 1
    h[2] *= 1e18                                # large magnitudes survive the max-scaling
    h[3] *= 1e-20
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = hidden_rms_q8(dev(h), dev(gamma.view(np.int16)).view(torch.bfloat16), 1e-6, f)
    xb = orc.hidden_rms_bf16(h, gamma, 1e-6)
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    z = q.codes.cpu().numpy()
    assert f.item() == 0
    diff = np.abs(z.astype(np.int32) - rz.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3, "codes differ only where a bf16 tie fell the other way"
    g = synth.activations(m, FFN, seed=5, scale=3.0)
    u = synth.activations(m, FFN, seed=6, scale=3.0)
    q2 = swiglu_pack_q8(dev(g), dev(u), f)
    rz2, ra2, rs2, _ = orc.q8_quantize(orc.swiglu_bf16(g, u), bf16_bits=True)
    d2 = np.abs(q2.codes.cpu().numpy().astype(np.int32) - rz2.astype(np.int32))
    assert f.item() == 0 and d2.max() <= 1 and (d2 != 0).mean() < 2e-3
    g[0, 0] = np.inf                            # a finite product must not mask a non-finite gate
    u[0, 0] = 0.0
    q3 = swiglu_pack_q8(dev(g), dev(u), f)
    assert f.item() == 1 and torch.isnan(q3.scales[0, 0]).item()


def test_mlp_failure_protocol(mlp):
    m = 4
    h, gamma = inputs(m, seed=8)
    ws = torch.empty(q8_mlp_workspace_bytes(m, HIDDEN, FFN), dtype=torch.uint8, device=DEV)
    out = torch.full((m, HIDDEN), 7.0, dtype=torch.float32, device=DEV)
    gd = dev(gamma.view(np.int16)).view(torch.bfloat16)
    # pre-launch rejection: nothing submitted, output untouched
    with pytest.raises(Q4KError) as e:
        q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], dev(h), gd, 1e-6, out, m, ws[:-8])
    assert e.value.code == L.ERR_INVALID_ARGUMENT and e.value.submitted is False
    assert (out == 7.0).all().item()
    with pytest.raises(Q4KError) as e:
        q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], dev(h), gd, -1.0, out, m, ws)
    assert e.value.submitted is False
    with pytest.raises(Q4KError) as e:      # output aliases the residual
        hd = dev(h)
        q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], hd, gd, 1e-6, hd, m, ws)
    assert e.value.submitted is False
    # post-launch failure: a NaN in the residual stream
    h[2, 5] = np.nan
    with pytest.raises(Q4KError) as e:
        q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], dev(h), gd, 1e-6, out, m, ws)
    assert e.value.code == L.ERR_INVALID_ARGUMENT and e.value.submitted is True and "nonfinite" in e.value.message
    pending = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], dev(h), gd, 1e-6, out, m, ws, pending_failure=pending)
    assert pending.item() == 1
    # the synchronous form refuses a capturing stream
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        g = torch.cuda.CUDAGraph()
        h2, _ = inputs(m, seed=9)
        hd = dev(h2)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            with pytest.raises(Q4KError):
                q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], hd, gd, 1e-6, out, m, ws)
            pending.zero_()
            q4k_q8_mlp(mlp[0][0], mlp[1][0], mlp[2][0], hd, gd, 1e-6, out, m, ws, pending_failure=pending)
        g.replay()
        torch.cuda.synchronize()
        ref, _ = cpu_chain(mlp, h2, gamma, 1e-6)
        assert_close_reference(out.cpu().numpy(), ref)


@pytest.mark.parametrize("m,hidden,ffn", [(1, 512, 1024), (8, 512, 1024), (16, 512, 1024), (5, 5120, 17408), (16, 5120, 17408)])
def test_mlp_fused_gate_up_activation_is_bitwise_the_unfused_one(m, hidden, ffn):
    """Up to sixteen tokens the chain runs gate, up and the SwiGLU -> Q8 pack as one launch whose reducer quantises.
    The Q8 activation it leaves in the workspace (codes, scales, sums of the down projection's input) must equal,
    bit for bit, what the separate launches produce: RMS + pack, two projections, swiglu_pack."""
    from qw38_b200.q4k_q8 import q4k_q8_project
    gate, up, down = (synth.device_weight(ffn, hidden, seed=11), synth.device_weight(ffn, hidden, seed=12),
                      synth.device_weight(hidden, ffn, seed=13))
    h = synth.activations(m, hidden, seed=m, scale=2.0)
    gamma = synth.f32_to_bf16_bits((np.random.default_rng(m).standard_normal(hidden) * 0.1).astype(np.float32))
    hd, gd = dev(h), dev(gamma.view(np.int16)).view(torch.bfloat16)
    ws = torch.zeros(q8_mlp_workspace_bytes(m, hidden, ffn), dtype=torch.uint8, device=DEV)
    out = torch.empty((m, hidden), dtype=torch.float32, device=DEV)
    assert q4k_q8_mlp(gate, up, down, hd, gd, 1e-6, out, m, ws) is True
    codes = ws[: m * ffn].view(torch.int8).view(m, ffn).clone()
    scales = ws[m * ffn: m * ffn + m * (ffn // 32) * 4].view(torch.float32).view(m, ffn // 32).clone()
    sums = ws[m * ffn + m * (ffn // 32) * 4: m * ffn + m * (ffn // 32) * 8].view(torch.int32).view(m, ffn // 32).clone()
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    xh = hidden_rms_q8(hd, gd, 1e-6, f)
    g = q4k_q8_project(gate, xh, kernel=L.KERNEL_GEMV_TMA)
    u = q4k_q8_project(up, xh, kernel=L.KERNEL_GEMV_TMA)
    q = swiglu_pack_q8(g, u, f)
    assert f.item() == 0
    assert torch.equal(codes, q.codes) and torch.equal(sums, q.sums) and torch.equal(scales, q.scales)
    ref = q4k_q8_project(down, q, residual=hd)
    assert torch.equal(out, ref)
