"""GPU parity tests of what the benchmark times and of the library's scratch, status and validation rules:
the full prefill shapes (sampled rows and a partial-dot dump), the MLP chain at the model's widths, the row-sharded
projection for more than sixteen tokens, activation scales beyond the fast path's exponent range, split-K scratch
under graph capture, and caller-workspace / static-entry pointer checks.  Everything goes through the C ABI; the CPU
oracle is the checker."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import _lib as L
from qw38_b200 import synth
from qw38_b200.q4k_q8 import (PrefillWeight, Q4KError, new_q8_input, pack_q8, q4k_q8_mlp, q4k_q8_project,
                              q4k_q8_project_static, q8_mlp_workspace_bytes, reserve_scratch)
from tests.helpers import assert_close_contract, assert_close_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(DEV).view(torch.bfloat16)


def flag() -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def kernel_status() -> int:
    v = ctypes.c_int(-1)
    assert L.load().q4k_kernel_status(ctypes.byref(v)) == 0
    return v.value


@pytest.mark.parametrize("m,n,k", [(2048, 17408, 5120), (8192, 17408, 5120)])
def test_timed_prefill_shapes_sampled(m, n, k):
    """The two largest shapes the benchmark times (64 token tiles x 136 row tiles in a persistent walk at m = 8192):
    sampled output rows over ALL tokens against the oracle, and a bit-exact partial dump of a 16-row slice."""
    w = synth.device_weight(n, k, seed=17)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=3, scale=0.5, outlier_frac=0.01))
    f = flag()
    q = pack_q8(bf16_tensor(xb), f)
    z, a, s, bad = orc.q8_quantize(xb, bf16_bits=True)
    assert f.item() == 0 and bad == 0 and (q.codes.cpu().numpy() == z).all()
    y = q4k_q8_project(w, q)
    for r0 in (0, 8 * 1000, n - 8):     # first tile, an interior tile, the last row group
        ws = w.row_slice(r0, 8)
        ref = orc.project_rows(ws.codes.cpu().numpy(), ws.scales.cpu().numpy(), 8, k, z, a, s, 0, 8)
        got = y[:, r0:r0 + 8].cpu().numpy()
        assert_close_reference(got, ref)
        assert_close_contract(got, ref)
    r0 = n // 2
    ws = w.row_slice(r0, 16)
    mt = 512                            # tokens of the dump: the first four token tiles
    part = torch.empty((mt, 16, k // 32), dtype=torch.int32, device=DEV)
    q4k_q8_project(ws, q.rows(0, mt), kernel=L.KERNEL_TCGEN05, partials=part)
    assert (part.cpu().numpy() == orc.dots(ws.codes.cpu().numpy(), 16, k, z[:mt])).all(), "bit-exact K32 partial dots"
    assert kernel_status() == 0


@pytest.mark.parametrize("m", [1, 127, 128, 512])
def test_mlp_chain_at_model_widths(m):
    """q4k_q8_mlp at hidden 5120 / ffn 17408 for the token counts of the reference's integration test
    (tests/q8_mlp_integration_test.cpp:75-80); the CPU chain is evaluated on sampled output rows of `down`."""
    hidden, ffn = 5120, 17408
    gate, up, down = (synth.device_weight(ffn, hidden, seed=41), synth.device_weight(ffn, hidden, seed=42),
                      synth.device_weight(hidden, ffn, seed=43))
    h = synth.activations(m, hidden, seed=m, scale=2.0)
    gamma = synth.f32_to_bf16_bits((np.random.default_rng(5).standard_normal(hidden) * 0.1).astype(np.float32))
    ws = torch.empty(q8_mlp_workspace_bytes(m, hidden, ffn), dtype=torch.uint8, device=DEV)
    out = torch.empty((m, hidden), dtype=torch.float32, device=DEV)
    hd = torch.from_numpy(h).to(DEV)
    assert q4k_q8_mlp(gate, up, down, hd, bf16_tensor(gamma), 1e-6, out, m, ws)
    # CPU chain: every gate/up row is needed (down contracts over all of ffn), so the host does the two big
    # projections in full once and `down` on sampled rows.
    xb = orc.hidden_rms_bf16(h, gamma, 1e-6)
    z, a, s, f1 = orc.q8_quantize(xb, bf16_bits=True)
    g = orc.project(gate.codes.cpu().numpy(), gate.scales.cpu().numpy(), ffn, hidden, z, a, s)
    u = orc.project(up.codes.cpu().numpy(), up.scales.cpu().numpy(), ffn, hidden, z, a, s)
    vb = orc.swiglu_bf16(g, u)
    z2, a2, s2, f2 = orc.q8_quantize(vb, bf16_bits=True)
    assert not (f1 | f2)
    got = out.cpu().numpy()
    # The SwiGLU producer rounds to bf16 before it quantises; where the device's and the host's exponential differ in
    # the last bit a bf16 tie falls the other way and ONE activation code of the 17408 moves by one.  That shifts an
    # output by one quantum of its group (up to about 1e-3 of the row's rms here), which the reference's 0.002|ref| does not
    # cover for outputs that cancel to near zero -- so the bound carries that quantum explicitly.
    for r0 in (0, 2560, hidden - 8):
        dsl = down.row_slice(r0, 8)
        ref = orc.project_rows(dsl.codes.cpu().numpy(), dsl.scales.cpu().numpy(), 8, ffn, z2, a2, s2, 0, 8) + h[:, r0:r0 + 8]
        err = np.abs(got[:, r0:r0 + 8].astype(np.float64) - ref)
        rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
        assert (err <= 0.02 + 0.002 * np.abs(ref) + 2e-3 * rms).all(), float((err / (np.abs(ref) + rms)).max())
    assert kernel_status() == 0


@pytest.mark.parametrize("m", [17, 64, 130])
def test_wide_activation_scales_take_the_slow_path(m):
    """The tensor-core kernel folds 2^49 into the activation scale; a scale beyond 2^78 would overflow there, and the
    affected super-blocks switch to the plain scales.  Rows with |x| up to 1e30 must still match the oracle."""
    n, k = 264, 1280
    codes, meta = synth.logical_q4k(n, k, seed=4)
    hc, hs = synth.split_tiles(codes, meta)
    w = PrefillWeight.from_host(hc, hs, n, k)
    x = synth.activations(m, k, seed=11)
    x[0, :] *= 1e30          # a whole token far outside the usual range
    x[m // 2, 300:340] *= 3e28   # one K32 group and a bit of an odd super-block
    x[m - 1, 1000] = 2e29
    f = flag()
    q = pack_q8(torch.from_numpy(x).to(DEV), f)
    z, a, s, _ = orc.q8_quantize(x)
    assert f.item() == 0 and a.max() > 2.0 ** 78
    part = torch.empty((m, n, k // 32), dtype=torch.int32, device=DEV)
    y = q4k_q8_project(w, q, kernel=L.KERNEL_TCGEN05, partials=part).cpu().numpy()
    assert (part.cpu().numpy() == orc.dots(hc, n, k, z)).all()
    ref = orc.project(hc, hs, n, k, z, a, s).astype(np.float64)
    assert np.isfinite(y).all()
    err = np.abs(y - ref)
    rms = np.sqrt((ref ** 2).mean(axis=1, keepdims=True))
    assert (err <= 2e-3 * np.maximum(np.abs(ref), 1e-3 * rms)).all()
    assert kernel_status() == 0


@pytest.mark.parametrize("m,k,world", [(17, 5120, 2), (64, 5120, 4), (130, 2560, 3)])
def test_project_gather_beyond_sixteen_tokens(m, k, world):
    """Row shards through the tensor-core kernel, whose writer stores into every rank's copy of the output and counts the
    projection as delivered.  Ranks are emulated on one GPU, one launch after the other (nothing waits on a kernel that
    has not run); every copy is compared with the oracle on sampled rows and with the unsharded projection."""
    from qw38_b200.q4k_q8 import peer_announce, peer_wait, q4k_q8_project_gather
    from qw38_b200.sharding import row_shard
    n = 2000
    w = synth.device_weight(n, k, seed=world + 10)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
    q = pack_q8(bf16_tensor(xb), flag())
    z, a, s, _ = orc.q8_quantize(xb, bf16_bits=True)
    full = q4k_q8_project(w, q)
    outs = [torch.full((m, n), -9.0, dtype=torch.float32, device=DEV) for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(world)]
    optr, fptr = [t.data_ptr() for t in outs], [t.data_ptr() for t in flags]
    for rnd in range(2):
        for rank in range(world):
            row0, rows, _ = row_shard(n, world, rank)
            q4k_q8_project_gather(w.row_slice(row0, rows), q, optr, fptr, rank, row0, n)
        for rank in range(world):
            peer_announce(fptr, rank)
        for rank in range(world):
            peer_wait(fptr, rank)
        torch.cuda.synchronize()
        for gidx in range(world):
            assert flags[gidx][:world].tolist() == [rnd + 1] * world
            got = outs[gidx].cpu().numpy()
            assert_close_contract(got, full.cpu().numpy())
            for r0 in (0, 992, n - 8):
                wsl = w.row_slice(r0, 8)
                ref = orc.project_rows(wsl.codes.cpu().numpy(), wsl.scales.cpu().numpy(), 8, k, z, a, s, 0, 8)
                assert_close_reference(got[:, r0:r0 + 8], ref)
            outs[gidx].fill_(-9.0)
    assert kernel_status() == 0


def test_scratch_growth_leaves_captured_graphs_valid():
    """A decode graph that uses the library's split-K scratch, then a larger call that makes the scratch grow, then the
    graph again: the block the graph captured must still be alive (blocks are retired, never freed), and the replay must
    reproduce the first result bit for bit.  Growth while a stream is capturing is refused with a clear message."""
    w = synth.device_weight(640, 17408, seed=2)
    xb = synth.f32_to_bf16_bits(synth.activations(8, 17408, seed=2))
    q = pack_q8(bf16_tensor(xb), flag())
    out = torch.zeros((8, 640), dtype=torch.float32, device=DEV)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        q4k_q8_project(w, q, out=out, kernel=L.KERNEL_GEMV_TMA, split_k=4)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            q4k_q8_project(w, q, out=out, kernel=L.KERNEL_GEMV_TMA, split_k=4)
        graph.replay()
    stream.synchronize()
    first = out.clone()
    # 16 slices x 512 x 5120 x 4 bytes = 168 MB of partial tiles: far beyond the initial 8 MiB
    big_w = synth.device_weight(5120, 17408, seed=3)
    big_q = pack_q8(bf16_tensor(synth.f32_to_bf16_bits(synth.activations(512, 17408, seed=4, scale=0.5))), flag())
    y = q4k_q8_project(big_w, big_q, kernel=L.KERNEL_TCGEN05, split_k=16)
    torch.cuda.synchronize()
    out.zero_()
    with torch.cuda.stream(stream):
        graph.replay()
    stream.synchronize()
    assert torch.equal(out, first), "the captured scratch block is still valid after the scratch grew"
    z, a, s, _ = orc.q8_quantize(synth.f32_to_bf16_bits(synth.activations(512, 17408, seed=4, scale=0.5)), bf16_bits=True)
    wsl = big_w.row_slice(0, 8)
    assert_close_reference(y[:, :8].cpu().numpy(), orc.project_rows(wsl.codes.cpu().numpy(), wsl.scales.cpu().numpy(), 8, 17408, z, a, s, 0, 8))
    # growth during capture: refused before anything is enqueued; q4k_reserve_scratch ahead of time makes it legal
    huge_q = pack_q8(bf16_tensor(synth.f32_to_bf16_bits(synth.activations(1024, 17408, seed=5, scale=0.5))), flag())
    o2 = torch.zeros((1024, 5120), dtype=torch.float32, device=DEV)
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(g2, stream=stream):
            o2.zero_()
            with pytest.raises(Q4KError) as e:
                q4k_q8_project(big_w, huge_q, out=o2, kernel=L.KERNEL_TCGEN05, split_k=16)
        assert "q4k_reserve_scratch" in e.value.message
    torch.cuda.synchronize()
    reserve_scratch(16 * 1024 * 5120 * 4)
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        q4k_q8_project(big_w, huge_q, out=o2, kernel=L.KERNEL_TCGEN05, split_k=16)
        stream.synchronize()
        with torch.cuda.graph(g3, stream=stream):
            q4k_q8_project(big_w, huge_q, out=o2, kernel=L.KERNEL_TCGEN05, split_k=16)
        g3.replay()
    stream.synchronize()
    assert kernel_status() == 0


@pytest.mark.parametrize("kern,m", [(L.KERNEL_GEMV_TMA, 8), (L.KERNEL_TCGEN05, 64), (L.KERNEL_MMA, 64)])
def test_caller_workspace_is_validated_on_every_kernel_family(kern, m):
    """A host pointer, a misaligned pointer or a short buffer as split-K workspace is an invalid argument on every
    branch, not a fault on the GPU; a good workspace gives the library-scratch result bit for bit."""
    n, k, split = 640, 5120, 4
    w = synth.device_weight(n, k, seed=6)
    q = pack_q8(bf16_tensor(synth.f32_to_bf16_bits(synth.activations(m, k, seed=6))), flag())
    want = q4k_q8_project(w, q, kernel=kern, split_k=split)
    need = L.load().q4k_project_workspace_bytes(m, n, split)
    good = torch.empty(need + 256, dtype=torch.uint8, device=DEV)
    got = q4k_q8_project(w, q, kernel=kern, split_k=split, workspace=good[:need])
    assert torch.equal(got, want)
    host = torch.empty(need, dtype=torch.uint8).pin_memory()
    for bad in (good[1:need + 1], good[:need - 4096], host):
        with pytest.raises(Q4KError) as e:
            q4k_q8_project(w, q, kernel=kern, split_k=split, workspace=bad)
        assert e.value.code == L.ERR_INVALID_ARGUMENT
    assert kernel_status() == 0


def test_static_entry_rejects_host_and_foreign_pointers():
    """The no-allocation entry runs the same operand checks as the allocating one: a host pointer (pinned memory is
    reachable from the GPU, so it would not even fault) is rejected before anything is launched."""
    n, k, m = 640, 2560, 16
    w = synth.device_weight(n, k, seed=8)
    q = pack_q8(bf16_tensor(synth.f32_to_bf16_bits(synth.activations(m, k, seed=8))), flag())
    host_out = torch.zeros((m, n), dtype=torch.float32).pin_memory()
    with pytest.raises(Q4KError) as e:
        q4k_q8_project_static(w, q, out=host_out, split_k=2)
    assert e.value.code == L.ERR_INVALID_ARGUMENT and "device memory" in e.value.message
    assert not host_out.any().item()
    host_q = new_q8_input(m, k, "cpu")
    with pytest.raises(Q4KError):
        q4k_q8_project_static(w, host_q, out=torch.zeros((m, n), dtype=torch.float32, device=DEV), split_k=2)
    out = torch.zeros((m, n), dtype=torch.float32, device=DEV)
    with pytest.raises(Q4KError):
        q4k_q8_project_static(w, q, out=out.view(-1)[: m * n - 1].view(-1), split_k=2)   # short output


def test_launch_overlap_with_settled_inputs_is_bitwise_the_serial_result():
    """Programmatic dependent launch through the tcgen05 kernel (and the decode kernel) with
    Q4K_FLAG_INPUT_SETTLED: both activation packs are enqueued before the projections, so no projection's
    input is the work of the launch directly before it, and the projections may compute beside their
    predecessors.  Chains of projections of different sizes -- few tiles (SMs left idle for the successor),
    split-K through the shared scratch and tickets, a residual -- must reproduce the serial results bit for
    bit, eagerly and as a replayed CUDA graph."""
    from qw38_b200 import set_launch_overlap, launch_overlap
    from qw38_b200.q4k_q8 import new_q8_input
    shapes = [(7168, 5120), (640, 5120), (34816 // 4, 5120), (1024, 17408), (5120, 5120)]
    ws = [synth.device_weight(n, k, seed=70 + i) for i, (n, k) in enumerate(shapes)]
    f = torch.zeros(1, dtype=torch.int32, device=DEV)
    tokens = (64, 40, 8, 1)
    xs = {m: {k: (torch.randn((m, k), device=DEV, generator=torch.Generator(device=DEV).manual_seed(m + k)) * 0.7).to(torch.bfloat16)
              for k in (5120, 17408)} for m in tokens}
    qs = {m: {k: new_q8_input(m, k) for k in (5120, 17408)} for m in tokens}
    res = {m: torch.randn((m, shapes[4][0]), device=DEV) for m in tokens}
    outs = {(m, i): torch.empty((m, n), dtype=torch.float32, device=DEV) for m in tokens for i, (n, _) in enumerate(shapes)}

    def chain(settled):
        for m in tokens:
            for k in (5120, 17408):
                pack_q8(xs[m][k], f, out=qs[m][k])
            for i, (n, k) in enumerate(shapes):
                q4k_q8_project(ws[i], qs[m][k], out=outs[(m, i)], residual=res[m] if i == 4 else None, trusted=True,
                               kernel=L.KERNEL_GEMV_TMA if m <= 16 else L.KERNEL_TCGEN05, input_settled=settled)

    assert not launch_overlap()
    chain(False)
    torch.cuda.synchronize()
    want = {key: t.clone() for key, t in outs.items()}
    try:
        set_launch_overlap(True)
        for settled in (False, True):
            for t in outs.values():
                t.fill_(-3.0)
            for _ in range(3):
                chain(settled)
            torch.cuda.synchronize()
            for key in outs:
                assert torch.equal(outs[key], want[key]), f"eager overlap (settled={settled}) differs at {key}"
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            chain(True)
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                chain(True)
                chain(True)
            for t in outs.values():
                t.fill_(-3.0)
            for _ in range(3):
                g.replay()
            stream.synchronize()
        for key in outs:
            assert torch.equal(outs[key], want[key]), f"graph overlap differs at {key}"
    finally:
        set_launch_overlap(False)
    assert f.item() == 0
    st = ctypes.c_int(0)
    L.load().q4k_kernel_status(ctypes.byref(st))
    assert st.value == 0
