"""GPU parity tests of the Q8 quantiser and the Q4_K x Q8 projection, through the C ABI.

The first block follows the reference's own tests/q4k_q8_test.cpp case by case (same matrix,
same activations, same token counts, same assertions); the rest covers the benchmark shapes.
Integer results (codes, sums, K32 partial dots) must be bit-exact against the CPU oracle;
fp32 outputs are held to the reference's 0.02+0.002|ref| and to the 2e-3 / 1e-4*||row|| contract."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from qw38_b200 import _lib as L
from qw38_b200 import synth
from qw38_b200.q4k_q8 import (PrefillWeight, Q4KError, Q8Input, export_q8_1, new_q8_input, pack_q8,
                              q4k_q8_project, q4k_q8_project_ragged, repack_blocks144)
from tests.helpers import assert_close_contract, assert_close_reference
from tests.test_oracle_pins import reference_test_input

pytestmark = pytest.mark.gpu
DEV = "cuda"


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def flag() -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return dev(bits.view(np.int16)).view(torch.bfloat16)


def host_q8(q: Q8Input):
    return q.codes.cpu().numpy(), q.scales.cpu().numpy(), q.sums.cpu().numpy()


@pytest.fixture(scope="module")
def fixture_a(golden):
    n, k = 137, 259
    w = PrefillWeight.from_host(golden["a_packed_codes"], golden["a_packed_scales"], n, k)
    return w, golden["a_packed_codes"], golden["a_packed_scales"]


def kernels_for(m):
    return (([L.KERNEL_GEMV_DP4A] if m <= 4 else []) + ([L.KERNEL_GEMV_MMA, L.KERNEL_GEMV_TMA] if m <= 16 else []) +
            [L.KERNEL_MMA, L.KERNEL_TCGEN05])


def kernel_status() -> int:
    import ctypes
    v = ctypes.c_int(-1)
    assert L.load().q4k_kernel_status(ctypes.byref(v)) == 0
    return v.value


SMALL_TILE = {}


@pytest.mark.parametrize("m", [1, 3, 33, 127, 128, 129, 256, 257, 511, 512])
def test_reference_case(fixture_a, m):
    w, hc, hs = fixture_a
    n, k, pk, G = 137, 259, 512, 16
    xb = reference_test_input(m, k)
    x = bf16_tensor(xb)
    f = flag()
    q = pack_q8(x, f)
    z, a, s = host_q8(q)
    rz, ra, rs, rf = orc.q8_quantize(xb, bf16_bits=True)
    assert f.item() == 0 and rf == 0                                       # finite pack
    assert (z == rz).all(), "exact codes, RNE and padding"
    assert (a.view(np.uint32) == ra.view(np.uint32)).all() and (s == rs).all(), "exact scales/sums"
    assert list(z[0, :5]) == [127, 0, 2, 0, -2], "halfway ties and saturation endpoint"
    assert s[0, 2] < 0
    y = q4k_q8_project(w, q).cpu().numpy()
    ref = orc.project(hc, hs, n, pk, rz, ra, rs)
    assert_close_reference(y, ref)
    assert_close_contract(y, ref)
    ref_dots = orc.dots(hc, n, pk, rz)
    assert np.abs(ref_dots).max() <= 32 * 15 * 127
    for kern in kernels_for(m):
        part = torch.full((m, n, G), -7, dtype=torch.int32, device=DEV)
        yk = q4k_q8_project(w, q, kernel=kern, partials=part).cpu().numpy()
        assert (part.cpu().numpy() == ref_dots).all(), f"bit-exact K32 partial dots, kernel {kern}"
        assert_close_reference(yk, ref)
    if m == 1:
        # 16-byte fast loads vs spans that are only 4-byte aligned; guard words at both ends.
        shifted_w = torch.zeros(w.codes.numel() + 8, dtype=torch.uint8, device=DEV)
        shifted_w[4:-4] = w.codes
        shifted_m = torch.zeros(w.scales.numel() + 4, dtype=torch.uint8, device=DEV)
        shifted_m[2:-2] = w.scales
        shifted_z = torch.full((pk + 8,), 99, dtype=torch.int8, device=DEV)
        shifted_z[4:-4] = q.codes[0]
        residual = dev(((np.arange(n) % 17) - 8).astype(np.float32) * 0.125)
        tma_kernels = (L.KERNEL_TCGEN05, L.KERNEL_GEMV_TMA)
        for kern in tma_kernels:        # TMA needs 16-byte aligned operands: a clear rejection, not a fault
            with pytest.raises(Q4KError):
                q4k_q8_project(PrefillWeight(shifted_w[4:-4], w.scales, n, k), q, kernel=kern)
        for kern in [L.KERNEL_AUTO] + [kk for kk in kernels_for(1) if kk not in tma_kernels]:
            base = q4k_q8_project(w, q, kernel=kern).cpu().numpy()[0]
            for variant in range(8):
                ww = PrefillWeight(shifted_w[4:-4] if variant & 1 else w.codes,
                                   shifted_m[2:-2] if variant & 4 else w.scales, n, k)
                qq = Q8Input(shifted_z[4:-4].view(1, pk) if variant & 2 else q.codes, q.scales, q.sums, 1, k, pk)
                guarded = torch.full((n + 2,), -12345.0, dtype=torch.float32, device=DEV)
                q4k_q8_project(ww, qq, out=guarded[1:-1].view(1, n), residual=residual.view(1, n), kernel=kern)
                got = guarded.cpu().numpy()
                assert (got[1:-1] == base + residual.cpu().numpy()).all(), "aligned/unaligned loads and residual agree exactly"
                assert got[0] == -12345.0 and got[-1] == -12345.0, "row-tail output guards"
    if m == 127:
        SMALL_TILE["y"] = y
    if m >= 128 and "y" in SMALL_TILE:
        assert (y[:127] == SMALL_TILE["y"]).all(), "rows do not depend on the token count"
    y2 = q4k_q8_project(w, q).cpu().numpy()
    assert (y2 == y).all(), "reused pack gives identical output"
    assert kernel_status() == 0, "no bounded wait inside a kernel gave up"
    z2, a2, s2 = host_q8(q)
    assert (z2 == z).all() and (a2.view(np.uint32) == a.view(np.uint32)).all() and (s2 == s).all(), "consumer preserves the pack"
    bad = Q8Input(q.codes.view(-1)[:1], q.scales, q.sums, m, k, pk)
    with pytest.raises(Q4KError) as e:
        q4k_q8_project(w, bad)
    assert e.value.code == L.ERR_INVALID_ARGUMENT
    badw = PrefillWeight(w.codes, w.scales, n, k, codes_bytes=w.codes.numel() - 1)
    with pytest.raises(Q4KError):
        q4k_q8_project(badw, q)
    for bits in (0x7F80, 0xFF80, 0x7FC0):
        xb2 = xb.copy()
        xb2[0, 0] = bits
        f.zero_()
        q2 = pack_q8(bf16_tensor(xb2), f)
        assert f.item() == 1 and torch.isnan(q2.scales[0, 0]).item(), "non-finite pack rejected, not finite zero"
        assert (q2.codes[0, :32] == 0).all().item()


def test_pack_rejects_bad_spans(fixture_a):
    x = torch.zeros((4, 259), dtype=torch.bfloat16, device=DEV)
    q = new_q8_input(4, 259)
    with pytest.raises(Q4KError):
        pack_q8(x, torch.zeros(1, dtype=torch.int32), out=q)            # host flag pointer
    with pytest.raises(Q4KError):
        pack_q8(x, q.sums.view(-1)[:1], out=q)                          # flag aliases an output
    big = torch.zeros(8, dtype=torch.int32, device=DEV)
    with pytest.raises(Q4KError):
        pack_q8(x, big.view(torch.int8)[1:5], out=q)                    # misaligned flag


@pytest.mark.parametrize("m,k", [(1, 5120), (5, 300), (16, 17408), (64, 1000)])
def test_pack_fp32_and_bf16_tails(m, k):
    x = synth.activations(m, k, seed=m + k, scale=3.0)
    x[0, : min(k, 32)] = 0.0                                              # a zero group
    x[-1, -1] = 1e-30
    for bits in (False, True):
        f = flag()
        if bits:
            xb = synth.f32_to_bf16_bits(x)
            q = pack_q8(bf16_tensor(xb), f)
            rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
        else:
            q = pack_q8(dev(x), f)
            rz, ra, rs, _ = orc.q8_quantize(x)
        z, a, s = host_q8(q)
        assert f.item() == 0
        assert (z == rz).all() and (a.view(np.uint32) == ra.view(np.uint32)).all() and (s == rs).all()


def test_q8_1_export_bit_exact():
    x = synth.activations(3, 5120, seed=8)
    q = pack_q8(dev(x), flag())
    rec = export_q8_1(q).cpu().numpy()
    z, a, s = host_q8(q)
    assert (rec == orc.q8_1_export(z, a, s)).all()


def test_repack_blocks144_bit_exact(golden):
    blocks = golden["b_blocks144"]
    rows, kk = golden["b_fit_codes"].shape
    w = repack_blocks144(dev(blocks.reshape(-1)), rows, kk)
    oc, om = orc.blocks144_to_split(blocks, rows, kk)
    assert (w.codes.cpu().numpy() == oc).all() and (w.scales.cpu().numpy() == om).all()
    codes, meta = synth.logical_q4k(21, 512, seed=3)
    w2 = repack_blocks144(dev(synth.blocks144(codes, meta).reshape(-1)), 21, 512)
    oc2, om2 = synth.split_tiles(codes, meta)
    assert (w2.codes.cpu().numpy() == oc2).all() and (w2.scales.cpu().numpy() == om2).all()


def run_and_check(w: PrefillWeight, hc, hs, x_f32=None, x_bits=None, rows=None, kernels=None, partial_rows=256):
    """Project on the GPU, compare with the oracle on all rows (rows=None) or on a sample."""
    n, pk = w.n, w.padded_k
    if x_bits is not None:
        q = pack_q8(bf16_tensor(x_bits), flag())
        rz, ra, rs, _ = orc.q8_quantize(x_bits, bf16_bits=True)
    else:
        q = pack_q8(dev(x_f32), flag())
        rz, ra, rs, _ = orc.q8_quantize(x_f32)
    z, a, s = host_q8(q)
    assert (z == rz).all() and (a.view(np.uint32) == ra.view(np.uint32)).all() and (s == rs).all()
    m = q.m
    for kern in kernels or [L.KERNEL_AUTO]:
        y = q4k_q8_project(w, q, kernel=kern).cpu().numpy()
        if rows is None:
            ref = orc.project(hc, hs, n, pk, rz, ra, rs)
            assert_close_reference(y, ref)
            assert_close_contract(y, ref)
        else:
            for r0, cnt in rows:
                ref = orc.project_rows(hc, hs, n, pk, rz, ra, rs, r0, cnt)
                assert_close_reference(y[:, r0:r0 + cnt], ref)
                assert_close_contract(y[:, r0:r0 + cnt], ref)
        # bit-exact partial dots on a row slice (a row group run is a view of the matrix)
        r0 = (n // 2) // 8 * 8
        cnt = min(partial_rows, n - r0)
        ws = w.row_slice(r0, cnt)
        part = torch.empty((m, cnt, pk // 32), dtype=torch.int32, device=DEV)
        ys = q4k_q8_project(ws, q, kernel=kern, partials=part).cpu().numpy()
        sl = slice(r0 // 8 * (pk // 256) * 1024, None)
        ref_dots = orc.dots(hc[sl], cnt, pk, rz)
        assert (part.cpu().numpy() == ref_dots).all(), "bit-exact K32 partial dots"
        # the slice may split K differently from the full matrix, so fp32 bits can differ
        assert_close_contract(ys, y[:, r0:r0 + cnt])
    return q


def test_config0_single_gemv():
    """M=1, K=5120, N=17408, seed 0, fp32 activation."""
    codes, meta = synth.logical_q4k(17408, 5120, seed=0)
    hc, hs = synth.split_tiles(codes, meta)
    assert hc.size + hs.size == 50135040
    w = PrefillWeight.from_host(hc, hs, 17408, 5120)
    x = synth.activations(1, 5120, seed=0)
    run_and_check(w, hc, hs, x_f32=x, kernels=[L.KERNEL_AUTO, L.KERNEL_GEMV_DP4A, L.KERNEL_GEMV_MMA, L.KERNEL_GEMV_TMA, L.KERNEL_MMA])


@pytest.mark.parametrize("m", [1, 2, 4, 8, 16])
@pytest.mark.parametrize("name,n,k", [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120),
                                      ("down", 5120, 17408)])
def test_config1_decode_projection_set(name, n, k, m):
    w = synth.device_weight(n, k, seed=n + k)
    hc, hs = w.codes.cpu().numpy(), w.scales.cpu().numpy()
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
    sample = [(0, 64), (n // 2 + 8, 40), (n - 72, 72)]
    kernels = [L.KERNEL_AUTO, L.KERNEL_GEMV_MMA, L.KERNEL_GEMV_TMA, L.KERNEL_TCGEN05] + ([L.KERNEL_MMA] if m <= 4 else [])
    run_and_check(w, hc, hs, x_bits=xb, rows=sample, kernels=kernels, partial_rows=128)


@pytest.mark.parametrize("m,n,k", [(512, 17408, 5120), (512, 5120, 17408), (2048, 5120, 17408)])
def test_config2_prefill_shapes_sampled(m, n, k):
    """Prefill shapes with 1% outlier channels x20; rows sampled, all tokens."""
    w = synth.device_weight(n, k, seed=7)
    hc, hs = w.codes.cpu().numpy(), w.scales.cpu().numpy()
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=2, scale=0.5, outlier_frac=0.01))
    run_and_check(w, hc, hs, x_bits=xb, rows=[(8, 24), (n - 16, 16)], kernels=[L.KERNEL_AUTO, L.KERNEL_TCGEN05, L.KERNEL_MMA],
                  partial_rows=16)
    assert kernel_status() == 0


@pytest.mark.parametrize("kern", [L.KERNEL_MMA, L.KERNEL_TCGEN05])
@pytest.mark.parametrize("split_k", [1, 2, 3, 5, 20])
def test_split_k_is_deterministic_and_exact(split_k, kern):
    n, k, m = 640, 5120, 16
    w = synth.device_weight(n, k, seed=5)
    hc, hs = w.codes.cpu().numpy(), w.scales.cpu().numpy()
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=9))
    q = pack_q8(bf16_tensor(xb), flag())
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    ref = orc.project(hc, hs, n, 5120, rz, ra, rs)
    part = torch.empty((m, n, 160), dtype=torch.int32, device=DEV)
    res = dev(synth.activations(m, n, seed=4))
    y = q4k_q8_project(w, q, kernel=kern, split_k=split_k, partials=part, residual=res).cpu().numpy()
    assert_close_contract(y - res.cpu().numpy(), ref)
    assert (part.cpu().numpy() == orc.dots(hc, n, 5120, rz)).all()
    for _ in range(3):
        again = q4k_q8_project(w, q, kernel=kern, split_k=split_k, residual=res).cpu().numpy()
        assert (again == y).all(), "slice sums are added in slice order, whatever the arrival order"
    ws_bytes = L.load().q4k_project_workspace_bytes(m, n, split_k)
    if ws_bytes:
        ws = torch.full((ws_bytes,), 0xAB, dtype=torch.uint8, device=DEV)   # dirty caller workspace
        mine = q4k_q8_project(w, q, kernel=kern, split_k=split_k, residual=res, workspace=ws).cpu().numpy()
        assert (mine == y).all()
        with pytest.raises(Q4KError):
            q4k_q8_project(w, q, kernel=kern, split_k=split_k, workspace=ws[: ws_bytes // 2])


@pytest.mark.parametrize("m", [3, 8, 9, 16])
@pytest.mark.parametrize("split_k,row_groups", [(1, 4), (2, 8), (3, 4), (5, 8), (8, 4)])
def test_cluster_split_k_is_deterministic_and_exact(m, split_k, row_groups):
    """K slices inside a thread-block cluster, added in rank order through distributed shared memory."""
    n, k = 1000, 5120                     # n % 64 != 0: inactive warps and a ragged last row group
    codes, meta = synth.logical_q4k(n, k, seed=6)
    hc, hs = synth.split_tiles(codes, meta)
    w = PrefillWeight.from_host(hc, hs, n, k)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
    q = pack_q8(bf16_tensor(xb), flag())
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    ref = orc.project(hc, hs, n, k, rz, ra, rs)
    part = torch.empty((m, n, 160), dtype=torch.int32, device=DEV)
    res = dev(synth.activations(m, n, seed=4))
    guarded = torch.full((m * n + 2,), -5.0, dtype=torch.float32, device=DEV)
    y = q4k_q8_project(w, q, out=guarded[1:-1].view(m, n), kernel=L.KERNEL_GEMV_MMA, split_k=split_k,
                       row_groups=row_groups, partials=part, residual=res).cpu().numpy()
    assert guarded[0].item() == -5.0 and guarded[-1].item() == -5.0
    assert_close_contract(y - res.cpu().numpy(), ref)
    assert (part.cpu().numpy() == orc.dots(hc, n, k, rz)).all()
    for _ in range(2):
        again = q4k_q8_project(w, q, kernel=L.KERNEL_GEMV_MMA, split_k=split_k, row_groups=row_groups, residual=res)
        assert (again.cpu().numpy() == y).all()
    with pytest.raises(Q4KError):
        q4k_q8_project(w, q, kernel=L.KERNEL_GEMV_MMA, split_k=9)


@pytest.mark.parametrize("m,split_k,warps", [(1, 0, 0), (3, 1, 20), (7, 2, 0), (8, 3, 7), (8, 0, 5), (9, 0, 0), (13, 2, 12),
                                             (16, 4, 0), (16, 20, 0), (12, 1, 20), (16, 2, 0)])
def test_gemv_tma_plans(m, split_k, warps):
    """Weights streamed by TMA, activations in registers: K slices of any width, ragged last slice,
    odd number of row groups, partial dots bit-exact, two runs bitwise equal, status word clean."""
    n, k = 1000, 5120                     # 125 row groups: the last 16-row tile is half outside the matrix
    codes, meta = synth.logical_q4k(n, k, seed=6)
    hc, hs = synth.split_tiles(codes, meta)
    w = PrefillWeight.from_host(hc, hs, n, k)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
    q = pack_q8(bf16_tensor(xb), flag())
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    ref = orc.project(hc, hs, n, k, rz, ra, rs)
    part = torch.empty((m, n, 160), dtype=torch.int32, device=DEV)
    res = dev(synth.activations(m, n, seed=4))
    guarded = torch.full((m * n + 2,), -5.0, dtype=torch.float32, device=DEV)
    y = q4k_q8_project(w, q, out=guarded[1:-1].view(m, n), kernel=L.KERNEL_GEMV_TMA, split_k=split_k,
                       row_groups=warps, partials=part, residual=res).cpu().numpy()
    assert guarded[0].item() == -5.0 and guarded[-1].item() == -5.0
    assert_close_contract(y - res.cpu().numpy(), ref)
    assert (part.cpu().numpy() == orc.dots(hc, n, k, rz)).all()
    for _ in range(2):
        again = q4k_q8_project(w, q, kernel=L.KERNEL_GEMV_TMA, split_k=split_k, row_groups=warps, residual=res)
        assert (again.cpu().numpy() == y).all()
    assert kernel_status() == 0
    with pytest.raises(Q4KError):
        q4k_q8_project(w, pack_q8(bf16_tensor(synth.f32_to_bf16_bits(synth.activations(17, k, seed=1))), flag()),
                       kernel=L.KERNEL_GEMV_TMA)


def test_launch_overlap_gives_identical_results():
    """Programmatic dependent launch: kernels start (and the TMA kernel streams weights) while the one
    before drains.  A chain pack -> four projections per token count, eager and as a CUDA graph, must
    reproduce the serialised results bit for bit, split-K scratch and tickets included."""
    from qw38_b200 import set_launch_overlap, launch_overlap
    shapes = [(1000, 5120), (520, 5120), (2048, 5120), (512, 17408)]     # the last one splits K four ways
    ws = [synth.device_weight(n, k, seed=40 + i) for i, (n, k) in enumerate(shapes)]
    xs = {m: {k: bf16_tensor(synth.f32_to_bf16_bits(synth.activations(m, k, seed=m + k))) for k in (5120, 17408)}
          for m in (1, 3, 8, 16)}
    f = flag()
    qs = {m: {k: new_q8_input(m, k) for k in (5120, 17408)} for m in xs}
    # explicit kernels: automatic dispatch of a single token depends on the switch under test
    kerns = {m: [L.KERNEL_GEMV_TMA] + ([L.KERNEL_GEMV_DP4A] if m <= 4 else []) for m in xs}
    outs = {(m, i, kern): torch.empty((m, n), dtype=torch.float32, device=DEV)
            for m in xs for i, (n, _) in enumerate(shapes) for kern in kerns[m]}

    def chain():
        for m in xs:
            for k in (5120, 17408):
                pack_q8(xs[m][k], f, out=qs[m][k])
            for i, (n, k) in enumerate(shapes):
                for kern in kerns[m]:
                    q4k_q8_project(ws[i], qs[m][k], out=outs[(m, i, kern)], kernel=kern, trusted=True)

    assert not launch_overlap()
    chain()
    torch.cuda.synchronize()
    want = {key: t.clone() for key, t in outs.items()}
    try:
        set_launch_overlap(True)
        assert launch_overlap()
        for t in outs.values():
            t.fill_(-3.0)
        for _ in range(3):
            chain()
        torch.cuda.synchronize()
        for key in outs:
            assert torch.equal(outs[key], want[key]), f"eager overlap differs at {key}"
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            chain()
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                chain()
                chain()
            for t in outs.values():
                t.fill_(-3.0)
            for _ in range(3):
                g.replay()
            stream.synchronize()
        for key in outs:
            assert torch.equal(outs[key], want[key]), f"graph overlap differs at {key}"
    finally:
        set_launch_overlap(False)
    assert f.item() == 0 and kernel_status() == 0


@pytest.mark.parametrize("m,k,world", [(3, 5120, 3), (16, 5120, 2), (8, 17408, 4)])
def test_project_gather_emulated_ranks(m, k, world):
    """Row shards whose projection kernel stores into every rank's copy of the output and then bumps the
    rank's arrival counter.  The ranks are emulated on one GPU: peer buffers are just other tensors, and the
    launches run one after the other, so nothing ever waits on a kernel that has not run."""
    from qw38_b200.q4k_q8 import q4k_q8_project_gather, peer_announce, peer_wait
    from qw38_b200.sharding import row_shard
    n = 2000
    w = synth.device_weight(n, k, seed=world)
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=m))
    q = pack_q8(bf16_tensor(xb), flag())
    res = dev(synth.activations(m, n, seed=9))
    full = q4k_q8_project(w, q, residual=res, kernel=L.KERNEL_GEMV_TMA)
    outs = [torch.full((m, n), -9.0, dtype=torch.float32, device=DEV) for _ in range(world)]
    flags = [torch.zeros(16, dtype=torch.int32, device=DEV) for _ in range(world)]
    optr, fptr = [t.data_ptr() for t in outs], [t.data_ptr() for t in flags]
    for rnd in range(2):                      # counters keep counting across steps
        for rank in range(world):
            row0, rows, _ = row_shard(n, world, rank)
            q4k_q8_project_gather(w.row_slice(row0, rows), q, optr, fptr, rank, row0, n, residual=res)
        for rank in range(world):         # one stream plays every rank: all announce before anyone waits
            peer_announce(fptr, rank)
        for rank in range(world):
            peer_wait(fptr, rank)
        torch.cuda.synchronize()
        for g in range(world):
            assert flags[g][:world].tolist() == [rnd + 1] * world
            err = (outs[g] - full).abs().max().item()
            assert err <= 1e-4 * full.abs().max().item(), f"rank {g}: {err}"
            outs[g].fill_(-9.0)
    assert kernel_status() == 0
    # A peer that never delivers: the wait runs out after ~1 ms of SM clocks and reports it; the context stays usable.
    flags[0][1] -= 1
    peer_wait(fptr, 0, limit_cycles=2_000_000)
    assert kernel_status() == 0x610
    assert kernel_status() == 0, "the read clears the word"
    with pytest.raises(Q4KError):
        q4k_q8_project_gather(w.row_slice(0, 1000), q, optr, fptr, world, 0, n)          # rank outside the world
    with pytest.raises(Q4KError):
        q4k_q8_project_gather(w.row_slice(1000, 1000), q, optr, fptr, 0, 1004, n)        # shard would overrun total_rows


def ragged_offsets():
    lens = [1] * 48 + [512, 237, 1024]
    return np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)


def test_config3_ragged_batch_equals_unbatched():
    """48 decode rows + prefill chunks {512, 237, 1024} packed into M=1821; each request's rows
    equal the same rows run alone: bit-exact int32 partials, fp32 within the contract."""
    offs = ragged_offsets()
    m, k, n = int(offs[-1]), 5120, 512          # 512-row slice of the gate+up matrix for the partial dump
    assert m == 1821
    w = synth.device_weight(n, k, seed=21)
    hc, hs = w.codes.cpu().numpy(), w.scales.cpu().numpy()
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=12))
    q = pack_q8(bf16_tensor(xb), flag())
    part = torch.empty((m, n, 160), dtype=torch.int32, device=DEV)
    y = q4k_q8_project_ragged(w, q, [int(v) for v in offs], partials=part)
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    assert (part.cpu().numpy() == orc.dots(hc, n, k, rz)).all()
    ref = orc.project(hc, hs, n, k, rz, ra, rs)
    assert_close_contract(y.cpu().numpy(), ref)
    for r in [0, 17, 47, 48, 49, 50]:
        r0, r1 = int(offs[r]), int(offs[r + 1])
        qa = pack_q8(bf16_tensor(xb[r0:r1]), flag())                       # the request on its own
        pa = torch.empty((r1 - r0, n, 160), dtype=torch.int32, device=DEV)
        ya = q4k_q8_project(w, qa, partials=pa)
        assert torch.equal(pa, part[r0:r1]), "int32 partials identical batched and unbatched"
        assert torch.equal(qa.codes, q.codes[r0:r1]) and torch.equal(qa.sums, q.sums[r0:r1])
        assert_close_contract(ya.cpu().numpy(), ref[r0:r1])
        assert_close_contract(y[r0:r1].cpu().numpy(), ya.cpu().numpy())
    with pytest.raises(Q4KError):
        q4k_q8_project_ragged(w, q, [0, 5, 5, 1821])
    with pytest.raises(Q4KError):
        q4k_q8_project_ragged(w, q, [0, 5, 1820])


def test_config3_ragged_full_width_sampled():
    offs = ragged_offsets()
    m, k, n = 1821, 5120, 34816
    w = synth.device_weight(n, k, seed=22)
    hc, hs = w.codes.cpu().numpy(), w.scales.cpu().numpy()
    xb = synth.f32_to_bf16_bits(synth.activations(m, k, seed=13))
    q = pack_q8(bf16_tensor(xb), flag())
    y = q4k_q8_project_ragged(w, q, [int(v) for v in offs]).cpu().numpy()
    rz, ra, rs, _ = orc.q8_quantize(xb, bf16_bits=True)
    for r0, cnt in [(0, 16), (17408, 16), (34800, 16)]:
        assert_close_contract(y[:, r0:r0 + cnt], orc.project_rows(hc, hs, n, k, rz, ra, rs, r0, cnt))
