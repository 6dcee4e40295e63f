"""Host-side mirror of the reference's Q4_K x Q8 operator interface (cuda/q4k_q8.hpp:14-49,
cuda/prefill.hpp:33-44) over the C ABI.  Same names, argument meaning and error behaviour;
torch supplies device memory and streams only -- every operation is a kernel of libq4k_b200."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import _lib as L


class Q4KError(RuntimeError):
    """A rejected or failed call.  `code` is the reference's ErrorCode (cuda/error.hpp:13-17):
    1 Status, 2 InvalidArgument, 3 Overflow."""

    def __init__(self, code: int, message: str):
        super().__init__(f"q4k error {code}: {message}")
        self.code = code
        self.message = message


def _check(status: int) -> None:
    if status != L.OK:
        raise Q4KError(status, L.load().q4k_last_error().decode())


def set_launch_overlap(enabled: bool) -> None:
    """Process-wide switch (q4k_set_launch_overlap): decode kernels may start, and stream weight tiles,
    while the preceding kernel of the stream drains.  Only while nothing in flight writes the weights."""
    L.load().q4k_set_launch_overlap(1 if enabled else 0)


def launch_overlap() -> bool:
    return bool(L.load().q4k_get_launch_overlap())


def pad_n(n: int) -> int:
    return (n + 7) // 8 * 8


def pad_k(k: int) -> int:
    return (k + 255) // 256 * 256


def _stream(stream) -> C.c_void_p:
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


@dataclass
class PrefillWeight:
    """Q4_K matrix in split tiles (struct PrefillWeight, cuda/prefill.hpp:33-44)."""
    codes: torch.Tensor   # uint8, padded_n * padded_k / 2 bytes
    scales: torch.Tensor  # uint8, padded_n * (padded_k / 256) * 16 bytes
    n: int
    k: int
    layout: int = L.LAYOUT_SPLIT_TILES
    quantizer: int = L.QUANTIZER_Q4K
    codes_bytes: Optional[int] = None    # override to build a malformed descriptor in tests
    scales_bytes: Optional[int] = None

    @property
    def padded_n(self) -> int:
        return pad_n(self.n)

    @property
    def padded_k(self) -> int:
        return pad_k(self.k)

    def c_struct(self) -> L.Weight:
        return L.Weight(self.codes.data_ptr(), self.scales.data_ptr(), self.layout, self.quantizer, self.n,
                        self.k, self.padded_n, self.padded_k,
                        self.codes.numel() if self.codes_bytes is None else self.codes_bytes,
                        self.scales.numel() if self.scales_bytes is None else self.scales_bytes)

    @staticmethod
    def from_host(codes, scales, n: int, k: int, device="cuda") -> "PrefillWeight":
        """codes / scales: numpy uint8 arrays already in split-tile order."""
        return PrefillWeight(torch.from_numpy(codes).to(device), torch.from_numpy(scales).to(device), n, k)

    def nbytes(self) -> int:
        return self.codes.numel() + self.scales.numel()

    def row_slice(self, row0: int, rows: int) -> "PrefillWeight":
        """Rows [row0, row0+rows) as a weight of its own (row0 % 8 == 0): a row group is one
        contiguous run of tiles, so an output-row shard is a view, not a copy."""
        if row0 % 8 != 0 or row0 + rows > self.n:
            raise ValueError("row shard must start on a multiple of 8 inside the matrix")
        tiles_k = self.padded_k // 256
        g0, g1 = row0 // 8, (row0 + rows + 7) // 8
        return PrefillWeight(self.codes[g0 * tiles_k * 1024:g1 * tiles_k * 1024],
                             self.scales[g0 * tiles_k * 128:g1 * tiles_k * 128], rows, self.k)


@dataclass
class Q8Input:
    """Quantised activations (struct Q8Input, cuda/q4k_q8.hpp:14-21)."""
    codes: torch.Tensor   # int8  [m, padded_k]
    scales: torch.Tensor  # fp32  [m, padded_k / 32]
    sums: torch.Tensor    # int32 [m, padded_k / 32]
    m: int
    k: int
    padded_k: int

    def c_struct(self) -> L.Q8:
        return L.Q8(self.codes.data_ptr(), self.scales.data_ptr(), self.sums.data_ptr(), self.codes.numel(),
                    self.scales.numel(), self.sums.numel(), self.m, self.k, self.padded_k)

    def rows(self, r0: int, r1: int) -> "Q8Input":
        return Q8Input(self.codes[r0:r1], self.scales[r0:r1], self.sums[r0:r1], r1 - r0, self.k, self.padded_k)


def new_q8_input(m: int, k: int, device="cuda") -> Q8Input:
    pk = pad_k(k)
    return Q8Input(torch.empty((m, pk), dtype=torch.int8, device=device),
                   torch.empty((m, pk // 32), dtype=torch.float32, device=device),
                   torch.empty((m, pk // 32), dtype=torch.int32, device=device), m, k, pk)


def pack_q8(x: torch.Tensor, failure: torch.Tensor, out: Optional[Q8Input] = None, stream=None) -> Q8Input:
    """pack_q8 (cuda/q4k_q8.hpp:32-34): bf16 (or fp32) rows [m, k] -> Q8.  `failure` is one
    int32 on the device that the caller cleared; a non-finite group sets it to 1."""
    lib = L.load()
    if x.dim() != 2 or not x.is_contiguous():
        raise Q4KError(L.ERR_INVALID_ARGUMENT, "pack_q8 takes a contiguous [m, k] tensor")
    m, k = x.shape
    if out is None:
        out = new_q8_input(m, k, x.device)
    if x.dtype == torch.bfloat16:
        fn = lib.q4k_pack_q8_bf16
    elif x.dtype == torch.float32:
        fn = lib.q4k_pack_q8_f32
    else:
        raise Q4KError(L.ERR_INVALID_ARGUMENT, "pack_q8 takes bf16 or fp32")
    _check(fn(_ptr(x), x.numel(), out.c_struct(), _ptr(failure), _stream(stream)))
    return out


def q4k_q8_project(weight: PrefillWeight, x: Q8Input, out: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None, *, kernel: int = L.KERNEL_AUTO, split_k: int = 0,
                   row_groups: int = 0, partials: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                   trusted: bool = False, input_settled: bool = False, stream=None) -> torch.Tensor:
    """q4k_q8_project (cuda/q4k_q8.hpp:35-37): fp32 out[token, row], token-major.
    `input_settled`: Q4K_FLAG_INPUT_SETTLED (x and residual were not written by the launch directly before)."""
    lib = L.load()
    if out is None:
        out = torch.empty((x.m, weight.n), dtype=torch.float32, device=x.codes.device)
    w = weight.c_struct()
    plain = kernel == L.KERNEL_AUTO and split_k == 0 and row_groups == 0 and partials is None and workspace is None and not trusted and not input_settled
    if plain:
        _check(lib.q4k_q8_project(C.byref(w), x.c_struct(), _ptr(out), out.numel(), _ptr(residual),
                                  0 if residual is None else residual.numel(), _stream(stream)))
    else:
        opt = L.ProjectOptions(kernel, split_k, row_groups, 0 if partials is None else partials.data_ptr(),
                               0 if partials is None else partials.numel(),
                               0 if workspace is None else workspace.data_ptr(),
                               0 if workspace is None else workspace.numel() * workspace.element_size(),
                               (L.FLAG_TRUSTED_SPANS if trusted else 0) | (L.FLAG_INPUT_SETTLED if input_settled else 0))
        _check(lib.q4k_q8_project_ex(C.byref(w), x.c_struct(), _ptr(out), out.numel(), _ptr(residual),
                                     0 if residual is None else residual.numel(), C.byref(opt), _stream(stream)))
    return out


def reserve_scratch(partial_bytes: int, stream=None) -> None:
    """Grow the library-owned split-K scratch of the current device to hold `partial_bytes` of partial tiles
    (q4k_reserve_scratch): once per device, before a graph is captured whose calls need that much."""
    _check(L.load().q4k_reserve_scratch(int(partial_bytes), _stream(stream)))


def q4k_q8_project_static(weight: PrefillWeight, x: Q8Input, out: Optional[torch.Tensor] = None,
                          residual: Optional[torch.Tensor] = None, *, split_k: int = 0, stream=None) -> torch.Tensor:
    """The projection for callers that may not allocate device memory: split-K scratch lives in a
    fixed array inside the library (8 MiB), so the call never reaches cudaMalloc.  `out` must be
    supplied by such callers; it is created here only as a convenience for tests."""
    lib = L.load()
    if out is None:
        out = torch.empty((x.m, weight.n), dtype=torch.float32, device=x.codes.device)
    w = weight.c_struct()
    _check(lib.q4k_q8_project_static(C.byref(w), x.c_struct(), _ptr(out), out.numel(), _ptr(residual),
                                     0 if residual is None else residual.numel(), split_k, _stream(stream)))
    return out


def q4k_q8_project_ragged(weight: PrefillWeight, x: Q8Input, row_offsets: Sequence[int],
                          out: Optional[torch.Tensor] = None, *, kernel: int = L.KERNEL_AUTO,
                          partials: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """Packed continuous batch: request r owns token rows [row_offsets[r], row_offsets[r+1])."""
    lib = L.load()
    if out is None:
        out = torch.empty((x.m, weight.n), dtype=torch.float32, device=x.codes.device)
    offs = (C.c_uint32 * len(row_offsets))(*row_offsets)
    w = weight.c_struct()
    opt = L.ProjectOptions(kernel, 0, 0, 0 if partials is None else partials.data_ptr(),
                           0 if partials is None else partials.numel(), 0, 0, 0)
    _check(lib.q4k_q8_project_ragged(C.byref(w), x.c_struct(), offs, len(row_offsets) - 1, _ptr(out),
                                     out.numel(), C.byref(opt), _stream(stream)))
    return out


def q4k_q8_project_gather(shard: PrefillWeight, x: Q8Input, outputs: Sequence[int], flags: Sequence[int], rank: int,
                          row_offset: int, total_rows: int, residual: Optional[torch.Tensor] = None, stream=None,
                          input_settled: bool = False) -> None:
    """Row-sharded decode projection with the gather fused in (q4k_q8_project_gather): `outputs[g]` /
    `flags[g]` are rank g's full [m, total_rows] fp32 buffer and zeroed uint32[16] flag array as device addresses
    valid in this process.  This rank's rows land in every buffer; flags[g][rank] is then incremented.
    `input_settled`: Q4K_FLAG_INPUT_SETTLED (x and residual were not written by the launch directly before)."""
    desc = L.GatherDesc()
    for g, (o, f) in enumerate(zip(outputs, flags)):
        desc.outputs[g] = int(o)
        desc.flags[g] = int(f)
    desc.ranks, desc.rank, desc.row_offset, desc.total_rows = len(outputs), rank, row_offset, total_rows
    desc.options = L.FLAG_INPUT_SETTLED if input_settled else 0
    _check(L.load().q4k_q8_project_gather(C.byref(shard.c_struct()), x.c_struct(), C.byref(desc), _ptr(residual),
                                          0 if residual is None else residual.numel(), _stream(stream)))


def peer_announce(flags: Sequence[int], rank: int, stream=None) -> None:
    """Enqueue only the announcement of this rank's finished gather projections (q4k_peer_announce)."""
    desc = L.GatherDesc()
    for g, f in enumerate(flags):
        desc.flags[g] = int(f)
    desc.ranks, desc.rank = len(flags), rank
    _check(L.load().q4k_peer_announce(C.byref(desc), _stream(stream)))


def peer_wait(flags: Sequence[int], rank: int, limit_cycles: int = 0, stream=None) -> None:
    """Enqueue the announcement of this rank's finished gather projections and the bounded wait for every
    rank's deliveries (q4k_peer_wait); `flags[g]` as for q4k_q8_project_gather."""
    desc = L.GatherDesc()
    for g, f in enumerate(flags):
        desc.flags[g] = int(f)
    desc.ranks, desc.rank = len(flags), rank
    _check(L.load().q4k_peer_wait(C.byref(desc), limit_cycles, _stream(stream)))


@dataclass
class DecodeMmvDesc:
    """One decode projection (struct DecodeMmvDesc, cuda/decode_mmv.hpp:103-121) under the Q8-K32 activation
    policy: `input` bf16 [m, k]; `output` bf16 or fp32 [m, n] by epilogue, or None for the in-place residual update."""
    weight: PrefillWeight
    input: torch.Tensor
    output: Optional[torch.Tensor]
    epilogue: int = L.EPILOGUE_STORE_BF16
    residual: Optional[torch.Tensor] = None
    activation_policy: int = L.ACTIVATION_Q8_K32

    def c_struct(self) -> L.DecodeDesc:
        m = self.input.shape[0] if self.input.dim() == 2 else 1
        return L.DecodeDesc(self.weight.c_struct(), self.input.data_ptr(), self.input.numel(),
                            0 if self.output is None else self.output.data_ptr(),
                            0 if self.output is None else self.output.numel(),
                            0 if self.residual is None else self.residual.data_ptr(),
                            0 if self.residual is None else self.residual.numel(), m, self.epilogue, self.activation_policy)


def decode_workspace(m: int, n_total: int, k: int, device="cuda") -> torch.Tensor:
    return torch.empty(L.load().q4k_decode_workspace_bytes(m, n_total, k), dtype=torch.uint8, device=device)


def launch_decode_mmv(desc: DecodeMmvDesc, workspace: torch.Tensor, failure: torch.Tensor, stream=None) -> None:
    """launch_decode_mmv (cuda/decode_mmv.hpp:207-209)."""
    d = desc.c_struct()
    _check(L.load().q4k_decode_mmv(C.byref(d), _ptr(workspace), workspace.numel(), _ptr(failure), _stream(stream)))


def launch_decode_mmv_paired(a: DecodeMmvDesc, b: DecodeMmvDesc, workspace: torch.Tensor, failure: torch.Tensor,
                             stream=None) -> None:
    """launch_decode_mmv_paired (cuda/decode_mmv.hpp:210-211): gate/up sharing one input; SwigluStoreBf16 lives here."""
    da, db = a.c_struct(), b.c_struct()
    _check(L.load().q4k_decode_mmv_paired(C.byref(da), C.byref(db), _ptr(workspace), workspace.numel(), _ptr(failure),
                                          _stream(stream)))


def launch_decode_mmv_ranges(ranges: Sequence[DecodeMmvDesc], workspace: torch.Tensor, failure: torch.Tensor,
                             stream=None) -> None:
    """launch_decode_mmv_ranges (cuda/decode_mmv.hpp:212-215): two or three output ranges over one input."""
    arr = (L.DecodeDesc * len(ranges))(*[r.c_struct() for r in ranges])
    _check(L.load().q4k_decode_mmv_ranges(arr, len(ranges), _ptr(workspace), workspace.numel(), _ptr(failure),
                                          _stream(stream)))


def prefill_project(projection: DecodeMmvDesc, workspace: torch.Tensor, failure: torch.Tensor, stream=None) -> None:
    """PrefillEngine::project (cuda/prefill.hpp:88-89) for a Q4_K weight: quantise -> MMQ -> PrefillEpilogue."""
    d = projection.c_struct()
    _check(L.load().q4k_prefill_project(C.byref(d), _ptr(workspace), workspace.numel(), _ptr(failure), _stream(stream)))


def prefill_paired_swiglu(gate: PrefillWeight, up: PrefillWeight, normalized: torch.Tensor, swiglu: torch.Tensor,
                          workspace: torch.Tensor, failure: torch.Tensor, stream=None) -> None:
    """PrefillEngine::paired_swiglu (cuda/prefill.hpp:90-93): swiglu = bf16(SiLU(gate x) * (up x))."""
    g, u = gate.c_struct(), up.c_struct()
    _check(L.load().q4k_prefill_paired_swiglu(C.byref(g), C.byref(u), _ptr(normalized), _ptr(swiglu), normalized.shape[0],
                                              _ptr(workspace), workspace.numel(), _ptr(failure), _stream(stream)))


def q8_mlp_workspace_bytes(m: int, hidden: int, ffn: int) -> int:
    return L.load().q4k_q8_mlp_workspace_bytes(m, hidden, ffn)


def q4k_q8_mlp(gate: PrefillWeight, up: PrefillWeight, down: PrefillWeight, residual: torch.Tensor,
               gamma: torch.Tensor, eps: float, out: torch.Tensor, m: int, workspace: torch.Tensor,
               pending_failure: Optional[torch.Tensor] = None, stream=None) -> bool:
    """q4k_q8_mlp (cuda/q4k_q8.hpp:44-49).  Returns `submitted`; raises Q4KError on rejection
    or, in the synchronous form (pending_failure None), on a non-finite producer."""
    lib = L.load()
    submitted = C.c_int(0)
    g, u, d = gate.c_struct(), up.c_struct(), down.c_struct()
    st = lib.q4k_q8_mlp(C.byref(g), C.byref(u), C.byref(d), _ptr(residual), _ptr(gamma), eps, _ptr(out), m,
                        _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(stream),
                        C.byref(submitted), _ptr(pending_failure))
    if st != L.OK:
        err = Q4KError(st, lib.q4k_last_error().decode())
        err.submitted = bool(submitted.value)
        raise err
    return bool(submitted.value)


def hidden_rms_q8(residual: torch.Tensor, gamma: torch.Tensor, eps: float, failure: torch.Tensor,
                  out: Optional[Q8Input] = None, stream=None) -> Q8Input:
    """launch_hidden_rms_q8 (cuda/activation.cu:536-548)."""
    m, hidden = residual.shape
    if out is None:
        out = new_q8_input(m, hidden, residual.device)
    _check(L.load().q4k_hidden_rms_q8(_ptr(residual), _ptr(gamma), eps, m, hidden, out.c_struct(), _ptr(failure),
                                      _stream(stream)))
    return out


def swiglu_pack_q8(gate: torch.Tensor, up: torch.Tensor, failure: torch.Tensor, out: Optional[Q8Input] = None,
                   stream=None) -> Q8Input:
    """swiglu_pack_kernel (cuda/q4k_q8.cu:52-61)."""
    m, ffn = gate.shape
    if out is None:
        out = new_q8_input(m, ffn, gate.device)
    _check(L.load().q4k_swiglu_pack_q8(_ptr(gate), _ptr(up), m, ffn, out.c_struct(), _ptr(failure), _stream(stream)))
    return out


def export_q8_1(x: Q8Input, stream=None) -> torch.Tensor:
    """36-byte records {fp16 d, fp16 s, 32 codes} per K32 group."""
    rec = torch.empty(x.scales.numel() * 36, dtype=torch.uint8, device=x.codes.device)
    _check(L.load().q4k_export_q8_1(x.c_struct(), _ptr(rec), rec.numel(), _stream(stream)))
    return rec


VALIDATE_ERRORS = {
    1: ("quantized.codes.padding", "Q4 padded coordinates must encode zero"),
    2: ("quantized.scales.padding", "padded Q4_K metadata must be zero"),
    3: ("quantized.scales", "Q4_K superblock scales must be nonnegative finite FP16"),
}


def validate_weight(weight: PrefillWeight, stream=None):
    """format::validate_cuda_v0 (src/format/unpack.cpp:89-226) on a resident weight.  Returns
    (0, 0) when admissible, else (kind, byte offset of the first offence in the reference's scan
    order); VALIDATE_ERRORS[kind] is the reference's (field, detail).  Synchronises."""
    verdict = torch.empty(2, dtype=torch.int64, device=weight.codes.device)
    _check(L.load().q4k_validate_weight(C.byref(weight.c_struct()), _ptr(verdict), _stream(stream)))
    kind, offset = verdict.cpu().tolist()
    return int(kind), int(offset)


def dequantize_bf16(weight: PrefillWeight, stream=None) -> torch.Tensor:
    """compiler::dequantize_to_bf16 (src/compiler/quantization/reference.cpp:141-166) from the resident
    weight: bfloat16 [n, k]."""
    out = torch.empty((weight.n, weight.k), dtype=torch.bfloat16, device=weight.codes.device)
    _check(L.load().q4k_dequantize_bf16(C.byref(weight.c_struct()), _ptr(out), out.numel(), _stream(stream)))
    return out


def unpack_logical(weight: PrefillWeight, stream=None):
    """format::unpack_cuda_v0 (src/format/unpack.cpp:262-380) from the resident weight:
    (levels int8 [n, k], metadata uint8 [n, k/256, 16])."""
    dev = weight.codes.device
    codes = torch.empty((weight.n, weight.k), dtype=torch.int8, device=dev)
    meta = torch.empty((weight.n, weight.k // 256, 16), dtype=torch.uint8, device=dev)
    _check(L.load().q4k_unpack_logical(C.byref(weight.c_struct()), _ptr(codes), codes.numel(), _ptr(meta), meta.numel(),
                                       _stream(stream)))
    return codes, meta


FIT_ERRORS = {
    1: "Q4_K input is nonfinite",
    2: "Q4_K fitting range exceeded",
    3: "Q4_K fitting reciprocal overflow",
    4: "Q4_K compression reciprocal overflow",
    5: "Q4_K FP16 scale overflow",
}


def _fit_dtype(weights: torch.Tensor) -> int:
    if weights.dtype == torch.float32:
        return 0
    if weights.dtype == torch.bfloat16:
        return 1
    raise Q4KError(2, "q4k.fit: weights must be float32 or bfloat16")


def _fit_raise(failure: torch.Tensor, status: torch.Tensor) -> None:
    """The reference stops at the first refused block in index order and returns its error
    (src/compiler/quantization/quantizer.cpp:176-181)."""
    if int(failure.item()):
        bad = torch.nonzero(status)[0]
        code = int(status[bad].item())
        raise Q4KError(2, f"q4k.fit: block {int(bad.item())}: {FIT_ERRORS.get(code, code)}")


def quantize_q4k_blocks(weights: torch.Tensor, stream=None, check: bool = True):
    """compiler::quantize_q4k_block (src/compiler/quantization/q4k.cpp:186-278) over every 256
    consecutive weights of a contiguous device tensor.  Returns (codes int8 [blocks, 256],
    metadata uint8 [blocks, 16], status uint8 [blocks]); with check (synchronises) a refused block
    raises the reference's message."""
    dtype = _fit_dtype(weights)
    if weights.numel() == 0 or weights.numel() % 256 or not weights.is_contiguous():
        raise Q4KError(2, "q4k.fit: weights must be contiguous and a multiple of 256 long")
    blocks = weights.numel() // 256
    dev = weights.device
    codes = torch.empty((blocks, 256), dtype=torch.int8, device=dev)
    meta = torch.empty((blocks, 16), dtype=torch.uint8, device=dev)
    status = torch.empty(blocks, dtype=torch.uint8, device=dev)
    failure = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(L.load().q4k_fit_blocks(_ptr(weights), dtype, blocks, _ptr(codes), _ptr(meta), _ptr(status), _ptr(failure),
                                   _stream(stream)))
    if check:
        _fit_raise(failure, status)
    return codes, meta, status


def quantize_q4k_weight(weights: torch.Tensor, stream=None, check: bool = True) -> PrefillWeight:
    """Row-major [n, k] float32/bfloat16 device weights (k % 256 == 0) -> split-tile Q4_K weight:
    the fitter followed by format::pack_cuda_v0 (src/format/pack.cpp:175-222), in one kernel."""
    dtype = _fit_dtype(weights)
    if weights.dim() != 2 or not weights.is_contiguous():
        raise Q4KError(2, "q4k.fit: weights must be a contiguous [n, k] matrix")
    n, k = weights.shape
    pn = pad_n(n)
    dev = weights.device
    codes = torch.empty(pn * k // 2, dtype=torch.uint8, device=dev)
    scales = torch.empty(pn * (k // 256) * 16, dtype=torch.uint8, device=dev)
    status = torch.empty(max(1, n * (k // 256)), dtype=torch.uint8, device=dev)
    failure = torch.zeros(1, dtype=torch.int32, device=dev)
    _check(L.load().q4k_fit_weight(_ptr(weights), dtype, n, k, _ptr(codes), codes.numel(), _ptr(scales), scales.numel(),
                                   _ptr(status), _ptr(failure), _stream(stream)))
    if check:
        _fit_raise(failure, status)
    return PrefillWeight(codes, scales, n, k)


def repack_blocks144(blocks: torch.Tensor, n: int, k: int, stream=None) -> PrefillWeight:
    """144-byte llama.cpp-native super-blocks (device uint8) -> split tiles."""
    pn = pad_n(n)
    codes = torch.empty(pn * k // 2, dtype=torch.uint8, device=blocks.device)
    scales = torch.empty(pn * (k // 256) * 16, dtype=torch.uint8, device=blocks.device)
    _check(L.load().q4k_repack_blocks144(_ptr(blocks), blocks.numel(), n, k, _ptr(codes), codes.numel(), _ptr(scales),
                                         scales.numel(), _stream(stream)))
    return PrefillWeight(codes, scales, n, k)
