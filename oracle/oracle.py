"""numpy binding of the CPU oracle (oracle/q4k_oracle.c) and, when it was built, of the
reference's own host code (oracle/_ref/libqw38_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the CPU-baseline
legs of bench.py, never by the qw38_b200 package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "libq4k_oracle.so"
REF_SO = HERE / "_ref" / "libqw38_ref.so"

_oracle = None
_ref = None


def build(native: bool = False) -> Path:
    """Compile q4k_oracle.c.  The default build uses a portable x86-64-v3 target so the file
    can travel between machines; native=True builds a -march=native copy for timing."""
    out = HERE / ("libq4k_oracle_native.so" if native else "libq4k_oracle.so")
    src = HERE / "q4k_oracle.c"
    if out.exists() and out.stat().st_mtime >= src.stat().st_mtime:
        return out
    march = "native" if native else "x86-64-v3"
    cmd = ["gcc", "-O3", f"-march={march}", "-ffp-contract=off", "-fno-fast-math", "-fopenmp", "-fPIC",
           "-shared", "-o", str(out), str(src), "-lm"]
    env = dict(os.environ)
    subprocess.run(cmd, check=True, env=env)
    return out


def build_ref(reference_root: str | None = None) -> Path | None:
    """Compile the reference's host sources where they lie (see oracle/Makefile).  The checkout is named by
    the argument, by the environment variable QW38_REFERENCE_ROOT, or is a directory "reference" beside this
    repository; when none of them holds the sources nothing is built and an existing library is used as it is."""
    reference_root = reference_root or os.environ.get("QW38_REFERENCE_ROOT") or str(HERE.parent.parent / "reference")
    if not reference_root or not (Path(reference_root) / "src" / "format").is_dir():
        return REF_SO if REF_SO.exists() else None
    subprocess.run(["make", "-C", str(HERE), "ref", f"REF={reference_root}"], check=True,
                   stdout=subprocess.DEVNULL)
    return REF_SO


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def lib(native: bool = False) -> C.CDLL:
    global _oracle
    if native:
        return C.CDLL(str(build(native=True)))
    if _oracle is None:
        _oracle = C.CDLL(str(build()))
        _oracle.orc_fp16_to_fp32.restype = C.c_float
        _oracle.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        _oracle.orc_bf16_to_fp32.restype = C.c_float
        _oracle.orc_fp32_to_fp16.restype = C.c_uint16
        _oracle.orc_fp32_to_fp16.argtypes = [C.c_float]
        _oracle.orc_fp32_to_bf16.restype = C.c_uint16
        _oracle.orc_fp32_to_bf16.argtypes = [C.c_float]
    return _oracle


def ref() -> C.CDLL | None:
    """The reference's own host code, or None when it was not built on this machine."""
    global _ref
    if _ref is None and REF_SO.exists():
        try:
            _ref = C.CDLL(str(REF_SO))
            _ref.ref_fp16_to_fp32.restype = C.c_float
            _ref.ref_fp16_to_fp32.argtypes = [C.c_uint16]
            _ref.ref_fp32_to_bf16.restype = C.c_uint16
            _ref.ref_fp32_to_bf16.argtypes = [C.c_float]
        except OSError:
            _ref = None
    return _ref


def num_threads() -> int:
    return lib().orc_num_threads()


def set_threads(threads: int, handle=None) -> int:
    """OpenMP team size of `handle` (a library returned by lib(); each loaded copy has its own OpenMP state)."""
    return (handle if handle is not None else lib()).orc_set_threads(int(threads))


def ref_gemv_packed(wcodes: np.ndarray, wmeta: np.ndarray, n: int, k: int, x_bits: np.ndarray) -> np.ndarray | None:
    """compiler::reference_gemv_packed (src/compiler/quantization/reference.cpp:230-279) from the reference's own
    host code: split-tile weight x bf16 activations (bit patterns) -> fp32 [n].  None when that library was not built."""
    r = ref()
    if r is None:
        return None
    y = np.zeros(n, dtype=np.float32)
    wc, wm = np.ascontiguousarray(wcodes), np.ascontiguousarray(wmeta)
    st = r.ref_gemv_packed_q4k(C.c_uint64(n), C.c_uint64(k), _p(wc), C.c_uint64(wc.size), _p(wm), C.c_uint64(wm.size),
                               _p(np.ascontiguousarray(x_bits, dtype=np.uint16)), _p(y))
    if st != 0:
        raise RuntimeError("reference_gemv_packed refused the operands")
    return y


# ---------------------------------------------------------------------------
def q8_quantize(x: np.ndarray, bf16_bits: bool = False):
    """x: fp32 [m, k] or bf16 bit patterns uint16 [m, k].  Returns codes, scales, sums, failure."""
    m, k = x.shape
    pk = (k + 255) // 256 * 256
    codes = np.zeros((m, pk), dtype=np.int8)
    scales = np.zeros((m, pk // 32), dtype=np.float32)
    sums = np.zeros((m, pk // 32), dtype=np.int32)
    failure = C.c_int(0)
    if bf16_bits:
        x = np.ascontiguousarray(x, dtype=np.uint16)
        lib().orc_q8_quantize_bf16(_p(x), m, k, pk, _p(codes), _p(scales), _p(sums), C.byref(failure))
    else:
        x = np.ascontiguousarray(x, dtype=np.float32)
        lib().orc_q8_quantize_f32(_p(x), m, k, pk, _p(codes), _p(scales), _p(sums), C.byref(failure))
    return codes, scales, sums, failure.value


def q8_1_export(codes, scales, sums) -> np.ndarray:
    groups = scales.size
    out = np.zeros(groups * 36, dtype=np.uint8)
    lib().orc_q8_1_export(_p(np.ascontiguousarray(codes)), _p(np.ascontiguousarray(scales)),
                          _p(np.ascontiguousarray(sums)), C.c_uint64(groups), _p(out))
    return out


def pack_split(codes: np.ndarray, meta: np.ndarray):
    """Logical codes [n, k] (0..15) + metadata [n, tiles_k, 16] -> split-tile bytes."""
    n, k = codes.shape
    pn, pk = (n + 7) // 8 * 8, (k + 255) // 256 * 256
    oc = np.zeros(pn * pk // 2, dtype=np.uint8)
    om = np.zeros(pn * (pk // 256) * 16, dtype=np.uint8)
    lib().orc_pack_split(_p(np.ascontiguousarray(codes, dtype=np.int8)), _p(np.ascontiguousarray(meta)),
                         C.c_uint64(n), C.c_uint64(k), _p(oc), _p(om))
    return oc, om


def blocks144_to_split(blocks: np.ndarray, n: int, k: int):
    pn = (n + 7) // 8 * 8
    oc = np.zeros(pn * k // 2, dtype=np.uint8)
    om = np.zeros(pn * (k // 256) * 16, dtype=np.uint8)
    lib().orc_blocks144_to_split(_p(np.ascontiguousarray(blocks)), C.c_uint64(n), C.c_uint64(k), _p(oc), _p(om))
    return oc, om


def blocks144_to_logical(blocks: np.ndarray, n: int, k: int):
    codes = np.zeros((n, k), dtype=np.int8)
    meta = np.zeros((n, k // 256, 16), dtype=np.uint8)
    lib().orc_blocks144_to_logical(_p(np.ascontiguousarray(blocks)), C.c_uint64(n), C.c_uint64(k), _p(codes), _p(meta))
    return codes, meta


def logical_to_blocks144(codes: np.ndarray, meta: np.ndarray) -> np.ndarray:
    n, k = codes.shape
    out = np.zeros((n, k // 256, 144), dtype=np.uint8)
    lib().orc_logical_to_blocks144(_p(np.ascontiguousarray(codes, dtype=np.int8)), _p(np.ascontiguousarray(meta)),
                                   C.c_uint64(n), C.c_uint64(k), _p(out))
    return out


def dequantize_bf16(codes: np.ndarray, meta: np.ndarray) -> np.ndarray:
    """Logical codes [n, k] (0..15) + metadata [n, k/256, 16] -> bf16 bits [n, k]:
    bf16_rne((d * sc) * q - dmin * mn), every operation rounded to fp32, as
    compiler::dequantize_to_bf16 (src/compiler/quantization/reference.cpp:141-166).  numpy float32
    arithmetic rounds each operation separately, which is what the reference's host build does."""
    n, k = codes.shape
    f32 = np.float32
    meta = np.ascontiguousarray(meta).reshape(n, k // 256, 16)
    d = meta[..., 0:2].copy().view(np.float16).astype(f32)[..., 0]
    dmin = meta[..., 2:4].copy().view(np.float16).astype(f32)[..., 0]
    p = meta[..., 4:].astype(np.uint32)
    sc = np.empty((n, k // 256, 8), dtype=np.uint32)
    mn = np.empty_like(sc)
    sc[..., :4], mn[..., :4] = p[..., 0:4] & 63, p[..., 4:8] & 63
    sc[..., 4:] = (p[..., 8:12] & 15) | ((p[..., 0:4] >> 6) << 4)
    mn[..., 4:] = (p[..., 8:12] >> 4) | ((p[..., 4:8] >> 6) << 4)
    step = (d[..., None] * sc.astype(f32)).astype(f32)
    offset = (dmin[..., None] * mn.astype(f32)).astype(f32)
    q = codes.reshape(n, k // 256, 8, 32).astype(f32)
    w = ((step[..., None] * q).astype(f32) - offset[..., None]).astype(f32).reshape(n, k)
    bits = w.view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def dots(wcodes: np.ndarray, n: int, padded_k: int, z: np.ndarray) -> np.ndarray:
    """Exact int32 K32 partial dots [m, n, padded_k/32]."""
    m = z.shape[0]
    out = np.zeros((m, n, padded_k // 32), dtype=np.int32)
    lib().orc_q4k_q8_dots(_p(wcodes), n, padded_k, _p(np.ascontiguousarray(z)), m, _p(out))
    return out


def project(wcodes, wmeta, n: int, padded_k: int, z, a, sums, residual=None, want64: bool = False):
    """fp32 [m, n] outputs of the reference equation accumulated in double."""
    m = z.shape[0]
    out = np.zeros((m, n), dtype=np.float32)
    out64 = np.zeros((m, n), dtype=np.float64) if want64 else None
    res = None if residual is None else np.ascontiguousarray(residual, dtype=np.float32)
    lib().orc_q4k_q8_project(_p(wcodes), _p(wmeta), n, padded_k, _p(np.ascontiguousarray(z)),
                             _p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(sums)), m, _p(res), _p(out),
                             _p(out64))
    return (out, out64) if want64 else out


def project_rows(wcodes, wmeta, n: int, padded_k: int, z, a, sums, row0: int, rows: int, native: bool = False,
                 handle=None):
    m = z.shape[0]
    out = np.zeros((m, rows), dtype=np.float32)
    h = handle if handle is not None else lib(native)
    h.orc_q4k_q8_project_rows(_p(wcodes), _p(wmeta), n, padded_k, _p(np.ascontiguousarray(z)),
                              _p(np.ascontiguousarray(a)), _p(np.ascontiguousarray(sums)), m, row0, rows, _p(out))
    return out


def swiglu_bf16(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    out = np.zeros(gate.shape, dtype=np.uint16)
    lib().orc_swiglu_bf16(_p(np.ascontiguousarray(gate, dtype=np.float32)),
                          _p(np.ascontiguousarray(up, dtype=np.float32)), C.c_uint64(gate.size), _p(out))
    return out


def hidden_rms_bf16(x: np.ndarray, gamma_bits: np.ndarray, eps: float) -> np.ndarray:
    m, h = x.shape
    out = np.zeros((m, h), dtype=np.uint16)
    lib().orc_hidden_rms_bf16(_p(np.ascontiguousarray(x, dtype=np.float32)),
                              _p(np.ascontiguousarray(gamma_bits, dtype=np.uint16)), C.c_float(eps), m, h, _p(out))
    return out


def bf16_gemv(wcodes, wmeta, n: int, k: int, padded_k: int, x_bits: np.ndarray) -> np.ndarray:
    y = np.zeros(n, dtype=np.float32)
    lib().orc_q4k_bf16_gemv(_p(wcodes), _p(wmeta), n, k, padded_k, _p(np.ascontiguousarray(x_bits, dtype=np.uint16)), _p(y))
    return y


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)
