"""q4k_q8_project_static: the projection entry point for callers that cannot allocate device
memory (their own arena owns the GPU, or an allocation's implicit synchronisation is not
acceptable on their path).  Its split-K scratch is a fixed array inside the library, so the
call must give the same numbers as the ordinary entry point without ever allocating -- on the
first call and again on the next one, which finds the array as the first call left it."""
import numpy as np
import pytest
import torch

from qw38_b200 import _lib as L
from qw38_b200 import synth
from qw38_b200.q4k_q8 import Q4KError, pack_q8, q4k_q8_project, q4k_q8_project_static
from tests.helpers import assert_close_contract

pytestmark = pytest.mark.gpu
DEV = "cuda"


def case(n, k, m, seed):
    w = synth.device_weight(n, k, seed=seed)
    x = torch.from_numpy(synth.f32_to_bf16_bits(synth.activations(m, k, seed=seed)).view(np.int16)).to(DEV).view(torch.bfloat16)
    q = pack_q8(x, torch.zeros(1, dtype=torch.int32, device=DEV))
    return w, q


def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row():
    for call, (n, k, m, split_k, seed) in enumerate([(640, 5120, 16, 4, 31), (1000 // 8 * 8, 2560, 40, 3, 32)]):
        w, q = case(n, k, m, seed)
        res = torch.from_numpy(synth.activations(m, n, seed=7)).to(DEV)
        want = q4k_q8_project(w, q, residual=res, kernel=L.KERNEL_MMA, split_k=split_k).cpu().numpy()
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        if call == 0:   # the first call on a device resolves the array's address (and loads the module)
            q4k_q8_project_static(w, q, out=out, residual=res, split_k=split_k)
            torch.cuda.synchronize()
        before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        got_t = q4k_q8_project_static(w, q, out=out, residual=res, split_k=split_k)
        torch.cuda.synchronize()
        # neither torch's allocator nor the driver (cudaMemGetInfo: a cudaMalloc inside the library would show here)
        assert torch.cuda.memory_allocated() == before and torch.cuda.mem_get_info()[0] == free_before
        got = got_t.cpu().numpy()
        del got_t   # (an alias of `out`: dropped here so that the next round's figures are not moved by its release)
        assert_close_contract(got, want)
        assert (got == want).all(), f"call {call}: same kernel, same slice order -> same bits"


def test_static_scratch_entry_rejects_what_does_not_fit():
    w, q = case(34816, 5120, 64, 33)           # 4 * 64 * 34816 * 4 bytes = 35.7 MB > 8 MiB
    out = torch.zeros((64, 34816), dtype=torch.float32, device=DEV)
    with pytest.raises(Q4KError) as e:
        q4k_q8_project_static(w, q, out=out, split_k=4)
    assert e.value.code == L.ERR_INVALID_ARGUMENT and "exceeds the built-in scratch" in e.value.message
    assert not out.any().item(), "a rejected call launches nothing"
    got = q4k_q8_project_static(w, q, out=out, split_k=1).cpu().numpy()   # no split: no scratch needed
    want = q4k_q8_project(w, q, kernel=L.KERNEL_MMA, split_k=1).cpu().numpy()
    assert (got == want).all()
