"""Runs one projection a few times so that a profiler can capture a single kernel:
    python -m qw38_b200.profile_case <n> <k> <m> <kernel id> [split_k] [row_groups]
Kernel ids are the Q4K_KERNEL_* values of include/q4k_b200.h (1 dp4a, 2 mma, 3 tcgen05, 4 cluster mma, 5 TMA gemv).
    python -m qw38_b200.profile_case fit <n> <k>      runs the Q4_K fitter on fp32 [n, k] weights instead,
    python -m qw38_b200.profile_case deq <n> <k>      the bf16 dequantiser on a resident [n, k] weight."""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from qw38_b200 import synth
from qw38_b200.q4k_q8 import pack_q8, q4k_q8_project, quantize_q4k_weight
if sys.argv[1] == "deq":
    from qw38_b200.q4k_q8 import dequantize_bf16
    wd = synth.device_weight(int(sys.argv[2]), int(sys.argv[3]), seed=0)
    for _ in range(3):
        o = dequantize_bf16(wd)
    torch.cuda.synchronize()
    print("ok", float(o.float().abs().mean()))
    sys.exit(0)
if sys.argv[1] == "fit":
    wf = torch.randn((int(sys.argv[2]), int(sys.argv[3])), device="cuda") * 0.02
    for _ in range(3):
        pw = quantize_q4k_weight(wf, check=False)
    torch.cuda.synchronize()
    print("ok", int(pw.codes.sum()))
    sys.exit(0)
n, k, m, kern = (int(a) for a in sys.argv[1:5])
sk = int(sys.argv[5]) if len(sys.argv) > 5 else 0
rg = int(sys.argv[6]) if len(sys.argv) > 6 else 0
w = synth.device_weight(n, k, seed=0)
f = torch.zeros(1, dtype=torch.int32, device="cuda")
q = pack_q8(torch.randn((m, k), device="cuda").to(torch.bfloat16), f)
out = torch.empty((m, n), dtype=torch.float32, device="cuda")
for _ in range(3):
    q4k_q8_project(w, q, out=out, kernel=kern, split_k=sk, row_groups=rg, trusted=True)
torch.cuda.synchronize()
print("ok", float(out.abs().mean()))
