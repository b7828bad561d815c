"""ncu workload: the two-phase prefill product (raw 16-bit decode + TMA-fed two-SM tcgen05 GEMM) on the
18944 x 3584 gate/up shape with 2048 tokens; three rounds of decode + GEMM (weights decoded to a 136 MB
scratch, activations 14 MB)."""
import sys
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch
from quantexperiments_b200.kernels import DenseStack, DeviceMatrix

R, C, T = 18944, 3584, 2048
g = torch.Generator(device="cuda").manual_seed(0)
W = (C // 8 * 12 + 31) // 32
tags = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g)
table = torch.randn(4096, 8, device="cuda", generator=g).half()
rs = (torch.rand(R, device="cuda", generator=g) * 0.02 + 0.01).half()
st = DenseStack([DeviceMatrix(tags, table, rs, K=4096, d=8, C=C)])
X = torch.randn(T, C, device="cuda", generator=g).bfloat16()
Y = torch.empty(T, R, device="cuda", dtype=torch.bfloat16)
for _ in range(3):
    st.gemm(X, Y)
torch.cuda.synchronize()
DenseStack.status("cuda")
print("ok")
