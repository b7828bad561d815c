"""ncu workload: the batch-1 table-lookup product on the 18944 x 3584 (gate/up) shape, 12 distinct
matrices (154 MB of packed weights, larger than L2) so that every launch streams from HBM."""
import sys
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch
from quantexperiments_b200.kernels import DeviceMatrix, L8Matrix, T16Matrix

R, C = 18944, 3584
which = sys.argv[1] if len(sys.argv) > 1 else "l8"
g = torch.Generator(device="cuda").manual_seed(0)
W = (C // 8 * 12 + 31) // 32
ms = []
for i in range(12):
    tags = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g)
    table = torch.randn(4096, 8, device="cuda", generator=g).half()
    rs = (torch.rand(R, device="cuda", generator=g) * 0.02 + 0.01).half()
    dm = DeviceMatrix(tags, table, rs, K=4096, d=8, C=C)
    ms.append(L8Matrix(dm) if which == "l8" else T16Matrix(dm))
x = torch.randn(C, device="cuda").bfloat16()
y = torch.empty(1, R, device="cuda", dtype=torch.bfloat16)
for rep in range(2):
    for m in ms:
        m.run(x, y[0]) if which == "l8" else m.run(x[None], y)
torch.cuda.synchronize()
print("ok")
