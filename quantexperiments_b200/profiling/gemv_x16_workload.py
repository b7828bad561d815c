"""ncu workload: the activation-stationary small-batch product (k_gemv_x16) on the stacked gate|up shape
37888 x 3584 with 16 tokens; three launches on staged activations (25.5 MB of tags; ncu flushes the caches before each captured launch)."""
import sys
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch
from quantexperiments_b200.kernels import DeviceMatrix, X16Matrix

R, C, B = 37888, 3584, 16
g = torch.Generator(device="cuda").manual_seed(0)
W = (C // 8 * 12 + 31) // 32
tags = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g)
table = torch.randn(4096, 8, device="cuda", generator=g).half()
rs = (torch.rand(R, device="cuda", generator=g) * 0.02 + 0.01).half()
xm = X16Matrix(DeviceMatrix(tags, table, rs, K=4096, d=8, C=C))
X = torch.randn(B, C, device="cuda", generator=g).bfloat16()
Y = torch.empty(B, R, device="cuda", dtype=torch.bfloat16)
xp = xm.prep(X, B)
for _ in range(3):
    xm.run_prepped(xp, Y, B)
torch.cuda.synchronize()
print("ok")
