"""ncu workload: nearest-codeword assignment (k_assign) of 148 x 2048 x 4 chunks against a 4096-word book,
unweighted then weighted, two launches each (39 MB of chunks per launch; the kernel is bound by fp32 FMAs)."""
import sys
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch
from quantexperiments_b200 import codebook as cb

n = 148 * 2048 * 4
g = torch.Generator(device="cuda").manual_seed(0)
x = torch.randn(n, 8, device="cuda", generator=g)
wt = torch.rand(n, 8, device="cuda", generator=g)
book = torch.randn(4096, 8, device="cuda", generator=g).half()
for w in (None, None, wt, wt):
    idx, err = cb.assign(x, book, wt=w)
torch.cuda.synchronize()
print("ok", int(idx[0]), float(err.mean()))
