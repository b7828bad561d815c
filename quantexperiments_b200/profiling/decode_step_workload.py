"""ncu workload: eager decode steps of a 4-layer Qwen2.5-7B-shaped engine (random init) at position 2048;
the last step runs between cudaProfilerStart/Stop (use --profile-from-start off). Argument: batch (1 or 32)."""
import sys
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch
from quantexperiments_b200.engine import Cfg, Qwen2BatchEngine, random_engine

B = int(sys.argv[1]) if len(sys.argv) > 1 else 1
eng = random_engine(Cfg(max_len=2304, layers=4), seed=0)
if B > 1:
    eng = Qwen2BatchEngine(eng, B)
eng.reset()
eng.pos.fill_(2048)
for _ in range(3):
    eng.step()
torch.cuda.synchronize()
torch.cuda.cudart().cudaProfilerStart()
eng.step()
torch.cuda.synchronize()
torch.cuda.cudart().cudaProfilerStop()
eng.check()
print("ok")
