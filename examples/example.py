"""The reference's example.lua in Python: start this in several terminals.

The first process founds the shared tensor at 127.0.0.1:50000, the others join it; each adds a tensor of ones per
iteration and prints what it sees.  Pass ``cuda`` as the first argument to keep the replica on a GPU.
"""
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))  # run from a checkout without installing

import sharedtensor  # noqa: E402

device = "cuda" if len(sys.argv) > 1 and sys.argv[1] == "cuda" else "cpu"
x = torch.arange(1, 5, dtype=torch.float32, device=device)
a = sharedtensor.createOrFetch("127.0.0.1", 50000, x)
try:
    while True:
        a.copyToTensor(x)
        results = torch.ones_like(x)       # "do something computationally intensive with x"
        a.addFromTensor(results)           # propagated asynchronously to every other process
        print(x.tolist())
        time.sleep(1)
except KeyboardInterrupt:
    a.close()
