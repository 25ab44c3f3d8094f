import glob
import importlib
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("int-flashattention_b200")


@pytest.fixture(scope="session")
def oracle():
    from oracle import intfa_oracle
    return intfa_oracle


def golden_names():
    return sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {k: z[k] for k in z.files}
    for k in ("q", "k", "v", "q8", "k8", "v8", "qs", "ks", "vs", "o"):
        out[k] = torch.from_numpy(out[k])
    out["variant"] = str(out["variant"])
    out["causal"] = bool(out["causal"])
    out["sm_scale"] = float(out["sm_scale"])
    out["block_m"] = int(out["block_m"])
    out["block_n"] = int(out["block_n"])
    return out


def make_qkv(seed, B, H, N, D, std=1.0, outlier=False, device="cpu"):
    """Seeded synthetic fp16 Q/K/V ~ N(0, std); optional x20 outlier channel shared by Q and K."""
    g = torch.Generator().manual_seed(seed)
    q, k, v = (std * torch.randn(B, H, N, D, generator=g) for _ in range(3))
    if outlier:
        ch = int(torch.randint(0, D, (1,), generator=g))
        q[..., ch] *= 20
        k[..., ch] *= 20
    return q.half().to(device), k.half().to(device), v.half().to(device)
