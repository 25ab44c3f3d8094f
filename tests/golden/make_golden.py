"""Generate the golden fixtures in this directory from the reference itself.

Runs the reference's UNMODIFIED Triton operators (flash_atten_full_int8.py,
flash_atten_int8.py) and quantisers (benchmark.py:96-107) on CPU tensors under
the Triton interpreter, with the autotune list pinned to one (BLOCK_M, BLOCK_N)
per case.  The reference's configs.py queries the GPU driver at import
(configs.py:7-8,17), so a stand-in `configs` module with the same exports is
placed in sys.modules first; nothing else of the reference is replaced.

Usage (only where a checkout of the reference is present; the fixtures are committed):
    python tests/golden/make_golden.py /path/to/reference [case name ...]
"""
import importlib
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import pytest
import torch
import triton
import triton.language as tl

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(ref_dir, block_m, block_n):
    stub = types.ModuleType("configs")
    stub.pytest, stub.torch, stub.triton, stub.tl = pytest, torch, triton, tl
    stub.is_hip = lambda: False
    stub.configs = [triton.Config({"BLOCK_M": block_m, "BLOCK_N": block_n}, num_stages=3, num_warps=4)]
    stub.keep = lambda conf: True
    sys.modules["configs"] = stub
    if ref_dir not in sys.path:
        sys.path.insert(0, ref_dir)
    for name in ("flash_atten_full_int8", "flash_atten_int8"):
        sys.modules.pop(name, None)
    full = importlib.import_module("flash_atten_full_int8")
    half = importlib.import_module("flash_atten_int8")
    return full, half


def load_quantisers(ref_dir):
    """benchmark.py drags in plotting/bench imports; take only the two quantiser
    functions by executing their source lines (benchmark.py:96-107) unmodified."""
    src = open(os.path.join(ref_dir, "benchmark.py")).read().splitlines()
    body = "\n".join(src[95:107])
    ns = {"torch": torch}
    exec(compile(body, "benchmark.py[96:107]", "exec"), ns)
    return ns["quant_pertoken"], ns["quant_pertensor"]


def make_inputs(seed, B, H, N, D, dist, outlier=False):
    g = torch.Generator().manual_seed(seed)
    if dist == "normal":
        q, k, v = (torch.randn(B, H, N, D, generator=g) for _ in range(3))
    elif dist == "normal_half":
        q, k, v = (0.5 * torch.randn(B, H, N, D, generator=g) for _ in range(3))
    elif dist == "uniform":
        q, k, v = (torch.rand(B, H, N, D, generator=g) for _ in range(3))
    if outlier:
        ch = int(torch.randint(0, D, (1,), generator=g))
        q[..., ch] *= 20
        k[..., ch] *= 20
    return q.half(), k.half(), v.half()


CASES = [
    # name, variant, causal, B,H,N,D, BLOCK_M, BLOCK_N, sm_scale, dist, outlier
    ("c1_full_nc_d64", "full", False, 1, 4, 512, 64, 128, 64, 0.125, "normal", False),
    ("full_nc_d128_g128", "full", False, 1, 1, 256, 128, 128, 128, 128 ** -0.5, "normal", False),
    ("full_nc_d128_g64", "full", False, 1, 1, 256, 128, 128, 64, 128 ** -0.5, "normal", False),
    ("half_c_d128_g128", "half", True, 1, 1, 384, 128, 128, 128, 128 ** -0.5, "normal", True),
    ("half_c_d128_g64", "half", True, 1, 1, 256, 128, 128, 64, 128 ** -0.5, "normal", True),
    ("half_nc_d64", "half", False, 1, 2, 256, 64, 128, 64, 0.125, "normal", False),
    ("full_c_shipped_d64", "full", True, 1, 1, 256, 64, 128, 64, 0.125, "normal_half", False),
    ("acc_test_full_d32", "full", False, 1, 1, 32, 32, 32, 32, 1.0, "uniform", False),
    ("acc_test_half_d32", "half", False, 1, 1, 32, 32, 32, 32, 1.0, "uniform", False),
    # the largest head dim the ops accept (flash_atten_full_int8.py:193).  (The smallest, 16, passes the host
    # assertion but no kernel can be built for it: every BLOCK_N of configs.py:16 is >= 32 and
    # flash_atten_full_int8.py:88 / flash_atten_int8.py:82 assert BLOCK_N <= HEAD_DIM.)
    ("full_nc_d256_g128", "full", False, 1, 1, 256, 256, 128, 128, 0.0625, "normal", False),
    ("half_c_d256_g64", "half", True, 1, 1, 256, 256, 128, 64, 0.0625, "normal", True),
    # (The half-int8 op with V in float8_e5m2, flash_atten_int8.py:55-56,160, runs under the interpreter too, but its
    # emulation of the fp32 -> fp8 cast is not the GPU's: it adds the cut-off bit without carrying a mantissa overflow
    # into the exponent (triton/runtime/interpreter.py, _convert_float), so such outputs would pin the emulator, not
    # the reference.  No fixture is made for that branch.)
]


def main(ref_dir, only=()):
    quant_pertoken, quant_pertensor = load_quantisers(ref_dir)
    for i, (name, variant, causal, B, H, N, D, BM, BN, sm_scale, dist, outlier) in enumerate(CASES):
        if only and name not in only:
            continue
        full, half = load_reference(ref_dir, BM, BN)
        q, k, v = make_inputs(1000 + i, B, H, N, D, dist, outlier)
        q8, qs = quant_pertoken(q)
        k8, ks = quant_pertoken(k)
        v8, vs = quant_pertensor(v)
        if variant == "full":
            o = full.attention_full_int8(q8, k8, v8, qs, ks, vs, causal, sm_scale)
        else:
            o = half.attention_int8(q8, k8, v, qs, ks, causal, sm_scale)
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            variant=variant, causal=causal, sm_scale=np.float64(sm_scale), block_m=BM, block_n=BN,
            q=q.numpy(), k=k.numpy(), v=v.numpy(),
            q8=q8.numpy(), k8=k8.numpy(), v8=v8.numpy(),
            qs=qs.numpy(), ks=ks.numpy(), vs=vs.numpy(),
            o=o.numpy())
        print(name, "ok", tuple(o.shape), float(o.float().abs().mean()))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path to the reference checkout> [case name ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))
