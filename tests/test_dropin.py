"""The drop-in modules, driven the way the reference's benchmark.py drives its own: `from flash_atten_int8 import
attention_int8`, `from flash_atten_full_int8 import attention_full_int8` (benchmark.py:12-13), positional arguments,
scales as quant_pertoken / quant_pertensor make them (fp16), at the shapes of its acc_test call (benchmark.py:212:
N_CTX=32, HEAD_DIM=32) and of its bench sweep (HEAD_DIM=64, benchmark.py:23)."""
import importlib
import os
import sys

import pytest
import torch

DROPIN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "int-flashattention_b200", "dropin")


def _modules():
    if DROPIN not in sys.path:
        sys.path.insert(0, DROPIN)
    return importlib.import_module("flash_atten_int8"), importlib.import_module("flash_atten_full_int8")


def test_dropin_modules_export_the_reference_names():
    half, full = _modules()
    assert callable(half.attention_int8) and callable(full.attention_full_int8)
    # the other two modules benchmark.py imports (benchmark.py:9,11) resolve inside the drop-in directory as well
    fp, cfg = importlib.import_module("flash_atten_fp"), importlib.import_module("configs")
    assert os.path.dirname(os.path.abspath(fp.__file__)) == os.path.abspath(DROPIN)
    assert os.path.dirname(os.path.abspath(cfg.__file__)) == os.path.abspath(DROPIN)
    assert callable(fp.attention) and cfg.is_hip() is False and isinstance(cfg.configs, list) and cfg.keep(None)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
def test_float_baseline_pass_through(causal):
    """`attention(q, k, v, causal, sm_scale)` as benchmark.py:156,167 call it: fp16, then fp8 (e5m2) inputs."""
    _modules()
    fp = importlib.import_module("flash_atten_fp")
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(21)
    q, k, v = (torch.rand(1, 2, 128, 64, generator=g).half().to(dev) for _ in range(3))
    s = torch.matmul(q.float(), k.float().transpose(2, 3)) * 0.7
    if causal:
        s = s + torch.triu(torch.full((128, 128), float("-inf"), device=dev), 1)
    ref = torch.matmul(torch.softmax(s, dim=-1), v.float())
    out = fp.attention(q, k, v, causal, 0.7)
    assert out.dtype == torch.float16 and (out.float() - ref).abs().max() < 1e-2          # benchmark.py:242
    out8 = fp.attention(q.to(torch.float8_e5m2), k.to(torch.float8_e5m2), v.to(torch.float8_e5m2), causal, 0.7)
    assert out8.dtype == torch.float8_e5m2 and (out8.float() - ref).abs().max() < 0.2


@pytest.mark.gpu
@pytest.mark.parametrize("B,H,N,D", [(1, 2, 32, 32), (2, 4, 1024, 64)])
def test_acc_test_call_pattern(B, H, N, D, oracle):
    half, full = _modules()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(20)
    q, k, v = (torch.rand(B, H, N, D, generator=g).half() for _ in range(3))     # benchmark.py:140-142
    q8, qs = oracle.quant_pertoken(q)                                              # :158-160
    k8, ks = oracle.quant_pertoken(k)
    v8, vs = oracle.quant_pertensor(v)
    G = 32 if D == 32 else 64
    o_half = half.attention_int8(q8.to(dev), k8.to(dev), v.to(dev), qs.to(dev), ks.to(dev), False, 1.0)
    o_full = full.attention_full_int8(q8.to(dev), k8.to(dev), v8.to(dev), qs.to(dev), ks.to(dev), vs.to(dev), False, 1.0)
    r_half = oracle.attention_int8(q8, k8, v, qs, ks, False, 1.0, G=G)
    r_full = oracle.attention_full_int8(q8, k8, v8, qs, ks, vs, False, 1.0, G=G)
    for o, r in ((o_half, r_half), (o_full, r_full)):
        assert o.dtype == torch.float16 and o.shape == (B, H, N, D)
        e = oracle.err_metrics(o.cpu(), r)
        assert e["max_abs"] <= 4e-3 and e["mean_rel"] <= 3e-4, e
