"""GPU: intfa_quant_v_static, the V quantiser for hosts that may not allocate device memory
(plug-ins inside someone else's memory pool, serving callbacks that must not call cudaMalloc).
Its scratch is a fixed array inside the library, so the caller passes only inputs and outputs.

The call goes straight through the C ABI with caller-owned buffers and must reproduce
intfa_quant_v (caller-provided workspace) bit for bit -- the quantised tensors are integers and the
scales are fp16-valued, so the tolerance is zero, as for the other quantiser tests.  Two calls are
made back to back on different data: the second would inherit the first call's column maxima if the
entry point failed to clear the part of the shared array it uses.  This file sorts last so that a
run that stops at the first failure has already exercised everything else; it also passes alone in
a fresh process (its first call on the device performs the one-time symbol-address lookup).
"""
import ctypes
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _run_pair(L, lib, v, mode, dev):
    B, H, N, D = v.shape
    st = L._i64x3(*v.stride()[:3])
    shape = (B, H, D) if mode == L.VSCALE_PER_CHANNEL else (B, H)
    # existing entry point: caller-provided workspace
    ref8 = torch.empty((B, H, N, D), dtype=torch.int8, device=dev)
    refs = torch.empty(shape, dtype=torch.float32, device=dev)
    nbytes = lib.intfa_quant_v_workspace_bytes(B, H, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    L.check(lib.intfa_quant_v(v.data_ptr(), st, ref8.data_ptr(), refs.data_ptr(), mode, B, H, N, D,
                              ws.data_ptr(), nbytes, _stream(v)))
    # new entry point: outputs only, no workspace
    out8 = torch.full((B, H, N, D), 99, dtype=torch.int8, device=dev)
    outs = torch.full(shape, -1.0, dtype=torch.float32, device=dev)
    L.check(lib.intfa_quant_v_static(v.data_ptr(), st, out8.data_ptr(), outs.data_ptr(), mode, B, H, N, D, _stream(v)))
    torch.cuda.synchronize(dev)
    assert torch.equal(outs, refs)
    assert torch.equal(out8, ref8)


def test_static_scratch_quantiser_matches_workspace_quantiser():
    assert torch.cuda.is_available()
    dev = torch.device("cuda:0")
    L = importlib.import_module("int-flashattention_b200._lib")
    lib = L.load()
    g = torch.Generator().manual_seed(77)
    big = (3.0 * torch.randn(2, 4, 1024, 128, generator=g)).half().to(dev)     # large maxima first ...
    small = (0.05 * torch.randn(2, 4, 1024, 128, generator=g)).half().to(dev)  # ... then small ones: stale scratch would show
    with torch.cuda.device(dev):
        _run_pair(L, lib, big, L.VSCALE_PER_CHANNEL, dev)
        _run_pair(L, lib, small, L.VSCALE_PER_CHANNEL, dev)
        _run_pair(L, lib, small[:, :, :384, :64].contiguous(), L.VSCALE_PER_TENSOR, dev)


def test_static_scratch_quantiser_rejects_oversize():
    dev = torch.device("cuda:0")
    L = importlib.import_module("int-flashattention_b200._lib")
    lib = L.load()
    limit = lib.intfa_quant_v_static_max_words()
    assert limit == 65536
    B, H, N, D = 9, 64, 8, 128                      # B*H*D = 73728 > limit; tiny N keeps the buffers small
    v = torch.zeros((B, H, N, D), dtype=torch.float16, device=dev)
    out8 = torch.empty((B, H, N, D), dtype=torch.int8, device=dev)
    outs = torch.empty((B, H, D), dtype=torch.float32, device=dev)
    rc = lib.intfa_quant_v_static(v.data_ptr(), L._i64x3(*v.stride()[:3]), out8.data_ptr(), outs.data_ptr(),
                                  L.VSCALE_PER_CHANNEL, B, H, N, D, _stream(v))
    assert rc == L.ERR_TOO_LARGE
    assert "exceeds" in L.last_error()
