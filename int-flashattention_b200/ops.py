"""Python operator surface over libintfa.so, mirroring the reference's operators.

    attention_full_int8(q, k, v, q_scale, k_scale, v_scale, causal, sm_scale) -> o
        (flash_atten_full_int8.py:187,223)
    attention_int8(q, k, v, q_scale, k_scale, causal, sm_scale) -> o
        (flash_atten_int8.py:181,217)
    quant_pertoken / quant_pertensor (benchmark.py:96-107) and quant_perchannel
    int_flash_attention(q16, k16, v16, causal, sm_scale, variant): prologue + forward

Positional arguments and their meaning are the reference's.  Tensors must live on a
CUDA device; launches are asynchronous on torch's current stream of that device.
PyTorch is used for memory and streams only -- every computation runs in libintfa.so,
and there is no other path: a missing library or a CPU tensor raises.
"""
import ctypes

import torch

from . import _lib

_status = {}          # device index -> int32[1] tensor the kernels report bounded-wait expiry into


def default_G(head_dim, variant="full"):
    """Running-max granularity used when the caller does not choose one.  full-int8: the widest KV
    tile the reference's kernels allow for this head size (BLOCK_N <= HEAD_DIM,
    flash_atten_full_int8.py:88).  half-int8: 128 -- its result does not depend on G beyond fp16
    rounding, and 128-wide KV tiles are the faster ones at both head sizes."""
    if variant == "half":
        return 64 if head_dim == 256 else 128      # (fp16 V tiles of 128 keys x 256 channels do not fit next to K)
    return 128 if head_dim >= 128 else (64 if head_dim >= 64 else 32)


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _status_word(dev):
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status[idx]


def check_status(device=None):
    """Synchronise and raise if any kernel launched through this module on `device` gave up a
    bounded device-side wait.  Returns the raw status word (0 = fine)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _status_word(dev)
    val = int(word.item())
    if val != 0:
        word.zero_()
        raise _lib.IntfaError(_lib.ERR_DEVICE_WAIT,
                              "device-side wait expired (wait code %d, CTA %d)" % (val & 0xff, val >> 8))
    return val


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("int-flashattention_b200 runs on CUDA tensors only (there is no CPU path)")


def _tma_ok(t):
    es = t.element_size()
    return (t.stride(-1) == 1 and t.data_ptr() % 16 == 0
            and all(s > 0 and (s * es) % 16 == 0 for s in t.stride()[:-1]))


def _prep_main(t):
    """TMA wants a contiguous last dim and 16-byte multiples for every other stride."""
    return t if _tma_ok(t) else t.contiguous()


def _scales_f32(s):
    """[B,H,N] scale -> fp32 contiguous (fp16 as benchmark.py makes it is widened by the library)."""
    if s.dtype == torch.float32:
        if s.is_contiguous():
            return s if s.data_ptr() % 16 == 0 else s.clone()
        return s.contiguous()
    if s.dtype == torch.float16:
        src = s.contiguous()
        dst = torch.empty(src.shape, dtype=torch.float32, device=s.device)
        with torch.cuda.device(s.device):      # the library launches on the current device
            _lib.check(_lib.load().intfa_scales_f16_to_f32(src.data_ptr(), dst.data_ptr(), src.numel(), _stream(s)))
        return dst
    return s.to(torch.float32).contiguous()


def _fwd(variant, q, k, v, q_scale, k_scale, v_scale, causal, sm_scale, *, G=None, p_round="triton", kv_order="ascending",
         state=None, q_offset=0, kv_offset=0, return_state=False, return_lse=False, write_o=True,
         debug_tap=None, out_dtype=torch.float16, debug_wait=None):
    # shape constraints, as flash_atten_full_int8.py:189-193
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    _need_cuda(q, k, v, q_scale, k_scale, v_scale)
    lib = _lib.load()
    full = variant == "full"
    if q.dtype != torch.int8 or k.dtype != torch.int8:
        raise TypeError("q and k must be int8")
    if full and v.dtype != torch.int8:
        raise TypeError("full-int8: v must be int8")
    f8v = not full and v.dtype == torch.float8_e5m2       # V (and with it P) in fp8: flash_atten_int8.py:55-56
    if not full and not f8v and v.dtype != torch.float16:
        raise TypeError("half-int8: v must be float16 or float8_e5m2")
    B, H, Nq, D = q.shape
    Nk = k.shape[2]
    H_kv = k.shape[1]                          # grouped-query attention: fewer K/V heads than query heads
    if v.shape[1] != H_kv or H % H_kv != 0:
        raise ValueError("k and v must have the same number of heads, dividing the %d query heads" % H)
    if out_dtype not in (torch.float16, torch.bfloat16):
        raise TypeError("out_dtype must be torch.float16 or torch.bfloat16")
    if G is None:
        G = default_G(D, variant)
    q, k, v = _prep_main(q), _prep_main(k), _prep_main(v)
    qs, ks = _scales_f32(q_scale), _scales_f32(k_scale)
    if Nk % G:
        # the kernel fetches the K scales of a KV step G at a time: give every row room up to the next multiple of G
        ks_pad = torch.zeros(ks.shape[:2] + ((Nk + G - 1) // G * G,), dtype=torch.float32, device=ks.device)
        ks_pad[:, :, :Nk] = ks
        ks = ks_pad
    o = torch.empty((B, H, Nq, D) if write_o else (1, 1, 1, 8), dtype=out_dtype, device=q.device)  # :194-195

    P = _lib.IntfaFwdParams()
    P.q, P.k, P.v, P.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()
    P.q_scale, P.k_scale = qs.data_ptr(), ks.data_ptr()
    P.q_stride = _lib._i64x3(*q.stride()[:3])
    P.k_stride = _lib._i64x3(*k.stride()[:3])
    P.v_stride = _lib._i64x3(*v.stride()[:3])
    P.o_stride = _lib._i64x3(*o.stride()[:3])
    P.qs_stride = _lib._i64x2(*qs.stride()[:2])
    P.ks_stride = _lib._i64x2(*ks.stride()[:2])
    keep = [q, k, v, qs, ks, o]
    if full:
        vs = v_scale.to(torch.float32)
        if vs.dim() == 2:                      # (B,H): one scale per (batch, head), benchmark.py:102-107
            vs = vs.contiguous()
            P.vs_stride = _lib._i64x3(vs.stride(0), vs.stride(1), 0)
        elif vs.dim() == 3:                    # (B,H,D): per channel
            vs = vs.contiguous()
            P.vs_stride = _lib._i64x3(*vs.stride())
        elif vs.dim() == 4:                    # (B,H,ceil(Nk/G),D): one row per KV tile, the CUDA path's layout
            vs = vs.contiguous()
            if vs.shape[2] != (Nk + G - 1) // G:
                raise ValueError("per-tile v_scale needs ceil(Nk/G) = %d rows, got %d" % ((Nk + G - 1) // G, vs.shape[2]))
            P.vs_stride = _lib._i64x3(vs.stride(0), vs.stride(1), vs.stride(3))
            P.vs_stride_blk = vs.stride(2)
        else:
            raise ValueError("v_scale must have shape (B,H), (B,H,D) or (B,H,ceil(Nk/G),D)")
        P.v_scale = vs.data_ptr()
        keep.append(vs)
    P.B, P.H, P.Nq, P.Nk, P.D = B, H, Nq, Nk, D
    P.H_kv = H_kv
    P.o_dtype = 1 if out_dtype == torch.bfloat16 else 0
    P.variant = _lib.VARIANT_FULL if full else (_lib.VARIANT_HALF_FP8 if f8v else _lib.VARIANT_HALF)
    P.causal = 1 if causal else 0
    P.sm_scale = float(sm_scale)
    P.G = int(G)
    P.p_round = {"triton": 0, "rne": 1}[p_round]
    P.kv_order = {"ascending": 0, "descending": 1}[kv_order]
    P.q_offset, P.kv_offset = int(q_offset), int(kv_offset)
    lse = None
    if return_lse:
        lse = torch.empty((B, H, Nq), dtype=torch.float32, device=q.device)
        P.lse_out = lse.data_ptr()
    if state is not None or return_state:
        if state is None:
            m = torch.empty((B, H, Nq), dtype=torch.float32, device=q.device)
            l = torch.empty((B, H, Nq), dtype=torch.float32, device=q.device)
            acc = torch.empty((B, H, Nq, D), dtype=torch.float32, device=q.device)
        else:
            m, l, acc = state
            assert m.is_contiguous() and l.is_contiguous() and acc.is_contiguous()
            assert m.dtype == l.dtype == acc.dtype == torch.float32
            P.state_in = 1
        P.state_m, P.state_l, P.state_acc = m.data_ptr(), l.data_ptr(), acc.data_ptr()
        P.state_out = 1 if return_state else 0
        state = (m, l, acc)
    P.write_o = 1 if write_o else 0
    dbg = None
    if debug_tap is not None:
        tile, step = debug_tap
        dbg_s = torch.zeros((128, G), dtype=torch.int32, device=q.device)
        dbg_p = torch.zeros((128, G), dtype=torch.int8 if full else (torch.uint8 if f8v else torch.float16), device=q.device)
        P.dbg_s, P.dbg_p, P.dbg_tile, P.dbg_step = dbg_s.data_ptr(), dbg_p.data_ptr(), int(tile), int(step)
        dbg = (dbg_s, dbg_p)
    if debug_wait is not None:                 # test hooks of the bounded waits: (limit in kilo-cycles, K step to leave out)
        P.debug_wait_limit_kcycles, P.debug_skip_k_load = int(debug_wait[0]), int(debug_wait[1])
    P.status = _status_word(q.device).data_ptr()
    with torch.cuda.device(q.device):
        _lib.check(lib.intfa_fwd(ctypes.byref(P), _stream(q)))
    del keep
    out = [o if write_o else None]
    if return_state:
        out.append(state)
    if return_lse:
        out.append(lse)
    if dbg is not None:
        out.append(dbg)
    return out[0] if len(out) == 1 else tuple(out)


def attention_full_int8(q, k, v, q_scale, k_scale, v_scale, causal, sm_scale, **kw):
    """Full-int8 attention forward (int8 Q/K/V, int8 P).  Mirrors attention_full_int8 of
    flash_atten_full_int8.py:187,223.  With causal=True the running maximum is carried from the
    off-band to the on-band stage (as flash_atten_int8.py:66,157,166 does); the reference's
    full-int8 Triton kernel drops it (flash_atten_full_int8.py:71,166-179).
    Extra keyword arguments (not in the reference): G (running-max granularity, the reference's
    BLOCK_N), p_round ("triton" | "rne"), kv_order ("ascending" | "descending": the CUDA path walks the KV tiles
    last to first, csrc/flash_fwd_kernel_full_qi8.h:331-469), v_scale of shape (B,H,ceil(Nk/G),D) (one row per KV
    tile, the CUDA path's layout), state/q_offset/kv_offset/return_state (ring attention),
    return_lse, debug_tap, out_dtype (torch.float16 | torch.bfloat16).  k, v and their scales may have
    fewer heads than q (grouped-query attention: query head h reads K/V head h // (H // H_kv))."""
    return _fwd("full", q, k, v, q_scale, k_scale, v_scale, causal, sm_scale, **kw)


def attention_int8(q, k, v, q_scale, k_scale, causal, sm_scale, **kw):
    """Half-int8 attention forward (int8 Q/K, fp16 V and P).  Mirrors attention_int8 of
    flash_atten_int8.py:181,217.  V may also be torch.float8_e5m2: P is then cast to e5m2 as well and P V runs as an
    fp8 matrix product with fp32 accumulation (flash_atten_int8.py:55-56,160)."""
    return _fwd("half", q, k, v, q_scale, k_scale, None, causal, sm_scale, **kw)


# ---------------------------------------------------------------------------------------------
# quantisation prologue
# ---------------------------------------------------------------------------------------------
def _quant_in(X):
    _need_cuda(X)
    if X.dtype != torch.float16 or X.dim() != 4:
        raise TypeError("quantisers take a float16 [B,H,N,D] tensor")
    if X.stride(-1) != 1 or X.data_ptr() % 16 or any(s % 8 for s in X.stride()[:3]):
        X = X.contiguous()
    return X


def quant_pertoken(X):
    """benchmark.py:96-100.  Returns (int8 [B,H,N,D], scale [B,H,N]); the scale is fp32 holding
    the reference's fp16 value."""
    lib = _lib.load()
    X = _quant_in(X)
    B, H, N, D = X.shape
    x8 = torch.empty((B, H, N, D), dtype=torch.int8, device=X.device)
    scale = torch.empty((B, H, N), dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        _lib.check(lib.intfa_quant_pertoken(X.data_ptr(), _lib._i64x3(*X.stride()[:3]), x8.data_ptr(),
                                            scale.data_ptr(), B, H, N, D, _stream(X)))
    return x8, scale


def _quant_v(X, mode):
    lib = _lib.load()
    X = _quant_in(X)
    B, H, N, D = X.shape
    x8 = torch.empty((B, H, N, D), dtype=torch.int8, device=X.device)
    shape = (B, H, D) if mode == _lib.VSCALE_PER_CHANNEL else (B, H)
    scale = torch.empty(shape, dtype=torch.float32, device=X.device)
    nbytes = lib.intfa_quant_v_workspace_bytes(B, H, D)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=X.device)
    with torch.cuda.device(X.device):
        _lib.check(lib.intfa_quant_v(X.data_ptr(), _lib._i64x3(*X.stride()[:3]), x8.data_ptr(), scale.data_ptr(),
                                     mode, B, H, N, D, ws.data_ptr(), nbytes, _stream(X)))
    return x8, scale


def quant_qkv(q, k, v=None, v_mode="per_channel"):
    """The quantisation prologue of one attention call in two launches (one when v is None): per-token q and k
    (benchmark.py:96-100) and, in the same grid, the column absmax of v; then the v quantisation (benchmark.py:102-107
    or its per-channel form).  Bit-identical to quant_pertoken / quant_perchannel / quant_pertensor called one by one.
    Returns (q8, q_scale, k8, k_scale) and, with v, (v8, v_scale) appended."""
    lib = _lib.load()
    q, k = _quant_in(q).contiguous(), _quant_in(k).contiguous()
    B, H, Nq, D = q.shape
    Hkv, Nk = k.shape[1], k.shape[2]
    q8 = torch.empty((B, H, Nq, D), dtype=torch.int8, device=q.device)
    k8 = torch.empty((B, Hkv, Nk, D), dtype=torch.int8, device=q.device)
    qs = torch.empty((B, H, Nq), dtype=torch.float32, device=q.device)
    ks = torch.empty((B, Hkv, Nk), dtype=torch.float32, device=q.device)
    v8 = vs = ws = None
    mode = _lib.VSCALE_PER_CHANNEL if v_mode == "per_channel" else _lib.VSCALE_PER_TENSOR
    vptr = v8ptr = vsptr = wsptr = None
    vst = _lib._i64x3(0, 0, 0)
    nbytes = 0
    if v is not None:
        v = _quant_in(v)
        if v.shape != k.shape:
            raise ValueError("k and v must have the same shape")
        v8 = torch.empty((B, Hkv, Nk, D), dtype=torch.int8, device=q.device)
        vs = torch.empty((B, Hkv, D) if mode == _lib.VSCALE_PER_CHANNEL else (B, Hkv), dtype=torch.float32, device=q.device)
        nbytes = lib.intfa_quant_qkv_workspace_bytes(B, Hkv, Nk, D)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
        vptr, v8ptr, vsptr, wsptr, vst = v.data_ptr(), v8.data_ptr(), vs.data_ptr(), ws.data_ptr(), _lib._i64x3(*v.stride()[:3])
    with torch.cuda.device(q.device):
        _lib.check(lib.intfa_quant_qkv(q.data_ptr(), k.data_ptr(), vptr, vst, q8.data_ptr(), k8.data_ptr(), v8ptr,
                                       qs.data_ptr(), ks.data_ptr(), vsptr, mode, B, H, Hkv, Nq, Nk, D, wsptr, nbytes, _stream(q)))
    return (q8, qs, k8, ks) if v is None else (q8, qs, k8, ks, v8, vs)


def quant_v_with_allreduce(X, mode, group=None):
    """V quantisation for a token-sharded V: local column absmax, all-reduce(MAX) over `group`
    of the B*H*D fp32 bit patterns (order-preserving as int32 because they are non-negative),
    then the quantising pass.  Equals quantising the unsharded tensor bit for bit."""
    import torch.distributed as dist
    lib = _lib.load()
    X = _quant_in(X)
    B, H, N, D = X.shape
    mode_i = {"per_channel": _lib.VSCALE_PER_CHANNEL, "per_tensor": _lib.VSCALE_PER_TENSOR}.get(mode, mode)
    colmax = torch.zeros(B * H * D, dtype=torch.int32, device=X.device)
    st = _lib._i64x3(*X.stride()[:3])
    with torch.cuda.device(X.device):
        _lib.check(lib.intfa_v_colmax(X.data_ptr(), st, colmax.data_ptr(), B, H, N, D, _stream(X)))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(colmax, op=dist.ReduceOp.MAX, group=group)
    x8 = torch.empty((B, H, N, D), dtype=torch.int8, device=X.device)
    shape = (B, H, D) if mode_i == _lib.VSCALE_PER_CHANNEL else (B, H)
    scale = torch.empty(shape, dtype=torch.float32, device=X.device)
    with torch.cuda.device(X.device):
        _lib.check(lib.intfa_v_quant_from_colmax(X.data_ptr(), st, colmax.data_ptr(), x8.data_ptr(),
                                                 scale.data_ptr(), mode_i, B, H, N, D, _stream(X)))
    return x8, scale


def quant_pertensor(X):
    """benchmark.py:102-107: one scale per (batch, head).  Returns (int8, scale [B,H] fp32)."""
    return _quant_v(X, _lib.VSCALE_PER_TENSOR)


def quant_perchannel(X):
    """Per-channel V quantisation: one scale per (batch, head, channel). Returns (int8, scale [B,H,D] fp32)."""
    return _quant_v(X, _lib.VSCALE_PER_CHANNEL)


def int_flash_attention(q, k, v, causal, sm_scale, variant="full", v_mode="per_channel", **kw):
    """fp16 Q/K/V in, fp16 O out: fused quantisation prologue (per-token Q/K; per-channel or
    per-(batch,head) V for the full-int8 variant) followed by the INT8 attention forward.
    Argument order follows the reference's attention(q, k, v, causal, sm_scale) (flash_atten_fp.py:155)."""
    if variant == "full":
        q8, qs, k8, ks, v8, vs = quant_qkv(q, k, v, v_mode)
        return attention_full_int8(q8, k8, v8, qs, ks, vs, causal, sm_scale, **kw)
    q8, qs, k8, ks = quant_qkv(q, k)
    return attention_int8(q8, k8, v, qs, ks, causal, sm_scale, **kw)
