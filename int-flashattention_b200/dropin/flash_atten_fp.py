"""Drop-in for the reference module of the same name (benchmark.py:11): `attention(q, k, v, causal, sm_scale)`,
the floating-point baseline the reference's benchmark and accuracy scripts run next to the int8 operators
(flash_atten_fp.py:152-188).  It is not on the int8 path and gets no kernel of its own here: the call is handed to
PyTorch's scaled_dot_product_attention (a library kernel).  Like the reference's, it takes fp16 or fp8 (e5m2) tensors
[B,H,N,D], positional arguments only, and returns a tensor of q's dtype."""
import torch


def attention(q, k, v, causal, sm_scale):
    HEAD_DIM_Q, HEAD_DIM_K, HEAD_DIM_V = q.shape[-1], k.shape[-1], v.shape[-1]
    assert HEAD_DIM_Q == HEAD_DIM_K and HEAD_DIM_K == HEAD_DIM_V            # flash_atten_fp.py:157-159
    assert HEAD_DIM_K in {16, 32, 64, 128, 256}
    wide = [t if t.dtype in (torch.float16, torch.bfloat16) else t.to(torch.float16) for t in (q, k, v)]
    o = torch.nn.functional.scaled_dot_product_attention(wide[0], wide[1], wide[2], is_causal=bool(causal),
                                                         scale=float(sm_scale))
    return o.to(q.dtype)
