"""The full-int8 kernels quantise P as  trunc(fp16(fp16(fp16(p)*127) + 0.5))  (flash_atten_full_int8.py:49-51).
The CUDA code evaluates the last two steps as the low byte of  fp32 fma(y, 1.000489, 1.5*2^23)  with
y = fp16(fp16(p)*127).  P depends on p only through fp16(p), so the identity can be checked exhaustively:
every fp16 value in [0, 1]."""
import numpy as np

K_A = np.float32(1.000489)          # the constant in csrc/intfa_fwd_pipe_softmax.inc
K_MAGIC = np.float64(12582912.0)    # 1.5 * 2^23


def test_fma_rounding_equals_the_fp16_chain_for_every_fp16_p():
    p16 = np.arange(0, 0x3C00 + 1, dtype=np.uint16).view(np.float16)          # 0 .. 1.0
    y = (p16.astype(np.float64) * 127.0).astype(np.float16)                   # fp16(p16 * 127), correctly rounded
    t = (y.astype(np.float64) + 0.5).astype(np.float16)                       # fp16(y + 0.5)
    ref = np.trunc(t.astype(np.float64)).astype(np.int64)
    # fp32 fma: the exact product-sum fits a float64 (24-bit x 24-bit product next to 2^23), then ONE rounding to fp32
    u = (y.astype(np.float64) * np.float64(K_A) + K_MAGIC).astype(np.float32)
    got = (u.view(np.uint32) & 0xFF).astype(np.int64)
    assert np.array_equal(got, ref)
    assert ref.min() == 0 and ref.max() == 127


def test_source_uses_the_checked_constant():
    import os
    src = open(os.path.join(os.path.dirname(__file__), "..", "int-flashattention_b200", "csrc",
                            "intfa_fwd_pipe_softmax.inc")).read()
    assert "1.000489f" in src
