"""The full-int8 kernels quantise P as  trunc(fp16(fp16(fp16(p)*127) + 0.5))  (flash_atten_full_int8.py:49-51).
P depends on p only through fp16(p), so a cheaper evaluation can be checked exhaustively, on every fp16 value in
[0, 1].  The pipelined kernel uses  z = fp16 fma(fp16(p), 127, 0.5)  (ONE rounding where the reference has two),
then floor(z) as the low byte of  fp32(z) + 1.5*2^23  rounded toward minus infinity."""
import numpy as np

K_MAGIC = np.float64(12582912.0)    # 1.5 * 2^23


def test_single_fp16_fma_then_floor_equals_the_fp16_chain_for_every_fp16_p():
    p16 = np.arange(0, 0x3C00 + 1, dtype=np.uint16).view(np.float16)          # 0 .. 1.0
    y = (p16.astype(np.float64) * 127.0).astype(np.float16)
    t = (y.astype(np.float64) + 0.5).astype(np.float16)
    ref = np.trunc(t.astype(np.float64)).astype(np.int64)
    # fp16 fma: the exact p16*127 + 0.5 fits a float64, then ONE rounding (to nearest even) to fp16
    z = (p16.astype(np.float64) * 127.0 + 0.5).astype(np.float16)
    # fp32(z) + 1.5*2^23, rounded toward minus infinity: exact sum in float64, floor to the fp32 grid (spacing 1 there)
    u = np.floor(z.astype(np.float64) + K_MAGIC).astype(np.float32)
    got = (u.view(np.uint32) & 0xFF).astype(np.int64)
    assert np.array_equal(got, ref)
    assert ref.min() == 0 and ref.max() == 127


def test_source_uses_the_checked_constants():
    import os
    csrc = os.path.join(os.path.dirname(__file__), "..", "int-flashattention_b200", "csrc")
    pipe = open(os.path.join(csrc, "intfa_fwd_pipe_softmax.inc")).read()
    assert "0x57F057F0u, 0x38003800u" in pipe      # fp16x2 (127, 127) and (0.5, 0.5)
