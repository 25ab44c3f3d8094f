"""Attention on HOST-resident tensors: the copies to and from the device overlap the kernels.

The reference's operators take device tensors (flash_atten_full_int8.py:187-223); a caller whose
fp16 Q/K/V live in host memory pays 3 H2D copies and 1 D2H copy per call, which at PCIe rates cost
more than the attention itself.  `HostPipeline` keeps `depth` sets of device buffers and three
streams (copy-in, compute, copy-out): while one call's kernels run, the next call's inputs are
already on their way in and the previous call's output is on its way out.  Per call it performs
exactly `int_flash_attention(q, k, v, causal, sm_scale, variant)` -- prologue + forward -- on the
compute stream.
"""
import torch

from . import ops


class HostPipeline:
    """pipe = HostPipeline((B,H,N,D), device); pipe.submit(hq, hk, hv, ho) ...; pipe.synchronize().

    hq, hk, hv: fp16 host tensors of the given shape (pinned memory makes the copies asynchronous);
    ho: host tensor that receives o.  Calls complete in submission order; `ho` may be read after
    `synchronize()` (or after waiting on the event `submit` returns)."""

    def __init__(self, shape, device, *, causal=False, sm_scale=None, variant="full", depth=2,
                 out_dtype=torch.float16, **kw):
        self.device = torch.device(device)
        self.shape = tuple(shape)
        self.causal, self.variant, self.out_dtype, self.kw = causal, variant, out_dtype, kw
        self.sm_scale = float(sm_scale) if sm_scale is not None else self.shape[-1] ** -0.5
        self.depth = int(depth)
        assert self.depth >= 1
        self.s_in = torch.cuda.Stream(self.device)
        self.s_cmp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self.bufs = [tuple(torch.empty(self.shape, dtype=torch.float16, device=self.device) for _ in range(3))
                     for _ in range(self.depth)]
        self.inputs_free = [None] * self.depth     # event: the compute that read this slot's inputs is done
        self.n = 0
        # everything allocated above (on the caller's stream) is ready before the side streams touch it
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(cur)

    def submit(self, hq, hk, hv, ho):
        slot = self.n % self.depth
        self.n += 1
        dq, dk, dv = self.bufs[slot]
        with torch.cuda.stream(self.s_in):
            if self.inputs_free[slot] is not None:
                self.s_in.wait_event(self.inputs_free[slot])
            dq.copy_(hq, non_blocking=True)
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(self.s_in)
        with torch.cuda.stream(self.s_cmp):
            self.s_cmp.wait_event(ev_in)
            out = ops.int_flash_attention(dq, dk, dv, self.causal, self.sm_scale, variant=self.variant,
                                          out_dtype=self.out_dtype, **self.kw)
            ev_cmp = torch.cuda.Event()
            ev_cmp.record(self.s_cmp)
            self.inputs_free[slot] = ev_cmp
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(ev_cmp)
            ho.copy_(out, non_blocking=True)
            out.record_stream(self.s_out)            # keep the allocator from reusing it before the copy ran
            ev_out = torch.cuda.Event()
            ev_out.record(self.s_out)
        return ev_out

    def synchronize(self):
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.synchronize()
        ops.check_status(self.device)
