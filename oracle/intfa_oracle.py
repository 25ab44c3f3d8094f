"""CPU oracle for the INT8 FlashAttention forward path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain PyTorch-on-CPU tensor code, the arithmetic of the
reference's Triton operators and quantisers.  It exists so that the CUDA path
can be checked against an independent statement of the same math.  Only the
test-suite, the smoke check and the benchmark's CPU-baseline leg may import it;
the product package never does (it fails loudly when its CUDA library is missing).

Parity pin: the reference ships no golden vectors or assertions for this path.
The restatement is therefore pinned against outputs of the reference's own
Triton kernels executed under the Triton interpreter (fixtures under
tests/golden/, produced by tests/golden/make_golden.py).

Reference lines followed (paths relative to the reference project root):
  quant_pertoken            benchmark.py:96-100
  quant_pertensor           benchmark.py:102-107
  full-int8 inner loop      flash_atten_full_int8.py:30-70, prologue/epilogue :149-182
  half-int8 inner loop      flash_atten_int8.py:30-66, prologue/epilogue :141-176
  running max carried over the off-band -> on-band boundary as
                            flash_atten_int8.py:66,157,166 does (the full-int8
                            Triton kernel drops it, flash_atten_full_int8.py:71,166-179;
                            `carry_m=False` reproduces that behaviour).
"""
from __future__ import annotations

import numpy as np
import torch

LOG2E_F32 = np.float32(1.44269504)  # flash_atten_full_int8.py:157


# --------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------
def quant_pertoken(X: torch.Tensor):
    """benchmark.py:96-100 -- per-token absmax int8, arithmetic in X's dtype."""
    X_max, _ = torch.abs(X).max(dim=-1)
    X_scale = X_max / 127
    ret = torch.round(X / X_scale[:, :, :, None]).to(torch.int8)
    return ret, X_scale


def quant_pertensor(X: torch.Tensor):
    """benchmark.py:102-107 -- one scale per (batch, head)."""
    X_max, _ = torch.abs(X).max(dim=-1)
    X_max, _ = torch.max(X_max, dim=-1)
    X_scale = X_max / 127
    ret = torch.round(X / X_scale[:, :, None, None]).to(torch.int8)
    return ret, X_scale


def quant_perchannel(X: torch.Tensor):
    """Per-channel variant of benchmark.py:102-107: absmax over the token axis
    only, one scale per (batch, head, channel); same dtype-following arithmetic."""
    X_max, _ = torch.abs(X).max(dim=-2)
    X_scale = X_max / 127
    ret = torch.round(X / X_scale[:, :, None, :]).to(torch.int8)
    return ret, X_scale


def zero_safe(q8: torch.Tensor, scale: torch.Tensor, X: torch.Tensor, axis: int):
    """The reference divides 0/0 for an all-zero row (NaN -> undefined int8).
    The CUDA prologue defines that case as value 0 with scale 0; apply the same
    definition to an oracle result so the two can be compared bit for bit."""
    zero = scale == 0
    if zero.any():
        q8 = torch.where(zero.unsqueeze(axis).expand_as(q8), torch.zeros_like(q8), q8)
    return q8, scale


# --------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------
def qk_scale_f32(sm_scale: float) -> np.float32:
    """flash_atten_full_int8.py:156-157: fp32(sm_scale) * fp32(1.44269504)."""
    return np.float32(np.float32(sm_scale) * LOG2E_F32)


def _p_to_int8(p: torch.Tensor, p_round: str) -> torch.Tensor:
    if p_round == "triton":
        # flash_atten_full_int8.py:49-51: fp16 cast, fp16 *127, fp16 +0.5, truncating cast
        h = p.to(torch.float16)
        h = h * 127
        return (h + 0.5).to(torch.int8)
    if p_round == "rne":
        # csrc/flash_fwd_kernel_full_qi8.h:387-388 + csrc/utils.h:227-238 (fp32 *127, RNE, saturate)
        return torch.clamp(torch.round(p * np.float32(127.0)), -128, 127).to(torch.int8)
    raise ValueError(p_round)


def _imatmul(a8: torch.Tensor, b8: torch.Tensor) -> torch.Tensor:
    """Exact int8 x int8 -> int32 product through fp32 BLAS: every partial sum is an
    integer below 2**24 as long as the contraction length is <= 1024."""
    assert a8.shape[-1] <= 1024
    return torch.matmul(a8.to(torch.float32), b8.to(torch.float32))


def int8_attention(q8, k8, v, q_scale, k_scale, v_scale, causal, sm_scale, *,
                   variant="full", G=128, block_m=128, carry_m=True, p_round="triton", kv_order="ascending",
                   state=None, q_offset=0, kv_offset=0, return_state=False):
    """Blockwise restatement of _attn_fwd_full_int8 / _attn_fwd_int8.

    q8,k8 int8 [B,H,Nq|Nk,d]; v int8 (variant "full") or fp16 / float8_e5m2 ("half") [B,H,Nk,d];
    q_scale [B,H,Nq], k_scale [B,H,Nk] any float dtype (promoted to fp32 like
    flash_atten_full_int8.py:37-38); v_scale [B,H] or [B,H,d] (full only).
    KV is visited in groups of G columns (G = the reference's BLOCK_N), ascending like the Triton ops or, with
    kv_order="descending", last group first like the CUDA path (csrc/flash_fwd_kernel_full_qi8.h:331-469);
    v_scale may also be [B,H,ceil(Nk/G),d], one row per KV group, the CUDA path's layout
    (csrc/flash_fwd_kernel_full_qi8.h:156-160, csrc/mask.h:313-340);
    `block_m` is the reference's BLOCK_M and only decides which groups use the
    masked formula when causal.  `state`=(m,l,acc) continues a previous call
    (ring attention); q_offset/kv_offset are the global positions of row 0 / col 0.
    Returns o fp16 [B,H,Nq,d] (and optionally the (m,l,acc) state).

    Sequence lengths that are not multiples of the block sizes (the Triton ops leave them unchecked; the
    CUDA path masks them, csrc/mask.h:277-285): rows and columns are padded with zeros up to the next
    multiple, padded COLUMNS get the bias -1e6 of the masked formula (so p = 0 exactly) in the one KV
    group they fall into, padded rows are dropped from every result.
    """
    B, H, Nq_valid, d = q8.shape
    Nk_valid = k8.shape[2]
    assert block_m % G == 0 or G % block_m == 0
    pad_q = (-Nq_valid) % block_m
    pad_k = (-Nk_valid) % G
    if pad_q or pad_k:
        F = torch.nn.functional
        q8 = F.pad(q8, (0, 0, 0, pad_q))
        q_scale = F.pad(q_scale, (0, pad_q))
        k8 = F.pad(k8, (0, 0, 0, pad_k))
        k_scale = F.pad(k_scale, (0, pad_k))
        v = F.pad(v, (0, 0, 0, pad_k))
        if state is not None:
            state = (F.pad(state[0], (0, pad_q)), F.pad(state[1], (0, pad_q), value=1.0),
                     F.pad(state[2], (0, 0, 0, pad_q)))
    Nq, Nk = Nq_valid + pad_q, Nk_valid + pad_k
    c = torch.tensor(qk_scale_f32(sm_scale))
    qs = q_scale.to(torch.float32)
    ks = k_scale.to(torch.float32)
    full = variant == "full"
    if full:
        vs = v_scale.to(torch.float32)
        if vs.dim() == 2:
            vs = vs[:, :, None].expand(B, H, d)
        if vs.dim() == 3:
            vs = vs[:, :, None, :]                  # [B,H,1,d]: one row for every KV group
        # else [B,H,n_groups,d]
    if state is None:
        m = torch.full((B, H, Nq), float("-inf"), dtype=torch.float32)     # :152
        l = torch.ones((B, H, Nq), dtype=torch.float32)                    # :153
        acc = torch.zeros((B, H, Nq, d), dtype=torch.float32)              # :154
    else:
        m, l, acc = (t.clone() for t in state)

    def step(rows, n0, masked, m_r, l_r, acc_r):
        kj = k8[:, :, n0:n0 + G]
        S = _imatmul(q8[:, :, rows], kj.transpose(-1, -2))                 # :36 exact int32
        s = S * qs[:, :, rows, None]                                       # :37
        s = s * ks[:, :, None, n0:n0 + G]                                  # :38
        tail = n0 + G > Nk_valid                                          # the group holds padded columns
        if masked or tail:
            row_id = torch.arange(rows.start, rows.stop)[:, None] + q_offset
            col_id = torch.arange(n0, n0 + G)[None, :] + kv_offset
            vis = (row_id >= col_id) if masked else torch.ones(1, 1, dtype=torch.bool)
            vis = vis & (torch.arange(n0, n0 + G)[None, :] < Nk_valid)
            bias = torch.where(vis, torch.tensor(0.0), torch.tensor(-1.0e6))
            x = s * c + bias                                               # :41
            m_new = torch.maximum(m_r, x.max(-1).values)                   # :42
            x = x - m_new[..., None]                                       # :43
        else:
            m_new = torch.maximum(m_r, s.max(-1).values * c)               # :45
            x = s * c - m_new[..., None]                                   # :46
        p = torch.exp2(x)                                                  # :47
        l_ij = p.sum(-1)                                                   # :48 (un-quantised p)
        alpha = torch.exp2(m_r - m_new)                                    # :53
        l_new = l_r * alpha + l_ij                                         # :54
        acc_new = acc_r * alpha[..., None]                                 # :56
        vj = v[:, :, n0:n0 + G]
        if full:
            p8 = _p_to_int8(p, p_round)                                    # :49-51
            tmp = _imatmul(p8, vj)                                         # :59-60
            vs_j = vs if vs.shape[2] == 1 else vs[:, :, n0 // G:n0 // G + 1]
            tmp = tmp * vs_j / 127                                         # :61
            acc_new = acc_new + tmp                                        # :62
        else:
            if vj.dtype == torch.float8_e5m2:
                pq = p.to(torch.float8_e5m2)                               # flash_atten_int8.py:55-56 (V in fp8: P in fp8 too)
            else:
                pq = p.to(torch.float16)                                   # flash_atten_int8.py:58
            acc_new = acc_new + torch.matmul(pq.float(), vj.float())       # :59
        return m_new, l_new, acc_new

    groups = list(range(0, Nk, G))
    if kv_order == "descending":
        groups.reverse()
    elif kv_order != "ascending":
        raise ValueError(kv_order)
    if not causal:
        rows = slice(0, Nq)
        for n0 in groups:
            m, l, acc = step(rows, n0, False, m, l, acc)
    else:
        for r0 in range(0, Nq, block_m):
            rows = slice(r0, r0 + block_m)
            g_lo = r0 + q_offset            # first global row of the block
            m_r, l_r, acc_r = m[:, :, rows], l[:, :, rows], acc[:, :, rows]
            m_init = m_r.clone()
            for n0 in groups:
                gc = n0 + kv_offset
                if gc + G <= g_lo:                              # off-band, :19-20
                    m_r, l_r, acc_r = step(rows, n0, False, m_r, l_r, acc_r)
                elif gc < g_lo + block_m:                       # on-band, :21-23
                    if not carry_m and gc == g_lo:
                        # the shipped full-int8 kernel enters the on-band stage with the
                        # initial m_i again (flash_atten_full_int8.py:71,173)
                        m_r = m_init
                    m_r, l_r, acc_r = step(rows, n0, True, m_r, l_r, acc_r)
            m[:, :, rows], l[:, :, rows], acc[:, :, rows] = m_r, l_r, acc_r

    if pad_q:
        m, l, acc = m[:, :, :Nq_valid], l[:, :, :Nq_valid], acc[:, :, :Nq_valid]
    o = (acc / l[..., None]).to(torch.float16)                             # :181-182
    if return_state:
        return o, (m, l, acc)
    return o


def log2_lse(m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """flash_atten_int8.py:172 -- M = m_i + log2(l_i)."""
    return m + torch.log2(l)


def attention_full_int8(q, k, v, q_scale, k_scale, v_scale, causal, sm_scale, **kw):
    return int8_attention(q, k, v, q_scale, k_scale, v_scale, causal, sm_scale, variant="full", **kw)


def attention_int8(q, k, v, q_scale, k_scale, causal, sm_scale, **kw):
    return int8_attention(q, k, v, q_scale, k_scale, None, causal, sm_scale, variant="half", **kw)


# --------------------------------------------------------------------------
# exact attention (error-vs-exact yardstick) and error metrics
# --------------------------------------------------------------------------
def exact_attention(q, k, v, causal, sm_scale):
    """fp32 softmax(QK^T * sm_scale) V, the comparison of benchmark.py:152-154 (+ causal mask :225-228)."""
    qf, kf, vf = q.float(), k.float(), v.float()
    s = torch.matmul(qf, kf.transpose(-1, -2)) * sm_scale
    if causal:
        n, mk = s.shape[-2], s.shape[-1]
        keep = torch.arange(n)[:, None] >= torch.arange(mk)[None, :]
        s = s.masked_fill(~keep, float("-inf"))
    return torch.matmul(torch.softmax(s, dim=-1), vf)


def err_metrics(out, ref):
    """max-abs, mean-relative = mean|d|/mean|ref|, and the reference's own formula
    mean(|d|/(|ref|+1e-5)) (benchmark.py:114-115) over ALL elements."""
    o, r = out.double(), ref.double()
    d = (o - r).abs()
    return {
        "max_abs": d.max().item(),
        "mean_rel": (d.mean() / r.abs().mean()).item(),
        "mre_ref_formula": (d / (r.abs() + 1e-5)).mean().item(),
    }
