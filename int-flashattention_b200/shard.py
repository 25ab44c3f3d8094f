"""Multi-GPU decompositions of the INT8 attention forward (one process per GPU).

The reference has no multi-device code: its only decomposition is the launch grid over
(query block, batch*head) (flash_atten_full_int8.py:89-95, :203).  Two decompositions follow
from that structure:

* batch x heads sharding -- every (batch, head) pair is independent, so ranks take disjoint
  slices and never communicate (`bh_slice`).
* a sequence-parallel ring for long causal context -- every rank owns two half-chunks of the
  sequence ("zigzag": half-chunks r and 2P-1-r, which balances causal work), keeps its query
  rows and their running (m, l, acc) state, and receives int8 K/V half-chunks plus fp32 K scales
  from their owners with point-to-point send/recv, in ASCENDING global order, so that every query
  row visits its keys in the same order and at the same running-max granularity as a
  single-device pass (the full-int8 result depends on that order).  Transfers are posted ahead of
  the attention launches on a side stream (by default all of them at the start: the gathered int8
  K/V of the whole sequence is ~1 GiB at 131072 tokens x 32 heads), landing in local HBM.

The host logic here is backend-agnostic: it moves tensors with torch.distributed (NCCL on GPUs,
gloo in CPU tests) and calls an `attend` function for the per-chunk forward, which defaults to
the CUDA operator.
"""
import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------
# batch x heads sharding (no communication)
# ------------------------------------------------------------------------------------------
def bh_slice(B, H, world, rank):
    """Slice of the batch (or, when the batch is smaller than the world, of the heads) that `rank`
    owns.  Returns (dim, start, stop) with dim 0 = batch, 1 = heads.  Requires an even split."""
    if B % world == 0:
        per = B // world
        return 0, rank * per, (rank + 1) * per
    if (B * H) % world == 0 and world % B == 0:
        ranks_per_batch = world // B
        per = H // ranks_per_batch
        b = rank // ranks_per_batch
        h0 = (rank % ranks_per_batch) * per
        return 1, b * H + h0, b * H + h0 + per          # indices into the flattened B*H axis
    raise ValueError("batch=%d heads=%d do not split evenly over %d ranks" % (B, H, world))


def take_bh(t, B, H, world, rank):
    """Local shard of a [B,H,...] tensor under `bh_slice` (a view; no copy)."""
    dim, s, e = bh_slice(B, H, world, rank)
    if dim == 0:
        return t[s:e]
    b = s // H
    return t[b:b + 1, s - b * H:e - b * H]


# ------------------------------------------------------------------------------------------
# sequence-parallel ring (zigzag, ascending order)
# ------------------------------------------------------------------------------------------
def zigzag_chunks(world, rank):
    """Global half-chunk indices owned by `rank`: (rank, 2*world-1-rank)."""
    return rank, 2 * world - 1 - rank


def owner_of(chunk, world):
    return chunk if chunk < world else 2 * world - 1 - chunk


def needs(rank, chunk, world):
    """True if `rank` has a query half-chunk that attends (causally) to KV half-chunk `chunk`."""
    return chunk <= 2 * world - 1 - rank


def zigzag_split(x, world, rank, dim=2):
    """Local shard [.., 2*Nh, ..] of a full-sequence tensor: half-chunks (rank, 2P-1-rank) concatenated."""
    n = x.shape[dim]
    assert n % (2 * world) == 0
    nh = n // (2 * world)
    a, b = zigzag_chunks(world, rank)
    return torch.cat([x.narrow(dim, a * nh, nh), x.narrow(dim, b * nh, nh)], dim=dim)


def zigzag_merge(parts, world, dim=2):
    """Inverse of zigzag_split over the list of all ranks' local tensors."""
    nh = parts[0].shape[dim] // 2
    halves = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(world, r)
        halves[a] = p.narrow(dim, 0, nh)
        halves[b] = p.narrow(dim, nh, nh)
    return torch.cat(halves, dim=dim)


def _cuda_attend(variant, G):
    from . import ops

    def attend(q8, k8, v, qs, ks, vs, sm_scale, q_offset, kv_offset, state, last):
        kw = dict(G=G, state=state, q_offset=q_offset, kv_offset=kv_offset, return_state=not last, write_o=last)
        if variant == "full":
            out = ops.attention_full_int8(q8, k8, v, qs, ks, vs, True, sm_scale, **kw)
        else:
            out = ops.attention_int8(q8, k8, v, qs, ks, True, sm_scale, **kw)
        return (out, None) if last else (None, out[1])
    return attend


def ring_attention_causal(q8, k8, v, q_scale, k_scale, v_scale, sm_scale, *, variant="full", G=None,
                          group=None, attend=None, comm_stream=None, prefetch=None):
    """Causal attention over a sequence sharded zigzag across the ranks of `group`.

    Local inputs are [B,H,2*Nh,D] (q8,k8 int8; v int8 or fp16) with scales [B,H,2*Nh]; rows
    [0,Nh) are global half-chunk `rank`, rows [Nh,2Nh) are half-chunk 2P-1-rank.  v_scale must
    already be the GLOBAL V scale (see quantize_v_global).  `prefetch` = how many half-chunk
    transfers are posted ahead of the attention launches (None = all of them at the start).
    Returns the local o [B,H,2*Nh,D] fp16.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, H, N2, D = q8.shape
    nh = N2 // 2
    if attend is None:
        from . import ops
        attend = _cuda_attend(variant, G if G is not None else ops.default_G(D, variant))
    on_gpu = q8.is_cuda
    mine = zigzag_chunks(world, rank)
    q_half = [(q8[:, :, :nh], q_scale[:, :, :nh]), (q8[:, :, nh:], q_scale[:, :, nh:])]
    local_kv = {mine[0]: (k8[:, :, :nh].contiguous(), v[:, :, :nh].contiguous(), k_scale[:, :, :nh].contiguous().float()),
                mine[1]: (k8[:, :, nh:].contiguous(), v[:, :, nh:].contiguous(), k_scale[:, :, nh:].contiguous().float())}
    state = [None, None]
    out = [None, None]
    if on_gpu and comm_stream is None:
        comm_stream = torch.cuda.Stream(device=q8.device)
    n_chunks = 2 * world
    depth = n_chunks if prefetch is None else max(1, int(prefetch))
    free_bufs = []                      # receive buffers whose chunk has been consumed

    def post(c):
        """Start the transfer of KV half-chunk c (send if owned, recv if needed). Returns (tensors, works)."""
        own = owner_of(c, world)
        if own == rank:
            peers = [r for r in range(world) if r != rank and needs(r, c, world)]
            ops_ = [dist.P2POp(dist.isend, t, dist.get_global_rank(group, r) if group is not None else r, group)
                    for r in peers for t in local_kv[c]]
            tensors = local_kv[c]
        elif needs(rank, c, world):
            tensors = free_bufs.pop() if free_bufs else tuple(torch.empty_like(t) for t in local_kv[mine[0]])
            src = dist.get_global_rank(group, own) if group is not None else own
            ops_ = [dist.P2POp(dist.irecv, t, src, group) for t in tensors]
        else:
            return None, []
        if not ops_:
            return tensors, []
        if on_gpu:
            comm_stream.wait_stream(torch.cuda.current_stream(q8.device))   # a reused buffer: after its last reader
            with torch.cuda.stream(comm_stream):
                works = dist.batch_isend_irecv(ops_)
        else:
            works = dist.batch_isend_irecv(ops_)
        return tensors, works

    # transfers are posted `depth` half-chunks ahead of the attention launches, in ascending order on
    # every rank (so sends and receives of each pair match); by default all of them up front -- the
    # gathered int8 K/V of the whole sequence is small next to HBM
    pending = {}
    nxt = 0
    while nxt < min(depth, n_chunks):
        pending[nxt] = post(nxt)
        nxt += 1
    for c in range(n_chunks):
        tensors, works = pending.pop(c)
        for w in works:
            w.wait()                      # GPU: makes the current stream wait for the transfer
        if tensors is not None:
            kc, vc, ksc = tensors
            for h in range(2):
                g = mine[h]               # global half-chunk of this query half
                if c > g:
                    continue
                last = c == g
                qh, qsh = q_half[h]
                o, st = attend(qh, kc, vc, qsh, ksc, v_scale, sm_scale, g * nh, c * nh, state[h], last)
                if last:
                    out[h] = o
                else:
                    state[h] = st
            if owner_of(c, world) != rank:
                free_bufs.append(tensors)
        if nxt < n_chunks:
            pending[nxt] = post(nxt)
            nxt += 1
    return torch.cat(out, dim=2)


def quantize_v_global(v, mode, group=None):
    """Per-channel (or per-(batch,head)) V quantisation whose absmax spans the WHOLE sequence:
    local column absmax, all-reduce(MAX) of B*H*D values, then the quantising pass -- bit-identical
    to quantising the unsharded tensor on one device."""
    from . import ops
    return ops.quant_v_with_allreduce(v, mode, group)
