"""GPU (needs >= 2 devices, skipped otherwise): the sequence-parallel ring and the V all-reduce
quantiser over NCCL, one process per GPU, against a single-device pass on rank 0's GPU.
NVLS is switched off and ranks leave only between steps (no device-side waiting between ranks exists:
chunks land in local HBM through NCCL send/recv before the attention kernel reads them)."""
import importlib
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, make_qkv

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, variant, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        pkg = importlib.import_module("int-flashattention_b200")
        B, H, D = 1, 4, 128
        N = 256 * 2 * world
        q, k, v = make_qkv(51, B, H, N, D, std=0.5, device=dev)
        sp = lambda t: pkg.shard.zigzag_split(t, world, rank).contiguous()
        # quantise the LOCAL shards; per-channel V absmax is all-reduced so it equals the unsharded one
        q8, qs = pkg.quant_pertoken(sp(q))
        k8, ks = pkg.quant_pertoken(sp(k))
        v8, vs = pkg.shard.quantize_v_global(sp(v), "per_channel")
        fq8, fqs = pkg.quant_pertoken(q)
        fk8, fks = pkg.quant_pertoken(k)
        fv8, fvs = pkg.quant_perchannel(v)
        ok_quant = bool(torch.equal(v8, sp(fv8)) and torch.equal(vs, fvs) and torch.equal(q8, sp(fq8)))
        if variant == "full":
            one = pkg.attention_full_int8(fq8, fk8, fv8, fqs, fks, fvs, True, 0.09)
            loc = pkg.shard.ring_attention_causal(q8, k8, v8, qs, ks, vs, 0.09, variant="full")
        else:
            one = pkg.attention_int8(fq8, fk8, v, fqs, fks, True, 0.09)
            loc = pkg.shard.ring_attention_causal(q8, k8, sp(v), qs, ks, None, 0.09, variant="half")
        pkg.check_status(dev)
        want = sp(one)
        torch.save({"quant": ok_quant, "equal": bool(torch.equal(loc, want)),
                    "max": float((loc.float() - want.float()).abs().max())}, os.path.join(tmpdir, "r%d.pt" % rank))
        dist.barrier(device_ids=[rank])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["full", "half"])
def test_ring_equals_single_device_pass(variant, tmp_path):
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    mp.spawn(_worker, args=(world, _free_port(), variant, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), "r%d.pt" % r))
        assert res["quant"], res
        assert res["equal"], res        # ascending order + carried state = the single-device trajectory, bit for bit
