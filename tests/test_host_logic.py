"""CPU: sharding arithmetic and the ring schedule (world_size 2 and 4 over gloo).  The per-chunk
forward is supplied by the oracle here; on GPUs the same driver calls the CUDA operator."""
import importlib
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, make_qkv


def test_bh_slice_covers_everything(pkg):
    sh = pkg.shard
    for B, H, W in [(64, 64, 8), (4, 32, 2), (4, 32, 8), (1, 32, 8), (2, 8, 4)]:
        seen = []
        for r in range(W):
            dim, s, e = sh.bh_slice(B, H, W, r)
            seen += list(range(s, e)) if dim == 1 else [b * H + h for b in range(s, e) for h in range(H)]
        assert sorted(seen) == list(range(B * H))
    with pytest.raises(ValueError):
        sh.bh_slice(3, 5, 4, 0)


def test_take_bh_views(pkg):
    t = torch.arange(4 * 6 * 2).reshape(4, 6, 2)
    parts = [pkg.shard.take_bh(t, 4, 6, 2, r) for r in range(2)]
    assert torch.equal(torch.cat(parts, 0), t)
    t = torch.arange(2 * 8 * 3).reshape(2, 8, 3)
    parts = [pkg.shard.take_bh(t, 2, 8, 4, r) for r in range(4)]
    assert torch.equal(torch.cat([torch.cat(parts[:2], 1), torch.cat(parts[2:], 1)], 0), t)


def test_zigzag_roundtrip_and_balance(pkg):
    sh = pkg.shard
    x = torch.arange(2 * 1 * 64 * 3).reshape(2, 1, 64, 3)
    for W in (1, 2, 4, 8):
        parts = [sh.zigzag_split(x, W, r) for r in range(W)]
        assert torch.equal(sh.zigzag_merge(parts, W), x)
        owners = [sh.owner_of(c, W) for c in range(2 * W)]
        assert sorted(owners) == sorted(list(range(W)) * 2)
        # causal work per rank in half-chunk pairs (diagonal counts 1/2) is the same for every rank
        work = []
        for r in range(W):
            a, b = sh.zigzag_chunks(W, r)
            work.append((a + 0.5) + (b + 0.5))
            assert all(sh.needs(r, c, W) == (c <= b) for c in range(2 * W))
        assert len(set(work)) == 1


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ring_worker(rank, world, port, variant, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("int-flashattention_b200")
        from oracle import intfa_oracle as O
        B, H, N, D, G = 1, 2, 128 * 2 * world, 64, 64
        q, k, v = make_qkv(11, B, H, N, D, std=0.5)
        q8, qs = O.quant_pertoken(q)
        k8, ks = O.quant_pertoken(k)
        v8, vs = O.quant_perchannel(v)
        vv = v8 if variant == "full" else v
        full = O.int8_attention(q8, k8, vv, qs, ks, vs, True, 0.125, variant=variant, G=G)

        def attend(q8_, k8_, v_, qs_, ks_, vs_, sm, q_off, kv_off, state, last):
            o, st = O.int8_attention(q8_, k8_, v_, qs_, ks_, vs_, True, sm, variant=variant, G=G, state=state,
                                     q_offset=q_off, kv_offset=kv_off, return_state=True)
            return (o, None) if last else (None, st)

        sp = lambda t: pkg.shard.zigzag_split(t, world, rank)
        o_loc = pkg.shard.ring_attention_causal(sp(q8), sp(k8), sp(vv), sp(qs), sp(ks), vs, 0.125,
                                                variant=variant, G=G, attend=attend)
        want = sp(full)
        torch.save({"equal": bool(torch.equal(o_loc, want)),
                    "max": float((o_loc.float() - want.float()).abs().max())}, os.path.join(tmpdir, "r%d.pt" % rank))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,variant", [(2, "full"), (2, "half"), (4, "full")])
def test_ring_reproduces_single_pass(world, variant, tmp_path):
    """Ascending-order zigzag ring == single-device ascending pass, bit for bit (same trajectory)."""
    mp.spawn(_ring_worker, args=(world, _free_port(), variant, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        res = torch.load(os.path.join(str(tmp_path), "r%d.pt" % r))
        assert res["equal"], res
