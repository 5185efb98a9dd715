"""KV-split decode over a real NCCL communicator through the C ABI (flat_splitkv_decode_nccl): two ranks, one GPU
each, every rank holding half of one sequence's pages.  The merged result on both ranks equals the CPU oracle on the
whole sequence and the single-GPU decode.  The peer-memory route (flat_splitkv_decode_peer: one kernel that stores the
partial into both ranks' buffers, waits for the other's flag and merges) runs on the same ranks and must give the
same bits as the NCCL route, step after step (both receive buffers and their reuse).  Needs two GPUs; the plumbing around it (sharding, merge formula) is covered
on CPU with gloo in test_distributed_cpu.py."""
import os
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, result):
    sys.path.insert(0, ROOT)
    import importlib.util

    import torch.distributed as dist
    from __graft_entry__ import load_package
    fa = load_package()
    spec = importlib.util.spec_from_file_location("fd", os.path.join(ROOT, "flat-attention_b200", "distributed.py"))
    fd = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fd)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ctx = fa.Context(rank)
        Hq, Hkv, D, ps, theta, n = 32, 8, 128, 16, 5e5, 16 * 301 + 5
        g = torch.Generator().manual_seed(9)
        K = torch.randn(n, Hkv * D, generator=g).bfloat16()
        V = torch.randn(n, Hkv * D, generator=g).bfloat16()
        Q = torch.randn(1, Hq * D, generator=g).bfloat16()
        first, count = fd.shard_pages(n, ps, world, rank)
        pages = (count + ps - 1) // ps
        pool = pages + 2
        perm = np.random.default_rng(rank).permutation(pool).astype(np.int32)[:pages]
        Kc = torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16)
        Vc = torch.zeros(pool * ps, Hkv * D, dtype=torch.bfloat16)
        for i in range(pages):
            lo, hi = first + i * ps, min(first + count, first + (i + 1) * ps)
            Kc[perm[i] * ps:perm[i] * ps + hi - lo] = K[lo:hi]
            Vc[perm[i] * ps:perm[i] * ps + hi - lo] = V[lo:hi]
        lens, qpos, tab = np.array([count], np.int32), np.array([n - 1], np.int32), perm.reshape(1, pages)
        gathered = torch.empty(world * Hq * (D + 1), dtype=torch.float32, device="cuda")
        out = ctx.create_decode_output_buffer(fa.BF16, 1, Hq, D)
        dist.barrier()
        comm = fd.nccl_comm_ptr()
        for _ in range(2):  # twice: the gather buffer is reused
            ctx.splitkv_decode_nccl(comm, rank, world, fa.BF16, 1, Hq, Hkv, D, ps, pool, pages, torch.from_numpy(tab).cuda(),
                                    torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda(), tab, lens, fa.config(True),
                                    theta, Q.cuda(), Kc.cuda(), Vc.cuda(), gathered, out)
        ctx.synchronize()
        assert ctx.device_status() == 0
        o, l = ctx.split_decode_output(out, fa.BF16, 1, Hq, D)
        if rank == 0:
            from tests.test_gpu_decode_cache import oracle_decode
            eo, el = oracle_decode(Q[0].float().numpy(), K.float().numpy(), V.float().numpy(), Hq, Hkv, D, theta, n - 1, 0, True)
            result["o"] = float(np.abs(o.float().cpu().numpy().reshape(-1) - eo).max())
            result["l"] = float(np.abs(l.cpu().numpy().reshape(-1) - el).max())
        both = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(both, out)
        result["same_%d" % rank] = bool(torch.equal(both[0], both[1]))
        # the same step over peer memory: five steps, so both receive buffers are used and reused
        xchg = fd.connect_peer_exchange(fa.SplitKvPeerExchange(ctx, rank, world, Hq, D))
        out_peer = ctx.create_decode_output_buffer(fa.BF16, 1, Hq, D)
        peer_same = True
        for step in range(5):
            out_peer.zero_()
            ctx.splitkv_decode_peer(xchg, fa.BF16, 1, Hq, Hkv, D, ps, pool, pages, torch.from_numpy(tab).cuda(),
                                    torch.from_numpy(lens).cuda(), torch.from_numpy(qpos).cuda(), tab, lens, fa.config(True),
                                    theta, Q.cuda(), Kc.cuda(), Vc.cuda(), out_peer)
            ctx.synchronize()
            peer_same = peer_same and bool(torch.equal(out_peer, out))
        result["peer_same_%d" % rank] = peer_same
        result["peer_status_%d" % rank] = ctx.device_status()
        dist.barrier()  # nobody unmaps a buffer a peer may still store into
        xchg.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_splitkv_decode_over_nccl_two_ranks():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    result = mgr.dict()
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, result), nprocs=2, join=True)
    assert result["o"] <= 2e-2 and result["l"] <= 2e-3, dict(result)
    assert result["same_0"] and result["same_1"]
    assert result["peer_status_0"] == 0 and result["peer_status_1"] == 0, dict(result)
    assert result["peer_same_0"] and result["peer_same_1"], dict(result)
