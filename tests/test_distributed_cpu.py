"""Host-side multi-rank logic on CPU (gloo, world_size 2): unit / page sharding and the
all-gather + merge of split-KV partials.  No GPU and no product kernel is involved; the merge here is
the reference formula (the CUDA merge is covered by the gpu tests)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "flat-attention_b200"))
import distributed as fd  # noqa: E402


def test_shard_units_cover_everything_once():
    for n in (1, 7, 16, 32, 33):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                seen += list(fd.shard_units(n, world, r))
            assert seen == list(range(n))
            sizes = [len(fd.shard_units(n, world, r)) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_shard_pages_are_contiguous_and_page_aligned():
    for live, ps, world in ((131072, 16, 8), (1000, 16, 3), (5, 16, 4), (4097, 16, 2)):
        at = 0
        for r in range(world):
            first, count = fd.shard_pages(live, ps, world, r)
            if count:
                assert first == at and first % ps == 0
                at += count
        assert at == live


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, D, n = 6, 16, 101
        g = torch.Generator().manual_seed(0)
        scores = torch.randn(rows, n, generator=g) * 2
        v = torch.randn(n, D, generator=g)
        first, count = fd.shard_pages(n, 16, world, rank)
        s_loc, v_loc = scores[:, first:first + count], v[first:first + count]
        lse = torch.logsumexp(s_loc, dim=1)
        o = torch.softmax(s_loc, dim=1) @ v_loc
        packed = torch.cat([o.reshape(-1), lse])
        gathered = fd.all_gather_partials(packed)
        po = gathered[:, :rows * D].reshape(world, rows, D)
        pl = gathered[:, rows * D:]
        mo, ml = fd.merge_partials_reference(po, pl)
        eo, el = torch.softmax(scores, dim=1) @ v, torch.logsumexp(scores, dim=1)
        q.put((rank, float((mo - eo).abs().max()), float((ml - el).abs().max())))
    finally:
        dist.destroy_process_group()


def test_gather_and_merge_of_partials_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = [q.get(timeout=5) for _ in range(2)]
    assert sorted(r[0] for r in results) == [0, 1]
    for _, eo, el in results:
        assert eo < 1e-5 and el < 1e-5


def test_empty_slice_has_zero_weight():
    po = torch.randn(3, 4, 8)
    pl = torch.tensor([[0.5, 1.0, -2.0, 0.0], [float("-inf")] * 4, [1.5, 0.0, 0.3, -1.0]])
    mo, ml = fd.merge_partials_reference(po, pl)
    eo, el = fd.merge_partials_reference(po[[0, 2]], pl[[0, 2]])
    assert torch.allclose(mo, eo) and torch.allclose(ml, el)
