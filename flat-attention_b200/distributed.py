"""Multi-GPU plumbing of the attention path: one process per GPU, torch.distributed for the exchange.

The path shards without communication: every (batch, kv_head) unit — with its q_heads/kv_heads query
heads — is independent in forward, decode and backward (src/grouped.rs:101-108,
src/backward_grouped.rs:45-52), so ranks take contiguous blocks of units (`shard_units`), or whole
sequences for paged decode.  The one exchange is single-sequence long-context decode: the KV axis is cut
into one contiguous page range per rank (`shard_pages`), every rank computes the normalised partial
(O_i, LSE_i) of its slice, the partials are all-gathered (NCCL on GPUs, gloo in CPU tests) and merged
locally:  LSE = log sum_i exp(LSE_i),  O = sum_i exp(LSE_i - LSE) O_i.  The reference has no multi-device
code; this module has no counterpart there.
"""
from __future__ import annotations


def shard_units(n_units: int, world: int, rank: int) -> range:
    """Contiguous block of independent units for this rank; blocks differ by at most one unit."""
    base, extra = divmod(n_units, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def shard_pages(live_tokens: int, page_size: int, world: int, rank: int):
    """(first_token, token_count) of this rank's slice of one sequence, cut on page boundaries."""
    pages = (live_tokens + page_size - 1) // page_size
    r = shard_units(pages, world, rank)
    first = r.start * page_size
    last = min(live_tokens, r.stop * page_size)
    return first, max(0, last - first)


def merge_partials_reference(partial_o, partial_lse):
    """The merge formula on torch tensors ([parts, rows, D], [parts, rows]); used by CPU tests of the
    exchange (the product merge is the CUDA kernel behind flat_splitkv_merge_packed)."""
    import torch
    total = torch.logsumexp(partial_lse.double(), dim=0)
    w = torch.exp(partial_lse.double() - total)
    w = torch.where(torch.isfinite(partial_lse.double()), w, torch.zeros_like(w))
    return (w[:, :, None] * partial_o.double()).sum(0).float(), total.float()


def all_gather_partials(packed_partial, group=None):
    """All-gathers one packed [O(rows*D) | LSE(rows)] f32 block per rank into [world, rows*(D+1)]."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    flat = packed_partial.contiguous().reshape(-1)
    out = torch.empty(world * flat.numel(), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.view(world, flat.numel())


def splitkv_decode(ctx, fa, dtype, slice_args: dict, rows: int, head_dim: int, out, group=None):
    """One KV-split decode step: local partial on this rank's cache slice, all-gather, local merge.

    slice_args are the keyword arguments of Context.decode_paged_batched_partial except `out`.  Ranks
    whose slice is empty contribute LSE = -inf (weight 0).  Returns the gathered buffer (for inspection).
    """
    import torch
    import torch.distributed as dist
    partial = torch.empty(rows * (head_dim + 1), dtype=torch.float32, device=out.device)
    if slice_args is None:
        partial[:rows * head_dim] = 0
        partial[rows * head_dim:] = float("-inf")
    else:
        ctx.decode_paged_batched_partial(dtype, out=partial, **slice_args)
    gathered = all_gather_partials(partial, group)
    ctx.splitkv_merge_packed(dtype, dist.get_world_size(group), rows, head_dim, gathered, out)
    return gathered


def nccl_comm_ptr(group=None, device=None) -> int:
    """The ncclComm_t behind a torch.distributed NCCL process group, as an integer for the C ABI
    (flat_splitkv_decode_nccl).  The communicator exists once the group has run a collective on the device."""
    import torch
    import torch.distributed as dist
    pg = group if group is not None else dist.distributed_c10d._get_default_group()
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    backend = pg._get_backend(dev)
    if not hasattr(backend, "_comm_ptr"):
        raise RuntimeError("this torch build does not expose the NCCL communicator of a process group")
    return int(backend._comm_ptr())


def connect_peer_exchange(exchange, group=None):
    """Hands every rank's IPC handle of a `SplitKvPeerExchange` to every other rank (one all-gather of 64 bytes per
    rank through torch.distributed, any backend) and maps them: after this the exchange can run
    `Context.splitkv_decode_peer`.  Every rank of the group must make the call; when a rank cannot map a peer, every
    rank raises (nobody is left waiting in a collective)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    handles = [None] * world
    dist.all_gather_object(handles, exchange.handle(), group=group)
    error = None
    try:
        exchange.connect(b"".join(handles))
    except Exception as e:  # reported after the ranks have agreed on the outcome
        error = e
    device = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    ok = torch.tensor([0 if error else 1], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)  # also: every rank has mapped every buffer before any store
    if int(ok.item()) == 0:
        raise RuntimeError("peer exchange could not be connected on every rank: %r" % (error,))
    return exchange
