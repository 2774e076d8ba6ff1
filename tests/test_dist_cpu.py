"""Multi-rank host logic on CPU ranks (gloo, world size 2): row sharding + output all-gather of
the M-sharded GEMM, and the expert-parallel dispatch / combine exchange, each against the
single-process computation.  The compute steps are injected reference callables — the CUDA
kernels cannot run here — so what is tested is the partition, count-exchange and reorder logic."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import restate as R
from pretrain_b200 import dist as D


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world, *args):
    port = _free_port()
    mp.spawn(_entry, args=(fn, world, port, args), nprocs=world, join=True)


def _entry(rank, fn, world, port, args):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def test_row_shard_covers_rows_in_tiles():
    for m in (8192, 1000, 130, 128, 5):
        for world in (1, 2, 4, 8):
            spans = [D.row_shard(m, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(s[0] % 128 == 0 or s[0] == m for s in spans)   # empty tail shards start at m
    with pytest.raises(ValueError):
        D.row_shard(10, 2, 2)


def _sharded_gemm_rank(rank, world, m):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(m, 64, generator=g)
    b = torch.randn(64, 48, generator=g)
    lo, hi = D.row_shard(m, world, rank)
    plain = lambda x, y, fa, fb, dt, rw: (x @ y).to(dt)
    out = D.sharded_gemm(a[lo:hi], b, "bf16", "bf16", torch.float32, m, gemm=plain)
    assert torch.equal(out, a @ b)
    local = D.sharded_gemm(a[lo:hi], b, "bf16", "bf16", torch.float32, m, gather=False, gemm=plain)
    assert local.shape[0] == hi - lo
    with pytest.raises(ValueError):
        D.all_gather_rows(torch.zeros(hi - lo + 1, 48), m)


@pytest.mark.parametrize("m", [512, 300])           # even shards; ragged shards (256 + 44 rows)
def test_m_sharded_gemm_all_gather(m):
    _run(_sharded_gemm_rank, 2, m)


def _ref_ffn(rows, expert_ids, w_in, w_down):
    out = torch.zeros(rows.shape[0], w_down.shape[1], dtype=rows.dtype)
    for e in range(w_in.shape[0]):
        sel = expert_ids == e
        if sel.any():
            h = (rows[sel].float() @ w_in[e].float().t()).to(rows.dtype)
            h = R.silu_glu(*h.chunk(2, dim=-1))
            out[sel] = (h.float() @ w_down[e].float().t()).to(rows.dtype)
    return out


def _ep_rank(rank, world, skew):
    g = torch.Generator().manual_seed(3)
    t, d, e, k, i = 96, 32, 8, 2, 16
    x = torch.randn(world * t, d, generator=g).bfloat16()
    logits = torch.randn(world * t, e, generator=g)
    if skew:
        logits[:, 4:] -= 1e9                         # every token goes to rank 0's experts; rank 1 receives nothing
        logits[:, 1] -= 1e9                          # and one of those experts stays empty
    w_in = (0.1 * torch.randn(e, 2 * i, d, generator=g)).bfloat16()
    w_down = (0.1 * torch.randn(e, d, i, generator=g)).bfloat16()
    top_i, top_w = R.router_topk(logits, k)
    lo, hi = rank * t, (rank + 1) * t
    el = e // world
    out = D.expert_parallel_moe(x[lo:hi], top_i[lo:hi], top_w[lo:hi], w_in[rank * el:(rank + 1) * el],
                                w_down[rank * el:(rank + 1) * el], e, ffn=_ref_ffn)
    # single-process reference on all tokens
    y = _ref_ffn(x.repeat_interleave(k, 0), top_i.reshape(-1), w_in, w_down)
    ref = (y.view(world * t, k, d).float() * top_w.view(world * t, k, 1).float()).sum(1).bfloat16()
    assert torch.equal(out, ref[lo:hi])


@pytest.mark.parametrize("skew", [False, True])
def test_expert_parallel_dispatch_combine(skew):
    _run(_ep_rank, 2, skew)


def _ep_index_rank(rank, world, skew):
    """The index tables of the fused expert-parallel path (the host restatement of b200q_moe_ep_index), with the count
    exchange done over gloo: together the ranks' rows must tile every owner's expert segments exactly - no row claimed
    twice, none left out, senders in rank order, each sender's rows in its own stable order."""
    g = torch.Generator().manual_seed(11)
    t, e, k = 200, 8, 2
    logits = torch.randn(world * t, e, generator=g)
    if skew:
        logits[:, 4:] -= 1e9
        logits[:, 1] -= 1e9
    top_i, _ = R.router_topk(logits, k)
    lo, hi, el = rank * t, (rank + 1) * t, e // world
    mine = top_i[lo:hi]
    offs, padded_offs, row_of = R.moe_padded_plan(mine, e)
    all_offs = [torch.empty_like(offs) for _ in range(world)]
    dist.all_gather(all_offs, offs)
    all_offs = torch.stack(all_offs)
    row_base, own_offs, pair_peer, pair_row = R.ep_index(all_offs, rank, mine, row_of, padded_offs)
    # gather everyone's claims: (owner, row, global expert, sender, position in the sender's stable order)
    pos = row_of.long() - padded_offs.long()[mine.reshape(-1)]
    claim = torch.stack([pair_peer.long(), pair_row.long(), mine.reshape(-1), torch.full_like(pos, rank), pos], 1)
    claims = [torch.empty_like(claim) for _ in range(world)]
    dist.all_gather(claims, claim)
    claims = torch.cat(claims)
    own_lists = [torch.empty_like(own_offs) for _ in range(world)]
    dist.all_gather(own_lists, own_offs)
    for owner in range(world):
        c = claims[claims[:, 0] == owner]
        assert (c[:, 2] // el == owner).all()
        assert c[:, 1].unique().numel() == c.shape[0]                           # no row claimed twice
        ends = own_lists[owner].long()
        counts = torch.diff(ends, prepend=ends.new_zeros(1))
        start = 0
        for j in range(el):
            seg = c[c[:, 2] == owner * el + j]
            assert seg.shape[0] == counts[j]                                       # every pair of the expert has a row
            if seg.shape[0]:
                seg = seg[seg[:, 1].argsort()]
                assert torch.equal(seg[:, 1], start + torch.arange(seg.shape[0]))  # contiguous from the 128-aligned segment start
                key = seg[:, 3] * (2 * world * t) + seg[:, 4]
                assert (key[1:] > key[:-1]).all()                                  # rank order, then each sender's stable order
            start += (int(counts[j]) + 127) // 128 * 128


@pytest.mark.parametrize("skew", [False, True])
def test_expert_parallel_index_tables_tile_the_owners_buffers(skew):
    _run(_ep_index_rank, 2, skew)
