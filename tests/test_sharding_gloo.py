"""The multi-GPU path on the CPU: two gloo ranks shard a sparse and a dense decode problem by batch (each with its
own renumbered page pool) and a prefill problem by query token, run the oracle on their shard, and the
gathered result must equal the unsharded one bit for bit.  Also checks the max-over-ranks timing reduction
the benchmark uses."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashmla_b200 import sharding, workloads as wl
from oracle import attention, quant


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    w = wl.make_decode_workload(5, 2, 8, 64, 100, 400, seed=3, invalid_frac=0.05, with_sink=True)
    q, kv, idx, (lo, hi) = sharding.shard_decode_inputs(w.q, w.kv_rows, w.indices, world, rank)
    assert kv.shape[0] <= w.kv_rows.shape[0]
    out, lse, _ = attention.sparse_decode(q, quant.dequantize_rows(kv), idx, w.sm_scale, attn_sink=w.attn_sink)
    gathered = [None] * world
    dist.all_gather_object(gathered, (lo, hi, out, lse.contiguous()))
    p = wl.make_prefill_workload(7, 120, 4, 64, seed=4)
    pq, pidx, (plo, phi) = sharding.shard_prefill_inputs(p.q, p.indices, world, rank)
    pout = attention.sparse_prefill_fwd(pq, p.kv, pidx, p.sm_scale)[0]
    pg = [None] * world
    dist.all_gather_object(pg, (plo, phi, pout))
    dq, dk, dbt, dlens = _dense_problem()
    sq, sk, sbt, slens, (dlo, dhi) = sharding.shard_dense_decode_inputs(dq, dk, dbt, dlens, world, rank)
    assert sk.shape[0] < dk.shape[0]
    dout, dlse = attention.dense_decode(sq, sk, sbt, slens, 512, True)
    dg = [None] * world
    dist.all_gather_object(dg, (dlo, dhi, dout, dlse.contiguous()))
    t = torch.tensor([1.0 + rank], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        torch.save({"decode": gathered, "prefill": pg, "dense": dg, "tmax": float(t)}, os.path.join(out_dir, "r.pt"))
    dist.barrier()
    dist.destroy_process_group()


def _dense_problem():
    g = torch.Generator().manual_seed(11)
    b, s_q, h_q, page, max_blocks = 5, 2, 8, 64, 6
    lens = torch.tensor([300, 0, 64, 381, 130], dtype=torch.int32)
    block_table = torch.randperm(b * max_blocks, generator=g).to(torch.int32).view(b, max_blocks)
    q = torch.randn((b, s_q, h_q, 576), generator=g).to(torch.bfloat16)
    k = (torch.randn((b * max_blocks, page, 1, 576), generator=g) / 10).to(torch.bfloat16)
    return q, k, block_table, lens


def test_two_rank_sharding_reproduces_unsharded_results(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = torch.load(os.path.join(tmp_path, "r.pt"), weights_only=False)
    assert r["tmax"] == 2.0
    w = wl.make_decode_workload(5, 2, 8, 64, 100, 400, seed=3, invalid_frac=0.05, with_sink=True)
    ref_out, ref_lse, _ = attention.sparse_decode(w.q, quant.dequantize_rows(w.kv_rows), w.indices, w.sm_scale, attn_sink=w.attn_sink)
    parts = sorted(r["decode"], key=lambda x: x[0])
    assert [(a, b) for a, b, _, _ in parts] == [(0, 3), (3, 5)]
    assert torch.equal(torch.cat([x[2] for x in parts]), ref_out)
    assert torch.equal(torch.cat([x[3] for x in parts]), ref_lse.contiguous())
    p = wl.make_prefill_workload(7, 120, 4, 64, seed=4)
    pref = attention.sparse_prefill_fwd(p.q, p.kv, p.indices, p.sm_scale)[0]
    pp = sorted(r["prefill"], key=lambda x: x[0])
    assert torch.equal(torch.cat([x[2] for x in pp]), pref)
    dq, dk, dbt, dlens = _dense_problem()
    dref_out, dref_lse = attention.dense_decode(dq, dk, dbt, dlens, 512, True)
    dd = sorted(r["dense"], key=lambda x: x[0])
    assert torch.equal(torch.cat([x[2] for x in dd]), dref_out)
    assert torch.equal(torch.cat([x[3] for x in dd]), dref_lse.contiguous())


@pytest.mark.parametrize("n,world", [(128, 8), (7, 2), (3, 4), (0, 2)])
def test_shard_bounds_cover(n, world):
    spans = [sharding.shard_bounds(n, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == n
    assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    sizes = [hi - lo for lo, hi in spans]
    assert max(sizes) - min(sizes) <= 1


def test_dense_shard_of_empty_requests_and_more_ranks_than_requests():
    q, k, bt, lens = _dense_problem()
    zero = torch.zeros_like(lens)
    sq, sk, sbt, slens, (lo, hi) = sharding.shard_dense_decode_inputs(q, k, bt, zero, 2, 0)
    assert (lo, hi) == (0, 3) and sk.shape[0] == 1 and int(sbt.abs().sum()) == 0          # no page reached: one stand-in block
    out, lse = attention.dense_decode(sq, sk, sbt, slens, 512, False)
    assert float(out.float().abs().sum()) == 0.0 and bool(torch.isinf(lse).all())
    spans = []
    for r in range(8):                                                                     # 8 ranks, 5 requests
        sq, sk, sbt, slens, (lo, hi) = sharding.shard_dense_decode_inputs(q, k, bt, lens, 8, r)
        spans.append((lo, hi))
        assert sq.shape[0] == hi - lo == sbt.shape[0] == slens.shape[0]
        if hi > lo:
            ref = attention.dense_decode(q[lo:hi], k, bt[lo:hi], lens[lo:hi], 512, True)
            got = attention.dense_decode(sq, sk, sbt, slens, 512, True)
            assert torch.equal(ref[0], got[0]) and torch.equal(ref[1], got[1])
    assert spans[0][0] == 0 and spans[-1][1] == 5 and sum(hi - lo for lo, hi in spans) == 5
