"""world_size-2 gloo run of the vocabulary-sharded head's host logic on CPU: each rank
forms the per-row partials of its shard (here with the oracle standing in for the
kernel), one all-reduce sums them, and the telemetry equals the unsharded head."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from algebraic_transformer_b200.dist import init_from_env, vocab_shard
    from oracle import algebraic_ref as R
    r, w, _ = init_from_env(backend="gloo")
    assert (r, w) == (rank, world)
    g = torch.Generator().manual_seed(11)
    N, d, V = 96, 64, 1000                                # 8 tiles of 128 -> 4/4, ragged last tile
    h = torch.randn((N, d), generator=g).bfloat16()
    E = torch.randn((V, d), generator=g) * 0.1
    t = torch.randint(0, V, (N,), generator=g)
    lo, cnt = vocab_shard(V, rank, world)
    l, zt = R.fused_head_stats(h, E, t, 8, 2.0, vocab_lo=lo, vocab_hi=lo + cnt, vocab_total=V)
    stats = torch.stack([l, zt])
    dist.all_reduce(stats, op=dist.ReduceOp.SUM)
    pt, obj = R.fused_head_telemetry(stats[0], stats[1], 8, 2.0, R.likelihood_clamp(V, 8))
    obj0, pt0 = R.head_loss_dense(h, E, t, 8, 2.0)
    ok = torch.allclose(pt, pt0, rtol=2e-5, atol=1e-9) and abs(float(obj) - float(obj0)) < 1e-5
    # the "ce" kind: per-shard logsumexp and target logit, combined by the product's own host routine
    # (a MAX and a SUM all-reduce), against the unsharded cross-entropy; one shard holds a logit of 3e4
    from algebraic_transformer_b200.ops import combine_ce_statistics
    E2 = E.clone()
    E2[700] = 40.0 * torch.sign(h[5].float())               # z[5, 700] ~ 40 * sum |h_5| >> 88
    z = R.head_logits(h, E2)
    zs = z[:, lo:lo + cnt]
    in_shard = (t >= lo) & (t < lo + cnt)
    zt_s = torch.where(in_shard, zs.gather(-1, (t - lo).clamp(0, cnt - 1)[:, None])[:, 0], torch.zeros(N))
    ce_stats = torch.stack([torch.logsumexp(zs, dim=-1), zt_s])
    combine_ce_statistics(ce_stats, dist.group.WORLD)
    obj_ce, nll_ce = R.cross_entropy(z, t)
    ok = ok and torch.allclose(ce_stats[0] - ce_stats[1], nll_ce, rtol=1e-5, atol=1e-4) and float(z.max()) > 1000.0
    ret[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_vocab_sharded_head_on_gloo():
    world = 2
    port = 29600 + os.getpid() % 200
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}
