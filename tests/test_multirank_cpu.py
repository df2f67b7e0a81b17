"""The push-dispatch protocol on two CPU processes (gloo): each rank exchanges
only its per-expert counts and block-M with the other, computes the
destination row of each of its routes on its own, and the union of the plans
must be exactly the pool the world oracle lays out."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gc_moe_b200.heuristics import get_block_m_for_gc_moe
from oracle import gcmoe_oracle as O

E, H, K, CAP = 16, 256, 4, 1920


def _inputs(rank, tokens):
    xq, xsf, idx, w = O.make_tokens(tokens, H, E, K, seed=300 + rank)
    if tokens > 3:
        idx[2, 1] = -1
    return xq, xsf, idx, w


def _worker(rank, world, port, token_counts, result):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        xq, xsf, idx, w = _inputs(rank, token_counts[rank])
        own = np.bincount(idx.numpy().reshape(-1)[(idx.numpy().reshape(-1) >= 0) & (idx.numpy().reshape(-1) < E)],
                          minlength=E)
        # the all-to-all of counts and block-M: the only thing the ranks exchange before pushing rows
        mine = torch.tensor(list(own) + [get_block_m_for_gc_moe(world, E, CAP, token_counts[rank], K)])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        matrix = np.stack([g.numpy()[:E] for g in gathered])
        block_m_of = [int(g[E]) for g in gathered]
        plan = O.push_plan(rank, idx, matrix, block_m_of, E)
        # collect every rank's plan on every rank and compare with the world oracle
        plans = [None] * world
        dist.all_gather_object(plans, plan)
        everyone = [_inputs(r, token_counts[r]) for r in range(world)]
        d = O.dispatch([a[2].numpy() for a in everyone], [a[3].numpy() for a in everyone],
                       [a[0].view(torch.uint8).numpy() for a in everyone], [a[1].numpy() for a in everyone],
                       E, block_m_of)
        ok = True
        for r in range(world):
            seen = np.full((d[r].metadata.shape[0], 3), -1, np.int64)
            for s, pl in enumerate(plans):
                for owner, l, row, pos, token, slot in pl:
                    if owner != r:
                        continue
                    ok &= bool((seen[row] == -1).all())            # no two routes share a row
                    seen[row] = (s, token, slot)
                    ok &= int(d[r].index_lists[(l, s)][pos]) == token * K + slot
            ok &= bool(np.array_equal(seen, d[r].metadata))
            ok &= bool(np.array_equal(matrix[:, r * (E // world):(r + 1) * (E // world)], d[r].counts))
        result[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('token_counts', [(9, 14), (0, 7), (40, 40)])
def test_push_dispatch_protocol_two_ranks(token_counts):
    ctx = mp.get_context('spawn')
    result = ctx.Manager().dict()
    port = 29800 + sum(token_counts) % 50
    procs = [ctx.Process(target=_worker, args=(r, 2, port, token_counts, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert dict(result) == {0: True, 1: True}
