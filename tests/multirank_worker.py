"""Worker of the multi-GPU parity test: one process per GPU (torchrun), NCCL
for rendezvous only.  Every rank regenerates all ranks' seeded inputs, runs the
collective layer call on its own tokens, and compares what it holds afterwards
-- dispatch data products of its local experts and its y -- with the CPU oracle
of the whole world.  Prints one JSON line per rank; exit code 0 iff all pass."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import numpy as np
import torch
import torch.distributed as dist

import gc_moe_b200 as G
from gc_moe_b200 import quant
from gc_moe_b200.layout import round_up, sf_row_in_block
from oracle import gcmoe_oracle as O

COSINE_MIN, MAX_REL_ERR = 0.9999, 2.0 ** -6


def main():
    rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
    torch.cuda.set_device(int(os.environ.get('LOCAL_RANK', rank)))
    dev = torch.device('cuda', torch.cuda.current_device())
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    dist.init_process_group('nccl', device_id=dev)
    group = dist.group.WORLD
    host_group = dist.new_group(backend='gloo')     # host-side decisions (who failed) never touch the GPUs

    def anyone_failed():
        """Every rank learns whether ANY rank has recorded a failure, so that all of them
        skip the remaining collective calls together instead of leaving peers to wait
        for a rank that has gone."""
        flag = torch.tensor([1 if failures else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=host_group)
        return bool(flag.item())
    E, H, I, K, CAP = 8 * world, 1024, 512, 4, 1920
    EL = E // world

    g = torch.Generator(device=dev).manual_seed(5)
    packs = []
    for rows, k in ((2 * I, H), (H, I)):
        w = torch.randn((E, rows, k), device=dev, generator=g) * 0.02
        packs.append(quant.quantize_weights_fp4(w))
    (q1, c1), (q2, c2) = packs
    mine = slice(rank * EL, (rank + 1) * EL)
    l1, l2 = G.transform_weights_for_gc_moe(
        (q1[mine].contiguous(), quant.weight_scales_mn_major(c1[mine].contiguous())),
        (q2[mine].contiguous(), quant.weight_scales_mn_major(c2[mine].contiguous())))
    cpu_w = [t.cpu() for t in (q1, c1, q2, c2)]
    buf = G.get_symm_buffer_for_gc_moe(group, E, CAP, K, H, I)
    stats = torch.zeros(EL, dtype=torch.int32, device=dev)
    failures, report = [], {}

    def inputs_of(case, r):
        tokens = case['tokens'][r]
        xq, xsf, idx, w = O.make_tokens(tokens, H, E, K, seed=case['seed'] * 100 + r)
        if case.get('invalid') and tokens:
            idx[::3, 0] = -1
            idx[1::4, 1] = E + 2
        if case.get('hot') is not None and tokens:
            idx[:, 0] = case['hot']
            idx[:, 1] = (case['hot'] + 1) % E
        if case.get('to_rank0') and tokens:
            idx = idx % EL             # every route goes to an expert of rank 0
            idx[:, 1:] = (idx[:, :1] + torch.arange(1, K)) % EL   # k distinct experts per token
        return xq, xsf, idx, w

    def stage(inp):
        xq, xsf, idx, w = inp
        t = xq.shape[0]
        buf.x[:t].copy_(xq.to(dev)); buf.x_sf[:t].copy_(xsf.to(dev))
        buf.topk_idx[:t].copy_(idx.to(dev)); buf.topk_weights[:t].copy_(w.to(dev))

    def check(name, cond):
        if not cond:
            failures.append(name)

    cases = [
        {'name': 'uniform', 'tokens': [24] * world, 'seed': 1},
        {'name': 'asymmetric', 'tokens': [(37 * (r + 1)) % 90 for r in range(world)], 'seed': 2},
        {'name': 'one_idle', 'tokens': [0 if r == 0 else 16 for r in range(world)], 'seed': 3},
        {'name': 'invalid_routes', 'tokens': [20] * world, 'seed': 4, 'invalid': True},
        {'name': 'hot_expert', 'tokens': [150] * world, 'seed': 5, 'hot': 1},
        {'name': 'single_token', 'tokens': [1] * world, 'seed': 6},
        # the reference's asymmetric vectors (scripts/run.sh:313-391): nobody, one rank only,
        # a ramp, ranks in different tile regimes (block-M 16 next to 96)
        {'name': 'all_idle', 'tokens': [0] * world, 'seed': 7},
        {'name': 'one_active', 'tokens': [33 if r == world - 1 else 0 for r in range(world)], 'seed': 8},
        {'name': 'ramp', 'tokens': [5 + 40 * r for r in range(world)], 'seed': 9},
        {'name': 'mixed_regimes', 'tokens': [400 if r % 2 else 3 for r in range(world)], 'seed': 10},
        # one rank enters the call late, with no barrier in front: its peers' GEMM launches
        # (and their down tiles) run while its rows are still on their way
        {'name': 'late_rank', 'tokens': [48] * world, 'seed': 11, 'late': world - 1, 'hot': 2},
        {'name': 'late_rank_decode', 'tokens': [2] * world, 'seed': 12, 'late': 0},
    ]
    # every block-M switch of this geometry, one token either side (scripts/run.sh:292-311)
    switches = [t for t in range(1, 700)
                if G.get_block_m_for_gc_moe(world, E, CAP, t, K) != G.get_block_m_for_gc_moe(world, E, CAP, t - 1, K)]
    for t in switches[:6]:
        cases.append({'name': f'boundary_{t - 1}', 'tokens': [t - 1] * world, 'seed': 100 + t})
        cases.append({'name': f'boundary_{t}', 'tokens': [t] * world, 'seed': 200 + t})
    expected_stats = np.zeros(EL, np.int64)
    for case in cases:
        all_inputs = [inputs_of(case, r) for r in range(world)]
        bms = [G.get_block_m_for_gc_moe(world, E, CAP, case['tokens'][r], K) for r in range(world)]
        ref = O.moe_layer([a[0] for a in all_inputs], [a[1] for a in all_inputs],
                          [a[2] for a in all_inputs], [a[3] for a in all_inputs], *cpu_w, bms, clamp=10.0)
        t = case['tokens'][rank]
        stage(all_inputs[rank])
        y = torch.full((t, H), float('nan'), dtype=torch.bfloat16, device=dev)
        gen = int(buf.region('recv_parity').view(torch.int32)[0].item()) & 1
        dist.barrier()
        if case.get('late') == rank:
            import time
            time.sleep(0.05)           # host-side skew only: the GPUs keep running
        G.fp8_fp4_gc_moe(y, l1, l2, buf, cumulative_local_expert_recv_stats=stats, activation_clamp=10.0)
        torch.cuda.synchronize()
        try:
            buf.raise_on_device_error()
        except RuntimeError as exc:
            failures.append(f"{case['name']}: {exc}")
        if anyone_failed():
            break
        dist.barrier()
        d, bm = ref.dispatch[rank], bms[rank]
        expected_stats += d.counts.sum(0)
        counts = buf.region('expert_recv_count').view(torch.int64)[gen * world * EL:(gen + 1) * world * EL]
        check(case['name'] + ':counts', np.array_equal(counts.cpu().numpy().reshape(world, EL), d.counts))
        check(case['name'] + ':pool_blocks', int(buf.region('routed_pool_blocks').view(torch.int32)[0]) == d.pool_blocks)
        rows = d.pool_blocks * bm
        valid = np.nonzero(d.metadata[:, 0] >= 0)[0]
        meta = buf.region('token_src_metadata').view(torch.int32).reshape(-1, 3)[:rows].cpu().numpy()
        check(case['name'] + ':metadata', np.array_equal(meta[valid], d.metadata[valid]))
        acts = buf.l1_acts.view(torch.uint8)[:rows].cpu().numpy()
        check(case['name'] + ':rows', np.array_equal(acts[valid], d.rows[valid]))
        wts = buf.buffer.narrow(0, buf.layout.views['l1_topk_weights'].offset, rows * 4).view(torch.float32).cpu().numpy()
        check(case['name'] + ':weights', np.array_equal(wts[valid], d.weights[valid]))
        sf = buf.l1_acts_sf[:d.pool_blocks * round_up(bm, 128)].cpu().numpy()
        sf_rows = np.array([(r // bm) * round_up(bm, 128) + sf_row_in_block(r % bm) for r in valid], dtype=np.int64)
        check(case['name'] + ':scales', np.array_equal(sf[sf_rows], d.sf_words[valid]) if len(valid) else True)
        table = buf.region('src_token_topk_idx').view(torch.int32).reshape(E, CAP)[:EL * world].cpu().numpy().reshape(EL, world, CAP)
        check(case['name'] + ':index_table', all(np.array_equal(table[l, s, :len(v)].astype(np.uint32), v)
                                                 for (l, s), v in d.index_lists.items()))
        yc = y.cpu()
        if t:
            cos, err = O.cosine(yc, ref.y[rank]), O.max_rel_err(yc, ref.y[rank])
            report[case['name']] = [round(cos, 9), err]
            check(case['name'] + ':y', bool(torch.isfinite(yc.float()).all()) and cos >= COSINE_MIN and err <= MAX_REL_ERR)
    if not anyone_failed():
        check('stats', np.array_equal(stats.cpu().numpy(), expected_stats))

    # Graph capture + alternating replays at fixed addresses, all routed work of every
    # rank sent to rank 0's experts (the reference's readiness protocol,
    # tests/test_gc_moe_readiness.py:97-99,148,165-178): y is pre-filled with NaN and
    # each replay must reproduce its own eager result, not the other input's.
    if not anyone_failed():
        a = {'tokens': [12] * world, 'seed': 21, 'to_rank0': True}
        b = {'tokens': [12] * world, 'seed': 22, 'to_rank0': True}
        y = torch.empty((12, H), dtype=torch.bfloat16, device=dev)
        eager = []
        for case in (a, b):
            stage(inputs_of(case, rank)); dist.barrier()
            G.fp8_fp4_gc_moe(y, l1, l2, buf, activation_clamp=10.0)
            torch.cuda.synchronize(); dist.barrier()
            eager.append(y.cpu().clone())
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                G.fp8_fp4_gc_moe(y, l1, l2, buf, activation_clamp=10.0)
        torch.cuda.current_stream().wait_stream(side)
        assert not torch.equal(eager[0], eager[1])
        for it in range(40):
            stage(inputs_of((a, b)[it & 1], rank))
            y.fill_(float('nan'))
            torch.cuda.synchronize(); dist.barrier()
            graph.replay()
            torch.cuda.synchronize()
            check(f'replay{it}', torch.equal(y.cpu().view(torch.int16), eager[it & 1].view(torch.int16)))
        try:
            buf.raise_on_device_error()
        except RuntimeError as exc:
            failures.append(f'replay: {exc}')
        dist.barrier()
    # Fused shared expert together with expert parallelism: every rank applies the
    # (replicated) shared expert to its own tokens while its routes go to their owners.
    if not anyone_failed():
        sbuf = G.get_symm_buffer_for_gc_moe(group, E, CAP, K, H, I, 1)
        gs = torch.Generator().manual_seed(11)
        sw1, sc1 = O.quantize_block_fp8(torch.randn((2 * I, H), generator=gs) * 0.02)
        sw2, sc2 = O.quantize_block_fp8(torch.randn((H, I), generator=gs) * 0.02)
        shared = {'w1': sw1, 'w1_codes': sc1, 'w2': sw2, 'w2_codes': sc2}
        sl1, sl2 = G.transform_weights_for_gc_moe(
            (sw1.to(dev), O.expand_block_sf_rows(sc1, 2 * I).to(dev)),
            (sw2.to(dev), O.expand_block_sf_rows(sc2, H).to(dev)))
        case = {'tokens': [(11 * (r + 2)) % 50 for r in range(world)], 'seed': 31}
        all_inputs = [inputs_of(case, r) for r in range(world)]
        bms = [G.get_block_m_for_gc_moe(world, E, CAP, case['tokens'][r], K) for r in range(world)]
        ref = O.moe_layer([a[0] for a in all_inputs], [a[1] for a in all_inputs], [a[2] for a in all_inputs],
                          [a[3] for a in all_inputs], *cpu_w, bms, clamp=10.0, shared=shared)
        t = case['tokens'][rank]
        xq, xsf, idx, w = all_inputs[rank]
        sbuf.x[:t].copy_(xq.to(dev)); sbuf.x_sf[:t].copy_(xsf.to(dev))
        sbuf.topk_idx[:t].copy_(idx.to(dev)); sbuf.topk_weights[:t].copy_(w.to(dev))
        tt = torch.arange(t)
        u = tt % bms[rank]
        rows = (tt // bms[rank]) * ((bms[rank] + 127) // 128 * 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32
        if t:
            sbuf.shared_l1_acts_sf[rows.to(dev)] = xsf.to(dev)
        y = torch.full((t, H), float('nan'), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize(); dist.barrier()
        G.fp8_fp4_gc_moe(y, l1, l2, sbuf, sl1, sl2, activation_clamp=10.0, shared_recipe=(1, 128, 128))
        torch.cuda.synchronize()
        try:
            sbuf.raise_on_device_error()
            if t:
                cos, err = O.cosine(y.cpu(), ref.y[rank]), O.max_rel_err(y.cpu(), ref.y[rank])
                report['shared_expert'] = [round(cos, 9), err]
                check('shared_expert:y', cos >= COSINE_MIN and err <= MAX_REL_ERR)
        except RuntimeError as exc:
            failures.append(f'shared_expert: {exc}')
        dist.barrier()
        sbuf.destroy()
    print(json.dumps({'rank': rank, 'world': world, 'failures': failures, 'y': report}), flush=True)
    buf.destroy()
    dist.destroy_process_group()
    sys.exit(1 if failures else 0)


if __name__ == '__main__':
    main()
