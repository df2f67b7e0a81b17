"""Benchmark of the MoE layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Metric: MoE layer latency in microseconds under CUDA-graph replay, max over
ranks.  One step = one layer call (graph replay) at each token count of the
workload's sweep; `value` is the mean latency of a layer call over the sweep.

* 1 GPU: the single-GPU configuration of the benchmark spec -- hidden 4096, 64
  routed experts, top-8, intermediate 2048, tokens in {1, 8, 32, 128, 256},
  uniform random routing.
* N > 1 GPUs: the expert-parallel decode configuration -- hidden 7168, 256
  routed experts sharded evenly over the N ranks, top-8, intermediate 2048,
  tokens per rank in {1, 2, 4, ..., 256}, router logits N(0,1) plus a
  Zipf(1.1) per-expert bias; dispatch and combine run over NVLink peer stores
  inside the layer's kernels (no NCCL on the data path).

FP8 e4m3 activations and FP4 e2m1 weights with UE8M0 scales per 32 elements of
K; all inputs are seeded synthetic tensors of those shapes and distributions.

`--impl reference` times the reference operator's own CPU path for this layer
(its PyTorch dequantise-and-matmul forward, restated in oracle/gcmoe_oracle.py)
on the host cores of rank 0, on a bounded sample of each call.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = 'MoE layer latency us (graph replay, max over ranks) @1-256 tok/rank'
L2_FLUSH_BYTES = 512 << 20    # > 126 MB of L2
ROOFLINE_TOKENS = 32          # every local expert is hit: the weight-streaming regime
INPUT_SETS = 2                # alternating token sets per token count


class Workload:
    def __init__(self, world: int, only_tokens: int = 0):
        self.world = world
        if world == 1:
            self.name = 'single-GPU config: H4096 E64 top8 I2048, tokens {1,8,32,128,256}, uniform routing'
            self.hidden, self.experts, self.topk, self.inter = 4096, 64, 8, 2048
            self.sweep = (1, 8, 32, 128, 256)
            self.zipf = None
            self.cpu_fraction = 8
        else:
            self.name = (f'expert-parallel decode config on {world} GPUs: H7168 E256 ({256 // world}/rank) top8 I2048, '
                         'tokens/rank {1,2,4,8,16,32,64,128,256}, router logits N(0,1) + Zipf(1.1) expert bias')
            self.hidden, self.experts, self.topk, self.inter = 7168, 256, 8, 2048
            self.sweep = (1, 2, 4, 8, 16, 32, 64, 128, 256)
            self.zipf = 1.1
            self.cpu_fraction = 32
        if only_tokens:
            self.sweep = (only_tokens,)
        self.capacity = 256
        self.local_experts = self.experts // world

    def expert_bytes(self) -> int:
        """FP4 payload + UE8M0/32 scales of one expert's W1 and W2: the weight
        working-set model of the reference's benchmark (benchmark_gc_moe.py:248-309)."""
        return 3 * self.inter * self.hidden * 17 // 32

    def expert_bias(self, device):
        """log p_e with p_e ~ 1 / rank_e^1.1 over a fixed seeded permutation."""
        if self.zipf is None:
            return None
        perm = torch.randperm(self.experts, generator=torch.Generator().manual_seed(99)).float() + 1
        return torch.log(perm.pow(-self.zipf) / perm.pow(-self.zipf).sum()).to(device)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while timing runs."""

    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int):
        self.index, self.samples, self.proc, self.first_timed = index, [], None, 0

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--id={self.index}', f'--query-gpu={self.FIELDS}',
                 '--format=csv,noheader,nounits', '-lms', '20'],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(',')]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def wait_first(self, seconds: float) -> None:
        """nvidia-smi needs a second or more to start on an 8-GPU box: do not begin
        the timed region before it delivers samples."""
        deadline = time.time() + seconds
        while self.proc is not None and not self.samples and time.time() < deadline:
            time.sleep(0.05)

    def mark_timed(self) -> None:
        self.first_timed = len(self.samples)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.1)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['unavailable']}
        timed = self.samples[self.first_timed:] or self.samples     # samples during warm-up + timed region
        clocks = sorted(int(s[0]) for s in timed)
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == 'Active' for s in self.samples)]
        return {'sm_mhz': clocks[len(clocks) // 2], 'sm_max_mhz': int(self.samples[0][1]),
                'reasons': reasons, 'samples': len(clocks)}


def make_inputs(wl: Workload, device, rank: int):
    """Seeded synthetic weights N(0, 0.02) -> FP4 for this rank's experts; per
    token count INPUT_SETS token sets N(0,1) -> FP8 with router logits N(0,1)
    (+ expert bias), top-k and softmax over the selected k."""
    from gc_moe_b200 import quant
    g = torch.Generator(device=device).manual_seed(1234 + 7919 * rank)
    packs = []
    for rows, k in ((2 * wl.inter, wl.hidden), (wl.hidden, wl.inter)):
        payload = torch.empty((wl.local_experts, rows, k // 2), dtype=torch.int8, device=device)
        codes = torch.empty((wl.local_experts, rows, k // 32), dtype=torch.uint8, device=device)
        for e in range(wl.local_experts):      # one expert at a time keeps the fp32 staging small
            w = torch.randn((rows, k), device=device, generator=g) * 0.02
            payload[e], codes[e] = quant.quantize_weights_fp4(w)
        packs.append((payload, codes))
    bias = wl.expert_bias(device)
    tokens = {}
    for t in wl.sweep:
        sets = []
        for _ in range(INPUT_SETS):
            x = torch.randn((t, wl.hidden), device=device, generator=g).to(torch.bfloat16)
            xq, xsf = quant.quantize_activations(x)
            logits = torch.randn((t, wl.experts), device=device, generator=g)
            idx, wts = quant.route(logits if bias is None else logits + bias, wl.topk)
            sets.append((xq, xsf, idx, wts))
        tokens[t] = sets
    return packs, tokens


def run_ours(args):
    import torch.distributed as dist
    import gc_moe_b200 as G
    from gc_moe_b200 import _native, operator, quant
    from gc_moe_b200.contract import validate_call

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    else:
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29531')
        dist.init_process_group('gloo', rank=0, world_size=1)
    group = dist.group.WORLD
    wl = Workload(world, args.only_tokens)
    sweep = wl.sweep

    ((w1, c1), (w2, c2)), tokens = make_inputs(wl, device, rank)
    l1, l2 = G.transform_weights_for_gc_moe((w1, quant.weight_scales_mn_major(c1)),
                                            (w2, quant.weight_scales_mn_major(c2)))
    del w1, w2, c1, c2
    buf = G.get_symm_buffer_for_gc_moe(group, wl.experts, wl.capacity, wl.topk, wl.hidden, wl.inter)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    stream = torch.cuda.Stream(device=device)
    lib = _native.library()

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def stage(t, which):
        xq, xsf, idx, wts = tokens[t][which]
        buf.x[:t].copy_(xq); buf.x_sf[:t].copy_(xsf)
        buf.topk_idx[:t].copy_(idx); buf.topk_weights[:t].copy_(wts)

    ys, graphs, plans, active = {}, {}, {}, {}
    with torch.cuda.stream(stream):
        for t in sweep:
            ys[t] = torch.empty((t, wl.hidden), dtype=torch.bfloat16, device=device)
            # experts of THIS rank hit by the world's tokens (set 0)
            idx_all = [tokens[t][0][2]]
            if world > 1:
                gathered = [torch.empty_like(idx_all[0]) for _ in range(world)]
                dist.all_gather(gathered, idx_all[0])
                idx_all = gathered
            hit = torch.unique(torch.cat(idx_all))
            active[t] = int(((hit >= rank * wl.local_experts) & (hit < (rank + 1) * wl.local_experts)).sum())
            stage(t, 0)
            barrier()
            G.fp8_fp4_gc_moe(ys[t], l1, l2, buf, activation_clamp=10.0)       # eager warm call
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                G.fp8_fp4_gc_moe(ys[t], l1, l2, buf, activation_clamp=10.0)
            graphs[t] = graph
            cfg = validate_call(ys[t], l1, l2, buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True, None, None)
            plans[t] = operator.get_plan(cfg, ys[t], l1, l2, buf, None, None, None)
    barrier()
    buf.raise_on_device_error()

    n = len(sweep)
    start = [torch.cuda.Event(enable_timing=True) for _ in range(n * args.steps)]
    stop = [torch.cuda.Event(enable_timing=True) for _ in range(n * args.steps)]

    def one_sweep(step, record):
        for j, t in enumerate(sweep):
            stage(t, step % INPUT_SETS)           # alternate token sets: different experts each replay
            flush.zero_()                         # evict weights and workspace from L2
            if record:
                start[step * n + j].record(stream)
            graphs[t].replay()
            if record:
                stop[step * n + j].record(stream)

    with torch.cuda.stream(stream):
        with ClockSampler(local_rank) as clocks:
            clocks.wait_first(8.0)
            barrier()                 # nvidia-smi starts at different speeds per rank: enter the loop together
            clocks.mark_timed()
            for s in range(args.warmup):
                one_sweep(s, False)
            barrier()
            wall0 = time.perf_counter()
            for s in range(args.steps):
                one_sweep(s, True)
            barrier()
            wall = time.perf_counter() - wall0
    buf.raise_on_device_error()
    per_t = {t: [start[s * n + j].elapsed_time(stop[s * n + j]) * 1e3 for s in range(args.steps)]
             for j, t in enumerate(sweep)}
    local = torch.tensor([sum(sum(v) for v in per_t.values())] + [sum(per_t[t]) / args.steps for t in sweep],
                         dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(local, op=dist.ReduceOp.MAX)       # max over ranks
    total_us = float(local[0])
    latency = {str(t): round(float(local[1 + j]), 2) for j, t in enumerate(sweep)}

    # ---- reference protocol for context: windows of back-to-back replays, no flush inside
    b2b = {}
    if not args.skip_baselines:
        w0, w1e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        windows = []
        with torch.cuda.stream(stream):
            for t in sweep:
                stage(t, 0)
                barrier()
                flush.zero_()
                w0.record(stream)
                for _ in range(50):
                    graphs[t].replay()
                w1e.record(stream)
                barrier()
                windows.append(w0.elapsed_time(w1e) * 1e3 / 50)
        loc = torch.tensor(windows, dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(loc, op=dist.ReduceOp.MAX)
        b2b = {str(t): round(float(loc[j]), 2) for j, t in enumerate(sweep)}

    # ---- per-kernel timing for the roofline: one complete layer call enqueued as three
    # separate launches (dispatch | expert GEMMs | combine), which therefore run one after
    # the other instead of overlapping as they do inside a layer call.
    t = ROOFLINE_TOKENS if ROOFLINE_TOKENS in sweep else sweep[-1]
    cstream = ctypes.c_void_p(stream.cuda_stream)
    kev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    parts = {'dispatch': [], 'expert_gemms': [], 'combine': []}
    with torch.cuda.stream(stream):
        stage(t, 0)
        for _ in range(7):
            barrier()
            flush.zero_()
            kev[0].record(stream)
            for j, mask in enumerate((1, 6, 8)):
                _native.raise_for(lib.gcmoe_launch_kernels(plans[t].handle, mask, cstream))
                kev[j + 1].record(stream)
            stream.synchronize()
            for j, name in enumerate(parts):
                parts[name].append(kev[j].elapsed_time(kev[j + 1]) * 1e3)
        barrier()
    buf.raise_on_device_error()
    kernel_us = {name: sorted(v[2:])[len(v[2:]) // 2] for name, v in parts.items()}
    peaks_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))['hbm_gbs']), 'measured'
    else:
        peak, peak_src = 6650.0, 'fallback'
    l1_bytes = active[t] * wl.expert_bytes()
    achieved = l1_bytes / (kernel_us['expert_gemms'] * 1e-6) / 1e9
    roofline = {'bound': 'hbm', 'kernel': 'grouped_gemm_kernel (gate/up + down tiles of all active experts, one launch)', 'tokens': t, 'rank': rank,
                'achieved': round(achieved, 1), 'peak': peak, 'peak_source': peak_src,
                'unit': 'GB/s', 'frac': round(achieved / peak, 4),
                'algorithmic_bytes': l1_bytes, 'launch_us': round(kernel_us['expert_gemms'], 2),
                'traffic': None,
                'layer_frac_by_tokens_rank0': {
                    str(tt): round(active[tt] * wl.expert_bytes() / (float(latency[str(tt)]) * 1e-6) / 1e9 / peak, 4)
                    for tt in sweep},
                'kernel_us_at_tokens': {k: round(v, 2) for k, v in kernel_us.items()}}

    # ---- end to end through the public API with host buffers
    e2e_us, h2d, d2h = None, 0, 0
    if not args.skip_baselines:
        host = {}
        for t in sweep:
            xq, xsf, idx, wts = tokens[t][0]
            host[t] = ([v.cpu().pin_memory() for v in (xq.view(torch.uint8), xsf, idx, wts)],
                       torch.empty((t, wl.hidden), dtype=torch.bfloat16).pin_memory())
        h2d = sum(sum(v.numel() * v.element_size() for v in host[t][0]) for t in sweep)
        d2h = sum(host[t][1].numel() * 2 for t in sweep)

        def e2e_sweep():
            for t in sweep:
                (hx, hsf, hidx, hw), hy = host[t]
                buf.x[:t].view(torch.uint8).copy_(hx, non_blocking=True)
                buf.x_sf[:t].copy_(hsf, non_blocking=True)
                buf.topk_idx[:t].copy_(hidx, non_blocking=True)
                buf.topk_weights[:t].copy_(hw, non_blocking=True)
                G.fp8_fp4_gc_moe(ys[t], l1, l2, buf, activation_clamp=10.0)
                hy.copy_(ys[t], non_blocking=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            for _ in range(max(args.warmup, 3)):
                e2e_sweep()
            barrier()
            e0.record(stream)
            for _ in range(args.steps):
                e2e_sweep()
            e1.record(stream)
            barrier()
        e2e_local = torch.tensor([e0.elapsed_time(e1) * 1e3], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(e2e_local, op=dist.ReduceOp.MAX)
        e2e_us = float(e2e_local[0]) / (args.steps * n)
        buf.raise_on_device_error()

    value = total_us / (args.steps * n)
    line = {
        'metric': METRIC, 'value': round(value, 2), 'unit': 'us', 'n_gpus': world,
        'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': round(total_us / args.steps / 1e3, 5),
        'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8xfp4->bf16',
        'data': 'synthetic',
        'config': {'workload': wl.name + '; one step = one layer call per token count',
                   'parallelism': f'ep{world}' if world > 1 else 'single',
                   'experts_active_rank0': active,
                   'l2': 'flushed (512 MB memset) before every timed replay; token sets alternate between replays',
                   'timing': 'CUDA events around each graph replay on the launch stream, max over ranks'},
        'latency_us_by_tokens': latency,
        'latency_us_back_to_back_by_tokens': b2b,
        'tokens_per_s_by_tokens': {str(t): round(world * t / (float(latency[str(t)]) * 1e-6)) for t in sweep},
        'e2e': {'value': round(e2e_us, 2) if e2e_us is not None else None, 'unit': 'us',
                'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
        'gpu_launches': args.steps * n * lib.gcmoe_kernels_per_launch(plans[sweep[0]].handle),
        'roofline': roofline, 'clocks': clocks.summary(), 'wall_s_timed_region': round(wall, 3),
    }
    if world == 1 and not args.skip_baselines:
        ref = CpuReference(wl, fraction=max(1, wl.cpu_fraction // 2))
        line['cpu_baseline'] = ref.describe(ref.step_us())
    barrier()
    graphs.clear()              # captured graphs are retired before their workspace goes
    buf.destroy()
    if world == 1 and (args.large_token or not args.skip_baselines):
        del l1, l2, plans
        torch.cuda.empty_cache()
        line['large_token'] = large_token_leg(device, group, stream, flush)
    return line if rank == 0 else None


def large_token_leg(device, group, stream, flush, samples: int = 5) -> dict:
    """The tensor-bound regime of the same kernels on one GPU: hidden 7168,
    intermediate 2048, 32 local experts, 4096 tokens with uniform top-8 routing
    = 32768 rows, about 1024 per expert (the per-rank shape of the
    4096-tokens-per-rank configuration, with the expert count cut to 32 so that
    the case stays near 2 GB on the device).  Reports the expert-GEMM launch
    against the FP8-rate tensor peak: FLOPs = 6 x rows x H x I."""
    import gc_moe_b200 as G
    from gc_moe_b200 import _native, operator, quant
    from gc_moe_b200.contract import validate_call
    wl = Workload(1)
    wl.hidden, wl.experts, wl.topk, wl.inter, wl.zipf = 7168, 32, 8, 2048, None
    wl.local_experts, wl.sweep, wl.capacity = 32, (4096,), 4096
    t = 4096
    ((w1, c1), (w2, c2)), tokens = make_inputs(wl, device, 0)
    l1, l2 = G.transform_weights_for_gc_moe((w1, quant.weight_scales_mn_major(c1)),
                                            (w2, quant.weight_scales_mn_major(c2)))
    del w1, w2, c1, c2
    buf = G.get_symm_buffer_for_gc_moe(group, wl.experts, wl.capacity, wl.topk, wl.hidden, wl.inter)
    lib = _native.library()
    xq, xsf, idx, wts = tokens[t][0]
    buf.x[:t].copy_(xq); buf.x_sf[:t].copy_(xsf); buf.topk_idx[:t].copy_(idx); buf.topk_weights[:t].copy_(wts)
    y = torch.empty((t, wl.hidden), dtype=torch.bfloat16, device=device)
    cfg = validate_call(y, l1, l2, buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True, None, None)
    plan = operator.get_plan(cfg, y, l1, l2, buf, None, None, None)
    cstream = ctypes.c_void_p(stream.cuda_stream)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    out = {}
    with torch.cuda.stream(stream):
        for _ in range(3):
            lib.gcmoe_launch(plan.handle, cstream)
        stream.synchronize()
        buf.raise_on_device_error()
        for name, mask in (('layer', 15), ('expert_gemms', 6)):
            times = []
            for _ in range(samples):
                flush.zero_()
                k0.record(stream)
                if mask == 15:
                    lib.gcmoe_launch(plan.handle, cstream)
                else:
                    lib.gcmoe_launch_kernels(plan.handle, mask, cstream)
                k1.record(stream)
                stream.synchronize()
                times.append(k0.elapsed_time(k1) * 1e3)
            out[name] = sorted(times)[len(times) // 2]
    buf.raise_on_device_error()
    rows = int((idx >= 0).sum())
    flops = 6.0 * rows * wl.hidden * wl.inter
    achieved = flops / (out['expert_gemms'] * 1e-6) / 1e12
    peaks_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(peaks_path):
        bf16, src = float(json.load(open(peaks_path))['bf16_tflops']), 'measured'
    else:
        bf16, src = 1590.0, 'fallback'
    buf.destroy()
    return {'workload': 'H7168 I2048, 32 experts, 4096 tokens x top-8 = 32768 rows, uniform routing, 1 GPU',
            'block_m': cfg.block_m, 'bound': 'tensor', 'kernel': 'grouped_gemm_kernel (one launch)',
            'layer_us': round(out['layer'], 1), 'launch_us': round(out['expert_gemms'], 1),
            'achieved': round(achieved, 1), 'unit': 'TFLOP/s',
            'peak': round(2 * bf16, 1),
            'peak_source': f'2 x {src} dense bf16 cuBLAS burst ({bf16} TFLOP/s): the FP8-rate MMA kinds run at '
                           'twice the bf16 rate and no FP8 figure is measured on this pool',
            'frac': round(achieved / (2 * bf16), 4), 'frac_of_bf16_peak': round(achieved / bf16, 4)}


class CpuReference:
    """Reference CPU path on the host cores (the oracle port of the reference's
    PyTorch dequantise-and-matmul forward) for the WORLD's tokens in one
    process, on a bounded sample: for each token count of the sweep, the first
    1/fraction of the active experts, with the time scaled back by
    active/sampled (the cost is linear in the active experts)."""

    def __init__(self, wl: Workload, fraction: int):
        from oracle import gcmoe_oracle as O
        self.O, self.wl, self.fraction = O, wl, fraction
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.sample_experts = max(1, wl.experts // fraction)
        g = torch.Generator().manual_seed(7)
        w1 = torch.randn((self.sample_experts, 2 * wl.inter, wl.hidden), generator=g) * 0.02
        w2 = torch.randn((self.sample_experts, wl.hidden, wl.inter), generator=g) * 0.02
        self.q1, self.c1 = O.quantize_weight_fp4(w1)
        self.q2, self.c2 = O.quantize_weight_fp4(w2)
        bias = wl.expert_bias('cpu')
        self.calls = []
        for t in wl.sweep:
            xq, xsf, idx, wts = O.make_tokens(t * wl.world, wl.hidden, wl.experts, wl.topk, seed=50 + t,
                                              expert_bias=bias)
            active = torch.unique(idx).tolist()
            chosen = active[:max(1, -(-len(active) // fraction))][:self.sample_experts]
            sub = torch.full_like(idx, -1)
            for i, e in enumerate(chosen):
                sub[idx == e] = i
            self.calls.append((xq, xsf, sub, wts, len(active) / len(chosen)))

    def step_us(self) -> float:
        """Mean scaled latency of a layer call over one pass of the sweep."""
        total = 0.0
        for xq, xsf, sub, wts, scale in self.calls:
            t0 = time.perf_counter()
            self.O.moe_layer([xq], [xsf], [sub], [wts], self.q1, self.c1, self.q2, self.c2, [16], clamp=10.0)
            total += (time.perf_counter() - t0) * scale
        return total / len(self.calls) * 1e6

    def describe(self, value: float) -> dict:
        return {'value': round(value, 1), 'unit': 'us', 'cores': self.cores, 'kind': 'port',
                'sample': f'per token count in {list(self.wl.sweep)} (tokens of all {self.wl.world} rank(s) in one '
                          f'process): the first 1/{self.fraction} of the active experts (dequantise, both matmuls, '
                          'epilogues, combine); time scaled by active/sampled'}


def run_reference(args):
    if int(os.environ.get('RANK', '0')) != 0:
        return None
    world = int(os.environ.get('WORLD_SIZE', '1'))
    wl = Workload(world, args.only_tokens)
    ref = CpuReference(wl, fraction=wl.cpu_fraction)
    for _ in range(args.warmup):
        ref.step_us()
    steps = [ref.step_us() for _ in range(args.steps)]
    value = sum(steps) / len(steps)
    return {
        'impl': 'reference', 'metric': METRIC, 'value': round(value, 1), 'unit': 'us',
        'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': round(value * len(wl.sweep) / 1e3, 3), 'higher_is_better': False,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp32 (dequantised)', 'data': 'synthetic',
        'config': {'workload': wl.name + '; reference CPU path (oracle port), bounded sample per call'},
        'cpu_baseline': ref.describe(value),
        'e2e': {'value': round(value, 1), 'unit': 'us', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=('ours', 'reference'))
    ap.add_argument('--only-tokens', type=int, default=0,
                    help='profiling aid: run this single token count instead of the sweep')
    ap.add_argument('--skip-baselines', action='store_true',
                    help='profiling aid: skip the end-to-end, back-to-back and CPU-baseline legs')
    ap.add_argument('--large-token', action='store_true',
                    help='profiling aid: run the large-token leg even with --skip-baselines')
    args = ap.parse_args()
    if args.impl == 'ours':
        args.warmup = max(args.warmup, 3)
    line = run_reference(args) if args.impl == 'reference' else run_ours(args)
    if line is not None:
        print(json.dumps(line))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
