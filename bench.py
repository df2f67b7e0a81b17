"""Benchmark of the MoE layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Metric: MoE layer latency in microseconds under CUDA-graph replay (max over
ranks).  At one GPU the workload is the single-GPU configuration of the
benchmark spec: hidden 4096, 64 routed experts, top-8, intermediate 2048, FP8
e4m3 activations and FP4 e2m1 weights with UE8M0/32 scales, uniform random
routing, tokens in {1, 8, 32, 128, 256}.  One step = one layer call at each of
the five token counts; `value` is the mean latency of a layer call over the
sweep.  Inputs are seeded synthetic tensors of those shapes and distributions.

`--impl reference` times the reference operator's own CPU path for this layer
(its PyTorch dequantise-and-matmul forward, restated in oracle/gcmoe_oracle.py)
on the host cores, on a bounded sample of each call.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

HIDDEN, EXPERTS, TOPK, INTER = 4096, 64, 8, 2048
SWEEP = (1, 8, 32, 128, 256)
CAPACITY = 256
ROOFLINE_TOKENS = 32          # every expert is hit: the weight-streaming regime
METRIC = 'MoE layer latency us (graph replay, max over ranks) @1-256 tok/rank'
L2_FLUSH_BYTES = 512 << 20    # > 126 MB of L2


def expert_bytes() -> int:
    """FP4 payload + UE8M0/32 scales of one expert's W1 and W2: the weight
    working set model of the reference's benchmark (benchmark_gc_moe.py:248-309)."""
    return 3 * INTER * HIDDEN * 17 // 32


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while timing runs."""

    FIELDS = ('clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,'
              'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
              'clocks_event_reasons.sw_power_cap')

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--id={self.index}', f'--query-gpu={self.FIELDS}',
                 '--format=csv,noheader,nounits', '-lms', '100'],
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

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['unavailable']}
        clocks = sorted(int(s[0]) for s in self.samples)
        names = ('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap')
        reasons = [n for i, n in enumerate(names) if any(s[2 + i] == 'Active' for s in self.samples)]
        return {'sm_mhz': clocks[len(clocks) // 2], 'sm_max_mhz': int(self.samples[0][1]),
                'reasons': reasons, 'samples': len(clocks)}


def make_inputs(device, rank: int):
    """Seeded synthetic weights N(0, 0.02) -> FP4, per-T tokens N(0,1) -> FP8,
    router logits N(0,1), top-k + softmax over the selected k."""
    from gc_moe_b200 import quant
    g = torch.Generator(device=device).manual_seed(1234 + 7919 * rank)
    packs = []
    for rows, k in ((2 * INTER, HIDDEN), (HIDDEN, INTER)):
        payload = torch.empty((EXPERTS, rows, k // 2), dtype=torch.int8, device=device)
        codes = torch.empty((EXPERTS, rows, k // 32), dtype=torch.uint8, device=device)
        for e in range(EXPERTS):      # one expert at a time keeps the fp32 staging small
            w = torch.randn((rows, k), device=device, generator=g) * 0.02
            payload[e], codes[e] = quant.quantize_weights_fp4(w)
        packs.append((payload, codes))
    tokens = {}
    for t in SWEEP:
        x = torch.randn((t, HIDDEN), device=device, generator=g).to(torch.bfloat16)
        xq, xsf = quant.quantize_activations(x)
        idx, wts = quant.route(torch.randn((t, EXPERTS), device=device, generator=g), TOPK)
        tokens[t] = (xq, xsf, idx, wts)
    return packs, tokens


def run_ours(args) -> dict:
    import torch.distributed as dist
    import gc_moe_b200 as G
    from gc_moe_b200 import _native, operator, quant
    from gc_moe_b200.contract import validate_call
    import ctypes

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local_rank = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local_rank)
    device = torch.device('cuda', local_rank)
    if world > 1:
        dist.init_process_group('nccl', device_id=device)
    # The expert-parallel exchange over NVLink is not built yet: every rank
    # runs the single-GPU workload on its own replica (no data-path collective).
    if not dist.is_initialized():
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('MASTER_PORT', '29531')
        dist.init_process_group('gloo', rank=0, world_size=1)
        solo = dist.group.WORLD
    else:
        solo = dist.new_group([rank], backend='gloo', use_local_synchronization=True)

    ((w1, c1), (w2, c2)), tokens = make_inputs(device, rank)
    l1, l2 = G.transform_weights_for_gc_moe((w1, quant.weight_scales_mn_major(c1)),
                                            (w2, quant.weight_scales_mn_major(c2)))
    del w1, w2, c1, c2
    buf = G.get_symm_buffer_for_gc_moe(solo, EXPERTS, CAPACITY, TOPK, HIDDEN, INTER)
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    stream = torch.cuda.Stream(device=device)
    lib = _native.library()

    ys, graphs, plans, active = {}, {}, {}, {}
    with torch.cuda.stream(stream):
        for t in SWEEP:
            xq, xsf, idx, wts = tokens[t]
            ys[t] = torch.empty((t, HIDDEN), dtype=torch.bfloat16, device=device)
            active[t] = int(torch.unique(idx).numel())

            def stage(t=t, xq=xq, xsf=xsf, idx=idx, wts=wts):
                buf.x[:t].copy_(xq); buf.x_sf[:t].copy_(xsf)
                buf.topk_idx[:t].copy_(idx); buf.topk_weights[:t].copy_(wts)
            stage()
            G.fp8_fp4_gc_moe(ys[t], l1, l2, buf, activation_clamp=10.0)       # eager warm call
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                G.fp8_fp4_gc_moe(ys[t], l1, l2, buf, activation_clamp=10.0)
            graphs[t] = (graph, stage)
            cfg = validate_call(ys[t], l1, l2, buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True, None, None)
            plans[t] = operator.get_plan(cfg, ys[t], l1, l2, buf, None, None, None)
    buf.raise_on_device_error()

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    start = [torch.cuda.Event(enable_timing=True) for _ in range(len(SWEEP) * args.steps)]
    stop = [torch.cuda.Event(enable_timing=True) for _ in range(len(SWEEP) * args.steps)]

    def sweep(record_from=None):
        for j, t in enumerate(SWEEP):
            graph, stage = graphs[t]
            stage()
            flush.zero_()                         # evict weights and workspace from L2
            if record_from is not None:
                start[record_from + j].record(stream)
            graph.replay()
            if record_from is not None:
                stop[record_from + j].record(stream)

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            sweep()
        barrier()
        with ClockSampler(local_rank) as clocks:
            wall0 = time.perf_counter()
            for s in range(args.steps):
                sweep(record_from=s * len(SWEEP))
            barrier()
            wall = time.perf_counter() - wall0
    per_t = {t: [] for t in SWEEP}
    for s in range(args.steps):
        for j, t in enumerate(SWEEP):
            per_t[t].append(start[s * len(SWEEP) + j].elapsed_time(stop[s * len(SWEEP) + j]) * 1e3)
    step_us = [sum(per_t[t][s] for t in SWEEP) for s in range(args.steps)]
    local = torch.tensor([sum(step_us)] + [sum(per_t[t]) / args.steps for t in SWEEP],
                         dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(local, op=dist.ReduceOp.MAX)       # max over ranks
    total_us = float(local[0])
    latency = {str(t): round(float(local[1 + j]), 2) for j, t in enumerate(SWEEP)}

    # ---- per-kernel timing of the dominant kernel (gate/up GEMM) for the roofline
    t = ROOFLINE_TOKENS
    cstream = ctypes.c_void_p(stream.cuda_stream)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    kernel_us = {}
    with torch.cuda.stream(stream):
        graphs[t][1]()
        lib.gcmoe_launch_kernels(plans[t].handle, 1, cstream)
        for name, mask in (('gate_up_gemm', 2), ('down_gemm', 4), ('dispatch', 1), ('combine', 8)):
            samples = []
            for _ in range(5):
                flush.zero_()
                k0.record(stream)
                lib.gcmoe_launch_kernels(plans[t].handle, mask, cstream)
                k1.record(stream)
                stream.synchronize()
                samples.append(k0.elapsed_time(k1) * 1e3)
            kernel_us[name] = sorted(samples)[len(samples) // 2]
    peaks_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))['hbm_gbs']), 'measured'
    else:
        peak, peak_src = 6650.0, 'fallback'
    l1_bytes = active[t] * expert_bytes() * 2 // 3
    achieved = l1_bytes / (kernel_us['gate_up_gemm'] * 1e-6) / 1e9
    roofline = {'bound': 'hbm', 'kernel': 'grouped_gemm_kernel<gate/up>', 'tokens': t,
                'achieved': round(achieved, 1), 'peak': peak, 'peak_source': peak_src,
                'unit': 'GB/s', 'frac': round(achieved / peak, 4),
                'algorithmic_bytes': l1_bytes, 'launch_us': round(kernel_us['gate_up_gemm'], 2),
                'traffic': None,
                'layer_frac_by_tokens': {str(tt): round(active[tt] * expert_bytes() / (float(latency[str(tt)]) * 1e-6) / 1e9 / peak, 4)
                                         for tt in SWEEP},
                'kernel_us_at_tokens': {k: round(v, 2) for k, v in kernel_us.items()}}

    e2e_us, h2d, d2h = None, 0, 0
    if not args.skip_baselines:
        # ---- end to end through the public API with host buffers
        host = {}
        for t in SWEEP:
            xq, xsf, idx, wts = tokens[t]
            host[t] = ([v.cpu().pin_memory() for v in (xq.view(torch.uint8), xsf, idx, wts)],
                       torch.empty((t, HIDDEN), dtype=torch.bfloat16).pin_memory())
        h2d = sum(sum(v.numel() * v.element_size() for v in host[t][0]) for t in SWEEP)
        d2h = sum(host[t][1].numel() * 2 for t in SWEEP)

        def e2e_sweep():
            for t in SWEEP:
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
        e2e_us = float(e2e_local[0]) / (args.steps * len(SWEEP))
        buf.raise_on_device_error()

    value = total_us / (args.steps * len(SWEEP))
    line = {
        'metric': METRIC, 'value': round(value, 2), 'unit': 'us', 'n_gpus': world,
        'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': round(total_us / args.steps / 1e3, 5),
        'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8xfp4->bf16',
        'data': 'synthetic',
        'config': {'workload': 'single-GPU config: H4096 E64 top8 I2048, tokens {1,8,32,128,256}, uniform routing; '
                               'one step = one layer call per token count',
                   'parallelism': 'replicas' if world > 1 else 'single', 'experts_active': active,
                   'l2': 'flushed (512 MB memset) before every timed replay',
                   'timing': 'CUDA events around each graph replay on the launch stream'},
        'latency_us_by_tokens': latency,
        'tokens_per_s_by_tokens': {str(t): round(world * t / (float(latency[str(t)]) * 1e-6)) for t in SWEEP},
        'e2e': {'value': round(e2e_us, 2) if e2e_us is not None else None, 'unit': 'us', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
        'gpu_launches': args.steps * len(SWEEP) * lib.gcmoe_kernels_per_launch(plans[SWEEP[0]].handle),
        'roofline': roofline, 'clocks': clocks.summary(), 'wall_s_timed_region': round(wall, 3),
    }
    if world == 1 and not args.skip_baselines:
        line['cpu_baseline'] = cpu_baseline(fraction=4, repeats=1)
    buf.destroy()
    return line if rank == 0 else None


class CpuReference:
    """Reference CPU path on the host cores (the oracle port of the reference's
    PyTorch dequantise-and-matmul forward), on a bounded sample: for each token
    count of the sweep, the first 1/fraction of the active experts, with the
    time scaled back by active/sampled (the cost is linear in active experts)."""

    def __init__(self, fraction: int):
        from oracle import gcmoe_oracle as O
        self.O, self.fraction = O, fraction
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.sample_experts = max(1, EXPERTS // fraction)
        g = torch.Generator().manual_seed(7)
        w1 = torch.randn((self.sample_experts, 2 * INTER, HIDDEN), generator=g) * 0.02
        w2 = torch.randn((self.sample_experts, HIDDEN, INTER), generator=g) * 0.02
        self.q1, self.c1 = O.quantize_weight_fp4(w1)
        self.q2, self.c2 = O.quantize_weight_fp4(w2)
        self.calls = []
        for t in SWEEP:
            xq, xsf, idx, wts = O.make_tokens(t, HIDDEN, EXPERTS, TOPK, seed=50 + t)
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
                'sample': f'per token count in {list(SWEEP)}: the first 1/{self.fraction} of the active experts '
                          '(dequantise, both matmuls, epilogues, combine); time scaled by active/sampled'}


def cpu_baseline(fraction: int, repeats: int) -> dict:
    ref = CpuReference(fraction)
    values = [ref.step_us() for _ in range(repeats)]
    return ref.describe(sum(values) / len(values))


def run_reference(args) -> dict | None:
    if int(os.environ.get('RANK', '0')) != 0:
        return None
    ref = CpuReference(fraction=8)
    for _ in range(args.warmup):
        ref.step_us()
    steps = [ref.step_us() for _ in range(args.steps)]
    value = sum(steps) / len(steps)
    return {
        'impl': 'reference', 'metric': METRIC, 'value': round(value, 1), 'unit': 'us',
        'n_gpus': int(os.environ.get('WORLD_SIZE', '1')), 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': round(value * len(SWEEP) / 1e3, 3), 'higher_is_better': False,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp32 (dequantised)', 'data': 'synthetic',
        'config': {'workload': 'single-GPU config: H4096 E64 top8 I2048, tokens {1,8,32,128,256}, uniform routing; '
                               'reference CPU path (oracle port), bounded sample per call'},
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
                    help='profiling aid: skip the end-to-end and CPU-baseline legs')
    args = ap.parse_args()
    if args.only_tokens:
        global SWEEP, ROOFLINE_TOKENS
        SWEEP, ROOFLINE_TOKENS = (args.only_tokens,), args.only_tokens
    args.warmup = max(args.warmup, 3) if args.impl == 'ours' else args.warmup
    line = run_reference(args) if args.impl == 'reference' else run_ours(args)
    if line is not None:
        print(json.dumps(line))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
