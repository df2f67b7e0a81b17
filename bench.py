"""Benchmark of the MoE layer hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Metric: MoE layer latency in microseconds under CUDA-graph replay, max over
ranks.  One step = one layer call (graph replay) at each token count of the
workload's sweep; `value` is the mean latency of a layer call over the sweep.

Headline workload (`value`, `e2e`, `roofline`):
* 1 GPU: the single-GPU configuration of the benchmark spec -- hidden 4096, 64
  routed experts, top-8, intermediate 2048, tokens in {1, 8, 32, 128, 256},
  uniform random routing.
* N > 1 GPUs: the expert-parallel decode configuration -- hidden 7168, 256
  routed experts sharded evenly over the N ranks, top-8, intermediate 2048,
  tokens per rank in {1, 2, 4, ..., 256}, router logits N(0,1) plus a
  Zipf(1.1) per-expert bias; dispatch and combine run over NVLink peer stores
  inside the layer's kernels (no NCCL on the data path).

Every line also carries, under `configs`, the two other configurations of the
spec on the same N GPUs (experts resharded 256 / N per rank):
* `c3`: hidden 6144, 256 routed experts top-8 (intermediate 2048) plus the
  fused FP8 shared expert (intermediate 4096, 128 x 128 block scales), uniform
  routing, tokens per rank in {1, 16, 64, 256};
* `c4`: the large-token regime: hidden 7168, 256 experts top-8, 4096 tokens per
  rank, 26 hot experts that draw half of the assignments (Gumbel top-8 without
  replacement); tokens/s and the fraction of the tensor peak;
and a `parity` block: one call of the headline workload (8 tokens per rank)
checked against the CPU oracle of the whole group -- the integer dispatch
products of every rank bit-exact, y within tolerance -- so that a multi-GPU
bench line is also a multi-GPU parity record.  A parity failure exits non-zero.

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
# Device-side waits give up after this long.  The library's default of 2 s is short when a rank
# of a loaded 8-GPU box falls behind during set-up; nothing in the timed regions waits that long.
os.environ.setdefault('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', '10')

import torch  # noqa: E402

METRIC = 'MoE layer latency us (graph replay, max over ranks) @1-256 tok/rank'
L2_FLUSH_BYTES = 512 << 20    # > 126 MB of L2
ROOFLINE_TOKENS = 32          # every local expert is hit: the weight-streaming regime
INPUT_SETS = 2                # alternating token sets per token count
COSINE_MIN, MAX_REL_ERR = 0.9999, 2.0 ** -6      # parity block: same bounds as tests/test_gpu_layer.py
CPU_FRACTION = {'c1': 4, 'c2': 16}                # share of the active experts the CPU arms run (both arms)


class Workload:
    """Geometry, routing model and token sweep of one benchmark configuration."""

    def __init__(self, world: int, kind: str, only_tokens: int = 0):
        self.world, self.kind = world, kind
        self.topk, self.inter, self.shared_inter, self.zipf, self.hot = 8, 2048, 0, None, 0
        self.capacity = 256
        if kind == 'c1':
            self.name = 'single-GPU config: H4096 E64 top8 I2048, tokens {1,8,32,128,256}, uniform routing'
            self.hidden, self.experts, self.sweep = 4096, 64, (1, 8, 32, 128, 256)
        elif kind == 'c2':
            self.name = (f'expert-parallel decode config on {world} GPUs: H7168 E256 ({256 // world}/rank) top8 I2048, '
                         'tokens/rank {1,2,4,8,16,32,64,128,256}, router logits N(0,1) + Zipf(1.1) expert bias')
            self.hidden, self.experts, self.sweep = 7168, 256, (1, 2, 4, 8, 16, 32, 64, 128, 256)
            self.zipf = 1.1
        elif kind == 'c3':
            self.name = (f'fused shared expert on {world} GPU(s): H6144 E256 ({256 // world}/rank) top8 I2048 + shared '
                         'FP8 expert I4096 with 128x128 block scales, tokens/rank {1,16,64,256}, uniform routing')
            self.hidden, self.experts, self.sweep, self.shared_inter = 6144, 256, (1, 16, 64, 256), 4096
        elif kind == 'c4':
            self.name = (f'large-token regime on {world} GPU(s): H7168 E256 ({256 // world}/rank) top8 I2048, 4096 '
                         'tokens/rank, 26 hot experts draw half of the assignments (Gumbel top-8 without replacement)')
            self.hidden, self.experts, self.sweep, self.hot, self.capacity = 7168, 256, (4096,), 26, 4096
        elif kind == 'lt':
            self.name = 'H7168 I2048, 32 experts, 4096 tokens x top-8 = 32768 rows, uniform routing, 1 GPU'
            self.hidden, self.experts, self.sweep, self.capacity = 7168, 32, (4096,), 4096
        else:
            raise ValueError(kind)
        if only_tokens:
            self.sweep = (only_tokens,)
        self.local_experts = self.experts // world
        self.shared_experts = self.shared_inter // self.inter
        self._gen = None

    def expert_bytes(self) -> int:
        """FP4 payload + UE8M0/32 scales of one expert's W1 and W2: the weight
        working-set model of the reference's benchmark (benchmark_gc_moe.py:248-309)."""
        return 3 * self.inter * self.hidden * 17 // 32

    def shared_bytes(self) -> int:
        """FP8 payload + K128 scale words of the fused shared expert."""
        if not self.shared_inter:
            return 0
        h, s = self.hidden, self.shared_inter
        return 3 * s * h + 4 * (2 * s * -(-h // 512) + h * -(-s // 512))

    def hot_experts(self):
        order = torch.randperm(self.experts, generator=torch.Generator().manual_seed(99))
        return order[:self.hot]

    def route(self, logits, device):
        """Expert ids and weights for router logits N(0,1) under this workload's model."""
        from gc_moe_b200 import quant
        if self.zipf is not None:
            # log p_e with p_e ~ 1 / rank_e^1.1 over a fixed seeded permutation
            perm = torch.randperm(self.experts, generator=torch.Generator().manual_seed(99)).float() + 1
            logits = logits + torch.log(perm.pow(-self.zipf) / perm.pow(-self.zipf).sum()).to(device)
        elif self.hot:
            # Gumbel top-k without replacement on log w_e: the hot experts share half of the mass
            w = torch.full((self.experts,), 0.5 / (self.experts - self.hot))
            w[self.hot_experts()] = 0.5 / self.hot
            u = torch.rand(logits.shape, device=device, generator=self._gen).clamp_min(1e-20)
            logits = torch.log(w).to(device) - torch.log(-torch.log(u))
        return quant.route(logits, self.topk)


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


WEIGHT_SHAPES = lambda wl: ((2 * wl.inter, wl.hidden), (wl.hidden, wl.inter))   # noqa: E731  W1, W2 rows x K


def make_inputs(wl: Workload, device, rank: int):
    """Seeded synthetic weights N(0, 0.02) -> FP4 for this rank's experts (and
    the replicated FP8 shared expert); per token count INPUT_SETS token sets
    N(0,1) -> FP8 with router logits N(0,1) routed by the workload's model,
    top-k and softmax over the selected k."""
    from gc_moe_b200 import quant
    g = torch.Generator(device=device).manual_seed(1234 + 7919 * rank)
    wl._gen = g
    packs = []
    for rows, k in WEIGHT_SHAPES(wl):
        payload = torch.empty((wl.local_experts, rows, k // 2), dtype=torch.int8, device=device)
        codes = torch.empty((wl.local_experts, rows, k // 32), dtype=torch.uint8, device=device)
        for e in range(wl.local_experts):      # one expert at a time keeps the fp32 staging small
            w = torch.randn((rows, k), device=device, generator=g) * 0.02
            payload[e], codes[e] = quant.quantize_weights_fp4(w)
        packs.append((payload, codes))
    shared = None
    if wl.shared_inter:
        gs = torch.Generator(device=device).manual_seed(4321)       # the same shared expert on every rank
        shared = []
        for rows, k in ((2 * wl.shared_inter, wl.hidden), (wl.hidden, wl.shared_inter)):
            q, codes = quant.quantize_weights_fp8_blocks(torch.randn((rows, k), device=device, generator=gs) * 0.02)
            shared.append((q, quant.expand_block_scales(codes, rows)))
    tokens = {}
    for t in wl.sweep:
        sets = []
        for _ in range(INPUT_SETS):
            x = torch.randn((t, wl.hidden), device=device, generator=g).to(torch.bfloat16)
            xq, xsf = quant.quantize_activations(x)
            logits = torch.randn((t, wl.experts), device=device, generator=g)
            idx, wts = wl.route(logits, device)
            sets.append((xq, xsf, idx, wts))
        tokens[t] = sets
    return packs, shared, tokens


def median(values):
    values = sorted(values)
    return values[len(values) // 2]


class Env:
    """Process-wide state of one bench run: device, stream, group, helpers."""

    def __init__(self):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get('WORLD_SIZE', '1'))
        self.rank = int(os.environ.get('RANK', '0'))
        self.local_rank = int(os.environ.get('LOCAL_RANK', '0'))
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device('cuda', self.local_rank)
        if self.world > 1:
            dist.init_process_group('nccl', device_id=self.device)
        else:
            os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
            os.environ.setdefault('MASTER_PORT', '29531')
            dist.init_process_group('gloo', rank=0, world_size=1)
        self.group = dist.group.WORLD
        self.flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=self.device)
        self.stream = torch.cuda.Stream(device=self.device)
        self.token = torch.zeros(1, device=self.device)
        peaks_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
        if os.path.exists(peaks_path):
            peaks = json.load(open(peaks_path))
            self.hbm_peak, self.bf16_peak = float(peaks['hbm_gbs']), float(peaks['bf16_tflops'])
            self.peak_source = 'measured'
        else:
            self.hbm_peak, self.bf16_peak, self.peak_source = 6650.0, 1590.0, 'fallback'

    def barrier(self):
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.device)

    def align(self):
        """Bring the ranks' streams to the same point on the device before a timed
        region: a one-element all-reduce that the launch stream waits for (no host
        synchronisation), so an event pair does not include waiting for a peer that
        is still staging inputs or flushing its L2."""
        if self.world > 1:
            self.dist.all_reduce(self.token)

    def max_over_ranks(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t]

    def gather(self, values):
        """[world][len(values)] on every rank."""
        t = torch.tensor(values, dtype=torch.float64, device=self.device)
        if self.world == 1:
            return [t.tolist()]
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [o.tolist() for o in out]

    def gather_cpu(self, t):
        """The ranks' tensors (same shape on every rank) as CPU tensors, on every rank."""
        if self.world == 1:
            return [t.cpu()]
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t.contiguous())
        return [o.cpu() for o in out]


class LayerBench:
    """One configuration on this process group: weights, workspace, one captured
    graph per token count, and the timing legs."""

    def __init__(self, env: Env, wl: Workload):
        import gc_moe_b200 as G
        from gc_moe_b200 import _native, operator, quant
        from gc_moe_b200.contract import validate_call
        self.env, self.wl, self.G, self.lib = env, wl, G, _native.library()
        dev = env.device
        ((w1, c1), (w2, c2)), shared, self.tokens = make_inputs(wl, dev, env.rank)
        self.l1, self.l2 = G.transform_weights_for_gc_moe((w1, quant.weight_scales_mn_major(c1)),
                                                          (w2, quant.weight_scales_mn_major(c2)))
        del w1, w2, c1, c2
        self.sl1 = self.sl2 = None
        self.kw = dict(activation_clamp=10.0)
        if shared is not None:
            self.sl1, self.sl2 = G.transform_weights_for_gc_moe(shared[0], shared[1])
            self.kw['shared_recipe'] = (1, 128, 128)
        self.buf = G.get_symm_buffer_for_gc_moe(env.group, wl.experts, wl.capacity, wl.topk, wl.hidden, wl.inter,
                                                wl.shared_experts)
        self.ys, self.graphs, self.plans, self.block_m = {}, {}, {}, {}
        self.stats = {}          # per token count: model inputs from the actual routes of set 0, all ranks
        lo, hi = env.rank * wl.local_experts, (env.rank + 1) * wl.local_experts
        with torch.cuda.stream(env.stream):
            for t in wl.sweep:
                self.ys[t] = torch.empty((t, wl.hidden), dtype=torch.bfloat16, device=dev)
                self.block_m[t] = G.get_block_m_for_gc_moe(env.world, wl.experts, self.buf.num_max_tokens_per_rank, t,
                                                           wl.topk)
                idx = self.tokens[t][0][2]
                idx_all = [idx]
                if env.world > 1:
                    idx_all = [torch.empty_like(idx) for _ in range(env.world)]
                    env.dist.all_gather(idx_all, idx)
                counts = torch.bincount(torch.cat(idx_all).reshape(-1), minlength=wl.experts)
                mine = counts[lo:hi]
                local = int(((idx >= lo) & (idx < hi)).sum())
                recv = int(mine.sum())
                per_rank = env.gather([float((mine > 0).sum()), float(recv), float(recv - local),
                                       float(idx.numel() - local)])
                self.stats[t] = {'active': [int(v[0]) for v in per_rank], 'recv_rows': [int(v[1]) for v in per_rank],
                                 'remote_in': [int(v[2]) for v in per_rank], 'remote_out': [int(v[3]) for v in per_rank]}
                if wl.hot:
                    hot = wl.hot_experts().to(dev)
                    self.stats[t]['hot_share'] = round(float(counts[hot].sum()) / max(1, int(counts.sum())), 4)
                self.stage(t, 0)
                env.barrier()
                self.call(t)                                                   # eager warm call
                env.barrier()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=env.stream):
                    self.call(t)
                self.graphs[t] = graph
                cfg = validate_call(self.ys[t], self.l1, self.l2, self.buf, self.sl1, self.sl2, None, (1, 1, 32), 'swiglu',
                                    10.0, True, self.kw.get('shared_recipe'), None)
                assert cfg.block_m == self.block_m[t]
                self.plans[t] = operator.get_plan(cfg, self.ys[t], self.l1, self.l2,
                                                  self.buf._for_call(cfg.shared_experts), self.sl1, self.sl2, None)
        env.barrier()
        self.buf.raise_on_device_error()

    def busiest(self, t) -> int:
        """The rank that sets the latency: most rows received, then most active experts."""
        s = self.stats[t]
        return max(range(self.env.world), key=lambda r: (s['recv_rows'][r], s['active'][r]))

    def call(self, t):
        self.G.fp8_fp4_gc_moe(self.ys[t], self.l1, self.l2, self.buf, self.sl1, self.sl2, **self.kw)

    def stage(self, t, which):
        xq, xsf, idx, wts = self.tokens[t][which]
        b = self.buf
        b.x[:t].copy_(xq); b.x_sf[:t].copy_(xsf)
        b.topk_idx[:t].copy_(idx); b.topk_weights[:t].copy_(wts)
        if self.wl.shared_inter:
            # caller-side staging of the shared expert's input scales in block-M order
            bm = self.block_m[t]
            tt = torch.arange(t, device=xq.device)
            u = tt % bm
            rows = (tt // bm) * ((bm + 127) // 128 * 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32
            b.shared_l1_acts_sf[rows] = xsf

    # ---- timing legs -------------------------------------------------------------------
    def time_flushed(self, steps, warmup, clocks=None):
        """Per token count: graph replays, each after an L2 flush and a switch of the
        token set, ranks aligned on the device; CUDA events on the launch stream.
        Returns ({t: mean us, max over ranks}, total us max over ranks, wall seconds)."""
        env, sweep = self.env, self.wl.sweep
        n = len(sweep)
        start = [torch.cuda.Event(enable_timing=True) for _ in range(n * steps)]
        stop = [torch.cuda.Event(enable_timing=True) for _ in range(n * steps)]

        def one_sweep(step, record):
            for j, t in enumerate(sweep):
                self.stage(t, step % INPUT_SETS)      # alternate token sets: different experts each replay
                env.flush.zero_()                     # evict weights and workspace from L2
                env.align()
                if record:
                    start[step * n + j].record(env.stream)
                self.graphs[t].replay()
                if record:
                    stop[step * n + j].record(env.stream)

        with torch.cuda.stream(env.stream):
            env.barrier()
            if clocks is not None:
                clocks.mark_timed()
            for s in range(warmup):
                one_sweep(s, False)
            env.barrier()
            wall0 = time.perf_counter()
            for s in range(steps):
                one_sweep(s, True)
            env.barrier()
            wall = time.perf_counter() - wall0
        self.buf.raise_on_device_error()
        per_t = [sum(start[s * n + j].elapsed_time(stop[s * n + j]) * 1e3 for s in range(steps)) / steps
                 for j in range(n)]
        reduced = env.max_over_ranks([sum(per_t) * steps] + per_t)
        return {t: reduced[1 + j] for j, t in enumerate(sweep)}, reduced[0], wall

    def time_back_to_back(self, windows, warm_windows, replays=100):
        """The reference's own protocol (benchmarks/benchmark_gc_moe.py:113-179): windows
        of back-to-back replays of one token count with fixed inputs; barrier, L2 flush
        and a 5 ms pause between windows only; per-rank median over the measured
        windows, max over ranks."""
        env = self.env
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        out = []
        with torch.cuda.stream(env.stream):
            for t in self.wl.sweep:
                self.stage(t, 0)
                samples = []
                for w in range(warm_windows + windows):
                    env.barrier()
                    env.flush.zero_()
                    torch.cuda.synchronize(env.device)
                    time.sleep(0.005)
                    env.align()
                    w0.record(env.stream)
                    for _ in range(replays):
                        self.graphs[t].replay()
                    w1.record(env.stream)
                    env.stream.synchronize()
                    if w >= warm_windows:
                        samples.append(w0.elapsed_time(w1) * 1e3 / replays)
                out.append(median(samples))
        self.buf.raise_on_device_error()
        reduced = env.max_over_ranks(out)
        return {t: reduced[j] for j, t in enumerate(self.wl.sweep)}

    def time_kernels(self, t, samples=7):
        """One complete layer call enqueued as three separate launches (dispatch |
        expert GEMMs | combine), which therefore run one after the other instead of
        overlapping as they do inside a layer call; ranks aligned before each call, L2
        flushed.  Returns per rank [dispatch, gemm, combine] medians in us."""
        from gc_moe_b200 import _native
        env = self.env
        cstream = ctypes.c_void_p(env.stream.cuda_stream)
        kev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        parts = [[], [], []]
        with torch.cuda.stream(env.stream):
            self.stage(t, 0)
            for _ in range(samples):
                env.barrier()
                env.flush.zero_()
                env.align()
                kev[0].record(env.stream)
                for j, mask in enumerate((1, 6, 8)):
                    _native.raise_for(self.lib.gcmoe_launch_kernels(self.plans[t].handle, mask, cstream))
                    kev[j + 1].record(env.stream)
                env.stream.synchronize()
                for j in range(3):
                    parts[j].append(kev[j].elapsed_time(kev[j + 1]) * 1e3)
            env.barrier()
        self.buf.raise_on_device_error()
        return env.gather([median(v[2:]) for v in parts])

    def time_e2e(self, steps, warmup):
        """Through the public API with HOST buffers: every call copies its quantised
        inputs from pinned host memory, runs the layer and reads y back."""
        env, wl = self.env, self.wl
        host = {}
        for t in wl.sweep:
            xq, xsf, idx, wts = self.tokens[t][0]
            host[t] = ([v.cpu().pin_memory() for v in (xq.view(torch.uint8), xsf, idx, wts)],
                       torch.empty((t, wl.hidden), dtype=torch.bfloat16).pin_memory())
        h2d = sum(sum(v.numel() * v.element_size() for v in host[t][0]) for t in wl.sweep)
        d2h = sum(host[t][1].numel() * 2 for t in wl.sweep)
        b = self.buf

        def sweep_once():
            for t in wl.sweep:
                (hx, hsf, hidx, hw), hy = host[t]
                b.x[:t].view(torch.uint8).copy_(hx, non_blocking=True)
                b.x_sf[:t].copy_(hsf, non_blocking=True)
                b.topk_idx[:t].copy_(hidx, non_blocking=True)
                b.topk_weights[:t].copy_(hw, non_blocking=True)
                self.call(t)
                hy.copy_(self.ys[t], non_blocking=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(env.stream):
            for _ in range(max(warmup, 3)):
                sweep_once()
            env.barrier()
            env.align()
            e0.record(env.stream)
            for _ in range(steps):
                sweep_once()
            e1.record(env.stream)
            env.barrier()
        us = env.max_over_ranks([e0.elapsed_time(e1) * 1e3])[0] / (steps * len(wl.sweep))
        self.buf.raise_on_device_error()
        return us, h2d, d2h

    def model(self, t, rank, latency_us):
        """The reference benchmark's workload model for one rank
        (benchmarks/benchmark_gc_moe.py:235-384): weight + scale working set of the
        experts that were hit, FLOPs of the rows received, useful NVLink payload of
        the remote assignments (H + H/32 in, 2H out per assignment)."""
        wl, s = self.wl, self.stats[t]
        weight_bytes = s['active'][rank] * wl.expert_bytes() + wl.shared_bytes()
        flops = 6.0 * s['recv_rows'][rank] * wl.hidden * wl.inter + 6.0 * t * wl.hidden * wl.shared_inter
        nvlink = (s['remote_in'][rank] + s['remote_out'][rank]) * (3 * wl.hidden + wl.hidden // 32) // 2
        sec = latency_us * 1e-6
        return {'rank': rank, 'active_experts': s['active'][rank], 'recv_rows': s['recv_rows'][rank],
                'weight_bytes': weight_bytes, 'weight_gbs': round(weight_bytes / sec / 1e9, 1),
                'frac_of_hbm_peak': round(weight_bytes / sec / 1e9 / self.env.hbm_peak, 4),
                'tflops': round(flops / sec / 1e12, 1),
                'nvlink_useful_payload_bytes': nvlink, 'nvlink_useful_payload_gbs': round(nvlink / sec / 1e9, 1)}

    def close(self):
        self.env.barrier()
        self.graphs.clear()          # captured graphs are retired before their workspace goes
        self.plans.clear()
        self.buf.destroy()
        del self.l1, self.l2, self.sl1, self.sl2, self.tokens
        torch.cuda.empty_cache()


def parity_block(env: Env, lb: LayerBench, tokens: int = 8) -> dict:
    """One call of the bench's own workload against the CPU oracle of the whole group:
    every rank compares the integer dispatch products in its arena with the oracle's
    (bit-exact), rank 0 compares every rank's y (cosine, maximum error relative to the
    largest output magnitude).  Outside every timed region."""
    import numpy as np
    import gc_moe_b200 as G
    from gc_moe_b200 import quant
    from gc_moe_b200.layout import round_up, sf_row_in_block
    from oracle import gcmoe_oracle as O
    wl, dist, dev, world, rank = lb.wl, env.dist, env.device, env.world, env.rank
    g = torch.Generator(device=dev).manual_seed(555 + 31 * rank)
    wl._gen = g
    x = torch.randn((tokens, wl.hidden), device=dev, generator=g).to(torch.bfloat16)
    xq, xsf = quant.quantize_activations(x)
    idx, wts = wl.route(torch.randn((tokens, wl.experts), device=dev, generator=g), dev)
    all_xq = [t.view(torch.float8_e4m3fn) for t in env.gather_cpu(xq.view(torch.uint8))]
    all_xsf, all_idx, all_w = env.gather_cpu(xsf), env.gather_cpu(idx), env.gather_cpu(wts)
    b = lb.buf
    y = torch.full((tokens, wl.hidden), float('nan'), dtype=torch.bfloat16, device=dev)
    with torch.cuda.stream(env.stream):
        b.x[:tokens].copy_(xq); b.x_sf[:tokens].copy_(xsf)
        b.topk_idx[:tokens].copy_(idx); b.topk_weights[:tokens].copy_(wts)
        gen = int(b.region('recv_parity').view(torch.int32)[0].item()) & 1
        env.barrier()
        G.fp8_fp4_gc_moe(y, lb.l1, lb.l2, b, lb.sl1, lb.sl2, **lb.kw)
        env.barrier()
    b.raise_on_device_error()
    # ---- integer products of this rank against the oracle's dispatch of the whole group
    bms = [G.get_block_m_for_gc_moe(world, wl.experts, b.num_max_tokens_per_rank, tokens, wl.topk)] * world
    d = O.dispatch([t.numpy() for t in all_idx], [t.numpy() for t in all_w],
                   [t.view(torch.uint8).numpy() for t in all_xq], [t.numpy() for t in all_xsf], wl.experts, bms)[rank]
    el, bm = wl.local_experts, bms[rank]
    counts = b.region('expert_recv_count').view(torch.int64)[gen * world * el:(gen + 1) * world * el]
    exact = bool(np.array_equal(counts.cpu().numpy().reshape(world, el), d.counts))
    exact &= int(b.region('routed_pool_blocks').view(torch.int32)[0]) == d.pool_blocks
    rows = d.pool_blocks * bm
    valid = np.nonzero(d.metadata[:, 0] >= 0)[0]
    meta = b.region('token_src_metadata').view(torch.int32).reshape(-1, 3)[:rows].cpu().numpy()
    exact &= bool(np.array_equal(meta[valid], d.metadata[valid]))
    acts = b.l1_acts.view(torch.uint8)[:rows].cpu().numpy()
    exact &= bool(np.array_equal(acts[valid], d.rows[valid]))
    route_w = b.buffer.narrow(0, b.layout.views['l1_topk_weights'].offset, rows * 4).view(torch.float32).cpu().numpy()
    exact &= bool(np.array_equal(route_w[valid], d.weights[valid]))
    sf = b.l1_acts_sf[:d.pool_blocks * round_up(bm, 128)].cpu().numpy()
    sf_rows = np.array([(r // bm) * round_up(bm, 128) + sf_row_in_block(r % bm) for r in valid], dtype=np.int64)
    if len(valid):
        exact &= bool(np.array_equal(sf[sf_rows], d.sf_words[valid]))
    table = (b.region('src_token_topk_idx').view(torch.int32).reshape(-1, b.layout.capacity)[:el * world]
             .cpu().numpy().reshape(el, world, -1))
    exact &= all(np.array_equal(table[l, s, :len(v)].astype(np.uint32), v) for (l, s), v in d.index_lists.items())
    integers_exact = all(f[0] == 1.0 for f in env.gather([1.0 if exact else 0.0]))
    # ---- y of every rank on rank 0.  The oracle reads the original-layout weights of the experts
    # that were hit; they were dropped after the transform, so every rank regenerates its own
    # (same generator, same order) and sends the hit ones to rank 0.
    every = torch.cat(all_idx).reshape(-1)
    hit = torch.unique(every[(every >= 0) & (every < wl.experts)]).tolist()
    ys = env.gather_cpu(y)
    result = {'tokens_per_rank': tokens, 'ranks_checked': world, 'active_experts': len(hit),
              'integers_exact': integers_exact, 'tolerance': {'cosine_min': COSINE_MIN, 'max_rel_err': MAX_REL_ERR}}
    gw = torch.Generator(device=dev).manual_seed(1234 + 7919 * rank)
    mine = {e - rank * el for e in hit if rank * el <= e < (rank + 1) * el}
    kept = {}
    for which, (rws, k) in enumerate(WEIGHT_SHAPES(wl)):
        for e in range(el):
            w = torch.randn((rws, k), device=dev, generator=gw) * 0.02
            if e in mine:
                kept[(which, e)] = quant.quantize_weights_fp4(w)
    pieces = {}
    for e in hit:
        r = e // el
        for which, (rws, k) in enumerate(WEIGHT_SHAPES(wl)):
            if r == 0:
                if rank == 0:
                    pieces[(which, e)] = tuple(v.cpu() for v in kept[(which, e)])
            elif rank == r:
                payload, codes = kept[(which, e - r * el)]
                dist.send(payload.contiguous(), 0)
                dist.send(codes.contiguous(), 0)
            elif rank == 0:
                payload = torch.empty((rws, k // 2), dtype=torch.int8, device=dev)
                codes = torch.empty((rws, k // 32), dtype=torch.uint8, device=dev)
                dist.recv(payload, r)
                dist.recv(codes, r)
                pieces[(which, e)] = (payload.cpu(), codes.cpu())
    if rank == 0:
        class HitExperts:
            """Stand-in for an [E, ...] weight tensor that holds only the experts that were hit."""

            def __init__(self, which, part, shape):
                self.which, self.part, self.shape = which, part, shape

            def __getitem__(self, e):
                return pieces[(self.which, int(e))][self.part]
        w1 = HitExperts(0, 0, (wl.experts, 2 * wl.inter, wl.hidden // 2))
        w2 = HitExperts(1, 0, (wl.experts, wl.hidden, wl.inter // 2))
        ref = O.moe_layer(all_xq, all_xsf, all_idx, all_w, w1, HitExperts(0, 1, None), w2, HitExperts(1, 1, None),
                          bms, clamp=10.0)
        cos = [O.cosine(ys[r], ref.y[r]) for r in range(world)]
        err = [O.max_rel_err(ys[r], ref.y[r]) for r in range(world)]
        finite = all(bool(torch.isfinite(v.float()).all()) for v in ys)
        result.update({'cosine_min': round(min(cos), 9), 'max_rel_err': max(err),
                       'pass': bool(integers_exact and finite and min(cos) >= COSINE_MIN and max(err) <= MAX_REL_ERR)})
    env.barrier()
    return result


def headline(env: Env, args):
    wl = Workload(env.world, 'c1' if env.world == 1 else 'c2', args.only_tokens)
    lb = LayerBench(env, wl)
    sweep, n = wl.sweep, len(wl.sweep)
    with ClockSampler(env.local_rank) as clocks:
        clocks.wait_first(8.0)
        latency, total_us, wall = lb.time_flushed(args.steps, args.warmup, clocks)
    b2b = {}
    if not args.skip_baselines:
        full = args.steps >= 20
        b2b = lb.time_back_to_back(30 if full else max(3, args.steps), 10 if full else 2)
    # ---- per-kernel times (busiest rank and max over ranks) and the roofline of the dominant kernel
    kernel_tokens = [t for t in (1, 8, 32, 256) if t in sweep] or [sweep[-1]]
    if args.skip_baselines:
        kernel_tokens = [t for t in kernel_tokens if t == ROOFLINE_TOKENS] or kernel_tokens[-1:]
    kernels = {}
    for t in kernel_tokens:
        per_rank = lb.time_kernels(t)
        r = lb.busiest(t)
        kernels[str(t)] = {'busiest_rank': r,
                           'dispatch': round(per_rank[r][0], 2), 'expert_gemms': round(per_rank[r][1], 2),
                           'combine': round(per_rank[r][2], 2),
                           'max_over_ranks': [round(max(v[j] for v in per_rank), 2) for j in range(3)]}
    t = ROOFLINE_TOKENS if str(ROOFLINE_TOKENS) in kernels else kernel_tokens[-1]
    r = kernels[str(t)]['busiest_rank']
    gemm_us = kernels[str(t)]['expert_gemms']
    bytes_ = lb.stats[t]['active'][r] * wl.expert_bytes()
    achieved = bytes_ / (gemm_us * 1e-6) / 1e9
    roofline = {'bound': 'hbm', 'kernel': 'grouped_gemm_kernel (gate/up + down tiles of all active experts, one launch)',
                'tokens': t, 'rank': r, 'rank_choice': 'busiest: most rows received, then most active experts',
                'achieved': round(achieved, 1), 'peak': env.hbm_peak, 'peak_source': env.peak_source,
                'unit': 'GB/s', 'frac': round(achieved / env.hbm_peak, 4),
                'algorithmic_bytes': bytes_, 'launch_us': round(gemm_us, 2),
                'traffic': None,
                'traffic_note': 'not measured in this run; the ncu summary of this kernel gives dram read + write per launch',
                'kernel_us_by_tokens': kernels,
                'layer_model_by_tokens_busiest_rank': {str(tt): lb.model(tt, lb.busiest(tt), latency[tt]) for tt in sweep}}
    e2e_us, h2d, d2h = (None, 0, 0) if args.skip_baselines else lb.time_e2e(args.steps, args.warmup)
    line = {
        'metric': METRIC, 'value': round(total_us / (args.steps * n), 2), 'unit': 'us', 'n_gpus': env.world,
        'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': round(total_us / args.steps / 1e3, 5),
        'higher_is_better': False, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'fp8xfp4->bf16',
        'data': 'synthetic',
        'config': {'workload': wl.name + '; one step = one layer call per token count',
                   'parallelism': f'ep{env.world}' if env.world > 1 else 'single',
                   'experts_active_by_tokens_per_rank': {str(t): lb.stats[t]['active'] for t in sweep},
                   'block_m_by_tokens': {str(t): lb.block_m[t] for t in sweep},
                   'l2': 'flushed (512 MB memset) before every timed replay; token sets alternate between replays',
                   'timing': 'CUDA events around each graph replay on the launch stream after a device-side '
                             'alignment of the ranks, max over ranks'},
        'latency_us_by_tokens': {str(t): round(latency[t], 2) for t in sweep},
        'latency_us_back_to_back_by_tokens': {str(t): round(v, 2) for t, v in b2b.items()},
        'back_to_back_protocol': 'median over windows of 100 replays; barrier, L2 flush and 5 ms between windows; '
                                 'max over ranks',
        'tokens_per_s_by_tokens': {str(t): round(env.world * t / (latency[t] * 1e-6)) for t in sweep},
        'e2e': {'value': round(e2e_us, 2) if e2e_us is not None else None, 'unit': 'us',
                'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
        'gpu_launches': args.steps * sum(lb.lib.gcmoe_kernels_per_launch(lb.plans[t].handle) for t in sweep),
        'roofline': roofline, 'clocks': clocks.summary(), 'wall_s_timed_region': round(wall, 3),
    }
    return line, lb


def side_config(env: Env, kind: str, steps: int, warmup: int) -> dict:
    """C3 or C4 on this process group: flushed graph-replay latency per token count,
    per-kernel times and the workload model on the busiest rank."""
    wl = Workload(env.world, kind)
    lb = LayerBench(env, wl)
    latency, _, _ = lb.time_flushed(steps, warmup)
    out = {'workload': wl.name, 'steps': steps, 'block_m_by_tokens': {str(t): lb.block_m[t] for t in wl.sweep},
           'latency_us_by_tokens': {str(t): round(latency[t], 2) for t in wl.sweep},
           'tokens_per_s_by_tokens': {str(t): round(env.world * t / (latency[t] * 1e-6)) for t in wl.sweep},
           'model_busiest_rank_by_tokens': {str(t): lb.model(t, lb.busiest(t), latency[t]) for t in wl.sweep}}
    t = wl.sweep[-1] if kind == 'c4' else (64 if 64 in wl.sweep else wl.sweep[-1])
    per_rank = lb.time_kernels(t, samples=5)
    r = lb.busiest(t)
    gemm_us = per_rank[r][1]
    s = lb.stats[t]
    out['kernel_us'] = {'tokens': t, 'busiest_rank': r, 'dispatch': round(per_rank[r][0], 2),
                        'expert_gemms': round(gemm_us, 2), 'combine': round(per_rank[r][2], 2)}
    if kind == 'c4':
        tf = 6.0 * s['recv_rows'][r] * wl.hidden * wl.inter / (gemm_us * 1e-6) / 1e12
        out['hot_share_realised'] = s.get('hot_share')
        out['roofline'] = {'bound': 'tensor', 'kernel': 'grouped_gemm_kernel (one launch)', 'rank': r,
                           'recv_rows': s['recv_rows'][r], 'launch_us': round(gemm_us, 1),
                           'achieved': round(tf, 1), 'unit': 'TFLOP/s', 'peak': round(2 * env.bf16_peak, 1),
                           'peak_source': f'2 x {env.peak_source} dense bf16 cuBLAS burst: kind::mxf8f6f4 with an FP8 '
                                          'operand runs at the FP8 rate; no FP8 figure is measured on this pool',
                           'frac': round(tf / (2 * env.bf16_peak), 4),
                           'frac_of_fp4_peak': round(tf / (4 * env.bf16_peak), 4)}
    else:
        bytes_ = s['active'][r] * wl.expert_bytes() + wl.shared_bytes()
        gbs = bytes_ / (gemm_us * 1e-6) / 1e9
        out['roofline'] = {'bound': 'hbm', 'kernel': 'grouped_gemm_kernel (one launch)', 'rank': r, 'tokens': t,
                           'algorithmic_bytes': bytes_, 'launch_us': round(gemm_us, 2), 'achieved': round(gbs, 1),
                           'unit': 'GB/s', 'peak': env.hbm_peak, 'peak_source': env.peak_source,
                           'frac': round(gbs / env.hbm_peak, 4)}
    lb.close()
    return out


def large_token_leg(env: Env, samples: int = 5) -> dict:
    """The tensor-bound regime of the same kernels on one GPU at the per-rank shape of
    the 8-GPU large-token configuration: hidden 7168, intermediate 2048, 32 local
    experts, 4096 tokens with uniform top-8 routing = 32768 rows, about 1024 per
    expert (the ncu summary of the large-token regime is of this case).  Reports the
    expert-GEMM launch against the FP8-rate tensor peak: FLOPs = 6 x rows x H x I."""
    from gc_moe_b200 import _native
    wl = Workload(1, 'lt')
    lb = LayerBench(env, wl)
    t = 4096
    cstream = ctypes.c_void_p(env.stream.cuda_stream)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    layer = []
    with torch.cuda.stream(env.stream):
        for _ in range(samples + 2):
            env.flush.zero_()
            k0.record(env.stream)
            _native.raise_for(lb.lib.gcmoe_launch(lb.plans[t].handle, cstream))
            k1.record(env.stream)
            env.stream.synchronize()
            layer.append(k0.elapsed_time(k1) * 1e3)
    per_rank = lb.time_kernels(t, samples=samples + 2)
    gemm_us = per_rank[0][1]
    rows = lb.stats[t]['recv_rows'][0]
    achieved = 6.0 * rows * wl.hidden * wl.inter / (gemm_us * 1e-6) / 1e12
    out = {'workload': wl.name, 'block_m': lb.block_m[t], 'bound': 'tensor', 'kernel': 'grouped_gemm_kernel (one launch)',
           'layer_us': round(median(layer[2:]), 1), 'launch_us': round(gemm_us, 1),
           'achieved': round(achieved, 1), 'unit': 'TFLOP/s', 'peak': round(2 * env.bf16_peak, 1),
           'peak_source': f'2 x {env.peak_source} dense bf16 cuBLAS burst ({env.bf16_peak} TFLOP/s): the FP8-rate MMA '
                          'kinds run at twice the bf16 rate and no FP8 figure is measured on this pool',
           'frac': round(achieved / (2 * env.bf16_peak), 4), 'frac_of_bf16_peak': round(achieved / env.bf16_peak, 4)}
    lb.close()
    return out


def run_ours(args):
    env = Env()
    line, lb = headline(env, args)
    failed = False
    if not args.skip_parity:
        line['parity'] = parity_block(env, lb, 8)
        failed = env.rank == 0 and not line['parity'].get('pass', False)
    if env.world == 1 and not args.skip_baselines:
        ref = CpuReference(lb.wl, fraction=CPU_FRACTION[lb.wl.kind])
        line['cpu_baseline'] = ref.describe(ref.step_us())
    lb.close()
    if not args.skip_configs and not args.only_tokens:
        line['configs'] = {'c3': side_config(env, 'c3', max(3, min(args.steps, 10)), 3),
                           'c4': side_config(env, 'c4', max(3, min(args.steps, 5)), 3)}
    if env.world == 1 and (args.large_token or not args.skip_baselines):
        line['large_token'] = large_token_leg(env)
    failed = env.max_over_ranks([1.0 if failed else 0.0])[0] != 0.0
    return (line if env.rank == 0 else None), failed


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
        bias = None
        if wl.zipf is not None:
            perm = torch.randperm(wl.experts, generator=torch.Generator().manual_seed(99)).float() + 1
            bias = torch.log(perm.pow(-wl.zipf) / perm.pow(-wl.zipf).sum())
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
        total, raw = 0.0, 0.0
        for xq, xsf, sub, wts, scale in self.calls:
            t0 = time.perf_counter()
            self.O.moe_layer([xq], [xsf], [sub], [wts], self.q1, self.c1, self.q2, self.c2, [16], clamp=10.0)
            dt = time.perf_counter() - t0
            raw += dt
            total += dt * scale
        self.last_unscaled_us = raw / len(self.calls) * 1e6      # what the host cores actually ran
        return total / len(self.calls) * 1e6

    def describe(self, value: float) -> dict:
        return {'value': round(value, 1), 'unit': 'us', 'cores': self.cores, 'kind': 'port',
                'unscaled_us_per_call_actually_run': round(getattr(self, 'last_unscaled_us', 0.0), 1),
                'sample': f'per token count in {list(self.wl.sweep)} (tokens of all {self.wl.world} rank(s) in one '
                          f'process): the first 1/{self.fraction} of the active experts (dequantise, both matmuls, '
                          'epilogues, combine) is run and timed; the reported value is that time scaled by '
                          'active/sampled, an extrapolation (the cost is linear in the active experts); the same '
                          "fraction in the GPU arm's cpu_baseline and in --impl reference"}


def run_reference(args):
    if int(os.environ.get('RANK', '0')) != 0:
        return None
    world = int(os.environ.get('WORLD_SIZE', '1'))
    wl = Workload(world, 'c1' if world == 1 else 'c2', args.only_tokens)
    ref = CpuReference(wl, fraction=CPU_FRACTION[wl.kind])
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
    ap.add_argument('--skip-configs', action='store_true',
                    help='profiling aid: skip the c3 and c4 configurations')
    ap.add_argument('--skip-parity', action='store_true', help='profiling aid: skip the parity block')
    ap.add_argument('--large-token', action='store_true',
                    help='profiling aid: run the large-token leg even with --skip-baselines')
    args = ap.parse_args()
    # Standard output carries the one JSON line and nothing else: libraries that write to file
    # descriptor 1 themselves (NCCL prints its version there under NCCL_DEBUG=VERSION) are sent to
    # standard error for the length of the run.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    failed = False
    if args.impl == 'ours':
        args.warmup = max(args.warmup, 3)
        line, failed = run_ours(args)
    else:
        line = run_reference(args)
    sys.stdout.flush()
    if line is not None:
        os.write(json_fd, (json.dumps(line) + '\n').encode())
    os.close(json_fd)
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()
    if failed:
        sys.exit(3)


if __name__ == '__main__':
    main()
