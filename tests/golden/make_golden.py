"""Generate the golden fixtures of this directory from the reference's own
importable Python code.  Run in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

Nothing else reads the reference; the tests only read the files written here.
Sources: gc_moe/layout/gc_moe.py (layout offsets), gc_moe/jit_kernels/
heuristics/gc_moe.py (block-M and ring sizing), gc_moe/gc/__init__.py and
gc_moe/jit_kernels/impls/runtime_utils.py (weight transform),
tests/test_sm120_gc_moe.py (dequantisers and the dequantise-and-matmul
forward the reference uses as its own accuracy reference).
"""

import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, 'tests'))
    sys.path.insert(0, ROOT)
    from gc_moe.layout.gc_moe import GCBufferLayout, SIGNAL_OFFSETS
    from gc_moe.jit_kernels.heuristics.gc_moe import get_block_m_for_gc_moe, get_ring_tokens
    from gc_moe.gc import _gc_interleave_rows, _gc_transpose_sf
    from gc_moe.jit_kernels.impls.runtime_utils import repack_fp4_weights, repack_fp8_weights
    import test_sm120_gc_moe as ref_tests
    from oracle import gcmoe_oracle as O

    host = {'signal_offsets': SIGNAL_OFFSETS, 'layouts': [], 'block_m': [], 'ring': []}
    geometries = [  # P, E, cap, k, H, I, sms, S
        (1, 8, 1920, 2, 1024, 512, 148, 0), (1, 64, 1920, 8, 4096, 2048, 148, 0),
        (8, 256, 1920, 8, 7168, 2048, 148, 0), (8, 256, 1920, 8, 6144, 2048, 148, 2),
        (8, 256, 5760, 8, 7168, 2048, 148, 0), (2, 256, 1920, 8, 6144, 2048, 148, 2),
        (4, 384, 1920, 6, 5120, 2304, 140, 1), (1, 256, 5760, 8, 7168, 2048, 148, 0)]
    for p, e, cap, k, h, i, sms, s in geometries:
        ring, sf_ring = get_ring_tokens(p, e, cap, k, h, i, sms)
        host['ring'].append({'args': [p, e, cap, k, h, i, sms], 'ring': [ring, sf_ring]})
        lay = GCBufferLayout(p, e, cap, k, h, i, ring, sf_ring, s)
        host['layouts'].append({
            'args': [p, e, cap, k, h, i, ring, sf_ring, s], 'nbytes': lay.nbytes,
            'num_max_pool_tokens': lay.num_max_pool_tokens, 'workspace': lay.workspace_offsets,
            'views': {n: [v.offset, v.nbytes, list(v.shape), v.dtype,
                          list(v.stride) if v.stride else None] for n, v in lay.views.items()}})
    for p, e, k in [(1, 8, 2), (1, 64, 8), (8, 256, 8), (8, 384, 6), (2, 256, 8), (4, 256, 8),
                    (32, 256, 8), (1, 256, 8), (72, 1152, 8)]:
        for cap in (1920, 5760):
            tokens = sorted(set(list(range(0, 300)) + list(range(300, cap + 1, 37)) + [cap]))
            host['block_m'].append({'args': [p, e, cap, k], 'tokens': tokens,
                                    'block_m': [get_block_m_for_gc_moe(p, e, cap, t, k) for t in tokens]})
    with open(os.path.join(HERE, 'host_geometry.json'), 'w') as f:
        json.dump(host, f, indent=0, sort_keys=True)

    # Weight transform: seeded bytes in, digests + one small full tensor out.
    g = torch.Generator().manual_seed(11)
    w1 = torch.randint(-128, 128, (3, 256, 128), dtype=torch.int8, generator=g)     # E=3, 2I=256, H=256
    w2 = torch.randint(-128, 128, (3, 256, 64), dtype=torch.int8, generator=g)      # H=256, I=128
    sf1 = torch.randint(0, 2 ** 31 - 1, (3, 2, 256), dtype=torch.int32, generator=g).transpose(1, 2)
    sf2 = torch.randint(0, 2 ** 31 - 1, (3, 1, 256), dtype=torch.int32, generator=g).transpose(1, 2)
    s8a = torch.randint(0, 255, (256, 256), dtype=torch.uint8, generator=g)
    out = {'w1': repack_fp4_weights(_gc_interleave_rows(w1)), 'w2': repack_fp4_weights(w2),
           'sf1': _gc_transpose_sf(_gc_interleave_rows(sf1)), 'sf2': _gc_transpose_sf(sf2),
           'fp8': repack_fp8_weights(_gc_interleave_rows(s8a.view(torch.float8_e4m3fn))).view(torch.uint8)}
    np.savez_compressed(os.path.join(HERE, 'weight_transform.npz'),
                        in_w1=w1.numpy(), in_w2=w2.numpy(), in_sf1=sf1.contiguous().numpy(),
                        in_sf2=sf2.contiguous().numpy(), in_fp8=s8a.numpy(),
                        **{'out_' + k: v.contiguous().numpy() for k, v in out.items()},
                        out_sf1_strides=np.array(out['sf1'].stride()),
                        out_sf2_strides=np.array(out['sf2'].stride()))

    # Dequantise-and-matmul forward of the reference on the CPU-runnable
    # configuration (16 tokens, hidden 1024, 8 experts, top-2, intermediate 512)
    # and a second case with invalid routes and no clamp.
    cases = {}
    for name, (e, h, i, k, t, clamp, seed, drop) in {
            'c0': (8, 1024, 512, 2, 16, 10.0, 0, False),
            'c0_noclamp_invalid': (8, 1024, 512, 2, 24, None, 5, True)}.items():
        q1, c1, q2, c2 = O.make_weights(e, h, i, seed=seed)
        xq, xsf, idx, w = O.make_tokens(t, h, e, k, seed=seed + 1)
        if drop:
            idx[::3, 0] = -1
        y = ref_tests.reference_processed_moe_forward(xq, xsf, idx, w, q1, c1, q2, c2, i, clamp)
        cases[name] = {'args': [e, h, i, k, t, clamp, seed, drop], 'y': y.view(torch.int16).numpy(),
                       'inputs_sha': sha(q1) + sha(c1) + sha(q2) + sha(c2) + sha(xq) + sha(xsf)
                       + sha(idx) + sha(w),
                       'w1_dequant_sha': sha(ref_tests.dequantize_mxfp4(q1[0], c1[0])),
                       'x_dequant_sha': sha(ref_tests.dequantize_activation(xq, xsf))}
    np.savez_compressed(os.path.join(HERE, 'processed_forward.npz'),
                        **{f'{n}_y': c['y'] for n, c in cases.items()})
    with open(os.path.join(HERE, 'processed_forward.json'), 'w') as f:
        json.dump({n: {k: v for k, v in c.items() if k != 'y'} for n, c in cases.items()}, f,
                  indent=0, sort_keys=True)

    # Shared expert forward (FP8 weights, 128x128 block scales) of the reference.
    g = torch.Generator().manual_seed(3)
    h, i_s, t = 512, 256, 12
    sw1, sc1 = O.quantize_block_fp8(torch.randn((2 * i_s, h), generator=g) * 0.05)
    sw2, sc2 = O.quantize_block_fp8(torch.randn((h, i_s), generator=g) * 0.05)
    xq, xsf, _, _ = O.make_tokens(t, h, 8, 2, seed=9)
    x = ref_tests.dequantize_activation(xq, xsf)
    scales = [torch.exp2(c.float() - 127) for c in (sc1, sc2)]
    ys = ref_tests.reference_shared_forward(x, ((sw1, scales[0]), (sw2, scales[1])), 10.0, gran_k=128)
    np.savez_compressed(os.path.join(HERE, 'shared_forward.npz'), y=ys.view(torch.int16).numpy(),
                        sw1=sw1.view(torch.uint8).numpy(), sc1=sc1.numpy(),
                        sw2=sw2.view(torch.uint8).numpy(), sc2=sc2.numpy(),
                        xq=xq.view(torch.uint8).numpy(), xsf=xsf.numpy())
    print('golden fixtures written to', HERE)


if __name__ == '__main__':
    if len(sys.argv) != 2:
        sys.exit('usage: python tests/golden/make_golden.py <path of the reference checkout>')
    main(sys.argv[1])
