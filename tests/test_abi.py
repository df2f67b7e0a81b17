"""The C-ABI library loads on a machine without a GPU and exports every
function include/gcmoe.h declares, with the struct sizes the binding assumes."""
import ctypes
import os
import re
import subprocess

import pytest

from gc_moe_b200 import _native, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, 'include', 'gcmoe.h')


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(gcmoe_[a-z0-9_]+)\s*\(', text)))


@pytest.fixture(scope='module')
def lib():
    build.build()
    return _native.library()


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
    assert sorted(_native.EXPORTED_SYMBOLS) == names


def test_struct_sizes_match_the_header(tmp_path):
    src = tmp_path / 'sizes.c'
    src.write_text('#include <stdio.h>\n#include "gcmoe.h"\nint main(void){printf("%zu %zu %zu %zu\\n",'
                   'sizeof(gcmoe_problem),sizeof(gcmoe_buffers),offsetof(gcmoe_buffers,y),'
                   'offsetof(gcmoe_problem,clamp));return 0;}\n')
    exe = tmp_path / 'sizes'
    subprocess.run(['gcc', '-I', os.path.join(ROOT, 'include'), str(src), '-o', str(exe)], check=True)
    sizes = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(_native.Problem), ctypes.sizeof(_native.Buffers),
                     _native.Buffers.y.offset, _native.Problem.clamp.offset]


def test_version_and_argument_errors_need_no_gpu(lib):
    assert lib.gcmoe_version() >= 100
    prob = _native.Problem(num_ranks=1, rank=0, num_experts=8, capacity=1920, topk=2, hidden=1024,
                           intermediate=512, num_tokens=4, block_m=16, ring_tokens=5760,
                           sf_ring_tokens=46080)
    assert lib.gcmoe_scratch_bytes(ctypes.byref(prob)) >= 8 * 4 + 17 * 4
    handle = ctypes.c_void_p()
    bufs = _native.Buffers()
    for bad, exc in ((dict(block_m=24), ValueError), (dict(hidden=1000), NotImplementedError),
                     (dict(num_tokens=5000), ValueError), (dict(rank=3), ValueError),
                     (dict(ring_tokens=1920), NotImplementedError)):
        p = _native.Problem.from_buffer_copy(prob)
        for k, v in bad.items():
            setattr(p, k, v)
        rc = lib.gcmoe_plan_create(ctypes.byref(p), ctypes.byref(bufs), ctypes.byref(handle))
        assert rc < 0 and not handle.value
        with pytest.raises(exc):
            _native.raise_for(rc)
    # a well-formed problem with null buffers is a contract violation, not a crash
    rc = lib.gcmoe_plan_create(ctypes.byref(prob), ctypes.byref(bufs), ctypes.byref(handle))
    assert rc == _native.ERR_INVALID and 'arena' in _native.last_error()
    assert lib.gcmoe_launch(None, None) == _native.ERR_INVALID


def test_stage_inputs_struct_and_argument_errors_need_no_gpu(lib, tmp_path):
    src = tmp_path / 'stage.c'
    src.write_text('#include <stdio.h>\n#include "gcmoe.h"\nint main(void){printf("%zu %zu\\n",'
                   'sizeof(gcmoe_stage_args),offsetof(gcmoe_stage_args,shared_sf_rows));return 0;}\n')
    exe = tmp_path / 'stage'
    subprocess.run(['gcc', '-I', os.path.join(ROOT, 'include'), str(src), '-o', str(exe)], check=True)
    sizes = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(_native.StageArgs), _native.StageArgs.shared_sf_rows.offset]

    assert lib.gcmoe_stage_inputs(None, None) == _native.ERR_INVALID
    good = dict(x=0x1000, router_logits=0x2000, x_q=0x3000, x_sf=0x4000, topk_idx=0x5000, topk_weights=0x6000,
                num_tokens=4, hidden=1024, num_experts=8, topk=2, block_m=16)
    for bad in (dict(hidden=1000), dict(topk=0), dict(topk=33), dict(x=0x1004), dict(x_q=0), dict(num_experts=1),
                dict(num_experts=4096), dict(router_logits=0), dict(shared_sf=0x7000, shared_sf_rows=64, num_tokens=200),
                dict(shared_sf=0x7000, shared_sf_rows=128, block_m=24)):
        args = _native.StageArgs(**{**good, **bad})
        assert lib.gcmoe_stage_inputs(ctypes.byref(args), None) == _native.ERR_INVALID, bad
    # no tokens: nothing to do, nothing launched
    assert lib.gcmoe_stage_inputs(ctypes.byref(_native.StageArgs(**{**good, 'num_tokens': 0})), None) == 0


def test_static_scratch_limits_are_checked_before_any_cuda_call(lib):
    """The entry point for callers that cannot allocate holds its scratch in a fixed
    64 KiB array: both ways of outgrowing it are refused with a message that names
    the limit that was exceeded (no GPU needed: the checks come first)."""
    bufs = _native.Buffers()
    many_experts = _native.Problem(num_ranks=1, rank=0, num_experts=256, capacity=1920, topk=8, hidden=1024,
                                   intermediate=512, num_tokens=4, block_m=16, ring_tokens=1920 * 40,
                                   sf_ring_tokens=1920 * 40 * 16)
    assert lib.gcmoe_launch_static_scratch(ctypes.byref(many_experts), ctypes.byref(bufs), None) == _native.ERR_UNSUPPORTED
    assert 'local experts exceed the 128' in _native.last_error()
    # 32 local experts are fine, but the tile counters of a 4096-token, top-8 ring are not
    big_ring = _native.Problem(num_ranks=1, rank=0, num_experts=32, capacity=5760, topk=8, hidden=7168,
                               intermediate=2048, num_tokens=4096, block_m=240, ring_tokens=376320,
                               sf_ring_tokens=376320 * 16)
    assert lib.gcmoe_scratch_bytes(ctypes.byref(big_ring)) > 65536
    assert lib.gcmoe_launch_static_scratch(ctypes.byref(big_ring), ctypes.byref(bufs), None) == _native.ERR_UNSUPPORTED
    message = _native.last_error()
    assert 'tile counters' in message and 'ring of 376320 rows' in message and 'local experts exceed' not in message
    assert lib.gcmoe_static_scratch_status(None, None) == _native.ERR_INVALID
