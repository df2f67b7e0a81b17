"""Environment knobs the operator honours, parsed the way the reference parses
them (gc_moe/runtime/gc_moe.py:29-49, gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:166-180).
Host logic only."""
import types

import pytest
import torch

from gc_moe_b200 import operator


@pytest.fixture
def sms(monkeypatch):
    monkeypatch.setattr(torch.cuda, 'current_device', lambda: 0)
    monkeypatch.setattr(torch.cuda, 'get_device_properties',
                        lambda index: types.SimpleNamespace(multi_processor_count=148))


def test_dispatch_sms_default_and_valid_requests(monkeypatch, sms):
    monkeypatch.delenv('GC_MOE_DISPATCH_SMS', raising=False)
    assert operator._dispatch_sms() == 0            # the library's own default
    for raw, value in (('8', 8), ('16', 16), ('2', 2), ('147', 147)):
        monkeypatch.setenv('GC_MOE_DISPATCH_SMS', raw)
        assert operator._dispatch_sms() == value


@pytest.mark.parametrize('raw', ['', ' 8', '8 ', '+8', '0x8', '8.0', 'eight', '99999999999'])
def test_dispatch_sms_strict_parsing(monkeypatch, sms, raw):
    monkeypatch.setenv('GC_MOE_DISPATCH_SMS', raw)
    with pytest.raises(ValueError, match='invalid value for GC_MOE_DISPATCH_SMS'):
        operator._dispatch_sms()


@pytest.mark.parametrize('raw', ['-1', '0', '1', '148', '1000'])
def test_dispatch_sms_outside_the_device_is_refused(monkeypatch, sms, raw):
    monkeypatch.setenv('GC_MOE_DISPATCH_SMS', raw)
    with pytest.raises(ValueError, match='invalid dispatch SM request'):
        operator._dispatch_sms()


def test_barrier_timeout_parsing(monkeypatch):
    monkeypatch.delenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', raising=False)
    assert operator._timeout_ms() == 2000
    monkeypatch.setenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', '7')
    assert operator._timeout_ms() == 7000
    for bad in ('0', '-3', 'x', '1.5'):
        monkeypatch.setenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', bad)
        with pytest.raises(ValueError):
            operator._timeout_ms()
