"""The checkers the GPU parity tests use must themselves reject what they claim to reject:
the classified comparison of the requantised intermediate is exercised here on synthetic
bytes (no GPU)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from _cases import check_requantised_intermediate, sf_rows_of_pool
from gc_moe_b200.layout import round_up


def synthetic(rows=40, inter=256, bm=16, seed=3):
    rng = np.random.default_rng(seed)
    acts = rng.integers(0, 0x7F, size=(rows, inter), dtype=np.uint8) | (rng.integers(0, 2, size=(rows, inter), dtype=np.uint8) << 7)
    sf = rng.integers(100, 140, size=(rows, inter // 32), dtype=np.uint8)
    metadata = np.zeros((rows, 3), dtype=np.int32)
    metadata[5::7, 0] = -1                      # padding rows of the pool are not compared
    ref = SimpleNamespace(dispatch=[SimpleNamespace(metadata=metadata)],
                          l2_acts=[torch.from_numpy(acts.copy())], l2_sf=[torch.from_numpy(sf.copy())])
    ring = np.zeros((round_up(rows, bm) // bm * round_up(bm, 128), inter // 32), dtype=np.uint8)
    ring[sf_rows_of_pool(np.arange(rows), bm)] = sf
    prod = {'l2_acts': acts.copy(), 'l2_acts_sf': ring}
    return prod, ref, bm


def test_identical_bytes_pass_and_padding_rows_are_ignored():
    prod, ref, bm = synthetic()
    prod['l2_acts'][5] ^= 0x55                  # a padding row
    check_requantised_intermediate(prod, ref, bm, 'synthetic')


def test_one_code_step_passes_below_the_fraction_and_fails_above_it():
    prod, ref, bm = synthetic()
    prod['l2_acts'][0, 0] = (prod['l2_acts'][0, 0] & 0x80) | ((prod['l2_acts'][0, 0] & 0x7F) + 1)
    check_requantised_intermediate(prod, ref, bm, 'synthetic', max_fraction=1e-3)
    for c in range(1, 40):
        prod['l2_acts'][0, c] = (prod['l2_acts'][0, c] & 0x80) | ((prod['l2_acts'][0, c] & 0x7F) ^ 1)
    with pytest.raises(AssertionError):
        check_requantised_intermediate(prod, ref, bm, 'synthetic', max_fraction=1e-3)


def test_two_code_steps_or_a_sign_flip_fail():
    prod, ref, bm = synthetic()
    prod['l2_acts'][1, 3] = (prod['l2_acts'][1, 3] & 0x80) | (((prod['l2_acts'][1, 3] & 0x7F) + 2) % 0x7F)
    with pytest.raises(AssertionError):
        check_requantised_intermediate(prod, ref, bm, 'synthetic')
    prod, ref, bm = synthetic()
    prod['l2_acts'][2, 9] = (prod['l2_acts'][2, 9] ^ 0x80) | 0x10
    with pytest.raises(AssertionError):
        check_requantised_intermediate(prod, ref, bm, 'synthetic')


def test_a_moved_scale_byte_excuses_its_group_only_and_only_by_one_step():
    prod, ref, bm = synthetic()
    ring_row = sf_rows_of_pool(np.array([3]), bm)[0]
    prod['l2_acts_sf'][ring_row, 1] += 1
    prod['l2_acts'][3, 32:64] ^= 0x3C           # the group's payload follows its scale
    check_requantised_intermediate(prod, ref, bm, 'synthetic', max_fraction=1e-2)
    prod['l2_acts'][3, 64] ^= 0x3C              # a byte of the next group does not
    with pytest.raises(AssertionError):
        check_requantised_intermediate(prod, ref, bm, 'synthetic', max_fraction=1e-2)
    prod, ref, bm = synthetic()
    prod['l2_acts_sf'][ring_row, 1] += 2
    with pytest.raises(AssertionError):
        check_requantised_intermediate(prod, ref, bm, 'synthetic', max_fraction=1e-2)
