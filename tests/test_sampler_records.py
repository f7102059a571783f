"""What the sampler sends to the device per row and per token (host side; no GPU needed)."""
import struct
import types

import numpy as np

from vllm_cpp_b200.sampling.sampler import Sampler, SamplingOptions


def as_float(i):
    return struct.unpack("<f", struct.pack("<i", int(i)))[0]


def test_records_hold_the_options_bit_for_bit_and_all_fit_int32():
    opts = [SamplingOptions(0.7, 0.8, 1.1, seed=(1 << 63) + 12345), SamplingOptions(0.0, 1.0, 1.0, seed=7),
            SamplingOptions(1.5, 1.0, 0.0, seed=0xFFFFFFFF)]
    flat, use_counts, no_nucleus = Sampler.records(opts, [3, 0, (1 << 31) + 5], [2, 0, 1])
    rec = np.asarray(flat, dtype=np.int64).reshape(3, 8)
    assert np.all(rec >= -(1 << 31)) and np.all(rec < (1 << 31))
    rec32 = rec.astype(np.int32)
    assert [as_float(rec32[i, 0]) for i in range(3)] == [np.float32(0.7), 0.0, 1.5]
    assert as_float(rec32[0, 1]) == np.float32(0.8) and as_float(rec32[0, 2]) == np.float32(1.1)
    assert rec32[0, 3] == 2 and rec32[1, 3] == -1 and rec32[2, 3] == -1      # the count row only where a penalty applies
    assert as_float(rec32[2, 2]) == 1.0                                     # penalty 0 means none
    seed0 = (int(rec32[0, 5]) & 0xFFFFFFFF) << 32 | (int(rec32[0, 4]) & 0xFFFFFFFF)
    assert seed0 == (1 << 63) + 12345
    assert int(rec32[2, 4]) & 0xFFFFFFFF == 0xFFFFFFFF and int(rec32[2, 6]) & 0xFFFFFFFF == (1 << 31) + 5
    assert use_counts and not no_nucleus                                    # row 0 has a penalty and cuts a nucleus


def test_which_kernels_a_step_needs():
    greedy = SamplingOptions(0.0, 0.5, 1.0)              # top-p means nothing to a greedy row
    plain = SamplingOptions(0.9, 1.0, 1.0)
    assert Sampler.records([greedy, plain], [0, 0], [0, 1])[1:] == (False, True)
    assert Sampler.records([plain, SamplingOptions(0.9, 0.95, 1.0)], [0, 0], [0, 1])[1:] == (False, False)
    assert Sampler.records([SamplingOptions(0.0, 1.0, 1.3)], [0], [4])[1:] == (True, True)
    assert Sampler.records([], [], []) == ([], False, True)


def test_token_slots_mark_the_tokens_of_penalised_requests():
    e = lambda slot, n: types.SimpleNamespace(slot=slot, tokens=[0] * n)
    assert Sampler.token_slots([e(0, 1), e(3, 2), e(1, 3)], {3, 0}) == [1, 4, 4, 0, 0, 0]
    assert Sampler.token_slots([], {1}) == []
