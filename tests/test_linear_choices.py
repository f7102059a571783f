"""How a product is cut into k-slices (host-side decisions of parts/linear.py; no GPU needed)."""
import pytest

from vllm_cpp_b200 import ops
from vllm_cpp_b200.parts.linear import MAX_SPLIT_TOKENS, choose_splits, token_tile


def test_k_slices_fill_the_sms_of_the_benchmark_model():
    assert choose_splits(6144, 8, 4096) == 3         # decoding: 48 feature tiles x 3 = 144 units on 148 SMs
    assert choose_splits(4096, 8, 4096) == 4         # 32 x 4 = 128
    assert choose_splits(24576, 8, 4096) == 3        # 192 x 3 = 576: four rounds less a few units
    assert choose_splits(4096, 8, 12288) == 4
    assert choose_splits(6144, 256, 4096) == 3       # 48 units of 128 x 256 -> 144
    assert choose_splits(4096, 256, 12288) == 4      # 32 units -> 128
    assert choose_splits(4096, 512, 4096) == 2       # 64 units -> 128
    assert choose_splits(4096, 1024, 4096) == 1      # 128 units already
    assert choose_splits(24576, 2048, 4096) == 1


@pytest.mark.parametrize("M,K", [(6144, 4096), (4096, 12288), (151936, 4096), (896, 896), (128, 64), (300, 200)])
def test_k_slices_are_whole_and_never_empty(M, K):
    total_kb = -(-K // 64)
    for T in (1, 7, 16, 33, 64, 128, 129, 300, 512, 1000, 1024, 1025, 4096):
        s = choose_splits(M, T, K)
        assert 1 <= s <= 8
        if T > MAX_SPLIT_TOKENS:
            assert s == 1                            # units in plenty: partial sums would only cost traffic
        eff = ops.gemm_effective_splits(K, s)
        per = -(-total_kb // eff)
        assert 1 <= eff <= min(s, total_kb) and per * (eff - 1) < total_kb <= per * eff
        assert eff == 1 or per >= 8 or total_kb < 16  # no slice shorter than eight k-blocks where there is a choice


def test_token_tiles():
    assert [token_tile(t) for t in (1, 16, 17, 64, 65, 128, 129, 5000)] == [16, 16, 32, 64, 128, 128, 256, 256]
    assert ops.gemm_effective_splits(4096, 3) == 3 and ops.gemm_effective_splits(4096, 5) == 5
    assert ops.gemm_effective_splits(128, 8) == 2 and ops.gemm_effective_splits(64, 4) == 1
    assert ops.gemm_effective_splits(4096, 7) == 7   # 64 k-blocks in slices of ten: seven slices, the last one shorter
