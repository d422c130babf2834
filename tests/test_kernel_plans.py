"""The host-side plans that pick kernel variants from a step's shape (pure Python: no GPU, no library)."""
import pytest

from glassbox_b200 import kernels


@pytest.mark.parametrize("nkv", [1, 3, 5, 32])
@pytest.mark.parametrize("context", [16, 100, 512, 1024, 4096, 8192, 65536])
def test_decode_attention_plan_keeps_its_promises(nkv, context):
    """For every batch size: at least one split; the eight-warp variant never asks for more blocks than SMs (a second
    block of eight warps does not fit beside the first) nor for more partial results per head than its merge holds at
    once; 16 keys per iteration only at head size 64; the plan depends on the shape alone."""
    for rows in list(range(1, 70)) + [128, 500]:
        splits, block_keys, warps = kernels.decode_mma_plan(rows, nkv, 64, context)
        assert splits >= 1 and warps in (4, 8) and block_keys in (0, 16)
        assert (splits, block_keys, warps) == kernels.decode_mma_plan(rows, nkv, 64, context)
        if warps == 4 and block_keys == 16:
            assert splits <= 4                                           # clusters of 5 and 7 place badly
        if warps == 8:
            assert rows * nkv * splits <= 148
            assert splits * warps <= 64
            if block_keys == 16:
                assert context <= 1024 * splits
        assert splits == 1 or splits * 128 <= max(context, 512) * 2      # no split without keys of its own
        # other head sizes have no 16-key or eight-warp variant
        s2, b2, w2 = kernels.decode_mma_plan(rows, nkv, 128, context)
        assert b2 == 0 and w2 == 4 and s2 >= 1


def test_decode_attention_plan_examples():
    """The shapes the benchmark runs (SmolLM2-135M: 3 kv heads, context 4096)."""
    assert kernels.decode_mma_plan(1, 3, 64, 4096) == (8, 16, 8)
    assert kernels.decode_mma_plan(8, 3, 64, 4096) == (6, 16, 8)
    assert kernels.decode_mma_plan(16, 3, 64, 4096) == (3, 0, 8)        # 1,365 keys a block: 32 keys per iteration
    assert kernels.decode_mma_plan(64, 3, 64, 4096) == (2, 16, 4)
    # large batches: the split count whose waves of resident blocks end soonest
    assert kernels.decode_mma_plan(8, 32, 64, 4096) == (3, 16, 4)       # 256 pairs: 2 splits would leave a short second wave
    assert kernels.decode_mma_plan(48, 3, 64, 4096) == (2, 16, 4)       # 144 pairs: 3 splits no longer fit one wave
    assert kernels.decode_mma_plan(13, 32, 64, 4096) == (1, 16, 4)      # 416 pairs fit one wave by themselves
    assert kernels.decode_mma_plan(64, 32, 64, 4096) == (1, 16, 4)
    assert kernels.decode_mma_plan(64, 5, 64, 4096) == (1, 16, 4)
