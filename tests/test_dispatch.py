"""Which matrix-product kernel the operations layer picks for a size (no GPU needed: the choice is a function of
the sizes, the dtypes and the options)."""
import torch

from synaptix_b200 import ops

BF = torch.bfloat16


def pick(M, N, K, dtype=BF):
    return ops._weight_stream_kernel(M, N, K, dtype, dtype)


def test_weight_streaming_kernel_by_rows_and_size():
    qkv, o, gate_up, down, head = (6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728), (151936, 2560)
    for shape in (qkv, o, gate_up, down, head):
        assert pick(1, *shape) == "skinny"                                        # one row: mma.sync throughout
    for M in (2, 3, 8):
        assert pick(M, *qkv) == "ws" and pick(M, *gate_up) == "ws" and pick(M, *down) == "ws"
        assert pick(M, *o) == "skinny"                                            # under 15 M elements
        assert pick(M, *head) == "skinny"                                         # more outputs than the tcgen05 stream takes
    for M in (9, 16):
        assert all(pick(M, *s) == "ws" for s in (qkv, o, gate_up, down))
        assert pick(M, *head) == "skinny"
    for M in (17, 64, 128, 144, 160):
        assert all(pick(M, *s) == "ws" for s in (qkv, o, gate_up, down))
        assert pick(M, *head) is None                                             # the persistent tcgen05 product
    assert pick(161, *qkv) is None


def test_sizes_and_dtypes_the_fast_products_refuse():
    assert pick(8, 64, 100) is None                      # K no multiple of 8: the plain product
    assert pick(8, 64, 72) == "ws"                       # K a multiple of 8 but not of 32: only the tcgen05 stream
    assert pick(1, 64, 72) == "ws"
    assert pick(8, 64, 64, torch.float32) is None        # the 32-bit path has its own kernels
    with ops.options(gemm_ws=False):
        assert pick(8, 19456, 2560) == "skinny" and pick(64, 19456, 2560) is None and pick(8, 64, 72) is None


def test_which_products_add_themselves_into_the_residual_stream():
    assert not ops.residual_product_fusable(1, 2560, 4096, BF) and not ops.residual_product_fusable(1, 2560, 9728, BF)
    assert all(ops.residual_product_fusable(M, 2560, 4096, BF) for M in (2, 3, 8, 16, 17, 64, 128, 160))
    assert ops.norm_fusable(1, 2560, BF) and not ops.norm_fusable(2, 2560, BF)
    assert not ops.residual_product_fusable(161, 2560, 4096, BF)
    assert not ops.residual_product_fusable(8, 2560, 4096, torch.float32)
    with ops.options(fused_residual=False):
        assert not ops.residual_product_fusable(8, 2560, 4096, BF)


def test_the_tile_product_splits_uniformly_only_a_handful_of_tiles():
    """``plan_splits`` (the two-kernel form of the tcgen05 product): one row of tiles that leaves SMs idle, or up to a
    dozen tiles; several rows of more tiles run whole (or cut by the persistent kernel)."""
    from synaptix_b200.ops.gemm_tc import plan_splits
    assert plan_splits(64, 2560, 4096, 148) > 1            # 10 tiles of 256 columns
    assert plan_splits(200, 1000, 3072, 148) > 1           # 8 tiles in two rows
    assert plan_splits(512, 2560, 4096, 148) == 1          # 40 tiles in four rows
    assert plan_splits(256, 6144, 2560, 148) == 1
    assert plan_splits(2048, 2560, 4096, 148) == 1         # more tiles than three quarters of the SMs
    assert plan_splits(64, 151936, 2560, 148) == 1
