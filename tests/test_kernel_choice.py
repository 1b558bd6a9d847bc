"""Which product kernel a shape goes to (pure host-side decisions, no GPU): the table that the
measurements in the kernels' doc strings led to."""
import pytest

from gguf2bin_b200.kernels_bf16 import _normed_loses, _tc_shape, _wstream_case


@pytest.mark.parametrize("M,N,K,want", [
    # big weights (N and K of 2,048 and more): from 9 to 64 rows; narrow outputs up to 96 rows
    (8, 4096, 4096, False), (9, 4096, 4096, True), (64, 6144, 4096, True), (128, 24576, 4096, False),
    (65, 24576, 4096, False), (65, 4096, 12288, True), (96, 5120, 5120, True), (97, 4096, 12288, False),
    (129, 4096, 4096, False), (64, 151936, 4096, True),
    # ... unless the matrix is small
    (16, 4096, 2048, False), (17, 4096, 2048, True), (32, 2048, 2048, False), (33, 2048, 2048, True),
    (16, 12288, 2048, True),
    # up to 8 rows: only the largest matrices (a vocabulary is one) or a very long K
    (8, 5120, 17408, True), (1, 2048, 6144, True), (4, 19456, 2560, True), (8, 4096, 12288, True),
    (8, 2560, 4096, False), (8, 6144, 4096, False), (1, 4096, 2048, False), (8, 151936, 4096, True), (1, 151936, 2048, True),
    # a small model's layers: from 17 rows; narrow outputs except the short one at up to 32 rows
    (16, 1024, 3072, False), (32, 1024, 2048, False), (32, 1024, 3072, True), (64, 1024, 2048, True),
    (128, 1024, 3072, True),
    # wide outputs with a short K: up to 48 rows, or up to 64 rows and 4,096 outputs
    (48, 6144, 1024, True), (64, 4096, 1024, True), (64, 6144, 1024, False), (96, 4096, 1024, False),
    # a vocabulary with a short K: from 9 to 64 rows; shapes that are too small
    (64, 151936, 1024, True), (9, 151936, 1024, True), (8, 151936, 1024, False), (65, 151936, 1024, False),
    (64, 512, 4096, False), (64, 4096, 512, False),
])
def test_which_few_row_products_split_k_over_a_cluster(M, N, K, want):
    assert _wstream_case(M, N, K) is want


def test_tile_shape_of_a_few_row_product():
    assert _tc_shape(64, 4096, None, 4096) == (0, 0, 3)             # the cluster kernel picks its own shape
    assert _tc_shape(100, 151936, None, 1024) == (128, 3, False)    # a vocabulary beyond 64 rows: wide tiles, one per CTA
    assert _tc_shape(100, 4096, None, 1024) == (64, 8, False)


@pytest.mark.parametrize("M,N,K,want", [
    (8, 6144, 4096, False), (8, 24576, 4096, True), (8, 34816, 5120, True), (1, 12288, 2048, False),
    (9, 6144, 4096, True), (16, 24576, 4096, True), (16, 4096, 1024, False), (8, 151936, 4096, True),
    (8, 151936, 1024, False),
])
def test_when_the_product_does_not_take_the_norm_along(M, N, K, want):
    assert _normed_loses(M, N, K) is want


def test_wide_products_of_65_to_128_rows_go_to_the_persistent_kernel():
    assert _tc_shape(100, 24576, None, 4096) == (0, 0, False)      # no output to write as tiles: the launcher's own choice
    import torch
    out = torch.empty(100, 12288, dtype=torch.bfloat16)
    if out.data_ptr() % 16 == 0:
        assert _tc_shape(100, 24576, out, 4096) == (0, 0, True)
    assert _tc_shape(100, 4096, out, 12288) == (0, 0, True)        # narrow output beyond 96 rows
    assert _tc_shape(90, 4096, out, 12288) == (0, 0, 3)


def test_prompts_of_a_thousand_rows_and_a_long_k_go_to_pairs_of_ctas():
    import torch
    out = torch.empty(8, 8, dtype=torch.bfloat16)                   # stands for an aligned output
    if out.data_ptr() % 16:
        return
    out = out.as_strided((1, 8), (8, 1))
    assert _tc_shape(2048, 6144, out, 4096) == (256, 6, 2)
    assert _tc_shape(1024, 5120, out, 17408) == (256, 6, 2)
    assert _tc_shape(1024, 4096, out, 12288) == (256, 6, 2)          # 64 tiles of 256 x 256
    assert _tc_shape(1000, 6144, out, 4096) == (0, 0, True)
    assert _tc_shape(2048, 6144, out, 1024) == (0, 0, True)          # the short K of a small model
    assert _tc_shape(2048, 1024, out, 4096) == (0, 0, True)          # few tiles: the persistent kernel may split K
