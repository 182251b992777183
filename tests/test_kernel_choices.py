"""Which product a step of few rows takes: decided on the host, so checked without a GPU."""

from kairyu_b200 import kernels


def test_few_rows_by_row_count_and_width():
    assert all(kernels.few_rows(rows) for rows in (1, 2, 8))
    assert not kernels.few_rows(0)
    # 9 to 16 rows: the weight-streaming product and its fusions only in a narrow model
    assert not kernels.few_rows(9) and not kernels.few_rows(16, 4096) and not kernels.few_rows(12, 8192)
    assert kernels.few_rows(9, 2048) and kernels.few_rows(16, 2048) and kernels.few_rows(12, 1024)
    assert not kernels.few_rows(17, 2048)
    assert kernels.SKINNY_FAST_ROWS <= kernels.SKINNY_MAX_ROWS


def test_the_gated_tcgen05_product_wants_a_large_weight():
    hidden_8b = 2 * 14336 * 4096 * 2   # gate and up of the Llama-3.1-8B shape, bytes
    hidden_1b = 2 * 8192 * 2048 * 2
    assert hidden_1b < kernels.TC5_MIN_WEIGHT_BYTES <= hidden_8b
