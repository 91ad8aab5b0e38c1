"""Host-side choices of how a product is cut into blocks (no GPU needed)."""

import pytest

from enginekernel_b200.ops import kernels


@pytest.mark.parametrize("n_out,k,epi", [
    (6144, 2560, kernels.EPI_BF16), (2560, 4096, kernels.EPI_BF16), (9728, 2560, kernels.EPI_SWIGLU),
    (2560, 9728, kernels.EPI_BF16), (151936, 2560, kernels.EPI_F32), (1024, 1024, kernels.EPI_BF16),
    (4096, 12288, kernels.EPI_BF16), (128, 64, kernels.EPI_BF16), (20011, 2560, kernels.EPI_F32),
])
def test_k_split_of_the_swapped_form(n_out, k, epi):
    split = kernels.swap_k_split(n_out, k, epi)
    tiles = -(-n_out // (64 if epi == kernels.EPI_SWIGLU else 128))
    k_blocks = -(-k // 64)
    assert 1 <= split <= kernels.TC_MAX_CLUSTER
    assert split & (split - 1) == 0                        # clusters of 3, 5, 6, 7 blocks run slowly
    assert split == 1 or tiles * split <= 2 * kernels.sm_count()      # one filling of the machine
    assert split == 1 or k_blocks // split >= 8            # a block keeps a ring's worth of K


def test_the_benchmark_shape_gets_the_splits_the_profiles_name():
    assert kernels.swap_k_split(6144, 2560, kernels.EPI_BF16) == 4      # q/k/v
    assert kernels.swap_k_split(2560, 4096, kernels.EPI_BF16) == 8      # attention output
    assert kernels.swap_k_split(9728, 2560, kernels.EPI_SWIGLU) == 1    # gate/up
    assert kernels.swap_k_split(2560, 9728, kernels.EPI_BF16) == 8      # down
