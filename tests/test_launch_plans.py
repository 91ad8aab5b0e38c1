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


def test_launch_record_groups_costs_and_issues_again():
    """The record behind the per-kernel tables, without a GPU: entries keep their order, are named
    with their label, sum their costs by name, and are issued again by name."""
    from enginekernel_b200.ops import lib
    issued = []
    with lib.LaunchRecord() as rec:
        assert lib.recording()
        lib.record_library_call("library_matmul[8x4]", lambda: issued.append("a"), bytes=100, flops=64)
        lib.record_library_call("library_matmul[2x4]", lambda: issued.append("b"), bytes=10, flops=16)
        lib.record_library_call("library_matmul[8x4]", lambda: issued.append("c"), bytes=100, flops=64)
        with pytest.raises(RuntimeError):
            lib.LaunchRecord().__enter__()                 # one record at a time
    assert not lib.recording()
    lib.record_library_call("late", lambda: issued.append("x"))        # nothing is active: not kept
    assert rec.names() == ["library_matmul[8x4]", "library_matmul[2x4]"]
    assert rec.cost("library_matmul[8x4]") == {"bytes": 200, "flops": 128, "launches": 2}
    assert rec.cost() == {"bytes": 210, "flops": 144, "launches": 3}
    assert rec.issue(0, "library_matmul[8x4]") == 2 and issued == ["a", "c"]
    assert rec.issue(0) == 3 and issued == ["a", "c", "a", "b", "c"]
