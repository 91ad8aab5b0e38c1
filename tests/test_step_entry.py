"""A step entry's tokens as one host tensor: lists, tuples, tensors, and what is not a token id."""

import pytest
import torch

from enginekernel_b200.engine.runner import StepEntry


def test_tokens_are_converted_once_and_exactly():
    e = StepEntry(3, [5, 0, 151935, 7])
    t = e.token_tensor()
    assert t.dtype == torch.int64 and t.tolist() == [5, 0, 151935, 7]
    assert e.token_tensor() is t                                   # kept for the step that follows the check
    assert StepEntry(0, (9,)).token_tensor().tolist() == [9]
    assert StepEntry(0, []).token_tensor().numel() == 0
    assert StepEntry(0, torch.tensor([4, 5], dtype=torch.int32)).token_tensor().tolist() == [4, 5]
    assert StepEntry(0, range(3)).token_tensor().tolist() == [0, 1, 2]


def test_numbers_that_are_not_plain_ints_go_the_slow_way():
    assert StepEntry(0, [1.0, 2]).token_tensor().tolist() == [1, 2]
    import numpy as np
    assert StepEntry(0, list(np.array([3, 4], dtype=np.int32))).token_tensor().tolist() == [3, 4]
    with pytest.raises((ValueError, TypeError)):
        StepEntry(0, ["a"]).token_tensor()


def test_negative_and_large_ids_survive_to_the_range_check():
    t = StepEntry(0, [-1, 2 ** 40]).token_tensor()
    assert int(t.min()) == -1 and int(t.max()) == 2 ** 40
