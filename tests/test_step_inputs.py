"""What the step function takes as a row's token ids and wanted places, before anything
reaches the device: lists, arrays or tensors of integers, laid out without a loop over the
tokens; anything that is no flat sequence of integers is refused."""
import numpy as np
import pytest
import torch

from minfer_b200.engine.step import StepError, _int_array


def test_rows_of_integers_in_every_form():
    for given in ([1, 2, 3], (1, 2, 3), np.array([1, 2, 3], dtype=np.int32),
                  torch.tensor([1, 2, 3]), [1.0, 2.0, 3.0], [np.int64(1), 2, 3]):
        got = _int_array(given, "token ids")
        assert got.dtype == np.int64 and got.tolist() == [1, 2, 3]
    assert _int_array([], "wanted places").tolist() == []


@pytest.mark.parametrize("bad", [[1.5], ["a"], [[1, 2], [3, 4]], [[1], [2, 3]], [None]])
def test_rows_that_are_no_flat_sequence_of_integers_are_refused(bad):
    with pytest.raises(StepError):
        _int_array(bad, "token ids")
