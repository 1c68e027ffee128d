"""Host-side pieces of the engine binding that need no GPU."""
import numpy as np
import torch

from ft_b200 import engine


def test_row_ranges_travel_inside_the_q_entries_table():
    q_entries = np.arange(7, dtype=np.int32)
    ranges = np.stack([np.arange(7), np.arange(7) + 3], axis=1).astype(np.int32)
    packed = engine.pack_row_ranges(q_entries, ranges)
    assert packed.dtype == np.int32 and packed.shape == (3 * 7 + 2,)
    assert packed[-2] == engine.ROW_RANGE_MAGIC and packed[-1] == 7
    t = torch.from_numpy(packed)
    for view in (t, t.clone(), t.contiguous(), torch.from_numpy(packed.copy())):
        rows, got = engine.split_q_entries(view)
        assert rows == 7
        np.testing.assert_array_equal(got.numpy(), ranges)
    # a table in the reference's format (request ids only) has no trailer, whatever its length
    for n in (0, 1, 5, 8, 23):
        rows, got = engine.split_q_entries(torch.arange(n, dtype=torch.int32))
        assert rows == n and got is None


def test_pack_row_ranges_rejects_a_mismatched_table():
    try:
        engine.pack_row_ranges(np.arange(4, dtype=np.int32), np.zeros((3, 2), dtype=np.int32))
    except ValueError:
        return
    raise AssertionError("a range table of the wrong length was accepted")


def test_range_lookup_works_on_inference_tensors():
    """A serving host decodes under torch.inference_mode(); such tensors have no version counter."""
    with torch.inference_mode():
        t = torch.arange(23, dtype=torch.int32)
        rows, got = engine.split_q_entries(t)
    assert rows == 23 and got is None
