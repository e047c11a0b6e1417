"""Helpers shared by the tensor classes (python/src/gelib/gelib_common.py:15-20 of GElib)."""


def common_batch(x, y):
    """Batch size of a binary operation: equal batches, or one of them 1 (broadcast)."""
    assert x.dim() >= 1
    assert y.dim() >= 1
    if x.size(0) > 1 and y.size(0) > 1:
        assert x.size(0) == y.size(0)
    return max(x.size(0), y.size(0))
