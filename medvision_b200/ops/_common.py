import torch


def parse_output_size(output_size, ndim, name="output_size"):
    """int -> the same size on every axis; tuple of ``ndim`` ints -> as given.  Anything else
    (a list included) is a TypeError, as in medvision/ops/roi_align_nd.py:14-26."""
    if isinstance(output_size, int):
        return (output_size,) * ndim
    if isinstance(output_size, tuple):
        assert len(output_size) == ndim
        for v in output_size:
            assert isinstance(v, int)
        return output_size
    raise TypeError(f'"{name}" must be an integer or tuple of integers')
