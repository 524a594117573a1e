"""Row-wise top-k on the device (radix select).  Same call contract as the reference's
`topk` / `topk_idx` (sklearn_numba_dpex/common/topk.py:112-270); the reference leaves the
output order and the choice among tied threshold values undefined, here the output is by
descending value, ties by ascending index."""
from ..kmeans.drivers import _topk_call


def topk(array_in, k, group_sizes=None):
    """The k greatest values of each row of `array_in` (1-D or 2-D CUDA tensor).
    `group_sizes` is accepted for signature compatibility and ignored."""
    return _topk_call(array_in, int(k), True, False)[0]


def topk_idx(array_in, k, group_sizes=None):
    """int64 indices of the k greatest values of each row of `array_in`."""
    return _topk_call(array_in, int(k), False, True)[1]
