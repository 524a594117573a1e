"""xoroshiro128++ restated with Python integers (test infrastructure only).

Follows sklearn_numba_dpex/common/random.py:
  * SplitMix64 seeding of state 0 ................ random.py:198-203, 245-249
  * 2**64 jump between consecutive states ........ random.py:205-231, 256-261
  * next(): rotl 17 / 49 / 28, shift 21 .......... random.py:275-292
  * uint64 -> [0, 1) float32 / float64 ........... random.py:78-104
  * seed drawn from a numpy RandomState .......... random.py:156-157
"""
import numpy as np

_M64 = (1 << 64) - 1


def _rotl(x, k):
    return ((x << k) & _M64) | (x >> (64 - k))


def _splitmix64_next(state):
    state = (state + 0x9E3779B97F4A7C15) & _M64
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return state, z ^ (z >> 31)


class Xoroshiro128ppStates:
    """`n_states` generators, state i+1 being state i advanced by 2**64 steps."""

    def __init__(self, n_states, seed, subsequence_start=0):
        if hasattr(seed, "randint"):
            seed = int(seed.randint(0, np.iinfo(np.int64).max - 1))
        seed = int(seed) & _M64
        self.states = []
        if n_states < 1:
            return
        sm, s0 = _splitmix64_next(seed)
        _, s1 = _splitmix64_next(sm)
        self.states.append([s0, s1])
        for _ in range(subsequence_start):
            self._jump(0)
        for idx in range(1, n_states):
            self.states.append(list(self.states[idx - 1]))
            self._jump(idx)

    def next(self, idx=0):
        s0, s1 = self.states[idx]
        result = (_rotl((s0 + s1) & _M64, 17) + s0) & _M64
        s1 ^= s0
        self.states[idx][0] = _rotl(s0, 49) ^ s1 ^ ((s1 << 21) & _M64)
        self.states[idx][1] = _rotl(s1, 28)
        return result

    def _jump(self, idx):
        a0 = a1 = 0
        for const in (0x2BD7A6A6E99C2DDC, 0x0992CCAF6A6FCA05):
            for b in range(64):
                if const & (1 << b):
                    a0 ^= self.states[idx][0]
                    a1 ^= self.states[idx][1]
                self.next(idx)
        self.states[idx][0] = a0
        self.states[idx][1] = a1

    def uniform(self, idx, dtype):
        return uint64_to_unit_float(self.next(idx), dtype)

    def as_array(self):
        return np.array(self.states, dtype=np.uint64).reshape(-1, 2)


def uint64_to_unit_float(x, dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return np.float32(x >> 40) * (np.float32(1) / np.float32(1 << 24))
    if dtype == np.float64:
        return np.float64(x >> 11) * (np.float64(1) / np.float64(1 << 53))
    raise ValueError(f"Expected float32 or float64 but got {dtype}")
