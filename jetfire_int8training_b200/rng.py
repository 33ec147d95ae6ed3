"""Host-side state of the stochastic-rounding generator.

Every stochastic operator call consumes one `offset`; the kernels derive the noise of element e of that call from
Philox4x32-10 with key = seed and counter = (e // 4, offset), so calls never share noise and a (seed, offset) pair
reproduces a call bit for bit.  The seed defaults to torch.initial_seed() at first use.
"""
import threading

import torch

_lock = threading.Lock()
_seed = None
_offset = 0


def manual_seed(seed, offset=0):
    global _seed, _offset
    with _lock:
        _seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        _offset = int(offset)


def get_state():
    return _seed, _offset


def next_key():
    """(seed, offset) for one stochastic operator call."""
    global _seed, _offset
    with _lock:
        if _seed is None:
            _seed = int(torch.initial_seed()) & 0xFFFFFFFFFFFFFFFF
        key = (_seed, _offset)
        _offset += 1
        return key
