"""Cache of prepared (split / packed) weight forms for the tensor-core kernels, shared by the SO3Linear,
dense and radial-chain front-ends.  Keyed on the weight tensors' storage address and version, so an in-place
update or a new tensor invalidates the entry; an entry keeps its weight tensors alive so the address cannot
be reused while it exists.  An entry remembers the stream it was built on and an event recorded behind the
build: a later call on another stream waits for that event (and tells the allocator about the new reader)
before it uses the entry.  Plays the part of the reference's plan LRU
(fasteq/ops/auto_schedule/eqlinear_plan.py:38-41, :81-100, :167-187).

Inside CUDA-graph capture a prepared form would be baked into the graph and go stale when the weights
change, so the cache is bypassed there unless the caller declares the weights frozen (``frozen_weights``)."""
from __future__ import annotations

from collections import OrderedDict
from contextlib import contextmanager
from typing import Callable, Optional, Sequence, Tuple

import torch

# key -> (weights kept alive, prepared tensor, event recorded after the build, ids of the streams ordered behind it)
_CACHE: "OrderedDict[Tuple, Tuple[tuple, torch.Tensor, torch.cuda.Event, set]]" = OrderedDict()
_BYTES = [0]
_BUDGET = [256 << 20]
_FROZEN = [0]


def set_budget(max_bytes: Optional[int]) -> None:
    _BUDGET[0] = (256 << 20) if max_bytes is None else int(max_bytes)
    if _BUDGET[0] <= 0:
        clear()


def clear() -> None:
    _CACHE.clear()
    _BYTES[0] = 0


@contextmanager
def frozen_weights():
    """Inside this block prepared weights may be used while a CUDA graph is being captured: the caller
    promises not to change the weights for as long as the graph is replayed."""
    _FROZEN[0] += 1
    try:
        yield
    finally:
        _FROZEN[0] -= 1


def snapshot() -> list:
    """References to everything cached right now (hold them to keep graph-captured pointers valid)."""
    return [v[1] for v in _CACHE.values()]


def get(weights: Sequence[torch.Tensor], tag: Tuple, build: Callable[[], Optional[torch.Tensor]]) -> Optional[torch.Tensor]:
    """The prepared form of ``weights`` for ``tag``, building it with ``build()`` on a miss; ``None`` when the
    cache must not be used (disabled, capture without ``frozen_weights``, or ``build`` declined)."""
    if _BUDGET[0] <= 0:
        return None
    capturing = torch.cuda.is_current_stream_capturing()
    if capturing and not _FROZEN[0]:
        return None
    key = tuple((w.data_ptr(), w._version, w.numel()) for w in weights) + (str(weights[0].device), tag)
    hit = _CACHE.get(key)
    if hit is not None:
        _CACHE.move_to_end(key)
        val = hit[1]
        if not capturing:
            cur = torch.cuda.current_stream(val.device)
            if cur.cuda_stream not in hit[3]:
                cur.wait_event(hit[2])
                val.record_stream(cur)
                hit[3].add(cur.cuda_stream)
        return val
    if capturing:
        return None            # nothing persistent may be allocated inside a capture
    val = build()
    if val is None:
        return None
    cur = torch.cuda.current_stream(val.device)
    done = torch.cuda.Event()
    done.record(cur)
    nbytes = val.numel() * val.element_size()
    while _CACHE and _BYTES[0] + nbytes > _BUDGET[0]:
        _, old = _CACHE.popitem(last=False)
        _BYTES[0] -= old[1].numel() * old[1].element_size()
    _CACHE[key] = (tuple(weights), val, done, {cur.cuda_stream})
    _BYTES[0] += nbytes
    return val
