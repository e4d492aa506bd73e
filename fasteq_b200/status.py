"""One call that reads (and clears) the device status words of every kernel family loaded in this process.

Every kernel with a bounded wait or an index check records why it gave up or what it skipped in a status word
instead of trapping (wait timed out, index outside its operand); results of that launch are then not to be used.
The words live per generated module (tensor product, symmetric contraction) and per family in the core library
(tcgen05 GEMMs and the radial chain, edge geometry).  Reading synchronises the device."""
from __future__ import annotations

from typing import Dict

import torch


def device_status() -> Dict[str, int]:
    """``{}`` when every status word is zero, else ``{kernel family or module: code}``; all words are cleared."""
    out: Dict[str, int] = {}
    if not torch.cuda.is_available():
        return out
    from .ops import uniform1d_jit as u1d
    from .ops import stc_uniform1d_jit as stc
    from .ops.dense import tensorcore_device_status
    from .ops.edge_geometry import edge_geometry_device_status
    with u1d._lock:
        mods = list(u1d._MODULES.items())
    for (spec, direction, needs, tun), mod in mods:
        code = mod.device_status()
        if code:
            out[f"u1d {direction} u={spec.u} {spec.dtype} w{spec.w_segs}/o{spec.out_segs} needs={tuple(needs)}"] = code
    for key, mod in list(stc._MODULES.items()):
        code = mod.device_status()
        if code:
            out[f"stc {key[1:]}"] = code
    for name, fn in (("tcgen05 gemm / radial chain", tensorcore_device_status), ("edge geometry", edge_geometry_device_status)):
        code = fn()
        if code:
            out[name] = code
    return out
