"""Partitioning of one contraction over the GPUs of a box by an external (output) mode.

A mode that lives in C and in exactly one input can be cut into `world` equal slices: every
rank contracts its slice of that input with the whole other input and owns the matching slice of
C; no rank needs anything from another, so there is no collective on the data path.  When the
cut mode is the slowest mode of the tensors that carry it, each slice is one contiguous block.
"""
from __future__ import annotations

from dataclasses import replace

import numpy as np


def shard_equation(eq, mode: str, world: int, rank: int):
    """Local descriptor of `rank` (same modes, extent[mode] / world) and the slice it owns."""
    if mode not in eq.modeC or (mode in eq.modeA) == (mode in eq.modeB):
        raise ValueError(f"mode '{mode}' is not an external mode of this contraction")
    full = int(eq.extent[mode])
    if full % world:
        raise ValueError(f"extent {full} of mode '{mode}' does not divide over {world} ranks")
    local = full // world
    ext = dict(eq.extent)
    ext[mode] = local
    return replace(eq, extent=ext), slice(rank * local, (rank + 1) * local)


def grow_equation(eq, mode: str, world: int):
    """Weak scaling: the global problem whose `mode` extent is `world` times the per-GPU one."""
    ext = dict(eq.extent)
    ext[mode] = int(ext[mode]) * world
    return replace(eq, extent=ext)


def take_slice(tensor: np.ndarray, modes: str, extent: dict, mode: str, sl: slice) -> np.ndarray:
    """Slice of a column-major tensor (flat, first mode fastest) along `mode`, again flat."""
    if mode not in modes:
        return tensor
    shape = [int(extent[m]) for m in modes][::-1]          # numpy order: slowest first
    nd = tensor.reshape(shape)
    axis = len(modes) - 1 - modes.index(mode)
    index = [slice(None)] * len(modes)
    index[axis] = sl
    return np.ascontiguousarray(nd[tuple(index)]).ravel()


def put_slice(dst: np.ndarray, part: np.ndarray, modes: str, extent: dict, mode: str, sl: slice) -> None:
    """Inverse of take_slice for the output tensor: writes `part` into dst's slice."""
    shape = [int(extent[m]) for m in modes][::-1]
    nd = dst.reshape(shape)
    axis = len(modes) - 1 - modes.index(mode)
    index = [slice(None)] * len(modes)
    index[axis] = sl
    local_shape = list(shape)
    local_shape[axis] = sl.stop - sl.start
    nd[tuple(index)] = part.reshape(local_shape)


def shard_contracted(eq, mode: str, world: int, rank: int):
    """Cut a CONTRACTED mode: every rank sums over its slice of `mode` and produces a full-size
    partial C; the partials must then be added (reduce-scatter over NVLink leaves each rank with
    1/world of C).  Returns the local descriptor and the slice of `mode` the rank owns."""
    if mode in eq.modeC or mode not in eq.modeA or mode not in eq.modeB:
        raise ValueError(f"mode '{mode}' is not a contracted mode of this contraction")
    full = int(eq.extent[mode])
    if full % world:
        raise ValueError(f"extent {full} of mode '{mode}' does not divide over {world} ranks")
    local = full // world
    ext = dict(eq.extent)
    ext[mode] = local
    return replace(eq, extent=ext), slice(rank * local, (rank + 1) * local)


def owner_range(n_elements: int, world: int, owner: int) -> slice:
    """Contracted-mode split: C is cut into `world` contiguous ranges along its slowest mode and range o
    belongs to rank o (tcontb_run_ksplit_* in include/tcontb.h).  The range as a slice of the flat tensor."""
    if n_elements % world:
        raise ValueError(f"{n_elements} elements of C do not cut into {world} equal ranges")
    n = n_elements // world
    return slice(owner * n, (owner + 1) * n)


def sum_owner_slots(slots) -> np.ndarray:
    """What an owner does with the `world` partial ranges stored into its slots: add them in rank order
    (the order is fixed, so the result does not depend on which peer's stores arrived first)."""
    out = np.array(slots[0], dtype=slots[0].dtype, copy=True)
    for part in slots[1:]:
        out += part
    return out
