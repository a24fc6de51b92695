"""Expert placement pattern handling (reference: omni_planner/expert_mapping.py:12-280).

A pattern is a 0/1 array ``[world, moe_layers, experts]`` (``.npy`` as produced by the offline tool, or the text
format of the C++ loader).  ``ExpertMapping`` validates it, owns the int32 selector tensor ``[layers, experts]`` that
the router kernel reads, and wraps the C++ ``PlacementMapping``."""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from . import _native as nat


def base_pattern(world: int, layers: int, experts: int) -> np.ndarray:
    p = np.zeros((world, layers, experts), dtype=np.int32)
    per = experts // world
    for r in range(world):
        p[r, :, r * per:(r + 1) * per] = 1
    return p


def pattern_from_placement(placement: np.ndarray, world: int, slots: int, experts: int) -> np.ndarray:
    """[layers, world*slots] expert ids (or -1) -> 0/1 pattern [world, layers, experts]."""
    layers = placement.shape[0]
    p = np.zeros((world, layers, experts), dtype=np.int32)
    for l in range(layers):
        for pos, e in enumerate(placement[l]):
            if e >= 0:
                p[pos // slots, l, e] = 1
    return p


class ExpertMapping:
    def __init__(self, pattern: Optional[np.ndarray], world: int, rank: int, layers: int, experts: int,
                 redundant_per_rank: int = 0, ranks_per_host: int = 8, device="cpu"):
        if pattern is None:
            pattern = base_pattern(world, layers, experts)
        pattern = np.ascontiguousarray(pattern, dtype=np.int32)
        if pattern.shape != (world, layers, experts):
            raise ValueError(f"pattern shape {pattern.shape} != {(world, layers, experts)}")
        if not np.isin(pattern, (0, 1)).all():
            raise ValueError("pattern entries must be 0 or 1")
        per_rank = pattern.sum(axis=2)
        if (per_rank > experts // world + redundant_per_rank).any():
            raise ValueError("pattern places more experts on a rank than it has slots")
        if (pattern.sum(axis=0) == 0).any():
            raise ValueError("pattern leaves an expert without a replica")
        self.pattern, self.world, self.rank, self.layers, self.experts = pattern, world, rank, layers, experts
        self.redundant_per_rank = redundant_per_rank
        self.device = torch.device(device)
        # the C++ side writes host memory; the device copy is refreshed after every selector update
        self._selector_host = np.zeros((layers, experts), dtype=np.int32)
        self.selector_dev = torch.zeros(layers, experts, dtype=torch.int32, device=self.device)
        L = nat.lib()
        self.handle = L.omni_pl_mapping_create(pattern.ctypes.data, world, layers, experts, rank, redundant_per_rank,
                                               ranks_per_host, None)
        if not self.handle:
            raise ValueError("the placement core rejected the pattern")
        self.slots_per_rank = L.omni_pl_mapping_slots_per_rank(self.handle)
        self.refresh_selector()

    def refresh_selector(self) -> None:
        nat.lib().omni_pl_mapping_copy_selector(self.handle, self._selector_host.ctypes.data)
        self.selector_dev.copy_(torch.from_numpy(self._selector_host), non_blocking=False)

    # ---- getters with the reference's names
    def get_num_of_redundant_experts(self, moe_layer: int = 0) -> int:
        return self.slots_per_rank * self.world - self.experts

    def expert_at(self, layer: int, global_pos: int) -> int:
        return nat.lib().omni_pl_mapping_expert_at(self.handle, layer, global_pos)

    def get_redundant_count(self, layer: int, expert: int) -> int:
        return nat.lib().omni_pl_mapping_redundant_count(self.handle, layer, expert)

    def local_slots_of(self, layer: int, expert: int) -> list:
        base = self.rank * self.slots_per_rank
        return [s for s in range(self.slots_per_rank) if self.expert_at(layer, base + s) == expert]

    def logical_of_slot(self, layer: int, slot: int) -> int:
        return self.expert_at(layer, self.rank * self.slots_per_rank + slot)

    def is_expert_on_current_rank(self, layer: int, expert: int) -> bool:
        return bool(self.local_slots_of(layer, expert))

    def placement(self) -> np.ndarray:
        P = self.world * self.slots_per_rank
        return np.array([[self.expert_at(l, p) for p in range(P)] for l in range(self.layers)], dtype=np.int32)

    def update(self, layer: int, global_pos: int, old_expert: int, new_expert: int) -> bool:
        ok = bool(nat.lib().omni_pl_mapping_update(self.handle, layer, global_pos, old_expert, new_expert))
        if ok:
            self.refresh_selector()
        return ok

    def close(self) -> None:
        if self.handle:
            nat.lib().omni_pl_mapping_destroy(self.handle)
            self.handle = None
