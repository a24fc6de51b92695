"""ctypes binding of ``libomni_placement.so`` (the C++ placement core in ``csrc/placement``)."""
from __future__ import annotations

import ctypes
from pathlib import Path

_PATH = Path(__file__).resolve().parents[2] / "_lib" / "libomni_placement.so"
_lib = None

COPY_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong)
ALLGATHER_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong)
SENDRECV_FN = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_ulonglong)
BARRIER_FN = ctypes.CFUNCTYPE(None)


def lib():
    global _lib
    if _lib is None:
        if not _PATH.exists():
            from ...build import build_placement
            build_placement()
        L = ctypes.CDLL(str(_PATH))
        vp, ci, cd, ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_double, ctypes.c_ulonglong
        for name, res, args in [
            ("omni_pl_mapping_create", vp, [vp, ci, ci, ci, ci, ci, ci, vp]),
            ("omni_pl_mapping_destroy", None, [vp]),
            ("omni_pl_mapping_slots_per_rank", ci, [vp]),
            ("omni_pl_mapping_expert_at", ci, [vp, ci, ci]),
            ("omni_pl_mapping_redundant_count", ci, [vp, ci, ci]),
            ("omni_pl_mapping_selector", ci, [vp, ci, ci]),
            ("omni_pl_mapping_copy_selector", None, [vp, vp]),
            ("omni_pl_mapping_update", ci, [vp, ci, ci, ci, ci]),
            ("omni_pl_weights_create", vp, [ci, ci]),
            ("omni_pl_weights_destroy", None, [vp]),
            ("omni_pl_weights_add", None, [vp, ci, ci, vp, ull]),
            ("omni_pl_weights_set_initialized", None, [vp]),
            ("omni_pl_weights_expert_bytes", ull, [vp]),
            ("omni_pl_activation_create", vp, [vp, ci, ci, ci, ci, ci]),
            ("omni_pl_activation_destroy", None, [vp]),
            ("omni_pl_activation_collect_from_txt", ci, [vp, ctypes.c_char_p]),
            ("omni_pl_activation_dump", None, [vp, ctypes.c_char_p]),
            ("omni_pl_activation_delta", ctypes.c_longlong, [vp, ci, ci]),
            ("omni_pl_distribution_create", vp, [ci, ci, ull, ALLGATHER_FN, SENDRECV_FN, BARRIER_FN]),
            ("omni_pl_distribution_create_device", vp, [ci, ci, ull, ALLGATHER_FN, SENDRECV_FN, BARRIER_FN, vp, vp]),
            ("omni_pl_distribution_destroy", None, [vp]),
            ("omni_pl_placement_create", vp, [vp, vp, vp, vp, ci, cd]),
            ("omni_pl_placement_destroy", None, [vp]),
            ("omni_pl_placement_start", None, [vp]),
            ("omni_pl_placement_stop", None, [vp]),
            ("omni_pl_placement_run_round", ci, [vp]),
            ("omni_pl_do_placement_optimizer", ci, [vp]),
            ("omni_pl_placement_rounds", ci, [vp]),
            ("omni_pl_placement_ready_rounds", ci, [vp]),
            ("omni_pl_placement_skipped", ci, [vp]),
            ("omni_pl_placement_last_instructions", ci, [vp, vp, ci]),
            ("omni_pl_weights_init_shm", ci, [vp, ctypes.c_char_p, ci, ci]),
            ("omni_pl_weights_replicate", None, [vp, vp]),
            ("omni_pl_weights_replica_complete", ci, [vp]),
            ("omni_pl_weights_replica_has", ci, [vp, ci, ci]),
            ("omni_pl_weights_replica_bytes", ull, [vp]),
            ("omni_pl_weights_close_shm", None, [vp, ci]),
            ("omni_pl_placement_get_ema", ci, [vp, vp, ci]),
            ("omni_pl_placement_set_ema", ci, [vp, vp, ci]),
            ("omni_pl_static_placement", ci, [vp, ci, ci, ci, ci, ci, vp]),
            ("omni_pl_greedy_instructions", ci, [vp, vp, ci, ci, ci, ci, ci, vp, ci]),
            ("omni_pl_static_instructions", ci, [vp, vp, ci, ci, ci, ci, ci, ci, ci, cd, vp, ci, vp]),
            ("omni_pl_set_copy_hooks", None, [COPY_FN, COPY_FN, COPY_FN]),
            ("omni_pl_set_ut_memcpy", None, []),
            ("omni_pl_unset_ut_memcpy", None, []),
        ]:
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib
