"""Omni-Attention KV compression."""
from __future__ import annotations

from .omni_attn import (OmniAttentionSpec, OmniAttnConfig, OmniAttnState, OmniKVCacheManager,  # noqa: F401
                        compute_omni_attn_metadata_ref, default_pattern)


def apply_omni_attn_patch(engine, config: dict, is_kv_consumer: bool = True) -> None:
    """Switch an engine to Omni-Attention (reference entry: omni/accelerators/cache/__init__.py:28-69): replaces the
    KV manager by the two-pool manager, re-allocates compressed layers' caches as per-request windows, and makes
    the runner build window metadata.  Decode then runs eagerly (the window tables are not part of the captured
    graphs) and speculative decoding is not combined with it."""
    runner = engine.worker.runner
    if runner.tpr != 1:
        raise ValueError("Omni-Attention is not combined with speculative decoding here")
    if engine.cfg.enable_chunked_prefill or engine.cfg.enable_prefix_caching:
        # A later chunk (or a request that starts from cached blocks) attends over what earlier tokens left in the cache.
        # A compressed layer keeps only its window of them, so the result would differ from a prefill that sees the whole
        # prompt at once - which is what the layer pattern was chosen for.  The reference runs Omni-Attention on decode
        # instances, whose prompts are prefilled elsewhere (omni/accelerators/cache/__init__.py:28-69).
        raise ValueError("Omni-Attention cannot be combined with chunked prefill or prefix caching")
    n_layers = runner.model.num_kv_layers
    cfg = OmniAttnConfig.from_dict(config, n_layers)
    state = OmniAttnState(cfg, engine.cfg.block_size)
    n_window = engine.cfg.max_num_seqs * state.spec.blocks_per_request + 1
    runner.enable_omni_attn(state, n_window)
    engine.kv = OmniKVCacheManager(engine.kv.num_blocks, engine.cfg.block_size, state.spec, n_window)
