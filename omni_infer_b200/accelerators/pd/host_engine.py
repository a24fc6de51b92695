"""The connector as a class of the host engine's V1 connector interface (reference: LLMDataDistConnector is a
``KVConnectorBase_V1`` split by role, omni/accelerators/pd/llmdatadist_connector_v1.py:87-181).  One object per role:
the scheduler-role object answers the scheduler's questions, the worker-role object owns the cache tensors and the
transfers; both delegate to the connector pair of this package.  Imported only when the host engine asks its connector
factory for ``B200PeerPushConnectorV1`` (or the reference's name, kept as an alias)."""
from __future__ import annotations

from typing import Any, Optional

try:
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1, KVConnectorMetadata, KVConnectorRole
except Exception:  # noqa: BLE001  (no host engine here: the class below then stands on plain objects)
    KVConnectorBase_V1, KVConnectorMetadata = object, object

    class KVConnectorRole:  # type: ignore[no-redef]
        SCHEDULER, WORKER = 0, 1

from . import create_connectors
from .connector import ConnectorMetadata


class _Meta(KVConnectorMetadata):     # what travels from the scheduler-role object to the worker-role object each step
    def __init__(self, inner: ConnectorMetadata):
        self.inner = inner


def _config_dict(kv_transfer_config) -> dict:
    """The host engine's KVTransferConfig (or a plain mapping) as the dictionary ``create_connectors`` takes."""
    if isinstance(kv_transfer_config, dict):
        return dict(kv_transfer_config)
    d = dict(getattr(kv_transfer_config, "kv_connector_extra_config", None) or {})
    for k in ("kv_role", "engine_id", "kv_rank", "kv_parallel_size"):
        v = getattr(kv_transfer_config, k, None)
        if v is not None:
            d.setdefault(k, v)
    return d


class B200PeerPushConnectorV1(KVConnectorBase_V1):
    def __init__(self, vllm_config: Any, role: Any, kv_cache_config: Any = None):
        if KVConnectorBase_V1 is not object:
            super().__init__(vllm_config, role, kv_cache_config)
        cfg = _config_dict(vllm_config.kv_transfer_config)
        block_size = int(getattr(getattr(vllm_config, "cache_config", None), "block_size", None) or 128)
        spec = getattr(vllm_config, "speculative_config", None)
        self.sched, self.worker = create_connectors(cfg, block_size, int(getattr(spec, "num_speculative_tokens", 0) or 0))
        self.connector_role = role

    # ------------------------------------------------------------------ scheduler role
    def get_num_new_matched_tokens(self, request, num_computed_tokens: int):
        return self.sched.get_num_new_matched_tokens(request, num_computed_tokens)

    def update_state_after_alloc(self, request, blocks, num_external_tokens: int) -> None:
        if num_external_tokens <= 0:
            return
        # the host engine hands over its block object; this package's scheduler keeps the ids on the request
        ids = blocks.get_block_ids()[0] if hasattr(blocks, "get_block_ids") else list(getattr(request, "block_ids", blocks) or [])
        if not getattr(request, "block_ids", None):
            request.block_ids = list(ids)
        self.sched.update_state_after_alloc(request, num_external_tokens)

    def build_connector_meta(self, scheduler_output=None):
        return _Meta(self.sched.build_connector_meta())

    def request_finished(self, request, block_ids: list):
        return self.sched.request_finished(request, block_ids)

    # ------------------------------------------------------------------ worker role
    def register_kv_caches(self, kv_caches) -> None:
        self.worker.register_kv_caches(list(kv_caches.values()) if isinstance(kv_caches, dict) else kv_caches)

    def bind_connector_metadata(self, connector_metadata) -> None:
        if KVConnectorBase_V1 is not object:
            super().bind_connector_metadata(connector_metadata)
        self.worker.bind_connector_metadata(getattr(connector_metadata, "inner", connector_metadata))

    def start_load_kv(self, forward_context=None, **kwargs) -> None:
        self.worker.start_load_kv()

    def wait_for_layer_load(self, layer_name: str) -> None:
        """Transfers complete per request, not per layer: a request only becomes runnable once all of its blocks have
        arrived (it waits in WAITING_FOR_REMOTE_KVS), so there is nothing to wait for inside a forward pass."""

    def save_kv_layer(self, layer_name: str, kv_layer, attn_metadata=None, **kwargs) -> None:
        """The prefill instance's forward pass writes its own paged cache; the push reads from there afterwards."""

    def wait_for_save(self) -> None:
        self.worker.wait_for_save()

    def get_finished(self, finished_req_ids: Optional[set] = None):
        sent, received = self.worker.get_finished(finished_req_ids)
        return (sent or None), (received or None)

    def get_block_ids_with_load_errors(self) -> set:
        return set()

    def shutdown(self) -> None:
        self.worker.close()
