"""PD disaggregation: KV connector, block push, instance topology."""
from __future__ import annotations

import itertools

from .connector import ConnectorMetadata, InProcessHub, SchedulerConnector, WorkerConnector  # noqa: F401

CONNECTOR_NAME = "B200PeerPushConnectorV1"       # the reference registers "AscendHcclConnectorV1"
_ids = itertools.count()


COMPAT_NAMES = ("AscendHcclConnectorV1",)       # accepted so that existing kv-transfer configs keep working
_REGISTERED: dict = {}


def register() -> dict:
    """Entry point ``vllm.general_plugins`` / ``kv_connectors`` (reference: omni/accelerators/pd/__init__.py):
    registers the connector under its name (and the reference's name as an alias) in this package's table and,
    when the host engine imports, with that engine's connector factory."""
    mod, cls = "omni_infer_b200.accelerators.pd.connector", "WorkerConnector"
    for name in (CONNECTOR_NAME, *COMPAT_NAMES):
        _REGISTERED[name] = (mod, cls)
    try:
        from vllm.distributed.kv_transfer.kv_connector.factory import KVConnectorFactory
        for name in (CONNECTOR_NAME, *COMPAT_NAMES):
            if name not in getattr(KVConnectorFactory, "_registry", {}):
                # the host engine gets the class that speaks its connector interface and delegates to this package's pair
                KVConnectorFactory.register_connector(name, "omni_infer_b200.accelerators.pd.host_engine", "B200PeerPushConnectorV1")
    except Exception:  # noqa: BLE001  (no host engine: the in-repo engine uses create_connectors directly)
        pass
    return {name: mod for name in _REGISTERED}


def get_connector_class(name: str):
    """Resolve a connector name from a kv-transfer config to its class."""
    import importlib
    if not _REGISTERED:
        register()
    mod, cls = _REGISTERED[name]
    return getattr(importlib.import_module(mod), cls)


def create_connectors(kv_transfer_config: dict, block_size: int = 128, num_speculative_tokens: int = 0):
    """kv_transfer_config: {"kv_role": "kv_producer"|"kv_consumer"|"kv_both", "engine_id": str,
    "endpoint": "tcp://host:port" | "inproc://name", "transport": "inproc"|"tcp", timeouts...}."""
    c = dict(kv_transfer_config)
    role = c.get("kv_role", "kv_both")
    eid = c.get("engine_id", f"engine-{next(_ids)}")
    endpoint = c.get("endpoint", f"inproc://{eid}")
    transport = c.get("transport", "inproc" if endpoint.startswith("inproc") else "tcp")
    from .topology import from_env
    topo = from_env()
    worker = WorkerConnector(role, eid, endpoint, transport, float(c.get("sync_timeout_s", 20.0)), int(c.get("retries", 3)),
                             float(c.get("retry_wait_s", 2.0)), authkey=c.get("authkey"),
                             handover_ttl_s=float(c.get("handover_ttl_s", 120.0)),
                             known_producers=topo.control_endpoints("prefill") | topo.control_endpoints("mixed") if topo else None,
                             known_consumers=topo.control_endpoints("decode") | topo.control_endpoints("mixed") if topo else None)
    sched = SchedulerConnector(role, eid, endpoint, block_size, num_speculative_tokens,
                               worker=worker if c.get("async_pull_kv", True) else None)
    return sched, worker
