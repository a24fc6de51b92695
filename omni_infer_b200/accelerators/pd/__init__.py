"""PD disaggregation: KV connector, block push, instance topology."""
from __future__ import annotations

import itertools

from .connector import ConnectorMetadata, InProcessHub, SchedulerConnector, WorkerConnector  # noqa: F401

CONNECTOR_NAME = "B200PeerPushConnectorV1"       # the reference registers "AscendHcclConnectorV1"
_ids = itertools.count()


def register() -> dict:
    """Entry point kept from the reference's ``vllm.general_plugins`` hook ``kv_connectors``."""
    return {CONNECTOR_NAME: "omni_infer_b200.accelerators.pd.connector"}


def create_connectors(kv_transfer_config: dict, block_size: int = 128, num_speculative_tokens: int = 0):
    """kv_transfer_config: {"kv_role": "kv_producer"|"kv_consumer"|"kv_both", "engine_id": str,
    "endpoint": "tcp://host:port" | "inproc://name", "transport": "inproc"|"tcp", timeouts...}."""
    c = dict(kv_transfer_config)
    role = c.get("kv_role", "kv_both")
    eid = c.get("engine_id", f"engine-{next(_ids)}")
    endpoint = c.get("endpoint", f"inproc://{eid}")
    transport = c.get("transport", "inproc" if endpoint.startswith("inproc") else "tcp")
    worker = WorkerConnector(role, eid, endpoint, transport, float(c.get("sync_timeout_s", 20.0)), int(c.get("retries", 3)),
                             float(c.get("retry_wait_s", 2.0)))
    sched = SchedulerConnector(role, eid, endpoint, block_size, num_speculative_tokens,
                               worker=worker if c.get("async_pull_kv", True) else None)
    return sched, worker
