"""Instance topology for PD deployments on one box: which process serves which role on which GPUs and where its
control endpoint listens.  Plays the part of the reference's rank tables (omni/accelerators/pd/ranktable/*.py,
tools/scripts/pd_ranktable_tools.py) - no device IP addresses are needed on an NVSwitch domain."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass
class Instance:
    name: str
    role: str                  # prefill | decode | mixed
    gpus: list
    api_port: int
    control_port: int
    host: str = "127.0.0.1"
    cluster_id: int = 0

    @property
    def control_endpoint(self) -> str:
        return f"tcp://{self.host}:{self.control_port}"


@dataclass
class Topology:
    instances: list = field(default_factory=list)

    def by_role(self, role: str) -> list:
        return [i for i in self.instances if i.role == role]

    def to_json(self) -> str:
        return json.dumps({"instances": [asdict(i) for i in self.instances]}, indent=1)

    @classmethod
    def from_json(cls, text: str) -> "Topology":
        d = json.loads(text)
        return cls([Instance(**i) for i in d.get("instances", [])])

    @classmethod
    def load(cls, path: str) -> "Topology":
        return cls.from_json(Path(path).read_text())

    def save(self, path: str) -> None:
        Path(path).write_text(self.to_json())


def generate(n_prefill: int, n_decode: int, gpus_per_prefill: int = 1, gpus_per_decode: int = 1, base_api_port: int = 9000,
             base_control_port: int = 5568, host: str = "127.0.0.1") -> Topology:
    """``gen`` mode of the rank-table tool: lay instances out over consecutive GPUs."""
    t = Topology()
    gpu = 0
    for i in range(n_prefill):
        t.instances.append(Instance(f"prefill-{i}", "prefill", list(range(gpu, gpu + gpus_per_prefill)), base_api_port + i,
                                    base_control_port + i, host, cluster_id=i))
        gpu += gpus_per_prefill
    for j in range(n_decode):
        t.instances.append(Instance(f"decode-{j}", "decode", list(range(gpu, gpu + gpus_per_decode)),
                                    base_api_port + 100 + j, base_control_port + 100 + j, host, cluster_id=n_prefill + j))
        gpu += gpus_per_decode
    return t


def merge(*tops: Topology) -> Topology:
    """``merge`` modes of the rank-table tool: concatenate, re-number cluster ids, reject duplicate names/ports."""
    out = Topology()
    seen = set()
    for t in tops:
        for i in t.instances:
            key = (i.host, i.api_port)
            if i.name in {x.name for x in out.instances} or key in seen:
                raise ValueError(f"duplicate instance {i.name} / port {key}")
            seen.add(key)
            out.instances.append(Instance(**{**asdict(i), "cluster_id": len(out.instances)}))
    return out
