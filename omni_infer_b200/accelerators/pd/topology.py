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

    def control_endpoints(self, role=None) -> set:
        """Control endpoints of the instances (of one role): who a KV exchange may come from or go to."""
        return {i.control_endpoint for i in self.instances if role is None or i.role == role}

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


def from_env(var: str = "OMNI_TOPOLOGY"):
    """The deployment's table named by the environment (set by the launchers and the playbook), or None.  An unreadable
    file is reported and treated as absent: the table restricts who may exchange KV, it is not needed to run."""
    import logging
    import os
    path = os.environ.get(var, "")
    if not path:
        return None
    try:
        return Topology.load(path)
    except (OSError, ValueError, TypeError, KeyError) as e:
        logging.getLogger("omni_infer_b200.pd").warning("topology file %s is unreadable (%s): not used", path, e)
        return None


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


def main(argv=None) -> int:
    """Command line of the tool, with the reference's option names (tools/scripts/pd_ranktable_tools.py:43-70):

        python -m omni_infer_b200.accelerators.pd.topology --mode gen --prefill-server-list 0,1 2,3 \
               --decode-server-list 4,5,6,7 --save-dir tables/
        python -m omni_infer_b200.accelerators.pd.topology --mode merge --global-ranktable-list a.json b.json --save-dir tables/

    ``gen`` takes one GPU list per instance (all prefill instances must have the same size, and all decode instances:
    they are the tensor-parallel width) and writes ``global_topology.json`` plus one ``local_<name>.json`` per instance;
    ``merge`` (also ``merge-local`` / ``merge-all``) concatenates tables into one."""
    import argparse
    import os

    ap = argparse.ArgumentParser(description=main.__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--mode", default="gen", choices=["gen", "merge", "merge-local", "merge-all"])
    ap.add_argument("--api-server", action="store_true", help="accepted for compatibility: every instance has an API server here")
    ap.add_argument("--prefill-server-list", nargs="*", default=[])
    ap.add_argument("--decode-server-list", nargs="*", default=[])
    ap.add_argument("--save-dir", default="./")
    ap.add_argument("--global-ranktable-list", nargs="*", default=[])
    ap.add_argument("--local-ranktable-list", nargs="*", default=[])
    ap.add_argument("--base-api-port", type=int, default=9000)
    ap.add_argument("--base-control-port", type=int, default=5568)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--index-offset", type=int, default=0,
                    help="first instance number of this call's names (a table per host, merged later, needs distinct names)")
    a = ap.parse_args(argv)
    os.makedirs(a.save_dir, exist_ok=True)
    if a.mode == "gen":
        pre = [[int(x) for x in s.split(",") if x != ""] for s in a.prefill_server_list]
        dec = [[int(x) for x in s.split(",") if x != ""] for s in a.decode_server_list]
        for name, group in (("prefill", pre), ("decode", dec)):
            if len({len(g) for g in group}) > 1:
                raise SystemExit(f"every {name} instance must span the same number of GPUs (its tensor-parallel size)")
        used = [g for grp in pre + dec for g in grp]
        if len(used) != len(set(used)):
            raise SystemExit("a GPU is listed for more than one instance")
        t = Topology()
        for i, g in enumerate(pre):
            t.instances.append(Instance(f"prefill-{a.index_offset + i}", "prefill", g, a.base_api_port + i, a.base_control_port + i,
                                        a.host, cluster_id=i))
        for j, g in enumerate(dec):
            t.instances.append(Instance(f"decode-{a.index_offset + j}", "decode", g, a.base_api_port + 100 + j,
                                        a.base_control_port + 100 + j, a.host,
                                        cluster_id=len(pre) + j))
        t.save(os.path.join(a.save_dir, "global_topology.json"))
        for inst in t.instances:
            Topology([inst]).save(os.path.join(a.save_dir, f"local_{inst.name}.json"))
        print(json.dumps({"instances": len(t.instances), "saved": os.path.join(a.save_dir, "global_topology.json")}))
        return 0
    files = list(a.global_ranktable_list) + list(a.local_ranktable_list)
    if not files:
        raise SystemExit("merge needs --global-ranktable-list and / or --local-ranktable-list")
    merged = merge(*[Topology.load(f) for f in files])
    out = os.path.join(a.save_dir, "global_topology.json")
    merged.save(out)
    print(json.dumps({"instances": len(merged.instances), "saved": out}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
