#!/usr/bin/env python
"""What the nodes of a deployment have published in the registry: node ids and liveness, node metadata (host
pool file, SSD and remote block files), and the number of block records per node and tier. Works against every
kind of registry the configuration accepts: a ``RegistryServer`` (``tcp://host:port`` / ``ipc://path`` / host +
port) or a Redis server (``redis://[:password@]host[:port][/db]``).
(Reference counterpart: benchmarks/redis_check.py.)

    python benchmarks/registry_check.py --host redis://10.0.0.5 --password secret
    python benchmarks/registry_check.py --host tcp://10.0.0.5:6379 --json
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flexkv_b200.cache.registry import connect  # noqa: E402

TIERS = (("CPUB", "host"), ("SSDB", "ssd"), ("PCFSB", "remote files"))


def inspect(client, samples: int = 2) -> dict:
    """One dict per node: liveness record, metadata and block-record counts per tier (with a few sample records)."""
    node_keys = sorted(client.scan("node:"), key=lambda k: int(k.split(":")[1]))
    meta_keys = client.scan("meta:")
    ids = sorted({int(k.split(":")[1]) for k in node_keys} | {int(k.split(":")[1]) for k in meta_keys})
    out = {"nodes": []}
    for nid in ids:
        node = client.hgetall(f"node:{nid}")
        rec = {"node_id": nid, "alive": bool(node), "node": node,
               "meta": {k: client.hgetall(k) for k in sorted(meta_keys) if int(k.split(":")[1]) == nid}, "blocks": {}}
        for kind, name in TIERS:
            keys = client.scan(f"{kind}:block:{nid}:")
            rec["blocks"][name] = {"records": len(keys),
                                   "sample": [client.hgetall(k) for k in sorted(keys)[:samples]]}
        out["nodes"].append(rec)
    # block records of nodes that are gone (their heartbeat key expired): nobody serves them any more
    orphans = {}
    for kind, name in TIERS:
        for k in client.scan(f"{kind}:block:"):
            nid = int(k.split(":")[2])
            if nid not in ids:
                orphans.setdefault(nid, {}).setdefault(name, 0)
                orphans[nid][name] += 1
    out["records_of_unknown_nodes"] = orphans
    return out


def render(report: dict) -> str:
    lines = []
    for n in report["nodes"]:
        state = "alive" if n["alive"] else "EXPIRED (metadata or records left behind)"
        lines.append(f"node {n['node_id']}: {state}")
        for k, v in n["node"].items():
            lines.append(f"    {k} = {v}")
        for key, meta in n["meta"].items():
            lines.append(f"  {key}")
            for k, v in meta.items():
                text = str(v)
                lines.append(f"    {k} = {text if len(text) <= 100 else text[:97] + '...'}")
        for name, b in n["blocks"].items():
            lines.append(f"  {name}: {b['records']} block records")
            for s in b["sample"]:
                lines.append(f"    e.g. {s}")
    if report["records_of_unknown_nodes"]:
        lines.append(f"records of nodes without a liveness key: {report['records_of_unknown_nodes']}")
    if not report["nodes"]:
        lines.append("no node has registered")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host", default="127.0.0.1", help="redis_host of the deployment (tcp://, ipc://, redis:// or a host name)")
    ap.add_argument("--port", type=int, default=6379)
    ap.add_argument("--password", default=None)
    ap.add_argument("--samples", type=int, default=2)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    report = inspect(connect(a.host, a.port, a.password), a.samples)
    print(json.dumps(report, default=str, indent=1) if a.json else render(report))


if __name__ == "__main__":
    main()
