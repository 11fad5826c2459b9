"""Reorder a hostfile so that ranks that are adjacent in the file are close in the network.

    python -m aws_ofi_nccl_b200.utils.hostfile_topologify --input hostfile --output hostfile.sorted \
        [--topology topology.json]

The topology is a list of instances with their network nodes from the outermost layer to the one
nearest the instance, in the shape `aws ec2 describe-instance-topology` prints:

    {"Instances": [{"InstanceId": "i-0a", "NetworkNodes": ["nn-1", "nn-7", "nn-42"]}, ...]}

together with the private DNS name or IP of each instance ("PrivateDnsName" / "PrivateIpAddress" /
"Hostname", any of them) that the hostfile uses.  Without --topology the tool asks EC2 through boto3
(DescribeInstances + DescribeInstanceTopology) when boto3 and credentials are available.  Hosts are
sorted by their network-node path, which places instances under the same leaf next to each other,
then leaves under the same spine, and so on; hosts the topology does not know keep their relative
order at the end.  Ring and tree collectives over consecutive ranks then cross as few upper-layer
links as possible (reference: contrib/scripts/topology_aware/hostfile-topologify.py).
"""
from __future__ import annotations

import argparse
import json
import sys


def load_topology(path: str) -> dict[str, list[str]]:
    """host name or address -> network nodes (outermost first)."""
    with open(path) as f:
        doc = json.load(f)
    out: dict[str, list[str]] = {}
    for inst in doc.get("Instances", doc if isinstance(doc, list) else []):
        nodes = list(inst.get("NetworkNodes", []))
        for key in ("Hostname", "PrivateDnsName", "PrivateIpAddress", "InstanceId"):
            name = inst.get(key)
            if name:
                out[str(name)] = nodes
                out.setdefault(str(name).split(".")[0], nodes)   # short host name
    return out


def query_ec2(hosts: list[str]) -> dict[str, list[str]]:
    """Ask EC2 for the topology of the instances behind `hosts` (private DNS names or IPs)."""
    try:
        import boto3
    except ImportError as e:
        raise SystemExit("no --topology file given and boto3 is not installed") from e
    ec2 = boto3.client("ec2")
    by_id: dict[str, str] = {}
    for flt in ("private-dns-name", "private-ip-address"):
        for i in range(0, len(hosts), 100):
            page = ec2.describe_instances(Filters=[{"Name": flt, "Values": hosts[i:i + 100]}])
            for res in page.get("Reservations", []):
                for inst in res.get("Instances", []):
                    name = inst.get("PrivateDnsName") if flt == "private-dns-name" else inst.get("PrivateIpAddress")
                    if name:
                        by_id[inst["InstanceId"]] = name
    out: dict[str, list[str]] = {}
    ids = list(by_id)
    for i in range(0, len(ids), 100):
        page = ec2.describe_instance_topology(InstanceIds=ids[i:i + 100])
        for inst in page.get("Instances", []):
            out[by_id[inst["InstanceId"]]] = list(inst.get("NetworkNodes", []))
    return out


def topologify(hosts: list[str], topo: dict[str, list[str]]) -> list[str]:
    known = [(topo.get(h) or topo.get(h.split(".")[0]), i, h) for i, h in enumerate(hosts)]
    placed = sorted((k for k in known if k[0]), key=lambda k: (k[0], k[1]))
    unknown = [k for k in known if not k[0]]
    return [h for _, _, h in placed] + [h for _, _, h in unknown]


def crossings(hosts: list[str], topo: dict[str, list[str]]) -> int:
    """Number of adjacent pairs in the file that do not share their nearest network node."""
    n = 0
    for a, b in zip(hosts, hosts[1:]):
        pa, pb = topo.get(a) or topo.get(a.split(".")[0]), topo.get(b) or topo.get(b.split(".")[0])
        if not pa or not pb or pa[-1] != pb[-1]:
            n += 1
    return n


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    ap.add_argument("--input", required=True, help="hostfile, one host per line (slots / comments after the name are kept)")
    ap.add_argument("--output", help="sorted hostfile (default: standard output)")
    ap.add_argument("--topology", help="JSON in the shape of `aws ec2 describe-instance-topology`")
    args = ap.parse_args(argv)
    with open(args.input) as f:
        lines = [ln.rstrip("\n") for ln in f if ln.strip() and not ln.lstrip().startswith("#")]
    names = [ln.split()[0] for ln in lines]
    topo = load_topology(args.topology) if args.topology else query_ec2(names)
    order = topologify(names, topo)
    line_of = {}
    for name, ln in zip(names, lines):
        line_of.setdefault(name, []).append(ln)
    text = "\n".join(line_of[h].pop(0) for h in order) + "\n"
    if args.output:
        with open(args.output, "w") as f:
            f.write(text)
    else:
        sys.stdout.write(text)
    print(f"adjacent pairs on different leaf nodes: {crossings(names, topo)} -> {crossings(order, topo)}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
