"""CPU tests of the stand-alone tools: hostfile ordering and the plugin's CUDA-linkage rule."""
import json
import subprocess
import sys


def test_hostfile_is_grouped_by_network_nodes(tmp_path):
    from aws_ofi_nccl_b200.utils import hostfile_topologify as ht

    topo = {"Instances": [
        {"InstanceId": "i-1", "PrivateDnsName": "ip-10-0-0-1.ec2.internal", "NetworkNodes": ["nn-a", "nn-s1", "nn-l1"]},
        {"InstanceId": "i-2", "PrivateDnsName": "ip-10-0-0-2.ec2.internal", "NetworkNodes": ["nn-a", "nn-s2", "nn-l3"]},
        {"InstanceId": "i-3", "PrivateDnsName": "ip-10-0-0-3.ec2.internal", "NetworkNodes": ["nn-a", "nn-s1", "nn-l1"]},
        {"InstanceId": "i-4", "PrivateDnsName": "ip-10-0-0-4.ec2.internal", "NetworkNodes": ["nn-a", "nn-s1", "nn-l2"]},
        {"InstanceId": "i-5", "PrivateDnsName": "ip-10-0-0-5.ec2.internal", "NetworkNodes": ["nn-a", "nn-s2", "nn-l3"]},
    ]}
    tfile = tmp_path / "topo.json"
    tfile.write_text(json.dumps(topo))
    hosts = tmp_path / "hostfile"
    hosts.write_text("# job 42\nip-10-0-0-1 slots=8\nip-10-0-0-2 slots=8\nip-10-0-0-3 slots=8\nunknown-host slots=8\n"
                     "ip-10-0-0-4 slots=8\nip-10-0-0-5 slots=8\n")
    out = tmp_path / "sorted"
    res = subprocess.run([sys.executable, "-m", "aws_ofi_nccl_b200.utils.hostfile_topologify", "--input", str(hosts),
                          "--output", str(out), "--topology", str(tfile)], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    got = [ln.split()[0] for ln in out.read_text().splitlines()]
    # same leaf together, leaves of one spine together, unknown hosts last, slots kept
    assert got == ["ip-10-0-0-1", "ip-10-0-0-3", "ip-10-0-0-4", "ip-10-0-0-2", "ip-10-0-0-5", "unknown-host"]
    assert all("slots=8" in ln for ln in out.read_text().splitlines())
    table = ht.load_topology(str(tfile))
    assert ht.crossings(got[:5], table) == 2 < ht.crossings(["ip-10-0-0-1", "ip-10-0-0-2", "ip-10-0-0-3", "ip-10-0-0-4", "ip-10-0-0-5"], table)


def test_plugin_links_no_cuda_library_and_imports_no_cuda_symbol(built):
    """The plugin must load on a machine without a GPU driver: nothing of libcuda / libcudart may be
    linked or imported (everything goes through dlopen + cuGetProcAddress), and no dynamic C++
    run-time either (a second libstdc++ next to NCCL's crashed)."""
    so = built / "libnccl-net-ofi-b200.so"
    needed = subprocess.run(["readelf", "-d", str(so)], capture_output=True, text=True).stdout
    libs = [ln.split("[")[1].rstrip("]") for ln in needed.splitlines() if "(NEEDED)" in ln]
    assert not [l for l in libs if l.startswith(("libcuda", "libcudart", "libnccl", "libstdc++"))], libs
    undefined = subprocess.run(["nm", "-D", "--undefined-only", str(so)], capture_output=True, text=True).stdout
    bad = [ln.split()[-1] for ln in undefined.splitlines() if ln.split() and ln.split()[-1].split("@")[0].startswith(("cu", "nccl"))
           and not ln.split()[-1].startswith("__cu")]
    assert not bad, bad
