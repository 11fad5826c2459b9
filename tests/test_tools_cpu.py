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


def test_calibration_table_feeds_the_measured_tuner(built, tmp_path, monkeypatch):
    """tuner_calibrate merges the per-(algorithm, protocol) jobs into the table format the plugin's
    measured tuner parses; the jobs themselves (torchrun on GPUs) are replaced by canned timings in
    which Ring/LL wins below 64 KiB and Ring/Simple above."""
    from aws_ofi_nccl_b200.utils import tuner_calibrate as tc

    def fake_run(cmd, env=None, cwd=None, timeout=600.0):
        """Stands in for utils.proc.run_job: (returncode, stdout, stderr)."""
        algo, proto = env["NCCL_ALGO"], env["NCCL_PROTO"]
        if algo != "Ring":
            return 1, "", ""   # "not available here"
        rows = []
        for size in (1 << 10, 1 << 14, 1 << 18, 1 << 22, 1 << 26):
            if proto == "LL":
                t = 10.0 + size / 20e3      # low latency, poor bandwidth (us)
            elif proto == "Simple":
                t = 30.0 + size / 300e3     # high latency, good bandwidth
            else:
                continue
            rows.append({"coll": tc.COLLS["all_reduce"], "bytes": size, "time_us": t})
        return 0, "noise\nCALIBRATION_ROWS " + json.dumps(rows) + "\n", ""

    monkeypatch.setattr(tc, "run_job", fake_run)
    table = tmp_path / "measured.json"
    assert tc.main(["--gpus", "8", "--out", str(table), "--algos", "Ring", "Tree", "--protos", "LL", "Simple"]) == 0
    doc = json.loads(table.read_text())
    assert doc["world"] == 8 and len(doc["rows"]) == 10
    assert {(r["algo"], r["proto"]) for r in doc["rows"]} == {(tc.ALGOS["Ring"], tc.PROTOS["LL"]), (tc.ALGOS["Ring"], tc.PROTOS["Simple"])}
    monkeypatch.undo()
    res = subprocess.run([sys.executable, "-m", "aws_ofi_nccl_b200.utils.tuner_cli", "--json", "--platform", "DGX B200",
                          "--nodes", "1", "--tuner-type", "Measured", "--table", str(table), "--collectives", "all_reduce"],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr[-2000:]
    (out,) = json.loads(res.stdout)
    rows = out["collectives"]["all_reduce"]
    assert rows[0]["decision"][:2] == ["Ring", "LL"] and rows[-1]["decision"][:2] == ["Ring", "Simple"]
    # the crossover of the two canned cost lines is at 20 us * (1 / (1/20e3 - 1/300e3)) = 428 571 bytes
    switch = next(r["from_bytes"] for r in rows if r["decision"][1] == "Simple")
    assert 64 << 10 < switch < 4 << 20


def test_packaging_install_steps_produce_a_loadable_plugin(built, tmp_path):
    """The install steps of the Debian rules file and of the RPM spec, run against the built tree
    into a scratch root: the shared object and the two names NCCL searches for land in the library
    directory, and a C program can dlopen the plugin through the installed `libnccl-net.so` name."""
    import ctypes
    import os
    import re
    import subprocess

    repo = REPO if "REPO" in globals() else os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    work = tmp_path / "tree"
    work.mkdir()
    os.symlink(os.path.join(repo, "aws-ofi-nccl_b200"), work / "aws-ofi-nccl_b200")
    # Debian: the override_dh_auto_install target, with the variable dpkg-buildpackage exports
    res = subprocess.run(["make", "-f", os.path.join(repo, "contrib", "debian", "rules"), "override_dh_auto_install",
                          "DEB_HOST_MULTIARCH=x86_64-linux-gnu"], cwd=work, capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    libdir = work / "debian" / "libnccl-net-ofi-b200" / "usr" / "lib" / "x86_64-linux-gnu"
    for name in ("libnccl-net-ofi-b200.so", "libnccl-net.so", "libnccl-tuner-ofi-b200.so"):
        assert (libdir / name).exists(), name
    assert os.readlink(libdir / "libnccl-net.so") == "libnccl-net-ofi-b200.so"
    lib = ctypes.CDLL(str(libdir / "libnccl-net.so"))
    assert hasattr(lib, "ncclNetPlugin_v11") and hasattr(lib, "ncclTunerPlugin_v6")
    # RPM: the %install section with its macros expanded by hand
    spec = open(os.path.join(repo, "contrib", "fedora", "aws-ofi-nccl-b200.spec")).read()
    install = spec[spec.index("%install") + len("%install"):spec.index("%files")]
    root = tmp_path / "buildroot"
    script = install.replace("%{buildroot}", str(root)).replace("%{_libdir}", "/usr/lib64")
    assert "%{" not in script, script
    res = subprocess.run(["sh", "-ec", script], cwd=work, capture_output=True, text=True, timeout=60)
    assert res.returncode == 0, res.stdout + res.stderr
    listed = re.findall(r"^%\{_libdir\}/(\S+)$", spec[spec.index("%files"):], flags=re.M)
    assert sorted(listed) == sorted(os.listdir(root / "usr" / "lib64"))


def test_parameter_listing_comes_from_the_library_and_the_committed_table_matches(built):
    """`utils.params` asks the built library for its parameters: an environment override shows up
    with its source, the compatibility prefix of the reference works, and docs/PARAMETERS.md is the
    tool's own markdown output."""
    import json
    import os
    import subprocess
    import sys

    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, B200NET_COPY_BATCH_DEPTH="3", OFI_NCCL_EAGER_MAX_SIZE="4096")
    env.pop("B200NET_EAGER_MAX_SIZE", None)
    out = subprocess.run([sys.executable, "-m", "aws_ofi_nccl_b200.utils.params", "--json"], cwd=repo, env=env,
                         capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    rows = {r["name"]: r for r in json.loads(out.stdout)}
    assert len(rows) > 40
    assert rows["COPY_BATCH_DEPTH"]["value"] == "3" and rows["COPY_BATCH_DEPTH"]["source"] == "environment"
    assert rows["EAGER_MAX_SIZE"]["value"] == "4096" and rows["EAGER_MAX_SIZE"]["source"] == "environment"
    assert rows["COPY_BATCH"]["source"] == "default" and rows["COPY_BATCH"]["doc"]
    clean = {k: v for k, v in os.environ.items() if not k.startswith(("B200NET_", "OFI_NCCL_"))}
    md = subprocess.run([sys.executable, "-m", "aws_ofi_nccl_b200.utils.params", "--markdown"], cwd=repo, env=clean,
                        capture_output=True, text=True, timeout=60)
    assert md.returncode == 0, md.stderr
    committed = open(os.path.join(repo, "docs", "PARAMETERS.md")).read()
    assert md.stdout.strip() in committed, "docs/PARAMETERS.md is stale: regenerate it with utils.params --markdown"


def test_channel_sweep_rows_become_a_measured_table():
    """bench_plugin rows per forced channel count -> rows of the measured tuner's table: collective
    ids of the ABI, algorithm / protocol left open, failed checks and all_to_all dropped."""
    from aws_ofi_nccl_b200.utils import tuner_calibrate as tc

    per = {2: [{"coll": "all_reduce", "bytes": 1 << 20, "us": 123.44, "busbw_GBs": 1.0, "correct": True},
               {"coll": "all_to_all", "bytes": 1 << 20, "us": 50.0, "busbw_GBs": 1.0, "correct": True}],
           8: [{"coll": "all_gather", "bytes": 1 << 20, "us": 67.0, "busbw_GBs": 1.0, "correct": True},
               {"coll": "reduce_scatter", "bytes": 1 << 20, "us": 66.0, "busbw_GBs": 1.0, "correct": False}]}
    table = tc.plugin_rows_to_table(2, per)
    assert table["world"] == 2
    assert table["rows"] == [
        {"coll": 4, "algo": -1, "proto": -1, "nchannels": 2, "bytes": 1 << 20, "time_us": 123.4},
        {"coll": 2, "algo": -1, "proto": -1, "nchannels": 8, "bytes": 1 << 20, "time_us": 67.0}]
