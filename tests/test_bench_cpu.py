"""The CPU arm of bench.py (`--impl reference`) prints one JSON line with the contract's keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "2",
                          "--warmup", "3"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["higher_is_better"] is True
    assert line["value"] > 1e3 and line["ms_per_step"] > 0
    # the reference's own bench_router.py when it has been staged under oracle/_ref, else the port
    from oracle import ref_runner

    assert line["cpu_baseline"]["kind"] == ("reference" if ref_runner.available() else "port")
    assert line["cpu_baseline"]["cores"] >= 1 and line["steps"] == 2 and line["warmup"] == 3
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["gpu_launches"] == 0
    # same workload string as the GPU arm prints, so that the two lines compare like for like
    sys.path.insert(0, ROOT)
    import bench

    assert line["config"] == bench.CONFIG and line["config"]["workload"] == bench.WORKLOAD


def test_reference_runner_falls_back_to_the_port_when_nothing_is_staged(monkeypatch):
    sys.path.insert(0, ROOT)
    import bench
    from oracle import ref_runner

    monkeypatch.setattr(ref_runner, "available", lambda: False)
    r = bench.run_cpu_reference(1, 1)
    assert r["kind"] == "port" and r["value"] > 1e3 and set(r["breakdown_ms"]) == {"t_logit", "t_select", "t_pack"}


def test_non_zero_ranks_of_the_reference_arm_stay_silent():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_numa_helpers_parse_sysfs(tmp_path, monkeypatch):
    """The helpers that place pinned staging buffers next to the GPU: cpulist parsing, the sysfs walk
    with a fake tree and a fake PCI address, and the affinity context manager leaving the thread's
    affinity as it found it."""
    import os

    from moe_routers_b200 import host

    assert host.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert host.parse_cpulist("") == set()

    class FakeLib:
        def moe_device_pci_bus_id(self, device, buf, n):
            buf.value = b"0000:1B:00.0"
            return 0

    import moe_routers_b200._lib as _lib

    monkeypatch.setattr(_lib, "lib", FakeLib())
    dev_dir = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev_dir.mkdir(parents=True)
    (dev_dir / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("4-7\n")
    assert host.local_cpus("cuda:0", sysfs=str(tmp_path)) == {4, 5, 6, 7}
    (dev_dir / "numa_node").write_text("-1\n")
    assert host.local_cpus("cuda:0", sysfs=str(tmp_path)) == set()
    assert host.local_cpus("cuda:0", sysfs=str(tmp_path / "missing")) == set()

    before = os.sched_getaffinity(0)
    one = {sorted(before)[0]}
    with host.numa_local("cuda:0", cpus=one):
        assert os.sched_getaffinity(0) == one
    assert os.sched_getaffinity(0) == before
    with host.numa_local("cuda:0", cpus={10 ** 6}):  # not in the allowed set: nothing changes
        assert os.sched_getaffinity(0) == before
