"""Node-smoke collectors, orchestrator and aggregator on recorded tool output (no GPU, nothing is changed on the host)."""
import json

from primus_b200.tools.preflight.node_smoke import collectors as C
from primus_b200.tools.preflight.node_smoke import run_node_smoke, summarize_cluster, write_report
from primus_b200.tools.preflight.node_smoke.orchestrator import node_status_from

TOPO = """\tGPU0\tGPU1\tGPU2\tNIC0\tCPU Affinity
GPU0\t X \tNV18\tNV18\tPIX\t0-55
GPU1\tNV18\t X \tNV18\tSYS\t0-55
GPU2\tNV18\tNV18\t X \tSYS\t56-111
NIC0\tPIX\tSYS\tSYS\t X
"""
TOPO_BAD = TOPO.replace("GPU2\tNV18\tNV18", "GPU2\tNV18\tSYS")


def fake_run(outputs):
    def run(cmd, timeout=20.0):
        key = " ".join(cmd)
        for k, v in outputs.items():
            if k in key:
                return v
        return ""
    return run


def test_dmesg_collector_finds_xid_and_passes_clean_log():
    bad = C.collect_dmesg_errors(fake_run({"dmesg": "[Tue] NVRM: Xid (PCI:0000:19:00): 79, pid=1, GPU has fallen off the bus.\n"
                                                    "[Tue] something harmless\n"}))
    assert bad["status"] == "FAIL" and bad["xids"] == [79] and "fallen" in bad["matches"]
    ok = C.collect_dmesg_errors(fake_run({"dmesg": "[Tue] eth0: link up\n"}))
    assert ok["status"] == "PASS" and not ok["matches"]
    assert C.collect_dmesg_errors(fake_run({}))["status"] == "SKIP"


def test_gpu_metrics_processes_clock_and_topology():
    q = "0, 45, 300.1, 1000.0, 10, 183359, 0, 0, No, 5, 5, 16, 16\n1, 50, 310.0, 1000.0, 90000, 183359, 2, 2, Yes, 5, 5, 8, 16\n"
    m = C.collect_gpu_metrics(fake_run({"--query-gpu=index,temperature": q}))
    assert m["status"] == "FAIL" and m["gpus"][0]["problems"] == []
    assert {"uncorrected ECC errors", "page retirement pending (needs a reset)", "PCIe link narrower than its maximum",
            "memory already in use"} <= set(m["gpus"][1]["problems"])
    p = C.collect_gpu_processes(fake_run({"--query-compute-apps": "4242, python, 1000 MiB, GPU-abc\n"}), self_pid=1)
    assert p["status"] == "WARN" and p["foreign"] == 1
    assert C.collect_gpu_processes(fake_run({"--query-compute-apps": "4242, python, 1000 MiB, GPU-abc\n"}), self_pid=4242)["status"] == "PASS"
    clk = C.collect_clock_state(fake_run({"timedatectl": "yes\n", "--query-gpu=index,clocks.sm": "0, 1965, 1965, 1965, 0x0\n1, 1200, 1965, 1200, 0x0\n"}))
    assert clk["status"] == "WARN" and clk["gpus"][1].get("locked_low") and not clk["gpus"][0].get("locked_low")
    good = C.collect_nvlink_topology(fake_run({"topo -m": TOPO, "nvlink --status": "GPU 0\n\t Link 0: 50 GB/s\n"}))
    assert good["status"] == "PASS" and good["gpus"] == 3
    bad = C.collect_nvlink_topology(fake_run({"topo -m": TOPO_BAD, "nvlink --status": "\t Link 3: <inactive>\n"}))
    assert bad["status"] == "FAIL" and bad["non_nvlink_pairs"] and bad["inactive_links"]


def test_nic_selector_and_host_limits(tmp_path):
    net, ib = tmp_path / "net", tmp_path / "ib"
    for n, st in (("eth0", "up"), ("eth1", "down"), ("lo", "unknown")):
        (net / n).mkdir(parents=True)
        (net / n / "operstate").write_text(st + "\n")
    for dev, st in (("mlx5_0", "4: ACTIVE"), ("mlx5_1", "1: DOWN")):
        (ib / dev / "ports" / "1").mkdir(parents=True)
        (ib / dev / "ports" / "1" / "state").write_text(st + "\n")
    allp = C.collect_nic_status(selector="", sys_net=str(net), sys_ib=str(ib))
    assert allp["status"] == "FAIL" and allp["down"][0]["device"] == "mlx5_1"
    assert C.collect_nic_status(selector="mlx5_0", sys_net=str(net), sys_ib=str(ib))["status"] == "PASS"
    assert C.collect_nic_status(selector="^mlx5_1", sys_net=str(net), sys_ib=str(ib))["status"] == "PASS"
    assert C.collect_nic_status(selector="=eth1", sys_net=str(net), sys_ib=str(ib))["status"] == "FAIL"
    lim = C.collect_host_limits(ulimit_l_min_gb=0.0, shm_min_gb=0.0)
    assert "memlock_gib" in lim and lim["nofile"] > 0


def test_orchestrator_and_aggregator(tmp_path):
    def spawn(cmd, timeout):
        gpu = int(cmd[cmd.index("--gpu") + 1])
        tf = 1300.0 if gpu != 2 else 900.0
        return {"gpu": gpu, "checks": [{"check": "tier1 training step", "status": "PASS", "losses": [10.4, 10.3]},
                                       {"check": "tier2 square bf16 GEMM", "status": "PASS" if tf >= 1100 else "FAIL", "tflops": tf,
                                        "threshold": 1100.0},
                                       {"check": "tier2 HBM copy", "status": "PASS", "gbs": 6400.0, "threshold": 5000.0}]}
    run = fake_run({"topo -m": TOPO, "dmesg": "clean\n", "timedatectl": "yes\n"})
    rep = run_node_smoke(tier=2, gpus=[0, 1, 2, 3], dump_dir=str(tmp_path), spawn=spawn, run=run)
    assert rep["status"] == "FAIL" and (tmp_path / (rep["hostname"] + ".json")).exists()
    assert node_status_from({"a": {"status": "WARN"}}, []) == "WARN" and node_status_from({"a": {"status": "PASS"}}, []) == "PASS"
    other = json.loads(json.dumps(rep))
    other["hostname"] = "node-b"
    other["status"] = "PASS"
    other["collectors"]["fingerprint"]["digest"] = "different"
    for g in other["per_gpu"]:
        for c in g["checks"]:
            c["status"] = "PASS"
            if "tflops" in c:
                c["tflops"] = 1310.0
    third = json.loads(json.dumps(other))
    third["hostname"] = "node-c"
    third["collectors"]["fingerprint"]["digest"] = rep["collectors"]["fingerprint"]["digest"]
    s = summarize_cluster([rep, other, third])
    assert s["nodes"] == 3 and s["fail"] == 1 and s["failing_nodes"] == [rep["hostname"]]
    assert s["fingerprint_outliers"] == ["node-b"]
    assert any(x["gpu"] == 2 and x["metric"] == "tflops" for x in s["slow_gpus"])
    write_report(s, str(tmp_path / "report.md"))
    assert "exclude: " + rep["hostname"] in (tmp_path / "report.md").read_text()
