"""The perftest runner's bookkeeping, with a fake in place of the process launch (no GPU, no torchrun)."""
import json

from perftest import runner


def test_command_lines_use_loopback_rendezvous():
    one = runner.command("kernel_case", ["--kernel", "gemm"], 1, python="py")
    assert one == ["py", "-m", "perftest.kernel_case", "--kernel", "gemm"]
    many = runner.command("coll", ["--algos", "best"], 8, python="py")
    assert many[:3] == ["py", "-m", "torch.distributed.run"] and "--nproc-per-node=8" in many
    assert many[many.index("--master-addr") + 1] == "127.0.0.1"
    assert many[-4:] == ["-m", "perftest.coll", "--algos", "best"]


def test_run_list_collects_rows_failures_and_skips_unsupported_pe_counts(tmp_path):
    calls = []

    def fake(cmd, timeout, env=None):
        calls.append(cmd)
        if "perftest.host" in cmd:
            return 124, "partial output\n", 600.0  # a time-out
        return 0, 'noise\n{"test": "put_bw", "GBps": 650.0}\n{"test": "get_bw", "GBps": 630.0}\n', 1.5

    summary = runner.run_list("p2p", [1, 2], tmp_path, 600.0, runner=fake, python="py")
    # the p2p drivers need exactly two PEs: the 1-PE pass is skipped
    assert [s["npes"] for s in summary] == [2, 2] and len(calls) == 2
    ok, bad = summary
    assert ok["driver"] == "rma" and ok["status"] == 0 and ok["rows"] == 2
    assert bad["driver"] == "host" and bad["status"] == 124 and bad["rows"] == 0
    rows = [json.loads(l) for l in (tmp_path / "p2p_rma_256M_n2.jsonl").read_text().splitlines()]
    assert rows[0]["test"] == "put_bw" and rows[1]["GBps"] == 630.0
    assert "partial output" in (tmp_path / "p2p_host_n2.log").read_text()


def test_run_one_times_out_and_terminates_only_its_child():
    import sys
    status, out, secs = runner.run_one([sys.executable, "-c", "import time; print('started', flush=True); time.sleep(30)"], timeout=1.0)
    assert status == 124 and "started" in out and secs < 20
    status, out, _ = runner.run_one([sys.executable, "-c", "print('{\"a\": 1}')"], timeout=30.0)
    assert status == 0 and out.strip() == '{"a": 1}'
