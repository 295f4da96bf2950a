"""Host-side pieces of bench.py that need no GPU: the DRAM-traffic record it reads for roofline.traffic, the operation
count of the workload, and the weight-shard bookkeeping of configuration 5."""
import importlib
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
bench = importlib.import_module("bench")


def test_traffic_record_parses_and_names_its_capture():
    t = bench.read_dram_traffic()
    assert t["source"].startswith("profiles/") and t["captured"]
    assert sorted(t["per_shape"]) == sorted(name for name, _, _ in bench.SHAPES)
    assert abs(t["bytes_per_launch"] - sum(t["per_shape"].values()) / 4) < 1
    # between the operand bytes alone and operands + full output, per launch
    for (name, n, k) in bench.SHAPES:
        assert 4096 * k * 0.4 < t["per_shape"][name] < 1.3 * (4096 * k + n * k + 2 * 4096 * n)


def test_missing_traffic_record_gives_null_not_a_built_in_number(monkeypatch, tmp_path):
    monkeypatch.setattr(bench, "TRAFFIC_RECORD", str(tmp_path / "absent.txt"))
    t = bench.read_dram_traffic()
    assert t["bytes_per_launch"] is None and t["per_shape"] is None


def test_operation_count_of_the_workload():
    # 2 * M * N * K over the four CPM-Bee-10B linears at M = 4096: 4.12e11 + 1.37e11 + 3.44e11 + 3.44e11
    assert abs(bench.total_ops(4096) - 1.237e12) / 1.237e12 < 1e-3
    assert bench.total_ops(16384) == 4 * bench.total_ops(4096)


def test_cfg5_row_blocks_divide_every_weight_for_every_world_size():
    for world in (1, 2, 4, 8):
        assert bench.CFG5_BLOCKS % world == 0
        for _, n, _ in bench.SHAPES:
            assert n % bench.CFG5_BLOCKS == 0 and (n // world) % 16 == 0
