"""Host-side pieces of ``bench.py`` that the reported numbers rest on: the algorithmic FLOP count of the
headline workload, the map from a rank's local rows to global sequence positions that the ring check
samples with, and the ingestion of an ncu raw-page CSV into ``profiles/traffic.json`` (the source of
``roofline.traffic``).  No GPU needed."""

import argparse
import json

import pytest
import torch

import bench
from torch_neuronx_b200 import ring


def test_flop_count_equals_a_brute_force_count_of_visible_pairs():
    # 4 * E * (visible (query, key) pairs): causal, clipped by each batch's key length, over the query heads
    L, hq, e = 37, 3, 8
    lens = torch.tensor([37, 20, 1, 29])
    pairs = 0
    for n in lens.tolist():
        for i in range(L):
            pairs += min(i + 1, n)
    assert bench.c3_flops(lens, hq=hq, L=L, e=e) == 4.0 * e * hq * pairs
    # the benchmark's own shape: the bound without padding is the causal square
    full = torch.full((4,), 4096)
    assert bench.c3_flops(full) == 4.0 * 128 * 32 * 4 * (4096 * 4097 // 2)


@pytest.mark.parametrize("layout", ["zigzag", "contiguous"])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_local_rows_map_to_the_positions_the_shard_holds(layout, world):
    n = 16 * world
    pos = torch.arange(n).view(1, 1, n, 1)
    for rank in range(world):
        held = ring.shard_sequence(pos, rank, world, layout).flatten()
        got = bench._global_positions(torch.arange(held.numel()), rank, world, held.numel(), layout)
        assert torch.equal(got, held)


def test_ncu_csv_is_ingested_into_the_traffic_table(tmp_path, monkeypatch):
    csv_path = tmp_path / "raw.csv"
    csv_path.write_text(
        '"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","dram__bytes_write.sum"\n'
        '"","","us","Mbyte","Kbyte"\n'
        '"0","void other_kernel(int)","3.5","1.0","2.0"\n'
        '"1","void b200::prefill_persistent_kernel<128, 1, 0, 0>(...)","500.0","190.5","97,000.0"\n'
        '"2","void b200::prefill_persistent_kernel<128, 1, 0, 0>(...)","520.0","193.5","97,500.0"\n'
    )
    table = tmp_path / "traffic.json"
    table.write_text(json.dumps({"decode": {"dram_bytes_per_launch": 1.0}}))
    monkeypatch.setattr(bench, "TRAFFIC_JSON", str(table))
    args = argparse.Namespace(ingest_ncu=str(csv_path), profile="prefill", kernel="prefill_persistent_kernel",
                              algorithmic_bytes=325427200.0)
    bench.ingest_ncu(args)
    got = json.loads(table.read_text())
    assert got["decode"] == {"dram_bytes_per_launch": 1.0}                  # other cases are kept
    entry = got["prefill"]
    assert entry["launches_averaged"] == 2
    assert entry["dram_read_bytes"] == pytest.approx(192.0e6)
    assert entry["dram_write_bytes"] == pytest.approx(97.25e6)
    assert entry["dram_bytes_per_launch"] == pytest.approx(289.25e6)
    assert entry["gpu_time_us_under_ncu"] == pytest.approx(510.0)
    assert entry["algorithmic_bytes_per_launch"] == 325427200.0
    # and read back the way the roofline object reads it
    assert bench.measured_traffic("prefill")["dram_bytes_per_launch"] == pytest.approx(289.25e6)
    with pytest.raises(SystemExit):
        bench.ingest_ncu(argparse.Namespace(ingest_ncu=str(csv_path), profile="gpt2", kernel="no_such_kernel",
                                            algorithmic_bytes=1.0))
