"""Host-side arithmetic of bench.py: the FLOP counts behind the reported TFLOP/s, the L2 policy,
the workload descriptions and the data files the roofline line is built from."""
import json
import os

import bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_algorithmic_flops_of_the_benchmarked_configurations():
    c4 = bench.WORKLOADS["c4"]
    T, d = c4["B"] * c4["S"], c4["d"]
    # four projections forward and two gradients each, attention core with c = 1/2
    assert bench.algorithmic_flops(c4["B"], c4["S"], d, True) == 24.0 * T * d * d + 6.0 * c4["B"] * c4["S"] ** 2 * d
    assert abs(bench.algorithmic_flops(4, 8192, 2048, True) - 6.597e12) < 1e9
    assert bench.algorithmic_flops(1, 128, 64, False) == 2 * bench.algorithmic_flops(1, 128, 64, True) - 24.0 * 128 * 64 * 64
    # the reference computes the whole S x S product whatever the mask
    assert bench.reference_flops(2, 64, 64) == bench.algorithmic_flops(2, 64, 64, False)
    # the block adds two dense layers of width 4d: 16 T d^2 forward, 32 T d^2 backward
    assert bench.block_flops(32, 1024, 1024, False) - bench.algorithmic_flops(32, 1024, 1024, False) == 48.0 * 32 * 1024 * 1024 * 1024


def test_workloads_name_the_baseline_configurations():
    with open(os.path.join(ROOT, "BASELINE.json")) as f:
        configs = json.load(f)["configs"]
    for name, must in (("c2", ("batch=8", "seq=512", "d_model=512", "heads=8")),
                       ("c3", ("batch=16", "seq=2048", "d_model=1024", "heads=16")),
                       ("c4", ("batch=4", "seq=8192", "d_model=2048", "heads=16")),
                       ("c5", ("batch=32", "seq=1024", "d_model=1024", "heads=16"))):
        text = configs[int(name[1]) - 1]
        cfg = bench.WORKLOADS[name]
        described = "batch=%d, seq=%d, d_model=%d, heads=%d" % (cfg["B"], cfg["S"], cfg["d"], cfg["nh"])
        for piece in must:
            assert piece in text and piece in described, (name, piece)
    assert bench.DEFAULT_WORKLOAD == "c4"
    line = bench.workload_config("c4", bench.WORKLOADS["c4"], 8)
    assert line["global_batch"] == 32 and line["parallelism"].startswith("dp8") and "causal" in line["workload"]
    assert "model" not in line
    assert "encoder block" in bench.workload_config("c5", bench.WORKLOADS["c5"], 1)["workload"]


def test_l2_policy_flushes_only_what_could_stay_in_l2():
    flush, text = bench.l2_policy(bench.WORKLOADS["c2"])        # 14 * 8*512*512*4 B = 117 MB
    assert flush and "flush" in text
    for name in ("c3", "c4", "c5", "target"):
        flush, text = bench.l2_policy(bench.WORKLOADS[name])
        assert not flush and "larger than L2" in text, name


def test_peaks_and_traffic_files():
    pk = bench.load_peaks()
    assert pk["source"] in ("measured", "fallback")
    assert 1000 < pk["hbm"] < 10000 and 500 < pk["bf16_sustained"] <= pk["bf16"] < 3000
    caps = bench.load_kernel_traffic()
    assert {c["kernel"] for c in caps} >= {"attn_fwd_tc", "attn_bwd_tc"}
    for c in caps:
        assert c["dram_bytes"] > 0 and c["units"] > 0 and c["hs"] in (64, 128)
        assert os.path.exists(os.path.join(ROOT, "profiles", c["summary"])), c["summary"]
