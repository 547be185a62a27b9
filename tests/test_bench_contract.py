"""bench.py contract checks that need no GPU: the reference arm prints one JSON line with the keys the
driver reads, and the algorithmic byte / flop formulas agree with their definitions."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "tiny",
                          "--steps", "1", "--warmup", "1"], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "Mtokens/s" and line["higher_is_better"] is True
    for key in ("metric", "value", "n_gpus", "steps", "warmup", "ms_per_step", "scaling", "config", "cpu_baseline", "e2e"):
        assert key in line
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert line["value"] > 0


def test_algorithmic_formulas():
    sys.path.insert(0, ROOT)
    import bench
    B, H, L, d, bs, nnzb, e = 8, 8, 4096, 64, 64, 205, 2
    flops, fused_bytes, nnz = bench.algorithmic(B, H, L, d, bs, nnzb, e)
    assert nnz == nnzb * bs * bs
    assert flops == 12.0 * nnz * d * B * H                      # 2 SDDMM + 4 SpMM of 2*nnz*d each
    assert fused_bytes == 12.0 * L * d * e * B * H
    BH = B * H
    ld, v = BH * L * d * e, BH * nnz
    assert bench.stage_bytes("fused_fwd", BH, L, d, nnz, e, e, p_stored=True) == 4 * ld + 4 * BH * L + e * v
    assert bench.stage_bytes("bwd_row", BH, L, d, nnz, e, e) == 5 * ld + 2 * e * v
    assert bench.stage_bytes("spmm_dkdv", BH, L, d, nnz, e, e) == 2 * e * v + 4 * ld
    assert bench.stage_flops("bwd_row", BH, d, nnz) == 4.0 * nnz * d * BH


def test_workload_tables_are_consistent():
    """Every workload names a block size that divides L; the traffic table only names known workloads and stages."""
    sys.path.insert(0, ROOT)
    import bench
    for name, (B, H, L, d, bs, dens, dt) in bench.WORKLOADS.items():
        assert L % bs == 0 and d in (32, 64) and dt in ("bf16", "fp32") and 0 < dens <= 1, name
    for name, per_stage in bench.NCU_TRAFFIC.items():
        assert name in bench.WORKLOADS and name in bench.NCU_TRAFFIC_SOURCE
        B, H, L, d, bs, dens, dt = bench.WORKLOADS[name]
        esz = 2 if dt == "bf16" else 4
        nnz = int(round(dens * (L // bs) ** 2)) * bs * bs
        for stage, traffic in per_stage.items():
            # measured DRAM traffic of a launch is within a small factor of the algorithmic bytes
            stored = stage.endswith("+P")                # forward that also stores the probabilities
            alg = bench.stage_bytes(stage[:-2] if stored else stage, B * H, L, d, nnz, esz, esz,
                                    p_stored=stored or stage != "fused_fwd")
            assert 0.3 * alg < traffic < 1.5 * alg, (name, stage, traffic, alg)


def test_reference_arm_other_ranks_exit_quietly():
    """Under torchrun only rank 0 times the CPU path; the other ranks leave at once with status 0 and no line."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--workload", "tiny", "--steps", "1", "--warmup", "1"], stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip() == ""
