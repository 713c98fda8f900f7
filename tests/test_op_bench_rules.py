"""Tuning rules derived from op_bench records (cut_b200/op_bench.py) are what the C++ VariantSelector reads:
the derived file is loaded by the host library's selector and steers MatMulQBlocks' variant choice."""
import json
import os
import subprocess

from cut_b200 import op_bench

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HOST = os.path.join(ROOT, "cut_b200", "csrc", "host")
CPP = os.path.join(ROOT, "tests", "cpp")
OUT = os.path.join(CPP, "build")


def _row(v, us):
    return {"variant": v, "name": op_bench.BLOCK_VARIANT_NAMES[v], "median_us": us, "gflops": 1.0}


RECORDS = [
    {"shape": [1, 4096, 11008], "blocks_q4_0": [_row(0, 900.0), _row(1, 7.7)]},                      # built-in wins: no rule
    {"shape": [12, 4096, 11008], "blocks_q4_0": [_row(0, 9000.0), _row(1, 40.0), _row(2, 30.0)]},    # GEMM beats the mat-vec
    {"shape": [24, 4096, 11008], "blocks_q4_0": [_row(1, 40.1), _row(2, 40.6)]},                       # a 1 % edge: no rule
    {"shape": [32, 2048, 2048], "blocks_q4_0": [_row(1, 0.0)] and [_row(0, 5.0), _row(2, 9.0)]},     # SIMT beats the GEMM
    {"shape": [8, 2048, 5632], "blocks_q4_0": []},                                                    # nothing timed
]


def test_builtin_choice_matches_the_operator_node():
    assert op_bench.builtin_block_variant(1, 4096, 11008, False) == 1
    assert op_bench.builtin_block_variant(12, 4096, 11008, False) == 1
    assert op_bench.builtin_block_variant(16, 4096, 11008, False) == 2  # the fourth column tile on a large weight
    assert op_bench.builtin_block_variant(16, 2048, 2048, False) == 1
    assert op_bench.builtin_block_variant(8, 4096, 11008, True) == 1    # fp32 rows stay on the mat-vec
    assert op_bench.builtin_block_variant(9, 4096, 11008, True) == 2  # 18 virtual rows
    assert op_bench.builtin_block_variant(17, 4096, 11008, False) == 2
    assert op_bench.builtin_block_variant(4, 96, 8, False) == 0


def test_rules_only_where_the_measured_best_differs():
    doc = op_bench.derive_rules(RECORDS)
    cuda = doc["operators"]["MatMulQBlocks"]["backends"]["cuda"]
    assert cuda["default_variant"] == -1  # unmatched shapes keep the operator's own shape-dependent choice
    got = {tuple(r["conditions"]["shape"]): r["variant"] for r in cuda["rules"]}
    assert got == {(12, 4096, 11008): 2, (32, 2048, 2048): 0}


def test_derived_file_drives_the_cpp_selector(tmp_path):
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, "tuning_rules_check")
    r = subprocess.run(["g++", "-O1", "-std=c++17", f"-I{HOST}", "-o", exe, os.path.join(CPP, "tuning_rules_check.cpp"),
                        os.path.join(HOST, "cut_api.cpp")], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    path = tmp_path / "tuning_data.json"
    path.write_text(json.dumps(op_bench.derive_rules(RECORDS)))

    def select(default, *shape):
        out = subprocess.run([exe, str(path), "MatMulQBlocks", "cuda", str(default), *map(str, shape)], capture_output=True, text=True)
        assert out.returncode == 0, out.stdout + out.stderr
        return int(out.stdout.strip().splitlines()[-1])

    assert select(1, 12, 4096, 11008) == 2   # rule
    assert select(2, 32, 2048, 2048) == 0    # rule
    assert select(0, 1, 4096, 11008) == 0    # no rule for the shape: the caller's own choice stands
    assert select(2, 512, 4096, 14336) == 2
    # the committed rule file parses too
    shipped = os.path.join(ROOT, "cut_b200", "tuning_data.json")
    if os.path.exists(shipped):
        out = subprocess.run([exe, shipped, "MatMulQBlocks", "cuda", "1", "1", "4096", "11008"], capture_output=True, text=True)
        assert out.returncode == 0 and out.stdout.strip().splitlines()[-1].isdigit(), out.stdout + out.stderr
