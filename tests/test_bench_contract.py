"""The measurement script's behaviour that needs no GPU: what it answers for more
than one GPU and for the reference arm, and the arithmetic of its roofline figures."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def run_bench(*args):
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True)
    lines = [l for l in proc.stdout.splitlines() if l.strip()]
    return proc.returncode, lines


def test_more_than_one_gpu_is_answered_with_one_line_and_exit_code_2():
    code, lines = run_bench("--gpus", "2", "--steps", "3", "--warmup", "3")
    assert code == 2 and len(lines) == 1
    assert json.loads(lines[0])["n_gpus"] == 2


def test_the_reference_arm_says_why_it_is_unavailable():
    code, lines = run_bench("--impl", "reference", "--steps", "3", "--warmup", "3")
    assert code == 0 and len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]


def test_roofline_arithmetic_of_the_default_shape():
    import bench
    cfg = bench.SMOLLM2_1P7B
    total, weights, cache = bench.decode_bytes(cfg, cfg["num_hidden_layers"], 8, 8192)
    # 24 layers of (q, k, v, o: 4 x 2048^2; gate, up, down: 3 x 2048 x 8192; two norms) + head + final norm, bfloat16
    per_layer = 4 * 2048 * 2048 + 3 * 2048 * 8192 + 2 * 2048
    assert weights == 2 * (24 * per_layer + 49152 * 2048 + 2048)
    assert cache == 8 * 8192 * 24 * 2 * 2048 * 2 and total == weights + cache
    flops = bench.prefill_flops(cfg, 24, 2048)
    gemm = 2 * 2048 * (4 * 2048 * 2048 + 3 * 2048 * 8192)
    attention = 2 * 2048 * 2048 * 64 * 32                   # causal: half of the scores, half of the weighted sum
    assert flops == 24 * (gemm + attention) + 2 * 49152 * 2048
    for name, (label, shape) in bench.SHAPES.items():
        assert shape["num_attention_heads"] % shape["num_key_value_heads"] == 0 and label
