"""What ``bench.py`` promises without a GPU: more than one GPU is refused with one line and exit code 2, and the
workload and shape names it documents exist."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_more_than_one_gpu_is_refused_with_one_line_and_code_2():
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2", "--steps", "2", "--warmup", "1"],
                          capture_output=True, text=True, timeout=120)
    assert proc.returncode == 2
    lines = [line for line in proc.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0] and "single-GPU" in lines[0]


def test_workloads_are_the_two_serving_shapes():
    sys.path.insert(0, ROOT)
    import bench
    assert set(bench.WORKLOADS) == {"serve14b", "mixed32b"}
    s14, m32 = bench.WORKLOADS["serve14b"], bench.WORKLOADS["mixed32b"]
    assert s14["requests"] == 32 and s14["prompt_range"] == (128, 2048) and s14["new_tokens"] == 256
    assert m32["requests"] == 16 and m32["prompt_range"][1] + m32["new_tokens"] == 8192
    # the 32B shape's query width differs from its hidden size
    assert m32["shape"]["num_attention_heads"] * m32["shape"]["head_dim"] != m32["shape"]["hidden_size"]
    # the headline shape: 36 layers of the 8B sizes, batch 8 to context 4096 behind 2,048-token prompts
    assert bench.FULL_LAYERS == bench.SHAPE["num_hidden_layers"] == 36 and bench.CONTEXT == 4096 and bench.PROMPT == 2048
