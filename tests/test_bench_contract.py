"""What bench.py promises without a GPU: one GPU only, and a reference arm that answers."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_2():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--gpus", "2"], capture_output=True, text=True,
                       timeout=120)
    assert p.returncode == 2
    lines = [ln for ln in (p.stdout + p.stderr).splitlines() if ln.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_config_of_the_default_run_is_flat_and_short():
    """The record keeps at most 20 flat keys of `config`."""
    sys.path.insert(0, str(ROOT))
    try:
        import bench
    finally:
        sys.path.pop(0)
    cfg = bench.describe_config(dict(bench.LLAMA_8B), 8, 4096, 32, 32, 3840, 4096, "measured")
    assert cfg["head_dim"] == 128 and cfg["hidden"] == 4096 and cfg["vocab"] == 128256
    assert len(cfg) <= 20
    assert all(isinstance(v, (int, float, str)) for v in cfg.values())
    json.dumps(cfg)
    for key in ("layers", "layers_full", "hidden", "ffn", "q_heads", "kv_heads", "head_dim", "vocab", "page"):
        assert key in cfg


def test_serve_bench_roofline_arithmetic_and_arrivals():
    """The per-step roofline of the serving benchmark from a made-up step log, and the seeded
    arrival schedule."""
    from fastgen_b200.tools import serve_bench as sb

    cfg = sb.config_of("1b")
    d, f, v, hq, hkv, hd, layers = 2048, 8192, 128256, 32, 8, 64, 16
    matmul = layers * (d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * f)
    log = [
        dict(t_start=0.0, t_end=0.002, decode_tokens=10, prompt_tokens=0, kv_tokens=5000, key_pairs=5000),
        dict(t_start=0.002, t_end=0.012, decode_tokens=4, prompt_tokens=1020, kv_tokens=3000, key_pairs=400000),
        dict(t_start=0.012, t_end=0.013, decode_tokens=0, prompt_tokens=100, kv_tokens=100, key_pairs=5050),
    ]
    r = sb.roofline_of(log, cfg, weight_bytes=2_000_000_000, kv_bytes_per_token=32768, max_prefill=1024,
                       pk=dict(hbm_gbs=6537.3, tflops=1388.5, source="measured"))
    assert (r["steps_decode_only"], r["steps_prompt_heavy"], r["steps_mixed"]) == (1, 1, 1)
    read = 2_000_000_000 + 5000 * 32768
    assert abs(r["decode_hbm_gbs"] - read / 0.002 / 1e9) < 0.1 and r["decode_mean_batch"] == 10
    flops = 2 * matmul * 1024 + 4 * hd * hq * layers * 400000 + 2 * d * v * 4
    assert abs(r["prompt_tflops"] - flops / 0.010 / 1e12) < 0.1
    assert abs(r["prompt_tensor_frac"] - flops / 0.010 / 1e12 / 1388.5) < 1e-3
    t = sb.arrival_times(256, 1.0, 6)
    assert t[0] == 0.0 and abs(t[-1] - 1.0) < 1e-12 and t == sorted(t) and t == sb.arrival_times(256, 1.0, 6)
    assert sb.arrival_times(256, 1.0, 7) != t
