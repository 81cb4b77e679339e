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
