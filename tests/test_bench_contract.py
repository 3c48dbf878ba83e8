"""bench.py's bookkeeping without a GPU: algorithmic bytes of the headline workload, the config
block of the JSON line, and that the tensor-parallel binding covers its header."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_of_the_headline_workload():
    b = _bench()
    # packed Q4_K weights of the Llama-3-8B MLP + x in + y out + norm weight (bf16), batch 1
    assert b.algorithmic_bytes(1) == 99115008
    assert b.algorithmic_bytes(8) == 99229696
    assert b.algorithmic_bytes(1, 8192, 28672) == 3 * 8192 * 28672 * 144 // 256 + 2 * 8192 * 2 + 8192 * 2


def test_config_block_names_the_workload():
    b = _bench()
    c = b.config_dict(1, 1)
    assert "Llama-3-8B" in c["workload"] and c["parallelism"] == "single GPU" and "model" not in c
    c8 = b.config_dict(1, 8, "auto")
    assert c8["parallelism"].startswith("tp8") and c8["exchange"] == "auto"
    # nothing run-dependent in it: both arms of a run print the same dict
    assert b.config_dict(1, 1) == c
    hbm, tf, which = b.measured_peaks()
    assert hbm > 1000 and tf > 100 and which in ("measured", "fallback")


def test_tp_binding_covers_header():
    import re
    from mlxr_b200 import _capi
    text = open(os.path.join(ROOT, "include", "mlxr_b200_tp.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"MLXR_API\s+[^;(]*?\b(mlxr_tp_\w+)\s*\(", text))
    assert names and names == set(_capi.TP_PROTOTYPES)
