"""Host-side pieces of bench.py that need no GPU: both arms (this build and ``--impl reference``) must name the
workload with the same ``config`` dict, whatever flags select it."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_workload_config_names_the_workload_only():
    b = _bench()
    c1 = b.workload_config(64, 1)
    assert c1["tokens_per_gpu"] == 64 and c1["experts"] == 512 and c1["topk"] == 10 and c1["parallelism"] == "single GPU"
    assert "kernel_path" not in c1 and "zipf_s" not in c1 and "mtp" not in c1
    c8 = b.workload_config(192, 8, zipf=1.2, mtp_corr=0.98)
    assert c8["zipf_s"] == 1.2 and c8["mtp"] == {"positions_per_sequence": 6, "logit_correlation": 0.98}
    assert "64 routed experts per GPU" in c8["parallelism"]
    # a batch that is no multiple of the 1 + 5 positions carries no MTP grouping
    assert "mtp" not in b.workload_config(64, 1, mtp_corr=0.98)
    # the same call gives the same dict: what the two arms rely on
    assert b.workload_config(192, 8, 1.2, 0.98) == c8
