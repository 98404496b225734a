"""bench.py's bookkeeping that runs without a GPU: the ncu traffic figures are only used while the kernel
sources are the ones the capture ran, and the algorithmic per-edge figures follow the workload's shape."""
import importlib.util
import os
import shutil

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("pbg_bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_traffic_line_is_tied_to_the_kernel_sources(tmp_path):
    b = _bench()
    csrc = tmp_path / "pytorch-biggraph_b200" / "csrc"
    csrc.mkdir(parents=True)
    (csrc / "a.cu").write_text("__global__ void k() {}\n")
    (csrc / "b.cuh").write_text("// header\n")
    (tmp_path / "profiles").mkdir()
    b.ROOT = str(tmp_path)
    digest = b.csrc_digest()
    name = b.PROFILE_FILES[("c3", "bf16x6")]
    prof = tmp_path / "profiles" / name
    prof.write_text(f"# summary\ntraffic_per_edge_bytes: gather=10 score=20 grad=30 update=40 csrc_sha256={digest}\n")
    per_class, source = b.ncu_traffic_per_edge("c3", "bf16x6")
    assert per_class == {"gather": 10.0, "score": 20.0, "grad": 30.0, "update": 40.0} and digest in source
    # any change to a kernel source makes the capture describe other kernels: no figure, and the reason is given
    (csrc / "a.cu").write_text("__global__ void k() { }\n")
    assert b.csrc_digest() != digest
    per_class, why = b.ncu_traffic_per_edge("c3", "bf16x6")
    assert per_class is None and digest in why
    # no summary, or one without the line: no figure either
    prof.write_text("# summary without a traffic line\n")
    assert b.ncu_traffic_per_edge("c3", "bf16x6")[0] is None
    assert b.ncu_traffic_per_edge("c1", "bf16x6")[0] is None


def test_committed_summary_is_used_only_for_its_own_sources():
    """The committed summary either names the kernel sources in the tree (its figures are then used, and exceed
    the algorithmic bytes) or the bench says why it reports no traffic."""
    b = _bench()
    per_class, source = b.ncu_traffic_per_edge("c3", "bf16x6")
    if per_class is None:
        assert "other kernel sources" in source or "no traffic line" in source or "no ncu summary" in source
    else:
        assert b.csrc_digest() in source
        assert per_class["gather"] + per_class["score"] + per_class["grad"] + per_class["update"] > b.algorithmic(b.WORKLOADS["c3"])["bytes"]


def test_algorithmic_figures_of_the_headline_workload():
    b = _bench()
    alg = b.algorithmic(b.WORKLOADS["c3"])
    # per trained edge, dim 1024 with 100 chunk + 100 uniform negatives: 12 D (P + U) flops, (2 + 2 U / P)(12 D + 8) + 24 bytes
    assert alg["flops"] == 12 * 1024 * 200
    assert alg["bytes"] == 4 * (12 * 1024 + 8) + 24
