"""Benchmark timer, result writers, roofline arithmetic, sweep driver and configuration files (no GPU needed)."""
import json
import os
import subprocess
import sys

import pytest
import torch

import iris_b200 as iris
from iris_b200.utils import roofline
from iris_b200.utils.results import JSONWriter, validate_gemm

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_do_bench_cpu_modes():
    calls = {"fn": 0, "barrier": 0, "pre": 0}

    def fn():
        calls["fn"] += 1

    def barrier():
        calls["barrier"] += 1

    def pre():
        calls["pre"] += 1
    ms = iris.do_bench(fn, barrier, pre, n_warmup=2, n_repeat=5)
    assert ms >= 0.0
    assert calls["fn"] == 1 + 2 + 5 and calls["pre"] == 1 + 2 + 5
    assert calls["barrier"] == 2 + 2 * 7 + 1          # around the first call, twice per iteration, once at the end
    allv = iris.do_bench(fn, n_warmup=0, n_repeat=4, return_mode="all")
    assert len(allv) == 4
    q = iris.do_bench(fn, n_warmup=0, n_repeat=4, quantiles=[0.5, 0.9])
    assert len(q) == 2 and q[0] <= q[1]
    for mode in ("min", "max", "median", "mean"):
        assert iris.do_bench(fn, n_warmup=0, n_repeat=3, return_mode=mode) >= 0.0


def test_memset_tensor_cpu_and_asserts():
    t = torch.full((10,), 3, dtype=torch.int32)
    iris.memset_tensor(t, 7)
    assert t.tolist() == [7] * 10
    with pytest.raises(AssertionError):
        iris.memset_tensor(torch.zeros(4), 0)
    with pytest.raises(AssertionError):
        iris.memset_tensor(torch.zeros((4, 4), dtype=torch.int32).t(), 0)


def test_json_writer(tmp_path):
    path = tmp_path / "sub" / "log.json"
    w = JSONWriter(str(path))
    w.add_field("m", 8192)
    w.add_fields(world_size=8, fused_ms=0.37)
    w.flush()
    assert json.loads(path.read_text()) == {"m": 8192, "world_size": 8, "fused_ms": 0.37}
    JSONWriter("").flush()  # no file requested: nothing happens


def test_validate_gemm_cpu():
    a, b = torch.randn(16, 8), torch.randn(8, 4)
    assert validate_gemm(a, b, a @ b, atol=1e-3)
    bad = (a @ b).clone()
    bad[3, 2] += 5
    assert not validate_gemm(a, b, bad, atol=1e-3)


def test_roofline_numbers():
    pk = roofline.Peaks(6539.0, 1667.0, 1417.0, 770.0, "measured")
    r1 = roofline.all_scatter_roofline_us(8192, 14336, 4096, 1, pk)
    assert r1["bound"] == "compute" and abs(r1["target_us"] - 577.1) < 1.0
    r8 = roofline.all_scatter_roofline_us(8192, 14336, 4096, 8, pk)
    assert r8["bound"] == "link" and abs(r8["link_us"] - 267.0) < 1.0
    one = roofline.all_reduce_roofline_us(8192, 4096, 11008, 8, pk, "one_shot")
    two = roofline.all_reduce_roofline_us(8192, 4096, 11008, 8, pk, "two_shot")
    assert abs(one["link_us"] - 610.1) < 1.0 and abs(two["link_us"] - 152.5) < 1.0
    eff = roofline.effective_link_bandwidth({"m": 8192, "n": 14336, "world_size": 8, "fused_ms": 0.38})
    assert abs(eff["gbs_per_rank"] - 540.8) < 1.0
    assert roofline.load_peaks("/nonexistent.json").source == "fallback"


def test_config_files_and_sweep_dry_run():
    shapes = json.load(open(os.path.join(ROOT, "configs", "shapes.json")))["shapes"]
    assert any(s["name"] == "config3_all_scatter" and (s["m"], s["n"], s["k"]) == (8192, 14336, 4096) for s in shapes)
    assert {1, 128, 1024, 8192} <= {s["m"] for s in shapes if "config4" in s["name"]}
    tiling = json.load(open(os.path.join(ROOT, "configs", "tiling_b200.json")))
    assert tiling["default"]["BLK_M"] in (0, 128, 256) and tiling["default"]["BLK_N"] == 256
    # more than one tile shape in the table, every entry a shape the kernel has
    from iris_b200.utils.config import TileConfig
    shapes_used = set()
    for o in tiling["overrides"]:
        t = TileConfig(**{k: v for k, v in dict(tiling["default"], **o).items() if k not in ("m", "n", "k")})
        assert not t.problems(), (o, t.problems())
        shapes_used.add((t.BLK_M, t.BLK_N))
    assert len(shapes_used) >= 4
    out = subprocess.run([sys.executable, os.path.join(ROOT, "examples", "benchmark", "bench_all_shapes.py"), "-n",
                          "--gpus", "8", "--only", "config3_all_scatter", "config4_all_reduce_m128"],
                         capture_output=True, text=True, check=True).stdout
    assert "07_gemm_all_scatter/benchmark.py" in out and "-np 8" in out
    assert out.count("09_gemm_one_shot_all_reduce/benchmark.py") == 2 and "--variant two_shot" in out


def test_launcher_time_limit(tmp_path):
    from iris_b200.launch import launch
    slow = tmp_path / "slow.py"
    slow.write_text("import time\ntime.sleep(30)\n")
    code, _ = launch(2, [str(slow)], timeout_s=1.5, capture=True)
    assert code == 124


def test_kernel_resources_are_recorded_at_build_time():
    """ptxas figures per kernel: parsed from the compiler's output (device functions compiled out of line do not
    overwrite the kernel that calls them) and kept beside the library."""
    from iris_b200 import _build
    log = """
ptxas info    : Compiling entry function '_Z1kv' for 'sm_100a'
ptxas info    : Function properties for _Z1kv
    160 bytes stack frame, 186 bytes spill stores, 336 bytes spill loads
ptxas info    : Used 168 registers, used 4 barriers, 160 bytes cumulative stack size, 32 bytes smem
ptxas info    : Function properties for _Z6helperv
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Compiling entry function '_Z2k2v' for 'sm_100a'
ptxas info    : Function properties for _Z2k2v
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 32 registers, used 1 barriers
"""
    got = _build.parse_ptxas(log)
    assert got["_Z1kv"] == dict(registers=168, barriers=4, stack_bytes=160, spill_store_bytes=186,
                                spill_load_bytes=336, smem_bytes=32)
    assert got["_Z2k2v"]["registers"] == 32 and got["_Z2k2v"]["spill_store_bytes"] == 0
    _build.build_all()
    res = _build.kernel_resources()
    gemm = {k: v for k, v in res.items() if "fused_gemm_kernel<" in k}
    assert len(gemm) == 12   # cta_group x pull x 16-bit type, plus cta_group x (fp32, int8) without reducer warps
    for name, v in gemm.items():
        # 8 warps: at most 255; 10 warps (reducer kernels): 168 per thread, or the CTA would not fit the register file
        pull = ", true, " in name       # fused_gemm_kernel<cta_group, pull, element type>
        assert 0 < v["registers"] <= (168 if pull else 255), (name, v)
    # the main-loop kernels without reducer warps must not spill
    assert all(v["spill_store_bytes"] == 0 for k, v in gemm.items() if ", false, " in k)


def test_tile_trace_to_chrome():
    from iris_b200.utils.results import tile_trace_to_chrome
    recs = [dict(record=0, tile_id=0, cta_in_pair=0, mma_begin=1.0, mma_end=9.0, epi_begin=9.5, epi_end=12.0,
                 wait_begin=13.0, wait_end=20.0, pull_end=31.0),
            dict(record=1, tile_id=0, cta_in_pair=1, mma_begin=None, mma_end=None, epi_begin=9.6, epi_end=12.5,
                 wait_begin=None, wait_end=None, pull_end=None)]
    tr = tile_trace_to_chrome(recs, rank=3)
    ev = [e for e in tr["traceEvents"] if e["ph"] == "X"]
    assert {(e["name"], e["tid"]) for e in ev} == {("main loop", 0), ("epilogue", 1), ("flag wait", 2), ("sum", 2),
                                                   ("epilogue", 4)}
    assert all(e["pid"] == 3 and e["dur"] >= 0 for e in ev)
    sm = next(e for e in ev if e["name"] == "sum")
    assert sm["ts"] == 20.0 and sm["dur"] == 11.0
    import json
    json.dumps(tr)


def test_json_writer_records_its_environment(tmp_path):
    w = JSONWriter(str(tmp_path / "r.json"))
    w.add_field("x", 1)
    w.add_environment()
    w.flush()
    import json
    d = json.load(open(tmp_path / "r.json"))
    env = d["environment"]
    assert d["x"] == 1 and env["torch"] == torch.__version__ and "time_utc" in env and "host" in env
    assert ("gpu" in env) == torch.cuda.is_available()


def test_benchmark_points_validate_and_build_their_command():
    from iris_b200.utils.config import GemmPoint, TileConfig, load_points
    table = json.load(open(os.path.join(ROOT, "configs", "tiling_b200.json")))
    ok = GemmPoint("all_scatter", 8192, 14336, 4096, 8, name="c3")
    assert ok.problems() == [] and ok.per_rank_shape() == (8192, 1792, 4096)
    assert ok.tile(table) == TileConfig(BLK_M=256, BLK_N=256, gsize_m=8)        # the table's entry for 8192x1792x4096
    short = GemmPoint("atomic", 128, 4096, 11008, 8).tile(table)
    assert (short.BLK_M, short.BLK_N, short.ksplit) == (128, 64, 1)                # another tile shape for a short matrix
    cmd = ok.command("/r", table, output_file="o.json")
    assert cmd[:5] == ["python", "-m", "iris_b200.launch", "-np", "8"] and "/r/examples/07_gemm_all_scatter/benchmark.py" in cmd
    assert cmd[cmd.index("--output_file") + 1] == "o.json"
    assert GemmPoint("all_scatter", 8192, 14336, 4096, 3).problems() == ["N must divide by the number of ranks"]
    assert "K per rank" in GemmPoint("one_shot", 128, 4096, 11004, 4).problems()[0]
    assert GemmPoint("one_shot", 1, 4096, 11008, 8).problems() == []
    assert GemmPoint("one_shot", 1, 4096, 11008, 8).per_rank_shape() == (1, 4096, 1376)
    assert GemmPoint("one_shot", 1, 4096, 11008, 8).tile(table).gsize_m == 1       # an override of the table
    assert "ranks x 128" in GemmPoint("reduce_scatter", 1000, 4096, 4096, 8).problems()[0]
    assert GemmPoint("reduce_scatter", 16384, 4096, 4096, 8).problems() == []
    assert GemmPoint("atomic", 64, 4104, 4096, 2).problems() != [] and GemmPoint("atomic", 64, 4104, 4096, 1).problems() == []
    assert GemmPoint("nope", 1, 8, 8).problems() == ["unknown workload 'nope'"]
    shapes = json.load(open(os.path.join(ROOT, "configs", "shapes.json")))
    pts = load_points(shapes, (1, 2, 4, 8))
    assert len(pts) == 4 * sum(len(s["workloads"]) for s in shapes["shapes"])
    assert any(p.workload == "reduce_scatter" and p.world == 8 and not p.problems() for p in pts)


def test_sweep_points_carry_their_element_type():
    """A shape of the sweep file may name its element type; the command line passes it on, and int8 points never ask
    for tiles narrower than one 128-column sub-tile."""
    import json
    import os
    from iris_b200.utils.config import GemmPoint, load_points
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "configs", "shapes.json")) as f:
        shapes = json.load(f)
    pts = load_points(shapes, worlds=(1, 2))
    by_type = {p.dtype for p in pts}
    assert {"bf16", "fp16", "fp32", "int8"} <= by_type
    for p in pts:
        assert p.problems() == [], (p, p.problems())
    table = {"default": {"BLK_N": 64}, "overrides": []}
    cmd = GemmPoint("all_scatter", 8192, 14336, 4096, 2, dtype="int8").command("/repo", table)
    assert cmd[cmd.index("--datatype") + 1] == "int8" and cmd[cmd.index("--BLK_N") + 1] == "128"
    assert GemmPoint("two_shot", 8192, 4096, 11008, 2, dtype="int8").problems()


def _example_scripts():
    import glob
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pats = ["examples/[01]*/*.py", "examples/benchmark/*.py", "examples/benchmark/reference/*.py"]
    return sorted(p for pat in pats for p in glob.glob(os.path.join(root, pat)) if not p.endswith("_common.py"))


def test_every_example_prints_its_usage():
    """Every example and benchmark script parses its command line before it touches a device: `-h` exits 0 on a machine
    without a GPU and names the flags the READMEs use (a guard for edits to the shared drivers)."""
    import os
    import subprocess
    import sys
    scripts = _example_scripts()
    assert len(scripts) >= 20
    procs = [(s, subprocess.Popen([sys.executable, s, "-h"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
             for s in scripts]
    usage = {}
    for s, p in procs:
        out, _ = p.communicate(timeout=300)
        assert p.returncode == 0, (s, out[-400:])
        usage[os.path.relpath(s, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))] = out
    for flag in ("--datatype", "--BLK_N", "--push_kind", "--all_gather", "--tail_split", "--ksplit", "--variant"):
        assert flag in usage["examples/07_gemm_all_scatter/benchmark.py"], flag
    assert "--cuda_graph" in usage["examples/10_tp_block/tp_block.py"] and "--attention" in usage["examples/10_tp_block/tp_block.py"]
    assert "--blocks" in usage["examples/06_message_passing/message_passing_put.py"]
    assert "mp" in usage["examples/benchmark/profile_case.py"]
