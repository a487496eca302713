"""CPU-side checks: the library loads and exports what the header declares, the launch-shape
rules match the reference's unit tests, and bad arguments are refused before any device work."""
import ctypes
import os
import re

import pytest

import krea2_hrx_b200 as k
from krea2_hrx_b200 import _lib, kernels, shape

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "krea2_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(krea2_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    handle = k.lib()
    names = header_symbols()
    assert len(names) >= 40
    for name in names:
        assert hasattr(handle, name), f"{name} is declared but not exported"
    assert sorted(_lib.SIGNATURES) == names, "the ctypes table and the header disagree"


def test_only_rows_that_alias_are_padded():
    """src/kernels/shape.rs:121-123."""
    assert [shape.gemm_pitch(6144), shape.gemm_pitch(16384)] == [6144, 16448]
    assert [shape.gemm_pitch(3072), shape.gemm_pitch(8192)] == [3072, 8256]


def test_capacity_leaves_headroom_and_whole_key_blocks():
    """src/kernels/shape.rs:126-130."""
    assert shape.capacity(4115) == 4160
    assert shape.capacity(16) == 64
    assert shape.capacity(2048) == 2080


def test_attention_tiles_fit_every_supported_capacity():
    """src/kernels/shape.rs:133-141."""
    assert shape.attention_rows(8191) == 16 and shape.attention_rows(8192) == 32
    for tokens in list(shape.tokens_range())[::97] + [16, 16896]:
        rows = shape.attention_rows(tokens)
        assert shape.capacity(tokens) >= -(-tokens // rows) * rows


def test_the_grid_is_the_tiles_themselves():
    """src/kernels/shape.rs:144-148."""
    assert shape.gemm_grid_rows(4115) == 17
    assert shape.gemm_grid_rows(256) == 1
    assert shape.gemm_grid_rows(16) == 1


def test_tiles_sources_and_schedule():
    """src/kernels/shape.rs:67-99, blocks.rs:181-216."""
    assert shape.gemm_tile("gemm_down") is shape.GemmTile.Wide
    for stem in ("gemm_qkvg", "gemm_gu", "gemm_wo", "anything"):
        assert shape.gemm_tile(stem) is shape.GemmTile.Narrow
    assert shape.gemm_source("gemm_i8_resid_256", shape.GemmTile.Wide) == "gemm_i8_resid_256x256"
    assert shape.gemm_source("gemm_i8_256", shape.GemmTile.Wide) == "gemm_i8_256"
    assert (shape.GemmTile.Narrow.columns(), shape.GemmTile.Narrow.threads()) == (128, 256)
    assert (shape.GemmTile.Wide.columns(), shape.GemmTile.Wide.threads()) == (256, 512)
    assert shape.gemm_m_group() == 4
    assert not shape.gemm_schedule_rows(4095) and shape.gemm_schedule_rows(4096)


def test_shape_refuses_lengths_outside_the_range():
    """src/kernels/blocks.rs:27-36."""
    with pytest.raises(k.InvalidArgument, match="tokens must be 16..16896"):
        kernels.Shape.new(15)
    with pytest.raises(k.InvalidArgument):
        kernels.Shape.new(16897)
    s = kernels.Shape.new(4115)
    assert s.capacity == 4160
    jobs = {j.stem: j for j in s.jobs()}
    assert jobs["gemm_down"].source == "gemm_i8_resid_256x256"
    assert jobs["gemm_down"].config["schedule_rows"] == "1"
    assert jobs["gemm_down"].config["k_stride"] == "16448"
    assert "schedule_rows" not in jobs["gemm_wo"].config
    assert kernels.Shape.new(1043).jobs()[-1].config["schedule_rows"] == "0"
    assert jobs["prepare_gated_i8"].config["gate_stride"] == "15360"


def test_scalars_grid_and_workgroup():
    """src/kernels/mod.rs:77-135."""
    s = kernels.Scalars().index(7).float(0.5)
    assert s.indices == [7] and s.floats == [0.5]
    with pytest.raises(AssertionError):
        kernels.Scalars().index(1).index(2).index(3).index(4).index(5)
    assert kernels.grid("x", 3, 4) == (3, 4, 1)
    with pytest.raises(k.Internal, match="exceed the grid"):
        kernels.grid("x", 1 << 32, 1)
    assert kernels.workgroup("down", "gemm_i8_resid_256x256", 512) == (512, 1, 1)
    with pytest.raises(k.Internal, match="compiled for workgroup"):
        kernels.workgroup("down", "gemm_i8_resid_256x256", 256)


def test_session_dimensions_are_validated_without_a_device():
    """src/session/mod.rs:278-287 and tests/constructor.rs."""
    from krea2_hrx_b200 import session
    session.Session.validate_dimensions(4608, 28)
    for tokens, layers in [(15, 1), (16897, 1), (64, 0), (64, 29)]:
        with pytest.raises(k.InvalidArgument, match="tokens must be 16..16896 and layers must be 1..28"):
            session.Session.validate_dimensions(tokens, layers)
    assert session.QKVG == 15360 and session.GATE_OFFSET == 9216
    plan = session.Weights.plan_bytes(session.ModelDims(), 28)
    per_block = 15360 * 6144 + 6144 * 6144 + 32768 * 6144 + 6144 * 16448
    assert 28 * per_block < plan < 28 * per_block * 1.001


def _call(name, *args):
    fn = getattr(k.lib(), name)
    return fn(*args)


def test_bad_kernel_arguments_are_refused_before_any_device_work():
    """Config ranges of the kernels' config.decl lines; no CUDA call is made for these."""
    buf = ctypes.create_string_buffer(64)
    p = (ctypes.addressof(buf) + 15) & ~15
    cases = [
        ("krea2_prepare_plain_i8", (None, 3, p, p, p, 2000, 2048), "width"),
        ("krea2_prepare_plain_i8", (None, 3, p, p, p, 2048, 2047), "out_stride"),
        ("krea2_prepare_plain_i8", (None, 0, p, p, p, 2048, 2048), "tokens"),
        ("krea2_prepare_plain_i8", (None, 3, p + 2, p, p, 2048, 2048), "aligned"),
        ("krea2_prepare_gated_i8", (None, 3, p, p, p, p, 2048, 2048, 2000), "gate_stride"),
        ("krea2_prepare_norm_i8", (None, 3, p, p, p, p, p, p, 2048, 2048, -1.0), "eps"),
        ("krea2_gemm_i8_256", (None, 0, p, p, p, p, p, 128, 128, 128, 4), "m 0"),
        ("krea2_gemm_i8_256", (None, 1, p, p, p, p, p, 100, 128, 128, 4), "k_size"),
        ("krea2_gemm_i8_256", (None, 1, p, p, p, p, p, 128, 64, 128, 4), "k_stride"),
        ("krea2_gemm_i8_256", (None, 1, p, p, p, p, p, 128, 128, 100, 4), "n_size"),
        ("krea2_gemm_i8_256", (None, 1, p, p, p, p, p, 128, 128, 128, 5), "m_group"),
        ("krea2_gemm_i8_resid_256x256", (None, 1, p, p, p, p, p, p, 64, 64, 128, 4, 0), "n_size"),
        ("krea2_gemm_i8_resid_256x256", (None, 1, p, p, p, p, p, p, 64, 64, 256, 4, 2), "schedule_rows"),
        ("krea2_lora_transport", (None, 8, p, p, 3), "reverse"),
    ]
    for name, args, needle in cases:
        status = _call(name, *args)
        assert status == 1, (name, args)
        assert needle in k.lib().krea2_last_error().decode(), (name, k.lib().krea2_last_error())


def test_generic_launch_checks_names_counts_and_geometry():
    """Ops::launch (src/ops/mod.rs:673-693) refusals that need no device."""
    buf = ctypes.create_string_buffer(1 << 16)
    p = (ctypes.addressof(buf) + 15) & ~15

    def launch(name, config, rows, bindings, gx, gy, threads):
        entries = (_lib.ConfigEntry * max(1, len(config)))()
        for i, (key, value) in enumerate(config.items()):
            entries[i].key, entries[i].value, entries[i].fvalue = key.encode(), int(value), float(value)
        idx = (ctypes.c_uint64 * 1)(rows)
        binds = (_lib.Binding * max(1, len(bindings)))()
        for i, n in enumerate(bindings):
            binds[i].ptr, binds[i].bytes = p, n
        return k.lib().krea2_launch(None, name.encode(), entries, len(config), idx, 1, binds, len(bindings), gx, gy,
                                    threads), k.lib().krea2_last_error().decode()

    assert launch("nope", {}, 1, [], 1, 1, 256) == (1, "no kernel named nope")
    status, msg = launch("gemm_i8_256", {"k_size": 128, "k_stride": 128, "n_size": 128}, 17, [1] * 5, 1, 1, 256)
    assert status == 1 and "m_group" in msg
    cfg = {"k_size": 128, "k_stride": 128, "n_size": 128, "m_group": 4}
    status, msg = launch("gemm_i8_256", cfg, 17, [1 << 14] * 5, 1, 1, 512)
    assert status == 5 and "compiled for workgroup" in msg
    status, msg = launch("gemm_i8_256", cfg, 17, [1 << 14] * 5, 2, 1, 256)
    assert status == 1 and "grid" in msg
    status, msg = launch("gemm_i8_256", cfg, 17, [1 << 14] * 4, 1, 1, 256)
    assert status == 1 and "takes 5 buffers" in msg
    status, msg = launch("gemm_i8_256", cfg, 17, [1 << 14, 100, 1 << 14, 1 << 14, 1 << 14], 1, 1, 256)
    assert status == 1 and "buffer 1 spans 100 bytes" in msg
    status, msg = launch("prepare_plain_i8", {"width": 2048, "out_stride": 2048}, 3, [1 << 14] * 3, 4, 1, 256)
    assert status == 1 and "grid" in msg


def test_cpp_host_mirror_compiles_and_agrees(tmp_path):
    """include/krea2_b200.hpp (the C++ face shaped like the crate's modules) against the same rules."""
    import subprocess
    exe = tmp_path / "host_mirror"
    lib_dir = os.path.join(ROOT, "krea2_hrx_b200")
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "host_mirror.cpp"), "-o", str(exe), "-L", lib_dir, "-lkrea2_b200",
                    f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "host mirror ok" in out.stdout, out.stdout + out.stderr


def test_the_public_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own, with no C++ or torch types."""
    import subprocess
    source = tmp_path / "header_check.c"
    source.write_text('#include "krea2_b200.h"\nint main(void) { krea2_span_info span; krea2_dims dims; (void)span; (void)dims; '
                      "return krea2_shape_gemm_pitch(8192) == 8256 ? 0 : 1; }\n")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-fsyntax-only", "-I",
                    os.path.join(ROOT, "include"), str(source)], check=True)


def test_the_reference_arm_prints_the_benchmark_line(tmp_path):
    """`bench.py --impl reference` (the CPU port on the host cores) keeps the JSON contract of the GPU arm."""
    import json
    import subprocess
    import sys
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                           "--cpu-tokens", "64"], capture_output=True, text=True, check=True, cwd=str(tmp_path))
    line = json.loads(done.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "w8a8_path_int8_tops" and line["unit"] == "TOP/s"
    assert line["value"] > 0 and line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in line["config"]


def test_the_bench_reads_every_gemm_row_of_the_committed_dram_table():
    """`roofline.traffic` and `kernels.*.dram_over_algorithmic` come from `profiles/gemm_i8_dram_bytes_m4608.md`;
    a reworded table must not silently empty them.  The measured reads can never be below what a launch must read
    at least once, nor absurdly above it."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    table, where = bench.profiled_dram_bytes()
    assert where == os.path.join("profiles", "gemm_i8_dram_bytes_m4608.md")
    assert set(table) == set(bench.GEMM_LABELS) and len(table) == 4
    dims = dict(hidden=6144, kv_heads=12, head_dim=128, inter=16384)
    for label, (m, n, k) in bench.gemm_shapes(dims, 4608).items():
        read, written = table[label]
        operands = m * k + n * k
        assert 0.95 * operands <= read <= 3.0 * operands, (label, read, operands)
        assert 0 < written <= bench.gemm_algorithmic_bytes(label, m, n, k), label
