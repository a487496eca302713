"""The checkpoint reader and the device layout it derives, without a GPU: the reference's own unit
tests of the reader (src/checkpoint/file.rs:128-205) and of the plan (src/checkpoint/plan.rs:270-360,
restated on a small synthetic checkpoint), and every span's device image against the numpy restatement."""
import numpy as np
import pytest

from oracle import plan as plan_oracle

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200.checkpoint import Checkpoint, Segment  # noqa: E402


def write(tmp_path, name, header: str, payload: bytes):
    path = tmp_path / name
    raw = header.encode()
    path.write_bytes(len(raw).to_bytes(8, "little") + raw + payload)
    return path


def test_a_file_that_is_not_safetensors_is_refused_by_name():
    with pytest.raises(k.InvalidArgument, match=r"not a ComfyUI checkpoint \(\.safetensors\)"):
        Checkpoint("/models/krea2.bin")


def test_a_header_longer_than_the_file_is_refused(tmp_path):
    path = write(tmp_path, "long.safetensors", "{}", b"")
    raw = bytearray(path.read_bytes())
    raw[:8] = (2 ** 64 - 1).to_bytes(8, "little")
    path.write_bytes(bytes(raw))
    with pytest.raises(k.InvalidArgument, match=r"^cannot read "):
        Checkpoint(path)


def test_a_tensor_reaching_past_the_data_is_refused(tmp_path):
    path = write(tmp_path, "span.safetensors", '{"w":{"dtype":"I8","shape":[2,2],"data_offsets":[0,64]}}', bytes(4))
    with pytest.raises(k.InvalidArgument, match=r"^cannot read "):
        Checkpoint(path)


def test_tensors_read_back_with_their_dtype_shape_and_bytes(tmp_path):
    header = '''{"__metadata__":{"format":"pt"},
        "w":{"dtype":"I8","shape":[2,3],"data_offsets":[0,6]},
        "s":{"dtype":"F32","shape":[2],"data_offsets":[6,14]}}'''
    path = write(tmp_path, "read.safetensors", header, bytes([1, 2, 3, 4, 5, 6, 0, 0, 0, 0, 0, 0, 0, 0]))
    file = Checkpoint(path)
    assert file.get("w") == ("I8", (2, 3), bytes([1, 2, 3, 4, 5, 6]))
    assert file.get("s")[0] == "F32"
    assert not file.has("__metadata__"), "metadata is not a tensor"
    with pytest.raises(k.InvalidArgument, match=r"^missing tensor missing in "):
        file.get("missing")


def test_a_whole_model_save_reads_under_the_transformer_names(tmp_path):
    header = '''{"__metadata__":{"workflow":"{}"},
        "model.diffusion_model.blocks.0.attn.wq.weight":{"dtype":"I8","shape":[1],"data_offsets":[0,1]},
        "model.diffusion_model.first.weight":{"dtype":"I8","shape":[1],"data_offsets":[1,2]}}'''
    file = Checkpoint(write(tmp_path, "wrapped.safetensors", header, bytes([7, 9])))
    assert file.get("first.weight")[2] == bytes([9])
    assert file.block_count() == 1
    assert not file.has("model.diffusion_model.first.weight")


def test_names_without_a_shared_wrapper_are_kept(tmp_path):
    header = '''{"model.blocks.0.attn.wq.weight":{"dtype":"I8","shape":[1],"data_offsets":[0,1]},
        "first.weight":{"dtype":"I8","shape":[1],"data_offsets":[1,2]}}'''
    file = Checkpoint(write(tmp_path, "mixed.safetensors", header, bytes([7, 9])))
    assert file.has("model.blocks.0.attn.wq.weight") and file.has("first.weight")
    assert file.block_count() == 0


def test_malformed_headers_are_refused(tmp_path):
    for i, header in enumerate(['[1,2]', '{"w":{"dtype":"I8","shape":[2,2]}}', '{"w":{"dtype":"Q4","shape":[1],"data_offsets":[0,1]}}',
                                '{"w":{"dtype":"F32","shape":[3],"data_offsets":[0,4]}}', '{"w":{"dtype":"I8","shape":[1],"data_offsets":[0,1]}} x',
                                '{"w":{"dtype":"I8","shape":[1],"data_offsets":[2,1]}}']):
        with pytest.raises(k.InvalidArgument, match=r"^cannot read "):
            Checkpoint(write(tmp_path, f"bad{i}.safetensors", header, bytes(8)))


def test_header_strings_must_be_well_formed_text(tmp_path):
    """JSON text is UTF-8 without raw control characters, and an escaped surrogate needs its pair."""
    entry = b'{"dtype":"I8","shape":[1],"data_offsets":[0,1]}'
    for i, name in enumerate([b'w\x9a', b'w\xc0\xaf', b'w\xed\xa0\x80', b'w\x01', b'w\\ud83d', b'w\\ude00', b'w\\ud83dx']):
        path = tmp_path / f"text{i}.safetensors"
        header = b'{"' + name + b'":' + entry + b'}'
        path.write_bytes(len(header).to_bytes(8, "little") + header + bytes(8))
        with pytest.raises(k.InvalidArgument, match=r"^cannot read "):
            Checkpoint(path)
    header = b'{"w\\ud83d\\ude00\\u00e9\xc3\xa9":' + entry + b'}'
    path = tmp_path / "pair.safetensors"
    path.write_bytes(len(header).to_bytes(8, "little") + header + bytes(8))
    assert Checkpoint(path).names() == ["w\U0001f600\u00e9\u00e9"]


SMALL = dict(layers=2, hidden=2048, kv_heads=2, head_dim=128, inter=8192)


@pytest.fixture(scope="module")
def small(tmp_path_factory):
    tensors = plan_oracle.synthetic_blocks(np.random.default_rng(7), **SMALL)
    path = tmp_path_factory.mktemp("ckpt") / "small.safetensors"
    plan_oracle.write_safetensors(str(path), tensors, metadata={"format": "pt"})
    return path, tensors


def test_the_plan_lays_out_the_blocks(small):
    """plan.rs:290-325 at the small shape: fused rows, dense and padded pitches, aligned disjoint spans."""
    path, _ = small
    file = Checkpoint(path)
    plan = file.plan()
    assert plan.layers == 2 and file.dims() == ((2048, 2, 128, 8192), 2)
    qkvg = plan.span("blocks.0.qkvg.q")
    assert qkvg.rows == 2048 + 2 * 128 + 2 * 128 + 2048
    assert (qkvg.row_bytes, qkvg.device_row_bytes, len(qkvg.segments)) == (2048, 2048, 4)
    down = plan.span("blocks.0.down.q")  # rows of 8192 bytes take one 64-byte step of padding
    assert (down.rows, down.row_bytes, down.device_row_bytes, down.device_bytes) == (2048, 8192, 8256, 2048 * 8256)
    end = 0
    for span in sorted((plan.span(name) for name in plan.names), key=lambda s: s.device_offset):
        assert span.device_offset % 256 == 0 and span.device_offset >= end, "spans overlap"
        end = span.device_offset + span.device_bytes
    assert plan.total_bytes >= end
    assert plan.names == sorted(plan.names, key=lambda n: n.encode())


def test_the_gate_and_up_rows_interleave_in_sixteens(small):
    """plan.rs:327-360."""
    path, _ = small
    plan = Checkpoint(path).plan()
    gu = plan.span("blocks.0.gu.q")
    half = gu.rows // 2
    assert len(gu.segments) == half // 16 * 2
    assert gu.segments[0] == Segment("blocks.0.mlp.gate.weight", range(0, 16))
    assert gu.segments[1] == Segment("blocks.0.mlp.up.weight", range(0, 16))
    assert gu.segments[2] == Segment("blocks.0.mlp.gate.weight", range(16, 32))
    scales = plan.span("blocks.0.gu.s")
    assert (scales.device_bytes, scales.file_bytes, len(scales.segments)) == (gu.rows * 4, gu.rows * 4, 0)


@pytest.mark.parametrize("bf16_norms,prefix", [(False, ""), (True, "model.diffusion_model.")])
def test_every_span_assembles_to_the_restated_device_image(tmp_path, bf16_norms, prefix):
    """Offsets, extents, segments and bytes (rows re-pitched with zero padding, scales gathered in row order,
    bf16 norm vectors widened) against oracle/plan.py, for plain and wrapped names."""
    shape = dict(layers=2, hidden=2048, kv_heads=1, head_dim=128, inter=2048)
    tensors = plan_oracle.synthetic_blocks(np.random.default_rng(3), bf16_norms=bf16_norms, **shape)
    path = tmp_path / "model.safetensors"
    plan_oracle.write_safetensors(str(path), tensors, prefix=prefix)
    plan = Checkpoint(path).plan()
    want, total = plan_oracle.plan(tensors, shape["layers"])
    assert plan.names == list(want) and plan.total_bytes == total
    for name, expect in want.items():
        span = plan.span(name)
        assert span.device_offset == expect["offset"] and span.device_bytes == expect["image"].size, name
        assert (span.rows, span.row_bytes, span.device_row_bytes) == (expect["rows"], expect["row_bytes"], expect["pitch"]), name
        assert [(s.tensor, s.rows.start, s.rows.stop) for s in span.segments] == expect["segments"], name
        np.testing.assert_array_equal(plan.assemble(name), expect["image"], err_msg=name)


def test_a_checkpoint_with_inconsistent_blocks_is_refused_before_any_device_work(tmp_path):
    shape = dict(layers=1, hidden=2048, kv_heads=1, head_dim=128, inter=2048)
    tensors = plan_oracle.synthetic_blocks(np.random.default_rng(4), **shape)
    broken = dict(tensors)
    broken["blocks.0.mlp.up.weight"] = tensors["blocks.0.mlp.up.weight"][:-16]
    broken["blocks.0.mlp.up.weight_scale"] = tensors["blocks.0.mlp.up.weight_scale"][:-16]
    path = tmp_path / "broken.safetensors"
    plan_oracle.write_safetensors(str(path), broken)
    with pytest.raises(k.InvalidArgument, match="interleave shape"):
        Checkpoint(path).plan()
    missing = {n: t for n, t in tensors.items() if n != "blocks.0.attn.wo.weight_scale"}
    plan_oracle.write_safetensors(str(path), missing)
    with pytest.raises(k.InvalidArgument, match="missing tensor blocks.0.attn.wo.weight_scale"):
        Checkpoint(path).plan()
    wrong = dict(tensors)
    wrong["blocks.0.attn.wq.weight"] = tensors["blocks.0.attn.wq.weight"].astype(np.float32)
    plan_oracle.write_safetensors(str(path), wrong)
    with pytest.raises(k.InvalidArgument, match="not int8 ConvRot rows"):
        Checkpoint(path).plan()


# ------------------------------------------------------------------ Session::validate (tests/constructor.rs)
VALIDATE_CHILD = r'''
import ctypes, json, sys
lib = ctypes.CDLL(sys.argv[1])
lib.krea2_session_validate.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_size_t]
lib.krea2_last_error.restype = ctypes.c_char_p
out = []
for path, tokens, layers in json.loads(sys.argv[2]):
    status = lib.krea2_session_validate(path.encode(), tokens, layers)
    out.append([status, lib.krea2_last_error().decode()])
maps = open("/proc/self/maps").read()
print(json.dumps({"results": out, "driver_loaded": "libcuda.so" in maps}))
'''


def validate_in_child(calls):
    """Runs Session::validate in a process that imports neither torch nor anything else that could load the
    CUDA driver, and reports whether the driver library got mapped (tests/constructor.rs:31-36)."""
    import json
    import subprocess
    import sys
    from krea2_hrx_b200 import _lib
    done = subprocess.run([sys.executable, "-c", VALIDATE_CHILD, _lib.LIB_PATH, json.dumps(calls)],
                          capture_output=True, text=True, check=True)
    return json.loads(done.stdout.strip().splitlines()[-1])


def test_an_incomplete_checkpoint_and_invalid_dimensions_are_refused_before_the_gpu(tmp_path):
    """tests/constructor.rs:38-66."""
    path = write(tmp_path, "incomplete.safetensors",
                 '{"blocks.0.attn.wq.weight":{"dtype":"I8","shape":[16,6144],"data_offsets":[0,98304]}}', bytes(98304))
    calls = [[str(path), 16, 1]] * 3
    calls += [[str(path), tokens, layers] for tokens, layers in [(0, 1), (15, 1), (16897, 1), (16, 0), (16, 29), (2 ** 64 - 1, 1)]]
    calls += [[str(tmp_path), 16, 1]]
    report = validate_in_child(calls)
    results = report["results"]
    for status, message in results[:3]:
        assert status == 1 and "missing tensor" in message, message
    for status, message in results[3:9]:
        assert status == 1, message  # InvalidArgument
    assert results[9][0] == 1 and ".safetensors" in results[9][1]
    assert not report["driver_loaded"], "a rejected constructor loaded the CUDA driver"


def test_the_interleaved_gate_and_up_rows_are_validated_before_any_allocation(tmp_path):
    """tests/constructor.rs:68-110: mlp.up carries one scale too few; and separately, weights with no rows."""
    calls = []
    for zero_rows in (False, True):
        entries, offset = [], 0
        for name in ["attn.wq", "attn.wk", "attn.wv", "attn.gate", "attn.wo", "mlp.gate", "mlp.up", "mlp.down"]:
            rows = 0 if zero_rows else 16
            entries.append(f'"blocks.0.{name}.weight":{{"dtype":"I8","shape":[{rows},1],"data_offsets":[{offset},{offset + rows}]}}')
            offset += rows
            scales = 15 if name == "mlp.up" else 16
            entries.append(f'"blocks.0.{name}.weight_scale":{{"dtype":"F32","shape":[{scales}],"data_offsets":[{offset},{offset + scales * 4}]}}')
            offset += scales * 4
        path = write(tmp_path, f"tiny{int(zero_rows)}.safetensors", "{" + ",".join(entries) + "}", bytes(offset))
        calls.append([str(path), 16, 1])
    report = validate_in_child(calls)
    (status, message), (zero_status, zero_message) = report["results"]
    assert status == 1 and "scale count in blocks.0.mlp.up" in message, message
    assert zero_status == 1 and "invalid weight shape" in zero_message, zero_message
    assert not report["driver_loaded"], "a rejected constructor loaded the CUDA driver"
