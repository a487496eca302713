"""krea2_quantized_forward_static: the W8A8 projection for hosts that cannot give the library a
workspace or let it allocate one (a plugin inside an engine with a frozen device arena, a serving
loop that must stay out of the allocator).  Its scratch is an array inside the library image, so
the call is checked here, through the C ABI, against krea2_quantized_forward with an explicit
workspace: same bits, twice in a row (the second call finds the first call's bytes in the array).

Collected last on purpose: a run that stops at the first failure has then already run every
other test."""
import ctypes

import numpy as np
import pytest
import torch

import kat

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")


def _call_pair(rows, inputs, outputs, seed):
    from krea2_hrx_b200 import shape
    lib = k.lib()
    rng = np.random.default_rng(seed)
    pitch = shape.gemm_pitch(inputs)
    weight = torch.zeros((outputs, pitch), dtype=torch.int8)
    weight[:, :inputs] = torch.from_numpy(rng.integers(-127, 128, size=(outputs, inputs)).astype(np.int8))
    weight = weight.cuda()
    scales = torch.from_numpy(rng.uniform(1e-3, 1e-2, size=outputs).astype(np.float32)).cuda()
    x = torch.from_numpy(kat.bf16_bits_from_f32(rng.standard_normal((rows, inputs)).astype(np.float32)).view(np.int16))
    x = x.view(torch.bfloat16).cuda()
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.krea2_quantized_workspace_bytes(rows, inputs, outputs)
    workspace = torch.empty(need, dtype=torch.uint8, device="cuda")
    want = torch.zeros((rows, outputs), dtype=torch.bfloat16, device="cuda")
    status = lib.krea2_quantized_forward(stream, rows, x.data_ptr(), weight.data_ptr(), scales.data_ptr(),
                                         want.data_ptr(), inputs, outputs, workspace.data_ptr(), need)
    assert status == 0, lib.krea2_last_error()
    got = torch.zeros((rows, outputs), dtype=torch.bfloat16, device="cuda")
    status = lib.krea2_quantized_forward_static(stream, rows, x.data_ptr(), weight.data_ptr(), scales.data_ptr(),
                                                got.data_ptr(), inputs, outputs)
    assert status == 0, lib.krea2_last_error()
    torch.cuda.synchronize()
    return got.view(torch.int16).cpu().numpy(), want.view(torch.int16).cpu().numpy()


def test_static_workspace_call_matches_the_caller_workspace_call_twice_in_a_row():
    assert k.lib().krea2_quantized_static_workspace_bytes() == 4 << 20
    # two calls back to back with different shapes and data: the second one runs over the bytes the
    # first one left in the shared array
    got, want = _call_pair(rows=48, inputs=6144, outputs=512, seed=1)
    np.testing.assert_array_equal(got, want)
    got, want = _call_pair(rows=9, inputs=16384, outputs=256, seed=2)
    np.testing.assert_array_equal(got, want)
    assert k.device_status() == 0


def test_static_workspace_call_refuses_what_does_not_fit():
    lib = k.lib()
    buf = torch.zeros(1024, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    rows, inputs, outputs = 512, 16384, 6144
    assert lib.krea2_quantized_workspace_bytes(rows, inputs, outputs) > lib.krea2_quantized_static_workspace_bytes()
    status = lib.krea2_quantized_forward_static(None, rows, p, p, p, p, inputs, outputs)
    assert status == 1
    message = lib.krea2_last_error().decode()
    assert "built-in" in message and "krea2_quantized_forward" in message
