// One W8A8 projection on bf16 tensors, the whole of Quantized::forward
// (src/training/quantized.rs:51-112) as one call: bf16 -> f16 transport, prepare_plain_i8,
// gemm_i8_256, f16 -> bf16.  The four intermediates the reference takes from its buffer pool
// (:55-58) live in a workspace the caller passes.
#include <mutex>

#include "common.cuh"

namespace krea2 {
namespace {

// Workspace of krea2_quantized_forward_static: part of the library image, so every GPU that
// loads the library carries these 4 MiB until the process exits.  In host code this name is only
// a handle for cudaGetSymbolAddress; the device address it resolves to is what kernels receive.
constexpr size_t kStaticWorkspaceBytes = size_t(4) << 20;
static __device__ __align__(256) unsigned char g_static_workspace[kStaticWorkspaceBytes];

// Never launched.  It names the array in device code so that the device image keeps it even
// though every other use goes through cudaGetSymbolAddress on the host.
__global__ void static_workspace_anchor(unsigned char **out) { *out = g_static_workspace; }

size_t align256(size_t n) { return (n + 255) / 256 * 256; }

struct Layout {
    size_t transport, quantized, scales, out_f16, total;
};

Layout workspace_layout(size_t rows, size_t inputs, size_t outputs) {
    const size_t pitch = krea2_shape_gemm_pitch(inputs);
    Layout l;
    l.transport = 0;
    l.quantized = l.transport + align256(rows * inputs * 2);
    l.scales = l.quantized + align256(rows * pitch);
    l.out_f16 = l.scales + align256(rows * 4);
    l.total = l.out_f16 + align256(rows * outputs * 2);
    return l;
}

}  // namespace

int quantized_forward_in(cudaStream_t stream, size_t rows, const void *x, const void *weight, const float *scales,
                         void *out, size_t inputs, size_t outputs, uint8_t *workspace) {
    const size_t pitch = krea2_shape_gemm_pitch(inputs);
    const Layout l = workspace_layout(rows, inputs, outputs);
    uint8_t *transport = workspace + l.transport, *quantized = workspace + l.quantized;
    float *token_scales = reinterpret_cast<float *>(workspace + l.scales);
    uint8_t *out_f16 = workspace + l.out_f16;
    if (int s = krea2_lora_transport(stream, rows * inputs, x, transport, 1)) return s;
    if (int s = krea2_prepare_plain_i8(stream, rows, transport, quantized, token_scales, inputs, pitch)) return s;
    if (int s = krea2_gemm_i8_256(stream, rows, quantized, weight, scales, token_scales, out_f16, inputs, pitch, outputs,
                                  krea2_shape_gemm_m_group()))
        return s;
    return krea2_lora_transport(stream, rows * outputs, out_f16, out, 2);
}

int check_quantized(size_t rows, const void *x, const void *weight, const float *scales, void *out, size_t inputs,
                    size_t outputs) {
    KREA2_REQUIRE(rows >= 1 && rows <= 1048576, "quantized_forward: rows %zu outside 1..1048576", rows);
    KREA2_REQUIRE(inputs >= 2048 && inputs <= 32768 && inputs % 2048 == 0,
                  "quantized_forward: inputs %zu must be a multiple of 2048 in 2048..32768", inputs);
    KREA2_REQUIRE(outputs >= 128 && outputs <= 32768 && outputs % 128 == 0,
                  "quantized_forward: outputs %zu must be a multiple of 128 up to 32768", outputs);
    KREA2_REQUIRE(x && weight && scales && out, "quantized_forward: null buffer");
    KREA2_REQUIRE(aligned16(x) && aligned16(weight) && aligned16(scales) && aligned16(out),
                  "quantized_forward: buffers must be 16-byte aligned");
    return KREA2_OK;
}

}  // namespace krea2

using namespace krea2;

extern "C" size_t krea2_quantized_workspace_bytes(size_t rows, size_t inputs, size_t outputs) {
    return workspace_layout(rows, inputs, outputs).total;
}

extern "C" int krea2_quantized_forward(krea2_stream stream, size_t rows, const void *x, const void *weight,
                                       const float *scales, void *out, size_t inputs, size_t outputs,
                                       void *workspace, size_t workspace_bytes) {
    clear_error();
    if (int s = check_quantized(rows, x, weight, scales, out, inputs, outputs)) return s;
    const size_t need = workspace_layout(rows, inputs, outputs).total;
    KREA2_REQUIRE(workspace && aligned16(workspace) && workspace_bytes >= need,
                  "quantized_forward: the workspace spans %zu bytes, %zu are needed", workspace_bytes, need);
    return quantized_forward_in(static_cast<cudaStream_t>(stream), rows, x, weight, scales, out, inputs, outputs,
                                static_cast<uint8_t *>(workspace));
}

extern "C" size_t krea2_quantized_static_workspace_bytes(void) { return kStaticWorkspaceBytes; }

extern "C" int krea2_quantized_forward_static(krea2_stream stream, size_t rows, const void *x, const void *weight,
                                              const float *scales, void *out, size_t inputs, size_t outputs) {
    clear_error();
    if (int s = check_quantized(rows, x, weight, scales, out, inputs, outputs)) return s;
    const size_t need = workspace_layout(rows, inputs, outputs).total;
    KREA2_REQUIRE(need <= kStaticWorkspaceBytes,
                  "quantized_forward_static: %zu rows of %zu -> %zu need %zu bytes of scratch, the built-in "
                  "workspace holds %zu; use krea2_quantized_forward with a caller workspace",
                  rows, inputs, outputs, need, kStaticWorkspaceBytes);
    // Per device, once, with that device current: resolve the device address of the array.
    static std::mutex lock;
    static uint8_t *address[64] = {nullptr};
    int device = 0;
    KREA2_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(KREA2_INTERNAL, "device index %d out of range", device);
    // The array handed to the kernels is the current device's: a stream or buffers of another device would
    // make that device's kernels dereference an address that is not mapped there.
    if (stream) {
        int stream_device = device;
        if (cudaStreamGetDevice(static_cast<cudaStream_t>(stream), &stream_device) != cudaSuccess) {
            cudaGetLastError();  // a driver without the query: the buffer check below still applies
            stream_device = device;
        }
        KREA2_REQUIRE(stream_device == device,
                      "quantized_forward_static: the stream belongs to device %d but device %d is current", stream_device,
                      device);
    }
    cudaPointerAttributes where{};
    if (cudaPointerGetAttributes(&where, x) != cudaSuccess) cudaGetLastError();
    else
        KREA2_REQUIRE(where.type != cudaMemoryTypeDevice || where.device == device,
                      "quantized_forward_static: x lives on device %d but device %d is current", where.device, device);
    uint8_t *workspace = nullptr;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (!address[device]) {
            void *resolved = nullptr;
            cudaError_t status = cudaGetSymbolAddress(&resolved, g_static_workspace);
            if (status != cudaSuccess)
                return fail(KREA2_RUNTIME, "cudaGetSymbolAddress failed for the built-in workspace: %s",
                            cudaGetErrorString(status));
            address[device] = static_cast<uint8_t *>(resolved);
        }
        workspace = address[device];
    }
    return quantized_forward_in(static_cast<cudaStream_t>(stream), rows, x, weight, scales, out, inputs, outputs,
                                workspace);
}
