// Compiled and run by tests/test_host.py: the C++ face of the library against the reference's
// CPU unit tests (src/kernels/shape.rs:115-149) and its refusal of bad session dimensions
// (src/session/mod.rs:278-287), without touching a GPU.
#include <cstdio>
#include <cstring>

#include "krea2_b200.hpp"

#define EXPECT(cond)                                                    \
    do {                                                                \
        if (!(cond)) {                                                  \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main() {
    using namespace krea2;
    namespace shape = kernels::shape;
    EXPECT(shape::gemm_pitch(6144) == 6144 && shape::gemm_pitch(16384) == 16448);
    EXPECT(shape::capacity(4115) == 4160 && shape::capacity(16) == 64 && shape::capacity(2048) == 2080);
    EXPECT(shape::attention_rows(8191) == 16 && shape::attention_rows(8192) == 32);
    EXPECT(shape::gemm_grid_rows(4115) == 17 && shape::gemm_grid_rows(256) == 1 && shape::gemm_grid_rows(16) == 1);
    EXPECT(shape::gemm_tile("gemm_down") == shape::GemmTile::Wide && shape::gemm_tile("gemm_gu") == shape::GemmTile::Narrow);
    EXPECT(std::strcmp(shape::gemm_source("gemm_i8_resid_256", shape::GemmTile::Wide), "gemm_i8_resid_256x256") == 0);
    EXPECT(shape::columns(shape::GemmTile::Wide) == 256 && shape::threads(shape::GemmTile::Wide) == 512);
    EXPECT(!shape::gemm_schedule_rows(4095) && shape::gemm_schedule_rows(4096));
    EXPECT(shape::tokens().first == 16 && shape::tokens().second == 16896);
    EXPECT(session::QKVG == 15360 && session::GATE_OFFSET == 9216);
    kernels::Scalars scalars = kernels::Scalars().index(4608);
    EXPECT(scalars.index_count() == 1 && scalars.indices()[0] == 4608);
    bool refused = false;
    try {
        kernels::Scalars().index(1).index(2).index(3).index(4).index(5);
    } catch (const Internal &) {
        refused = true;
    }
    EXPECT(refused);
    refused = false;
    try {
        session::Session::validate_dimensions(15, 1);
    } catch (const InvalidArgument &e) {
        refused = std::strstr(e.what(), "tokens must be 16..16896") != nullptr;
    }
    EXPECT(refused);
    session::Session::validate_dimensions(4608, 28);
    refused = false;
    try {
        ops::launch(nullptr, "no_such_kernel", {}, kernels::Scalars().index(1), {}, 1, 1, 256);
    } catch (const InvalidArgument &e) {
        refused = std::strstr(e.what(), "no kernel named") != nullptr;
    }
    EXPECT(refused);
    std::printf("host mirror ok\n");
    return 0;
}
