// The B200 row of the reference's platform table and what the device itself reports, for the host that decides
// which rules fit (engine/gpu/platform/src/platform.rs:11-29 `Row`, :52-70 `Platform`; the row it refines is
// engine/gpu/platform/platforms/cuda-blackwell.json:1-21, which still describes sm_10x as an mma.sync
// [16, 8, 8] / [16, 8, 16] machine).  The row below is the text of tessera_b200/platforms/cuda-b200.json: the
// file a maintainer drops into engine/gpu/platform/platforms/ (it sorts before cuda-blackwell.json, so
// `row_for("cuda sm_100")` finds it first); a test holds the two copies equal.
#include <cstring>
#include <string>

#include "ts_common.cuh"
#include "ts_kernels.cuh"

namespace {

const char kRow[] =
    "{\"matches\": [\"cuda sm_100\"], \"tile\": [128, 256, 16], \"bf16_tile\": [128, 256, 16], \"pdl\": true, "
    "\"check\": [\"sm_100a\"], \"note\": \"B200: tcgen05.mma (128 x N x 16, N up to 256, f32 sums in TMEM) fed by TMA; the "
    "matmul and attention rules launch prebuilt kernels of libtessera_b200.so instead of printing tile text\", "
    "\"b200\": {\"library\": \"libtessera_b200.so\", \"abi\": 1, \"pair_tile\": [256, 256, 16], \"tmem_columns\": 512, "
    "\"cluster\": 8, \"group_bytes\": 232448, \"group_threads\": 1024, \"lanes\": 32, \"units\": 148}}";

}  // namespace

#pragma GCC visibility push(default)
extern "C" int ts_platform_info(char *out, size_t capacity) {
    TS_REQUIRE(out && capacity > 0, "platform info: no buffer");
    std::string text = std::string("{\"row\": ") + kRow + ", \"asked\": ";
    int count = 0, dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0 && cudaGetDevice(&dev) == cudaSuccess &&
        cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
        // what a backend asks its device before the table (platform.rs:72-84 `Asked`)
        int driver = 0, clock_khz = 0, bus_bits = 0;
        cudaDriverGetVersion(&driver);
        cudaDeviceGetAttribute(&clock_khz, cudaDevAttrMemoryClockRate, dev);
        cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, dev);
        char buf[640];
        snprintf(buf, sizeof(buf),
                 "{\"backend\": \"cuda\", \"arch\": \"sm_%d%d\", \"name\": \"%s\", \"driver\": \"%d\", \"units\": %d, "
                 "\"memory\": %llu, \"bandwidth\": %.0f, \"integrated\": false, \"limits\": {\"lanes\": %d, \"group_bytes\": %llu, "
                 "\"group_threads\": %d, \"compiler\": false, \"pdl\": %s}, \"fits\": %s}",
                 prop.major, prop.minor, prop.name, driver, prop.multiProcessorCount, (unsigned long long)prop.totalGlobalMem,
                 2.0 * clock_khz * 1e3 * (bus_bits / 8.0), prop.warpSize, (unsigned long long)prop.sharedMemPerBlockOptin,
                 prop.maxThreadsPerBlock, prop.major >= 9 ? "true" : "false", prop.major == 10 && prop.minor == 0 ? "true" : "false");
        text += buf;
    } else {
        cudaGetLastError();
        text += "null";  // no device: the row alone
    }
    text += "}";
    TS_REQUIRE(text.size() + 1 <= capacity, "platform info: %zu bytes do not fit in %zu", text.size() + 1, capacity);
    memcpy(out, text.c_str(), text.size() + 1);
    return TS_OK;
}
#pragma GCC visibility pop
