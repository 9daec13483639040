// Exercises the C++ host layer (candy_b200/host/candy_cuda.hpp) against libcandyq.so.
// argv[1] = "nogpu": checks that without a usable GPU the layer fails with an exception (no fallback).
// argv[1] = "gpu":   a small quantized linear; prints the result rows for the Python test to compare.
#include <cstdio>
#include <cstring>
#include <random>

#include "candy_cuda.hpp"

using namespace candy::cuda;

int main(int argc, char **argv) {
    const bool gpu = argc > 1 && !strcmp(argv[1], "gpu");
    if (!gpu) {
        int count = 0;
        cq_device_count(&count);
        if (count > 0) {
            printf("SKIP gpu present\n");
            return 0;
        }
        try {
            auto dev = Device::open(0);
            printf("FAIL opened a device without a GPU\n");
            return 1;
        } catch (const std::runtime_error &e) {
            printf("OK %s\n", e.what());
            return 0;
        }
    }
    auto dev = Device::open(0);
    const int64_t n = 48, k = 256, rows = 6;
    std::mt19937 rng(4);
    std::normal_distribution<float> nd(0.0f, 1.0f);
    std::vector<float> w(n * k), x(rows * k);
    for (auto &v : w) v = 0.02f * nd(rng);
    for (auto &v : x) v = nd(rng);
    QLinear lin(QStorage::quantize(dev, CQ_Q4_0, CQ_ORDER_GO_INTERLEAVED, n, k, w));
    std::vector<float> y = lin.forward(x, {2, 3, k}, CQ_ACT_F32);
    // error behaviour mirrors nn.Linear / MatMulForward
    int errors = 0;
    try {
        lin.forward(x, {k});
    } catch (const std::runtime_error &e) {
        errors += strstr(e.what(), "input rank must be >= 2") != nullptr;
    }
    try {
        lin.forward(std::vector<float>(2 * 128), {2, 128});
    } catch (const std::runtime_error &e) {
        errors += strstr(e.what(), "inner dims mismatch") != nullptr;
    }
    // dump: blocks, x, y for the caller to check against the oracle
    std::vector<uint8_t> blocks = lin.weight().data();
    FILE *f = fopen(argc > 2 ? argv[2] : "host_out.bin", "wb");
    if (!f) return 2;
    fwrite(blocks.data(), 1, blocks.size(), f);
    fwrite(x.data(), 4, x.size(), f);
    fwrite(y.data(), 4, y.size(), f);
    fclose(f);
    printf("OK errors=%d n=%lld k=%lld rows=%lld blocks=%zu\n", errors, (long long)n, (long long)k, (long long)rows, blocks.size());
    return errors == 2 ? 0 : 3;
}
