// Drives gradc::DataLoader (gradcraft_b200/gradc/nn.hpp) and prints one line per batch: batch size and an FNV-1a hash of
// the inputs and of the targets.  Usage: loader_check dataset.bin T n_batches B1 [B2 switch_at]
#include "gradc/gradc.hpp"

#include <cstdio>
#include <cstdlib>

static unsigned long long fnv(const int64_t* p, int64_t n) {
    unsigned long long h = 1469598103934665603ull;
    for (int64_t i = 0; i < n; ++i) { h ^= (unsigned long long)p[i]; h *= 1099511628211ull; }
    return h;
}

int main(int argc, char** argv) {
    if (argc < 5) { std::fprintf(stderr, "usage: loader_check dataset.bin T n_batches B1 [B2 switch_at]\n"); return 2; }
    const int64_t T = std::atoll(argv[2]), n = std::atoll(argv[3]), B1 = std::atoll(argv[4]);
    const int64_t B2 = argc > 6 ? std::atoll(argv[5]) : B1, sw = argc > 6 ? std::atoll(argv[6]) : n;
    gradc::DataLoader loader(argv[1], T, 67);
    for (int64_t i = 0; i < n; ++i) {
        const int64_t B = i < sw ? B1 : B2;
        auto [X, Y] = loader.next_batch(B, T, gradc::Device(gradc::DeviceType::CPU));
        std::printf("%lld %llu %llu\n", (long long)B, fnv(X.data_ptr(), B * T), fnv(Y.data_ptr(), B * T));
    }
    return 0;
}
