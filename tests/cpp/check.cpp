// The reference's two `check` functions, written by a C++ caller against the C++ spelling of
// the crate's host surface (include/ferro_kittens.hpp): `gemm::check`
// (examples/src/gemm.rs:591-610: two sizes, traversal widths 8, 1, 3, 6, exact) and
// `flash_forward::check` (examples/src/flash_forward.rs:570-572: 256 queries x 2 heads, causal,
// fp32 out, relative error <= 2^-8). The CPU references come from the oracle (test
// infrastructure); this program is a test, not part of the library.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime_api.h>

#include "ferro_kittens.hpp"

extern "C" {
void fko_gemm_stage(int which, size_t rows, size_t k, uint16_t* out);
size_t fko_gemm_check_c(const uint16_t* observed, size_t m, size_t n, size_t k, double* worst, size_t* first_wrong);
void fko_flash_stage(int which, size_t sequence, size_t heads, uint16_t* out);
void fko_flash_rows(const uint16_t* q, const uint16_t* k, const uint16_t* v, size_t sequence, size_t row0,
                    size_t rows, double scale, int causal, double* out, double* lse);
}

#define CUDA(call)                                                                           \
    do {                                                                                     \
        cudaError_t status_ = (call);                                                        \
        if (status_ != cudaSuccess) {                                                        \
            std::fprintf(stderr, "%s: %s\n", #call, cudaGetErrorString(status_));             \
            std::exit(2);                                                                    \
        }                                                                                    \
    } while (0)

template <class T>
static uint64_t stage(const std::vector<T>& host) {
    void* device = nullptr;
    CUDA(cudaMalloc(&device, host.size() * sizeof(T)));
    CUDA(cudaMemcpy(device, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice));
    return reinterpret_cast<uint64_t>(device);
}

static int gemm_check() {
    const size_t sizes[2][3] = {{512, 256, 256}, {4096, 4096, 256}};
    const uint32_t groups[4] = {kittens::gemm::GROUP, 1, 3, 6};
    for (const auto& size : sizes) {
        const size_t m = size[0], n = size[1], k = size[2];
        std::vector<uint16_t> a(m * k), b(n * k), c(m * n);
        fko_gemm_stage(0, m, k, a.data());
        fko_gemm_stage(1, n, k, b.data());
        const uint64_t a_dev = stage(a), b_dev = stage(b);
        void* c_dev = nullptr;
        uint32_t* status = nullptr;
        CUDA(cudaMalloc(&c_dev, c.size() * 2));
        CUDA(cudaMalloc(reinterpret_cast<void**>(&status), 32));
        double worst = 0.0;
        for (uint32_t group : groups) {
            CUDA(cudaMemset(c_dev, 0, c.size() * 2));
            CUDA(cudaMemset(status, 0, 32));
            kittens::gemm::run(nullptr, a_dev, b_dev, reinterpret_cast<uint64_t>(c_dev), m, n, k, group, status);
            kittens::watchdog::wait(nullptr);
            kittens::check(fk_status_check(status, nullptr));
            CUDA(cudaMemcpy(c.data(), c_dev, c.size() * 2, cudaMemcpyDeviceToHost));
            size_t first = 0;
            const size_t wrong = fko_gemm_check_c(c.data(), m, n, k, &worst, &first);
            if (wrong) {
                std::printf("gemm %zux%zux%zu group %u: %zu of %zu elements wrong, first at %zu\n", m, n, k, group,
                            wrong, m * n, first);
                return 1;
            }
        }
        std::printf("gemm %zux%zux%zu exact at groups [8, 1, 3, 6] (%u CTAs, %u B, worst |rel| %.2e)\n", m, n, k,
                    kittens::gemm::grid(m, n), fk_gemm_shared_bytes(), worst);
        cudaFree(reinterpret_cast<void*>(a_dev));
        cudaFree(reinterpret_cast<void*>(b_dev));
        cudaFree(c_dev);
        cudaFree(status);
    }
    return 0;
}

static int flash_check() {
    const size_t sequence = 256, heads = 2, head = 128;
    std::vector<uint16_t> q(heads * sequence * head), k(q.size()), v(q.size());
    fko_flash_stage(0, sequence, heads, q.data());
    fko_flash_stage(1, sequence, heads, k.data());
    fko_flash_stage(2, sequence, heads, v.data());
    const uint64_t q_dev = stage(q), k_dev = stage(k), v_dev = stage(v);
    float* out_dev = nullptr;
    uint32_t* status = nullptr;
    CUDA(cudaMalloc(reinterpret_cast<void**>(&out_dev), q.size() * 4));
    CUDA(cudaMalloc(reinterpret_cast<void**>(&status), 32));
    CUDA(cudaMemset(out_dev, 0, q.size() * 4));
    CUDA(cudaMemset(status, 0, 32));
    kittens::flash_forward::run(nullptr, q_dev, k_dev, v_dev, 0, out_dev, nullptr, heads, sequence,
                                kittens::flash_forward::SCALE, true, status);
    kittens::watchdog::wait(nullptr);
    kittens::check(fk_status_check(status, nullptr));
    std::vector<float> out(q.size());
    CUDA(cudaMemcpy(out.data(), out_dev, out.size() * 4, cudaMemcpyDeviceToHost));
    double worst = 0.0;
    std::vector<double> expected(sequence * head);
    for (size_t h = 0; h < heads; ++h) {
        fko_flash_rows(q.data() + h * sequence * head, k.data() + h * sequence * head, v.data() + h * sequence * head,
                       sequence, 0, sequence, kittens::flash_forward::SCALE, 1, expected.data(), nullptr);
        for (size_t i = 0; i < sequence * head; ++i) {
            const double error = std::fabs((out[h * sequence * head + i] - expected[i]) / expected[i]);
            if (!(error <= 1.0 / 256.0)) {
                std::printf("flash [%zu, %zu, %zu] = %g, want %g (%.2e)\n", h, i / head, i % head,
                            out[h * sequence * head + i], expected[i], error);
                return 1;
            }
            worst = error > worst ? error : worst;
        }
    }
    std::printf("flash %zux%zux%zu rows attended, worst relative error %.2e\n", heads, sequence, head, worst);
    return 0;
}

int main() {
    try {
        // Bad arguments come back as the crate's messages, before any launch.
        try {
            kittens::gemm::run(nullptr, 0x1000, 0x2000, 0x3000, 512, 256, 256, 0);
            std::printf("a zero traversal width was accepted\n");
            return 1;
        } catch (const kittens::Error& error) {
            if (std::string(error.what()).find("traversal group width of 0") == std::string::npos) throw;
        }
        if (gemm_check()) return 1;
        if (flash_check()) return 1;
    } catch (const kittens::Error& error) {
        std::printf("error %d: %s\n", error.code, error.what());
        return 1;
    }
    std::printf("check ok\n");
    return 0;
}
