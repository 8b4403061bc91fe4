// Torch-free driver over the C ABI: fill, run, check against a plain CPU loop, time.
// Plays the role of the reference's standalone smoke program (src/test.cu:27-65: fill Q, K, V with
// an LCG, launch, print a corner) but asserts instead of printing numbers to eyeball.
//
//   fa_b200_driver [B R L H [iters]]      exit code 0 = results within tolerance
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "fa_b200.h"

namespace {

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            return 2;                                                                     \
        }                                                                                 \
    } while (0)

// The reference fills with s = (s * 32767) % 65521 (src/test.cu:9-12); any LCG does: this one is a
// 64-bit multiplicative generator summed to a bell-shaped value in about [-2, 2].
struct Lcg {
    uint64_t s;
    float next() {
        float acc = 0.f;
        for (int i = 0; i < 4; ++i) {
            s = s * 6364136223846793005ull + 1442695040888963407ull;
            acc += static_cast<float>((s >> 40) & 0xFFFF) / 65536.f;
        }
        return acc - 2.f;
    }
};

// softmax(q k^T / sqrt(H)) v for one (batch, head, row), in double
void cpu_row(const std::vector<__half>& q, const std::vector<__half>& k, const std::vector<__half>& v, uint32_t L,
             uint32_t F, uint32_t H, uint32_t b, uint32_t h, uint32_t row, std::vector<double>& out) {
    std::vector<double> s(L);
    double mx = -1e300;
    const size_t qo = (static_cast<size_t>(b) * L + row) * F + h * H;
    for (uint32_t j = 0; j < L; ++j) {
        const size_t ko = (static_cast<size_t>(b) * L + j) * F + h * H;
        double acc = 0;
        for (uint32_t d = 0; d < H; ++d) acc += static_cast<double>(__half2float(q[qo + d])) * __half2float(k[ko + d]);
        s[j] = acc / std::sqrt(static_cast<double>(H));
        mx = s[j] > mx ? s[j] : mx;
    }
    double sum = 0;
    for (uint32_t j = 0; j < L; ++j) { s[j] = std::exp(s[j] - mx); sum += s[j]; }
    out.assign(H, 0.0);
    for (uint32_t j = 0; j < L; ++j) {
        const size_t vo = (static_cast<size_t>(b) * L + j) * F + h * H;
        for (uint32_t d = 0; d < H; ++d) out[d] += s[j] / sum * __half2float(v[vo + d]);
    }
}

}  // namespace

int main(int argc, char** argv) {
    uint32_t B = 2, R = 4, L = 600, H = 128;
    int iters = 20;
    if (argc >= 5) { B = std::atoi(argv[1]); R = std::atoi(argv[2]); L = std::atoi(argv[3]); H = std::atoi(argv[4]); }
    if (argc >= 6) iters = std::atoi(argv[5]);
    const uint32_t F = R * H;
    const size_t n = static_cast<size_t>(B) * L * F;

    std::vector<__half> q(n), k(n), v(n), y(n), y2(n);
    Lcg g{179};
    for (size_t i = 0; i < n; ++i) { q[i] = __float2half(g.next()); k[i] = __float2half(g.next()); v[i] = __float2half(g.next()); }

    // host-buffer entry point: one call does everything
    int rc = fa_b200_attention_forward_host(q.data(), k.data(), v.data(), nullptr, y.data(), B, L, F, H, 0, 0, 0);
    if (rc != FA_B200_OK) { std::fprintf(stderr, "host entry point: %s\n", fa_b200_strerror(rc)); return 1; }

    // device-pointer entry point, timed with events
    __half *dq, *dk, *dv, *dy;
    CK(cudaMalloc(&dq, n * 2)); CK(cudaMalloc(&dk, n * 2)); CK(cudaMalloc(&dv, n * 2)); CK(cudaMalloc(&dy, n * 2));
    CK(cudaMemcpy(dq, q.data(), n * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, k.data(), n * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, v.data(), n * 2, cudaMemcpyHostToDevice));
    cudaStream_t st;
    CK(cudaStreamCreate(&st));
    for (int i = 0; i < 3; ++i) {
        rc = fa_b200_attention_forward(dq, dk, dv, nullptr, dy, B, L, F, H, 0, 0, st, 0);
        if (rc != FA_B200_OK) { std::fprintf(stderr, "device entry point: %s\n", fa_b200_strerror(rc)); return 1; }
    }
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    CK(cudaEventRecord(e0, st));
    for (int i = 0; i < iters; ++i) rc |= fa_b200_attention_forward(dq, dk, dv, nullptr, dy, B, L, F, H, 0, 0, st, 0);
    CK(cudaEventRecord(e1, st));
    CK(cudaStreamSynchronize(st));
    if (rc != FA_B200_OK) { std::fprintf(stderr, "device entry point: %s\n", fa_b200_strerror(rc)); return 1; }
    float ms = 0;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    CK(cudaMemcpy(y2.data(), dy, n * 2, cudaMemcpyDeviceToHost));
    uint32_t status[2] = {0, 0};
    rc = fa_b200_read_status(0, status);
    if (rc != FA_B200_OK || status[0] != 0) { std::fprintf(stderr, "device status %u (%d)\n", status[0], rc); return 1; }

    // check: both entry points agree bit for bit; sampled rows against the CPU loop
    size_t differ = 0;
    for (size_t i = 0; i < n; ++i) differ += (__half_as_ushort(y[i]) != __half_as_ushort(y2[i]));
    double max_err = 0, sum_err = 0;
    size_t cnt = 0;
    std::vector<double> ref;
    const uint32_t rows[] = {0u, 1u, L / 3, L / 2, L - 1};
    for (uint32_t b = 0; b < B; ++b)
        for (uint32_t h = 0; h < R; ++h)
            for (uint32_t r : rows) {
                cpu_row(q, k, v, L, F, H, b, h, r, ref);
                const size_t yo = (static_cast<size_t>(b) * L + r) * F + h * H;
                for (uint32_t d = 0; d < H; ++d) {
                    const double e = std::fabs(ref[d] - __half2float(y[yo + d]));
                    max_err = e > max_err ? e : max_err;
                    sum_err += e;
                    ++cnt;
                }
            }
    const double flops = 4.0 * B * R * static_cast<double>(L) * L * H;
    std::printf("B=%u R=%u L=%u H=%u  %.1f us/call  %.1f TFLOP/s  max_abs=%.2e mean_abs=%.2e  entry points differ in %zu values\n",
                B, R, L, H, ms * 1000.f / iters, flops / (ms / iters * 1e-3) / 1e12, max_err, sum_err / cnt, differ);
    const bool ok = differ == 0 && max_err <= 2e-3 * 2.0 && sum_err / cnt <= 2e-4 * 2.0;   // inputs reach |2| here
    return ok ? 0 : 3;
}
