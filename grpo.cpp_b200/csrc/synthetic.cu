// Counter-based synthetic logits: every element is a pure function of (seed, global row, column),
// so any split of a batch over ranks produces the same rows, and a host restatement
// (workloads.synthetic_logits_rows) rebuilds any row bit for bit without moving the batch.
//
// The reference measures on arithmetic fixtures built on the host and copied over
// (bench/bench_grpo_loss_cuda.cu:60-102); a 12 GiB batch is built next to where it is used
// instead.  Element (r, v), with c = r * P + v:
//     s  = seed + (2c + 1) * 0x9E3779B97F4A7C15           (the splitmix64 stream of `seed`, outputs 2c+1, 2c+2)
//     h1 = mix64(s), h2 = mix64(s + 0x9E3779B97F4A7C15)
//     k  = sum of the eight 16-bit fields of h1 and h2 - 262140        (an integer in [-262140, 262140])
//     x  = float(k) * scale                                            (one fp32 multiply)
// Eight summed uniforms are close to normal (tails end at 4.9 standard deviations); scale =
// sigma / sqrt(8 * (65536^2 - 1) / 12) gives standard deviation sigma.  Columns [V, P) get `tail_fill`.
#include "common.cuh"

namespace grpo_b200 {
namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

__device__ __forceinline__ int fields16(unsigned long long h) {
    return static_cast<int>(h & 0xffffULL) + static_cast<int>((h >> 16) & 0xffffULL) +
           static_cast<int>((h >> 32) & 0xffffULL) + static_cast<int>(h >> 48);
}

__global__ void __launch_bounds__(256) synthetic_logits_kernel(float* __restrict__ out, long long n_rows,
                                                               long long row_offset, int V, int P, float scale,
                                                               unsigned long long seed, float tail_fill) {
    constexpr unsigned long long kGamma = 0x9E3779B97F4A7C15ULL;
    const long long total = n_rows * static_cast<long long>(P);
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / P;
        const int v = static_cast<int>(i - r * P);
        float x = tail_fill;
        if (v < V) {
            const unsigned long long c = static_cast<unsigned long long>(row_offset + r) * static_cast<unsigned long long>(P) +
                                         static_cast<unsigned long long>(v);
            const unsigned long long s = seed + (2ULL * c + 1ULL) * kGamma;
            const int k = fields16(mix64(s)) + fields16(mix64(s + kGamma)) - 262140;
            x = __fmul_rn(static_cast<float>(k), scale);
        }
        out[i] = x;
    }
}

}  // namespace

cudaError_t launch_synthetic_logits(float* out, long long n_rows, long long row_offset, int V, int P, float scale,
                                    unsigned long long seed, float tail_fill, cudaStream_t stream) {
    const long long total = n_rows * static_cast<long long>(P);
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 32) blocks = 148LL * 32;
    synthetic_logits_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(out, n_rows, row_offset, V, P, scale, seed,
                                                                              tail_fill);
    return cudaGetLastError();
}

}  // namespace grpo_b200
