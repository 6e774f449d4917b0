// Synthetic weights and activations on the device: the labelled SplitMix64 streams the benchmark
// configurations are defined on.  SplitMix64 (Sources/MferenceValidation/Support/PRNG/SplitMix64.swift:4-24)
// is counter based — draw i is mix(seed + (i+1)*gamma) — so every element can be produced independently;
// stream seeds are root ^ FNV-1a(label) (SeedTree.swift:12-19).
#include <cstdio>
#include <string>
#include <vector>

#include "common.cuh"

namespace mfb {

namespace {

__host__ __device__ __forceinline__ uint64_t splitmix_at(uint64_t seed, uint64_t index) {
    uint64_t z = seed + (index + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

uint64_t seed_for_label(uint64_t root, const std::string& label) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (unsigned char c : label) { h ^= (uint64_t)c; h *= 0x100000001B3ull; }
    return root ^ h;
}

// Box-Muller in double; value i consumes draws 2i and 2i+1.
__device__ __forceinline__ double normal_at(uint64_t seed, uint64_t i) {
    const uint64_t a = splitmix_at(seed, 2 * i), b = splitmix_at(seed, 2 * i + 1);
    const double u1 = (double)((a >> 11) + 1ull) * (1.0 / 9007199254740992.0);
    const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
    return __dmul_rn(sqrt(__dmul_rn(-2.0, log(u1))), cos(__dmul_rn(6.283185307179586476925286766559, u2)));
}

__device__ __forceinline__ void store_value(void* out, uint64_t i, double mean, double z, uint32_t dtype) {
    const float v = __double2float_rn(__dadd_rn(mean, z));
    if (dtype == MFB_DT_F32) ((float*)out)[i] = v;
    else ((uint16_t*)out)[i] = narrow16(v, (int)dtype);
}

__global__ void synth_normal_kernel(uint64_t seed, uint64_t n, double mean, double std, int absolute, uint32_t dtype,
                                    void* out) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        double z = __dmul_rn(normal_at(seed, i), std);
        if (absolute) z = fabs(z);
        store_value(out, i, mean, z, dtype);
    }
}

// grid.y = expert slot, grid.z = sub-tensor (0..8: gate q,s,b, up q,s,b, down q,s,b); grid.x strides the tensor.
__global__ void synth_pool_kernel(const uint64_t* __restrict__ seeds, uint32_t scale_dtype, uint64_t code_words,
                                  uint64_t n_groups, uint8_t* pool, uint64_t slot_stride, mfb_expert_offsets off) {
    const uint32_t e = blockIdx.y, sub = blockIdx.z, kind = sub % 3;
    const uint32_t* o = &off.gate_w;
    uint8_t* dst = pool + (uint64_t)e * slot_stride + o[sub];
    const uint64_t seed = seeds[(uint64_t)e * 9 + sub];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x, first = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (kind == 0) {
        for (uint64_t i = first; i < code_words; i += stride) ((uint64_t*)dst)[i] = splitmix_at(seed, i);
    } else {
        const double std = kind == 1 ? 0.02 : 0.01;
        for (uint64_t i = first; i < n_groups; i += stride) {
            double z = __dmul_rn(normal_at(seed, i), std);
            if (kind == 1) z = fabs(z);
            store_value(dst, i, 0.0, z, scale_dtype);
        }
    }
}

}  // namespace

cudaError_t launch_synth_pool(cudaStream_t s, const uint64_t* seeds_dev, uint32_t n_experts, uint32_t bits,
                              uint32_t scale_dtype, uint32_t d, uint32_t f, uint8_t* pool, uint64_t slot_stride,
                              mfb_expert_offsets off) {
    const uint64_t code_words = (uint64_t)d * f * bits / 64, n_groups = (uint64_t)d * f / 64;
    dim3 grid(32, n_experts, 9);
    synth_pool_kernel<<<grid, 256, 0, s>>>(seeds_dev, scale_dtype, code_words, n_groups, pool, slot_stride, off);
    return cudaGetLastError();
}

cudaError_t launch_synth_normal(cudaStream_t s, uint64_t seed, uint64_t n, double mean, double std, int absolute,
                                uint32_t dtype, void* out) {
    if (n == 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    synth_normal_kernel<<<blocks, 256, 0, s>>>(seed, n, mean, std, absolute, dtype, out);
    return cudaGetLastError();
}

}  // namespace mfb

extern "C" int32_t mfb_synth_expert_pool(void* stream, uint64_t root_seed, uint32_t layer, uint32_t first_expert,
                                         uint32_t n_experts, int32_t shared, uint32_t bits, uint32_t scale_dtype,
                                         uint32_t d, uint32_t f, uint8_t* pool, uint64_t slot_stride) {
    using namespace mfb;
    MFB_REQUIRE(pool != nullptr, MFB_ERR_INVALID_ARGUMENT, "synth: pool is NULL");
    MFB_REQUIRE(bits == 4 || bits == 2 || bits == 8, MFB_ERR_INVALID_ARGUMENT, "synth: bits must be 2, 4 or 8");
    MFB_REQUIRE(scale_dtype == MFB_DT_F16 || scale_dtype == MFB_DT_BF16, MFB_ERR_INVALID_ARGUMENT, "synth: scale dtype");
    MFB_REQUIRE(d % 64 == 0 && f % 64 == 0 && d && f, MFB_ERR_INVALID_ARGUMENT, "synth: d and f must be multiples of 64");
    mfb_expert_offsets off;
    uint64_t blob = 0;
    int32_t rc = mfb_expert_layout(bits, d, f, &off, &blob);
    if (rc != MFB_OK) return rc;
    const uint32_t n = shared ? 1u : n_experts;
    if (n == 0) return MFB_OK;
    MFB_REQUIRE(shared || slot_stride >= blob, MFB_ERR_INVALID_ARGUMENT, "synth: slot stride smaller than a blob");
    static const char* proj[3] = {"gate", "up", "down"};
    static const char* kind[3] = {"q", "s", "b"};
    std::vector<uint64_t> seeds((size_t)n * 9);
    for (uint32_t i = 0; i < n; ++i) {
        char who[48];
        if (shared) snprintf(who, sizeof who, "L%u.shared", layer);
        else snprintf(who, sizeof who, "L%u.e%u", layer, first_expert + i);
        for (int p = 0; p < 3; ++p)
            for (int k = 0; k < 3; ++k)
                seeds[(size_t)i * 9 + p * 3 + k] = seed_for_label(root_seed, std::string(who) + "." + proj[p] + "." + kind[k]);
    }
    uint64_t* dev = nullptr;
    MFB_CUDA(cudaMalloc(&dev, seeds.size() * sizeof(uint64_t)));
    cudaError_t e = cudaMemcpy(dev, seeds.data(), seeds.size() * sizeof(uint64_t), cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = launch_synth_pool((cudaStream_t)stream, dev, n, bits, scale_dtype, d, f,
                              shared ? pool : pool + (uint64_t)first_expert * slot_stride, slot_stride, off);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    cudaFree(dev);
    if (e != cudaSuccess) return cuda_fail(e, "synth pool");
    return MFB_OK;
}

extern "C" int32_t mfb_synth_normal(void* stream, uint64_t root_seed, const char* label, uint64_t n, double mean,
                                    double std, int32_t absolute, uint32_t dtype, void* out) {
    using namespace mfb;
    MFB_REQUIRE(out != nullptr && label != nullptr, MFB_ERR_INVALID_ARGUMENT, "synth: NULL argument");
    MFB_REQUIRE(dtype <= MFB_DT_F32, MFB_ERR_INVALID_ARGUMENT, "synth: dtype");
    MFB_CUDA(launch_synth_normal((cudaStream_t)stream, seed_for_label(root_seed, label), n, mean, std, absolute, dtype, out));
    return MFB_OK;
}
