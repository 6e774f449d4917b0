// Quantised gates and resident projections around the expert FFN: the INT8 affine gate GEMV (Qwen router, shared-expert
// scalar gate), the weights of hash-routed layers, the sigmoid gate on the shared expert's rows, and the INT4 affine
// GEMV of the resident projections.
#include "common.cuh"
#include "select.cuh"

namespace mfb {
namespace {

constexpr int QG_WARPS = 8;

// One warp per (token, row).  Summation order of router_gemv_gemma4_r4 (Sources/Mference/Metal/MoE/moe.metal:102-157)
// and prefill_qwen_shared_scalar_gate (Sources/Mference/Metal/Prefill/prefill.metal:37-80): per 64-element group lane l
// takes elements 2l and 2l+1, acc = fma(s, q0*x0 + q1*x1, acc); acc = fma(b, x0 + x1, acc), every product and sum
// rounded to fp32 (no contraction), then the xor butterfly used for the bf16 gate.
__global__ void __launch_bounds__(QG_WARPS * 32)
gemv_int8_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                 const void* __restrict__ x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                 const uint16_t* __restrict__ effective_scale, uint32_t M, uint32_t N, float* __restrict__ y) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * QG_WARPS + warp, t = blockIdx.y;
    if (r >= M || t >= n_tokens) return;
    const uint32_t groups = N / 64;
    const uint8_t* wr = W + (size_t)r * N;
    float acc = 0.0f;
    for (uint32_t g = 0; g < groups; ++g) {
        const float s = __uint_as_float((uint32_t)scales[(size_t)r * groups + g] << 16);
        const float b = __uint_as_float((uint32_t)biases[(size_t)r * groups + g] << 16);
        const uint32_t i0 = g * 64 + 2 * lane;
        const uint16_t q = *reinterpret_cast<const uint16_t*>(wr + i0);
        float x0 = load_act(x, (size_t)t * ldx + i0, x_dtype), x1 = load_act(x, (size_t)t * ldx + i0 + 1, x_dtype);
        if (effective_scale) {
            x0 = __fmul_rn(x0, __uint_as_float((uint32_t)effective_scale[i0] << 16));
            x1 = __fmul_rn(x1, __uint_as_float((uint32_t)effective_scale[i0 + 1] << 16));
        }
        const float dot = __fadd_rn(__fmul_rn((float)(q & 0xFFu), x0), __fmul_rn((float)(q >> 8), x1));
        acc = fmaf(s, dot, acc);
        acc = fmaf(b, __fadd_rn(x0, x1), acc);
    }
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) y[(size_t)t * M + r] = acc;
}

// router_hash_weights_k6(_par) (moe.metal:852-896): weights of given experts, serial sum in rank order on every lane.
__global__ void hash_weights_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ idx, uint32_t n_tokens,
                                    uint32_t num_experts, uint32_t top_k, float route_scale, uint16_t* __restrict__ out_w) {
    const uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= n_tokens) return;
    float own = 0.0f;
    if (lane < top_k) {
        const uint32_t e = idx[(size_t)t * top_k + lane];
        own = e < num_experts ? sqrtsoftplus(logits[(size_t)t * num_experts + e]) : 0.0f;
    }
    float sum = 0.0f;
    for (uint32_t i = 0; i < top_k; ++i) sum += __shfl_sync(0xFFFFFFFFu, own, i);
    const float inv = route_scale / (sum + 1e-20f);
    if (lane < top_k) out_w[(size_t)t * top_k + lane] = __half_as_ushort(__float2half_rn(own * inv));
}

// rows[t, :] *= sigmoid(fp16(gate[t])): the Qwen shared-expert scalar gate (utility.metal:49-59, prefill.metal:72-79;
// the gate logit passes through fp16 before the sigmoid, as the reference's buffer boundary does).
__global__ void shared_gate_scale_kernel(const float* __restrict__ gate, float* __restrict__ rows, uint64_t row_stride,
                                         uint32_t n_tokens, uint32_t d) {
    const uint32_t t = blockIdx.x;
    if (t >= n_tokens) return;
    const float g = __half2float(__float2half_rn(gate[t]));
    const float m = 1.0f / (1.0f + expf(-g));
    float* row = rows + (size_t)t * row_stride;
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) row[c] *= m;
}

// INT4 affine group-64 GEMV for up to eight activation rows per weight read (dequant_int4_gemv_simd and its multi-x
// form, Sources/Mference/Metal/Quant/dequant_int4.metal:248-288, 343-446): one warp per output row, a lane takes 16
// bytes (32 codes = half a group) of the row per step with one 128-bit load; activations staged once per block in
// shared memory as fp32.  Per group the factored form s * sum(q x) + b * sum(x), fp32.
template <int T>
__global__ void __launch_bounds__(QG_WARPS * 32)
gemv_int4_kernel(const uint8_t* __restrict__ W, const uint16_t* __restrict__ scales, const uint16_t* __restrict__ biases,
                 int scale_dtype, const void* __restrict__ x, int x_dtype, uint32_t ldx, uint32_t M, uint32_t N,
                 float* __restrict__ y) {
    extern __shared__ float xs[];   // [T][N]
    for (uint32_t i = threadIdx.x; i < T * N; i += blockDim.x) xs[i] = load_act(x, (size_t)(i / N) * ldx + i % N, x_dtype);
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t groups = N / 64;
    for (uint32_t r = blockIdx.x * QG_WARPS + warp; r < M; r += gridDim.x * QG_WARPS) {
        const uint8_t* wr = W + (size_t)r * (N / 2);
        float acc[T];
#pragma unroll
        for (int t = 0; t < T; ++t) acc[t] = 0.0f;
        for (uint32_t byte0 = lane * 16; byte0 < N / 2; byte0 += 512) {
            const uint4 q = *reinterpret_cast<const uint4*>(wr + byte0);
            const uint32_t k0 = byte0 * 2, g = k0 / 64;
            const float s = widen16(scales[(size_t)r * groups + g], scale_dtype), b = widen16(biases[(size_t)r * groups + g], scale_dtype);
            const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int t = 0; t < T; ++t) {
                const float* xv = xs + t * N + k0;
                float dot = 0.0f, sx = 0.0f;
#pragma unroll
                for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float xe = xv[wi * 8 + j];
                        dot = fmaf((float)((words[wi] >> (4 * j)) & 15u), xe, dot);
                        sx += xe;
                    }
                acc[t] = fmaf(s, dot, acc[t]);
                acc[t] = fmaf(b, sx, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < T; ++t) {
            float v = acc[t];
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (lane == 0) y[(size_t)t * M + r] = v;
        }
    }
}

template <int T>
cudaError_t launch_gemv_int4_t(cudaStream_t s, const uint8_t* W, const uint16_t* sc, const uint16_t* bi, int sdt, const void* x, int xdt,
                               uint32_t ldx, uint32_t M, uint32_t N, float* y, int sm_count) {
    const size_t smem = (size_t)T * N * sizeof(float);
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(gemv_int4_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const uint32_t blocks_needed = (M + QG_WARPS - 1) / QG_WARPS;
    const uint32_t grid = blocks_needed < (uint32_t)sm_count * 4 ? blocks_needed : (uint32_t)sm_count * 4;
    gemv_int4_kernel<T><<<grid, QG_WARPS * 32, smem, s>>>(W, sc, bi, sdt, x, xdt, ldx, M, N, y);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemv_int8(cudaStream_t s, const uint8_t* W, const void* scales, const void* biases, const void* x, int x_dtype,
                             uint32_t ldx, uint32_t n_tokens, const void* effective_scale, uint32_t M, uint32_t N, float* y) {
    if (n_tokens == 0 || M == 0) return cudaSuccess;
    dim3 grid((M + QG_WARPS - 1) / QG_WARPS, n_tokens);
    gemv_int8_kernel<<<grid, QG_WARPS * 32, 0, s>>>(W, (const uint16_t*)scales, (const uint16_t*)biases, x, x_dtype, ldx, n_tokens,
                                                    (const uint16_t*)effective_scale, M, N, y);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_shared_gate_scale(cudaStream_t s, const float* gate, float* rows, uint64_t row_stride, uint32_t n_tokens, uint32_t d) {
    if (n_tokens == 0) return cudaSuccess;
    shared_gate_scale_kernel<<<n_tokens, 256, 0, s>>>(gate, rows, row_stride, n_tokens, d);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace mfb

using namespace mfb;

extern "C" int32_t mfb_router_hash_weights(void* stream, const float* logits, const uint32_t* idx, uint32_t n_tokens,
                                           uint32_t num_experts, uint32_t top_k, float route_scale, uint16_t* out_w) {
    MFB_REQUIRE(logits && idx && out_w, MFB_ERR_INVALID_ARGUMENT, "hash_weights: NULL argument");
    MFB_REQUIRE(top_k >= 1 && top_k <= MFB_MAX_TOP_K && num_experts >= 1, MFB_ERR_INVALID_ARGUMENT, "hash_weights: top_k / num_experts out of range");
    if (n_tokens == 0) return MFB_OK;
    hash_weights_kernel<<<(n_tokens + 3) / 4, 128, 0, (cudaStream_t)stream>>>(logits, idx, n_tokens, num_experts, top_k, route_scale, out_w);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

extern "C" int32_t mfb_gemv_int8(void* stream, const uint8_t* W, const void* scales_bf16, const void* biases_bf16, const void* x,
                                 uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens, const void* effective_scale_bf16, uint32_t M,
                                 uint32_t N, float* y) {
    MFB_REQUIRE(W && scales_bf16 && biases_bf16 && x && y, MFB_ERR_INVALID_ARGUMENT, "gemv_int8: NULL argument");
    MFB_REQUIRE(N % 64 == 0 && N > 0 && ldx >= N, MFB_ERR_INVALID_ARGUMENT, "gemv_int8: N must be a positive multiple of 64 and ldx >= N");
    MFB_REQUIRE(x_dtype <= MFB_DT_F32, MFB_ERR_INVALID_ARGUMENT, "gemv_int8: activation dtype");
    MFB_CUDA(launch_gemv_int8((cudaStream_t)stream, W, scales_bf16, biases_bf16, x, (int)x_dtype, ldx, n_tokens, effective_scale_bf16, M, N, y));
    return MFB_OK;
}

extern "C" int32_t mfb_gemv_int4(void* stream, const uint8_t* W, const void* scales, const void* biases, uint32_t scale_dtype,
                                 const void* x, uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens, uint32_t M, uint32_t N, float* y) {
    MFB_REQUIRE(W && scales && biases && x && y, MFB_ERR_INVALID_ARGUMENT, "gemv_int4: NULL argument");
    MFB_REQUIRE(N % 64 == 0 && N > 0 && ldx >= N, MFB_ERR_INVALID_ARGUMENT, "gemv_int4: N must be a positive multiple of 64 and ldx >= N");
    MFB_REQUIRE(((uintptr_t)W % 16) == 0 && (N / 2) % 16 == 0, MFB_ERR_INVALID_ARGUMENT, "gemv_int4: rows must be 16-byte aligned");
    MFB_REQUIRE(n_tokens <= 8, MFB_ERR_CAPACITY, "gemv_int4: at most 8 activation rows per call (got %u)", n_tokens);
    MFB_REQUIRE((scale_dtype == MFB_DT_F16 || scale_dtype == MFB_DT_BF16) && x_dtype <= MFB_DT_F32, MFB_ERR_INVALID_ARGUMENT, "gemv_int4: dtype");
    MFB_REQUIRE((size_t)n_tokens * N * 4 <= 200 * 1024, MFB_ERR_UNSUPPORTED_SHAPE, "gemv_int4: the activation rows do not fit in shared memory");
    if (n_tokens == 0 || M == 0) return MFB_OK;
    int dev = 0, sms = 0;
    MFB_CUDA(cudaGetDevice(&dev));
    MFB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    cudaStream_t s = (cudaStream_t)stream;
    const uint16_t *sc = (const uint16_t*)scales, *bi = (const uint16_t*)biases;
    cudaError_t e = cudaSuccess;
    switch (n_tokens) {
        case 1: e = launch_gemv_int4_t<1>(s, W, sc, bi, (int)scale_dtype, x, (int)x_dtype, ldx, M, N, y, sms); break;
        case 2: e = launch_gemv_int4_t<2>(s, W, sc, bi, (int)scale_dtype, x, (int)x_dtype, ldx, M, N, y, sms); break;
        case 3: case 4: {
            // rows beyond n_tokens of the staged block would be read out of bounds: run 4 only on exactly 4
            if (n_tokens == 4) e = launch_gemv_int4_t<4>(s, W, sc, bi, (int)scale_dtype, x, (int)x_dtype, ldx, M, N, y, sms);
            else {
                e = launch_gemv_int4_t<2>(s, W, sc, bi, (int)scale_dtype, x, (int)x_dtype, ldx, M, N, y, sms);
                if (e == cudaSuccess)
                    e = launch_gemv_int4_t<1>(s, W, sc, bi, (int)scale_dtype, (const uint8_t*)x + (size_t)2 * ldx * (x_dtype == MFB_DT_F32 ? 4 : 2),
                                              (int)x_dtype, ldx, M, N, y + (size_t)2 * M, sms);
            }
            break;
        }
        default: {
            // 5 .. 8 rows: four at a time, then the rest
            e = launch_gemv_int4_t<4>(s, W, sc, bi, (int)scale_dtype, x, (int)x_dtype, ldx, M, N, y, sms);
            const uint32_t rest = n_tokens - 4;
            const uint8_t* x2 = (const uint8_t*)x + (size_t)4 * ldx * (x_dtype == MFB_DT_F32 ? 4 : 2);
            float* y2 = y + (size_t)4 * M;
            if (e == cudaSuccess) {
                int32_t rc = mfb_gemv_int4(stream, W, scales, biases, scale_dtype, x2, x_dtype, ldx, rest, M, N, y2);
                if (rc) return rc;
            }
        }
    }
    count_launches(1);
    MFB_CUDA(e);
    return MFB_OK;
}
