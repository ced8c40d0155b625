// V-Smooth preparation for the VC-Attention baseline: k-means grouping of V tokens per head and the
// permute / block-demean / quantise passes.  Restates the Triton kernels of
// src/open_vc_attn/_kernels/blackwell/v_smooth.py of the reference (_assign_values :10-39,
// _accumulate_centers :42-73, _block_stats :76-94, _block_write :97-134) as plain CUDA.
//
// All tensors are for one sequence: V, K, Q are [S,H,128] BF16, centres [H,K,128] BF16.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"

namespace ovc {
namespace {

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }

__device__ __forceinline__ uint8_t to_e4m3(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// labels[h][s] = argmin_k (|c_k|^2 - 2 v.c_k), first index on ties.  One thread per token, the head's
// centres in shared memory as float32.  grid (ceil(S/128), H), 128 threads, smem (K*128 + K) floats.
__global__ void __launch_bounds__(128) assign_kernel(const uint16_t* v, const uint16_t* centers, int32_t* labels,
                                                     long long S, int H, int K) {
    extern __shared__ float smem[];
    float* cen = smem;             // [K][128]
    float* norm = smem + K * kDim;  // [K]
    const int head = blockIdx.y;
    for (int i = threadIdx.x; i < K * kDim; i += 128)
        cen[i] = bf16_bits_to_float(centers[static_cast<long long>(head) * K * kDim + i]);
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += 128) {
        float n = 0.0f;
        for (int c = 0; c < kDim; ++c) n = __fadd_rn(n, __fmul_rn(cen[k * kDim + c], cen[k * kDim + c]));
        norm[k] = n;
    }
    __syncthreads();
    const long long token = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
    if (token >= S) return;
    const uint4* row = reinterpret_cast<const uint4*>(v + (token * H + head) * kDim);
    float x[kDim];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint4 raw = __ldg(row + i);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
    float best = INFINITY;
    int best_k = 0;
    for (int k = 0; k < K; ++k) {
        const float4* c4 = reinterpret_cast<const float4*>(cen + k * kDim);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const float4 c = c4[i];
            dot = fmaf(x[4 * i], c.x, dot);
            dot = fmaf(x[4 * i + 1], c.y, dot);
            dot = fmaf(x[4 * i + 2], c.z, dot);
            dot = fmaf(x[4 * i + 3], c.w, dot);
        }
        const float dist = fmaf(-2.0f, dot, norm[k]);
        if (dist < best) {
            best = dist;
            best_k = k;
        }
    }
    labels[static_cast<long long>(head) * S + token] = best_k;
}

constexpr int kTokensPerCta = 2048;

// Per-cluster sums and counts of one head: a warp takes one token at a time, each lane adds four channels
// to the CTA's shared accumulators; the CTA then adds its totals to global memory.
// grid (ceil(S/2048), H), 256 threads, smem (K*128 + K) floats.
__global__ void __launch_bounds__(256) accumulate_kernel(const uint16_t* v, const int32_t* labels, float* sums,
                                                         float* counts, long long S, int H, int K) {
    extern __shared__ float smem[];
    float* acc = smem;             // [K][128]
    float* cnt = smem + K * kDim;  // [K]
    const int head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < K * kDim + K; i += 256) smem[i] = 0.0f;
    __syncthreads();
    const long long first = static_cast<long long>(blockIdx.x) * kTokensPerCta;
    const long long last = min(first + kTokensPerCta, S);
    for (long long token = first + warp; token < last; token += 8) {
        const int label = labels[static_cast<long long>(head) * S + token];
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(v + (token * H + head) * kDim) + lane);
        float* dst = acc + label * kDim + 4 * lane;
        atomicAdd(dst, __uint_as_float(raw.x << 16));
        atomicAdd(dst + 1, __uint_as_float(raw.x & 0xFFFF0000u));
        atomicAdd(dst + 2, __uint_as_float(raw.y << 16));
        atomicAdd(dst + 3, __uint_as_float(raw.y & 0xFFFF0000u));
        if (lane == 0) atomicAdd(cnt + label, 1.0f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < K * kDim; i += 256)
        if (acc[i] != 0.0f) atomicAdd(sums + static_cast<long long>(head) * K * kDim + i, acc[i]);
    for (int i = threadIdx.x; i < K; i += 256)
        if (cnt[i] != 0.0f) atomicAdd(counts + head * K + i, cnt[i]);
}

// centres = count > 0 ? bf16(sum / count) : centres.  One thread per (head, cluster, channel).
__global__ void update_centers_kernel(const float* sums, const float* counts, uint16_t* centers, long long total) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float count = counts[i / kDim];
    if (count > 0.0f) {
        const __nv_bfloat16 b = __float2bfloat16_rn(__fdiv_rn(sums[i], count));
        centers[i] = *reinterpret_cast<const uint16_t*>(&b);
    }
}

// Per (head, block): V rows gathered in group order, block mean (rows summed in ascending order) and the
// running per-channel maximum of |v - mean|.  One thread per channel.  grid (blocks, H), 128 threads.
__global__ void __launch_bounds__(128) block_stats_kernel(const uint16_t* v, const long long* perm, float* means,
                                                          float* amax, long long S, int H, int blocks) {
    const int block = blockIdx.x, head = blockIdx.y, c = threadIdx.x;
    const long long first = static_cast<long long>(block) * kTile;
    const int count = static_cast<int>(min(static_cast<long long>(kTile), S - first));
    float x[kTile];
    float sum = 0.0f;
#pragma unroll
    for (int r = 0; r < kTile; ++r) {
        float value = 0.0f;
        if (r < count) {
            const long long token = perm[static_cast<long long>(head) * S + first + r];
            value = bf16_bits_to_float(v[(token * H + head) * kDim + c]);
            sum = __fadd_rn(sum, value);
        }
        x[r] = value;
    }
    const float mean = __fdiv_rn(sum, static_cast<float>(count));
    float m = 0.0f;
#pragma unroll
    for (int r = 0; r < kTile; ++r)
        if (r < count) m = fmaxf(m, fabsf(__fsub_rn(x[r], mean)));
    means[(static_cast<long long>(head) * blocks + block) * kDim + c] = mean;
    atomicMax(reinterpret_cast<int*>(amax + head * kDim + c), __float_as_int(m));
}

// Per (head, block): permuted K cast to FP8 (no scale), V residual codes (v - mean) / scale_c, block means in
// code units rounded to BF16, channel scales.  grid (blocks, H), 128 threads.
__global__ void __launch_bounds__(128) block_write_kernel(const uint16_t* k, const uint16_t* v, const long long* perm,
                                                          const float* means, const float* amax, uint8_t* k_out,
                                                          uint8_t* codes, float* means_out, float* scale_out,
                                                          long long S, int H, int blocks) {
    const int block = blockIdx.x, head = blockIdx.y, c = threadIdx.x;
    const long long first = static_cast<long long>(block) * kTile;
    const int count = static_cast<int>(min(static_cast<long long>(kTile), S - first));
    const float a = amax[head * kDim + c];
    const float scale = a > 0.0f ? __fdiv_rn(a, 448.0f) : 1.0f;
    const float mean = means[(static_cast<long long>(head) * blocks + block) * kDim + c];
    for (int r = 0; r < count; ++r) {
        const long long token = perm[static_cast<long long>(head) * S + first + r];
        const long long source = (token * H + head) * kDim + c;
        const long long target = ((first + r) * H + head) * kDim + c;
        const float value = bf16_bits_to_float(v[source]);
        const float code = fminf(fmaxf(__fdiv_rn(__fsub_rn(value, mean), scale), -448.0f), 448.0f);
        codes[target] = to_e4m3(code);
        k_out[target] = to_e4m3(bf16_bits_to_float(k[source]));
    }
    const __nv_bfloat16 rounded = __float2bfloat16_rn(__fdiv_rn(mean, scale));
    means_out[(static_cast<long long>(block) * H + head) * kDim + c] = __bfloat162float(rounded);
    if (block == 0) scale_out[head * kDim + c] = scale;
}

// Plain (unscaled) cast of 16-bit floats to FP8, eight elements per thread.
template <int DT>
__global__ void cast_kernel(const uint16_t* x, uint8_t* out, long long groups) {
    const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= groups) return;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x) + g);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t packed[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float lo, hi;
        if (DT == OVC_BF16) {
            lo = __uint_as_float(w[j] << 16);
            hi = __uint_as_float(w[j] & 0xFFFF0000u);
        } else {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            lo = p.x, hi = p.y;
        }
        const uint32_t pair = __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
        packed[j >> 1] |= pair << (16 * (j & 1));
    }
    reinterpret_cast<uint2*>(out)[g] = make_uint2(packed[0], packed[1]);
}

bool bad(long long S, long long H, long long K) { return S < 1 || H < 1 || H > 65535 || K < 1 || K > 128 || K > S; }

}  // namespace
}  // namespace ovc

using namespace ovc;

extern "C" {

int ovc_vs_assign(const void* v, const void* centers, int32_t* labels, int64_t S, int64_t H, int64_t K, void* stream) {
    if (!v || !centers || !labels || bad(S, H, K) || !aligned16(v)) return OVC_ERR_ARGUMENT;
    const size_t smem = sizeof(float) * (K * kDim + K);
    // Up to 128 centres of 128 floats plus their norms: above the 48 KB default (a per-device setting, host-side only).
    cudaError_t err = cudaFuncSetAttribute(assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * (kDim + 1) * 4);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const dim3 grid(static_cast<unsigned>(ceil_div(S, 128)), static_cast<unsigned>(H));
    assign_kernel<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(v), static_cast<const uint16_t*>(centers), labels, S, static_cast<int>(H), static_cast<int>(K));
    return check_launch();
}

int ovc_vs_accumulate(const void* v, const int32_t* labels, float* sums, float* counts, int64_t S, int64_t H, int64_t K,
                      void* stream) {
    if (!v || !labels || !sums || !counts || bad(S, H, K) || (reinterpret_cast<uintptr_t>(v) & 7u)) return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(sums, 0, sizeof(float) * H * K * kDim, s);
    if (err == cudaSuccess) err = cudaMemsetAsync(counts, 0, sizeof(float) * H * K, s);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const size_t smem = sizeof(float) * (K * kDim + K);
    err = cudaFuncSetAttribute(accumulate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * (kDim + 1) * 4);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const dim3 grid(static_cast<unsigned>(ceil_div(S, kTokensPerCta)), static_cast<unsigned>(H));
    accumulate_kernel<<<grid, 256, smem, s>>>(static_cast<const uint16_t*>(v), labels, sums, counts, S,
                                              static_cast<int>(H), static_cast<int>(K));
    return check_launch();
}

int ovc_vs_update_centers(const float* sums, const float* counts, void* centers, int64_t H, int64_t K, void* stream) {
    if (!sums || !counts || !centers || H < 1 || K < 1) return OVC_ERR_ARGUMENT;
    const long long total = H * K * kDim;
    update_centers_kernel<<<static_cast<unsigned>(ceil_div(total, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        sums, counts, static_cast<uint16_t*>(centers), total);
    return check_launch();
}

int ovc_vs_block_stats(const void* v, const int64_t* permutation, float* means, float* amax, int64_t S, int64_t H,
                       void* stream) {
    if (!v || !permutation || !means || !amax || bad(S, H, 1)) return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(amax, 0, sizeof(float) * H * kDim, s);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const int blocks = static_cast<int>(ceil_div(S, kTile));
    block_stats_kernel<<<dim3(blocks, static_cast<unsigned>(H)), 128, 0, s>>>(
        static_cast<const uint16_t*>(v), reinterpret_cast<const long long*>(permutation), means, amax, S,
        static_cast<int>(H), blocks);
    return check_launch();
}

int ovc_vs_block_write(const void* k, const void* v, const int64_t* permutation, const float* means, const float* amax,
                       void* k_out, void* codes, float* means_out, float* scale, int64_t S, int64_t H, void* stream) {
    if (!k || !v || !permutation || !means || !amax || !k_out || !codes || !means_out || !scale || bad(S, H, 1))
        return OVC_ERR_ARGUMENT;
    const int blocks = static_cast<int>(ceil_div(S, kTile));
    block_write_kernel<<<dim3(blocks, static_cast<unsigned>(H)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(k), static_cast<const uint16_t*>(v), reinterpret_cast<const long long*>(permutation),
        means, amax, static_cast<uint8_t*>(k_out), static_cast<uint8_t*>(codes), means_out, scale, S,
        static_cast<int>(H), blocks);
    return check_launch();
}

int ovc_cast_e4m3(const void* x, int dtype, void* out, int64_t elements, void* stream) {
    if (!x || !out || elements < 8 || elements % 8 != 0 || (dtype != OVC_F16 && dtype != OVC_BF16) || !aligned16(x) ||
        (reinterpret_cast<uintptr_t>(out) & 7u))
        return OVC_ERR_ARGUMENT;
    const long long groups = elements / 8;
    const unsigned grid = static_cast<unsigned>(ceil_div(groups, 256));
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == OVC_BF16) cast_kernel<OVC_BF16><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<uint8_t*>(out), groups);
    else cast_kernel<OVC_F16><<<grid, 256, 0, s>>>(static_cast<const uint16_t*>(x), static_cast<uint8_t*>(out), groups);
    return check_launch();
}

}  // extern "C"
