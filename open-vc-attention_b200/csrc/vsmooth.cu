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

__device__ __forceinline__ uint8_t to_e4m3(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// labels[h][s] = argmin_k (|c_k|^2 - 2 v.c_k), first index on ties.  The products v.c_k are a small GEMM
// ([tokens x 128] x [128 x K], K <= 128) on the tensor cores: mma.sync m16n8k16, BF16 inputs, FP32 accumulators.
// A warp owns 32 tokens (two 16-row tiles) whose rows it reads straight from global memory with 16-byte
// loads: lane (r, q) = (lane / 4, lane % 4) takes the 16-byte chunks q, q + 4, q + 8, q + 12 of rows r and
// r + 8.  The order in which the 128 channels are fed to the MMAs is free, so the k-slots of step `ks` are
// simply the words the lane already holds (2 ks and 2 ks + 1 of its 16); the centre words are fetched from
// shared memory with the same word index.  grid (ceil(S/128), H), 128 threads,
// smem K * 68 words (BF16 centres, rows padded by 4 words) + K floats (norms).
constexpr int kCenterStride = 68;  // 32-bit words per centre row in shared memory

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128) assign_kernel(const uint16_t* v, const uint16_t* centers, int32_t* labels,
                                                     long long S, int H, int K) {
    extern __shared__ uint32_t smem_words[];
    uint32_t* cen = smem_words;                                             // [K8][kCenterStride]
    const int K8 = (K + 7) / 8 * 8;
    float* norm = reinterpret_cast<float*>(smem_words + K8 * kCenterStride);  // [K8]
    const int head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t* cen_g = reinterpret_cast<const uint32_t*>(centers + static_cast<long long>(head) * K * kDim);
    for (int i = threadIdx.x; i < K8 * 64; i += 128) {
        const int k = i >> 6, w = i & 63;
        cen[k * kCenterStride + w] = k < K ? cen_g[k * 64 + w] : 0u;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < K8; k += 128) {
        float n = 0.0f;
        for (int w = 0; w < 64; ++w) {
            const uint32_t x = cen[k * kCenterStride + w];
            const float lo = __uint_as_float(x << 16), hi = __uint_as_float(x & 0xFFFF0000u);
            n = __fadd_rn(n, __fmul_rn(lo, lo));
            n = __fadd_rn(n, __fmul_rn(hi, hi));
        }
        norm[k] = k < K ? n : INFINITY;
    }
    __syncthreads();

    const int r = lane >> 2, q = lane & 3;
    const long long token0 = static_cast<long long>(blockIdx.x) * 128 + warp * 32;
    // a[tile][half][i]: word i (of 16) of row r + 8 * half of the 16-row tile
    uint32_t a[2][2][16];
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const long long token = token0 + 16 * tile + 8 * half + r;
            const uint4* row = reinterpret_cast<const uint4*>(v + (min(token, S - 1) * H + head) * kDim);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 x = __ldg(row + q + 4 * j);
                a[tile][half][4 * j] = x.x, a[tile][half][4 * j + 1] = x.y, a[tile][half][4 * j + 2] = x.z, a[tile][half][4 * j + 3] = x.w;
            }
        }
    float best[2][2] = {{INFINITY, INFINITY}, {INFINITY, INFINITY}};
    int best_k[2][2] = {{0, 0}, {0, 0}};
    for (int nt = 0; nt < K8 / 8; ++nt) {
        float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
        const uint32_t* crow = cen + (8 * nt + r) * kCenterStride;  // B fragment: centre n = 8 nt + lane / 4
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            // word index of the lane's words 2 ks and 2 ks + 1 within the 64-word row
            const int i0 = 2 * ks, i1 = 2 * ks + 1;
            const uint32_t b0 = crow[4 * (q + 4 * (i0 >> 2)) + (i0 & 3)];
            const uint32_t b1 = crow[4 * (q + 4 * (i1 >> 2)) + (i1 & 3)];
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                const uint32_t frag[4] = {a[tile][0][i0], a[tile][1][i0], a[tile][0][i1], a[tile][1][i1]};
                mma_bf16(acc[tile], frag, b0, b1);
            }
        }
        // acc[tile][0..1]: row r, centres 8 nt + 2 q + {0,1}; acc[tile][2..3]: row r + 8, same centres
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int k = 8 * nt + 2 * q + e;
                    const float dist = fmaf(-2.0f, acc[tile][2 * half + e], norm[k]);
                    if (dist < best[tile][half]) best[tile][half] = dist, best_k[tile][half] = k;
                }
    }
    // The four lanes of a row hold disjoint centres: smallest distance wins, smaller index on ties.
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            float d = best[tile][half];
            int k = best_k[tile][half];
#pragma unroll
            for (int step = 1; step <= 2; step <<= 1) {
                const float od = __shfl_xor_sync(0xFFFFFFFFu, d, step);
                const int ok = __shfl_xor_sync(0xFFFFFFFFu, k, step);
                if (od < d || (od == d && ok < k)) d = od, k = ok;
            }
            const long long token = token0 + 16 * tile + 8 * half + r;
            if (q == 0 && token < S) labels[static_cast<long long>(head) * S + token] = k;
        }
}

constexpr int kTokensPerCta = 1024;

// Per-cluster sums and counts of one head: a warp takes eight tokens at a time, each lane adds four channels
// per token to the CTA's shared accumulators; the CTA then adds its totals to global memory.
// grid (ceil(S/1024), H), 256 threads, smem (K*128 + K) floats.
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
    // Eight tokens per warp and step, so that eight row loads are in flight per lane.
    for (long long base = first + 8 * warp; base < last; base += 64) {
        const int my_label = (lane < 8 && base + lane < last) ? __ldg(labels + static_cast<long long>(head) * S + base + lane) : -1;
        uint2 raw[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            raw[t] = make_uint2(0u, 0u);
            if (base + t < last) raw[t] = __ldg(reinterpret_cast<const uint2*>(v + ((base + t) * H + head) * kDim) + lane);
        }
#pragma unroll
        for (int t = 0; t < 8; ++t) {
            const int label = __shfl_sync(0xFFFFFFFFu, my_label, t);
            if (label < 0) continue;
            // Channel 4 * lane + j lives at word 32 * j + lane of its cluster's row: one bank per lane.
            float* dst = acc + label * kDim + lane;
            atomicAdd(dst, __uint_as_float(raw[t].x << 16));
            atomicAdd(dst + 32, __uint_as_float(raw[t].x & 0xFFFF0000u));
            atomicAdd(dst + 64, __uint_as_float(raw[t].y << 16));
            atomicAdd(dst + 96, __uint_as_float(raw[t].y & 0xFFFF0000u));
            if (lane == 0) atomicAdd(cnt + label, 1.0f);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < K * kDim; i += 256) {
        const int w = i & (kDim - 1);  // word 32 * j + lane holds channel 4 * lane + j
        const int channel = 4 * (w & 31) + (w >> 5);
        if (acc[i] != 0.0f) atomicAdd(sums + static_cast<long long>(head) * K * kDim + (i - w) + channel, acc[i]);
    }
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

// The two block passes share one tiling: 256 threads per (block, head); thread t owns the eight channels
// 8*(t%16).. of the eight rows t/16 + 16 i of the 128-row block, so every load is 16 bytes and a warp reads
// two whole 256-byte rows (gathered through the permutation) per instruction.
__device__ __forceinline__ void load_rows8(const uint16_t* x, const long long* perm_row, long long first, int count, int H,
                                           int head, int rg, int cg, float (&val)[8][8]) {
    uint4 raw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = rg + 16 * i;
        raw[i] = make_uint4(0u, 0u, 0u, 0u);
        if (r < count) {
            const long long token = __ldg(perm_row + first + r);
            raw[i] = __ldg(reinterpret_cast<const uint4*>(x + (token * H + head) * kDim) + cg);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            val[i][2 * j] = __uint_as_float(w[j] << 16);
            val[i][2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
        }
    }
}

// Per (head, block): block mean and the running per-channel maximum of |v - mean|.  The sum of a channel
// is taken in a fixed order, so that results do not depend on scheduling: rows r = g + 16 i are added in
// ascending i into sixteen partial sums, which are then added in ascending g (rows past the end count as 0).
// grid (blocks, H), 256 threads.
__global__ void __launch_bounds__(256) block_stats_kernel(const uint16_t* v, const long long* perm, float* means,
                                                          float* amax, long long S, int H, int blocks) {
    __shared__ float partial[16][kDim];
    __shared__ float mean_s[kDim];
    const int block = blockIdx.x, head = blockIdx.y;
    const int cg = threadIdx.x & 15, rg = threadIdx.x >> 4;
    const long long first = static_cast<long long>(block) * kTile;
    const int count = static_cast<int>(min(static_cast<long long>(kTile), S - first));
    float val[8][8];
    load_rows8(v, perm + static_cast<long long>(head) * S, first, count, H, head, rg, cg, val);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        float sum = val[0][c];
#pragma unroll
        for (int i = 1; i < 8; ++i) sum = __fadd_rn(sum, val[i][c]);
        partial[rg][8 * cg + c] = sum;
    }
    __syncthreads();
    if (threadIdx.x < kDim) {
        float total = partial[0][threadIdx.x];
#pragma unroll
        for (int g = 1; g < 16; ++g) total = __fadd_rn(total, partial[g][threadIdx.x]);
        const float mean = div_full(total, static_cast<float>(count));
        mean_s[threadIdx.x] = mean;
        means[(static_cast<long long>(head) * blocks + block) * kDim + threadIdx.x] = mean;
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float mean = mean_s[8 * cg + c];
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (rg + 16 * i < count) m = fmaxf(m, fabsf(__fsub_rn(val[i][c], mean)));
        partial[rg][8 * cg + c] = m;
    }
    __syncthreads();
    if (threadIdx.x < kDim) {
        float m = partial[0][threadIdx.x];
#pragma unroll
        for (int g = 1; g < 16; ++g) m = fmaxf(m, partial[g][threadIdx.x]);
        atomicMax(reinterpret_cast<int*>(amax + head * kDim + threadIdx.x), __float_as_int(m));
    }
}

// Per (head, block): permuted K cast to FP8 (no scale), V residual codes (v - mean) / scale_c, block means in
// code units rounded to BF16, channel scales.  Same tiling; code rows are written as 8-byte pieces of a
// 128-byte row.  grid (blocks, H), 256 threads.
__global__ void __launch_bounds__(256) block_write_kernel(const uint16_t* k, const uint16_t* v, const long long* perm,
                                                          const float* means, const float* amax, uint8_t* k_out,
                                                          uint8_t* codes, float* means_out, float* scale_out,
                                                          long long S, int H, int blocks) {
    const int block = blockIdx.x, head = blockIdx.y;
    const int cg = threadIdx.x & 15, rg = threadIdx.x >> 4;
    const long long first = static_cast<long long>(block) * kTile;
    const int count = static_cast<int>(min(static_cast<long long>(kTile), S - first));
    float scale[8], mean[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float a = amax[head * kDim + 8 * cg + c];
        scale[c] = a > 0.0f ? div_full(a, 448.0f) : 1.0f;
        mean[c] = means[(static_cast<long long>(head) * blocks + block) * kDim + 8 * cg + c];
    }
    const long long* perm_row = perm + static_cast<long long>(head) * S;
    float val[8][8];
    load_rows8(v, perm_row, first, count, H, head, rg, cg, val);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = rg + 16 * i;
        if (r >= count) continue;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float code = fminf(fmaxf(div_full(__fsub_rn(val[i][c], mean[c]), scale[c]), -448.0f), 448.0f);
            const uint32_t byte = to_e4m3(code);
            if (c < 4) lo |= byte << (8 * c);
            else hi |= byte << (8 * (c - 4));
        }
        *reinterpret_cast<uint2*>(codes + ((first + r) * H + head) * kDim + 8 * cg) = make_uint2(lo, hi);
    }
    load_rows8(k, perm_row, first, count, H, head, rg, cg, val);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = rg + 16 * i;
        if (r >= count) continue;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t byte = to_e4m3(val[i][c]);
            if (c < 4) lo |= byte << (8 * c);
            else hi |= byte << (8 * (c - 4));
        }
        *reinterpret_cast<uint2*>(k_out + ((first + r) * H + head) * kDim + 8 * cg) = make_uint2(lo, hi);
    }
    if (rg == 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const __nv_bfloat16 rounded = __float2bfloat16_rn(div_full(mean[c], scale[c]));
            means_out[(static_cast<long long>(block) * H + head) * kDim + 8 * cg + c] = __bfloat162float(rounded);
            if (block == 0) scale_out[head * kDim + 8 * cg + c] = scale[c];
        }
    }
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
    if (!v || !centers || !labels || bad(S, H, K) || !aligned16(v) || (reinterpret_cast<uintptr_t>(centers) & 3u))
        return OVC_ERR_ARGUMENT;
    const int64_t K8 = (K + 7) / 8 * 8;
    const size_t smem = sizeof(uint32_t) * K8 * kCenterStride + sizeof(float) * K8;
    // Up to 128 padded centre rows plus their norms: no more than 35.3 KB, inside the default limit.
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
    if (!v || !permutation || !means || !amax || bad(S, H, 1) || !aligned16(v) ||
        (reinterpret_cast<uintptr_t>(permutation) & 7u))
        return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(amax, 0, sizeof(float) * H * kDim, s);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const int blocks = static_cast<int>(ceil_div(S, kTile));
    block_stats_kernel<<<dim3(blocks, static_cast<unsigned>(H)), 256, 0, s>>>(
        static_cast<const uint16_t*>(v), reinterpret_cast<const long long*>(permutation), means, amax, S,
        static_cast<int>(H), blocks);
    return check_launch();
}

int ovc_vs_block_write(const void* k, const void* v, const int64_t* permutation, const float* means, const float* amax,
                       void* k_out, void* codes, float* means_out, float* scale, int64_t S, int64_t H, void* stream) {
    if (!k || !v || !permutation || !means || !amax || !k_out || !codes || !means_out || !scale || bad(S, H, 1) ||
        !aligned16(k) || !aligned16(v) || (reinterpret_cast<uintptr_t>(permutation) & 7u) ||
        (reinterpret_cast<uintptr_t>(k_out) & 7u) || (reinterpret_cast<uintptr_t>(codes) & 7u))
        return OVC_ERR_ARGUMENT;
    const int blocks = static_cast<int>(ceil_div(S, kTile));
    block_write_kernel<<<dim3(blocks, static_cast<unsigned>(H)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
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
