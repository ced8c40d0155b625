// FP8 input preparation for ExpCast attention: HBM-bound kernels for sm_100a.
//
// Arithmetic follows the reference's Triton kernels operation for operation
// (src/open_vc_attn/quantization.py, src/open_vc_attn/preparation.py,
// src/open_vc_attn/v_repair.py in the reference project): amax floored at 1e-12,
// one division 448/amax, one multiply, clamp to +-448, round-to-nearest-even E4M3
// cast.  Triton lowers a float32 `/` to div.full.f32 (the dividend times an
// approximate reciprocal, not the IEEE quotient) and contracts `x - c * d` into one
// FMA; the kernels here issue the same instructions, because inputs with few mantissa
// bits put many scaled values exactly on E4M3 rounding ties, where the last bit of the
// scale decides the code.  Every global access is a 16-byte (or 8-byte for FP8 rows) vector
// access covering whole 128-byte lines per warp.

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>

#include "common.cuh"

namespace ovc {

static thread_local int g_last_cuda_error = 0;
void set_last_cuda_error(int code) { g_last_cuda_error = code; }

namespace {

constexpr float kQMax = 448.0f;
constexpr float kFloor = 1e-12f;

__device__ __forceinline__ uint4 ld_stream(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

// Eight 16-bit floats (one uint4) widened exactly to float32.
template <int DT>
__device__ __forceinline__ void widen8(const uint4& raw, float (&f)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (DT == OVC_BF16) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        } else {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
}

__device__ __forceinline__ float absmax8(const float (&f)[8], float m) {
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
    return m;
}

__device__ __forceinline__ float clamp448(float x) { return fminf(fmaxf(x, -kQMax), kQMax); }

// Four float32 -> four E4M3 bytes (a in the lowest byte), RNE.
__device__ __forceinline__ uint32_t cast4(float a, float b, float c, float d) {
    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return lo | (hi << 16);
}

__device__ __forceinline__ uint2 quantize8(const float (&f)[8], float scale) {
    uint2 out;
    out.x = cast4(clamp448(__fmul_rn(f[0], scale)), clamp448(__fmul_rn(f[1], scale)),
                  clamp448(__fmul_rn(f[2], scale)), clamp448(__fmul_rn(f[3], scale)));
    out.y = cast4(clamp448(__fmul_rn(f[4], scale)), clamp448(__fmul_rn(f[5], scale)),
                  clamp448(__fmul_rn(f[6], scale)), clamp448(__fmul_rn(f[7], scale)));
    return out;
}

__device__ __forceinline__ float4 decode4(uint32_t codes) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(codes & 0xFFFFu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(codes >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ float warp_max(float m) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
    return m;
}

// Max over the 128 threads of a CTA; every thread gets the result.
__device__ __forceinline__ float cta128_max(float m) {
    __shared__ float part[4];
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
    __syncthreads();
    return fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
}

struct BlockQuantArgs {
    const void* x[2];
    uint8_t* codes[2];
    float* descale[2];
    long long descale_stride[2];
    int sources;       // 1 or 2 tensors quantised by one launch
    float* amax_init;  // optional [H]: reset to 0 by the (block 0, source 0) CTAs
};

// Max over the 256 threads of a CTA; every thread gets the result.  `part` is caller-provided shared
// memory (8 floats) so that consecutive reductions can alternate between two buffers.
__device__ __forceinline__ float cta256_max(float m, float* part) {
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
    __syncthreads();
    return fmaxf(fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3])),
                 fmaxf(fmaxf(part[4], part[5]), fmaxf(part[6], part[7])));
}

constexpr int kBlocksPerCta = 4;  // consecutive 128-token blocks handled by one CTA of the Q/K quantiser

// Q/K quantiser.  One CTA walks kBlocksPerCta consecutive (128-token block, head) tiles of 128x128
// 16-bit values: 256 threads, 8 rows per thread, 16 bytes per row, the tile held in registers.  The
// loads of the next tile are issued before the current tile is reduced and stored, so the CTA barrier
// of the amax reduction does not leave the memory system idle.  grid (ceil(blocks/4), H, B*sources).
template <int DT>
__global__ void __launch_bounds__(256, 2) quant_block_kernel(BlockQuantArgs a, long long S, int H, int blocks) {
    __shared__ float part[2][8];
    const int which = blockIdx.z % a.sources;
    const long long batch = blockIdx.z / a.sources;
    const int head = blockIdx.y;
    const int c16 = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const long long row_pitch = static_cast<long long>(H) * kDim;  // elements
    const uint16_t* src = static_cast<const uint16_t*>(a.x[which]) + batch * S * row_pitch + head * kDim + c16 * 8;
    uint8_t* dst = a.codes[which] + batch * S * row_pitch + head * kDim + c16 * 8;
    float* descale = a.descale[which] + (batch * H + head) * a.descale_stride[which];
    const int first_blk = blockIdx.x * kBlocksPerCta;
    const int last_blk = min(first_blk + kBlocksPerCta, blocks);

    uint4 raw[8], next[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long row = static_cast<long long>(first_blk) * kTile + r0 + 16 * i;
        raw[i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
    }
    for (int blk = first_blk; blk < last_blk; ++blk) {
        if (blk + 1 < last_blk) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const long long row = static_cast<long long>(blk + 1) * kTile + r0 + 16 * i;
                next[i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
            }
        }
        float m = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float f[8];
            widen8<DT>(raw[i], f);
            m = absmax8(f, m);
        }
        const float amax = fmaxf(cta256_max(m, part[blk & 1]), kFloor);
        const float scale = div_full(kQMax, amax);
        if (threadIdx.x == 0) {
            descale[blk] = div_full(amax, kQMax);
            if (blk == 0 && a.descale_stride[which] > blocks) descale[blocks] = 1.0f;
            if (blk == 0 && which == 0 && a.amax_init != nullptr) a.amax_init[batch * H + head] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const long long row = static_cast<long long>(blk) * kTile + r0 + 16 * i;
            if (row < S) {
                float f[8];
                widen8<DT>(raw[i], f);
                *reinterpret_cast<uint2*>(dst + row * row_pitch) = quantize8(f, scale);
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) raw[i] = next[i];
    }
}

// Per-(batch, head) max |v| by atomic max over non-negative float bit patterns.  grid (blocks, H, B).
template <int DT>
__global__ void __launch_bounds__(128) head_amax_kernel(const void* v, float* amax, long long S, int H) {
    const int blk = blockIdx.x, head = blockIdx.y;
    const long long batch = blockIdx.z;
    const int c16 = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const long long row_pitch = static_cast<long long>(H) * kDim;
    const long long first = static_cast<long long>(blk) * kTile + r0;
    const uint16_t* src = static_cast<const uint16_t*>(v) + batch * S * row_pitch + head * kDim + c16 * 8;
    uint4 raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const long long row = first + 8 * i;
        raw[i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
    }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float f[8];
        widen8<DT>(raw[i], f);
        m = absmax8(f, m);
    }
    m = cta128_max(m);
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax + batch * H + head), __float_as_int(m));
}

// V cast with the per-(batch, head) scale, row-major output.  grid (blocks, H, B).
// With SCORE also emits the per-token squared rounding residual (score[h][s], B == 1).
template <int DT, bool SCORE>
__global__ void __launch_bounds__(128) head_cast_kernel(const void* v, const float* amax_in, uint8_t* codes,
                                                         float* descale_out, float* score, long long S, int H) {
    const int blk = blockIdx.x, head = blockIdx.y;
    const long long batch = blockIdx.z;
    const int c16 = threadIdx.x & 15, r0 = threadIdx.x >> 4;
    const long long row_pitch = static_cast<long long>(H) * kDim;
    const long long first = static_cast<long long>(blk) * kTile + r0;
    const uint16_t* src = static_cast<const uint16_t*>(v) + batch * S * row_pitch + head * kDim + c16 * 8;
    uint8_t* dst = codes + batch * S * row_pitch + head * kDim + c16 * 8;
    const float amax = fmaxf(amax_in[batch * H + head], kFloor);
    const float scale = div_full(kQMax, amax);
    const float descale = div_full(amax, kQMax);
    if (descale_out != nullptr && blk == 0 && threadIdx.x == 0) descale_out[batch * H + head] = descale;
    uint4 raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const long long row = first + 8 * i;
        raw[i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const long long row = first + 8 * i;
        float f[8];
        widen8<DT>(raw[i], f);
        const uint2 q = quantize8(f, scale);
        if (row < S) *reinterpret_cast<uint2*>(dst + row * row_pitch) = q;
        if (SCORE) {
            const float4 lo = decode4(q.x), hi = decode4(q.y);
            const float dec[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float r = __fmaf_rn(-dec[j], descale, f[j]);
                sum = __fadd_rn(sum, __fmul_rn(r, r));
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
            if (c16 == 0 && row < S) score[static_cast<long long>(head) * S + row] = sum;
        }
    }
}

// ---- transposition into the packed V layout [.., H, 128 channels, S_pad keys] --------------
//
// A 128-key x 128-channel byte tile is transposed through 16 KB of shared memory addressed as
// 32-bit words word[channel][key group of 4], with the group index XOR-ed by 2*(channel>>3) so
// that both the word stores (one instruction covers 16 channel chunks x 2 key groups) and the
// 16-byte reads (8 lanes cover one channel's 128 keys) are free of bank conflicts.

__device__ __forceinline__ void transpose4x4(const uint32_t (&a)[4], uint32_t (&o)[4]) {
    // a[i] = bytes of key i for channels c..c+3  ->  o[j] = bytes of channel c+j for keys 0..3
    const uint32_t t0 = __byte_perm(a[0], a[1], 0x5140), t1 = __byte_perm(a[2], a[3], 0x5140);
    const uint32_t t2 = __byte_perm(a[0], a[1], 0x7362), t3 = __byte_perm(a[2], a[3], 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410);
    o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410);
    o[3] = __byte_perm(t2, t3, 0x7632);
}

__device__ __forceinline__ void smem_put(uint32_t* words, int channel, int group, uint32_t value) {
    words[channel * 32 + (group ^ (2 * (channel >> 3)))] = value;
}

// After __syncthreads(): 256 threads write the tile to packed rows, 16 bytes per access.
__device__ __forceinline__ void smem_flush(const uint32_t* words, uint8_t* packed_head, long long S_pad, int tile) {
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int channel = idx >> 3, quad = idx & 7;
        const int s = 2 * (channel >> 3);
        const int base = (4 * quad) ^ (s & ~3);
        uint4 w = *reinterpret_cast<const uint4*>(words + channel * 32 + base);
        if (s & 2) w = make_uint4(w.z, w.w, w.x, w.y);
        *reinterpret_cast<uint4*>(packed_head + channel * S_pad + static_cast<long long>(tile) * kTile + 16 * quad) = w;
    }
}

// V cast + pack from 16-bit input.  grid (S_pad/128, H, B), 256 threads.
template <int DT>
__global__ void __launch_bounds__(256) cast_pack_kernel(const void* v, const float* amax_in, uint8_t* packed,
                                                         float* descale_out, long long S, int H, long long S_pad) {
    __shared__ __align__(16) uint32_t words[kDim * 32];
    const int tile = blockIdx.x, head = blockIdx.y;
    const long long batch = blockIdx.z;
    const int l16 = threadIdx.x & 15, kq = threadIdx.x >> 4;
    const long long row_pitch = static_cast<long long>(H) * kDim;
    const uint16_t* src = static_cast<const uint16_t*>(v) + batch * S * row_pitch + head * kDim + l16 * 8;
    const float amax = fmaxf(amax_in[batch * H + head], kFloor);
    const float scale = div_full(kQMax, amax);
    if (descale_out != nullptr && tile == 0 && threadIdx.x == 0)
        descale_out[batch * H + head] = div_full(amax, kQMax);
    uint4 raw[8];
#pragma unroll
    for (int gi = 0; gi < 2; ++gi)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long row = static_cast<long long>(tile) * kTile + 4 * (kq + 16 * gi) + i;
            raw[gi * 4 + i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
    for (int gi = 0; gi < 2; ++gi) {
        const int group = kq + 16 * gi;
        uint32_t lo[4], hi[4], o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float f[8];
            widen8<DT>(raw[gi * 4 + i], f);
            const uint2 q = quantize8(f, scale);
            lo[i] = q.x;
            hi[i] = q.y;
        }
        transpose4x4(lo, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) smem_put(words, l16 * 8 + j, group, o[j]);
        transpose4x4(hi, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) smem_put(words, l16 * 8 + 4 + j, group, o[j]);
    }
    __syncthreads();
    smem_flush(words, packed + (batch * H + head) * kDim * S_pad, S_pad, tile);
}

// FP8 byte transpose [B,S,H,128] -> [B,H,128,S_pad].  grid (S_pad/128, H, B), 256 threads.
__global__ void __launch_bounds__(256) pack_bytes_kernel(const uint8_t* codes, uint8_t* packed, long long S, int H,
                                                          long long S_pad) {
    __shared__ __align__(16) uint32_t words[kDim * 32];
    const int tile = blockIdx.x, head = blockIdx.y;
    const long long batch = blockIdx.z;
    const int l8 = threadIdx.x & 7, group = threadIdx.x >> 3;
    const long long row_pitch = static_cast<long long>(H) * kDim;
    const uint8_t* src = codes + batch * S * row_pitch + head * kDim + l8 * 16;
    uint4 raw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long row = static_cast<long long>(tile) * kTile + 4 * group + i;
        raw[i] = row < S ? ld_stream(src + row * row_pitch) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint32_t a[4], o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = k == 0 ? raw[i].x : k == 1 ? raw[i].y : k == 2 ? raw[i].z : raw[i].w;
        transpose4x4(a, o);
#pragma unroll
        for (int j = 0; j < 4; ++j) smem_put(words, l8 * 16 + 4 * k + j, group, o[j]);
    }
    __syncthreads();
    smem_flush(words, packed + (batch * H + head) * kDim * S_pad, S_pad, tile);
}

// Repair prefix rows: one warp per (repair row, head), four channels per lane.  grid (rows, H).
template <int DT>
__global__ void __launch_bounds__(32) repair_rows_kernel(uint8_t* k_all, uint8_t* v_all, const void* v_src,
                                                          const float* k_descale, const float* v_descale,
                                                          const int32_t* index, float* repair_kd, long long selected,
                                                          long long rows, long long S, int H, long long k_blocks) {
    const long long row = blockIdx.x;
    const int head = blockIdx.y, lane = threadIdx.x;
    const bool real = row < selected;
    const long long source = index[static_cast<long long>(head) * selected + (real ? row : 0)];
    const long long pitch = static_cast<long long>(H) * kDim;
    const long long target = row * pitch + head * kDim + 4 * lane;
    const long long origin = (rows + source) * pitch + head * kDim + 4 * lane;
    *reinterpret_cast<uint32_t*>(k_all + target) = *reinterpret_cast<const uint32_t*>(k_all + origin);
    if (lane == 0) repair_kd[static_cast<long long>(head) * rows + row] = k_descale[head * k_blocks + source / kTile];
    const float descale = v_descale[head];
    const uint2 orig = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(v_src) + source * pitch +
                                                       head * kDim + 4 * lane);
    float o[4];
    if (DT == OVC_BF16) {
        o[0] = __uint_as_float(orig.x << 16);
        o[1] = __uint_as_float(orig.x & 0xFFFF0000u);
        o[2] = __uint_as_float(orig.y << 16);
        o[3] = __uint_as_float(orig.y & 0xFFFF0000u);
    } else {
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&orig.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&orig.y));
        o[0] = a.x, o[1] = a.y, o[2] = b.x, o[3] = b.y;
    }
    const float4 dec = decode4(*reinterpret_cast<const uint32_t*>(v_all + origin));
    const float d[4] = {dec.x, dec.y, dec.z, dec.w};
    float c[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float residual = real ? __fmaf_rn(-d[j], descale, o[j]) : 0.0f;
        c[j] = clamp448(div_full(residual, descale));
    }
    *reinterpret_cast<uint32_t*>(v_all + target) = cast4(c[0], c[1], c[2], c[3]);
}

__global__ void div_full_kernel(const float* a, const float* b, float* q, long long n) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) q[i] = div_full(a[i], b[i]);
}

bool bad_dims(int64_t B, int64_t S, int64_t H) {
    return B < 1 || S < 1 || H < 1 || H > 65535 || B > 32767 || ceil_div(S, kTile) > 0x7FFFFFFF;
}

}  // namespace
}  // namespace ovc

using namespace ovc;

// ---- scratch that lives inside the library (used only by ovc_prepare_fused_static) --------------
//
// One float per head for the per-head max |v|.  Every GPU that loads the library holds these 16 KB
// until the process exits.  In host code the array's name is only a handle for the runtime: the
// device address has to be asked for, once per device, with that device current.
#define OVC_STATIC_MAX_HEADS 4096
static __device__ __align__(256) float g_static_amax[OVC_STATIC_MAX_HEADS];

namespace {

constexpr int kMaxDevices = 64;
// Filled on the first call per device; atomic so that host threads making that first call together agree.
std::atomic<float*> g_static_amax_ptr[kMaxDevices];

// Device address of g_static_amax on the current device (looked up on the first call per device).
int static_amax_pointer(float** out) {
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) {
        set_last_cuda_error(err);
        return OVC_ERR_CUDA;
    }
    if (device < 0 || device >= kMaxDevices) return OVC_ERR_ARGUMENT;
    float* ptr = g_static_amax_ptr[device].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_amax);
        if (err != cudaSuccess || ptr == nullptr) {
            set_last_cuda_error(err);
            return OVC_ERR_CUDA;
        }
        g_static_amax_ptr[device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return OVC_OK;
}

}  // namespace

extern "C" {

int ovc_version(void) { return 1; }

const char* ovc_error_string(int code) {
    switch (code) {
        case OVC_OK: return "ok";
        case OVC_ERR_ARGUMENT: return "invalid argument (null pointer, size, alignment or dtype)";
        case OVC_ERR_CUDA: return "CUDA runtime error (see ovc_last_cuda_error)";
        case OVC_ERR_DRIVER: return "tensor-map creation failed (see ovc_last_cuda_error)";
        case OVC_ERR_UNSUPPORTED: return "device is not sm_100";
        case OVC_ERR_TOO_LARGE: return "size exceeds the capacity of the library's built-in scratch memory";
        default: return "unknown error";
    }
}

int ovc_last_cuda_error(void) { return g_last_cuda_error; }

int ovc_quantize_per_block(const void* x, int dtype, int64_t B, int64_t S, int64_t H, void* codes, float* descale,
                           int64_t descale_stride, void* stream) {
    const int64_t blocks = ceil_div(S, kTile);
    if (!x || !codes || !descale || bad_dims(B, S, H) || (dtype != OVC_F16 && dtype != OVC_BF16) ||
        descale_stride < blocks || !aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 7u))
        return OVC_ERR_ARGUMENT;
    BlockQuantArgs a{};
    a.x[0] = x, a.codes[0] = static_cast<uint8_t*>(codes), a.descale[0] = descale, a.descale_stride[0] = descale_stride;
    a.sources = 1, a.amax_init = nullptr;
    const dim3 grid(static_cast<unsigned>(ceil_div(blocks, kBlocksPerCta)), static_cast<unsigned>(H), static_cast<unsigned>(B));
    auto s = static_cast<cudaStream_t>(stream);
    if (dtype == OVC_BF16) quant_block_kernel<OVC_BF16><<<grid, 256, 0, s>>>(a, S, static_cast<int>(H), static_cast<int>(blocks));
    else quant_block_kernel<OVC_F16><<<grid, 256, 0, s>>>(a, S, static_cast<int>(H), static_cast<int>(blocks));
    return check_launch();
}

int ovc_head_amax(const void* v, int dtype, int64_t B, int64_t S, int64_t H, float* amax, void* stream) {
    if (!v || !amax || bad_dims(B, S, H) || (dtype != OVC_F16 && dtype != OVC_BF16) || !aligned16(v)) return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    cudaError_t err = cudaMemsetAsync(amax, 0, sizeof(float) * B * H, s);
    if (err != cudaSuccess) { set_last_cuda_error(err); return OVC_ERR_CUDA; }
    const dim3 grid(static_cast<unsigned>(ceil_div(S, kTile)), static_cast<unsigned>(H), static_cast<unsigned>(B));
    if (dtype == OVC_BF16) head_amax_kernel<OVC_BF16><<<grid, 128, 0, s>>>(v, amax, S, static_cast<int>(H));
    else head_amax_kernel<OVC_F16><<<grid, 128, 0, s>>>(v, amax, S, static_cast<int>(H));
    return check_launch();
}

int ovc_quantize_per_head(const void* v, int dtype, int64_t B, int64_t S, int64_t H, const float* amax, void* codes,
                          float* descale, void* stream) {
    if (!v || !amax || !codes || !descale || bad_dims(B, S, H) || (dtype != OVC_F16 && dtype != OVC_BF16) ||
        !aligned16(v) || (reinterpret_cast<uintptr_t>(codes) & 7u))
        return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>(ceil_div(S, kTile)), static_cast<unsigned>(H), static_cast<unsigned>(B));
    auto* c = static_cast<uint8_t*>(codes);
    if (dtype == OVC_BF16) head_cast_kernel<OVC_BF16, false><<<grid, 128, 0, s>>>(v, amax, c, descale, nullptr, S, static_cast<int>(H));
    else head_cast_kernel<OVC_F16, false><<<grid, 128, 0, s>>>(v, amax, c, descale, nullptr, S, static_cast<int>(H));
    return check_launch();
}

int ovc_prepare_fused(const void* q, const void* k, const void* v, int dtype, int64_t S, int64_t H, void* q8, void* k8,
                      void* v_packed, float* q_descale, float* k_descale, float* v_descale, float* amax_ws,
                      void* stream) {
    if (!q || !k || !v || !q8 || !k8 || !v_packed || !q_descale || !k_descale || !v_descale || !amax_ws ||
        bad_dims(1, S, H) || (dtype != OVC_F16 && dtype != OVC_BF16) || !aligned16(q) || !aligned16(k) ||
        !aligned16(v) || !aligned16(v_packed) || (reinterpret_cast<uintptr_t>(q8) & 7u) ||
        (reinterpret_cast<uintptr_t>(k8) & 7u))
        return OVC_ERR_ARGUMENT;
    const int64_t blocks = ceil_div(S, kTile);
    const int64_t q_blocks = (blocks + 1) / 2 * 2;
    const int64_t S_pad = blocks * kTile;
    auto s = static_cast<cudaStream_t>(stream);
    const int h = static_cast<int>(H);
    BlockQuantArgs a{};
    a.x[0] = q, a.x[1] = k;
    a.codes[0] = static_cast<uint8_t*>(q8), a.codes[1] = static_cast<uint8_t*>(k8);
    a.descale[0] = q_descale, a.descale[1] = k_descale;
    a.descale_stride[0] = q_blocks, a.descale_stride[1] = blocks;
    a.sources = 2, a.amax_init = amax_ws;
    const dim3 grid_qk(static_cast<unsigned>(ceil_div(blocks, kBlocksPerCta)), static_cast<unsigned>(H), 2);
    const dim3 grid_v(static_cast<unsigned>(blocks), static_cast<unsigned>(H), 1);
    if (dtype == OVC_BF16) {
        quant_block_kernel<OVC_BF16><<<grid_qk, 256, 0, s>>>(a, S, h, static_cast<int>(blocks));
        head_amax_kernel<OVC_BF16><<<grid_v, 128, 0, s>>>(v, amax_ws, S, h);
        cast_pack_kernel<OVC_BF16><<<grid_v, 256, 0, s>>>(v, amax_ws, static_cast<uint8_t*>(v_packed), v_descale, S, h, S_pad);
    } else {
        quant_block_kernel<OVC_F16><<<grid_qk, 256, 0, s>>>(a, S, h, static_cast<int>(blocks));
        head_amax_kernel<OVC_F16><<<grid_v, 128, 0, s>>>(v, amax_ws, S, h);
        cast_pack_kernel<OVC_F16><<<grid_v, 256, 0, s>>>(v, amax_ws, static_cast<uint8_t*>(v_packed), v_descale, S, h, S_pad);
    }
    return check_launch();
}

int ovc_pack_v(const void* codes, int64_t B, int64_t S, int64_t H, void* packed, void* stream) {
    if (!codes || !packed || bad_dims(B, S, H) || !aligned16(codes) || !aligned16(packed)) return OVC_ERR_ARGUMENT;
    const int64_t S_pad = ceil_div(S, kTile) * kTile;
    const dim3 grid(static_cast<unsigned>(S_pad / kTile), static_cast<unsigned>(H), static_cast<unsigned>(B));
    pack_bytes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(codes), static_cast<uint8_t*>(packed), S, static_cast<int>(H), S_pad);
    return check_launch();
}

int ovc_copy_head_slice(void* dst, int64_t dst_heads, int64_t dst_first, const void* src, int64_t src_heads,
                        int64_t src_first, int64_t heads, int64_t S, int64_t bytes_per_head, int to_device, void* stream) {
    if (!dst || !src || S < 1 || heads < 1 || bytes_per_head < 1 || dst_first < 0 || src_first < 0 ||
        dst_first + heads > dst_heads || src_first + heads > src_heads)
        return OVC_ERR_ARGUMENT;
    // One 2-D copy: S rows (tokens) of `heads` consecutive heads each; the row pitch is the tensor's head count.
    const cudaError_t err = cudaMemcpy2DAsync(
        static_cast<char*>(dst) + dst_first * bytes_per_head, static_cast<size_t>(dst_heads * bytes_per_head),
        static_cast<const char*>(src) + src_first * bytes_per_head, static_cast<size_t>(src_heads * bytes_per_head),
        static_cast<size_t>(heads * bytes_per_head), static_cast<size_t>(S),
        to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream));
    if (err != cudaSuccess) {
        set_last_cuda_error(static_cast<int>(err));
        return OVC_ERR_CUDA;
    }
    return OVC_OK;
}

int ovc_div_full(const float* a, const float* b, float* q, int64_t n, void* stream) {
    if (!a || !b || !q || n < 1 || ceil_div(n, 256) > 0x7FFFFFFF) return OVC_ERR_ARGUMENT;
    div_full_kernel<<<static_cast<unsigned>(ceil_div(n, 256)), 256, 0, static_cast<cudaStream_t>(stream)>>>(a, b, q, n);
    return check_launch();
}

int ovc_repair_score(const void* v, int dtype, int64_t S, int64_t H, const float* amax, void* codes, float* score,
                     void* stream) {
    if (!v || !amax || !codes || !score || bad_dims(1, S, H) || (dtype != OVC_F16 && dtype != OVC_BF16) ||
        !aligned16(v) || (reinterpret_cast<uintptr_t>(codes) & 7u))
        return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>(ceil_div(S, kTile)), static_cast<unsigned>(H), 1);
    auto* c = static_cast<uint8_t*>(codes);
    if (dtype == OVC_BF16) head_cast_kernel<OVC_BF16, true><<<grid, 128, 0, s>>>(v, amax, c, nullptr, score, S, static_cast<int>(H));
    else head_cast_kernel<OVC_F16, true><<<grid, 128, 0, s>>>(v, amax, c, nullptr, score, S, static_cast<int>(H));
    return check_launch();
}

int ovc_repair_rows(void* k_all, void* v_all, const void* v_src, int dtype, const float* k_descale,
                    const float* v_descale, const int32_t* index, float* repair_kd, int64_t selected, int64_t rows,
                    int64_t S, int64_t H, int64_t k_blocks, void* stream) {
    if (!k_all || !v_all || !v_src || !k_descale || !v_descale || !index || !repair_kd || bad_dims(1, S, H) ||
        (dtype != OVC_F16 && dtype != OVC_BF16) || selected < 1 || rows < selected || rows % kTile != 0 ||
        rows > 0x7FFFFFFF || k_blocks < ceil_div(S, kTile) || (reinterpret_cast<uintptr_t>(k_all) & 3u) ||
        (reinterpret_cast<uintptr_t>(v_all) & 3u) || (reinterpret_cast<uintptr_t>(v_src) & 7u))
        return OVC_ERR_ARGUMENT;
    auto s = static_cast<cudaStream_t>(stream);
    const dim3 grid(static_cast<unsigned>(rows), static_cast<unsigned>(H), 1);
    auto* ka = static_cast<uint8_t*>(k_all);
    auto* va = static_cast<uint8_t*>(v_all);
    if (dtype == OVC_BF16)
        repair_rows_kernel<OVC_BF16><<<grid, 32, 0, s>>>(ka, va, v_src, k_descale, v_descale, index, repair_kd, selected, rows, S, static_cast<int>(H), k_blocks);
    else
        repair_rows_kernel<OVC_F16><<<grid, 32, 0, s>>>(ka, va, v_src, k_descale, v_descale, index, repair_kd, selected, rows, S, static_cast<int>(H), k_blocks);
    return check_launch();
}

int ovc_prepare_fused_static(const void* q, const void* k, const void* v, int dtype, int64_t S, int64_t H, void* q8,
                             void* k8, void* v_packed, float* q_descale, float* k_descale, float* v_descale,
                             void* stream) {
    if (H > OVC_STATIC_MAX_HEADS) return OVC_ERR_TOO_LARGE;
    float* scratch = nullptr;
    const int rc = static_amax_pointer(&scratch);
    if (rc != OVC_OK) return rc;
    // The first preparation kernel resets scratch[0..H) before the amax pass accumulates into it,
    // so nothing is carried over from the previous call.
    return ovc_prepare_fused(q, k, v, dtype, S, H, q8, k8, v_packed, q_descale, k_descale, v_descale, scratch, stream);
}


}  // extern "C"
