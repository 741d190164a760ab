// W4A16 path of compressed-tensors INT4 checkpoints (offset-binary codes, value =
// code - 8, one bf16 scale per 128 weights, fp32 activations):
//
//   int4_dot_k       partial[row*nbpr+b] = bf16(scale) * sum_{128} (code-8) * x
//                    reference tools/gen_int4_dot.py:88-147, head/tail and index algebra
//                    tools/gen_gemv_qdot.py:120-196
//   reduce_blocks_k  y[r] = partial[r*nbpr+0] + partial[r*nbpr+1] + ... in that order
//                    reference tools/gen_gemv_qdot.py:207-308
//   int4_dequant_k   y[8g+j] = (code_j - 8) * bf16(scale[g/16]), bit-exact
//                    reference tools/gen_int4_dot.py:162-223
//
// The reference runs one work-item per 64-byte block.  Here a warp owns whole weight
// rows (the nbpr blocks of a row are contiguous: address = w + ids[ew]*stride +
// local*64), lane l takes the 16-byte words l, l+32, ...; a block is 4 lanes, summed by
// two shuffles.  When every row reads the same activation row (the dense case) x is
// staged in shared memory once per CTA and R = 4 weight rows share every fetch of it,
// which keeps the shared-memory traffic below the weight stream.  Each nibble becomes a
// float without an integer conversion: PRMT drops the code into the low byte of
// 0x4B000000 (= 2^23 + code) and one fp32 subtract of 2^23 + 8 gives code - 8 exactly.
// The path is fp32 throughout (no integer accumulator exists on it).
#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct DotParams {
    const uint8_t* w;
    const float* x;
    float* partial;
    const uint16_t* scale;
    const uint32_t* ids;
    uint32_t items;          // work-items to produce: min(nblocks, grid*workgroup)
    uint32_t nbpr, rows_per_exp, stride, rows_per_w;
};

// eight codes of one packed word times eight activations, added into acc[0..3]
// (code j goes to accumulator j % 4, as in the reference)
__device__ __forceinline__ void fma_word(uint32_t w, const float4& xa, const float4& xb, float acc[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu;            // codes 0,2,4,6
    const uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;     // codes 1,3,5,7
    const uint32_t magic = 0x4B000000u;             // 2^23
    const float bias = 8388616.0f;                  // 2^23 + 8
    const float c0 = __uint_as_float(prmt(lo, magic, 0x7540u)) - bias;
    const float c1 = __uint_as_float(prmt(hi, magic, 0x7540u)) - bias;
    const float c2 = __uint_as_float(prmt(lo, magic, 0x7541u)) - bias;
    const float c3 = __uint_as_float(prmt(hi, magic, 0x7541u)) - bias;
    const float c4 = __uint_as_float(prmt(lo, magic, 0x7542u)) - bias;
    const float c5 = __uint_as_float(prmt(hi, magic, 0x7542u)) - bias;
    const float c6 = __uint_as_float(prmt(lo, magic, 0x7543u)) - bias;
    const float c7 = __uint_as_float(prmt(hi, magic, 0x7543u)) - bias;
    acc[0] = fmaf(c0, xa.x, acc[0]);
    acc[1] = fmaf(c1, xa.y, acc[1]);
    acc[2] = fmaf(c2, xa.z, acc[2]);
    acc[3] = fmaf(c3, xa.w, acc[3]);
    acc[0] = fmaf(c4, xb.x, acc[0]);
    acc[1] = fmaf(c5, xb.y, acc[1]);
    acc[2] = fmaf(c6, xb.z, acc[2]);
    acc[3] = fmaf(c7, xb.w, acc[3]);
}

// SHARED_X: all rows use activation row 0, staged in shared memory; R rows per warp step.
template <bool SHARED_X, int R>
__global__ void __launch_bounds__(kThreads)
int4_dot_kernel(const DotParams p) {
    extern __shared__ __align__(16) float s_x[];
    const int lane = threadIdx.x & 31;
    const int gwarp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int nwarp = gridDim.x * kWarps;
    const uint32_t nbpr = p.nbpr;
    const uint32_t rows = (p.items + nbpr - 1) / nbpr;       // the last row may be partial
    const int KW = nbpr * 16;                                // packed words per row
    pdl_wait();
    if (SHARED_X) {
        for (int i = threadIdx.x; i < (int)nbpr * 32; i += blockDim.x)
            reinterpret_cast<float4*>(s_x)[i] = reinterpret_cast<const float4*>(p.x)[i];
        __syncthreads();
    }
    for (uint32_t rb = gwarp; rb * R < rows; rb += nwarp) {
        const uint8_t* wrow[R];
        const uint16_t* srow[R];
        const float* xrow[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const uint32_t q1 = min(rb * R + r, rows - 1);
            const uint32_t ew = q1 / p.rows_per_w;
            const uint32_t e = q1 / p.rows_per_exp;
            const size_t base = (size_t)p.ids[ew] * p.stride;
            const size_t local = (size_t)(q1 - ew * p.rows_per_w) * nbpr;
            wrow[r] = p.w + base + local * 64;
            srow[r] = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(p.scale) + base / 32) + local;
            xrow[r] = SHARED_X ? s_x : p.x + (size_t)e * nbpr * 128;
        }
        for (int d0 = lane * 4; d0 < KW; d0 += 128) {
            const int b = d0 >> 4;                           // block inside the row
            float4 xv[8];
            if (SHARED_X) {
#pragma unroll
                for (int j = 0; j < 8; j++) xv[j] = *reinterpret_cast<const float4*>(s_x + d0 * 8 + j * 4);
            }
#pragma unroll
            for (int r = 0; r < R; r++) {
                const uint32_t q1 = rb * R + r;
                const uint4 w4 = ld_stream_v4(wrow[r] + (size_t)d0 * 4);
                const float sc = __uint_as_float((uint32_t)srow[r][b] << 16);
                if (!SHARED_X) {
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        xv[j] = *reinterpret_cast<const float4*>(xrow[r] + d0 * 8 + j * 4);
                }
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                fma_word(w4.x, xv[0], xv[1], acc);
                fma_word(w4.y, xv[2], xv[3], acc);
                fma_word(w4.z, xv[4], xv[5], acc);
                fma_word(w4.w, xv[6], xv[7], acc);
                float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                const uint32_t item = q1 * nbpr + b;
                if ((lane & 3) == 0 && q1 < rows && item < p.items) p.partial[item] = v * sc;
            }
        }
    }
    pdl_launch_dependents();
}

__global__ void __launch_bounds__(128)
reduce_blocks_kernel(const float* __restrict__ partial, float* __restrict__ y, uint32_t rows, uint32_t nbpr) {
    pdl_wait();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) {
        const float* p = partial + (size_t)r * nbpr;
        float s = 0.f;
        for (uint32_t j = 0; j < nbpr; j++) s += p[j];
        y[r] = s;
    }
    pdl_launch_dependents();
}

__global__ void __launch_bounds__(256)
int4_dequant_kernel(const uint32_t* __restrict__ w, const uint16_t* __restrict__ scale, float* __restrict__ y,
                    uint32_t nwords) {
    pdl_wait();
    const uint32_t g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g < nwords) {
        const uint32_t word = w[g];
        const float s = __uint_as_float((uint32_t)scale[g >> 4] << 16);
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = ((float)((word >> (4 * j)) & 0xFu) - 8.0f) * s;
        float4* dst = reinterpret_cast<float4*>(y + (size_t)g * 8);
        dst[0] = make_float4(o[0], o[1], o[2], o[3]);
        dst[1] = make_float4(o[4], o[5], o[6], o[7]);
    }
    pdl_launch_dependents();
}

// int4_dot_k(w, x, partial, nblocks, group_size, nbpr, magic_nbpr, rows_per_exp, magic_rpe,
//            scale, ids, stride, rows_per_w, magic_rpw).  The three magic multipliers are
// accepted and ignored (the kernel divides directly).
int launch_int4_dot(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "int4_dot_k";
    DotParams p = {};
    p.w = arg_ptr<const uint8_t>(a[0]);
    p.x = arg_ptr<const float>(a[1]);
    p.partial = arg_ptr<float>(a[2]);
    const uint32_t nblocks = arg_u32(a[3]);
    const uint32_t group_size = arg_u32(a[4]);
    p.nbpr = arg_u32(a[5]);
    p.rows_per_exp = arg_u32(a[7]);
    p.scale = arg_ptr<const uint16_t>(a[9]);
    p.ids = arg_ptr<const uint32_t>(a[10]);
    p.stride = arg_u32(a[11]);
    p.rows_per_w = arg_u32(a[12]);
    FM_REQUIRE(group_size == c.wx && c.wy == 1 && c.gy == 1, kn,
               "the group_size argument (%u) must equal the 1-D work-group size (%u)", group_size, c.wx);
    FM_REQUIRE(p.nbpr > 0 && p.rows_per_exp > 0 && p.rows_per_w > 0, kn, "nbpr, rows_per_exp, rows_per_w must be > 0");
    FM_REQUIRE(p.stride % 64 == 0, kn, "stride=%u must be a multiple of the 64-byte block", p.stride);
    const unsigned long long covered = (unsigned long long)c.gx * c.wx;
    p.items = (uint32_t)(covered < nblocks ? covered : nblocks);
    if (p.items == 0) return FM_OK;
    FM_REQUIRE(aligned(p.w, 16) && aligned(p.x, 16) && aligned(p.partial, 4) && aligned(p.scale, 2) &&
                   aligned(p.ids, 4), kn, "misaligned pointer (w and x need 16 bytes)");
    const uint32_t rows = (p.items + p.nbpr - 1) / p.nbpr;
    const uint32_t n_w = (rows + p.rows_per_w - 1) / p.rows_per_w;       // weight experts touched
    const uint32_t n_x = (rows + p.rows_per_exp - 1) / p.rows_per_exp;   // activation rows touched
    FM_RANGE(p.ids, (size_t)n_w * 4, kn, "ids");
    FM_RANGE(p.x, (size_t)n_x * p.nbpr * 512, kn, "x");
    FM_RANGE(p.partial, (size_t)p.items * 4, kn, "partial");
    // the weight/scale footprint depends on ids[], which lives on the device: the dense
    // layout (one expert, ids[0] = 0 by contract) is checked, expert tables are the caller's
    if (n_w == 1) {
        FM_RANGE(p.w, (size_t)rows * p.nbpr * 64, kn, "w (dense layout)");
        FM_RANGE(p.scale, (size_t)rows * p.nbpr * 2, kn, "scale (dense layout)");
    }
    const bool shared_x = n_x == 1;
    const size_t smem = shared_x ? (size_t)p.nbpr * 512 : 0;
    FM_REQUIRE(smem <= 200 * 1024, kn, "K=%u is too large for the shared-memory activation row", p.nbpr * 128);
    cudaError_t e;
    if (shared_x) {
        auto kern = int4_dot_kernel<true, 4>;
        if (smem > 48 * 1024) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return cuda_fail(kn, e);
        }
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        int grid = c.sm_count * (per_sm < 1 ? 1 : per_sm);
        const int need = (int)((rows + 4 * kWarps - 1) / (4 * kWarps));
        if (grid > need) grid = need;
        e = launch_kernel(kern, dim3(grid), dim3(kThreads), smem, c.stream, pdl_enabled(), p);
    } else {
        auto kern = int4_dot_kernel<false, 1>;
        int grid = c.sm_count * 8;
        const int need = (int)((rows + kWarps - 1) / kWarps);
        if (grid > need) grid = need;
        e = launch_kernel(kern, dim3(grid), dim3(kThreads), 0, c.stream, pdl_enabled(), p);
    }
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// reduce_blocks_k(partial, y, nrows, nbpr)
int launch_reduce_blocks(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "reduce_blocks_k";
    const float* partial = arg_ptr<const float>(a[0]);
    float* y = arg_ptr<float>(a[1]);
    const uint32_t nrows = arg_u32(a[2]), nbpr = arg_u32(a[3]);
    FM_REQUIRE(c.wy == 1 && c.gy == 1, kn, "1-D launch expected");
    const unsigned long long covered = (unsigned long long)c.gx * c.wx;
    const uint32_t rows = (uint32_t)(covered < nrows ? covered : nrows);
    if (rows == 0) return FM_OK;
    FM_REQUIRE(aligned(partial, 4) && aligned(y, 4), kn, "misaligned pointer");
    FM_RANGE(partial, (size_t)rows * nbpr * 4, kn, "partial");
    FM_RANGE(y, (size_t)rows * 4, kn, "y");
    cudaError_t e = launch_kernel(reduce_blocks_kernel, dim3((rows + 127) / 128), dim3(128), 0, c.stream,
                                  pdl_enabled(), partial, y, rows, nbpr);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// int4_dequant_k(w, scale, y, nwords, group_size)
int launch_int4_dequant(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "int4_dequant_k";
    const uint32_t* w = arg_ptr<const uint32_t>(a[0]);
    const uint16_t* scale = arg_ptr<const uint16_t>(a[1]);
    float* y = arg_ptr<float>(a[2]);
    const uint32_t nwords = arg_u32(a[3]), group_size = arg_u32(a[4]);
    FM_REQUIRE(group_size == c.wx && c.wy == 1 && c.gy == 1, kn,
               "the group_size argument (%u) must equal the 1-D work-group size (%u)", group_size, c.wx);
    const unsigned long long covered = (unsigned long long)c.gx * c.wx;
    const uint32_t words = (uint32_t)(covered < nwords ? covered : nwords);
    if (words == 0) return FM_OK;
    FM_REQUIRE(aligned(w, 4) && aligned(scale, 2) && aligned(y, 16), kn, "misaligned pointer (y needs 16 bytes)");
    FM_RANGE(w, (size_t)words * 4, kn, "w");
    FM_RANGE(scale, (size_t)((words + 15) / 16) * 2, kn, "scale");
    FM_RANGE(y, (size_t)words * 32, kn, "y");
    cudaError_t e = launch_kernel(int4_dequant_kernel, dim3((words + 255) / 256), dim3(256), 0, c.stream,
                                  pdl_enabled(), w, scale, y, words);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kInt4[] = {
    {"int4_dot_k", 14, launch_int4_dot, "pppiiiiiippiii"},
    {"reduce_blocks_k", 4, launch_reduce_blocks, "ppii"},
    {"int4_dequant_k", 5, launch_int4_dequant, "pppii"},
};

}  // namespace

const KernelEntry* int4_dot_kernels(int* n) {
    *n = (int)(sizeof(kInt4) / sizeof(kInt4[0]));
    return kInt4;
}

}  // namespace fm
