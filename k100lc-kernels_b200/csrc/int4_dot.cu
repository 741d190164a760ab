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
#include <cuda_bf16.h>
#include <stdlib.h>

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
// (code j goes to accumulator j % 4, as in the reference); two fp32 lanes per instruction
__device__ __forceinline__ void sub2(float& d0, float& d1, float a0, float a1, float b) {
    asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2,%3};\nmov.b64 rb, {%4,%4};\nadd.rn.f32x2 rd, ra, rb;\nmov.b64 {%0,%1}, rd;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b));
}
__device__ __forceinline__ void fma2(float& c0, float& c1, float a0, float a1, float b0, float b1) {
    asm("{\n.reg .b64 ra, rb, rc;\nmov.b64 ra, {%2,%3};\nmov.b64 rb, {%4,%5};\nmov.b64 rc, {%0,%1};\n"
        "fma.rn.f32x2 rc, ra, rb, rc;\nmov.b64 {%0,%1}, rc;\n}"
        : "+f"(c0), "+f"(c1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fma_word(uint32_t w, const float4& xa, const float4& xb, float acc[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu;            // codes 0,2,4,6
    const uint32_t hi = (w >> 4) & 0x0F0F0F0Fu;     // codes 1,3,5,7
    const uint32_t magic = 0x4B000000u;             // 2^23
    const float nbias = -8388616.0f;                // -(2^23 + 8)
    float c0, c1, c2, c3, c4, c5, c6, c7;
    sub2(c0, c1, __uint_as_float(prmt(lo, magic, 0x7540u)), __uint_as_float(prmt(hi, magic, 0x7540u)), nbias);
    sub2(c2, c3, __uint_as_float(prmt(lo, magic, 0x7541u)), __uint_as_float(prmt(hi, magic, 0x7541u)), nbias);
    sub2(c4, c5, __uint_as_float(prmt(lo, magic, 0x7542u)), __uint_as_float(prmt(hi, magic, 0x7542u)), nbias);
    sub2(c6, c7, __uint_as_float(prmt(lo, magic, 0x7543u)), __uint_as_float(prmt(hi, magic, 0x7543u)), nbias);
    fma2(acc[0], acc[1], c0, c1, xa.x, xa.y);
    fma2(acc[2], acc[3], c2, c3, xa.z, xa.w);
    fma2(acc[0], acc[1], c4, c5, xb.x, xb.y);
    fma2(acc[2], acc[3], c6, c7, xb.z, xb.w);
}

// Dense layout (one weight table, every row reads activation row 0): activation-stationary.
// A warp owns one 512-byte slice of every weight row (8 blocks of 128 weights; lane l the 16-byte
// word l of the slice, a block is 4 lanes) and keeps the 32 activations its lane needs in registers
// for the whole kernel: no shared memory, one 16-byte load per lane and row, UN rows in flight.
// The CTA has one warp per slice and walks rows blockIdx.x, blockIdx.x + gridDim.x, ...
template <int UN>
__global__ void __launch_bounds__(1024)
int4_dot_dense_kernel(const DotParams p) {
    const int lane = threadIdx.x & 31, slice = threadIdx.x >> 5;
    const uint32_t nbpr = p.nbpr;
    const uint32_t rows = (p.items + nbpr - 1) / nbpr;       // the last row may be partial
    const uint32_t word = slice * 32 + lane;                 // 16-byte word of the row
    const bool live = word < nbpr * 4;
    const uint32_t b = word >> 2;                            // block inside the row
    const size_t base = (size_t)p.ids[0] * p.stride;
    const uint8_t* w = p.w + base + (size_t)word * 16;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(p.scale) + base / 32) + b;
    const size_t row_bytes = (size_t)nbpr * 64;
    pdl_wait();
    float4 xv[8];
#pragma unroll
    for (int j = 0; j < 8; j++)
        xv[j] = live ? *reinterpret_cast<const float4*>(p.x + (size_t)word * 32 + j * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t r0 = blockIdx.x; r0 < rows; r0 += gridDim.x * UN) {
        uint4 w4[UN];
        uint32_t sb[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const uint32_t r = r0 + u * gridDim.x;
            const bool ok = live && r < rows;
            w4[u] = ok ? ld_stream_v4(w + (size_t)r * row_bytes) : make_uint4(0, 0, 0, 0);
            sb[u] = ok ? sc[(size_t)r * nbpr] : 0u;
        }
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const uint32_t r = r0 + u * gridDim.x;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            fma_word(w4[u].x, xv[0], xv[1], acc);
            fma_word(w4[u].y, xv[2], xv[3], acc);
            fma_word(w4[u].z, xv[4], xv[5], acc);
            fma_word(w4[u].w, xv[6], xv[7], acc);
            float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            const uint32_t item = r * nbpr + b;
            if ((lane & 3) == 0 && live && r < rows && item < p.items) p.partial[item] = v * __uint_as_float(sb[u] << 16);
        }
    }
    pdl_launch_dependents();
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

// Dense layout on the tensor cores.  The fp32 activations are split into three bf16 terms
// (x = x1 + x2 + x3 carries all 24 mantissa bits), the weights code - 8 are exact in bf16, so
// mma.sync m16n8k16 (bf16 in, fp32 accumulate) with the three terms as three columns of B gives
// the fp32 dot product to within accumulation rounding, and the add over the four lanes of a
// 128-block happens inside the MMA.  A warp owns one block index (so its B fragments — 32
// activations per lane — stay in registers) and walks 16-row units; lane (g, t) reads word t of
// a block for rows g and g + 8 (one 16-byte load each) and converts nibbles to bf16 two at a time:
// PRMT drops two codes into the low bytes of two 0x43xx halves (128 + code), one packed
// subtract of 136 gives code - 8.  6 instructions per 8 weights instead of 19.
constexpr int kDotWarps = 8;

// B fragments of int4_dot_mma_kernel, computed once per launch instead of once per warp:
// out[((b * 3 + term) * 4 + t) * 16 + (q * 4 + h * 2 + i)] = bf16 pair of the split term of
// x[128 b + 32 t + 8 q + 4 i + h] (low half) and x[... + 2] (high half)
__global__ void __launch_bounds__(256)
int4_dot_split_kernel(const float* __restrict__ x, uint32_t* __restrict__ out, uint32_t nbpr) {
    // the multiply kernel behind this one is launched as a programmatic dependent: it may start now and
    // fetch its first weights; it waits for this grid before it reads the fragments
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nbpr * 192) {
        const uint32_t e = idx & 15, t = (idx >> 4) & 3, term = (idx >> 6) % 3, b = idx / 192;
        const uint32_t q = e >> 2, h = (e >> 1) & 1, i = e & 1;
        const float* xs = x + (size_t)b * 128 + t * 32 + 8 * q + 4 * i + h;
        out[idx] = bf16_term(xs[0], (int)term) | (bf16_term(xs[2], (int)term) << 16);
    }
}

template <int UN>
__global__ void __launch_bounds__(kDotWarps * 32)
int4_dot_mma_kernel(const DotParams p, const uint32_t* __restrict__ frags) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t nbpr = p.nbpr;
    const uint32_t rows = (p.items + nbpr - 1) / nbpr;       // the last row may be partial
    const uint32_t bgroups = (nbpr + kDotWarps - 1) / kDotWarps;
    const uint32_t b = (blockIdx.x % bgroups) * kDotWarps + (threadIdx.x >> 5);   // this warp's block
    const uint32_t ucta = blockIdx.x / bgroups, nucta = gridDim.x / bgroups;       // row-unit walk of the CTA
    if (b >= nbpr || ucta >= nucta) return;
    const size_t base = (size_t)p.ids[0] * p.stride;
    const size_t row_bytes = (size_t)nbpr * 64;
    const uint8_t* w = p.w + base + (size_t)b * 64 + t * 16;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(reinterpret_cast<const uint8_t*>(p.scale) + base / 32) + b;
    const uint32_t nunits = (rows + 15) / 16;
    const uint4 zero8 = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // code 8 = weight 0
    uint4 wa[UN], wb[UN];
    const uint8_t* wnext = w + (size_t)(ucta * 16 + g) * row_bytes;   // row g of the next unit to fetch
    const size_t ustep = (size_t)nucta * 16 * row_bytes;
    auto fetch = [&](uint32_t u0) {
#pragma unroll
        for (int k = 0; k < UN; k++) {
            const uint32_t unit = u0 + k * nucta;
            const uint32_t ra = unit * 16 + g, rb = ra + 8;
            wa[k] = (unit < nunits && ra < rows) ? ld_stream_v4(wnext) : zero8;
            wb[k] = (unit < nunits && rb < rows) ? ld_stream_v4(wnext + 8 * row_bytes) : zero8;
            wnext += ustep;
        }
    };
    fetch(ucta);                                             // weights do not depend on the preceding kernel
    pdl_wait();

    // B fragments: MMA (q, h) uses, of the lane's 32 codes, codes 8q+h, 8q+2+h (b0) and 8q+4+h, 8q+6+h (b1);
    // column g of B is term g of the split (columns 3..7 are zero)
    uint32_t bf[4][2][2];
    {
        const uint4* fp = reinterpret_cast<const uint4*>(frags + ((size_t)(b * 3 + (g < 3 ? g : 0)) * 4 + t) * 16);
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const uint4 v = g < 3 ? fp[q] : make_uint4(0, 0, 0, 0);
            bf[q][0][0] = v.x; bf[q][0][1] = v.y; bf[q][1][0] = v.z; bf[q][1][1] = v.w;
        }
    }
    for (uint32_t u0 = ucta; u0 < nunits; u0 += nucta * UN) {
        uint4 ca[UN], cb[UN];
#pragma unroll
        for (int k = 0; k < UN; k++) {
            ca[k] = wa[k];
            cb[k] = wb[k];
        }
        fetch(u0 + nucta * UN);                              // next round (no loads past the end)
#pragma unroll
        for (int k = 0; k < UN; k++) {
            const uint32_t unit = u0 + k * nucta;
            if (unit >= nunits) break;
            const uint32_t ra = unit * 16 + g, rb = ra + 8;
            const uint32_t wav[4] = {ca[k].x, ca[k].y, ca[k].z, ca[k].w}, wbv[4] = {cb[k].x, cb[k].y, cb[k].z, cb[k].w};
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const uint32_t la = wav[q] & 0x0F0F0F0Fu, ha = (wav[q] >> 4) & 0x0F0F0F0Fu;
                const uint32_t lb = wbv[q] & 0x0F0F0F0Fu, hb = (wbv[q] >> 4) & 0x0F0F0F0Fu;
                const uint32_t m = 0x43434343u;
                // even codes (0,2 | 4,6), then odd codes (1,3 | 5,7)
                mma_bf16(c, bf16x2_sub136(prmt(la, m, 0x5140u)), bf16x2_sub136(prmt(lb, m, 0x5140u)),
                         bf16x2_sub136(prmt(la, m, 0x5342u)), bf16x2_sub136(prmt(lb, m, 0x5342u)), bf[q][0][0], bf[q][0][1]);
                mma_bf16(c, bf16x2_sub136(prmt(ha, m, 0x5140u)), bf16x2_sub136(prmt(hb, m, 0x5140u)),
                         bf16x2_sub136(prmt(ha, m, 0x5342u)), bf16x2_sub136(prmt(hb, m, 0x5342u)), bf[q][1][0], bf[q][1][1]);
            }
            // columns 0, 1 (lane t = 0) and 2 (lane t = 1) hold the three terms: smallest first
            const float va = __shfl_down_sync(0xffffffffu, c[0], 1), vb = __shfl_down_sync(0xffffffffu, c[2], 1);
            if (t == 0) {
                if (ra < rows && ra * nbpr + b < p.items)
                    p.partial[(size_t)ra * nbpr + b] = ((va + c[1]) + c[0]) * __uint_as_float((uint32_t)sc[(size_t)ra * nbpr] << 16);
                if (rb < rows && rb * nbpr + b < p.items)
                    p.partial[(size_t)rb * nbpr + b] = ((vb + c[3]) + c[2]) * __uint_as_float((uint32_t)sc[(size_t)rb * nbpr] << 16);
            }
        }
    }
    pdl_launch_dependents();
}

// 128 rows per CTA: their nbpr partial sums are one contiguous range, fetched coalesced into shared
// memory (row stride nbpr + 1 words: conflict-free), then every thread adds its row in index order.
__global__ void __launch_bounds__(128)
reduce_blocks_kernel(const float* __restrict__ partial, float* __restrict__ y, uint32_t rows, uint32_t nbpr) {
    extern __shared__ float s_part[];
    pdl_wait();
    const uint32_t row0 = blockIdx.x * 128;
    const uint32_t nrow = min(128u, rows - row0);
    const float* src = partial + (size_t)row0 * nbpr;
    for (uint32_t i = threadIdx.x; i < nrow * nbpr; i += 128) s_part[(i / nbpr) * (nbpr + 1) + i % nbpr] = src[i];
    __syncthreads();
    if (threadIdx.x < nrow) {
        const float* q = s_part + threadIdx.x * (nbpr + 1);
        float s = 0.f;
        for (uint32_t j = 0; j < nbpr; j++) s += q[j];
        y[row0 + threadIdx.x] = s;
    }
    pdl_launch_dependents();
}

// rows too long for the shared-memory tile: one thread per row straight from global memory
__global__ void __launch_bounds__(128)
reduce_blocks_long_kernel(const float* __restrict__ partial, float* __restrict__ y, uint32_t rows, uint32_t nbpr) {
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
    cudaError_t e;
    if (shared_x && n_w == 1 && p.nbpr <= 256) {
        // dense layer: one warp per 8 blocks of the row, rows strided over the CTAs
        static const int cfg = getenv("FM_DOT_CFG") ? atoi(getenv("FM_DOT_CFG")) : 0;
        if (cfg != 1) {                              // tensor-core kernel: one warp per block index, 16-row units
            auto kern = int4_dot_mma_kernel<2>;
            const int bgroups = (int)((p.nbpr + kDotWarps - 1) / kDotWarps);
            int per_sm = 0;
            e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDotWarps * 32, 0);
            if (e != cudaSuccess) return cuda_fail(kn, e);
            const int units = (int)((rows + 15) / 16);
            int ucta = c.sm_count * (per_sm < 1 ? 1 : per_sm) / bgroups;
            if (ucta < 1) ucta = 1;
            if (ucta > units) ucta = units;
            uint32_t* frags = static_cast<uint32_t*>(engine_scratch((size_t)p.nbpr * 192 * 4));
            FM_REQUIRE(frags != nullptr, kn, "the engine workspace is not available (FM_SCRATCH_MB=0?)");
            e = launch_kernel(int4_dot_split_kernel, dim3((p.nbpr * 192 + 255) / 256), dim3(256), 0, c.stream, pdl_enabled(),
                              p.x, frags, p.nbpr);
            if (e != cudaSuccess) return cuda_fail(kn, e);
            after_launch(kn);
            e = launch_kernel(kern, dim3(ucta * bgroups), dim3(kDotWarps * 32), 0, c.stream, true, p,
                              static_cast<const uint32_t*>(frags));
            return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
        }
        const int warps = (int)((p.nbpr + 7) / 8);
        auto kern = int4_dot_dense_kernel<4>;
        int per_sm = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, warps * 32, 0);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        int grid = c.sm_count * (per_sm < 1 ? 1 : per_sm);
        if ((uint32_t)grid > rows) grid = (int)rows;
        e = launch_kernel(kern, dim3(grid), dim3(warps * 32), 0, c.stream, pdl_enabled(), p);
    } else if (shared_x) {
        FM_REQUIRE(smem <= 200 * 1024, kn, "K=%u is too large for the shared-memory activation row", p.nbpr * 128);
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
    const size_t smem = (size_t)128 * (nbpr + 1) * 4;
    cudaError_t e = smem <= 48 * 1024
        ? launch_kernel(reduce_blocks_kernel, dim3((rows + 127) / 128), dim3(128), smem, c.stream, pdl_enabled(),
                        partial, y, rows, nbpr)
        : launch_kernel(reduce_blocks_long_kernel, dim3((rows + 127) / 128), dim3(128), 0, c.stream, pdl_enabled(),
                        partial, y, rows, nbpr);
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
