// NVFP4 decode GEMV: E2M1 weights, E4M3 scale per 16 weights, f32 global scale,
// int8 activations quantised per 16-block (nvfp4_quant_act).
//
//   nvfp4_gemv<A,B>, nvfp4_gemv_wide<A,B>   reference kernels/asm/k_nvfp4/003..026_*.s
//   (template argument A = number of activation rows M, B = weight rows per warp;
//    output [A][N]; a 256-thread work-group of the reference covers 4*B rows)
//
// Arithmetic (reference kernels/asm/k_nvfp4/011_*.s:11-62,117-184; oracle formula
// tools/selftest_all.py:1108-1114):
//   I[n,b] = sum_{k in 16-block b} (2*E2M1(w[n,k])) * q[m,k]            exact int32
//   y[m,n] = sum_b float(I[n,b]) * ((0.5*gscale*E4M3(ws[n,b])) * scale[m,b])
//
// Decode on B200: 2*E2M1 magnitudes {0,1,2,3,4,6,8,12} sit in one 8-byte table and a
// packed weight word is itself the PRMT selector: nibble = sign bit + 3-bit index,
// and PRMT's selector bit 3 means "replicate the selected byte's sign bit", which
// for table bytes < 0x80 yields 0.  So PRMT(table, w) gives the magnitudes of the
// four positive codes (0 elsewhere) and PRMT(table, w ^ 0x8888) those of the four
// negative codes; I = dp4a(pos, q) - dp4a(neg, q).  Activations are re-interleaved
// from the even/odd streams into natural k order once per CTA in shared memory.
// Streaming layout, persistence and the programmatic-dependent-launch prologue are
// those of the W4 GEMV (gemv_w4.cu).
#include <stdlib.h>

#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
struct Nvfp4Params {
    const uint32_t* wq;     // [N][K/8] E2M1 codes, low nibble = lower k
    const uint8_t* ws;      // [N][K/16] E4M3 block scales
    const uint32_t* qa;     // even-k int8 stream [M][K/2] bytes
    const uint32_t* qb;     // odd-k int8 stream
    const float* sc;        // [M][K/16]
    float* y;               // [M][N]
    int* iacc;              // optional dump [M][N][K/16]
    int N, K, rows;
    float gscale;
};

template <int M, int R, int KITER, bool DUMP>
__global__ void __launch_bounds__(kThreads)
nvfp4_gemv_kernel(const Nvfp4Params p) {
    extern __shared__ __align__(16) uint32_t smem[];
    const int KD = p.K >> 3;                 // packed words per weight row
    const int NB = p.K >> 4;                 // 16-blocks per row
    uint32_t* s_a = smem;                    // [M][K/4] natural-order int8
    float* s_sc = reinterpret_cast<float*>(s_a + M * (p.K >> 2));   // [M][NB]
    float* s_lut = s_sc + M * NB;            // [256] 0.5*gscale*E4M3(byte)

    const int lane = threadIdx.x & 31;
    const int gwarp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int nwarp = gridDim.x * kWarps;
    const int iters = KITER > 0 ? KITER : (KD + 127) >> 7;
    constexpr int UN = KITER > 0 ? KITER : 1;

    // one row block is always in flight: the loads of block rb + nwarp are issued right after block rb
    // has been consumed (weights and block scales do not depend on the preceding kernel)
    uint4 wreg[R][UN];
    uint32_t sbyte[R][UN];
    auto fetch = [&](int blk) {
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = blk * R + r;
            const bool live = row < p.rows;
#pragma unroll
            for (int it = 0; it < UN; it++) {
                const int d0 = it * 128 + lane * 4;
                wreg[r][it] = live ? ld_stream_v4(p.wq + (size_t)row * KD + d0) : make_uint4(0, 0, 0, 0);
                sbyte[r][it] = live ? ld_stream_u16(p.ws + (size_t)row * NB + (d0 >> 1)) : 0u;
            }
        }
    };
    int rb = gwarp;
    if (KITER > 0) fetch(rb);

    pdl_wait();
    constexpr bool AREG = M == 1 && KITER > 0;   // one token: its codes go straight from L2 into registers
    uint4 ra0[AREG ? UN : 1], ra1[AREG ? UN : 1];
    float2 rsc[AREG ? UN : 1];
    if (AREG) {
#pragma unroll
        for (int it = 0; it < UN; it++) {
            const int d0 = it * 128 + lane * 4;
            const uint4 e = *reinterpret_cast<const uint4*>(p.qa + d0), o = *reinterpret_cast<const uint4*>(p.qb + d0);
            ra0[it] = make_uint4(prmt(e.x, o.x, 0x5140u), prmt(e.x, o.x, 0x7362u), prmt(e.y, o.y, 0x5140u), prmt(e.y, o.y, 0x7362u));
            ra1[it] = make_uint4(prmt(e.z, o.z, 0x5140u), prmt(e.z, o.z, 0x7362u), prmt(e.w, o.w, 0x5140u), prmt(e.w, o.w, 0x7362u));
            rsc[it] = *reinterpret_cast<const float2*>(p.sc + (d0 >> 1));
        }
    } else {
        for (int i = threadIdx.x; i < M * KD; i += blockDim.x) {
            const uint32_t e = p.qa[i], o = p.qb[i];
            s_a[2 * i] = prmt(e, o, 0x5140u);        // k0 k1 k2 k3
            s_a[2 * i + 1] = prmt(e, o, 0x7362u);    // k4 k5 k6 k7
        }
        for (int i = threadIdx.x; i < M * NB; i += blockDim.x) s_sc[i] = p.sc[i];
    }
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_lut[i] = (0.5f * p.gscale) * e4m3_to_f32(i);
    __syncthreads();

    for (; rb * R < p.rows; rb += nwarp) {
        float acc[R][M];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int m = 0; m < M; m++) acc[r][m] = 0.f;


#pragma unroll 1
        for (int it0 = 0; it0 < iters; it0 += UN) {
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int it = it0 + u;
                const int d0 = it * 128 + lane * 4;
                const bool ok = KITER > 0 || d0 < KD;
                const int dc = ok ? d0 : 0;
                const int b0 = dc >> 1;                     // first of the lane's two 16-blocks
                uint4 w4[R];
                uint32_t sb[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if (KITER > 0) {
                        w4[r] = wreg[r][u];
                        sb[r] = sbyte[r][u];
                    } else {
                        const int row = rb * R + r;
                        const bool live = ok && row < p.rows;
                        w4[r] = live ? ld_stream_v4(p.wq + (size_t)row * KD + dc) : make_uint4(0, 0, 0, 0);
                        sb[r] = live ? ld_stream_u16(p.ws + (size_t)row * NB + b0) : 0u;
                    }
                }
#pragma unroll
                for (int m = 0; m < M; m++) {
                    const uint4 a0 = AREG ? ra0[u] : *reinterpret_cast<const uint4*>(s_a + m * (p.K >> 2) + 2 * dc);
                    const uint4 a1 = AREG ? ra1[u] : *reinterpret_cast<const uint4*>(s_a + m * (p.K >> 2) + 2 * dc + 4);
                    const float2 as = AREG ? rsc[u] : *reinterpret_cast<const float2*>(s_sc + m * NB + b0);
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        int i0 = dot8_e2m1(w4[r].x, a0.x, a0.y, 0);
                        i0 = dot8_e2m1(w4[r].y, a0.z, a0.w, i0);
                        int i1 = dot8_e2m1(w4[r].z, a1.x, a1.y, 0);
                        i1 = dot8_e2m1(w4[r].w, a1.z, a1.w, i1);
                        if (ok) {
                            acc[r][m] = fmaf((float)i0, s_lut[sb[r] & 0xFFu] * as.x, acc[r][m]);
                            acc[r][m] = fmaf((float)i1, s_lut[(sb[r] >> 8) & 0xFFu] * as.y, acc[r][m]);
                            if (DUMP) {
                                const int row = rb * R + r;
                                if (row < p.rows) {
                                    int* d = p.iacc + ((size_t)m * p.N + row) * NB + b0;
                                    d[0] = i0;
                                    d[1] = i1;
                                }
                            }
                        }
                    }
                }
            }
        }
        if (KITER > 0) fetch(rb + nwarp);                   // next block of this warp (no loads past the end)

#pragma unroll
        for (int r = 0; r < R; r++) {
            const int row = rb * R + r;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0 && row < p.rows) p.y[(size_t)m * p.N + row] = v;
            }
        }
    }
    pdl_launch_dependents();
}

template <int M, int R, int KITER, bool DUMP>
int run_variant(const char* kn, const LaunchCtx& c, const Nvfp4Params& p) {
    auto kern = nvfp4_gemv_kernel<M, R, KITER, DUMP>;
    const size_t smem = (size_t)M * (p.K + (p.K / 16) * 4) + 1024;
    FM_REQUIRE(smem <= 200 * 1024, kn, "K=%d needs %zu bytes of shared memory for %d tokens (limit 200 KiB)", p.K,
               smem, M);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
    }
    const int blocks_needed = (p.rows + R * kWarps - 1) / (R * kWarps);
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kThreads, smem);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    if (per_sm < 1) per_sm = 1;
    int grid = c.sm_count * per_sm;
    if (grid > blocks_needed) grid = blocks_needed;
    e = launch_kernel(kern, dim3(grid), dim3(kThreads), smem, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

template <int M, bool DUMP>
int dispatch(const char* kn, const LaunchCtx& c, const Nvfp4Params& p) {
    const int kiter = (p.K % 1024 == 0) ? p.K / 1024 : 0;
    if (DUMP) return run_variant<M, 1, 0, true>(kn, c, p);
    if (M == 1) {
        // (the register path reads the codes as 16-byte words)
        if (kiter == 5 && aligned(p.qa, 16) && aligned(p.qb, 16)) return run_variant<1, 1, 5, false>(kn, c, p);
        return run_variant<1, 1, 0, false>(kn, c, p);
    }
    if (kiter == 5) return run_variant<M, 2, 5, false>(kn, c, p);
    return run_variant<M, 2, 0, false>(kn, c, p);
}

int fill(const char* kn, const LaunchCtx& c, const uint64_t* a, Nvfp4Params& p, int M, int rows_per_wg, bool dump) {
    p.wq = arg_ptr<const uint32_t>(a[0]);
    p.ws = arg_ptr<const uint8_t>(a[1]);
    p.qa = arg_ptr<const uint32_t>(a[2]);
    p.qb = arg_ptr<const uint32_t>(a[3]);
    p.sc = arg_ptr<const float>(a[4]);
    p.y = arg_ptr<float>(a[5]);
    p.N = arg_i32(a[6]);
    p.K = arg_i32(a[7]);
    p.gscale = arg_f32(a[8]);
    FM_REQUIRE(c.wx == 256 && c.wy == 1 && c.gy == 1, kn,
               "work-group must be 256x1 threads on a 1-D grid; got %ux%u, grid y=%u", c.wx, c.wy, c.gy);
    FM_REQUIRE(p.N > 0 && p.K > 0 && p.K % 32 == 0, kn,
               "N=%d K=%d: K must be a positive multiple of 32 (16-byte weight words)", p.N, p.K);
    const long long covered = (long long)c.gx * rows_per_wg;
    p.rows = (int)(covered < p.N ? covered : p.N);
    FM_REQUIRE(aligned(p.wq, 16) && aligned(p.ws, 2) && aligned(p.qa, 4) && aligned(p.qb, 4) && aligned(p.sc, 8) &&
                   aligned(p.y, 4), kn, "misaligned pointer (weights need 16 bytes, scales 2/8, codes 4)");
    if (p.rows == 0) return 1;
    FM_RANGE(p.wq, (size_t)p.rows * (p.K / 2), kn, "wq");
    FM_RANGE(p.ws, (size_t)p.rows * (p.K / 16), kn, "ws");
    FM_RANGE(p.qa, (size_t)M * (p.K / 2), kn, "a");
    FM_RANGE(p.qb, (size_t)M * (p.K / 2), kn, "b");
    FM_RANGE(p.sc, (size_t)M * (p.K / 16) * 4, kn, "scale");
    FM_RANGE(p.y, ((size_t)(M - 1) * p.N + p.rows) * 4, kn, "y");
    if (dump) {
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, (size_t)M * p.N * (p.K / 16) * 4, kn, "iacc");
    }
    return 0;
}

// nvfp4_gemv<A,B> / nvfp4_gemv_wide<A,B> (wq, ws, a, b, scale, y, N, K, gscale)
template <int A, int B>
int launch_nvfp4(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "nvfp4_gemv<A,B>";
    Nvfp4Params p = {};
    const int rc = fill(kn, c, a, p, A, 4 * B, false);
    if (rc) return rc < 0 ? rc : FM_OK;
    return dispatch<A, false>(kn, c, p);
}

// nvfp4_gemv_iacc(wq, ws, a, b, scale, y, N, K, gscale, iacc, M): extension used by the
// parity tests; iacc int32 [M][N][K/16].
int launch_nvfp4_iacc(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "nvfp4_gemv_iacc";
    Nvfp4Params p = {};
    p.iacc = arg_ptr<int>(a[9]);
    const int M = arg_i32(a[10]);
    FM_REQUIRE(M >= 1 && M <= 4, kn, "M=%d must be 1..4", M);
    const int rc = fill(kn, c, a, p, M, 4, true);
    if (rc) return rc < 0 ? rc : FM_OK;
    switch (M) {
        case 1: return dispatch<1, true>(kn, c, p);
        case 2: return dispatch<2, true>(kn, c, p);
        case 3: return dispatch<3, true>(kn, c, p);
        default: return dispatch<4, true>(kn, c, p);
    }
}

#define NV(A, B) {"nvfp4_gemv<" #A "," #B ">", 9, launch_nvfp4<A, B>, "ppppppiif"}
#define NVW(A, B) {"nvfp4_gemv_wide<" #A "," #B ">", 9, launch_nvfp4<A, B>, "ppppppiif"}
const KernelEntry kNvfp4[] = {
    NV(1, 1), NV(1, 2), NV(1, 3), NV(1, 4), NV(2, 1), NV(2, 2), NV(2, 3), NV(2, 4),
    NV(3, 1), NV(3, 2), NV(3, 3), NV(3, 4), NV(4, 1), NV(4, 2), NV(4, 3), NV(4, 4),
    NVW(1, 1), NVW(1, 2), NVW(2, 1), NVW(2, 2), NVW(3, 1), NVW(3, 2), NVW(4, 1), NVW(4, 2),
    {"nvfp4_gemv_iacc", 11, launch_nvfp4_iacc, "ppppppiifpi"},
};

}  // namespace

const KernelEntry* gemv_nvfp4_kernels(int* n) {
    *n = (int)(sizeof(kNvfp4) / sizeof(kNvfp4[0]));
    return kNvfp4;
}

}  // namespace fm
