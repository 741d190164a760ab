// NVFP4 prefill GEMM  C[M,N] = A[M,K] . W[N,K]^T  with E2M1 weights, an E4M3 scale per 16 weights, an f32 global
// scale, and int8 activations quantised per (token, 16-block) by nvfp4_quant_act.
//
//   nvfp4_gemm_kernel, nvfp4_gemm_kernel_ng (wq, ws, a, b, scale, C, M, N, K, gscale)
//       reference kernels/asm/k_nvfp4/002_*.s and 025_*.s (the two files are the same code): 64 x 64 output tiles on a
//       2-D grid, 256 threads.  The reference never verified these two kernels (CHANGELOG.md:1380-1383), so the
//       arithmetic is defined here by extension of nvfp4_gemv (k_nvfp4/011_*.s:117-184): per (token m, row n, block b)
//           I = sum_{k in b} (2 * E2M1(w[n,k])) * q[m,k]                                     exact int32
//           C[m,n] = sum_b fmaf(float(I), (0.5 * gscale * E4M3(ws[n,b])) * scale[m,b], C)    b ascending
//       — "parity unpinned" by the reference's tests; the oracle is nvfp4_gemv's formula applied to M rows.
//   nvfp4_gemm_iacc (..., gscale, iacc)   the same kernel with the integers stored, iacc int32 [M][N][K/16].
//
// Mapping.  Per-block exactness asks for contractions of 16, so the tensor-core instruction is mma.sync m16n8k16
// (int8): 16 weight rows x 16 k times 16 k x 8 tokens.  The packed weight half-word of a lane (4 codes) is the PRMT
// selector into the table of doubled magnitudes: PRMT(table, w) gives the positive codes' magnitudes, PRMT(table,
// w ^ 0x8888) the negative ones; I = MMA(pos, q) - MMA(neg, q).  A CTA computes 128 weight rows x 64 tokens, its 8 warps 32 x 32 each
// (two row tiles, four token tiles), walking K in chunks of 128 (8 blocks) through double-buffered shared memory:
// the activation codes are re-interleaved from the even / odd streams into natural k order on their way in.
// The per-block scaling (one conversion, one multiply, one fused multiply-add per output element and block) is what
// bounds the kernel, not the tensor pipe.
#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int BN = 128, BM = 64, KC = 128, NBC = KC / 16;     // weight rows, tokens, k and blocks per chunk
constexpr int kThreads = 256;
constexpr int WP = 80;                                        // pitch of a packed weight row (64 bytes + pad)
constexpr int AP = 144;                                       // pitch of a token's 128 codes (+ pad)
struct Stage {
    uint8_t w[BN * WP];            // packed E2M1 codes
    uint8_t s[BN * NBC];           // E4M3 block scales
    uint8_t a[BM * AP];            // int8 activation codes, natural k order
    float sc[BM * NBC];            // activation block scales
};

struct GemmNvParams {
    const uint8_t* wq;     // [N][K/2]
    const uint8_t* ws;     // [N][K/16]
    const uint8_t* a;      // even codes [M][K/2]
    const uint8_t* b;      // odd codes [M][K/2]
    const float* scale;    // [M][K/16]
    float* C;              // [M][N]
    int* iacc;             // optional [M][N][K/16]
    int M, N, K;
    float gscale;
};

__device__ __forceinline__ void mma_k16(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0, const int (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%7,%8,%9,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                 : "r"(a0), "r"(a1), "r"(b0), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}
struct Prefetch {                  // one chunk on its way from global memory to shared memory, in registers
    uint4 w[2];
    uint2 s;
    uint4 e, o;
    float4 sc;
};

template <bool DUMP>
__global__ void __launch_bounds__(kThreads, DUMP ? 1 : 2)
nvfp4_gemm_kernel(const GemmNvParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Stage* st = reinterpret_cast<Stage*>(smem_raw);
    float* lut = reinterpret_cast<float*>(smem_raw + 2 * sizeof(Stage));          // [256] 0.5 * gscale * E4M3(byte)
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wn = warp & 3, wm = warp >> 2;                   // warp tile: rows wn*32.., tokens wm*32..
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const int KH = p.K >> 1, NB = p.K >> 4, nchunks = p.K / KC;
    for (int i = tid; i < 256; i += kThreads) lut[i] = (0.5f * p.gscale) * e4m3_to_f32(i);
    pdl_wait();

    // ---- loaders: thread -> its pieces of a chunk
    const int wrow = tid >> 2, wseg = tid & 3;                 // weights: rows wrow and wrow + 64, 16-byte segment wseg
    const int arow = tid >> 2, aseg = tid & 3;                 // activations: token arow, 16 even + 16 odd codes
    auto fetch = [&](int kc, Prefetch& f) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int n = n0 + wrow + h * 64;
            f.w[h] = n < p.N ? ld_stream_v4(p.wq + (size_t)n * KH + kc * 64 + wseg * 16) : make_uint4(0, 0, 0, 0);
        }
        if (tid < BN) {
            const int n = n0 + tid;
            f.s = n < p.N ? *reinterpret_cast<const uint2*>(p.ws + (size_t)n * NB + kc * NBC) : make_uint2(0, 0);
        }
        const int m = m0 + arow;
        if (m < p.M) {
            f.e = *reinterpret_cast<const uint4*>(p.a + (size_t)m * KH + kc * 64 + aseg * 16);
            f.o = *reinterpret_cast<const uint4*>(p.b + (size_t)m * KH + kc * 64 + aseg * 16);
        } else {
            f.e = f.o = make_uint4(0, 0, 0, 0);
        }
        if (tid < BM * 2) {
            const int mm = m0 + (tid >> 1);
            f.sc = mm < p.M ? *reinterpret_cast<const float4*>(p.scale + (size_t)mm * NB + kc * NBC + (tid & 1) * 4)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](Stage& s, const Prefetch& f) {
#pragma unroll
        for (int h = 0; h < 2; h++) *reinterpret_cast<uint4*>(s.w + (wrow + h * 64) * WP + wseg * 16) = f.w[h];
        if (tid < BN) *reinterpret_cast<uint2*>(s.s + tid * NBC) = f.s;
        // even / odd streams -> natural k order: 16 + 16 codes become 32 consecutive ones
        const uint32_t ev[4] = {f.e.x, f.e.y, f.e.z, f.e.w}, ov[4] = {f.o.x, f.o.y, f.o.z, f.o.w};
        uint32_t nat[8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            nat[2 * j] = prmt(ev[j], ov[j], 0x5140u);
            nat[2 * j + 1] = prmt(ev[j], ov[j], 0x7362u);
        }
        uint8_t* da = s.a + arow * AP + aseg * 32;
        *reinterpret_cast<uint4*>(da) = make_uint4(nat[0], nat[1], nat[2], nat[3]);
        *reinterpret_cast<uint4*>(da + 16) = make_uint4(nat[4], nat[5], nat[6], nat[7]);
        if (tid < BM * 2) *reinterpret_cast<float4*>(s.sc + (tid >> 1) * NBC + (tid & 1) * 4) = f.sc;
    };

    float acc[2][4][4];                                        // [row tile][token tile][fragment element]
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f;

    Prefetch pf;
    fetch(0, pf);
    stash(st[0], pf);
    __syncthreads();
    const int zero[4] = {0, 0, 0, 0};
    for (int kc = 0; kc < nchunks; kc++) {
        const Stage& s = st[kc & 1];
        if (kc + 1 < nchunks) fetch(kc + 1, pf);               // in flight while this chunk is multiplied
#pragma unroll 2
        for (int blk = 0; blk < NBC; blk++) {
            uint32_t bq[4];
            float sa[4][2];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int tok = wm * 32 + j * 8;
                bq[j] = *reinterpret_cast<const uint32_t*>(s.a + (tok + g) * AP + blk * 16 + 4 * t);
                sa[j][0] = s.sc[(tok + 2 * t) * NBC + blk];
                sa[j][1] = s.sc[(tok + 2 * t + 1) * NBC + blk];
            }
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const int ra = wn * 32 + i * 16 + g, rb = ra + 8;
                const uint32_t wa = *reinterpret_cast<const unsigned short*>(s.w + ra * WP + blk * 8 + 2 * t);
                const uint32_t wb = *reinterpret_cast<const unsigned short*>(s.w + rb * WP + blk * 8 + 2 * t);
                const uint32_t pa = prmt(kTabLo, kTabHi, wa), pb = prmt(kTabLo, kTabHi, wb);
                const uint32_t na = prmt(kTabLo, kTabHi, wa ^ 0x8888u), nb = prmt(kTabLo, kTabHi, wb ^ 0x8888u);
                const float la = lut[s.s[ra * NBC + blk]], lb = lut[s.s[rb * NBC + blk]];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    int d[4], dn[4], d2[4];
                    mma_k16(d, pa, pb, bq[j], zero);
                    mma_k16(dn, na, nb, bq[j], zero);
#pragma unroll
                    for (int e = 0; e < 4; e++) d2[e] = d[e] - dn[e];
                    acc[i][j][0] = fmaf((float)d2[0], la * sa[j][0], acc[i][j][0]);
                    acc[i][j][1] = fmaf((float)d2[1], la * sa[j][1], acc[i][j][1]);
                    acc[i][j][2] = fmaf((float)d2[2], lb * sa[j][0], acc[i][j][2]);
                    acc[i][j][3] = fmaf((float)d2[3], lb * sa[j][1], acc[i][j][3]);
                    if (DUMP) {
                        const int b = kc * NBC + blk;
                        const int na_ = n0 + ra, nb_ = n0 + rb, ma = m0 + wm * 32 + j * 8 + 2 * t;
                        if (ma < p.M && na_ < p.N) p.iacc[((size_t)ma * p.N + na_) * NB + b] = d2[0];
                        if (ma + 1 < p.M && na_ < p.N) p.iacc[((size_t)(ma + 1) * p.N + na_) * NB + b] = d2[1];
                        if (ma < p.M && nb_ < p.N) p.iacc[((size_t)ma * p.N + nb_) * NB + b] = d2[2];
                        if (ma + 1 < p.M && nb_ < p.N) p.iacc[((size_t)(ma + 1) * p.N + nb_) * NB + b] = d2[3];
                    }
                }
            }
        }
        if (kc + 1 < nchunks) stash(st[(kc + 1) & 1], pf);     // the other buffer: nobody reads it during this chunk
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int na_ = n0 + wn * 32 + i * 16 + g, ma = m0 + wm * 32 + j * 8 + 2 * t;
            if (ma < p.M && na_ < p.N) p.C[(size_t)ma * p.N + na_] = acc[i][j][0];
            if (ma + 1 < p.M && na_ < p.N) p.C[(size_t)(ma + 1) * p.N + na_] = acc[i][j][1];
            if (ma < p.M && na_ + 8 < p.N) p.C[(size_t)ma * p.N + na_ + 8] = acc[i][j][2];
            if (ma + 1 < p.M && na_ + 8 < p.N) p.C[(size_t)(ma + 1) * p.N + na_ + 8] = acc[i][j][3];
        }
    pdl_launch_dependents();
}

constexpr size_t kSmem = 2 * sizeof(Stage) + 1024;

template <bool DUMP>
int launch_nvfp4_gemm(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = DUMP ? "nvfp4_gemm_iacc" : "nvfp4_gemm_kernel";
    GemmNvParams p = {};
    p.wq = arg_ptr<const uint8_t>(a[0]);
    p.ws = arg_ptr<const uint8_t>(a[1]);
    p.a = arg_ptr<const uint8_t>(a[2]);
    p.b = arg_ptr<const uint8_t>(a[3]);
    p.scale = arg_ptr<const float>(a[4]);
    p.C = arg_ptr<float>(a[5]);
    p.M = arg_i32(a[6]);
    p.N = arg_i32(a[7]);
    p.K = arg_i32(a[8]);
    p.gscale = arg_f32(a[9]);
    FM_REQUIRE(c.wx == 256 && c.wy == 1, kn, "work-group must be 256 threads (got %ux%u)", c.wx, c.wy);
    FM_REQUIRE(p.M > 0 && p.N > 0 && p.K > 0 && p.K % KC == 0, kn, "M=%d N=%d K=%d: K must be a multiple of %d", p.M, p.N, p.K, KC);
    // the reference's geometry: 64 x 64 output tiles, grid x over N, grid y over M
    FM_REQUIRE(DUMP || ((long long)c.gx * 64 >= p.N && (long long)c.gy * 64 >= p.M), kn,
               "grid %ux%u does not cover ceil(N/64)=%d by ceil(M/64)=%d tiles; partial grids are not built", c.gx, c.gy,
               (p.N + 63) / 64, (p.M + 63) / 64);
    FM_REQUIRE(aligned(p.wq, 16) && aligned(p.ws, 8) && aligned(p.a, 16) && aligned(p.b, 16) && aligned(p.scale, 16) && aligned(p.C, 4),
               kn, "misaligned pointer (codes and activation scales need 16 bytes, block scales 8)");
    FM_RANGE(p.wq, (size_t)p.N * (p.K / 2), kn, "wq");
    FM_RANGE(p.ws, (size_t)p.N * (p.K / 16), kn, "ws");
    FM_RANGE(p.a, (size_t)p.M * (p.K / 2), kn, "a");
    FM_RANGE(p.b, (size_t)p.M * (p.K / 2), kn, "b");
    FM_RANGE(p.scale, (size_t)p.M * (p.K / 16) * 4, kn, "scale");
    FM_RANGE(p.C, (size_t)p.M * p.N * 4, kn, "C");
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[10]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, (size_t)p.M * p.N * (p.K / 16) * 4, kn, "iacc");
    }
    auto kern = nvfp4_gemm_kernel<DUMP>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    const dim3 grid((p.N + BN - 1) / BN, (p.M + BM - 1) / BM);
    cudaError_t e = launch_kernel(kern, grid, dim3(kThreads), kSmem, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kNvGemm[] = {
    {"nvfp4_gemm_kernel", 10, launch_nvfp4_gemm<false>, "ppppppiiif"},
    {"nvfp4_gemm_kernel_ng", 10, launch_nvfp4_gemm<false>, "ppppppiiif"},
    {"nvfp4_gemm_iacc", 11, launch_nvfp4_gemm<true>, "ppppppiiifp"},
};

}  // namespace

const KernelEntry* nvfp4_gemm_kernels(int* n) {
    *n = (int)(sizeof(kNvGemm) / sizeof(kNvGemm[0]));
    return kNvGemm;
}

}  // namespace fm
