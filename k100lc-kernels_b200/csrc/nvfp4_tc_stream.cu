// NVFP4 decode stream on the fifth-generation tensor cores: the E2M1 weight codes go from HBM to the MMA without
// passing through a register.
//
//   nvfp4_decode_stream (default consumer), nvfp4_decode_stream_iacc
//   arithmetic: reference kernels/asm/k_nvfp4/011_*.s:11-62,117-184 (nvfp4_gemv), tools/selftest_all.py:1108-1114:
//     I[n,b] = sum_{k in 16-block b} (2*E2M1(w[n,k])) * q[k]   (exact integer),
//     y[n]   = sum_b I[n,b] * (0.5 * gscale * E4M3(ws[n,b])) * asc[b]
//
// Why.  The SIMT and mma.sync consumers decode every nibble with integer instructions (PRMT, shifts, masks): 12 to 25
// issue slots per packed 32-bit word, which holds the stream at 10 us per 50 MB layer whatever feeds it.  tcgen05.mma
// kind::f8f6f4 reads E2M1 operands from shared memory itself, and TMA's 16U4_ALIGN16B tensor type unpacks the dense
// nibbles of global memory into the padded form that MMA wants (16 codes in 8 bytes, 8 bytes of padding), so the
// weights need no instruction at all.  The int8 activation q is split as q = 16*hi + lo with lo = q & 15 (0..15) and
// hi = q >> 4 (-8..7); both are exact in E4M3 and go in as B.  One MMA has K = 32 = two 16-blocks; they are kept apart
// by the columns of B: column n = part*2 + half holds part (lo / hi) of the codes of half `half` of every 32 k and
// zeros in the other half, so D[row][n] is the sum of one block alone.  Every product is a multiple of 1/2 below
// 2^7 and a block sum stays below 2^11: the fp32 accumulation is exact, I = 2*(D_lo + 16*D_hi) is the oracle's
// integer bit for bit (the _iacc entry stores it), and nothing is accumulated across MMAs — each MMA writes 16 fresh
// columns of tensor memory.
//
// Mapping.  Work unit: a tile of 128 rows of one layer, all of K; tile t goes to CTA t mod grid, so the layers
// complete in order.  Per tile K/256 stages; per stage
//   * copy lane: two TMA box copies (128 rows x 128 codes each -> 16 KB of shared memory each, 128-byte swizzle),
//     the stage's B image (prepared once per token by nvfp4_bimg_kernel: 512 bytes per 128 k for one token) and the
//     16 products asc[b]*gscale, all counted on one mbarrier;
//   * MMA lane: eight tcgen05.mma (M128 N16 K32) into a 128-column slice of tensor memory, one commit that frees the
//     stage and hands the slice to the epilogue;
//   * four epilogue warps: one thread per row; tcgen05.ld of the 32 block sums, I = lo + 16*hi, the E4M3 block scale
//     of the row (16 bytes per stage, read straight from global memory one stage ahead), one multiply and one fused
//     multiply-add per block; after the last stage the row's y goes to the local y and every other receiver.
// All waits are bounded (status 11..15); a wait that runs out raises the CTA-wide abort flag, the copy lane waits
// for the copies it issued, the MMA lane for its MMAs, and tensor memory is released before the CTA returns.
#include <cuda.h>
#include <stdlib.h>

#include "device_utils.cuh"
#include "fm_internal.h"
#include "stream_common.cuh"
#include "tc_utils.cuh"

namespace fm {
namespace {
using namespace tc;
using stream::StreamLayer;
using stream::StreamParams;

constexpr int TM = 128;                       // rows per tile = TMEM lanes
constexpr int SK = 256;                       // k per stage
constexpr int NCOL = 16;                      // columns of one MMA (4 per token: lo/hi x first/second block)
constexpr int STAGES = 6;
constexpr int NACC = 4;                       // 128-column slices of tensor memory
constexpr int ASG_SLOTS = 16;                 // > STAGES + NACC stages between a slot's write and its reuse
constexpr int A_BYTES = TM * SK;              // two boxes of 128 rows x 128 bytes (one byte of shared memory per code)
constexpr int B_BYTES = 2 * NCOL * 128;       // two 128-k chunks of 16 columns x 128 bytes
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int kThreads = 6 * 32;              // copy warp, MMA warp, four epilogue warps
constexpr int kSpin = 1 << 20;
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * STAGE_BYTES + ASG_SLOTS * 256 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory");
static_assert(ASG_SLOTS > STAGES + NACC, "slot reuse distance");

struct TcParams {
    StreamParams s;
    const CUtensorMap* maps;                  // [nlayers]: codes of a layer as [rows][K] 4-bit values, box 128 x 128
    const uint8_t* bimg;                      // [nlayers][K/256][kImgBytes]: B image + scale products of a stage
    int tiles_per_layer, ntiles;
    uint32_t box_tx;                          // bytes one box copy reports to its mbarrier (the packed source bytes)
};
constexpr int kImgBytes = 2 * 4 * 128 + 64;   // one token: rows 0..3 of both chunks, then 16 floats

struct __align__(16) Control {
    uint64_t full[STAGES], empty[STAGES];
    uint64_t acc_full[NACC], acc_empty[NACC];
    uint64_t drain;
    uint64_t stored;                          // the four epilogue warps have stored their rows of a tile (completion counters)
    uint32_t tmem_base;
    volatile int abort;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* b, uint32_t parity, Control* ctl, int* status, int code) {
    for (int i = 0; i < kSpin; i++) {
        if (mbar_try_wait(b, parity)) return true;
        if ((i & 63) == 63 && ctl->abort) return false;
    }
    ctl->abort = 1;
    atomicCAS(status, 0, code);
    return false;
}

// kind::f8f6f4: D fp32, A = E2M1, B = E4M3, both K-major, M = 128, N = 16
__device__ __forceinline__ uint32_t instr_desc() {
    return (1u << 4) | (5u << 7) | (0u << 10) | ((uint32_t)(NCOL >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
}

// E4M3 code in byte `i` of `w` as fp32 / 2^120: the 7 magnitude bits land in the exponent and the top of the
// mantissa, so normal and subnormal codes alike come out as value * 2^-120 (the arithmetic decode of the oracle:
// exponent 15 with mantissa 7 is 480, not a NaN)
__device__ __forceinline__ float e4m3_raw(uint32_t w, int i) {
    const uint32_t b = (w >> (8 * i)) & 0xFFu;
    return __uint_as_float(((b & 0x80u) << 24) | ((b & 0x7Fu) << 20));
}

// Integers 0..15 as E4M3 codes
__device__ __forceinline__ uint32_t e4m3_of_small(int v) {            // v in -15..15
    const uint32_t a = (uint32_t)(v < 0 ? -v : v);
    // 0; 1 = 0x38; 2,3 = 0x40 + 4*(a-2); 4..7 = 0x48 + 2*(a-4); 8..15 = 0x50 + (a-8)
    const uint32_t m = a == 0 ? 0u : a == 1 ? 0x38u : a < 4 ? 0x40u + 4u * (a - 2u) : a < 8 ? 0x48u + 2u * (a - 4u) : 0x50u + (a - 8u);
    return m | (v < 0 ? 0x80u : 0u);
}

// B image of every stage of every layer for one token.  grid (K/256, nlayers), 80 threads: thread i < 64 writes one
// 16-byte piece of the image, threads 64..79 one scale product each.
//   image [chunk 0..1][column n 0..3][128 bytes, 16-byte pieces XOR-swizzled by n], then asg[16] = asc * gscale
__global__ void __launch_bounds__(80)
nvfp4_bimg_kernel(const int8_t* __restrict__ qe, const int8_t* __restrict__ qo, const float* __restrict__ asc, float gscale,
                  uint8_t* __restrict__ bimg, int K) {
    pdl_wait();
    const int s = blockIdx.x, l = blockIdx.y, nst = K / SK, t = threadIdx.x;
    uint8_t* img = bimg + ((size_t)l * nst + s) * kImgBytes;
    if (t < 64) {
        const int ch = t >> 5, n = (t >> 3) & 3, phys = t & 7;
        const int c16 = phys ^ n;                          // logical 16-byte piece = 16 consecutive k
        const int part = n >> 1, half = n & 1;
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        if ((c16 & 1) == half) {
            const int k0 = s * SK + ch * 128 + c16 * 16;   // even
            const size_t o = (size_t)l * (K / 2) + k0 / 2;
            const uint2 e = *reinterpret_cast<const uint2*>(qe + o), od = *reinterpret_cast<const uint2*>(qo + o);
            const uint32_t ew[2] = {e.x, e.y}, ow[2] = {od.x, od.y};
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t src = (i & 1) ? ow[i >> 3] : ew[i >> 3];
                const int q = (int)(int8_t)((src >> (8 * ((i >> 1) & 3))) & 0xFFu);
                const int v = part ? (q >> 4) : (q & 15);
                out[i >> 2] |= e4m3_of_small(v) << (8 * (i & 3));
            }
        }
        *reinterpret_cast<uint4*>(img + ch * 512 + n * 128 + phys * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    } else {
        const int b = t - 64;
        reinterpret_cast<float*>(img + 1024)[b] = asc[(size_t)l * (K / 16) + s * 16 + b] * gscale;
    }
    pdl_launch_dependents();
}

template <bool DUMP>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_tc_stream_kernel(const TcParams pp) {
    const StreamParams& p = pp.s;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Control* ctl = reinterpret_cast<Control*>(smem);
    uint8_t* stages = smem + 1024;
    float* asg_ring = reinterpret_cast<float*>(stages + STAGES * STAGE_BYTES);     // [ASG_SLOTS][64]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nst = p.K / SK;
    const int G = (int)gridDim.x;
    const int my_tiles = ((int)blockIdx.x < pp.ntiles) ? (pp.ntiles - 1 - (int)blockIdx.x) / G + 1 : 0;
    const int total = my_tiles * nst;
    int* status = p.status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int a = 0; a < NACC; a++) {
            mbar_init(&ctl->acc_full[a], 1);
            mbar_init(&ctl->acc_empty[a], 4);
        }
        mbar_init(&ctl->drain, 1);
        mbar_init(&ctl->stored, 4);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // columns 4..15 of B are never written by a copy: they stay zero for the whole kernel
    for (int i = threadIdx.x; i < STAGES * (B_BYTES / 16); i += kThreads) {
        const int s = i / (B_BYTES / 16), o = i % (B_BYTES / 16);
        *reinterpret_cast<uint4*>(stages + s * STAGE_BYTES + A_BYTES + o * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) tmem_alloc(&ctl->tmem_base, NACC * 128);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    pdl_wait();

    if (warp == 0) {
        // ================================================================ copy lane
        if (lane == 0) {
            int issued = 0, it = 0;
            for (int t = (int)blockIdx.x; t < pp.ntiles && !ctl->abort; t += G) {
                const int l = t / pp.tiles_per_layer, r0 = (t % pp.tiles_per_layer) * TM;
                const CUtensorMap* map = pp.maps + l;
                const uint8_t* img = pp.bimg + (size_t)l * nst * kImgBytes;
                bool ok = true;
                for (int s = 0; s < nst; s++, it++) {
                    const int slot = it % STAGES;
                    if (it >= STAGES && !wait_or_abort(&ctl->empty[slot], ((it / STAGES) & 1) ^ 1, ctl, status, 11)) { ok = false; break; }
                    uint8_t* st = stages + slot * STAGE_BYTES;
                    mbar_expect_tx(&ctl->full[slot], 2 * pp.box_tx + kImgBytes);
                    tma_2d(st, map, s * SK, r0, &ctl->full[slot]);
                    tma_2d(st + TM * 128, map, s * SK + 128, r0, &ctl->full[slot]);
                    const uint8_t* im = img + (size_t)s * kImgBytes;
                    bulk_g2s(st + A_BYTES, im, 512, &ctl->full[slot]);
                    bulk_g2s(st + A_BYTES + 2048, im + 512, 512, &ctl->full[slot]);
                    bulk_g2s(asg_ring + (it % ASG_SLOTS) * 64, im + 1024, 64, &ctl->full[slot]);
                    issued = it + 1;
                }
                if (!ok) break;
            }
            if (ctl->abort) {
                for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; j++)
                    for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->full[j % STAGES], (j / STAGES) & 1); i++) {}
            }
        }
    } else if (warp == 1) {
        // ================================================================ MMA lane
        if (lane == 0) {
            const uint32_t idesc = instr_desc();
            const uint64_t adesc0 = smem_desc_sw128(smem_u32(stages));
            const uint64_t bdesc0 = smem_desc_sw128(smem_u32(stages) + A_BYTES);
            for (int it = 0; it < total; it++) {
                const int slot = it % STAGES, a = it % NACC;
                if (it >= NACC && !wait_or_abort(&ctl->acc_empty[a], ((it / NACC) & 1) ^ 1, ctl, status, 13)) break;
                if (!wait_or_abort(&ctl->full[slot], (it / STAGES) & 1, ctl, status, 12)) break;
                tc_fence_after();
                const uint64_t ad = adesc0 + (uint64_t)slot * (STAGE_BYTES >> 4), bd = bdesc0 + (uint64_t)slot * (STAGE_BYTES >> 4);
                const uint32_t d = tmem_base + a * 128;
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        tc_mma_f8f6f4(d + (c * 4 + j) * NCOL, ad + c * ((TM * 128) >> 4) + j * 2, bd + c * (2048 >> 4) + j * 2, idesc, 0);
                tc_commit(&ctl->empty[slot]);              // the stage may be refilled once these MMAs have read it
                tc_commit(&ctl->acc_full[a]);
            }
            tc_commit(&ctl->drain);
            for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->drain, 0); i++) {}
        }
    } else {
        // ================================================================ epilogue: one thread per row of the tile
        const int lq = warp & 3;                            // TMEM lane quarter this warp may read
        const int trow = lq * 32 + lane;
        const int nb = p.K / 16;                            // block scales per row
        int it = 0;
        int flagged = 0;                                    // layers below this one have their counters bumped
        int nev = 0;                                        // completed phases of `stored`
        for (int t = (int)blockIdx.x; t < pp.ntiles; t += G) {
            const int l = t / pp.tiles_per_layer, row = (t % pp.tiles_per_layer) * TM + trow;
            const bool live = row < p.rows;
            const StreamLayer L = p.layers[l];
            const uint8_t* wsr = L.ws + (size_t)(live ? row : 0) * nb;
            uint4 sc = ld_stream_v4(wsr);
            float y = 0.f;
            bool ok = true;
            for (int s = 0; s < nst; s++, it++) {
                const int a = it % NACC;
                const uint4 scn = (s + 1 < nst) ? ld_stream_v4(wsr + (s + 1) * 16) : sc;
                if (!wait_or_abort(&ctl->acc_full[a], (it / NACC) & 1, ctl, status, 14)) { ok = false; break; }
                tc_fence_after();
                uint32_t r[32];
                const uint32_t ta = tmem_base + ((uint32_t)(lq * 32) << 16) + a * 128;
#pragma unroll
                for (int j = 0; j < 8; j++) tmem_ld4(ta + j * NCOL, r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                const float4* ag = reinterpret_cast<const float4*>(asg_ring + (it % ASG_SLOTS) * 64);
                float asg[16];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 v = ag[j];
                    asg[4 * j] = v.x; asg[4 * j + 1] = v.y; asg[4 * j + 2] = v.z; asg[4 * j + 3] = v.w;
                }
                tmem_ld_wait(r);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);        // the slice is in registers
                const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (int j = 0; j < 8; j++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const int b = 2 * j + h;
                        // block sum: D_lo + 16 * D_hi (= I / 2), exact
                        const float tsum = fmaf(__uint_as_float(r[4 * j + 2 + h]), 16.f, __uint_as_float(r[4 * j + h]));
                        const float sw = e4m3_raw(scw[b >> 2], b & 3) * 0x1p120f;
                        y = fmaf(tsum, sw * asg[b], y);
                        if (DUMP && live) p.iacc[((size_t)l * p.rows + row) * nb + s * 16 + b] = (int)(2.f * tsum);
                    }
                sc = scn;
            }
            if (!ok) break;
            if (live) {
                float* dst = L.y + p.row_base + row;
                *dst = y;
#pragma unroll
                for (int q = 0; q < 8; q++)
                    if (q < p.npeers)
                        *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = y;
            }
            if (p.flags) {
                // every epilogue thread has stored its row: counters of the layers this CTA is now done with
                const int tn = t + G;
                const int upto = tn < pp.ntiles ? tn / pp.tiles_per_layer : p.nlayers;      // first layer still open
                if (upto > flagged) {
                    // (a warp cannot be a whole tile ahead of another one: the MMA lane needs all four to release a
                    //  slice and runs at most NACC stages ahead, and a tile has more stages than that)
                    __threadfence_system();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->stored);
                    if (warp == 2) {
                        if (!wait_or_abort(&ctl->stored, nev & 1, ctl, status, 15)) break;
                        for (int f = flagged + lane; f < upto; f += 32) {
                            unsigned* fl = p.flags + f;
                            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(fl) : "memory");
                            for (int q = 0; q < p.npeers; q++)
                                asm volatile("red.release.sys.global.add.u32 [%0], 1;"
                                             ::"l"(reinterpret_cast<char*>(fl) + p.peer_delta[q]) : "memory");
                        }
                    }
                    nev++;
                    flagged = upto;
                }
            }
        }
        // a CTA that had no tile at all (more CTAs than tiles) still counts once per layer
        if (p.flags && my_tiles == 0 && warp == 2) {
            for (int f = lane; f < p.nlayers; f += 32) {
                unsigned* fl = p.flags + f;
                asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(fl) : "memory");
                for (int q = 0; q < p.npeers; q++)
                    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(reinterpret_cast<char*>(fl) + p.peer_delta[q]) : "memory");
            }
        }
        __threadfence_system();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, NACC * 128);
    pdl_launch_dependents();
}

}  // namespace

// The launcher behind nvfp4_decode_stream: prepares the B images of all layers in the engine workspace, then the stream
// kernel.  Returns FM_OK after enqueueing both, a negative code after a rejection, or 1 when this path cannot take the
// launch (no tensor maps for the table, workspace cannot grow here) and the caller should use another consumer.
int nvfp4_tc_stream(const char* kn, const LaunchCtx& c, const stream::StreamParams& sp, float gscale, bool dump) {
    const int nst = sp.K / SK;
    if (sp.K % SK || nst <= NACC || sp.M != 1 || !sp.layers) return 1;
    const void* maps = stream_table_maps(sp.layers, sp.nlayers, sp.rows, sp.K);
    if (!maps) return 1;
    uint8_t* bimg = static_cast<uint8_t*>(engine_scratch((size_t)sp.nlayers * nst * kImgBytes));
    if (!bimg) return 1;
    TcParams pp = {};
    pp.s = sp;
    pp.maps = static_cast<const CUtensorMap*>(maps);
    pp.bimg = bimg;
    pp.tiles_per_layer = (sp.rows + TM - 1) / TM;
    pp.ntiles = pp.tiles_per_layer * sp.nlayers;
    pp.box_tx = TM * 64;                      // a box copy reports the packed bytes it read (measured), not the padded bytes it writes
    auto kern = dump ? nvfp4_tc_stream_kernel<true> : nvfp4_tc_stream_kernel<false>;
    static bool configured[2] = {false, false};
    if (!configured[dump]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured[dump] = true;
    }
    cudaError_t e = launch_kernel(nvfp4_bimg_kernel, dim3(nst, sp.nlayers), dim3(80), 0, c.stream, pdl_enabled(),
                                  reinterpret_cast<const int8_t*>(sp.ae), reinterpret_cast<const int8_t*>(sp.ao),
                                  reinterpret_cast<const float*>(sp.asc), gscale, bimg, sp.K);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    after_launch(kn);
    const int grid = c.sm_count < sp.rows ? c.sm_count : sp.rows;     // the CTA count the completion counters promise
    e = launch_kernel(kern, dim3(grid), dim3(kThreads), kSmemBytes, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

}  // namespace fm
