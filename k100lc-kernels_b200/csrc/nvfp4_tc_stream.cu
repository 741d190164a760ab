// NVFP4 decode stream on the fifth-generation tensor cores: the E2M1 weight codes go from HBM to the MMA as they
// are, without passing through a register.
//
//   nvfp4_decode_stream (default consumer), nvfp4_decode_stream_iacc
//   arithmetic: reference kernels/asm/k_nvfp4/011_*.s:11-62,117-184 (nvfp4_gemv), tools/selftest_all.py:1108-1114:
//     I[n,b] = sum_{k in 16-block b} (2*E2M1(w[n,k])) * q[k]   (exact integer),
//     y[n]   = sum_b I[n,b] * (0.5 * gscale * E4M3(ws[n,b])) * asc[b]
//
// Why.  The SIMT and mma.sync consumers decode every nibble with integer instructions (PRMT, shifts, masks): 12 to 25
// issue slots per packed 32-bit word, which holds the stream at 10 us per 50 MB layer whatever feeds it.
// tcgen05.mma kind::mxf4 reads densely packed E2M1 operands from shared memory — exactly the bytes of the reference
// layout — so a plain TMA box copy feeds it and the weights cost no instruction.  Both operands must then be E2M1, so
// the int8 activation code is written in balanced base 7, q = d0 + 7*d1 + 49*d2 with digits in -3..3 (all E2M1
// values), three columns of B per token.  One MMA has K = 64 = four 16-blocks; they are kept apart by the columns of
// B as well: column n = digit*4 + quarter carries the digit only at the k of that quarter of every 64 and zeros
// elsewhere, so D[row][n] is the sum over one block alone.  The block scale factors that this MMA kind multiplies
// in are all set to 1 (UE8M0 0x7F in every byte of the scale region of tensor memory).  Every product is a multiple
// of 1/2 below 2^5 and a block sum stays below 2^9: the fp32 accumulation is exact, I = 2*(D0 + 7*D1 + 49*D2) is the
// oracle's integer bit for bit (the _iacc entry stores it), and nothing is accumulated across MMAs — each MMA
// writes 16 fresh columns of tensor memory.
// (Built first and dropped: kind::f8f6f4 with TMA's unpacking 16U4_ALIGN16B tensor type and the activations as two
//  E4M3 halves.  Bit-exact too, but the padded shared-memory form — one byte per code — halves the weight bytes a CTA
//  can have in flight and doubles the MMAs per byte; the dense form needs neither.)
//
// Mapping.  Work unit: a tile of 128 rows of one layer, all of K; tile t goes to CTA t mod grid, so the layers
// complete in order.  Per tile K/256 stages; per stage
//   * a copy lane (two take the stages in turn): one TMA box copy (128 rows x 128 bytes = 256 codes per row, 128-byte
//     swizzle: the K-major layout the MMA reads), the stage's B image (prepared once per token by nvfp4_bimg_kernel:
//     12 columns x 128 bytes) and the 16 products asc[b]*gscale, all counted on one mbarrier; twelve stages = 192 KB
//     of weights in flight per SM;
//   * an MMA lane (four take the stages in turn): four tcgen05.mma (M128 N16 K64) into a 64-column slice of tensor
//     memory, one commit that frees the stage and one that hands the slice to the epilogue;
//   * eight epilogue warps, two per lane quarter of tensor memory taking the stages in turn: one thread per row;
//     tcgen05.ld of the 48 digit sums, I/2 = D0 + 7*D1 + 49*D2, the E4M3 block scale of the row (16 bytes per
//     stage through L1, requested four stages ahead), one multiply and one fused multiply-add per block; after the
//     last stage the two partial sums of a row meet and y goes to the local y and every receiver.
// All waits are bounded (status 11..17); a wait that runs out raises the CTA-wide abort flag, the copy lane waits
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
constexpr int NCOL = 16;                      // columns of one MMA: 3 digits x 4 quarters of its K = 64, 4 unused
constexpr int UCOL = 12;                      // columns of B that carry data
constexpr int STAGES = 12;
constexpr int NACC = 6;                       // 64-column slices of tensor memory
constexpr int ACC_COLS = 4 * NCOL;            // four MMAs per stage
constexpr int SF_COL = 448;                   // 16 columns of scale factors, all 1
constexpr int ASG_SLOTS = 24;                 // > STAGES + NACC stages between a slot's write and its reuse
constexpr int A_BYTES = TM * SK / 2;          // one box of 128 rows x 128 bytes, packed codes
constexpr int B_BYTES = NCOL * 128;           // 16 columns x 128 bytes
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
// Every role is a chain of barrier waits, and a wait costs a few hundred cycles even when the barrier is ready: one
// thread per role would hold the stream to its own pace.  So the stages go round NCOPY copy lanes and NMMA MMA lanes
// (one lane of a warp each), and round two epilogue warps per TMEM lane quarter.
constexpr int NCOPY = 2, NMMA = 4;
constexpr int EPI_WARP0 = NCOPY + NMMA;        // a multiple of 2; warp % 4 is the TMEM lane quarter a warp may read
constexpr int kThreads = (EPI_WARP0 + 8) * 32;
constexpr int kSpin = 1 << 20;
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * STAGE_BYTES + ASG_SLOTS * 64 + 2 * TM * 4 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory");
static_assert(ASG_SLOTS > STAGES + NACC, "slot reuse distance");

struct TcParams {
    StreamParams s;
    const CUtensorMap* maps;                  // [nlayers]: codes of a layer as [rows][K/2] bytes, box 128 bytes x 128 rows
    const uint8_t* bimg;                      // [nlayers][K/256][kImgBytes]: B image + scale products of a stage
    int tiles_per_layer, ntiles;
};
constexpr int kImgBytes = UCOL * 128 + 64;    // one token: columns 0..11, then 16 floats

struct __align__(16) Control {
    uint64_t full[STAGES], empty[STAGES];
    uint64_t acc_full[NACC], acc_empty[NACC];
    uint64_t drain[NMMA];
    uint64_t stored;                          // the four storing warps have stored their rows of a tile (completion counters)
    uint64_t ysum[4][2];                      // per lane quarter and buffer: the odd-stage warp has put its partial sums into ytmp
    uint64_t yfree[4][2];                     // ... and the even-stage warp has taken them out again
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

// kind::mxf4 (block-scaled): A = B = E2M1 (format 1), both K-major, N = 16, scale factors UE8M0 (bit 23),
// M = 128, K = 64 (bit 31 clear), scale-factor byte ids 0
__device__ __forceinline__ uint32_t instr_desc() {
    return (1u << 7) | (1u << 10) | ((uint32_t)(NCOL >> 3) << 17) | (1u << 23) | ((uint32_t)(TM >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_mxf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, 0, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%4], [%5], p;\n}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb) : "memory");
}

// E4M3 code in byte `i` of `w` as fp32 / 2^120: the 7 magnitude bits land in the exponent and the top of the
// mantissa, so normal and subnormal codes alike come out as value * 2^-120 (the arithmetic decode of the oracle:
// exponent 15 with mantissa 7 is 480, not a NaN)
__device__ __forceinline__ float e4m3_raw(uint32_t w, int i) {
    const uint32_t b = (w >> (8 * i)) & 0xFFu;
    return __uint_as_float(((b & 0x80u) << 24) | ((b & 0x7Fu) << 20));
}

// digit `which` (0..2) of q = d0 + 7*d1 + 49*d2, digits in -3..3, as an E2M1 code (1 -> 2, 2 -> 4, 3 -> 5, sign in bit 3)
__device__ __forceinline__ uint32_t digit_code(int q, int which) {
    const int q1 = (q + 3 + 126) / 7 - 18;                 // floor((q + 3) / 7)
    const int d0 = q - 7 * q1;
    const int d2 = (q1 + 3 + 21) / 7 - 3;
    const int d1 = q1 - 7 * d2;
    const int d = which == 0 ? d0 : which == 1 ? d1 : d2;
    const uint32_t a = (uint32_t)(d < 0 ? -d : d);
    return (a == 3 ? 5u : 2u * a) | (d < 0 ? 8u : 0u);
}

// B image of every stage of every layer for one token.  grid (K/256, nlayers), 112 threads: thread i < 96 writes one
// 16-byte piece of the image, threads 96..111 one scale product each.
//   image [column n = digit*4 + quarter, 0..11][128 bytes = 256 codes, 16-byte pieces XOR-swizzled by n & 7],
//   then asg[16] = asc * gscale
__global__ void __launch_bounds__(112)
nvfp4_bimg_kernel(const int8_t* __restrict__ qe, const int8_t* __restrict__ qo, const float* __restrict__ asc, float gscale,
                  uint8_t* __restrict__ bimg, int K) {
    pdl_wait();
    const int s = blockIdx.x, l = blockIdx.y, nst = K / SK, t = threadIdx.x;
    uint8_t* img = bimg + ((size_t)l * nst + s) * kImgBytes;
    if (t < 96) {
        const int n = t >> 3, phys = t & 7;
        const int c16 = phys ^ (n & 7);                    // logical 16-byte piece = 32 consecutive k = two quarters
        const int dg = n >> 2, qt = n & 3;
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        if ((qt >> 1) == (c16 & 1)) {
            const int h = qt & 1;                          // which half of the piece is this column's quarter
            const int k0 = s * SK + c16 * 32 + 16 * h;     // 16 codes from here: bytes 8h..8h+7 of the piece
            const size_t o = (size_t)l * (K / 2) + k0 / 2;
            const uint2 e = *reinterpret_cast<const uint2*>(qe + o), od = *reinterpret_cast<const uint2*>(qo + o);
            const uint32_t ew[2] = {e.x, e.y}, ow[2] = {od.x, od.y};
#pragma unroll
            for (int m = 0; m < 8; m++) {                  // byte m: code of k0 + 2m below, of k0 + 2m + 1 above
                const int qa = (int)(int8_t)((ew[m >> 2] >> (8 * (m & 3))) & 0xFFu);
                const int qb = (int)(int8_t)((ow[m >> 2] >> (8 * (m & 3))) & 0xFFu);
                out[2 * h + (m >> 2)] |= (digit_code(qa, dg) | (digit_code(qb, dg) << 4)) << (8 * (m & 3));
            }
        }
        *reinterpret_cast<uint4*>(img + n * 128 + phys * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    } else {
        const int b = t - 96;
        reinterpret_cast<float*>(img + UCOL * 128)[b] = asc[(size_t)l * (K / 16) + s * 16 + b] * gscale;
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
    float* asg_ring = reinterpret_cast<float*>(stages + STAGES * STAGE_BYTES);     // [ASG_SLOTS][16]
    float* ytmp = asg_ring + ASG_SLOTS * 16;                                       // [2][128] partial sums of the odd stages
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
        for (int m = 0; m < NMMA; m++) mbar_init(&ctl->drain[m], 1);
        mbar_init(&ctl->stored, 4);
        for (int q = 0; q < 8; q++) {
            mbar_init(&ctl->ysum[q >> 1][q & 1], 1);
            mbar_init(&ctl->yfree[q >> 1][q & 1], 1);
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // columns 12..15 of B are never written by a copy: they stay zero for the whole kernel
    for (int i = threadIdx.x; i < STAGES * (B_BYTES / 16); i += kThreads) {
        const int s = i / (B_BYTES / 16), o = i % (B_BYTES / 16);
        *reinterpret_cast<uint4*>(stages + s * STAGE_BYTES + A_BYTES + o * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == NCOPY) tmem_alloc(&ctl->tmem_base, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    if (warp >= EPI_WARP0 && warp < EPI_WARP0 + 4) {
        // scale factors of both operands: UE8M0 1.0 in every byte of 16 columns of all 128 lanes (each epilogue warp
        // writes its own lane quarter), whatever part of them an MMA reads
        const uint32_t one = 0x7F7F7F7Fu;
        asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};"
                     ::"r"(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + SF_COL), "r"(one) : "memory");
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_wait();

    if (warp < NCOPY) {
        // ================================================================ copy lanes (stage it belongs to lane it % NCOPY)
        if (lane == 0) {
            int issued = -1, it = 0;                       // `issued`: this lane's last stage with copies in flight
            for (int t = (int)blockIdx.x; t < pp.ntiles && !ctl->abort; t += G) {
                const int l = t / pp.tiles_per_layer, r0 = (t % pp.tiles_per_layer) * TM;
                const CUtensorMap* map = pp.maps + l;
                const uint8_t* img = pp.bimg + (size_t)l * nst * kImgBytes;
                bool ok = true;
                for (int s = 0; s < nst; s++, it++) {
                    if (it % NCOPY != warp) continue;
                    const int slot = it % STAGES;
                    if (it >= STAGES && !wait_or_abort(&ctl->empty[slot], ((it / STAGES) & 1) ^ 1, ctl, status, 11)) { ok = false; break; }
                    uint8_t* st = stages + slot * STAGE_BYTES;
                    mbar_expect_tx(&ctl->full[slot], A_BYTES + kImgBytes);
                    tma_2d(st, map, s * (SK / 2), r0, &ctl->full[slot]);
                    const uint8_t* im = img + (size_t)s * kImgBytes;
                    bulk_g2s(st + A_BYTES, im, UCOL * 128, &ctl->full[slot]);
                    bulk_g2s(asg_ring + (it % ASG_SLOTS) * 16, im + UCOL * 128, 64, &ctl->full[slot]);
                    issued = it;
                }
                if (!ok) break;
            }
            if (ctl->abort) {
                // leaving early: this lane's copies still in flight (its stages among the last STAGES) must land first
                for (int j = issued; j >= 0 && j > issued - STAGES; j -= NCOPY)
                    for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->full[j % STAGES], (j / STAGES) & 1); i++) {}
            }
        }
    } else if (warp < EPI_WARP0) {
        // ================================================================ MMA lanes (stage it belongs to lane it % NMMA)
        if (lane == 0) {
            const int m = warp - NCOPY;
            const uint32_t idesc = instr_desc();
            const uint64_t adesc0 = smem_desc_sw128(smem_u32(stages));
            const uint64_t bdesc0 = smem_desc_sw128(smem_u32(stages) + A_BYTES);
            for (int it = m; it < total; it += NMMA) {
                const int slot = it % STAGES, a = it % NACC;
                if (it >= NACC && !wait_or_abort(&ctl->acc_empty[a], ((it / NACC) & 1) ^ 1, ctl, status, 13)) break;
                if (!wait_or_abort(&ctl->full[slot], (it / STAGES) & 1, ctl, status, 12)) break;
                tc_fence_after();
                const uint64_t ad = adesc0 + (uint64_t)slot * (STAGE_BYTES >> 4), bd = bdesc0 + (uint64_t)slot * (STAGE_BYTES >> 4);
                const uint32_t d = tmem_base + a * ACC_COLS;
#pragma unroll
                for (int j = 0; j < 4; j++)            // 64 k = 32 bytes further along the rows of both operands
                    tc_mma_mxf4(d + j * NCOL, ad + j * 2, bd + j * 2, idesc, tmem_base + SF_COL, tmem_base + SF_COL + 4);
                tc_commit(&ctl->empty[slot]);              // the stage may be refilled once these MMAs have read it
                tc_commit(&ctl->acc_full[a]);
            }
            // nothing this lane issued may still be running when tensor memory is released
            tc_commit(&ctl->drain[m]);
            for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->drain[m], 0); i++) {}
        }
    } else {
        // ================================================================ epilogue: one thread per row of the tile
        // Two warps per TMEM lane quarter: the first takes the even stages, the second the odd ones, so a warp has two
        // stage times for the chain wait -> tcgen05.ld -> 16 blocks of arithmetic; each keeps its own partial sum of
        // the row and the second hands it over through shared memory at the end of the tile.
        const int lq = warp & 3;                            // TMEM lane quarter this warp may read
        const int ph = (warp - EPI_WARP0) >> 2;             // 0: even stages and the stores, 1: odd stages
        const int trow = lq * 32 + lane;
        const int nb = p.K / 16;                            // block scales per row
        int it = ph;                                        // this warp's next stage, counted over the whole kernel
        int flagged = 0;                                    // layers below this one have their counters bumped
        int nev = 0;                                        // completed phases of `stored`
        int ntile = 0;                                      // tiles this warp has finished
        // The E4M3 block scales of this thread's row, 16 bytes per stage, come straight from global memory through L1
        // (a row's 128-byte line serves eight stages; with L1 bypassed the same loads cost 2.6 us per layer more, and a
        // bulk L2 prefetch of the tile's scale block in front of them made nothing faster).  A load still takes longer
        // than a stage, so the scales are requested two of this warp's stages (four stages) ahead into a ring of
        // registers (the stage loop is unrolled to match: no register is moved, and a use never waits for a load
        // issued in the same stage); the ring runs across the tile boundary.
        constexpr int PF = 2;
        auto scale_row = [&](int t) -> const uint8_t* {
            const int l = t / pp.tiles_per_layer, row = (t % pp.tiles_per_layer) * TM + trow;
            return p.layers[l].ws + (size_t)(row < p.rows ? row : 0) * nb;
        };
        uint4 scr[PF];
        const uint8_t* wsr = (int)blockIdx.x < pp.ntiles ? scale_row((int)blockIdx.x) : nullptr;
        if (wsr) {
#pragma unroll
            for (int u = 0; u < PF; u++) scr[u] = __ldg(reinterpret_cast<const uint4*>(wsr + (ph + 2 * u) * 16));
        }
        for (int t = (int)blockIdx.x; t < pp.ntiles; t += G, ntile++) {
            const int l = t / pp.tiles_per_layer, row = (t % pp.tiles_per_layer) * TM + trow;
            const bool live = row < p.rows;
            const StreamLayer L = p.layers[l];
            const uint8_t* wsn = t + G < pp.ntiles ? scale_row(t + G) : wsr;      // the row of the next tile
            float y = 0.f;
            bool ok = true;
            for (int s0 = ph; s0 < nst && ok; s0 += 2 * PF) {
#pragma unroll
                for (int u = 0; u < PF; u++, it += 2) {
                    const int s = s0 + 2 * u, a = it % NACC;
                    const uint4 sc = scr[u];
                    scr[u] = __ldg(reinterpret_cast<const uint4*>(s + 2 * PF < nst ? wsr + (s + 2 * PF) * 16 : wsn + (s + 2 * PF - nst) * 16));
                    if (!wait_or_abort(&ctl->acc_full[a], (it / NACC) & 1, ctl, status, 14)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t ta = tmem_base + ((uint32_t)(lq * 32) << 16) + a * ACC_COLS;
                    uint32_t r[4][16];
#pragma unroll
                    for (int j = 0; j < 4; j++) tmem_ld16(ta + j * NCOL, r[j]);
                    const float4* ag = reinterpret_cast<const float4*>(asg_ring + (it % ASG_SLOTS) * 16);
                    float asg[16];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float4 v = ag[j];
                        asg[4 * j] = v.x; asg[4 * j + 1] = v.y; asg[4 * j + 2] = v.z; asg[4 * j + 3] = v.w;
                    }
                    tmem_ld_wait64(r);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);        // the slice is in registers
                    const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int qt = 0; qt < 4; qt++) {
                            const int b = 4 * j + qt;
                            // block sum: D0 + 7 * D1 + 49 * D2 (= I / 2), exact
                            const float tsum = fmaf(__uint_as_float(r[j][8 + qt]), 49.f,
                                                    fmaf(__uint_as_float(r[j][4 + qt]), 7.f, __uint_as_float(r[j][qt])));
                            const float sw = e4m3_raw(scw[j], qt) * 0x1p120f;
                            y = fmaf(tsum, sw * asg[b], y);
                            if (DUMP && live) p.iacc[((size_t)l * p.rows + row) * nb + s * 16 + b] = (int)(2.f * tsum);
                        }
                }
            }
            wsr = wsn;
            if (!ok) break;
            // The even and the odd stages are two pipelines of their own (own copy lane, MMA lanes, ring slots, slices of
            // tensor memory), so the two warps of a quarter can drift apart: the hand-over of the partial sums is what
            // ties them together.  Two buffers, each with a full / free barrier pair, so that every barrier is waited
            // on in consecutive phases.
            const int buf = ntile & 1;
            const uint32_t par = (ntile >> 1) & 1;
            if (ph == 1) {
                if (ntile >= 2 && !wait_or_abort(&ctl->yfree[lq][buf], par ^ 1, ctl, status, 17)) break;
                ytmp[buf * TM + trow] = y;
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->ysum[lq][buf]);
                continue;
            }
            if (!wait_or_abort(&ctl->ysum[lq][buf], par, ctl, status, 16)) break;
            y += ytmp[buf * TM + trow];
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->yfree[lq][buf]);
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
                    if (warp == EPI_WARP0) {
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
        if (p.flags && my_tiles == 0 && warp == EPI_WARP0) {
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
    if (warp == NCOPY) tmem_dealloc(tmem_base, 512);
    pdl_launch_dependents();
}

}  // namespace

// The launcher behind nvfp4_decode_stream: prepares the B images of all layers in the engine workspace, then the stream
// kernel.  Returns FM_OK after enqueueing both, a negative code after a rejection, or 1 when this path cannot take the
// launch (no tensor maps for the table, workspace cannot grow here) and the caller should use another consumer.
int nvfp4_tc_stream(const char* kn, const LaunchCtx& c, const stream::StreamParams& sp, float gscale, bool dump) {
    const int nst = sp.K / SK;
    if (sp.K % (4 * SK) || nst <= NACC || sp.M != 1 || !sp.layers) return 1;      // the epilogue unrolls the stages by four
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
    auto kern = dump ? nvfp4_tc_stream_kernel<true> : nvfp4_tc_stream_kernel<false>;
    static bool configured[2] = {false, false};
    if (!configured[dump]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured[dump] = true;
    }
    cudaError_t e = launch_kernel(nvfp4_bimg_kernel, dim3(nst, sp.nlayers), dim3(112), 0, c.stream, pdl_enabled(),
                                  reinterpret_cast<const int8_t*>(sp.ae), reinterpret_cast<const int8_t*>(sp.ao),
                                  reinterpret_cast<const float*>(sp.asc), gscale, bimg, sp.K);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    after_launch(kn);
    const int grid = c.sm_count < sp.rows ? c.sm_count : sp.rows;     // the CTA count the completion counters promise
    e = launch_kernel(kern, dim3(grid), dim3(kThreads), kSmemBytes, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

}  // namespace fm
