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
constexpr int SF_COL = 448;                   // 16 columns of scale factors, all 1
constexpr int ASG_SLOTS = 24;                 // > STAGES + NACC stages between a slot's write and its reuse
constexpr int A_BYTES = TM * SK / 2;          // one box of 128 rows x 128 bytes, packed codes
// Every role is a chain of barrier waits, and a wait costs a few hundred cycles even when the barrier is ready: one
// thread per role would hold the stream to its own pace.  So the stages go round NCOPY copy lanes and NMMA MMA lanes
// (one lane of a warp each), and round two epilogue warps per TMEM lane quarter.
constexpr int NCOPY = 2, NMMA = 4;
constexpr int EPI_WARP0 = NCOPY + NMMA;        // a multiple of 2; warp % 4 is the TMEM lane quarter a warp may read
constexpr int kThreads = (EPI_WARP0 + 8) * 32;
constexpr int kSpin = 1 << 20;
constexpr int kMaxStages = 12, kMaxAcc = 6;

// What depends on the number of tokens M (1..4): a token is 12 columns of B (3 digits x 4 quarters of an MMA's K = 64).
template <int M>
struct Geo {
    static constexpr int UCOL = 12 * M;                       // columns of B that carry data
    static constexpr int NCOL = (UCOL + 15) / 16 * 16;        // columns of one MMA
    static constexpr int B_BYTES = NCOL * 128;                // NCOL columns x 128 bytes
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int ACC_COLS = 4 * NCOL;                 // four MMAs per stage
    static constexpr int NACC = M == 1 ? 6 : 2;               // slices of tensor memory (even: a slice belongs to the even or the odd stages)
    static constexpr int STAGES = M == 1 ? 12 : M == 2 ? 10 : 8;
    // MMA lanes in use.  The barrier waits go by phase parity, which is only unambiguous while a waiter is never two
    // phases behind its barrier: a lane that takes every NMMA-th stage needs NMMA <= NACC (the slice it waits for was
    // released one phase after the one it saw last) and STAGES a multiple of NMMA and NCOPY (a slot's stages stay
    // with one lane).
    static constexpr int NMMA_USED = M == 1 ? NMMA : 2;
    static_assert(NMMA_USED <= NACC && NMMA_USED <= NMMA && STAGES % NMMA_USED == 0 && STAGES % NCOPY == 0, "lane / ring sizes");
    static constexpr int ASG = 16 * M;                        // scale products of a stage
    static constexpr int kImgBytes = UCOL * 128 + ASG * 4;    // B image of a stage, then its scale products
    static constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * STAGE_BYTES + ASG_SLOTS * ASG * 4 + 2 * M * TM * 4 + 1024;
    static_assert(kSmemBytes <= 227 * 1024, "shared memory");
    static_assert(NACC * ACC_COLS <= SF_COL, "tensor memory");
    static_assert(ASG_SLOTS > STAGES + NACC && STAGES <= kMaxStages && NACC <= kMaxAcc, "rings");
};

struct TcParams {
    StreamParams s;
    const CUtensorMap* maps;                  // [nlayers]: codes of a layer as [rows][K/2] bytes, box 128 bytes x 128 rows
    const uint8_t* bimg;                      // [nlayers][K/256][kImgBytes]: B image + scale products of a stage
    int tiles_per_layer, ntiles;
};

struct __align__(16) Control {
    uint64_t full[kMaxStages], empty[kMaxStages];
    uint64_t acc_full[kMaxAcc], acc_empty[kMaxAcc];
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

// kind::mxf4 (block-scaled): A = B = E2M1 (format 1), both K-major, N = ncol, scale factors UE8M0 (bit 23),
// M = 128, K = 64 (bit 31 clear), scale-factor byte ids 0
__device__ __forceinline__ uint32_t instr_desc(int ncol) {
    return (1u << 7) | (1u << 10) | ((uint32_t)(ncol >> 3) << 17) | (1u << 23) | ((uint32_t)(TM >> 4) << 24);
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

// B image of every stage of every layer.  grid (K/256, nlayers), 112 * M threads: thread i < 96 * M writes one 16-byte
// piece of the image, the next 16 * M one scale product each.
//   image [column n = token*12 + digit*4 + quarter][128 bytes = 256 codes, 16-byte pieces XOR-swizzled by n & 7],
//   then asg[token][16] = asc * gscale.  The codes of layer l, token k are rows l*M + k of qe / qo / asc.
template <int M>
__global__ void __launch_bounds__(112 * M)
nvfp4_bimg_kernel(const int8_t* __restrict__ qe, const int8_t* __restrict__ qo, const float* __restrict__ asc, float gscale,
                  uint8_t* __restrict__ bimg, int K) {
    using G = Geo<M>;
    pdl_wait();
    const int s = blockIdx.x, l = blockIdx.y, nst = K / SK, t = threadIdx.x;
    uint8_t* img = bimg + ((size_t)l * nst + s) * G::kImgBytes;
    if (t < 8 * G::UCOL) {
        const int n = t >> 3, phys = t & 7;
        const int c16 = phys ^ (n & 7);                    // logical 16-byte piece = 32 consecutive k = two quarters
        const int tok = n / 12, dg = (n % 12) >> 2, qt = n & 3;
        uint32_t out[4] = {0u, 0u, 0u, 0u};
        if ((qt >> 1) == (c16 & 1)) {
            const int h = qt & 1;                          // which half of the piece is this column's quarter
            const int k0 = s * SK + c16 * 32 + 16 * h;     // 16 codes from here: bytes 8h..8h+7 of the piece
            const size_t o = ((size_t)l * M + tok) * (K / 2) + k0 / 2;
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
        const int i = t - 8 * G::UCOL, tok = i >> 4, b = i & 15;
        reinterpret_cast<float*>(img + G::UCOL * 128)[i] = asc[((size_t)l * M + tok) * (K / 16) + s * 16 + b] * gscale;
    }
    pdl_launch_dependents();
}

template <int M, bool DUMP>
__global__ void __launch_bounds__(kThreads, 1)
nvfp4_tc_stream_kernel(const TcParams pp) {
    using Ge = Geo<M>;
    constexpr int STAGES = Ge::STAGES, STAGE_BYTES = Ge::STAGE_BYTES, B_BYTES = Ge::B_BYTES, NCOL = Ge::NCOL, UCOL = Ge::UCOL;
    constexpr int ACC_COLS = Ge::ACC_COLS, NACC = Ge::NACC, ASG = Ge::ASG, kImgBytes = Ge::kImgBytes;
    const StreamParams& p = pp.s;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Control* ctl = reinterpret_cast<Control*>(smem);
    uint8_t* stages = smem + 1024;
    float* asg_ring = reinterpret_cast<float*>(stages + STAGES * STAGE_BYTES);     // [ASG_SLOTS][M][16]
    float* ytmp = asg_ring + ASG_SLOTS * ASG;                                      // [2][M][128] partial sums of the odd stages
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
    // the columns of B behind the tokens' 12 each are never written by a copy: they stay zero for the whole kernel
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
                    bulk_g2s(asg_ring + (it % ASG_SLOTS) * ASG, im + UCOL * 128, ASG * 4, &ctl->full[slot]);
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
            constexpr int NL = Ge::NMMA_USED;              // lanes m >= NL have no stages
            const uint32_t idesc = instr_desc(NCOL);
            const uint64_t adesc0 = smem_desc_sw128(smem_u32(stages));
            const uint64_t bdesc0 = smem_desc_sw128(smem_u32(stages) + A_BYTES);
            for (int it = m; it < total && m < NL; it += NL) {
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
            float y[M];
#pragma unroll
            for (int k = 0; k < M; k++) y[k] = 0.f;
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
                    const float* ag = asg_ring + (it % ASG_SLOTS) * ASG;
                    const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
                    if constexpr (M == 1) {
                        uint32_t r[4][16];
#pragma unroll
                        for (int j = 0; j < 4; j++) tmem_ld16(ta + j * NCOL, r[j]);
                        float asg[16];
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float4 v = reinterpret_cast<const float4*>(ag)[j];
                            asg[4 * j] = v.x; asg[4 * j + 1] = v.y; asg[4 * j + 2] = v.z; asg[4 * j + 3] = v.w;
                        }
                        tmem_ld_wait64(r);
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);        // the slice is in registers
#pragma unroll
                        for (int j = 0; j < 4; j++)
#pragma unroll
                            for (int qt = 0; qt < 4; qt++) {
                                const int b = 4 * j + qt;
                                // block sum: D0 + 7 * D1 + 49 * D2 (= I / 2), exact
                                const float tsum = fmaf(__uint_as_float(r[j][8 + qt]), 49.f,
                                                        fmaf(__uint_as_float(r[j][4 + qt]), 7.f, __uint_as_float(r[j][qt])));
                                const float sw = e4m3_raw(scw[j], qt) * 0x1p120f;
                                y[0] = fmaf(tsum, sw * asg[b], y[0]);
                                if (DUMP && live) p.iacc[((size_t)l * p.rows + row) * nb + s * 16 + b] = (int)(2.f * tsum);
                            }
                    } else {
                        // several tokens: the slice is taken one MMA (64 k, four blocks, NCOL columns) at a time; a token's
                        // 12 digit sums are registers 12*token .. 12*token + 11 of it
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint32_t r[NCOL];
#pragma unroll
                            for (int v = 0; v < NCOL / 16; v++) tmem_ld16(ta + j * NCOL + v * 16, r + v * 16);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int v = 0; v < UCOL; v++) asm volatile("" : "+r"(r[v]) :: "memory");   // no use ahead of the wait
                            if (j == 3) {
                                tc_fence_before();
                                __syncwarp();
                                if (lane == 0) mbar_arrive(&ctl->acc_empty[a]);    // the last of the slice is in registers
                            }
                            float sw[4];
#pragma unroll
                            for (int qt = 0; qt < 4; qt++) sw[qt] = e4m3_raw(scw[j], qt) * 0x1p120f;
#pragma unroll
                            for (int k = 0; k < M; k++)
#pragma unroll
                                for (int qt = 0; qt < 4; qt++) {
                                    const int b = 4 * j + qt;
                                    const float tsum = fmaf(__uint_as_float(r[12 * k + 8 + qt]), 49.f,
                                                            fmaf(__uint_as_float(r[12 * k + 4 + qt]), 7.f, __uint_as_float(r[12 * k + qt])));
                                    y[k] = fmaf(tsum, sw[qt] * ag[k * 16 + b], y[k]);
                                    if (DUMP && live)
                                        p.iacc[(((size_t)l * M + k) * p.rows + row) * nb + s * 16 + b] = (int)(2.f * tsum);
                                }
                        }
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
#pragma unroll
                for (int k = 0; k < M; k++) ytmp[(buf * M + k) * TM + trow] = y[k];
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->ysum[lq][buf]);
                continue;
            }
            if (!wait_or_abort(&ctl->ysum[lq][buf], par, ctl, status, 16)) break;
#pragma unroll
            for (int k = 0; k < M; k++) y[k] += ytmp[(buf * M + k) * TM + trow];
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->yfree[lq][buf]);
            if (live) {
#pragma unroll
                for (int k = 0; k < M; k++) {                              // y of a layer is token-major
                    float* dst = L.y + (size_t)k * p.ystride + p.row_base + row;
                    *dst = y[k];
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if (q < p.npeers)
                            *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = y[k];
                }
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

namespace {
template <int M>
int run_tc(const char* kn, const LaunchCtx& c, const stream::StreamParams& sp, float gscale, bool dump, const void* maps) {
    using G = Geo<M>;
    const int nst = sp.K / SK;
    if (nst <= G::NACC) return 1;
    uint8_t* bimg = static_cast<uint8_t*>(engine_scratch((size_t)sp.nlayers * nst * G::kImgBytes));
    if (!bimg) return 1;
    TcParams pp = {};
    pp.s = sp;
    pp.maps = static_cast<const CUtensorMap*>(maps);
    pp.bimg = bimg;
    pp.tiles_per_layer = (sp.rows + TM - 1) / TM;
    pp.ntiles = pp.tiles_per_layer * sp.nlayers;
    auto kern = dump ? nvfp4_tc_stream_kernel<M, true> : nvfp4_tc_stream_kernel<M, false>;
    static bool configured[2] = {false, false};
    if (!configured[dump]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured[dump] = true;
    }
    cudaError_t e = launch_kernel(nvfp4_bimg_kernel<M>, dim3(nst, sp.nlayers), dim3(112 * M), 0, c.stream, pdl_enabled(),
                                  reinterpret_cast<const int8_t*>(sp.ae), reinterpret_cast<const int8_t*>(sp.ao),
                                  reinterpret_cast<const float*>(sp.asc), gscale, bimg, sp.K);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    after_launch(kn);
    const int grid = c.sm_count < sp.rows ? c.sm_count : sp.rows;     // the CTA count the completion counters promise
    e = launch_kernel(kern, dim3(grid), dim3(kThreads), G::kSmemBytes, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}
}  // namespace

// The launcher behind nvfp4_decode_stream (sp.M = 1) and nvfp4_decode_stream_m (2..4 tokens per layer): prepares the B
// images of all layers in the engine workspace, then the stream kernel.  Returns FM_OK after enqueueing both, a negative
// code after a rejection, or 1 when this path cannot take the launch (no tensor maps for the table, workspace cannot
// grow here) and the caller should use another consumer.
int nvfp4_tc_stream(const char* kn, const LaunchCtx& c, const stream::StreamParams& sp, float gscale, bool dump) {
    if (sp.K % (4 * SK) || sp.M < 1 || sp.M > 4 || !sp.layers) return 1;      // the epilogue unrolls the stages by four
    const void* maps = stream_table_maps(sp.layers, sp.nlayers, sp.rows, sp.K);
    if (!maps) return 1;
    switch (sp.M) {
        case 1: return run_tc<1>(kn, c, sp, gscale, dump, maps);
        case 2: return run_tc<2>(kn, c, sp, gscale, dump, maps);
        case 3: return run_tc<3>(kn, c, sp, gscale, dump, maps);
        default: return run_tc<4>(kn, c, sp, gscale, dump, maps);
    }
}

}  // namespace fm
