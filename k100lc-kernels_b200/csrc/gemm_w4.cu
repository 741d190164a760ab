// Prefill GEMM C[M,N] = A[M,K] . W[N,K]^T with int4 weights and int4 or int8 activations,
// one f32 scale per 128 k on both sides, on the Blackwell tensor cores (tcgen05, TMEM).
//
//   gemm_w4a4_flat, gemm_w4a4     reference kernels/gemm_core.h:59-206,
//                                 tools/gen_gemm_flat.py:36-67 (SIMT v_dot8_i32_i4 there)
//   gemm_w4a8                     no reference kernel; same contract with the int8 codes of
//                                 quant_rows_a8_k as A
//   gemm_w4a4_iacc, gemm_w4a8_iacc   the same kernel with the int32 accumulators dumped
//
// Arithmetic (reference gemm_core.h:144-188): per (m, n, 128-group g) the exact integer
//   I = sum_{k in g} a[m,k] * w[n,k]; then, g ascending,
//   C[m,n] = fmaf(float(I), sa[g*M+m] * sb[g*N+n], C[m,n])   (scale product rounded first).
//
// Mapping.  One persistent CTA per SM walks 128 x 128 output tiles (m fastest, so the CTAs
// that run together share a weight tile in L2).  Per tile and per 128-k group:
//   * two threads issue TMA copies: one the int8 activation tile (128 rows x 128 bytes, 128-byte
//     swizzle — exactly the K-major layout tcgen05.mma reads) into a 4-deep ring together with
//     the two scale vectors of the group, the other the packed weight tile (128 rows x 64 bytes,
//     64-byte swizzle) into an 8-deep ring of its own that the producers free early.  int4 activations are widened to int8 (16*v) once per call by
//     a small kernel in front, into an engine-owned workspace, so the GEMM never repeats
//     that for every column tile;
//   * four producer warps turn every weight nibble into the int8 value 16*v by masking it
//     in place in the high half of its byte ((w & 0xF0F0F0F0) for odd k,
//     ((w << 4) & 0xF0F0F0F0) for even k — the two's-complement nibble is then the byte's
//     sign and magnitude), shared memory to shared memory, into the un-swizzled core-matrix
//     layout (8 rows x 16 bytes).  Both operands use the same k order inside a word
//     (k0,k2,k4,k6,k1,k3,k5,k7); int8 activations arrive in that order from quant_rows_a8_k;
//   * two threads (even and odd steps) issue four tcgen05.mma.kind::i8 (M=128, N=128, K=32) per group
//     into one of four int32 accumulators in tensor memory (all 512 columns) and commit to an mbarrier;
//   * sixteen epilogue warps (one TMEM lane = one token row, a quarter of the columns each) drain the
//     accumulator with tcgen05.ld, convert, and fold it into 32 fp32 running sums per thread with the
//     group's scale product.  The integer in TMEM is 256*I (W4A4) or 16*I (W4A8); the
//     power of two is divided out of the scale, which leaves the fused multiply-add
//     bit-identical to fmaf(float(I), sa*sb, C).
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, the
// status word is set, all roles leave their loops, tensor memory is released and the
// kernel returns.
#include <cuda.h>          // CUtensorMap and its enums; the encoder itself is resolved at run time
#include <stdlib.h>

#include "device_utils.cuh"
#include "fm_internal.h"
#include "tc_utils.cuh"

namespace fm {
namespace {
using namespace tc;

constexpr int BM = 128, BN = 128, GK = 128;       // tile and quantisation group
constexpr int STAGES = 4;
constexpr int NACC = 4;                            // int32 accumulators in tensor memory (4 x 128 columns = all of it)
constexpr int SCALE_SLOTS = 16;                    // > 2 * NACC groups between a slot's write and its reuse
// Warps come in groups of four (the unit of setmaxnreg): four groups of epilogue warps, one group
// with the two MMA issuers and the copy lane, one group of producers.
constexpr int EPI_WARPS = 16;                      // four per TMEM lane quarter: each takes a quarter of the columns
constexpr int MMA_WARP = EPI_WARPS;                // first of the two MMA issuer warps (even / odd steps)
constexpr int TMA_WARP = EPI_WARPS + 2;            // lane 0 copies activations and scales; warp EPI_WARPS + 3 the packed weights
constexpr int PROD_WARP0 = EPI_WARPS + 4;          // first of the 4 producer warps
constexpr int kThreads = (EPI_WARPS + 4 + 4) * 32;
// 768 threads start with 80 registers each; the epilogue (32 running sums + 32 loaded integers per
// thread, and half of the scale products) takes 96, the other two groups shrink to 48: 4*128*96 + 2*128*48 =
// 61440 of 65536.  (Asking for all of the register file, 104, made setmaxnreg.inc wait forever.)
constexpr int kRegsEpilogue = 96, kRegsOther = 48;
static_assert(STAGES == NACC, "stage and accumulator share one completion barrier");
constexpr int BP_STAGES = 8;                       // ring of packed weight tiles: fetched far ahead, freed by the producers
static_assert(SCALE_SLOTS >= BP_STAGES + 2 * NACC, "scale slot reuse distance (see the weight copy lane)");
constexpr int A_BYTES = BM * GK;                   // int8 activation tile of one group, 128-byte swizzle
constexpr int BX_BYTES = BN * GK;                  // expanded int8 weight tile, core-matrix layout
constexpr int BP_BYTES = BN * GK / 2;              // packed weight tile as copied, 64-byte swizzle
constexpr int STAGE_BYTES = A_BYTES + BX_BYTES;    // what the MMA reads: freed when its MMAs have completed
constexpr int LBO = (BN / 8) * 128;                // weights: bytes between core matrices adjacent in K
constexpr int SBO = 128;                           // weights: bytes between 8-row groups
constexpr int kSpin = 1 << 17;

struct GemmParams {
    const float* sa;        // [K/128][M]
    const float* sb;        // [K/128][N]
    float* C;               // [M][N]
    int* dump;              // optional [wm1-wm0][wn1-wn0][K/128]: the integers of the window rows [wm0,wm1) x columns [wn0,wn1)
    int wm0, wm1, wn0, wn1;
    int M, N, K;
    float inv;              // 1/16 (int8 activations) or 1/256 (int4 activations widened to 16*v)
    int shift;              // log2 of the same factor, for the integer dump
};

struct __align__(16) Control {          // head of the dynamic shared memory
    uint64_t bp_full[BP_STAGES];         // weight copy lane -> producers: packed weight tile landed
    uint64_t bp_free[BP_STAGES];         // producers -> weight copy lane: packed tile is in registers
    uint64_t full[STAGES];               // -> MMA: activation tile landed (copy, byte count) and weight tile
                                         //    expanded (one arrival per producer warp)
    uint64_t drain[2];                   // MMA issuers: everything they issued has completed
    uint64_t acc_full[NACC];             // MMA -> epilogue: accumulator complete; -> copy lane: stage consumed
    uint64_t acc_empty[NACC];            // epilogue -> MMA: accumulator drained
    uint32_t tmem_base;
    volatile int abort;
};

#ifndef FM_GEMM_SPIN
#define FM_GEMM_SPIN 0
#endif
// bounded wait that also gives up when another role has raised the abort flag
__device__ __forceinline__ bool wait_or_abort(uint64_t* b, uint32_t parity, Control* ctl, int* status, int code) {
    for (int i = 0; i < kSpin; i++) {
        if (FM_GEMM_SPIN ? mbar_test_wait(b, parity) : mbar_try_wait(b, parity)) return true;
        if ((i & 63) == 63 && ctl->abort) return false;
    }
    ctl->abort = 1;
    if (status) atomicCAS(status, 0, code);
    return false;
}

// two fp32 lanes per instruction (sm_100 packed fp32): per lane identical to fmul / fmaf
__device__ __forceinline__ void mul2(float& d0, float& d1, float a, float b0, float b1) {
    asm("{\n.reg .b64 ra, rb, rd;\nmov.b64 ra, {%2,%2};\nmov.b64 rb, {%3,%4};\nmul.rn.f32x2 rd, ra, rb;\nmov.b64 {%0,%1}, rd;\n}"
        : "=f"(d0), "=f"(d1) : "f"(a), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fma2(float& c0, float& c1, float a0, float a1, float b0, float b1) {
    asm("{\n.reg .b64 ra, rb, rc;\nmov.b64 ra, {%2,%3};\nmov.b64 rb, {%4,%5};\nmov.b64 rc, {%0,%1};\n"
        "fma.rn.f32x2 rc, ra, rb, rc;\nmov.b64 {%0,%1}, rc;\n}"
        : "+f"(c0), "+f"(c1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

// Weights: K-major, no swizzle: start address, LBO (next core matrix in K), SBO (next 8-row group)
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)((LBO >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((SBO >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;                       // descriptor version of sm_100
    return d;                                     // layout type 0 (no swizzle), base offset 0
}
// kind::i8, signed x signed -> s32, both operands K-major, M = 128, N = 128
__device__ __forceinline__ uint32_t instr_desc() {
    uint32_t d = 0;
    d |= 2u << 4;                                 // D format: s32
    d |= 1u << 7;                                 // A format: s8
    d |= 1u << 10;                                // B format: s8
    d |= (uint32_t)(BN >> 3) << 17;               // N
    d |= (uint32_t)(BM >> 4) << 24;               // M
    return d;
}

// 0 while every bounded wait of the GEMM kernels has been satisfied; otherwise the code of
// the first one that ran out (1 stage not free, 2 weights not expanded, 3 accumulator not drained,
// 4 accumulator not complete, 6 packed weights and scales not landed, 7 expanded tile
// not free, 8 packed tile not free).  Read and cleared by fm_gemm_status().
__device__ int g_gemm_status;

__device__ __forceinline__ uint32_t even16(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }   // 16*v of k0,k2,k4,k6
__device__ __forceinline__ uint32_t odd16(uint32_t w) { return w & 0xF0F0F0F0u; }           // 16*v of k1,k3,k5,k7

// Position of a role in its sequence of (tile, group) steps.  The divisions that turn a tile
// index into coordinates run once per tile; per group only the counter moves (each role's loop
// is a serial chain of dependent instructions, so per-step index arithmetic is on the critical path).
struct Cursor {
    int g, m0, n0, t;
    __device__ __forceinline__ void set_tile(int tile, int tiles_m) {
        t = tile;
        m0 = (tile % tiles_m) * BM;
        n0 = (tile / tiles_m) * BN;
    }
    __device__ __forceinline__ void next(int G, int tiles_m, int stride) {
        if (++g == G) {
            g = 0;
            set_tile(t + stride, tiles_m);
        }
    }
};

// int4 activations [M][K/8] packed words -> int8 16*v in the word-internal order k0,k2,k4,k6,k1,k3,k5,k7
__global__ void __launch_bounds__(256)
expand_a4_kernel(const uint4* __restrict__ aq, uint4* __restrict__ out, size_t n16) {
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 w = aq[i];
        out[2 * i] = make_uint4(even16(w.x), odd16(w.x), even16(w.y), odd16(w.y));
        out[2 * i + 1] = make_uint4(even16(w.z), odd16(w.z), even16(w.w), odd16(w.w));
    }
    pdl_launch_dependents();
}

// tmA: int8 activations [M][K], box 128 bytes x 128 rows, 128-byte swizzle.
// tmB: packed weights [N][K/2] bytes, box 64 bytes x 128 rows, 64-byte swizzle (rows past N read as 0).
// DUMP: also store the integers.  (The epilogue's multiplies and fused multiply-adds are the packed two-lane forms:
// the same arithmetic as one-lane instructions measured 0.398 ms against 0.361 ms at M = 2048.)
template <bool DUMP>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // the swizzled tiles need a 1024-byte aligned base whatever the offset of the dynamic window is
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    Control* ctl = reinterpret_cast<Control*>(smem);
    uint8_t* stages = smem + 1024;                                   // STAGES x (A, expanded W)
    uint8_t* bp_ring = stages + STAGES * STAGE_BYTES;                // BP_STAGES x packed W
    float* sc_ring = reinterpret_cast<float*>(bp_ring + BP_STAGES * BP_BYTES);   // [SLOTS][2][128]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.K / GK;
    const int tiles_m = p.M / BM, tiles_n = (p.N + BN - 1) / BN;
    const int ntiles = tiles_m * tiles_n;
    const int my_tiles = ((int)blockIdx.x < ntiles) ? (ntiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total = my_tiles * G;                                  // (tile, group) steps of this CTA
    int* status = &g_gemm_status;

    if (threadIdx.x == 0) {
        // one arrival per WARP on the software barriers (hundreds of per-thread arrivals on one
        // barrier word would serialise)
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&ctl->full[s], 5);
        }
        for (int s = 0; s < BP_STAGES; s++) {
            mbar_init(&ctl->bp_full[s], 1);
            mbar_init(&ctl->bp_free[s], 4);
        }
        mbar_init(&ctl->drain[0], 1);
        mbar_init(&ctl->drain[1], 1);
        for (int b = 0; b < NACC; b++) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], EPI_WARPS);
        }
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&ctl->tmem_base, NACC * BN);    // NACC 128-column int32 accumulators
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    pdl_wait();

    // Every group of four warps begins by resizing its register file; all four warps of a group run the
    // same setmaxnreg instruction before they split into their roles.
    if (warp >= PROD_WARP0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        // ================================================================ producers
        // lane -> (q: which 16 packed bytes = 32 k of the row, rr: row inside an 8-row group); warp pw takes
        // the 8-row groups pw, pw + 4, pw + 8, pw + 12
        const int pw = warp - PROD_WARP0, q = lane >> 3, rr = lane & 7;
        for (int it = 0; it < total; it++) {
            const int s = it % STAGES, sp = it % BP_STAGES;
            if (!wait_or_abort(&ctl->bp_full[sp], (it / BP_STAGES) & 1, ctl, status, 6)) break;
            uint8_t* Bx = stages + s * STAGE_BYTES + A_BYTES;
            const uint8_t* Bp = bp_ring + sp * BP_BYTES;
            uint4 w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = (i * 4 + pw) * 8 + rr;               // 64-byte swizzle: chunk ^= (row / 2) % 4
                w[i] = *reinterpret_cast<const uint4*>(Bp + row * 64 + ((q ^ ((row >> 1) & 3)) << 4));
            }
            // the expanded tile of stage s was read by the MMAs of step it - STAGES
            if (it >= STAGES && !wait_or_abort(&ctl->acc_full[s], ((it / STAGES) & 1) ^ 1, ctl, status, 7)) break;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                uint8_t* dst = Bx + (2 * q) * LBO + (i * 4 + pw) * SBO + rr * 16;
                *reinterpret_cast<uint4*>(dst) = make_uint4(even16(w[i].x), odd16(w[i].x), even16(w[i].y), odd16(w[i].y));
                *reinterpret_cast<uint4*>(dst + LBO) = make_uint4(even16(w[i].z), odd16(w[i].z), even16(w[i].w), odd16(w[i].w));
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->full[s]);
                mbar_arrive(&ctl->bp_free[sp]);                      // the packed tile may be refilled
            }
        }
    } else if (warp >= EPI_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsOther));
        if (warp == TMA_WARP) {
            // ================================================================ copy lane
            if (lane == 0) {
                Cursor ld;
                ld.g = 0;
                ld.set_tile((int)blockIdx.x, tiles_m);
                int issued = 0;
                for (int it = 0; it < total; it++, ld.next(G, tiles_m, (int)gridDim.x)) {
                    const int s = it % STAGES;
                    // stage s was read by the MMAs of step it - STAGES
                    if (it >= STAGES && !wait_or_abort(&ctl->acc_full[s], ((it / STAGES) & 1) ^ 1, ctl, status, 1)) break;
                    uint8_t* st = stages + s * STAGE_BYTES;
                    mbar_expect_tx(&ctl->full[s], A_BYTES);
                    tma_2d(st, &tmA, ld.g * GK, ld.m0, &ctl->full[s]);
                    issued = it + 1;
                }
                if (ctl->abort) {
                    // leaving early: the copies already issued must have landed before the CTA's shared
                    // memory is given up (bounded like every other wait; nothing is reported twice)
                    for (int j = issued > STAGES ? issued - STAGES : 0; j < issued; j++) {
                        for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->full[j % STAGES], (j / STAGES) & 1); i++) {}
                    }
                }
            }
        } else if (warp == TMA_WARP + 1) {
            // ================================================================ weight copy lane
            // the packed weight tiles run up to BP_STAGES steps ahead of the producers, so their trip
            // from L2 is off the critical path
            if (lane == 0) {
                Cursor ld;
                ld.g = 0;
                ld.set_tile((int)blockIdx.x, tiles_m);
                int issued = 0;
                for (int it = 0; it < total; it++, ld.next(G, tiles_m, (int)gridDim.x)) {
                    const int sp = it % BP_STAGES;
                    if (it >= BP_STAGES && !wait_or_abort(&ctl->bp_free[sp], ((it / BP_STAGES) & 1) ^ 1, ctl, status, 8)) break;
                    const uint32_t nb = (uint32_t)min(BN, p.N - ld.n0) * 4u;
                    mbar_expect_tx(&ctl->bp_full[sp], BP_BYTES + BM * 4 + nb);
                    tma_2d(bp_ring + sp * BP_BYTES, &tmB, ld.g * (GK / 2), ld.n0, &ctl->bp_full[sp]);
                    // The scales of the step travel with it.  Slot it % 16 was last used by step it - 16: the
                    // producers have finished step it - 8 (bp_free), for which they waited for the MMAs of step
                    // it - 12, which were issued after the epilogue had drained step it - 16.
                    // They complete on the packed tile's barrier: the producers wait for it, the MMAs wait for
                    // the producers and the epilogue waits for the MMAs.
                    float* sc = sc_ring + (it % SCALE_SLOTS) * 256;
                    bulk_g2s(sc, p.sa + (size_t)ld.g * p.M + ld.m0, BM * 4, &ctl->bp_full[sp]);
                    bulk_g2s(sc + 128, p.sb + (size_t)ld.g * p.N + ld.n0, nb, &ctl->bp_full[sp]);
                    issued = it + 1;
                }
                if (ctl->abort) {
                    for (int j = issued > BP_STAGES ? issued - BP_STAGES : 0; j < issued; j++)
                        for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->bp_full[j % BP_STAGES], (j / BP_STAGES) & 1); i++) {}
                }
            }
        } else if (warp < TMA_WARP) {
            // ================================================================ MMA issuers
            // Two threads, one for the even and one for the odd steps: a step is two barrier waits (each a
            // few hundred cycles of latency even when the barrier is ready) around 256 cycles of MMA, so
            // one thread alone would keep the tensor pipe idle three quarters of the time.  Steps use
            // distinct stages and accumulators, and every thread commits its own MMAs.
            if (lane == 0) {
                const int par = warp - MMA_WARP;
                // everything that does not depend on the step is computed once: this single thread is
                // on the critical path of every group, so its loop body is kept to a few instructions
                const uint32_t idesc = instr_desc();
                const uint64_t adesc0 = smem_desc_sw128(smem_u32(stages));
                const uint64_t bdesc0 = smem_desc(smem_u32(stages) + A_BYTES);
                constexpr uint64_t kStageStep = STAGE_BYTES >> 4;        // descriptor units of 16 bytes
                constexpr uint64_t kAStep = 32 >> 4, kBStep = (2 * LBO) >> 4;   // 32 k further along the row
                for (int it = par; it < total; it += 2) {
                    const int s = it % STAGES;                  // == accumulator index (STAGES == NACC)
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it >= NACC && !wait_or_abort(&ctl->acc_empty[s], ph ^ 1, ctl, status, 3)) break;
                    if (!wait_or_abort(&ctl->full[s], ph, ctl, status, 2)) break;
                    tc_fence_after();
                    const uint64_t ad = adesc0 + s * kStageStep, bd = bdesc0 + s * kStageStep;
                    const uint32_t d = tmem_base + s * BN;
                    tc_mma_i8(d, ad, bd, idesc, 0);
                    tc_mma_i8(d, ad + kAStep, bd + kBStep, idesc, 1);
                    tc_mma_i8(d, ad + 2 * kAStep, bd + 2 * kBStep, idesc, 1);
                    tc_mma_i8(d, ad + 3 * kAStep, bd + 3 * kBStep, idesc, 1);
                    // one commit per group: STAGES == NACC, so one barrier tells the copy lane "stage
                    // consumed" and the epilogue "accumulator complete"
                    tc_commit(&ctl->acc_full[s]);
                }
                // nothing this thread issued may still be running when tensor memory is released (the
                // epilogue has consumed every step unless the kernel is aborting)
                tc_commit(&ctl->drain[par]);
                for (int i = 0; i < kSpin && !mbar_try_wait(&ctl->drain[par], 0); i++) {}
            }
        }
    } else {
        // ================================================================ epilogue
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
        // warp w drains TMEM lanes 32*(w%4).. (a hardware rule) and columns 32*(w/4)..+31
        constexpr int CPW = BN / (EPI_WARPS / 4);                    // columns per warp: 32
        const int lq = warp & 3, ch = warp >> 2;
        const int mrow = lq * 32 + lane;                             // TMEM lane = row of the tile
        const float inv = p.inv;                                     // the integer in TMEM is 16*I or 256*I
        float facc[CPW];
#pragma unroll
        for (int j = 0; j < CPW; j++) facc[j] = 0.f;
        Cursor cur;
        cur.g = 0;
        cur.set_tile((int)blockIdx.x, tiles_m);
        for (int it = 0; it < total; it++, cur.next(G, tiles_m, (int)gridDim.x)) {
            const int b = it % NACC, slot = it % SCALE_SLOTS, g = cur.g;
            const int m0 = cur.m0, n0 = cur.n0 + ch * CPW;
            if (!wait_or_abort(&ctl->acc_full[b], (it / NACC) & 1, ctl, status, 4)) break;
            tc_fence_after();
            // (the scales landed with the packed weight tile, before the producers expanded it for these MMAs)
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(lq * 32) << 16) + b * BN + ch * CPW, r);
            // while the accumulator is on its way: the scale products, rounded to fp32 first
            const float sa = sc_ring[slot * 256 + mrow] * inv;
            const float* sbv = sc_ring + slot * 256 + 128 + ch * CPW;
            constexpr int PRE = CPW / 2;                            // products computed ahead (register budget)
            float sc[PRE];
#pragma unroll
            for (int j = 0; j < PRE; j += 4) {
                const float4 sb4 = *reinterpret_cast<const float4*>(sbv + j);   // one broadcast load for four columns
                mul2(sc[j], sc[j + 1], sa, sb4.x, sb4.y);
                mul2(sc[j + 2], sc[j + 3], sa, sb4.z, sb4.w);
            }
            tmem_ld_wait(r);
#pragma unroll
            for (int j = 0; j < CPW; j += 4) {
                float s0, s1, s2, s3;
                if (j < PRE) {
                    s0 = sc[j]; s1 = sc[j + 1]; s2 = sc[j + 2]; s3 = sc[j + 3];
                } else {
                    const float4 sb4 = *reinterpret_cast<const float4*>(sbv + j);
                    mul2(s0, s1, sa, sb4.x, sb4.y);
                    mul2(s2, s3, sa, sb4.z, sb4.w);
                }
                // (a magic-number conversion on the FMA pipe was measured slower: the epilogue is bound by
                //  issue slots, and the conversion unit is otherwise idle)
                const float f0 = (float)(int)r[j], f1 = (float)(int)r[j + 1];
                const float f2 = (float)(int)r[j + 2], f3 = (float)(int)r[j + 3];
                fma2(facc[j], facc[j + 1], f0, f1, s0, s1);
                fma2(facc[j + 2], facc[j + 3], f2, f3, s2, s3);
                if (DUMP) {
                    const int mm = m0 + mrow;
                    if (mm >= p.wm0 && mm < p.wm1) {
#pragma unroll
                        for (int u = 0; u < 4; u++) {
                            const int nn = n0 + j + u;
                            if (nn >= p.wn0 && nn < p.wn1)
                                p.dump[((size_t)(mm - p.wm0) * (p.wn1 - p.wn0) + (nn - p.wn0)) * G + g] = (int)r[j + u] >> p.shift;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
            if (g == G - 1) {                                        // tile finished: write C and clear
                float* crow = p.C + (size_t)(m0 + mrow) * p.N + n0;
                if (n0 + CPW <= p.N) {
#pragma unroll
                    for (int j = 0; j < CPW; j += 4)
                        *reinterpret_cast<float4*>(crow + j) = make_float4(facc[j], facc[j + 1], facc[j + 2], facc[j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < CPW; j++)
                        if (n0 + j < p.N) crow[j] = facc[j];
                }
#pragma unroll
                for (int j = 0; j < CPW; j++) facc[j] = 0.f;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, NACC * BN);
    pdl_launch_dependents();
}

// mma_i8_peak: the rate at which the tensor cores complete tcgen05.mma.kind::i8 (M=128, N=128, K=32, the shape the
// GEMM issues) when nothing else limits them — operands already in shared memory (zeros), one thread per CTA issuing
// `iters` MMAs back to back into two alternating accumulators, one commit, one bounded wait.  The denominator of the
// GEMM's tensor roofline, measured on the device the GEMM runs on.
__global__ void __launch_bounds__(128, 1)
mma_i8_peak_kernel(int iters, long long* cycles, int* status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ uint64_t bar;
    __shared__ uint32_t tbase;
    for (int i = threadIdx.x; i < 2 * BX_BYTES / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) tmem_alloc(&tbase, 2 * BN);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) {
        const uint32_t idesc = instr_desc();
        const uint64_t ad = smem_desc(smem_u32(smem)), bd = smem_desc(smem_u32(smem) + BX_BYTES);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i++) tc_mma_i8(tbase + (i & 1) * BN, ad, bd, idesc, 1);
        tc_commit(&bar);
        bool ok = false;
        for (int i = 0; i < (1 << 24) && !ok; i++) ok = mbar_try_wait(&bar, 0);
        const long long t1 = clock64();
        if (!ok) atomicCAS(status, 0, 9);
        if (cycles) cycles[blockIdx.x] = t1 - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tbase, 2 * BN);
}

// mma_i8_peak(cycles, iters): one CTA per SM; cycles = device int64 [SM count] (or 0): clocks from the first issue to
// the completion of the last MMA on each SM.  2 * 128 * 128 * 32 * iters integer operations per CTA.
int launch_mma_peak(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "mma_i8_peak";
    long long* cycles = arg_ptr<long long>(a[0]);
    const int iters = arg_i32(a[1]);
    FM_REQUIRE(iters > 0 && iters <= (1 << 20), kn, "iters=%d must be 1..1048576", iters);
    if (cycles) {
        FM_REQUIRE(aligned(cycles, 8), kn, "misaligned cycle array");
        FM_RANGE(cycles, (size_t)c.sm_count * 8, kn, "cycles");
    }
    constexpr size_t smem = 2 * BX_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(mma_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int* status = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&status), g_gemm_status) != cudaSuccess) return cuda_fail(kn, cudaGetLastError());
    cudaError_t e = launch_kernel(mma_i8_peak_kernel, dim3(c.sm_count), dim3(128), smem, c.stream, false, iters, cycles, status);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// ------------------------------------------------------------------------- host side
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * STAGE_BYTES + (size_t)BP_STAGES * BP_BYTES + SCALE_SLOTS * 256 * 4 + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory");

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// the driver's tensor-map encoder, looked up through the runtime (no link against the driver library)
EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}
// bytes [rows][row_bytes], row-major and dense; box = box_bytes x 128 rows
bool make_map(CUtensorMap* m, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes, CUtensorMapSwizzle sw,
              CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {box_bytes, 128};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, sw, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// aq: packed int4 [M][K/8] words (A8 false) or int8 [M][K] (A8 true)
template <bool A8, bool DUMP>
int run_gemm(const char* kn, const LaunchCtx& c, const GemmParams& p, const void* aq, const void* wq) {
    auto kern = gemm_w4_kernel<DUMP>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    const void* a8 = aq;
    if (!A8) {                                       // widen the int4 codes once, in front of the GEMM
        const size_t bytes = (size_t)p.M * p.K;
        void* ws = engine_scratch(bytes);
        FM_REQUIRE(ws != nullptr, kn,
                   "the %zu-byte workspace for the widened activations cannot be allocated here (inside a graph "
                   "capture it must exist already: run this shape once outside the capture)", bytes);
        const size_t n16 = bytes / 32;
        const int blocks = (int)((n16 + 255) / 256 < (size_t)c.sm_count * 8 ? (n16 + 255) / 256 : (size_t)c.sm_count * 8);
        cudaError_t e = launch_kernel(expand_a4_kernel, dim3(blocks), dim3(256), 0, c.stream, pdl_enabled(),
                                      static_cast<const uint4*>(aq), static_cast<uint4*>(ws), n16);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        after_launch(kn);
        a8 = ws;
    }
    CUtensorMap tmA, tmB;
    FM_REQUIRE(make_map(&tmA, a8, p.M, p.K, 128, CU_TENSOR_MAP_SWIZZLE_128B) &&
               make_map(&tmB, wq, p.N, p.K / 2, 64, CU_TENSOR_MAP_SWIZZLE_64B), kn,
               "cuTensorMapEncodeTiled is unavailable or refused M=%d N=%d K=%d", p.M, p.N, p.K);
    const int ntiles = (p.M / BM) * ((p.N + BN - 1) / BN);
    const int grid = ntiles < c.sm_count ? ntiles : c.sm_count;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(kThreads), kSmemBytes, c.stream, pdl_enabled(), tmA, tmB, p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

struct GemmArgs {                                   // the by-name arguments before they are split up
    const uint32_t* aq;
    const uint32_t* wq;
    GemmParams p;
};

// shared checks; tiles_needed = number of reference work-groups (128 x 64 tiles) the grid must cover
template <bool A8>
int check_gemm(const char* kn, const LaunchCtx& c, GemmArgs& ga, long long groups_given, bool dump) {
    GemmParams& p = ga.p;
    FM_REQUIRE(c.wx == 256 && c.wy == 1, kn, "work-group must be 256 threads (got %ux%u)", c.wx, c.wy);
    FM_REQUIRE(p.M > 0 && p.N > 0 && p.K > 0 && p.M % 128 == 0 && p.N % 64 == 0 && p.K % 128 == 0, kn,
               "M=%d N=%d K=%d: M must be a multiple of 128, N of 64, K of 128", p.M, p.N, p.K);
    const long long need = (long long)(p.N / 64) * (p.M / 128);
    FM_REQUIRE(groups_given >= need, kn, "the grid covers %lld of the %lld 128x64 tiles; partial grids are not built",
               groups_given, need);
    FM_REQUIRE(aligned(ga.aq, 16) && aligned(ga.wq, 16) && aligned(p.sa, 16) && aligned(p.sb, 16) && aligned(p.C, 16), kn,
               "misaligned pointer (codes, scales and C need 16 bytes)");
    const int G = p.K / 128;
    FM_RANGE(ga.aq, A8 ? (size_t)p.M * p.K : (size_t)p.M * (p.K / 2), kn, "aq");
    FM_RANGE(ga.wq, (size_t)p.N * (p.K / 2), kn, "wq");
    p.inv = A8 ? (1.0f / 16.0f) : (1.0f / 256.0f);
    p.shift = A8 ? 4 : 8;
    FM_RANGE(p.sa, (size_t)G * p.M * 4, kn, "asc");
    FM_RANGE(p.sb, (size_t)G * p.N * 4, kn, "wsc");
    FM_RANGE(p.C, (size_t)p.M * p.N * 4, kn, "C");
    if (dump) {
        FM_REQUIRE(aligned(p.dump, 4), kn, "misaligned accumulator dump");
        FM_REQUIRE(0 <= p.wm0 && p.wm0 < p.wm1 && p.wm1 <= p.M && 0 <= p.wn0 && p.wn0 < p.wn1 && p.wn1 <= p.N, kn,
                   "dump window rows [%d,%d) x columns [%d,%d) is empty or outside M=%d N=%d", p.wm0, p.wm1, p.wn0, p.wn1, p.M, p.N);
        FM_RANGE(p.dump, (size_t)(p.wm1 - p.wm0) * (p.wn1 - p.wn0) * G * 4, kn, "iacc");
    }
    return FM_OK;
}

void fill(GemmArgs& ga, const uint64_t* a) {
    GemmParams& p = ga.p;
    ga.aq = arg_ptr<const uint32_t>(a[0]);
    ga.wq = arg_ptr<const uint32_t>(a[1]);
    p.sa = arg_ptr<const float>(a[2]);
    p.sb = arg_ptr<const float>(a[3]);
    p.C = arg_ptr<float>(a[4]);
    p.M = arg_i32(a[5]);
    p.N = arg_i32(a[6]);
    p.K = arg_i32(a[7]);
}

// gemm_w4a4_flat(aq, wq, asc, wsc, C, M, N, K, nbn, magic): 1-D grid of nbn * M/128 work-groups;
// nbn must be N/64; the magic multiplier is accepted and ignored.
int launch_gemm_flat(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gemm_w4a4_flat";
    GemmArgs ga = {};
    GemmParams& p = ga.p;
    fill(ga, a);
    FM_REQUIRE(c.gy == 1, kn, "1-D grid expected");
    FM_REQUIRE(p.N > 0 && arg_i32(a[8]) == p.N / 64, kn, "nbn=%d must equal N/64=%d", arg_i32(a[8]), p.N / 64);
    const int rc = check_gemm<false>(kn, c, ga, c.gx, false);
    return rc ? rc : run_gemm<false, false>(kn, c, p, ga.aq, ga.wq);
}

// gemm_w4a4(aq, wq, asc, wsc, C, M, N, K): grid x = N/64, grid y = M/128 (a 1-D launch covers M = 128)
int launch_gemm_2d(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gemm_w4a4";
    GemmArgs ga = {};
    GemmParams& p = ga.p;
    fill(ga, a);
    FM_REQUIRE(p.N > 0 && p.M > 0 && (long long)c.gx >= p.N / 64 && (long long)c.gy >= p.M / 128, kn,
               "grid %ux%u does not cover N/64=%d by M/128=%d work-groups", c.gx, c.gy, p.N / 64, p.M / 128);
    const int rc = check_gemm<false>(kn, c, ga, (long long)(p.N / 64) * (p.M / 128), false);
    return rc ? rc : run_gemm<false, false>(kn, c, p, ga.aq, ga.wq);
}

// gemm_w4a8(aq8, wq, asc, wsc, C, M, N, K): aq8 = int8 codes of quant_rows_a8_k; 1-D grid of N/64 * M/128
int launch_gemm_a8(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gemm_w4a8";
    GemmArgs ga = {};
    GemmParams& p = ga.p;
    fill(ga, a);
    FM_REQUIRE(c.gy == 1, kn, "1-D grid expected");
    const int rc = check_gemm<true>(kn, c, ga, c.gx, false);
    return rc ? rc : run_gemm<true, false>(kn, c, p, ga.aq, ga.wq);
}

// gemm_w4a4_iacc / gemm_w4a8_iacc (aq, wq, asc, wsc, C, M, N, K, iacc): iacc int32 [M][N][K/128]
// gemm_w4a4_iacc_win / gemm_w4a8_iacc_win (..., iacc, m0, m1, n0, n1): the whole GEMM runs, the integers of the
// window rows [m0,m1) x columns [n0,n1) go to iacc int32 [m1-m0][n1-n0][K/128] (the full dump of the
// M=2048 x N=17408 shape would be 5.7 GB)
template <bool A8, bool WIN>
int launch_gemm_iacc(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = A8 ? (WIN ? "gemm_w4a8_iacc_win" : "gemm_w4a8_iacc") : (WIN ? "gemm_w4a4_iacc_win" : "gemm_w4a4_iacc");
    GemmArgs ga = {};
    GemmParams& p = ga.p;
    fill(ga, a);
    p.dump = arg_ptr<int>(a[8]);
    p.wm0 = WIN ? arg_i32(a[9]) : 0;
    p.wm1 = WIN ? arg_i32(a[10]) : p.M;
    p.wn0 = WIN ? arg_i32(a[11]) : 0;
    p.wn1 = WIN ? arg_i32(a[12]) : p.N;
    const int rc = check_gemm<A8>(kn, c, ga, 1LL << 40, true);
    return rc ? rc : run_gemm<A8, true>(kn, c, p, ga.aq, ga.wq);
}

const KernelEntry kGemm[] = {
    {"gemm_w4a4_flat", 10, launch_gemm_flat, "pppppiiiii"},
    {"gemm_w4a4", 8, launch_gemm_2d, "pppppiii"},
    {"gemm_w4a8", 8, launch_gemm_a8, "pppppiii"},
    {"gemm_w4a4_iacc", 9, launch_gemm_iacc<false, false>, "pppppiiip"},
    {"gemm_w4a8_iacc", 9, launch_gemm_iacc<true, false>, "pppppiiip"},
    {"mma_i8_peak", 2, launch_mma_peak, "pi"},
    {"gemm_w4a4_iacc_win", 13, launch_gemm_iacc<false, true>, "pppppiiipiiii"},
    {"gemm_w4a8_iacc_win", 13, launch_gemm_iacc<true, true>, "pppppiiipiiii"},
};

}  // namespace

const KernelEntry* gemm_w4_kernels(int* n) {
    *n = (int)(sizeof(kGemm) / sizeof(kGemm[0]));
    return kGemm;
}

// Maps for a 5120-k chunk of 16 rows of a packed weight matrix whose rows are longer than the chunk (and of their
// group scales): the weight map sees a row as pieces of 512 bytes, so that a box of (512 bytes, 5 pieces, 16 rows) lands
// as 16 contiguous rows of 2560 bytes; the scale map is [rows][spitch bytes] with a box of 80 bytes x 16 rows.  Pieces
// and bytes past the end of a row read as zero.
bool encode_chunk_maps(void* wmap128, void* smap128, const void* wbase, const void* sbase, uint64_t rows, uint64_t wpitch,
                       uint64_t spitch) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (!enc || wpitch % 512 || spitch % 16) return false;
    const cuuint64_t wd[3] = {128, wpitch / 512, rows};
    const cuuint64_t ws[2] = {512, wpitch};
    const cuuint32_t wb[3] = {128, 5, 16}, e3[3] = {1, 1, 1};
    if (enc(static_cast<CUtensorMap*>(wmap128), CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(wbase), wd, ws, wb, e3,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    const cuuint64_t sd[2] = {spitch / 4, rows};
    const cuuint64_t ss[1] = {spitch};
    const cuuint32_t sb[2] = {20, 16}, e2[2] = {1, 1};
    return enc(static_cast<CUtensorMap*>(smap128), CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(sbase), sd, ss, sb, e2,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
bool encode_bytes_rows_map(void* map128, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_bytes) {
    // (256-byte L2 promotion: the next stage's 128 bytes of a row come along; 1 % over 128 bytes or none)
    return make_map(static_cast<CUtensorMap*>(map128), base, rows, row_bytes, box_bytes,
                    box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}
// status word of the GEMM kernels: drains the stream, reads it and clears it
int gemm_read_status(cudaStream_t stream) {
    int v = 0, zero = 0;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    return v;
}

}  // namespace fm
