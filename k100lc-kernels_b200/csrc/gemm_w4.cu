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
// that run together share a weight tile in L2).  Per tile and per group:
//   * four producer warps read the packed rows of A and W for this group (64 B per row),
//     turn every nibble into the int8 value 16*v by masking it in place in the high half
//     of its byte ((w & 0xF0F0F0F0) for odd k, ((w << 4) & 0xF0F0F0F0) for even k — the
//     two's-complement nibble is then the byte's sign and magnitude), and store the bytes
//     in the K-major core-matrix layout tcgen05.mma reads (8 rows x 16 bytes per core
//     matrix, no swizzle).  Both operands use the same k order inside a word
//     (k0,k2,k4,k6,k1,k3,k5,k7); int8 activations arrive in that order from
//     quant_rows_a8_k and are copied.  A 4-deep ring of such stages feeds the tensor core;
//   * one thread issues four tcgen05.mma.kind::i8 (M=128, N=128, K=32) per group into one
//     of four int32 accumulators in tensor memory (all 512 columns) and commits to an mbarrier;
//   * eight epilogue warps (one TMEM lane = one token row, half of the columns each) drain the
//     accumulator with tcgen05.ld, convert, and fold it into 64 fp32 running sums per thread with the
//     group's scale product.  The integer in TMEM is 256*I (W4A4) or 16*I (W4A8); the
//     power of two is divided out of the scale, which leaves the fused multiply-add
//     bit-identical to fmaf(float(I), sa*sb, C).
// Every mbarrier wait is bounded; a wait that runs out raises a CTA-wide abort flag, the
// status word is set, all roles leave their loops, tensor memory is released and the
// kernel returns.
#include <stdlib.h>

#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int BM = 128, BN = 128, GK = 128;       // tile and quantisation group
constexpr int STAGES = 4;
constexpr int NACC = 4;                            // int32 accumulators in tensor memory (4 x 128 columns = all of it)
constexpr int SCALE_SLOTS = 16;                    // > STAGES + NACC groups in flight
constexpr int EPI_WARPS = 8;                       // two per TMEM lane quarter: each takes half of the columns
constexpr int MMA_WARP = EPI_WARPS;                // warp index of the MMA issuer
constexpr int PROD_WARP0 = EPI_WARPS + 1;          // first of the 4 producer warps
constexpr int kThreads = (EPI_WARPS + 1 + 4) * 32;
static_assert(STAGES == NACC, "stage and accumulator share one completion barrier");
constexpr int TILE_BYTES = BM * GK;                // one int8 operand tile of one group: 16 KB
constexpr int STAGE_BYTES = 2 * TILE_BYTES;
constexpr int LBO = (BM / 8) * 128;                // bytes between core matrices adjacent in K
constexpr int SBO = 128;                           // bytes between 8-row groups
constexpr int kSpin = 1 << 17;

struct GemmParams {
    const uint32_t* aq;     // A4: [M][K/8] packed nibbles; A8: [M][K] int8, 8-permuted
    const uint32_t* wq;     // [N][K/8] packed nibbles
    const float* sa;        // [K/128][M]
    const float* sb;        // [K/128][N]
    float* C;               // [M][N]
    int* dump;              // optional [M][N][K/128]
    int M, N, K;
};

struct __align__(16) Control {          // head of the dynamic shared memory
    uint64_t full[STAGES];               // producers -> MMA: stage written
    uint64_t acc_full[NACC];             // MMA -> epilogue: accumulator complete; -> producers: stage consumed
    uint64_t acc_empty[NACC];            // epilogue -> MMA: accumulator drained
    uint64_t sc_full[SCALE_SLOTS];       // producers -> epilogue: scales of a group written
    uint32_t tmem_base;
    volatile int abort;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
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

// ---- tcgen05 wrappers ---------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 columns of 32-bit: thread t of the warp gets lane t, columns c..c+31
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
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

// K-major, no swizzle: start address, LBO (next core matrix in K), SBO (next 8-row group)
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
// the first one that ran out (1 stage not free, 2 stage not full, 3 accumulator not drained,
// 4 accumulator not complete, 5 scales not written).  Read and cleared by fm_gemm_status().
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

// A8: activations are int8 (quant_rows_a8_k) instead of packed int4.  DUMP: store the integers.
template <bool A8, bool DUMP>
__global__ void __launch_bounds__(kThreads, 1)
gemm_w4_kernel(const GemmParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    Control* ctl = reinterpret_cast<Control*>(smem);
    uint8_t* stages = smem + 1024;                                   // STAGES x (A tile, B tile)
    float* sc_ring = reinterpret_cast<float*>(stages + STAGES * STAGE_BYTES);   // [SLOTS][2][128]
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
        for (int s = 0; s < STAGES; s++) mbar_init(&ctl->full[s], 4);
        for (int b = 0; b < NACC; b++) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], EPI_WARPS);
        }
        for (int s = 0; s < SCALE_SLOTS; s++) mbar_init(&ctl->sc_full[s], 4);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) tmem_alloc(&ctl->tmem_base, NACC * BN);    // NACC 128-column int32 accumulators
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ctl->tmem_base;
    pdl_wait();

    if (warp >= PROD_WARP0) {
        // ================================================================ producers
        const int pw = warp - PROD_WARP0, q = lane >> 3, rr = lane & 7, pt = pw * 32 + lane;
        const int KW = p.K >> 3;                                     // packed words per row
        constexpr int NA = A8 ? 8 : 4;
        uint4 bufA[2][NA], bufB[2][4];
        float fsa[2], fsb[2];
        Cursor ld;                                                   // position of the loads (one step ahead)
        ld.g = 0;
        ld.set_tile((int)blockIdx.x, tiles_m);
        auto issue = [&](uint4* a, uint4* b, float& sa, float& sb) {  // loads of the step at `ld`, then advance
            const int m0 = ld.m0, n0 = ld.n0, g = ld.g;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int row = (i * 4 + pw) * 8 + rr;
                if (A8) {
                    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.aq) + (size_t)(m0 + row) * p.K + g * GK;
                    a[2 * i] = *reinterpret_cast<const uint4*>(src + q * 16);
                    a[2 * i + 1] = *reinterpret_cast<const uint4*>(src + (q + 4) * 16);
                } else {
                    a[i] = *reinterpret_cast<const uint4*>(p.aq + (size_t)(m0 + row) * KW + g * 16 + q * 4);
                }
                b[i] = (n0 + row < p.N) ? ld_stream_v4(p.wq + (size_t)(n0 + row) * KW + g * 16 + q * 4)
                                        : make_uint4(0, 0, 0, 0);
            }
            sa = p.sa[(size_t)g * p.M + m0 + pt];
            sb = (n0 + pt < p.N) ? p.sb[(size_t)g * p.N + n0 + pt] : 0.f;
            ld.next(G, tiles_m, (int)gridDim.x);
        };
        auto expand_store = [&](uint8_t* tile, int r8, const uint4& w) {   // 4 packed words -> 32 int8
            uint8_t* dst = tile + (2 * q) * LBO + r8 * SBO + rr * 16;
            *reinterpret_cast<uint4*>(dst) = make_uint4(even16(w.x), odd16(w.x), even16(w.y), odd16(w.y));
            *reinterpret_cast<uint4*>(dst + LBO) = make_uint4(even16(w.z), odd16(w.z), even16(w.w), odd16(w.w));
        };
        auto step = [&](int it, const uint4* a, const uint4* b, float sa, float sb) -> bool {
            const int s = it % STAGES;
            if (it >= STAGES && !wait_or_abort(&ctl->acc_full[s], ((it / STAGES) & 1) ^ 1, ctl, status, 1)) return false;
            uint8_t* At = stages + s * STAGE_BYTES;
            uint8_t* Bt = At + TILE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int r8 = i * 4 + pw;
                if (A8) {
                    *reinterpret_cast<uint4*>(At + q * LBO + r8 * SBO + rr * 16) = a[2 * i];
                    *reinterpret_cast<uint4*>(At + (q + 4) * LBO + r8 * SBO + rr * 16) = a[2 * i + 1];
                } else {
                    expand_store(At, r8, a[i]);
                }
                expand_store(Bt, r8, b[i]);
            }
            const int slot = it % SCALE_SLOTS;
            sc_ring[slot * 256 + pt] = sa;
            sc_ring[slot * 256 + 128 + pt] = sb;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&ctl->full[s]);
                mbar_arrive(&ctl->sc_full[slot]);
            }
            return true;
        };
        if (total > 0) issue(bufA[0], bufB[0], fsa[0], fsb[0]);
        for (int it = 0; it < total; it += 2) {
            if (it + 1 < total) issue(bufA[1], bufB[1], fsa[1], fsb[1]);
            if (!step(it, bufA[0], bufB[0], fsa[0], fsb[0])) break;
            if (it + 1 >= total) break;
            if (it + 2 < total) issue(bufA[0], bufB[0], fsa[0], fsb[0]);
            if (!step(it + 1, bufA[1], bufB[1], fsa[1], fsb[1])) break;
        }
    } else if (warp == MMA_WARP) {
        // ================================================================ MMA issuer
        if (lane == 0) {
            // everything that does not depend on the step is computed once: this single thread is
            // on the critical path of every group, so its loop body is kept to a few instructions
            const uint32_t idesc = instr_desc();
            const uint64_t adesc0 = smem_desc(smem_u32(stages));
            const uint64_t bdesc0 = smem_desc(smem_u32(stages) + TILE_BYTES);
            constexpr uint64_t kStageStep = STAGE_BYTES >> 4, kKStep = (2 * LBO) >> 4;   // descriptor units of 16 bytes
            for (int it = 0; it < total; it++) {
                const int s = it % STAGES;                  // == accumulator index (STAGES == NACC)
                const uint32_t ph = (it / STAGES) & 1;
                if (it >= NACC && !wait_or_abort(&ctl->acc_empty[s], ph ^ 1, ctl, status, 3)) break;
                if (!wait_or_abort(&ctl->full[s], ph, ctl, status, 2)) break;
                tc_fence_after();
                const uint64_t ad = adesc0 + s * kStageStep, bd = bdesc0 + s * kStageStep;
                const uint32_t d = tmem_base + s * BN;
                tc_mma_i8(d, ad, bd, idesc, 0);
                tc_mma_i8(d, ad + kKStep, bd + kKStep, idesc, 1);
                tc_mma_i8(d, ad + 2 * kKStep, bd + 2 * kKStep, idesc, 1);
                tc_mma_i8(d, ad + 3 * kKStep, bd + 3 * kKStep, idesc, 1);
                // one commit per group: STAGES == NACC, so one barrier tells the producers "stage
                // consumed" and the epilogue "accumulator complete"
                tc_commit(&ctl->acc_full[s]);
            }
        }
    } else {
        // ================================================================ epilogue
        // warp w drains TMEM lanes 32*(w%4).. (a hardware rule) and columns 64*(w/4)..+63
        constexpr int CPW = BN / (EPI_WARPS / 4);                    // columns per warp: 64
        const int lq = warp & 3, ch = warp >> 2;
        const int mrow = lq * 32 + lane;                             // TMEM lane = row of the tile
        const float inv = A8 ? (1.0f / 16.0f) : (1.0f / 256.0f);     // the integer in TMEM is 16*I or 256*I
        float facc[CPW];
#pragma unroll
        for (int j = 0; j < CPW; j++) facc[j] = 0.f;
        Cursor cur;
        cur.g = 0;
        cur.set_tile((int)blockIdx.x, tiles_m);
        for (int it = 0; it < total; it++, cur.next(G, tiles_m, (int)gridDim.x)) {
            const int b = it % NACC, slot = it % SCALE_SLOTS, g = cur.g;
            const int m0 = cur.m0, n0 = cur.n0 + ch * CPW;
            if (!wait_or_abort(&ctl->sc_full[slot], (it / SCALE_SLOTS) & 1, ctl, status, 5)) break;
            if (!wait_or_abort(&ctl->acc_full[b], (it / NACC) & 1, ctl, status, 4)) break;
            tc_fence_after();
            const float sa = sc_ring[slot * 256 + mrow] * inv;
            const float* sbv = sc_ring + slot * 256 + 128 + ch * CPW;
#pragma unroll
            for (int c = 0; c < CPW / 32; c++) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(lq * 32) << 16) + b * BN + ch * CPW + c * 32, r);
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const int col = c * 32 + j;
                    const float2 sb2 = *reinterpret_cast<const float2*>(sbv + col);
                    float s0, s1;
                    mul2(s0, s1, sa, sb2.x, sb2.y);                  // scale product, rounded to fp32 first
                    fma2(facc[col], facc[col + 1], (float)(int)r[j], (float)(int)r[j + 1], s0, s1);
                    if (DUMP) {
                        int* d = p.dump + ((size_t)(m0 + mrow) * p.N + n0 + col) * G + g;
                        if (n0 + col < p.N) d[0] = (int)r[j] >> (A8 ? 4 : 8);
                        if (n0 + col + 1 < p.N) d[G] = (int)r[j + 1] >> (A8 ? 4 : 8);
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

// ------------------------------------------------------------------------- host side
constexpr size_t kSmemBytes = 1024 + (size_t)STAGES * STAGE_BYTES + SCALE_SLOTS * 256 * 4 + 16 * 1024;

template <bool A8, bool DUMP>
int run_gemm(const char* kn, const LaunchCtx& c, const GemmParams& p) {
    auto kern = gemm_w4_kernel<A8, DUMP>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    const int ntiles = (p.M / BM) * ((p.N + BN - 1) / BN);
    const int grid = ntiles < c.sm_count ? ntiles : c.sm_count;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(kThreads), kSmemBytes, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// shared checks; tiles_needed = number of reference work-groups (128 x 64 tiles) the grid must cover
template <bool A8>
int check_gemm(const char* kn, const LaunchCtx& c, GemmParams& p, long long groups_given, bool dump) {
    FM_REQUIRE(c.wx == 256 && c.wy == 1, kn, "work-group must be 256 threads (got %ux%u)", c.wx, c.wy);
    FM_REQUIRE(p.M > 0 && p.N > 0 && p.K > 0 && p.M % 128 == 0 && p.N % 64 == 0 && p.K % 128 == 0, kn,
               "M=%d N=%d K=%d: M must be a multiple of 128, N of 64, K of 128", p.M, p.N, p.K);
    const long long need = (long long)(p.N / 64) * (p.M / 128);
    FM_REQUIRE(groups_given >= need, kn, "the grid covers %lld of the %lld 128x64 tiles; partial grids are not built",
               groups_given, need);
    FM_REQUIRE(aligned(p.aq, 16) && aligned(p.wq, 16) && aligned(p.sa, 4) && aligned(p.sb, 4) && aligned(p.C, 16), kn,
               "misaligned pointer (codes and C need 16 bytes)");
    const int G = p.K / 128;
    FM_RANGE(p.aq, A8 ? (size_t)p.M * p.K : (size_t)p.M * (p.K / 2), kn, "aq");
    FM_RANGE(p.wq, (size_t)p.N * (p.K / 2), kn, "wq");
    FM_RANGE(p.sa, (size_t)G * p.M * 4, kn, "asc");
    FM_RANGE(p.sb, (size_t)G * p.N * 4, kn, "wsc");
    FM_RANGE(p.C, (size_t)p.M * p.N * 4, kn, "C");
    if (dump) {
        FM_REQUIRE(aligned(p.dump, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.dump, (size_t)p.M * p.N * G * 4, kn, "iacc");
    }
    return FM_OK;
}

void fill(GemmParams& p, const uint64_t* a) {
    p.aq = arg_ptr<const uint32_t>(a[0]);
    p.wq = arg_ptr<const uint32_t>(a[1]);
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
    GemmParams p = {};
    fill(p, a);
    FM_REQUIRE(c.gy == 1, kn, "1-D grid expected");
    FM_REQUIRE(p.N > 0 && arg_i32(a[8]) == p.N / 64, kn, "nbn=%d must equal N/64=%d", arg_i32(a[8]), p.N / 64);
    const int rc = check_gemm<false>(kn, c, p, c.gx, false);
    return rc ? rc : run_gemm<false, false>(kn, c, p);
}

// gemm_w4a4(aq, wq, asc, wsc, C, M, N, K): grid x = N/64, grid y = M/128 (a 1-D launch covers M = 128)
int launch_gemm_2d(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gemm_w4a4";
    GemmParams p = {};
    fill(p, a);
    FM_REQUIRE(p.N > 0 && p.M > 0 && (long long)c.gx >= p.N / 64 && (long long)c.gy >= p.M / 128, kn,
               "grid %ux%u does not cover N/64=%d by M/128=%d work-groups", c.gx, c.gy, p.N / 64, p.M / 128);
    const int rc = check_gemm<false>(kn, c, p, (long long)(p.N / 64) * (p.M / 128), false);
    return rc ? rc : run_gemm<false, false>(kn, c, p);
}

// gemm_w4a8(aq8, wq, asc, wsc, C, M, N, K): aq8 = int8 codes of quant_rows_a8_k; 1-D grid of N/64 * M/128
int launch_gemm_a8(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gemm_w4a8";
    GemmParams p = {};
    fill(p, a);
    FM_REQUIRE(c.gy == 1, kn, "1-D grid expected");
    const int rc = check_gemm<true>(kn, c, p, c.gx, false);
    return rc ? rc : run_gemm<true, false>(kn, c, p);
}

// gemm_w4a4_iacc / gemm_w4a8_iacc (aq, wq, asc, wsc, C, M, N, K, iacc): iacc int32 [M][N][K/128]
template <bool A8>
int launch_gemm_iacc(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = A8 ? "gemm_w4a8_iacc" : "gemm_w4a4_iacc";
    GemmParams p = {};
    fill(p, a);
    p.dump = arg_ptr<int>(a[8]);
    const int rc = check_gemm<A8>(kn, c, p, 1LL << 40, true);
    return rc ? rc : run_gemm<A8, true>(kn, c, p);
}

const KernelEntry kGemm[] = {
    {"gemm_w4a4_flat", 10, launch_gemm_flat, "pppppiiiii"},
    {"gemm_w4a4", 8, launch_gemm_2d, "pppppiii"},
    {"gemm_w4a8", 8, launch_gemm_a8, "pppppiii"},
    {"gemm_w4a4_iacc", 9, launch_gemm_iacc<false>, "pppppiiip"},
    {"gemm_w4a8_iacc", 9, launch_gemm_iacc<true>, "pppppiiip"},
};

}  // namespace

const KernelEntry* gemm_w4_kernels(int* n) {
    *n = (int)(sizeof(kGemm) / sizeof(kGemm[0]));
    return kGemm;
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
