// w4a8_decode_stream / w4a4_decode_stream / w4a8_decode_stream_m / nvfp4_decode_stream / w4a16_decode_stream:
// one launch for the GEMVs of a whole stack of independent W4A8 (W4A4, NVFP4, W4A16)
// decode layers (M = 1), software-pipelined across layers so that HBM never idles at a
// layer boundary.  The activation codes of all layers come from one 2-D launch of the
// ordinary quant_act kernel (grid y = layer) that precedes it.
//
// The reference streams its 400-layer decode benchmark as 800 back-to-back launches on
// one in-order queue (tools/bench_decode.py:272-317).  On B200 one 17408 x 5120 layer is
// ~6.5 us of HBM time, the same order as a kernel's launch, ramp-up and drain, so the
// per-layer launches (which stay available by name) leave a quarter of the bandwidth
// unused.  This kernel keeps the arithmetic of gemv_w4a8 (reference
// kernels/gemv_w4a8_core.h:76-219) — identical int32 group accumulators, fp32 afterwards
// — and changes only the schedule:
//   * persistent grid, one CTA per SM; CTA c owns the contiguous rows
//     [c*rows/G, (c+1)*rows/G) of EVERY layer, so its weight bytes are contiguous;
//   * the last warp (one elected lane) is the producer: it walks layers and row chunks
//     and issues 1-D bulk async copies (cp.async.bulk) of CW rows of packed
//     weights plus their f16 scales into a shared-memory ring, completion counted on an
//     mbarrier per stage; once per layer it also copies that layer's int8 codes, scales
//     and group sums (5.4 KB) into a double-buffered tile;
//   * warps 0..CW-1 are consumers: warp w takes row w of a stage, lane l the 16-byte
//     words l, l+32, .. of that row (LDS.128) into registers; nibbles -> dp4a against the token's codes held in registers, two
//     shuffles per 128-group, f16 scale * act scale * float(I), butterfly, lane 0 stores y.
//   * W4A8 has a second consumer (the default) that feeds a stage of 16 rows to the tensor
//     cores as one m16 tile (mma.sync int8), described at w4a8_stream_mma_kernel below: 40 %
//     fewer instructions per weight byte, which matters because a sustained stream runs at
//     the board's power limit, where every instruction saved is SM clock (and with it L2 and
//     fabric bandwidth) kept.
// Every wait on an mbarrier is bounded; a wait that runs out sets *status and the
// thread leaves the kernel.
//
// Layers must be independent of each other (no layer reads another layer's y): the
// kernel orders nothing between layers.
#include <cuda_fp16.h>
#include <stdlib.h>

#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int kSpinLimit = 1 << 22;
constexpr int kOutCap = 512;           // rows of one CTA whose y values of a layer are collected in shared memory

struct StreamLayer {                   // one entry of the device-side layer table (32 bytes)
    const uint8_t* wq;                 // [rows][K/2] packed two's-complement nibbles
    const uint8_t* ws;                 // [rows][K/128] f16
    const float* x;                    // [K] fp32 activations of this layer
    float* y;                          // [>= row_base + rows] fp32 output of this layer
};

struct StreamParams {
    const StreamLayer* layers;
    const uint8_t *ae, *ao, *asc, *asu;   // quant_act outputs of all layers: [nlayers][K/2], .., [nlayers][K/128]
    int nlayers, rows, K, row_base;
    int npeers;                        // additional GPUs that receive y (0 on one GPU)
    const long long* peer_delta;       // [npeers] byte offset from a local y address to the peer's copy
    int* status;                       // 0 ok, else first failure code
    int M, ystride;                    // tokens per layer and floats between their outputs (multi-token kernel only)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
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
// bounded wait: false (and *status = code) when the limit runs out
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, int* status, int code) {
    for (int i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(b, parity)) return true;
    atomicCAS(status, 0, code);
    return false;
}
// Pins a value in program order: volatile statements are not reordered with each other, so an
// mbarrier.arrive that follows cannot be scheduled ahead of the arithmetic that produced `v`
// (and with it ahead of the shared-memory loads that arithmetic consumed).
__device__ __forceinline__ void consumed(float v) { asm volatile("" ::"f"(v) : "memory"); }
// 1-D bulk async copy global -> this CTA's shared memory
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Output tile.  A CTA's y values of one layer (at most kOutCap rows, else they are stored one by
// one) are collected in shared memory and written out once per layer by one warp as coalesced
// 128-byte stores: to the local y and to every additional copy (other GPUs' y over NVLink, a
// pinned host buffer over PCIe).  Per-row 4- or 64-byte stores are fine for HBM but throttle
// the kernel when they cross a link.  ydone[b] counts the consumer warps that have finished the
// layer, yfree[b] is set by the writer when the tile may be overwritten (two tiles alternate).
// The writer is a warp of its own, so that a slow link never holds up a consumer.
__device__ __forceinline__ void write_out(const StreamParams& p, const float* tile, float* y, int n, int lane) {
    for (int i = lane; i < n; i += 32) {
        const float v = tile[i];
        y[i] = v;
        for (int q = 0; q < p.npeers; q++)
            *reinterpret_cast<float*>(reinterpret_cast<char*>(y + i) + p.peer_delta[q]) = v;
    }
}

// KITER: K = KITER * 1024.  CW: consumer warps = weight rows per ring stage.  STAGES: ring depth.
// Warp roles: 0..CW-1 consumers, CW producer (one lane), CW+1 writer of the output tile.
// A4: int4 activations of quant_act4 (packed nibbles + one scale per 32 k) instead of the int8
//     codes of quant_act; the nibbles are sign-extended to int8 in registers at each layer start
//     and the integers are lane-private (a 16-byte word is one 32-sub-group).
template <bool A4, int KITER, int CW, int STAGES>
__global__ void __launch_bounds__((CW + 2) * 32, 1)
w4_stream_kernel(const StreamParams p) {
    constexpr int K = KITER * 1024, NG = K / 128;
    constexpr int ROWB = K / 2, SCB = NG * 2;
    constexpr int STAGE_W = CW * ROWB, STAGE = STAGE_W + CW * SCB;
    constexpr int ACT = A4 ? K / 2 + (K / 32) * 4        // packed nibbles, sub-group scales
                           : K + NG * 8;               // even codes, odd codes, scales, sums
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);      // [STAGES] weights landed
    uint64_t* empty = full + STAGES;                          // [STAGES] weights copied to registers
    uint64_t* act_ready = empty + STAGES;                     // [2] codes of a layer are in shared memory
    uint64_t* act_free = act_ready + 2;                       // [2] every consumer has its register copy
    uint64_t* ydone = act_free + 2;                           // [2] output tile complete
    uint64_t* yfree = ydone + 2;                              // [2] output tile written out
    uint8_t* ring = smem + 256;
    uint8_t* act = ring + (size_t)STAGES * STAGE;             // [2][ACT]
    float* ytile = reinterpret_cast<float*>(act + 2 * ACT);   // [2][kOutCap]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&act_ready[b], 1);
            mbar_init(&act_free[b], CW);
            mbar_init(&ydone[b], CW);
            mbar_init(&yfree[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();                                          // the codes come from the preceding quant_act

    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int nst = (r1 - r0 + CW - 1) / CW;             // stages per layer for this CTA
    const bool tiled = (r1 - r0) <= kOutCap;

    if (warp == CW) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            auto copy_codes = [&](int l) -> bool {       // layer l's codes -> act[l & 1]
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(&act_free[b], ((l >> 1) & 1) ^ 1, p.status, 4)) return false;
                uint8_t* ab = act + (size_t)b * ACT;
                mbar_expect_tx(&act_ready[b], ACT);
                if (A4) {
                    bulk_g2s(ab, p.ae + (size_t)l * (K / 2), K / 2, &act_ready[b]);                  // aq
                    bulk_g2s(ab + K / 2, p.asc + (size_t)l * (K / 32 * 4), K / 32 * 4, &act_ready[b]);
                } else {
                    bulk_g2s(ab, p.ae + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                    bulk_g2s(ab + K / 2, p.ao + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                    bulk_g2s(ab + K, p.asc + (size_t)l * (NG * 4), NG * 4, &act_ready[b]);
                    bulk_g2s(ab + K + NG * 4, p.asu + (size_t)l * (NG * 4), NG * 4, &act_ready[b]);
                }
                return true;
            };
            int c = 0;
            const uint8_t* wq = p.layers[0].wq;
            const uint8_t* ws = p.layers[0].ws;
            if (!copy_codes(0)) return;
            for (int l = 0; l < p.nlayers; l++) {
                // next layer's addresses and codes are fetched while this layer's weights stream
                const int ln = min(l + 1, p.nlayers - 1);
                const uint8_t* wq_n = p.layers[ln].wq;
                const uint8_t* ws_n = p.layers[ln].ws;
                for (int j = 0; j < nst; j++, c++) {
                    const int s = c % STAGES;
                    if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) & 1) ^ 1, p.status, 1)) return;
                    const int row = r0 + j * CW;
                    const int nr = min(CW, r1 - row);
                    uint8_t* dst = ring + (size_t)s * STAGE;
                    mbar_expect_tx(&full[s], (uint32_t)(nr * (ROWB + SCB)));
                    bulk_g2s(dst, wq + (size_t)row * ROWB, (uint32_t)(nr * ROWB), &full[s]);
                    bulk_g2s(dst + STAGE_W, ws + (size_t)row * SCB, (uint32_t)(nr * SCB), &full[s]);
                    if (j == 0 && l + 1 < p.nlayers && !copy_codes(l + 1)) return;
                }
                wq = wq_n;
                ws = ws_n;
            }
        }
        return;
    }

    if (warp == CW + 1) {                                    // writer: one coalesced pass per layer over the output tile
        if (!tiled) return;
        for (int l = 0; l < p.nlayers; l++) {
            if (!mbar_wait(&ydone[l & 1], (l >> 1) & 1, p.status, 8)) return;
            write_out(p, ytile + (l & 1) * kOutCap, p.layers[l].y + p.row_base + r0, r1 - r0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&yfree[l & 1]);
        }
        if (p.npeers) __threadfence_system();
        return;
    }

    // ---------------------------------------------------------------- consumers
    int c = 0;
    for (int l = 0; l < p.nlayers; l++) {
        const uint8_t* ab = act + (size_t)(l & 1) * ACT;
        float* yt = ytile + (l & 1) * kOutCap;
        if (tiled && l >= 2 && !mbar_wait(&yfree[l & 1], ((l >> 1) & 1) ^ 1, p.status, 7)) return;
        if (!mbar_wait(&act_ready[l & 1], (l >> 1) & 1, p.status, 2)) return;
        // register copy of the token's codes for this lane's words
        uint4 ae[KITER], ao[KITER];
        float asc[KITER];
        int asu8[KITER];
#pragma unroll
        for (int it = 0; it < KITER; it++) {
            const int d0 = it * 128 + lane * 4;
            if (A4) {
                const uint4 a = *reinterpret_cast<const uint4*>(ab + d0 * 4);      // 32 nibbles = one sub-group
                ae[it] = make_uint4(sext_nibbles(a.x & 0x0F0F0F0Fu), sext_nibbles(a.y & 0x0F0F0F0Fu),
                                    sext_nibbles(a.z & 0x0F0F0F0Fu), sext_nibbles(a.w & 0x0F0F0F0Fu));
                ao[it] = make_uint4(sext_nibbles((a.x >> 4) & 0x0F0F0F0Fu), sext_nibbles((a.y >> 4) & 0x0F0F0F0Fu),
                                    sext_nibbles((a.z >> 4) & 0x0F0F0F0Fu), sext_nibbles((a.w >> 4) & 0x0F0F0F0Fu));
                asc[it] = *reinterpret_cast<const float*>(ab + K / 2 + (d0 >> 2) * 4);
                int su = 0;
                su = dot4(ae[it].x, 0x01010101u, su); su = dot4(ao[it].x, 0x01010101u, su);
                su = dot4(ae[it].y, 0x01010101u, su); su = dot4(ao[it].y, 0x01010101u, su);
                su = dot4(ae[it].z, 0x01010101u, su); su = dot4(ao[it].z, 0x01010101u, su);
                su = dot4(ae[it].w, 0x01010101u, su); su = dot4(ao[it].w, 0x01010101u, su);
                asu8[it] = 8 * su;
            } else {
                ae[it] = *reinterpret_cast<const uint4*>(ab + d0 * 4);
                ao[it] = *reinterpret_cast<const uint4*>(ab + K / 2 + d0 * 4);
                asc[it] = *reinterpret_cast<const float*>(ab + K + (d0 >> 4) * 4);
                asu8[it] = 8 * *reinterpret_cast<const int*>(ab + K + NG * 4 + (d0 >> 4) * 4);
            }
        }
        float* y = p.layers[l].y + p.row_base;

        for (int j = 0; j < nst; j++, c++) {
            const int s = c % STAGES;
            if (!mbar_wait(&full[s], (c / STAGES) & 1, p.status, 3)) return;
            const int row = r0 + j * CW + warp;
            const bool live = row < r1;
            const uint8_t* st = ring + (size_t)s * STAGE;
            const uint4* wrow = reinterpret_cast<const uint4*>(st + (size_t)warp * ROWB);
            const __half* srow = reinterpret_cast<const __half*>(st + STAGE_W + (size_t)warp * SCB);
            // `live` is uniform over the warp (one row per warp), so dead rows of a partial last
            // stage skip the loads and the arithmetic altogether
            uint4 w[KITER];
            float sw[KITER];
            if (live) {
#pragma unroll
                for (int it = 0; it < KITER; it++) {
                    w[it] = wrow[it * 32 + lane];
                    sw[it] = __half2float(srow[(it * 128 + lane * 4) >> 4]);
                }
            }
            float acc = 0.f;
            if (live) {
#pragma unroll
                for (int it = 0; it < KITER; it++) {
                    int v = dot32_u(w[it], ae[it], ao[it]);
                    if (!A4) {
                        v += __shfl_xor_sync(0xffffffffu, v, 1);
                        v += __shfl_xor_sync(0xffffffffu, v, 2);
                    }
                    if (A4 || (lane & 3) == 0) acc += (sw[it] * asc[it]) * (float)(v - asu8[it]);
                }
            }
            // Release only now: the arithmetic above has consumed every register loaded from the stage
            // (and, in a layer's first stage, from the code tile), so those loads have completed.  An
            // arrive issued right behind the loads can overtake them, and the refill would race with them.
            consumed(acc);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                if (j == 0) mbar_arrive(&act_free[l & 1]);
            }
            if (!live) continue;
            acc = warp_sum(acc);
            if (lane == 0) {
                if (tiled) {
                    yt[row - r0] = acc;
                } else {
                    y[row] = acc;
                    for (int q = 0; q < p.npeers; q++)       // all-gather by direct peer stores over NVLink
                        *reinterpret_cast<float*>(reinterpret_cast<char*>(y + row) + p.peer_delta[q]) = acc;
                }
            }
        }
        if (tiled) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ydone[l & 1]);
        }
    }
    if (p.npeers) __threadfence_system();                    // peer stores are visible before the kernel ends
}

// ------------------------------------------------------------------------------------
// Tensor-core consumer (W4A8, one token).  The dp4a consumer above is bound by the ALU pipe
// (two LOP3 and two dp4a per packed word, plus shuffles).  Here a stage of 16 weight rows is
// one m16 tile: each of the 8 consumer warps takes 5 of the 40 groups of all 16 rows and
// multiplies them with mma.sync m16n8k32 (int8 x int8 -> int32; the token is column 0 of B).
// Per packed word only the two nibble masks remain: low nibbles as bytes u = n ^ 8 (signed
// operand), high nibbles in place as unsigned bytes 16*u (the u8 x s8 form), two accumulators,
//   I[n,g] = acc_lo + (acc_hi >> 4) - 8 * sum(q)        exactly, no shuffles,
// because the MMA itself adds over the four lanes that share a group.  Warp w scales groups
// w, w+8, ..., w+32 in fp32 and the eight per-warp partial sums of a row are added by one
// warp per stage (rotating) through a small shared-memory tile, as the tree
// ((p0+p4)+(p2+p6)) + ((p1+p5)+(p3+p7)): the association of the dp4a consumer's lane
// partials and xor-butterfly, so both variants (and gemv_w4a8) give the same bits.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int STAGES>
__global__ void __launch_bounds__(10 * 32, 1)
w4a8_stream_mma_kernel(const StreamParams p) {
    constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;   // 8 consumer warps x 5 groups, 16 rows per stage
    constexpr int ROWB = K / 2, SCB = NG * 2;
    constexpr int STAGE_W = ROWS * ROWB, STAGE = STAGE_W + ROWS * SCB;
    constexpr int ACT = K + NG * 8;
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + STAGES;
    uint64_t* act_ready = empty + STAGES;     // [2]
    uint64_t* act_free = act_ready + 2;       // [2]
    uint64_t* red_full = act_free + 2;        // [2] all eight partial sums of a stage are written
    uint64_t* red_free = red_full + 2;        // [2] the reducer has read them
    uint64_t* ydone = red_free + 2;           // [2] output tile complete
    uint64_t* yfree = ydone + 2;              // [2] output tile written out
    uint8_t* ring = smem + 256;
    uint8_t* act = ring + (size_t)STAGES * STAGE;
    float* red = reinterpret_cast<float*>(act + 2 * ACT);             // [2][CW][ROWS]
    float* ytile = red + 2 * CW * ROWS;                               // [2][kOutCap]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&act_ready[b], 1);
            mbar_init(&act_free[b], CW);
            mbar_init(&red_full[b], CW);
            mbar_init(&red_free[b], 1);
            mbar_init(&ydone[b], CW);
            mbar_init(&yfree[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();

    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int nst = (r1 - r0 + ROWS - 1) / ROWS;
    const bool tiled = (r1 - r0) <= kOutCap;

    if (warp == CW) {
        if (lane == 0) {                                   // producer: identical to the dp4a kernel's
            auto copy_codes = [&](int l) -> bool {
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(&act_free[b], ((l >> 1) & 1) ^ 1, p.status, 4)) return false;
                uint8_t* ab = act + (size_t)b * ACT;
                mbar_expect_tx(&act_ready[b], ACT);
                bulk_g2s(ab, p.ae + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                bulk_g2s(ab + K / 2, p.ao + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                bulk_g2s(ab + K, p.asc + (size_t)l * (NG * 4), NG * 4, &act_ready[b]);
                bulk_g2s(ab + K + NG * 4, p.asu + (size_t)l * (NG * 4), NG * 4, &act_ready[b]);
                return true;
            };
            int c = 0;
            const uint8_t* wq = p.layers[0].wq;
            const uint8_t* ws = p.layers[0].ws;
            if (!copy_codes(0)) return;
            for (int l = 0; l < p.nlayers; l++) {
                const int ln = min(l + 1, p.nlayers - 1);
                const uint8_t* wq_n = p.layers[ln].wq;
                const uint8_t* ws_n = p.layers[ln].ws;
                for (int j = 0; j < nst; j++, c++) {
                    const int s = c % STAGES;
                    if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) & 1) ^ 1, p.status, 1)) return;
                    const int row = r0 + j * ROWS;
                    const int nr = min(ROWS, r1 - row);
                    uint8_t* dst = ring + (size_t)s * STAGE;
                    mbar_expect_tx(&full[s], (uint32_t)(nr * (ROWB + SCB)));
                    bulk_g2s(dst, wq + (size_t)row * ROWB, (uint32_t)(nr * ROWB), &full[s]);
                    bulk_g2s(dst + STAGE_W, ws + (size_t)row * SCB, (uint32_t)(nr * SCB), &full[s]);
                    if (j == 0 && l + 1 < p.nlayers && !copy_codes(l + 1)) return;
                }
                wq = wq_n;
                ws = ws_n;
            }
        }
        return;
    }

    if (warp == CW + 1) {                                    // writer: one coalesced pass per layer over the output tile
        if (!tiled) return;
        for (int l = 0; l < p.nlayers; l++) {
            if (!mbar_wait(&ydone[l & 1], (l >> 1) & 1, p.status, 8)) return;
            write_out(p, ytile + (l & 1) * kOutCap, p.layers[l].y + p.row_base + r0, r1 - r0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&yfree[l & 1]);
        }
        if (p.npeers) __threadfence_system();
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;                 // fragment coordinates: rows g and g+8, k slot t
    int c = 0;
    for (int l = 0; l < p.nlayers; l++) {
        const uint8_t* ab = act + (size_t)(l & 1) * ACT;
        float* yt = ytile + (l & 1) * kOutCap;
        if (tiled && l >= 2 && !mbar_wait(&yfree[l & 1], ((l >> 1) & 1) ^ 1, p.status, 7)) return;
        if (!mbar_wait(&act_ready[l & 1], (l >> 1) & 1, p.status, 2)) return;
        uint4 be[GPW], bo[GPW];                            // B fragments: codes of the token for this lane's k slots
        float sa[GPW];
        int su8[GPW];
#pragma unroll
        for (int j = 0; j < GPW; j++) {
            const int gg = j * CW + warp;                   // this warp's groups: warp, warp + 8, ...
            be[j] = *reinterpret_cast<const uint4*>(ab + (gg * 16 + 4 * t) * 4);
            bo[j] = *reinterpret_cast<const uint4*>(ab + K / 2 + (gg * 16 + 4 * t) * 4);
            sa[j] = *reinterpret_cast<const float*>(ab + K + gg * 4);
            su8[j] = 8 * *reinterpret_cast<const int*>(ab + K + NG * 4 + gg * 4);
        }
        float* y = p.layers[l].y + p.row_base;

        for (int jst = 0; jst < nst; jst++, c++) {
            const int s = c % STAGES;
            if (!mbar_wait(&full[s], (c / STAGES) & 1, p.status, 3)) return;
            const uint8_t* st = ring + (size_t)s * STAGE;
            uint4 xa[GPW], xb[GPW];                        // packed words of rows g and g+8
            float swa[GPW], swb[GPW];
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                const int gg = j * CW + warp;                   // this warp's groups: warp, warp + 8, ...
                xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * ROWB + gg * 64 + t * 16);
                xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * ROWB + gg * 64 + t * 16);
                swa[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + g * SCB + gg * 2));
                swb[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + (g + 8) * SCB + gg * 2));
            }
            float fa = 0.f, fb = 0.f;                       // partial y of rows g and g+8 over this warp's groups
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
                const uint32_t m_lo = 0x0F0F0F0Fu, x_lo = 0x08080808u, m_hi = 0xF0F0F0F0u, x_hi = 0x80808080u;
                mma_s8(lo, (xa[j].x & m_lo) ^ x_lo, (xb[j].x & m_lo) ^ x_lo, (xa[j].y & m_lo) ^ x_lo, (xb[j].y & m_lo) ^ x_lo,
                       be[j].x, be[j].y);
                mma_s8(lo, (xa[j].z & m_lo) ^ x_lo, (xb[j].z & m_lo) ^ x_lo, (xa[j].w & m_lo) ^ x_lo, (xb[j].w & m_lo) ^ x_lo,
                       be[j].z, be[j].w);
                mma_u8(hi, (xa[j].x & m_hi) ^ x_hi, (xb[j].x & m_hi) ^ x_hi, (xa[j].y & m_hi) ^ x_hi, (xb[j].y & m_hi) ^ x_hi,
                       bo[j].x, bo[j].y);
                mma_u8(hi, (xa[j].z & m_hi) ^ x_hi, (xb[j].z & m_hi) ^ x_hi, (xa[j].w & m_hi) ^ x_hi, (xb[j].w & m_hi) ^ x_hi,
                       bo[j].z, bo[j].w);
                // column 0 (the token) of the accumulator tile sits in the lanes with t == 0
                const int ia = lo[0] + (hi[0] >> 4) - su8[j];
                const int ib = lo[2] + (hi[2] >> 4) - su8[j];
                fa += (swa[j] * sa[j]) * (float)ia;
                fb += (swb[j] * sa[j]) * (float)ib;
            }
            // Release only now: the MMAs and multiplies above have consumed every register loaded from
            // the stage (and, in a layer's first stage, from the code tile), so those loads have
            // completed.  An arrive issued right behind the loads can overtake them.
            consumed(fa + fb);
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                if (jst == 0) mbar_arrive(&act_free[l & 1]);
            }
            const int rb = c & 1;
            if (c >= 2 && !mbar_wait(&red_free[rb], ((c >> 1) & 1) ^ 1, p.status, 5)) return;
            if (t == 0) {
                red[(rb * CW + warp) * ROWS + g] = fa;
                red[(rb * CW + warp) * ROWS + g + 8] = fb;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_full[rb]);
            if (warp == (c % CW)) {                         // this stage's reducer: fixed order over the warps
                if (!mbar_wait(&red_full[rb], (c >> 1) & 1, p.status, 6)) return;
                const int row = r0 + jst * ROWS + lane;
                float acc = 0.f;
                if (lane < ROWS) {
                    const float* pr = red + rb * CW * ROWS + lane;
                    acc = ((pr[0 * ROWS] + pr[4 * ROWS]) + (pr[2 * ROWS] + pr[6 * ROWS])) +
                          ((pr[1 * ROWS] + pr[5 * ROWS]) + (pr[3 * ROWS] + pr[7 * ROWS]));
                }
                consumed(acc);                              // the partial sums are read before the tile is released
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_free[rb]);
                if (lane < ROWS && row < r1) {
                    if (tiled) {
                        yt[row - r0] = acc;
                    } else {
                        y[row] = acc;
                        for (int q = 0; q < p.npeers; q++)
                            *reinterpret_cast<float*>(reinterpret_cast<char*>(y + row) + p.peer_delta[q]) = acc;
                    }
                }
            }
        }
        if (tiled) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ydone[l & 1]);
        }
    }
    if (p.npeers) __threadfence_system();
}

// ------------------------------------------------------------------------------------
// Several tokens per layer (W4A8, M = 2..4): the tensor-core consumer with the tokens as the
// columns of the MMA, so a small decode batch streams the weights once.  Same ring, barriers and
// roles as w4a8_stream_mma_kernel; what differs: the code tile of a layer holds M tokens
// ([M][K/2] even codes, [M][K/2] odd codes, [M][NG] scales, [M][NG] sums — the layout one 2-D
// quant_act launch with grid y = layer * M + token leaves behind), lane (g, t) feeds token
// min(g, M-1) as column g and owns the sums of rows g, g + 8 for tokens 2t and 2t + 1, and y of
// a layer is token-major: y[token * ystride + row].
__device__ __forceinline__ void write_out_m(const StreamParams& p, const float* tile, float* y, int n, int lane, int M) {
    for (int i = lane; i < n * M; i += 32) {
        const int tok = i / n, row = i - tok * n;            // token-major walk: coalesced global stores
        const float v = tile[row * M + tok];
        float* dst = y + (size_t)tok * p.ystride + row;
        *dst = v;
        for (int q = 0; q < p.npeers; q++)
            *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = v;
    }
}

template <int STAGES, int M>
__global__ void __launch_bounds__(10 * 32, 1)
w4a8_stream_mma_m_kernel(const StreamParams p) {
    constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;
    constexpr int ROWB = K / 2, SCB = NG * 2;
    constexpr int STAGE_W = ROWS * ROWB, STAGE = STAGE_W + ROWS * SCB;
    constexpr int ACT = M * (K + NG * 8);
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + STAGES;
    uint64_t* act_ready = empty + STAGES;     // [2]
    uint64_t* act_free = act_ready + 2;       // [2]
    uint64_t* red_full = act_free + 2;        // [2]
    uint64_t* red_free = red_full + 2;        // [2]
    uint64_t* ydone = red_free + 2;           // [2]
    uint64_t* yfree = ydone + 2;              // [2]
    uint8_t* ring = smem + 256;
    uint8_t* act = ring + (size_t)STAGES * STAGE;
    float* red = reinterpret_cast<float*>(act + 2 * ACT);             // [2][CW][ROWS][M]
    float* ytile = red + 2 * CW * ROWS * M;                           // [2][kOutCap]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&act_ready[b], 1);
            mbar_init(&act_free[b], CW);
            mbar_init(&red_full[b], CW);
            mbar_init(&red_free[b], 1);
            mbar_init(&ydone[b], CW);
            mbar_init(&yfree[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();

    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int nst = (r1 - r0 + ROWS - 1) / ROWS;
    const bool tiled = (r1 - r0) * M <= kOutCap;

    if (warp == CW) {
        if (lane == 0) {                                   // producer
            auto copy_codes = [&](int l) -> bool {
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(&act_free[b], ((l >> 1) & 1) ^ 1, p.status, 4)) return false;
                uint8_t* ab = act + (size_t)b * ACT;
                mbar_expect_tx(&act_ready[b], ACT);
                bulk_g2s(ab, p.ae + (size_t)l * M * (K / 2), M * (K / 2), &act_ready[b]);
                bulk_g2s(ab + M * (K / 2), p.ao + (size_t)l * M * (K / 2), M * (K / 2), &act_ready[b]);
                bulk_g2s(ab + M * K, p.asc + (size_t)l * M * (NG * 4), M * NG * 4, &act_ready[b]);
                bulk_g2s(ab + M * K + M * NG * 4, p.asu + (size_t)l * M * (NG * 4), M * NG * 4, &act_ready[b]);
                return true;
            };
            int c = 0;
            const uint8_t* wq = p.layers[0].wq;
            const uint8_t* ws = p.layers[0].ws;
            if (!copy_codes(0)) return;
            for (int l = 0; l < p.nlayers; l++) {
                const int ln = min(l + 1, p.nlayers - 1);
                const uint8_t* wq_n = p.layers[ln].wq;
                const uint8_t* ws_n = p.layers[ln].ws;
                for (int j = 0; j < nst; j++, c++) {
                    const int s = c % STAGES;
                    if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) & 1) ^ 1, p.status, 1)) return;
                    const int row = r0 + j * ROWS;
                    const int nr = min(ROWS, r1 - row);
                    uint8_t* dst = ring + (size_t)s * STAGE;
                    mbar_expect_tx(&full[s], (uint32_t)(nr * (ROWB + SCB)));
                    bulk_g2s(dst, wq + (size_t)row * ROWB, (uint32_t)(nr * ROWB), &full[s]);
                    bulk_g2s(dst + STAGE_W, ws + (size_t)row * SCB, (uint32_t)(nr * SCB), &full[s]);
                    if (j == 0 && l + 1 < p.nlayers && !copy_codes(l + 1)) return;
                }
                wq = wq_n;
                ws = ws_n;
            }
        }
        return;
    }

    if (warp == CW + 1) {                                    // writer
        if (!tiled) return;
        for (int l = 0; l < p.nlayers; l++) {
            if (!mbar_wait(&ydone[l & 1], (l >> 1) & 1, p.status, 8)) return;
            write_out_m(p, ytile + (l & 1) * kOutCap, p.layers[l].y + p.row_base + r0, r1 - r0, lane, M);
            __syncwarp();
            if (lane == 0) mbar_arrive(&yfree[l & 1]);
        }
        if (p.npeers) __threadfence_system();
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    const int tk = g < M ? g : M - 1;                      // token fed as column g (columns >= M are never read)
    const int t0 = 2 * t, t1 = 2 * t + 1;                  // tokens whose sums this lane owns
    int c = 0;
    for (int l = 0; l < p.nlayers; l++) {
        const uint8_t* ab = act + (size_t)(l & 1) * ACT;
        float* yt = ytile + (l & 1) * kOutCap;
        if (tiled && l >= 2 && !mbar_wait(&yfree[l & 1], ((l >> 1) & 1) ^ 1, p.status, 7)) return;
        if (!mbar_wait(&act_ready[l & 1], (l >> 1) & 1, p.status, 2)) return;
        uint4 be[GPW], bo[GPW];
        float sa0[GPW], sa1[GPW];
        int su0[GPW], su1[GPW];
#pragma unroll
        for (int j = 0; j < GPW; j++) {
            const int gg = j * CW + warp;
            be[j] = *reinterpret_cast<const uint4*>(ab + tk * (K / 2) + (gg * 16 + 4 * t) * 4);
            bo[j] = *reinterpret_cast<const uint4*>(ab + M * (K / 2) + tk * (K / 2) + (gg * 16 + 4 * t) * 4);
            const float* scp = reinterpret_cast<const float*>(ab + M * K);
            const int* sup = reinterpret_cast<const int*>(ab + M * K + M * NG * 4);
            sa0[j] = t0 < M ? scp[t0 * NG + gg] : 0.f;
            sa1[j] = t1 < M ? scp[t1 * NG + gg] : 0.f;
            su0[j] = t0 < M ? 8 * sup[t0 * NG + gg] : 0;
            su1[j] = t1 < M ? 8 * sup[t1 * NG + gg] : 0;
        }
        float* y = p.layers[l].y + p.row_base;

        for (int jst = 0; jst < nst; jst++, c++) {
            const int s = c % STAGES;
            if (!mbar_wait(&full[s], (c / STAGES) & 1, p.status, 3)) return;
            const uint8_t* st = ring + (size_t)s * STAGE;
            uint4 xa[GPW], xb[GPW];
            float swa[GPW], swb[GPW];
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                const int gg = j * CW + warp;
                xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * ROWB + gg * 64 + t * 16);
                xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * ROWB + gg * 64 + t * 16);
                swa[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + g * SCB + gg * 2));
                swb[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + (g + 8) * SCB + gg * 2));
            }
            float fa0 = 0.f, fa1 = 0.f, fb0 = 0.f, fb1 = 0.f;   // rows g, g+8 x tokens t0, t1 over this warp's groups
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
                const uint32_t m_lo = 0x0F0F0F0Fu, x_lo = 0x08080808u, m_hi = 0xF0F0F0F0u, x_hi = 0x80808080u;
                mma_s8(lo, (xa[j].x & m_lo) ^ x_lo, (xb[j].x & m_lo) ^ x_lo, (xa[j].y & m_lo) ^ x_lo, (xb[j].y & m_lo) ^ x_lo,
                       be[j].x, be[j].y);
                mma_s8(lo, (xa[j].z & m_lo) ^ x_lo, (xb[j].z & m_lo) ^ x_lo, (xa[j].w & m_lo) ^ x_lo, (xb[j].w & m_lo) ^ x_lo,
                       be[j].z, be[j].w);
                mma_u8(hi, (xa[j].x & m_hi) ^ x_hi, (xb[j].x & m_hi) ^ x_hi, (xa[j].y & m_hi) ^ x_hi, (xb[j].y & m_hi) ^ x_hi,
                       bo[j].x, bo[j].y);
                mma_u8(hi, (xa[j].z & m_hi) ^ x_hi, (xb[j].z & m_hi) ^ x_hi, (xa[j].w & m_hi) ^ x_hi, (xb[j].w & m_hi) ^ x_hi,
                       bo[j].z, bo[j].w);
                // accumulator columns 2t and 2t+1 of this lane are tokens t0 and t1
                fa0 += (swa[j] * sa0[j]) * (float)(lo[0] + (hi[0] >> 4) - su0[j]);
                fa1 += (swa[j] * sa1[j]) * (float)(lo[1] + (hi[1] >> 4) - su1[j]);
                fb0 += (swb[j] * sa0[j]) * (float)(lo[2] + (hi[2] >> 4) - su0[j]);
                fb1 += (swb[j] * sa1[j]) * (float)(lo[3] + (hi[3] >> 4) - su1[j]);
            }
            // release only after the loaded registers have been consumed (see the one-token kernel)
            consumed((fa0 + fa1) + (fb0 + fb1));
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                if (jst == 0) mbar_arrive(&act_free[l & 1]);
            }
            const int rb = c & 1;
            if (c >= 2 && !mbar_wait(&red_free[rb], ((c >> 1) & 1) ^ 1, p.status, 5)) return;
            float* rw = red + (size_t)(rb * CW + warp) * ROWS * M;
            if (t0 < M) {
                rw[g * M + t0] = fa0;
                rw[(g + 8) * M + t0] = fb0;
            }
            if (t1 < M) {
                rw[g * M + t1] = fa1;
                rw[(g + 8) * M + t1] = fb1;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_full[rb]);
            if (warp == (c % CW)) {                         // this stage's reducer: fixed order over the warps
                if (!mbar_wait(&red_full[rb], (c >> 1) & 1, p.status, 6)) return;
                float acc[(ROWS * M + 31) / 32];
#pragma unroll
                for (int k = 0; k < (ROWS * M + 31) / 32; k++) {
                    const int i = k * 32 + lane;
                    acc[k] = 0.f;
                    if (i < ROWS * M) {
                        const float* pr = red + (size_t)rb * CW * ROWS * M + i;
                        constexpr int W = ROWS * M;
                        acc[k] = ((pr[0 * W] + pr[4 * W]) + (pr[2 * W] + pr[6 * W])) + ((pr[1 * W] + pr[5 * W]) + (pr[3 * W] + pr[7 * W]));
                    }
                    consumed(acc[k]);                       // read before the tile is released
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_free[rb]);
#pragma unroll
                for (int k = 0; k < (ROWS * M + 31) / 32; k++) {
                    const int i = k * 32 + lane;
                    const int rr = i / M, tok = i - rr * M, row = r0 + jst * ROWS + rr;
                    if (i < ROWS * M && row < r1) {
                        if (tiled) {
                            yt[(row - r0) * M + tok] = acc[k];
                        } else {
                            float* dst = y + (size_t)tok * p.ystride + row;
                            *dst = acc[k];
                            for (int q = 0; q < p.npeers; q++)
                                *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = acc[k];
                        }
                    }
                }
            }
        }
        if (tiled) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ydone[l & 1]);
        }
    }
    if (p.npeers) __threadfence_system();
}

template <int STAGES, int M>
int run_stream_mma_m(const char* kn, const LaunchCtx& c, const StreamParams& p) {
    constexpr int K = 5120;
    constexpr size_t smem = 256 + (size_t)STAGES * 16 * (K / 2 + 80) + 2 * M * (K + 320) + 2 * 8 * 16 * M * 4 + 2 * kOutCap * 4;
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = w4a8_stream_mma_m_kernel<STAGES, M>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > p.rows) grid = p.rows;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(10 * 32), smem, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

template <int STAGES>
int run_stream_mma(const char* kn, const LaunchCtx& c, const StreamParams& p) {
    constexpr int K = 5120;
    constexpr size_t smem = 256 + (size_t)STAGES * 16 * (K / 2 + 80) + 2 * (K + 320) + 2 * 8 * 16 * 4 + 2 * kOutCap * 4;
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = w4a8_stream_mma_kernel<STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > p.rows) grid = p.rows;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(10 * 32), smem, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

template <bool A4, int KITER, int CW, int STAGES>
int run_stream(const char* kn, const LaunchCtx& c, const StreamParams& p) {
    constexpr int K = KITER * 1024;
    constexpr size_t smem = 256 + (size_t)STAGES * CW * (K / 2 + (K / 128) * 2) + 2 * (K + (K / 128) * 8) + 2 * kOutCap * 4;
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = w4_stream_kernel<A4, KITER, CW, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > p.rows) grid = p.rows;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3((CW + 2) * 32), smem, c.stream, pdl_enabled(), p);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// w4a8_decode_stream(layers, nlayers, rows, K, row_base, npeers, peer_delta, status, ae, ao, asc, asu)
//   layers      device array of nlayers x {wq, ws, x, y} pointers (32 bytes each), filled by
//               fm_stream_table (which range-checks every pointer in it)
//   rows        weight rows held by this GPU (N, or N / number of GPUs)
//   row_base    first output index of this GPU's rows inside each layer's y
//   npeers      0, or the number of other copies of y that also receive the rows (other GPUs'
//               buffers and/or a pinned host buffer: up to 8);
//   peer_delta  device array of npeers signed byte offsets (peer y address - local y address),
//               filled by fm_stream_peers from allocations opened with fm_ipc_import
//   status      device int, must be 0 before the launch; non-zero afterwards = a bounded
//               wait ran out (1 producer/ring, 2 codes not landed, 3 consumer/ring, 4 code tile not free,
//               5 / 6 partial-sum tile of the tensor-core variant)
//   ae, ao, asc, asu   outputs of quant_act launched with grid y = nlayers over x [nlayers][K]:
//               int8 codes [nlayers][K/2] twice, f32 scales and int32 sums [nlayers][K/128]
// grid and work-group arguments are ignored (persistent: one CTA per SM).
// w4a4_decode_stream(layers, nlayers, rows, K, row_base, npeers, peer_delta, status, aq, asc): the same
// with the outputs of quant_act4 (grid y = nlayers): packed nibbles [nlayers][K/2], scales [nlayers][K/32].
template <bool A4>
int launch_w4_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = A4 ? "w4a4_decode_stream" : "w4a8_decode_stream";
    StreamParams p = {};
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.nlayers = arg_i32(a[1]);
    p.rows = arg_i32(a[2]);
    p.K = arg_i32(a[3]);
    p.row_base = arg_i32(a[4]);
    p.npeers = arg_i32(a[5]);
    p.peer_delta = arg_ptr<const long long>(a[6]);
    p.status = arg_ptr<int>(a[7]);
    p.ae = arg_ptr<const uint8_t>(a[8]);
    if (A4) {
        p.asc = arg_ptr<const uint8_t>(a[9]);
    } else {
        p.ao = arg_ptr<const uint8_t>(a[9]);
        p.asc = arg_ptr<const uint8_t>(a[10]);
        p.asu = arg_ptr<const uint8_t>(a[11]);
    }
    FM_REQUIRE(p.K == 5120, kn, "K=%d: the fused stream is built for K = 5120 only; launch the per-layer kernels", p.K);
    FM_REQUIRE(p.nlayers >= 0 && p.rows > 0 && p.row_base >= 0 && p.npeers >= 0 && p.npeers <= 8, kn,
               "bad nlayers/rows/row_base/npeers");
    if (p.nlayers == 0) return FM_OK;
    FM_REQUIRE(aligned(p.layers, 8) && aligned(p.status, 4), kn, "misaligned layer table or status");
    FM_RANGE(p.layers, (size_t)p.nlayers * sizeof(StreamLayer), kn, "layers");
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d "
               "(or was overwritten since), or the peer offsets do not come from fm_stream_peers for its outputs",
               (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.asc, 16) && (A4 || (aligned(p.ao, 16) && aligned(p.asu, 16))), kn,
               "the activation code arrays must be 16-byte aligned");
    FM_RANGE(p.ae, (size_t)p.nlayers * (p.K / 2), kn, A4 ? "aq" : "ae");
    FM_RANGE(p.asc, (size_t)p.nlayers * (p.K / (A4 ? 32 : 128)) * 4, kn, "asc");
    if (!A4) {
        FM_RANGE(p.ao, (size_t)p.nlayers * (p.K / 2), kn, "ao");
        FM_RANGE(p.asu, (size_t)p.nlayers * (p.K / 128) * 4, kn, "asu");
    }
    // consumer: W4A8 defaults to the tensor-core variant; $FM_STREAM_CFG=1 (and W4A4 always) takes
    // the dp4a consumer.  Both keep 16 rows x 5 stages = 211 KB in flight per SM and give the same bits.
    static const int cfg = getenv("FM_STREAM_CFG") ? atoi(getenv("FM_STREAM_CFG")) : 0;
    if (!A4 && cfg != 1) return run_stream_mma<5>(kn, c, p);
    return run_stream<A4, 5, 16, 5>(kn, c, p);
}

// ------------------------------------------------------------------------------------
// NVFP4 (E2M1 weights, E4M3 scale per 16 weights, f32 global scale, int8 activations per 16-block;
// reference kernels/asm/k_nvfp4/011_*.s): the same ring with the arithmetic of nvfp4_gemv<1,1> —
// identical integers per block, identical fp32 association — so both give the same bits.
// A stage is 12 rows of 2560 packed bytes + 320 scale bytes; the code tile of a layer holds the
// even / odd int8 streams and the 320 block scales of the token (nvfp4_quant_act's outputs),
// re-interleaved into natural k order in registers once per layer.
struct Nvfp4StreamParams {
    StreamParams s;                    // layers[].ws are E4M3 bytes [rows][K/16]; s.ae = even codes, s.ao = odd codes, s.asc = scales
    float gscale;
};

template <int CW, int STAGES>
__global__ void __launch_bounds__((CW + 2) * 32, 1)
nvfp4_stream_kernel(const Nvfp4StreamParams pp) {
    const StreamParams& p = pp.s;
    constexpr int K = 5120, KITER = 5, NB = K / 16;
    constexpr int ROWB = K / 2, SCB = NB;
    constexpr int STAGE_W = CW * ROWB, STAGE = STAGE_W + CW * SCB;
    constexpr int ACT = K + NB * 4;                      // even codes, odd codes, block scales
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + STAGES;
    uint64_t* act_ready = empty + STAGES;
    uint64_t* act_free = act_ready + 2;
    uint64_t* ydone = act_free + 2;
    uint64_t* yfree = ydone + 2;
    uint8_t* ring = smem + 256;
    uint8_t* act = ring + (size_t)STAGES * STAGE;
    float* ytile = reinterpret_cast<float*>(act + 2 * ACT);   // [2][kOutCap]
    float* s_lut = ytile + 2 * kOutCap;                       // [256] 0.5 * gscale * E4M3(byte)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&act_ready[b], 1);
            mbar_init(&act_free[b], CW);
            mbar_init(&ydone[b], CW);
            mbar_init(&yfree[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < 256; i += blockDim.x) s_lut[i] = (0.5f * pp.gscale) * e4m3_to_f32(i);
    __syncthreads();
    pdl_wait();

    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int nst = (r1 - r0 + CW - 1) / CW;
    const bool tiled = (r1 - r0) <= kOutCap;

    if (warp == CW) {
        if (lane == 0) {                                   // producer
            auto copy_codes = [&](int l) -> bool {
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(&act_free[b], ((l >> 1) & 1) ^ 1, p.status, 4)) return false;
                uint8_t* ab = act + (size_t)b * ACT;
                mbar_expect_tx(&act_ready[b], ACT);
                bulk_g2s(ab, p.ae + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                bulk_g2s(ab + K / 2, p.ao + (size_t)l * (K / 2), K / 2, &act_ready[b]);
                bulk_g2s(ab + K, p.asc + (size_t)l * (NB * 4), NB * 4, &act_ready[b]);
                return true;
            };
            int c = 0;
            const uint8_t* wq = p.layers[0].wq;
            const uint8_t* ws = p.layers[0].ws;
            if (!copy_codes(0)) return;
            for (int l = 0; l < p.nlayers; l++) {
                const int ln = min(l + 1, p.nlayers - 1);
                const uint8_t* wq_n = p.layers[ln].wq;
                const uint8_t* ws_n = p.layers[ln].ws;
                for (int j = 0; j < nst; j++, c++) {
                    const int s = c % STAGES;
                    if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) & 1) ^ 1, p.status, 1)) return;
                    const int row = r0 + j * CW;
                    const int nr = min(CW, r1 - row);
                    uint8_t* dst = ring + (size_t)s * STAGE;
                    mbar_expect_tx(&full[s], (uint32_t)(nr * (ROWB + SCB)));
                    bulk_g2s(dst, wq + (size_t)row * ROWB, (uint32_t)(nr * ROWB), &full[s]);
                    bulk_g2s(dst + STAGE_W, ws + (size_t)row * SCB, (uint32_t)(nr * SCB), &full[s]);
                    if (j == 0 && l + 1 < p.nlayers && !copy_codes(l + 1)) return;
                }
                wq = wq_n;
                ws = ws_n;
            }
        }
        return;
    }

    if (warp == CW + 1) {                                    // writer
        if (!tiled) return;
        for (int l = 0; l < p.nlayers; l++) {
            if (!mbar_wait(&ydone[l & 1], (l >> 1) & 1, p.status, 8)) return;
            write_out(p, ytile + (l & 1) * kOutCap, p.layers[l].y + p.row_base + r0, r1 - r0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&yfree[l & 1]);
        }
        if (p.npeers) __threadfence_system();
        return;
    }

    // ---------------------------------------------------------------- consumers: warp w takes row w of a stage
    int c = 0;
    for (int l = 0; l < p.nlayers; l++) {
        const uint8_t* ab = act + (size_t)(l & 1) * ACT;
        float* yt = ytile + (l & 1) * kOutCap;
        if (tiled && l >= 2 && !mbar_wait(&yfree[l & 1], ((l >> 1) & 1) ^ 1, p.status, 7)) return;
        if (!mbar_wait(&act_ready[l & 1], (l >> 1) & 1, p.status, 2)) return;
        uint4 a0[KITER], a1[KITER];                        // the token's codes of this lane's 32 k per step, natural order
        float2 asc[KITER];                                 // and the scales of its two 16-blocks
#pragma unroll
        for (int it = 0; it < KITER; it++) {
            const int d0 = it * 128 + lane * 4;
            const uint4 e = *reinterpret_cast<const uint4*>(ab + d0 * 4), o = *reinterpret_cast<const uint4*>(ab + K / 2 + d0 * 4);
            a0[it] = make_uint4(prmt(e.x, o.x, 0x5140u), prmt(e.x, o.x, 0x7362u), prmt(e.y, o.y, 0x5140u), prmt(e.y, o.y, 0x7362u));
            a1[it] = make_uint4(prmt(e.z, o.z, 0x5140u), prmt(e.z, o.z, 0x7362u), prmt(e.w, o.w, 0x5140u), prmt(e.w, o.w, 0x7362u));
            asc[it] = *reinterpret_cast<const float2*>(ab + K + (d0 >> 1) * 4);
        }
        float* y = p.layers[l].y + p.row_base;

        for (int j = 0; j < nst; j++, c++) {
            const int s = c % STAGES;
            if (!mbar_wait(&full[s], (c / STAGES) & 1, p.status, 3)) return;
            const int row = r0 + j * CW + warp;
            const bool live = row < r1;
            const uint8_t* st = ring + (size_t)s * STAGE;
            float acc = 0.f;
            if (live) {
                const uint4* wrow = reinterpret_cast<const uint4*>(st + (size_t)warp * ROWB);
                const uint8_t* srow = st + STAGE_W + (size_t)warp * SCB;
                uint4 w[KITER];
                uint32_t sb[KITER];
#pragma unroll
                for (int it = 0; it < KITER; it++) {
                    w[it] = wrow[it * 32 + lane];
                    sb[it] = *reinterpret_cast<const unsigned short*>(srow + ((it * 128 + lane * 4) >> 1));
                }
#pragma unroll
                for (int it = 0; it < KITER; it++) {
                    int i0 = dot8_e2m1(w[it].x, a0[it].x, a0[it].y, 0);
                    i0 = dot8_e2m1(w[it].y, a0[it].z, a0[it].w, i0);
                    int i1 = dot8_e2m1(w[it].z, a1[it].x, a1[it].y, 0);
                    i1 = dot8_e2m1(w[it].w, a1[it].z, a1[it].w, i1);
                    acc = fmaf((float)i0, s_lut[sb[it] & 0xFFu] * asc[it].x, acc);
                    acc = fmaf((float)i1, s_lut[(sb[it] >> 8) & 0xFFu] * asc[it].y, acc);
                }
            }
            consumed(acc);                                  // release only after the loaded data has been used
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                if (j == 0) mbar_arrive(&act_free[l & 1]);
            }
            if (!live) continue;
            acc = warp_sum(acc);
            if (lane == 0) {
                if (tiled) {
                    yt[row - r0] = acc;
                } else {
                    y[row] = acc;
                    for (int q = 0; q < p.npeers; q++)
                        *reinterpret_cast<float*>(reinterpret_cast<char*>(y + row) + p.peer_delta[q]) = acc;
                }
            }
        }
        if (tiled) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ydone[l & 1]);
        }
    }
    if (p.npeers) __threadfence_system();
}

// nvfp4_decode_stream(layers, nlayers, rows, K, row_base, npeers, peer_delta, status, qa, qb, sc, gscale):
// the layer table's ws entries are the E4M3 block scales [rows][K/16] (the table must have been validated
// with room for them: fm_stream_table records how many bytes follow every ws pointer inside its allocation);
// qa / qb / sc are nvfp4_quant_act's outputs for all layers: [nlayers][K/2], [nlayers][K/2], [nlayers][K/16].
int launch_nvfp4_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "nvfp4_decode_stream";
    Nvfp4StreamParams pp = {};
    StreamParams& p = pp.s;
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.nlayers = arg_i32(a[1]);
    p.rows = arg_i32(a[2]);
    p.K = arg_i32(a[3]);
    p.row_base = arg_i32(a[4]);
    p.npeers = arg_i32(a[5]);
    p.peer_delta = arg_ptr<const long long>(a[6]);
    p.status = arg_ptr<int>(a[7]);
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    pp.gscale = arg_f32(a[11]);
    FM_REQUIRE(p.K == 5120, kn, "K=%d: the fused stream is built for K = 5120 only; launch the per-layer kernels", p.K);
    FM_REQUIRE(p.nlayers >= 0 && p.rows > 0 && p.row_base >= 0 && p.npeers >= 0 && p.npeers <= 8, kn,
               "bad nlayers/rows/row_base/npeers");
    if (p.nlayers == 0) return FM_OK;
    FM_REQUIRE(aligned(p.layers, 8) && aligned(p.status, 4), kn, "misaligned layer table or status");
    FM_RANGE(p.layers, (size_t)p.nlayers * sizeof(StreamLayer), kn, "layers");
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers, false,
                               (size_t)p.rows * (p.K / 16)), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d (or was "
               "overwritten since), a ws entry has fewer than rows*K/16 bytes behind it, or the peer offsets do not come "
               "from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.ao, 16) && aligned(p.asc, 16), kn, "the activation code arrays must be 16-byte aligned");
    FM_RANGE(p.ae, (size_t)p.nlayers * (p.K / 2), kn, "qa");
    FM_RANGE(p.ao, (size_t)p.nlayers * (p.K / 2), kn, "qb");
    FM_RANGE(p.asc, (size_t)p.nlayers * (p.K / 16) * 4, kn, "sc");
    constexpr int CW = 12, STAGES = 5, K = 5120;
    constexpr size_t smem = 256 + (size_t)STAGES * CW * (K / 2 + K / 16) + 2 * (K + (K / 16) * 4) + 2 * kOutCap * 4 + 1024;
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = nvfp4_stream_kernel<CW, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > p.rows) grid = p.rows;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3((CW + 2) * 32), smem, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// ------------------------------------------------------------------------------------
// W4A16 (compressed-tensors INT4: offset-binary codes, bf16 scale per 128 weights, fp32 activations;
// reference tools/gen_int4_dot.py:88-147): the ring with the tensor-core arithmetic of int4_dot_k.
// The fp32 activations of every layer are split once, by a small kernel in front, into three bf16
// terms laid out as the B fragments of mma.sync m16n8k16 (30 720 bytes per layer); the code tile of
// a layer is that fragment array.  8 consumer warps take 5 of the 40 blocks each: two codes per PRMT
// into 0x43xx halves (128 + code), one packed subtract of 136, eight MMAs per block; columns 0..2
// of the accumulator are the three terms, their sum times the block's bf16 scale is the block's
// contribution, and the per-warp sums meet in the shared tile as in the int8 kernel.
__global__ void __launch_bounds__(256)
w4a16_split_layers_kernel(const StreamLayer* __restrict__ layers, uint32_t* __restrict__ out, uint32_t nbpr) {
    pdl_wait();
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < nbpr * 192) {
        const uint32_t e = idx & 15, t = (idx >> 4) & 3, term = (idx >> 6) % 3, b = idx / 192;
        const uint32_t q = e >> 2, h = (e >> 1) & 1, i = e & 1;
        const float* xs = layers[blockIdx.y].x + (size_t)b * 128 + t * 32 + 8 * q + 4 * i + h;
        out[(size_t)blockIdx.y * nbpr * 192 + idx] = bf16_term(xs[0], (int)term) | (bf16_term(xs[2], (int)term) << 16);
    }
}

struct W4a16StreamParams {
    StreamParams s;                    // layers[].wq offset-binary codes, layers[].ws bf16 scales [rows][K/128]
    const uint32_t* frags;             // [nlayers][40 * 192] B fragments of the activations
};

template <int STAGES>
__global__ void __launch_bounds__(10 * 32, 1)
w4a16_stream_kernel(const W4a16StreamParams pp) {
    const StreamParams& p = pp.s;
    constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;
    constexpr int ROWB = K / 2, SCB = NG * 2;
    constexpr int STAGE_W = ROWS * ROWB, STAGE = STAGE_W + ROWS * SCB;
    constexpr int ACT = NG * 192 * 4;                    // fragment array of one layer
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + STAGES;
    uint64_t* act_ready = empty + STAGES;
    uint64_t* act_free = act_ready + 2;
    uint64_t* red_full = act_free + 2;
    uint64_t* red_free = red_full + 2;
    uint64_t* ydone = red_free + 2;
    uint64_t* yfree = ydone + 2;
    uint8_t* ring = smem + 256;
    uint8_t* act = ring + (size_t)STAGES * STAGE;
    float* red = reinterpret_cast<float*>(act + 2 * ACT);             // [2][CW][ROWS]
    float* ytile = red + 2 * CW * ROWS;                               // [2][kOutCap]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CW);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(&act_ready[b], 1);
            mbar_init(&act_free[b], CW);
            mbar_init(&red_full[b], CW);
            mbar_init(&red_free[b], 1);
            mbar_init(&ydone[b], CW);
            mbar_init(&yfree[b], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();

    const int r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    const int r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    const int nst = (r1 - r0 + ROWS - 1) / ROWS;
    const bool tiled = (r1 - r0) <= kOutCap;

    if (warp == CW) {
        if (lane == 0) {                                   // producer
            auto copy_frags = [&](int l) -> bool {
                const int b = l & 1;
                if (l >= 2 && !mbar_wait(&act_free[b], ((l >> 1) & 1) ^ 1, p.status, 4)) return false;
                mbar_expect_tx(&act_ready[b], ACT);
                bulk_g2s(act + (size_t)b * ACT, pp.frags + (size_t)l * (NG * 192), ACT, &act_ready[b]);
                return true;
            };
            int c = 0;
            const uint8_t* wq = p.layers[0].wq;
            const uint8_t* ws = p.layers[0].ws;
            if (!copy_frags(0)) return;
            for (int l = 0; l < p.nlayers; l++) {
                const int ln = min(l + 1, p.nlayers - 1);
                const uint8_t* wq_n = p.layers[ln].wq;
                const uint8_t* ws_n = p.layers[ln].ws;
                for (int j = 0; j < nst; j++, c++) {
                    const int s = c % STAGES;
                    if (c >= STAGES && !mbar_wait(&empty[s], ((c / STAGES) & 1) ^ 1, p.status, 1)) return;
                    const int row = r0 + j * ROWS;
                    const int nr = min(ROWS, r1 - row);
                    uint8_t* dst = ring + (size_t)s * STAGE;
                    mbar_expect_tx(&full[s], (uint32_t)(nr * (ROWB + SCB)));
                    bulk_g2s(dst, wq + (size_t)row * ROWB, (uint32_t)(nr * ROWB), &full[s]);
                    bulk_g2s(dst + STAGE_W, ws + (size_t)row * SCB, (uint32_t)(nr * SCB), &full[s]);
                    if (j == 0 && l + 1 < p.nlayers && !copy_frags(l + 1)) return;
                }
                wq = wq_n;
                ws = ws_n;
            }
        }
        return;
    }

    if (warp == CW + 1) {                                    // writer
        if (!tiled) return;
        for (int l = 0; l < p.nlayers; l++) {
            if (!mbar_wait(&ydone[l & 1], (l >> 1) & 1, p.status, 8)) return;
            write_out(p, ytile + (l & 1) * kOutCap, p.layers[l].y + p.row_base + r0, r1 - r0, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&yfree[l & 1]);
        }
        if (p.npeers) __threadfence_system();
        return;
    }

    // ---------------------------------------------------------------- consumers
    const int g = lane >> 2, t = lane & 3;
    int c = 0;
    for (int l = 0; l < p.nlayers; l++) {
        const uint32_t* ft = reinterpret_cast<const uint32_t*>(act + (size_t)(l & 1) * ACT);
        float* yt = ytile + (l & 1) * kOutCap;
        if (tiled && l >= 2 && !mbar_wait(&yfree[l & 1], ((l >> 1) & 1) ^ 1, p.status, 7)) return;
        if (!mbar_wait(&act_ready[l & 1], (l >> 1) & 1, p.status, 2)) return;
        uint4 bf[GPW][4];                                  // B fragments of this warp's blocks: {b0,b1 of (q,0), b0,b1 of (q,1)}
#pragma unroll
        for (int j = 0; j < GPW; j++) {
            const int b = j * CW + warp;
            const uint4* fp = reinterpret_cast<const uint4*>(ft + ((size_t)(b * 3 + (g < 3 ? g : 0)) * 4 + t) * 16);
#pragma unroll
            for (int q = 0; q < 4; q++) bf[j][q] = g < 3 ? fp[q] : make_uint4(0, 0, 0, 0);
        }
        float* y = p.layers[l].y + p.row_base;

        for (int jst = 0; jst < nst; jst++, c++) {
            const int s = c % STAGES;
            if (!mbar_wait(&full[s], (c / STAGES) & 1, p.status, 3)) return;
            const uint8_t* st = ring + (size_t)s * STAGE;
            uint4 xa[GPW], xb[GPW];
            float swa[GPW], swb[GPW];
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                const int b = j * CW + warp;
                xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * ROWB + b * 64 + t * 16);
                xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * ROWB + b * 64 + t * 16);
                swa[j] = __uint_as_float((uint32_t)*reinterpret_cast<const unsigned short*>(st + STAGE_W + g * SCB + b * 2) << 16);
                swb[j] = __uint_as_float((uint32_t)*reinterpret_cast<const unsigned short*>(st + STAGE_W + (g + 8) * SCB + b * 2) << 16);
            }
            float fa = 0.f, fb = 0.f;
#pragma unroll
            for (int j = 0; j < GPW; j++) {
                const uint32_t wav[4] = {xa[j].x, xa[j].y, xa[j].z, xa[j].w}, wbv[4] = {xb[j].x, xb[j].y, xb[j].z, xb[j].w};
                float cc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t la = wav[q] & 0x0F0F0F0Fu, ha = (wav[q] >> 4) & 0x0F0F0F0Fu;
                    const uint32_t lb = wbv[q] & 0x0F0F0F0Fu, hb = (wbv[q] >> 4) & 0x0F0F0F0Fu;
                    const uint32_t m = 0x43434343u;
                    mma_bf16(cc, bf16x2_sub136(prmt(la, m, 0x5140u)), bf16x2_sub136(prmt(lb, m, 0x5140u)),
                             bf16x2_sub136(prmt(la, m, 0x5342u)), bf16x2_sub136(prmt(lb, m, 0x5342u)), bf[j][q].x, bf[j][q].y);
                    mma_bf16(cc, bf16x2_sub136(prmt(ha, m, 0x5140u)), bf16x2_sub136(prmt(hb, m, 0x5140u)),
                             bf16x2_sub136(prmt(ha, m, 0x5342u)), bf16x2_sub136(prmt(hb, m, 0x5342u)), bf[j][q].z, bf[j][q].w);
                }
                // columns 0, 1 (lane t = 0) and 2 (lane t = 1) hold the three terms: smallest first
                const float va = __shfl_down_sync(0xffffffffu, cc[0], 1), vb = __shfl_down_sync(0xffffffffu, cc[2], 1);
                fa += swa[j] * ((va + cc[1]) + cc[0]);
                fb += swb[j] * ((vb + cc[3]) + cc[2]);
            }
            consumed(fa + fb);                              // release only after the loaded data has been used
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&empty[s]);
                if (jst == 0) mbar_arrive(&act_free[l & 1]);
            }
            const int rb = c & 1;
            if (c >= 2 && !mbar_wait(&red_free[rb], ((c >> 1) & 1) ^ 1, p.status, 5)) return;
            if (t == 0) {
                red[(rb * CW + warp) * ROWS + g] = fa;
                red[(rb * CW + warp) * ROWS + g + 8] = fb;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_full[rb]);
            if (warp == (c % CW)) {
                if (!mbar_wait(&red_full[rb], (c >> 1) & 1, p.status, 6)) return;
                const int row = r0 + jst * ROWS + lane;
                float acc = 0.f;
                if (lane < ROWS) {
                    const float* pr = red + rb * CW * ROWS + lane;
                    acc = ((pr[0 * ROWS] + pr[4 * ROWS]) + (pr[2 * ROWS] + pr[6 * ROWS])) +
                          ((pr[1 * ROWS] + pr[5 * ROWS]) + (pr[3 * ROWS] + pr[7 * ROWS]));
                }
                consumed(acc);
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_free[rb]);
                if (lane < ROWS && row < r1) {
                    if (tiled) {
                        yt[row - r0] = acc;
                    } else {
                        y[row] = acc;
                        for (int q = 0; q < p.npeers; q++)
                            *reinterpret_cast<float*>(reinterpret_cast<char*>(y + row) + p.peer_delta[q]) = acc;
                    }
                }
            }
        }
        if (tiled) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&ydone[l & 1]);
        }
    }
    if (p.npeers) __threadfence_system();
}

// w4a16_decode_stream(layers, nlayers, rows, K, row_base, npeers, peer_delta, status): the table's x entries
// (fp32 activations [K] per layer) are read here — fm_stream_table must have seen a valid x for every layer —,
// wq are compressed-tensors codes, ws bf16 scales.  Launches the split kernel (grid y = layer) into the engine
// workspace (30 720 bytes per layer), then the stream kernel.
int launch_w4a16_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "w4a16_decode_stream";
    W4a16StreamParams pp = {};
    StreamParams& p = pp.s;
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.nlayers = arg_i32(a[1]);
    p.rows = arg_i32(a[2]);
    p.K = arg_i32(a[3]);
    p.row_base = arg_i32(a[4]);
    p.npeers = arg_i32(a[5]);
    p.peer_delta = arg_ptr<const long long>(a[6]);
    p.status = arg_ptr<int>(a[7]);
    FM_REQUIRE(p.K == 5120, kn, "K=%d: the fused stream is built for K = 5120 only; launch the per-layer kernels", p.K);
    FM_REQUIRE(p.nlayers >= 0 && p.rows > 0 && p.row_base >= 0 && p.npeers >= 0 && p.npeers <= 8, kn,
               "bad nlayers/rows/row_base/npeers");
    if (p.nlayers == 0) return FM_OK;
    FM_REQUIRE(aligned(p.layers, 8) && aligned(p.status, 4), kn, "misaligned layer table or status");
    FM_RANGE(p.layers, (size_t)p.nlayers * sizeof(StreamLayer), kn, "layers");
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers, false, 0, true), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d (or was "
               "overwritten since), an x entry is missing, or the peer offsets do not come from fm_stream_peers for its "
               "outputs", (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    constexpr int NG = 40;
    uint32_t* frags = static_cast<uint32_t*>(engine_scratch((size_t)p.nlayers * NG * 192 * 4));
    FM_REQUIRE(frags != nullptr, kn, "the engine workspace cannot hold %d x 30720 bytes here (FM_SCRATCH_MB, or a first use "
               "inside a graph capture)", p.nlayers);
    pp.frags = frags;
    cudaError_t e = launch_kernel(w4a16_split_layers_kernel, dim3((NG * 192 + 255) / 256, p.nlayers), dim3(256), 0, c.stream,
                                  pdl_enabled(), p.layers, frags, (uint32_t)NG);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    after_launch(kn);
    constexpr int STAGES = 3, K = 5120;
    constexpr size_t smem = 256 + (size_t)STAGES * 16 * (K / 2 + 80) + 2 * (NG * 192 * 4) + 2 * 8 * 16 * 4 + 2 * kOutCap * 4;
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = w4a16_stream_kernel<STAGES>;
    static bool configured = false;
    if (!configured) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > p.rows) grid = p.rows;
    e = launch_kernel(kern, dim3(grid), dim3(10 * 32), smem, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// w4a8_decode_stream_m(layers, nlayers, rows, K, row_base, npeers, peer_delta, status, ae, ao, asc, asu, M, ystride):
// M = 2..4 tokens per layer.  The code arrays hold [nlayers * M] tokens (one 2-D quant_act launch with grid
// y = nlayers * M over x[nlayers][M][K]); y of a layer is token-major, y[token * ystride + row_base + row].  The
// layer table must have been validated by fm_stream_table with row_base + (M - 1) * ystride as its row_base
// argument, which is what makes every token's rows lie inside the checked footprint of y.
int launch_w4a8_stream_m(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "w4a8_decode_stream_m";
    StreamParams p = {};
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.nlayers = arg_i32(a[1]);
    p.rows = arg_i32(a[2]);
    p.K = arg_i32(a[3]);
    p.row_base = arg_i32(a[4]);
    p.npeers = arg_i32(a[5]);
    p.peer_delta = arg_ptr<const long long>(a[6]);
    p.status = arg_ptr<int>(a[7]);
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    p.asu = arg_ptr<const uint8_t>(a[11]);
    p.M = arg_i32(a[12]);
    p.ystride = arg_i32(a[13]);
    FM_REQUIRE(p.K == 5120, kn, "K=%d: the fused stream is built for K = 5120 only; launch the per-layer kernels", p.K);
    FM_REQUIRE(p.M >= 2 && p.M <= 4, kn, "M=%d: this kernel takes 2..4 tokens (w4a8_decode_stream takes one)", p.M);
    FM_REQUIRE(p.nlayers >= 0 && p.rows > 0 && p.row_base >= 0 && p.npeers >= 0 && p.npeers <= 8, kn,
               "bad nlayers/rows/row_base/npeers");
    FM_REQUIRE(p.ystride >= p.row_base + p.rows && (long long)(p.M - 1) * p.ystride + p.row_base < (1LL << 31), kn,
               "ystride=%d must be at least row_base + rows = %d", p.ystride, p.row_base + p.rows);
    if (p.nlayers == 0) return FM_OK;
    FM_REQUIRE(aligned(p.layers, 8) && aligned(p.status, 4), kn, "misaligned layer table or status");
    FM_RANGE(p.layers, (size_t)p.nlayers * sizeof(StreamLayer), kn, "layers");
    const int vbase = p.row_base + (p.M - 1) * p.ystride;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, vbase, p.peer_delta, p.npeers, true), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d and the row_base "
               "argument row_base + (M - 1) * ystride = %d (or was overwritten since), or the peer offsets do not come "
               "from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers, p.rows, p.K, vbase);
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.asc, 16) && aligned(p.ao, 16) && aligned(p.asu, 16), kn,
               "the activation code arrays must be 16-byte aligned");
    const size_t tokens = (size_t)p.nlayers * p.M;
    FM_RANGE(p.ae, tokens * (p.K / 2), kn, "ae");
    FM_RANGE(p.ao, tokens * (p.K / 2), kn, "ao");
    FM_RANGE(p.asc, tokens * (p.K / 128) * 4, kn, "asc");
    FM_RANGE(p.asu, tokens * (p.K / 128) * 4, kn, "asu");
    switch (p.M) {
        case 2: return run_stream_mma_m<4, 2>(kn, c, p);
        case 3: return run_stream_mma_m<4, 3>(kn, c, p);
        default: return run_stream_mma_m<4, 4>(kn, c, p);
    }
}

const KernelEntry kStream[] = {
    {"w4a8_decode_stream", 12, launch_w4_stream<false>, "piiiiipppppp"},
    {"w4a4_decode_stream", 10, launch_w4_stream<true>, "piiiiipppp"},
    {"w4a8_decode_stream_m", 14, launch_w4a8_stream_m, "piiiiippppppii"},
    {"nvfp4_decode_stream", 12, launch_nvfp4_stream, "piiiiipppppf"},
    {"w4a16_decode_stream", 8, launch_w4a16_stream, "piiiiipp"},
};

}  // namespace

const KernelEntry* stream_kernels(int* n) {
    *n = (int)(sizeof(kStream) / sizeof(kStream[0]));
    return kStream;
}

}  // namespace fm
