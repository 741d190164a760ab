// w4a8_decode_stream / w4a4_decode_stream / w4a8_decode_stream_m / nvfp4_decode_stream / w4a16_decode_stream:
// one launch for the GEMVs of a whole stack of independent decode layers, software-pipelined across
// layers so that HBM never idles at a layer boundary.  The activation codes of all layers come from one
// 2-D launch of the ordinary quantiser kernel (grid y = layer) that precedes it.
//
// The reference streams its 400-layer decode benchmark as 800 back-to-back launches on one in-order
// queue (tools/bench_decode.py:272-317).  On B200 one 17408 x 5120 layer is ~6.5 us of HBM time, the
// same order as a kernel's launch, ramp-up and drain, so the per-layer launches (which stay available by
// name) leave a quarter of the bandwidth unused.  These kernels keep the arithmetic of the per-layer
// kernels — identical integer accumulators, fp32 afterwards — and change only the schedule; the roles
// of the warps, the ring and the barriers are in stream_common.cuh, this file holds what differs per
// quantisation format (the "policies") and the by-name launchers.
//
// Layers must be independent of each other (no layer reads another layer's y): the kernels order nothing
// between layers.  A caller that consumes a layer's gathered y while later layers still stream passes a
// flags array: every CTA adds one to flags[layer] on every receiver once its rows of that layer are
// visible there, and stream_flag_wait (below) or a host poll of a pinned copy acquires them.
#include <cuda_fp16.h>
#include <stdlib.h>

#include "fm_internal.h"
#include "stream_common.cuh"

namespace fm {
namespace {

using namespace stream;

__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// D = A * B (no accumulator input: the first MMA of a chain needs no zeroed registers)
__device__ __forceinline__ void mma_s8_first(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
struct PlainParams {
    StreamParams s;
};

// Partial sums of the tensor-core consumers.  The CW warps of a group each hold, for the 16 rows of a
// stage, the sum over their own share of K; they meet in a small shared tile (two per group, alternating)
// and one warp per stage (rotating) adds them in the fixed order ((p0+p4)+(p2+p6)) + ((p1+p5)+(p3+p7)) —
// the association of a warp's lane partials under an xor butterfly, so the tensor-core and the dp4a
// kernels give the same bits — and emits the y values.  `vals` are this lane's partials, `idx` their
// positions inside the tile of ROWS * M values (negative: none).
template <class P, int NV>
__device__ __forceinline__ bool reduce_and_emit(const Cta& c, int grp, int w, int cg, const float (&vals)[NV],
                                                const int (&idx)[NV], float* yt, float* y, int row0) {
    constexpr int CW = P::CW, W = P::ROWS * P::M;
    static_assert(CW == 8, "the reduction tree is written for eight warps");
    const int rb = grp * 2 + (cg & 1);
    if (cg >= 2 && !cta_wait(c, &c.bars->red_free[rb], ((cg >> 1) & 1) ^ 1, 5)) return false;
    float* rw = c.red + ((size_t)rb * CW + w) * W;
#pragma unroll
    for (int i = 0; i < NV; i++)
        if (idx[i] >= 0) rw[idx[i]] = vals[i];
    __syncwarp();
    if (c.lane == 0) mbar_arrive(&c.bars->red_full[rb]);
    if (w == (cg % CW)) {                              // this stage's reducer
        if (!cta_wait(c, &c.bars->red_full[rb], (cg >> 1) & 1, 6)) return false;
        constexpr int NK = (W + 31) / 32;
        float acc[NK];
#pragma unroll
        for (int k = 0; k < NK; k++) {
            const int i = k * 32 + c.lane;
            acc[k] = 0.f;
            if (i < W) {
                const float* pr = c.red + (size_t)rb * CW * W + i;
                acc[k] = ((pr[0 * W] + pr[4 * W]) + (pr[2 * W] + pr[6 * W])) + ((pr[1 * W] + pr[5 * W]) + (pr[3 * W] + pr[7 * W]));
            }
            consumed(acc[k]);                          // read before the tile is released
        }
        __syncwarp();
        if (c.lane == 0) mbar_arrive(&c.bars->red_free[rb]);
#pragma unroll
        for (int k = 0; k < NK; k++) {
            const int i = k * 32 + c.lane;
            const int rr = i / P::M, tok = i - rr * P::M, row = row0 + rr;
            if (i < W && row < c.r1) emit<P::M>(c, yt, y, row, tok, acc[k]);
        }
    }
    return true;
}

// ------------------------------------------------------------------------------------
// W4A8 on the tensor cores (reference arithmetic: kernels/gemv_w4a8_core.h:76-219).  A stage of 16
// weight rows is one m16 tile: each of the 8 warps of a group takes 5 of the 40 groups of all 16 rows and
// multiplies them with mma.sync m16n8k32 (int8 x int8 -> int32; the tokens are the columns of B).
// Per packed word only the two nibble masks remain: low nibbles as bytes u = n ^ 8 (signed operand),
// high nibbles in place as unsigned bytes 16*u (the u8 x s8 form), two accumulators,
//   I[n,g] = acc_lo + (acc_hi >> 4) - 8 * sum(q)        exactly, no shuffles,
// because the MMA itself adds over the four lanes that share a group.  Lane (g, t) feeds token
// min(g, M-1) as column g and owns rows g, g + 8 of tokens 2t, 2t + 1.
//   M       tokens per layer (1..4); the code tile of a layer is [M][K/2] even codes, [M][K/2] odd codes,
//           [M][NG] scales, [M][NG] sums — what a 2-D quant_act launch with grid y = layer * M + token leaves
//   NGROUPS consumer groups that take the stages in turn (2: a group has two stage times for its own stage)
//   AIS     the code tile travels inside every stage (no per-layer state at all) instead of in tiles of its own
//   BREG    (tiles of their own only) a warp keeps its B fragments of the layer in registers
//   PAD     bytes added to the pitch of a row inside a stage (64: the two rows of a quarter-warp's 16-byte
//           loads fall into different banks; the rows are then copied one by one)
//   DUMP    also store the integer accumulators
//   VAR     the layers have shapes of their own (StreamParams::var): rows per layer, row pitch, chunks of longer rows
//   ROT     whole stages are dealt out to the CTAs, from a position that moves with the layer (stream_common.cuh: var_rows)
template <int M_, int STAGES_, int NGROUPS_, bool AIS, int NACT_, bool BREG, int PAD, bool DUMP, int NPROD_ = 1, bool VAR_ = false,
          bool ROT_ = false>
struct W4A8Mma {
    using Params = PlainParams;
    static constexpr int M = M_, STAGES = STAGES_, NGROUPS = NGROUPS_, NACT = AIS ? 1 : NACT_;
    static constexpr bool ACT_IN_STAGE = AIS, VAR = VAR_, ROT = ROT_;
    static_assert(!VAR || (AIS && M_ == 1 && !DUMP && PAD == 0), "per-layer shapes: one token, codes inside the stage");
    static_assert(!ROT || (!VAR && !BREG), "moving row ranges: the shapes are the table's, no fragments held over a layer");
    static constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;
    static constexpr int ROWB = K / 2, SCB = NG * 2, PITCH = ROWB + PAD;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB;
    static constexpr int ACT = M * (K + NG * 8);
    static constexpr int STAGE = (OFF_ACT + (AIS ? ACT : 0) + 127) & ~127;
    static constexpr int RED = CW * ROWS * M, EXTRA = 0, NPROD = NPROD_;
    static constexpr int kThreads = (NGROUPS * CW + 1 + NPROD) * 32;
    static_assert(!(AIS && BREG), "fragments in registers need a tile that outlives the stage");

    __device__ static void init_extra(const Params&, uint8_t*) {}
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) {
        const StreamParams& p = pp.s;
        if (VAR) {                                       // the chunk's codes, by the layer's own pointers
            const VarLayer v = p.var[l];
            bulk_g2s(dst, v.ae, K / 2, bar);
            bulk_g2s(dst + K / 2, v.ao, K / 2, bar);
            bulk_g2s(dst + K, v.asc, NG * 4, bar);
            bulk_g2s(dst + K + NG * 4, v.asu, NG * 4, bar);
            return;
        }
        bulk_g2s(dst, p.ae + (size_t)l * M * (K / 2), M * (K / 2), bar);
        bulk_g2s(dst + M * (K / 2), p.ao + (size_t)l * M * (K / 2), M * (K / 2), bar);
        bulk_g2s(dst + M * K, p.asc + (size_t)l * M * (NG * 4), M * NG * 4, bar);
        bulk_g2s(dst + M * K + M * NG * 4, p.asu + (size_t)l * M * (NG * 4), M * NG * 4, bar);
    }

    struct Frag {                                        // B operand of one group for this lane
        uint4 be, bo;
        float sa0, sa1;
        int su0, su1;
    };
    __device__ static __forceinline__ Frag load_frag(const uint8_t* ab, int gg, int g, int t) {
        const int tk = g < M ? g : M - 1, t0 = 2 * t, t1 = 2 * t + 1;
        Frag f;
        f.be = *reinterpret_cast<const uint4*>(ab + tk * (K / 2) + (gg * 16 + 4 * t) * 4);
        f.bo = *reinterpret_cast<const uint4*>(ab + M * (K / 2) + tk * (K / 2) + (gg * 16 + 4 * t) * 4);
        const float* scp = reinterpret_cast<const float*>(ab + M * K);
        const int* sup = reinterpret_cast<const int*>(ab + M * K + M * NG * 4);
        f.sa0 = t0 < M ? scp[t0 * NG + gg] : 0.f;
        f.su0 = t0 < M ? 8 * sup[t0 * NG + gg] : 0;
        f.sa1 = (M > 1 && t1 < M) ? scp[t1 * NG + gg] : 0.f;
        f.su1 = (M > 1 && t1 < M) ? 8 * sup[t1 * NG + gg] : 0;
        return f;
    }

    __device__ static void consume(const Cta& cta, const Params& pp, int grp, int w) {
        Cta c = cta;                                     // (rows and stages of the CTA follow the layer when VAR)
        const StreamParams& p = pp.s;
        const int lane = c.lane, g = lane >> 2, t = lane & 3;
        const int t0 = 2 * t, t1 = 2 * t + 1;
        int cg = 0;                                      // stages this group has taken so far
        int c0 = 0;                                      // stages of the layers before this one
        for (int l = 0; l < p.nlayers; c0 += c.nst, l++) {
            set_geom<W4A8Mma>(c, l);
            // a short chunk (the end of a row that is no multiple of 5120 k) has fewer 128-groups: the others would
            // multiply zeros by zeros, so a warp skips them
            int ngr = NG;
            if (VAR) ngr = p.var[l].wbytes >> 6;
            const int jf = ((grp - c0) % NGROUPS + NGROUPS) % NGROUPS;     // this group's first stage of the layer
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + (VAR ? 0 : p.row_base);      // (VAR: always through the tile, the writer adds the base)
            if (!layer_enter<W4A8Mma>(c, l)) return;
            const uint8_t* tile = c.act + (size_t)(l % NACT) * ACT;
            Frag fr[BREG ? GPW : 1];
            bool held = false;                           // the tile has not been released yet
            if (BREG) {
                if (jf < c.nst) {
#pragma unroll
                    for (int j = 0; j < GPW; j++) fr[j] = load_frag(tile, j * CW + w, g, t);
                    held = true;
                } else {
                    act_release<W4A8Mma>(c, l);
                }
            }
            for (int jst = jf; jst < c.nst; jst += NGROUPS, cg++) {
                const int cc = c0 + jst, s = cc % STAGES;
                if (!stage_wait<W4A8Mma>(c, cc)) return;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                const uint8_t* ab = AIS ? st + OFF_ACT : tile;
                uint4 xa[GPW], xb[GPW];                  // packed words of rows g and g + 8
                float swa[GPW], swb[GPW];
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int gg = j * CW + w;           // this warp's groups: w, w + 8, ...
                    if (VAR && gg >= ngr) continue;
                    xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * PITCH + gg * 64 + t * 16);
                    xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * PITCH + gg * 64 + t * 16);
                    swa[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + g * SCB + gg * 2));
                    swb[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + (g + 8) * SCB + gg * 2));
                }
                float fa0 = 0.f, fa1 = 0.f, fb0 = 0.f, fb1 = 0.f;    // rows g, g + 8 x tokens t0, t1 over this warp's groups
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int gg = j * CW + w;
                    if (VAR && gg >= ngr) continue;
                    const Frag f = BREG ? fr[j] : load_frag(ab, gg, g, t);
                    int lo[4] = {0, 0, 0, 0}, hi[4] = {0, 0, 0, 0};
                    const uint32_t m_lo = 0x0F0F0F0Fu, x_lo = 0x08080808u, m_hi = 0xF0F0F0F0u, x_hi = 0x80808080u;
                    mma_s8(lo, (xa[j].x & m_lo) ^ x_lo, (xb[j].x & m_lo) ^ x_lo, (xa[j].y & m_lo) ^ x_lo, (xb[j].y & m_lo) ^ x_lo,
                           f.be.x, f.be.y);
                    mma_s8(lo, (xa[j].z & m_lo) ^ x_lo, (xb[j].z & m_lo) ^ x_lo, (xa[j].w & m_lo) ^ x_lo, (xb[j].w & m_lo) ^ x_lo,
                           f.be.z, f.be.w);
                    mma_u8(hi, (xa[j].x & m_hi) ^ x_hi, (xb[j].x & m_hi) ^ x_hi, (xa[j].y & m_hi) ^ x_hi, (xb[j].y & m_hi) ^ x_hi,
                           f.bo.x, f.bo.y);
                    mma_u8(hi, (xa[j].z & m_hi) ^ x_hi, (xb[j].z & m_hi) ^ x_hi, (xa[j].w & m_hi) ^ x_hi, (xb[j].w & m_hi) ^ x_hi,
                           f.bo.z, f.bo.w);
                    // accumulator columns 2t and 2t + 1 of this lane are tokens t0 and t1
                    const int ia0 = lo[0] + (hi[0] >> 4) - f.su0, ib0 = lo[2] + (hi[2] >> 4) - f.su0;
                    fa0 += (swa[j] * f.sa0) * (float)ia0;
                    fb0 += (swb[j] * f.sa0) * (float)ib0;
                    int ia1 = 0, ib1 = 0;
                    if (M > 1) {
                        ia1 = lo[1] + (hi[1] >> 4) - f.su1;
                        ib1 = lo[3] + (hi[3] >> 4) - f.su1;
                        fa1 += (swa[j] * f.sa1) * (float)ia1;
                        fb1 += (swb[j] * f.sa1) * (float)ib1;
                    }
                    if (DUMP) {
                        const int ra = c.r0 + jst * ROWS + g, rb = ra + 8;
                        int* d = p.iacc + (size_t)l * M * p.rows * NG + gg;
                        if (t0 < M && ra < c.r1) d[((size_t)t0 * p.rows + ra) * NG] = ia0;
                        if (t0 < M && rb < c.r1) d[((size_t)t0 * p.rows + rb) * NG] = ib0;
                        if (M > 1 && t1 < M && ra < c.r1) d[((size_t)t1 * p.rows + ra) * NG] = ia1;
                        if (M > 1 && t1 < M && rb < c.r1) d[((size_t)t1 * p.rows + rb) * NG] = ib1;
                    }
                }
                // Release only now: the MMAs and multiplies above have consumed every register loaded from
                // the stage (and from the code tile), so those loads have completed.  An arrive issued right
                // behind the loads can overtake them, and the refill would race with them.
                consumed((fa0 + fa1) + (fb0 + fb1));
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                if (BREG && held) {
                    act_release<W4A8Mma>(c, l);
                    held = false;
                }
                const float vals[4] = {fa0, fb0, fa1, fb1};
                const int idx[4] = {t0 < M ? g * M + t0 : -1, t0 < M ? (g + 8) * M + t0 : -1,
                                    (M > 1 && t1 < M) ? g * M + t1 : -1, (M > 1 && t1 < M) ? (g + 8) * M + t1 : -1};
                if (!reduce_and_emit<W4A8Mma>(c, grp, w, cg, vals, idx, yt, y, c.r0 + jst * ROWS)) return;
            }
            if (!BREG) act_release<W4A8Mma>(c, l);
            layer_done(c, l);
        }
    }
};

// ------------------------------------------------------------------------------------
// Read ceiling of the W4A8 stream: the producer, the ring, the stage geometry and the copies (weights, scales and the
// token's codes inside every stage) of the default W4A8 schedule, with consumers that release every stage as soon as it
// has landed — no shared-memory read, no arithmetic, no output.  What this kernel takes per token is what the memory
// system allows this access pattern; the distance of w4a8_decode_stream from it is what its arithmetic costs.
template <int STAGES_, int NPROD_, bool ROT_ = false>
struct W4A8ReadCeiling {
    using Params = PlainParams;
    using Base = W4A8Mma<1, STAGES_, 2, true, 1, false, 0, false, NPROD_>;
    static constexpr int M = 1, STAGES = STAGES_, NGROUPS = 2, NACT = 1;
    static constexpr bool ACT_IN_STAGE = true, NO_OUTPUT = true, ROT = ROT_;
    static constexpr int K = Base::K, NG = Base::NG, CW = Base::CW, ROWS = Base::ROWS;
    static constexpr int ROWB = Base::ROWB, SCB = Base::SCB, PITCH = Base::PITCH;
    static constexpr int STAGE_W = Base::STAGE_W, OFF_ACT = Base::OFF_ACT, ACT = Base::ACT, STAGE = Base::STAGE;
    static constexpr int RED = Base::RED, EXTRA = 0, NPROD = NPROD_;
    static constexpr int kThreads = Base::kThreads;

    __device__ static void init_extra(const Params&, uint8_t*) {}
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) { Base::copy_act(pp, l, dst, bar); }
    __device__ static void consume(const Cta& cta, const Params& pp, int grp, int w) {
        Cta c = cta;
        const StreamParams& p = pp.s;
        int c0 = 0;
        for (int l = 0; l < p.nlayers; c0 += c.nst, l++) {
            set_geom<W4A8ReadCeiling>(c, l);
            const int jf = ((grp - c0) % NGROUPS + NGROUPS) % NGROUPS;
            for (int jst = jf; jst < c.nst; jst += NGROUPS) {
                const int cc = c0 + jst, s = cc % STAGES;
                if (!stage_wait<W4A8ReadCeiling>(c, cc)) return;
                __syncwarp();
                if (c.lane == 0) mbar_arrive(&c.bars->empty[s]);
            }
        }
        (void)w;
    }
};

// ------------------------------------------------------------------------------------
// W4A4 on the tensor cores (reference arithmetic: kernels/gemv_w4a4_core.h:48-134): the schedule of W4A8Mma
// with the token's codes inside every stage and, per (row, 32-sub-group), the exact integer
//   J = sum_{k in sub-group} w[n,k] * q[k]         y += (f16(ws[n, sg / 4]) * asc[sg]) * float(J).
// A lane's 16-byte word is one sub-group, but an MMA adds over the k slots of all four lanes of a row; the
// sub-groups are kept apart by the columns of B: column 2t carries the token's codes only in the k slots that
// lane t feeds (zero elsewhere), so accumulator column 2t — which lane t owns — is lane t's own sub-group.
// Both operands are formed as 16 x their value with one or two logic instructions per register (a two's-
// complement nibble in the upper half of a byte is the signed byte 16 * v): J = acc >> 8, exactly, with no
// correction term.  The four lanes of a row then add their sub-groups with two shuffles.
// Several tokens (M_ = 2..4): accumulator column 2t + 1, which lane t owns as well, takes a second token of the same
// sub-group (column g carries token g & 1 in the k slots of lane g >> 1), so two tokens cost what one does; tokens
// 2 and 3 are a second set of MMAs over the same A registers.  The code tile of a layer is [M][K/2] nibbles, then
// [M][K/32] scales (a 2-D quant_act4 launch with grid y = layer * M + token).
// ROT_: whole stages are dealt out to the CTAs, from a position that moves with the layer (stream_common.cuh: var_rows).
template <int STAGES_, int NGROUPS_, bool DUMP, int NPROD_ = 1, int M_ = 1, bool ROT_ = false>
struct W4A4Mma {
    using Params = PlainParams;
    static constexpr int M = M_, STAGES = STAGES_, NGROUPS = NGROUPS_, NACT = 1;
    static constexpr bool ACT_IN_STAGE = true, ROT = ROT_;
    static constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;
    static constexpr int ROWB = K / 2, SCB = NG * 2, PITCH = ROWB;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB;
    static constexpr int ACT = M * (K / 2 + (K / 32) * 4);      // packed nibbles, sub-group scales
    static constexpr int STAGE = (OFF_ACT + ACT + 127) & ~127;
    static constexpr int RED = CW * ROWS * M, EXTRA = 0;
    static constexpr int NPROD = NPROD_;
    static constexpr int kThreads = (NGROUPS * CW + 1 + NPROD) * 32;
    static constexpr int NSET = (M + 1) / 2;                    // MMA sets of two tokens

    __device__ static void init_extra(const Params&, uint8_t*) {}
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) {
        const StreamParams& p = pp.s;
        bulk_g2s(dst, p.ae + (size_t)l * M * (K / 2), M * (K / 2), bar);                     // aq
        bulk_g2s(dst + M * (K / 2), p.asc + (size_t)l * M * (K / 32 * 4), M * (K / 32 * 4), bar);
    }

    __device__ static void consume(const Cta& cta, const Params& pp, int grp, int w) {
        Cta c = cta;                                     // (rows and stages of the CTA follow the layer when ROT)
        const StreamParams& p = pp.s;
        const int lane = c.lane, g = lane >> 2, t = lane & 3;
        // this lane's B registers carry column g: token (g & 1) of a set, in the k slots that lane g >> 1 feeds
        uint32_t bmask[NSET];
        int btok[NSET];
#pragma unroll
        for (int si = 0; si < NSET; si++) {
            const int tok = 2 * si + (g & 1);
            bmask[si] = ((g >> 1) == t && tok < M) ? 0xF0F0F0F0u : 0u;
            btok[si] = tok < M ? tok : M - 1;
        }
        int cg = 0;
        int c0 = 0;                                      // stages of the layers before this one
        for (int l = 0; l < p.nlayers; c0 += c.nst, l++) {
            set_geom<W4A4Mma>(c, l);
            const int jf = ((grp - c0) % NGROUPS + NGROUPS) % NGROUPS;
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + p.row_base;
            if (!layer_enter<W4A4Mma>(c, l)) return;
            for (int jst = jf; jst < c.nst; jst += NGROUPS, cg++) {
                const int cc = c0 + jst, s = cc % STAGES;
                if (!stage_wait<W4A4Mma>(c, cc)) return;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                const uint8_t* ab = st + OFF_ACT;
                uint4 xa[GPW], xb[GPW];
                float swa[GPW], swb[GPW];
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int gg = j * CW + w;
                    xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * PITCH + gg * 64 + t * 16);
                    xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * PITCH + gg * 64 + t * 16);
                    swa[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + g * SCB + gg * 2));
                    swb[j] = __half2float(*reinterpret_cast<const __half*>(st + STAGE_W + (g + 8) * SCB + gg * 2));
                }
                float fa[2 * NSET], fb[2 * NSET];                // rows g, g + 8 x tokens 2*set, 2*set + 1 (this lane's sub-groups)
#pragma unroll
                for (int k = 0; k < 2 * NSET; k++) fa[k] = fb[k] = 0.f;
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int gg = j * CW + w;
                    const uint32_t m_hi = 0xF0F0F0F0u;
                    // even k: low nibbles moved to the upper half of their bytes; odd k: high nibbles in place
                    const uint32_t ea0 = (xa[j].x << 4) & m_hi, eb0 = (xb[j].x << 4) & m_hi, ea1 = (xa[j].y << 4) & m_hi, eb1 = (xb[j].y << 4) & m_hi;
                    const uint32_t ea2 = (xa[j].z << 4) & m_hi, eb2 = (xb[j].z << 4) & m_hi, ea3 = (xa[j].w << 4) & m_hi, eb3 = (xb[j].w << 4) & m_hi;
                    const uint32_t oa0 = xa[j].x & m_hi, ob0 = xb[j].x & m_hi, oa1 = xa[j].y & m_hi, ob1 = xb[j].y & m_hi;
                    const uint32_t oa2 = xa[j].z & m_hi, ob2 = xb[j].z & m_hi, oa3 = xa[j].w & m_hi, ob3 = xb[j].w & m_hi;
#pragma unroll
                    for (int si = 0; si < NSET; si++) {
                        // the 32 codes of sub-group t of this lane's column token
                        const uint4 a = *reinterpret_cast<const uint4*>(ab + btok[si] * (K / 2) + gg * 64 + t * 16);
                        const uint32_t bm = bmask[si];
                        int acc[4] = {0, 0, 0, 0};
                        mma_s8(acc, ea0, eb0, ea1, eb1, (a.x << 4) & bm, (a.y << 4) & bm);
                        mma_s8(acc, ea2, eb2, ea3, eb3, (a.z << 4) & bm, (a.w << 4) & bm);
                        mma_s8(acc, oa0, ob0, oa1, ob1, a.x & bm, a.y & bm);
                        mma_s8(acc, oa2, ob2, oa3, ob3, a.z & bm, a.w & bm);
#pragma unroll
                        for (int h = 0; h < 2; h++) {            // accumulator columns 2t, 2t + 1: tokens 2*si, 2*si + 1
                            const int tok = 2 * si + h;
                            if (tok >= M) continue;
                            const float sa = *reinterpret_cast<const float*>(ab + M * (K / 2) + (tok * (K / 32) + gg * 4 + t) * 4);
                            const int ia = acc[h] >> 8, ib = acc[2 + h] >> 8;      // rows g, g + 8: 256 * J exactly
                            fa[tok] += (swa[j] * sa) * (float)ia;
                            fb[tok] += (swb[j] * sa) * (float)ib;
                            if (DUMP) {
                                const int ra = c.r0 + jst * ROWS + g, rb = ra + 8, sg = gg * 4 + t;
                                int* d = p.iacc + ((size_t)l * M + tok) * p.rows * (K / 32) + sg;
                                if (ra < c.r1) d[(size_t)ra * (K / 32)] = ia;
                                if (rb < c.r1) d[(size_t)rb * (K / 32)] = ib;
                            }
                        }
                    }
                }
                float chk = 0.f;
#pragma unroll
                for (int k = 0; k < M; k++) chk += fa[k] + fb[k];
                consumed(chk);                           // release only after the loaded data has been used
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                // the four lanes of a row hold the sums over their own sub-groups
                float vals[2 * M];
                int idx[2 * M];
#pragma unroll
                for (int k = 0; k < M; k++) {
                    float va = fa[k], vb = fb[k];
                    va += __shfl_xor_sync(0xffffffffu, va, 1);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 1);
                    va += __shfl_xor_sync(0xffffffffu, va, 2);
                    vb += __shfl_xor_sync(0xffffffffu, vb, 2);
                    vals[2 * k] = va;
                    vals[2 * k + 1] = vb;
                    idx[2 * k] = t == 0 ? g * M + k : -1;
                    idx[2 * k + 1] = t == 0 ? (g + 8) * M + k : -1;
                }
                if (!reduce_and_emit<W4A4Mma>(c, grp, w, cg, vals, idx, yt, y, c.r0 + jst * ROWS)) return;
            }
            layer_done(c, l);
        }
    }
};

// ------------------------------------------------------------------------------------
// dp4a consumer (W4A4 always; W4A8 as the alternative to the tensor-core consumer): one warp per row of
// a stage, lane l the 16-byte words l, l + 32, .. of that row (LDS.128) into registers; nibbles -> dp4a
// against the token's codes held in registers, two shuffles per 128-group (W4A8) or none (W4A4: a
// 16-byte word is one 32-sub-group), f16 scale * act scale * float(I), butterfly, lane 0 emits y.
//   A4   int4 activations of quant_act4 (packed nibbles + one scale per 32 k) instead of the int8 codes of
//        quant_act; the nibbles are sign-extended to int8 in registers at each layer start.
template <bool A4, int STAGES_, int NACT_, bool DUMP>
struct W4Dp4a {
    using Params = PlainParams;
    static constexpr int M = 1, STAGES = STAGES_, NGROUPS = 1, NACT = NACT_;
    static constexpr bool ACT_IN_STAGE = false;
    static constexpr int K = 5120, KITER = K / 1024, NG = K / 128, CW = 16, ROWS = CW;
    static constexpr int ROWB = K / 2, SCB = NG * 2, PITCH = ROWB;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB, STAGE = OFF_ACT;
    static constexpr int ACT = A4 ? K / 2 + (K / 32) * 4      // packed nibbles, sub-group scales
                                  : K + NG * 8;             // even codes, odd codes, scales, sums
    static constexpr int RED = 0, EXTRA = 0;
    static constexpr int NPROD = 1;
    static constexpr int kThreads = (CW + 2) * 32;

    __device__ static void init_extra(const Params&, uint8_t*) {}
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) {
        const StreamParams& p = pp.s;
        if (A4) {
            bulk_g2s(dst, p.ae + (size_t)l * (K / 2), K / 2, bar);                               // aq
            bulk_g2s(dst + K / 2, p.asc + (size_t)l * (K / 32 * 4), K / 32 * 4, bar);
        } else {
            bulk_g2s(dst, p.ae + (size_t)l * (K / 2), K / 2, bar);
            bulk_g2s(dst + K / 2, p.ao + (size_t)l * (K / 2), K / 2, bar);
            bulk_g2s(dst + K, p.asc + (size_t)l * (NG * 4), NG * 4, bar);
            bulk_g2s(dst + K + NG * 4, p.asu + (size_t)l * (NG * 4), NG * 4, bar);
        }
    }

    __device__ static void consume(const Cta& c, const Params& pp, int, int w) {
        const StreamParams& p = pp.s;
        const int lane = c.lane;
        int cc = 0;
        for (int l = 0; l < p.nlayers; l++) {
            if (!layer_enter<W4Dp4a>(c, l)) return;
            const uint8_t* ab = c.act + (size_t)(l % NACT) * ACT;
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + p.row_base;
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
            for (int j = 0; j < c.nst; j++, cc++) {
                const int s = cc % STAGES;
                if (!stage_wait<W4Dp4a>(c, cc)) return;
                const int row = c.r0 + j * CW + w;
                const bool live = row < c.r1;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                const uint4* wrow = reinterpret_cast<const uint4*>(st + (size_t)w * ROWB);
                const __half* srow = reinterpret_cast<const __half*>(st + STAGE_W + (size_t)w * SCB);
                // `live` is uniform over the warp (one row per warp), so dead rows of a partial last
                // stage skip the loads and the arithmetic altogether
                float acc = 0.f;
                if (live) {
                    uint4 wv[KITER];
                    float sw[KITER];
#pragma unroll
                    for (int it = 0; it < KITER; it++) {
                        wv[it] = wrow[it * 32 + lane];
                        sw[it] = __half2float(srow[(it * 128 + lane * 4) >> 4]);
                    }
#pragma unroll
                    for (int it = 0; it < KITER; it++) {
                        int v = dot32_u(wv[it], ae[it], ao[it]);
                        if (!A4) {
                            v += __shfl_xor_sync(0xffffffffu, v, 1);
                            v += __shfl_xor_sync(0xffffffffu, v, 2);
                        }
                        const int I = v - asu8[it];
                        if (A4 || (lane & 3) == 0) {
                            acc += (sw[it] * asc[it]) * (float)I;
                            if (DUMP) {
                                const int unit = A4 ? (it * 128 + lane * 4) >> 2 : (it * 128 + lane * 4) >> 4;
                                p.iacc[((size_t)l * p.rows + row) * (A4 ? K / 32 : NG) + unit] = I;
                            }
                        }
                    }
                }
                // Release only now: the arithmetic above has consumed every register loaded from the stage
                // (and, in a layer's first stage, from the code tile), so those loads have completed.
                consumed(acc);
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                if (j == 0) act_release<W4Dp4a>(c, l);
                if (!live) continue;
                acc = warp_sum(acc);
                if (lane == 0) emit<1>(c, yt, y, row, 0, acc);
            }
            layer_done(c, l);
        }
    }
};

// ------------------------------------------------------------------------------------
// NVFP4 (E2M1 weights, E4M3 scale per 16 weights, f32 global scale, int8 activations per 16-block;
// reference kernels/asm/k_nvfp4/011_*.s:117-184): per (row, 16-block) the exact integer
//   I = sum (2 * E2M1(w)) * q,   y += float(I) * ((0.5 * gscale * E4M3(ws)) * scale_act)   in block order.
// The code tile of a layer holds the even / odd int8 streams and the 320 block scales of the token
// (nvfp4_quant_act's outputs).
struct Nvfp4Params {
    StreamParams s;                    // layers[].ws are E4M3 bytes [rows][K/16]; s.ae = even codes, s.ao = odd codes, s.asc = scales
    float gscale;
};

__device__ __forceinline__ void nvfp4_copy_act(const StreamParams& p, int l, uint8_t* dst, uint64_t* bar) {
    constexpr int K = 5120, NB = K / 16;
    bulk_g2s(dst, p.ae + (size_t)l * (K / 2), K / 2, bar);
    bulk_g2s(dst + K / 2, p.ao + (size_t)l * (K / 2), K / 2, bar);
    bulk_g2s(dst + K, p.asc + (size_t)l * (NB * 4), NB * 4, bar);
}
__device__ __forceinline__ void nvfp4_init_lut(float gscale, uint8_t* extra) {
    float* lut = reinterpret_cast<float*>(extra);            // [256] 0.5 * gscale * E4M3(byte)
    for (int i = threadIdx.x; i < 256; i += blockDim.x) lut[i] = (0.5f * gscale) * e4m3_to_f32(i);
}

// Tensor-core consumer.  The packed word is the PRMT selector into the table of doubled magnitudes
// {0,1,2,3,4,6,8,12}: PRMT(table, w) gives the magnitudes of the positive codes of four nibbles (0 for the
// negative ones: selector bit 3 is "replicate the sign bit", which is 0 for table bytes < 0x80) and
// PRMT(table, w ^ 0x8888) those of the negative codes, so  I = MMA(pos, q) - MMA(neg, q)  with mma.sync
// m16n8k32 (int8).  One MMA adds over the k slots of all four lanes of a row, but a lane's 16-byte word holds
// two 16-blocks of its own; the blocks are kept apart by the columns of B: column 2t carries the token's codes
// only in the k slots that lane t feeds (zero elsewhere), so accumulator column 2t — which lane t owns — is
// the sum over lane t's own eight codes, and two MMAs (the two words of a block) complete a block.  A stage
// of 16 rows is one m16 tile; the 8 warps take 5 of the 40 chunks of 128 k each (8 blocks), as in the W4A8
// kernel.  Per packed word: 7 integer instructions and one MMA, against 12 with dp4a.
template <int STAGES_, int NGROUPS_, int NACT_, bool DUMP>
struct Nvfp4Mma {
    using Params = Nvfp4Params;
    static constexpr int M = 1, STAGES = STAGES_, NGROUPS = NGROUPS_, NACT = NACT_;
    static constexpr bool ACT_IN_STAGE = false;
    static constexpr int K = 5120, NB = K / 16, NC = K / 128, CW = 8, GPW = NC / CW, ROWS = 16;
    static constexpr int ROWB = K / 2, SCB = NB, PITCH = ROWB;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB, STAGE = OFF_ACT;
    static constexpr int ACT = K + NB * 4;
    static constexpr int RED = CW * ROWS, EXTRA = 1024;
    static constexpr int NPROD = 1;
    static constexpr int kThreads = (NGROUPS * CW + 2) * 32;

    __device__ static void init_extra(const Params& pp, uint8_t* extra) { nvfp4_init_lut(pp.gscale, extra); }
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) { nvfp4_copy_act(pp.s, l, dst, bar); }

    __device__ static void consume(const Cta& c, const Params& pp, int grp, int w) {
        const StreamParams& p = pp.s;
        const float* lut = reinterpret_cast<const float*>(c.extra);
        const int lane = c.lane, g = lane >> 2, t = lane & 3;
        const bool feeds = g == 2 * t;                   // this lane's B registers carry column 2t
        int cg = 0;
        for (int l = 0; l < p.nlayers; l++) {
            const int c0 = l * c.nst;
            const int jf = ((grp - c0) % NGROUPS + NGROUPS) % NGROUPS;
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + p.row_base;
            if (!layer_enter<Nvfp4Mma>(c, l)) return;
            const uint8_t* ab = c.act + (size_t)(l % NACT) * ACT;
            uint32_t b0[GPW][4], b1[GPW][4];             // B fragments: codes k0..k3 / k4..k7 of the lane's four words per chunk
            float2 asc[GPW];                             // activation scales of the lane's two blocks per chunk
            bool held = jf < c.nst;
            if (held) {
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int gg = j * CW + w;
                    const uint4 e = *reinterpret_cast<const uint4*>(ab + gg * 64 + t * 16);
                    const uint4 o = *reinterpret_cast<const uint4*>(ab + K / 2 + gg * 64 + t * 16);
                    const uint32_t ev[4] = {e.x, e.y, e.z, e.w}, ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        b0[j][q] = feeds ? prmt(ev[q], ov[q], 0x5140u) : 0u;      // k0 k1 k2 k3 of word q
                        b1[j][q] = feeds ? prmt(ev[q], ov[q], 0x7362u) : 0u;      // k4 k5 k6 k7
                    }
                    asc[j] = *reinterpret_cast<const float2*>(ab + K + (gg * 8 + 2 * t) * 4);
                }
            } else {
                act_release<Nvfp4Mma>(c, l);
            }
            for (int jst = jf; jst < c.nst; jst += NGROUPS, cg++) {
                const int cc = c0 + jst, s = cc % STAGES;
                if (!stage_wait<Nvfp4Mma>(c, cc)) return;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                uint4 xa[GPW], xb[GPW];
                uint32_t sba[GPW], sbb[GPW];             // E4M3 bytes of the lane's two blocks, rows g and g + 8
                auto load_chunk = [&](int j) {
                    const int gg = j * CW + w;
                    xa[j] = *reinterpret_cast<const uint4*>(st + (size_t)g * PITCH + gg * 64 + t * 16);
                    xb[j] = *reinterpret_cast<const uint4*>(st + (size_t)(g + 8) * PITCH + gg * 64 + t * 16);
                    sba[j] = *reinterpret_cast<const unsigned short*>(st + STAGE_W + g * SCB + gg * 8 + 2 * t);
                    sbb[j] = *reinterpret_cast<const unsigned short*>(st + STAGE_W + (g + 8) * SCB + gg * 8 + 2 * t);
                };
                if (NGROUPS == 1) {                      // registers to spare: everything in flight at once
#pragma unroll
                    for (int j = 0; j < GPW; j++) load_chunk(j);
                } else {
                    load_chunk(0);
                }
                float fa = 0.f, fb = 0.f;
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    if (NGROUPS > 1) {                   // one chunk ahead only (96 registers per thread with 18 warps)
                        if (j + 1 < GPW) load_chunk(j + 1);
                        asm volatile("" ::: "memory");
                    }
                    const uint32_t wa[4] = {xa[j].x, xa[j].y, xa[j].z, xa[j].w}, wb[4] = {xb[j].x, xb[j].y, xb[j].z, xb[j].w};
#pragma unroll
                    for (int blk = 0; blk < 2; blk++) {
                        int cp[4], cn[4];
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int q = blk * 2 + h;
                            const uint32_t pa = wa[q], pb = wb[q], na = pa ^ 0x88888888u, nb = pb ^ 0x88888888u;
                            const uint32_t p0 = prmt(kTabLo, kTabHi, pa), p1 = prmt(kTabLo, kTabHi, pb);
                            const uint32_t p2 = prmt(kTabLo, kTabHi, pa >> 16), p3 = prmt(kTabLo, kTabHi, pb >> 16);
                            const uint32_t n0 = prmt(kTabLo, kTabHi, na), n1 = prmt(kTabLo, kTabHi, nb);
                            const uint32_t n2 = prmt(kTabLo, kTabHi, na >> 16), n3 = prmt(kTabLo, kTabHi, nb >> 16);
                            if (h == 0) {
                                mma_s8_first(cp, p0, p1, p2, p3, b0[j][q], b1[j][q]);
                                mma_s8_first(cn, n0, n1, n2, n3, b0[j][q], b1[j][q]);
                            } else {
                                mma_s8(cp, p0, p1, p2, p3, b0[j][q], b1[j][q]);
                                mma_s8(cn, n0, n1, n2, n3, b0[j][q], b1[j][q]);
                            }
                        }
                        const int ia = cp[0] - cn[0], ib = cp[2] - cn[2];       // rows g, g + 8, column 2t
                        const float sact = blk ? asc[j].y : asc[j].x;
                        fa = fmaf((float)ia, lut[(sba[j] >> (8 * blk)) & 0xFFu] * sact, fa);
                        fb = fmaf((float)ib, lut[(sbb[j] >> (8 * blk)) & 0xFFu] * sact, fb);
                        if (DUMP) {
                            const int ra = c.r0 + jst * ROWS + g, rb = ra + 8, bi = (j * CW + w) * 8 + 2 * t + blk;
                            if (ra < c.r1) p.iacc[((size_t)l * p.rows + ra) * NB + bi] = ia;
                            if (rb < c.r1) p.iacc[((size_t)l * p.rows + rb) * NB + bi] = ib;
                        }
                    }
                }
                consumed(fa + fb);                       // release only after the loaded data has been used
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                if (held) {
                    act_release<Nvfp4Mma>(c, l);
                    held = false;
                }
                // the four lanes of a row hold the sums over their own blocks
                fa += __shfl_xor_sync(0xffffffffu, fa, 1);
                fb += __shfl_xor_sync(0xffffffffu, fb, 1);
                fa += __shfl_xor_sync(0xffffffffu, fa, 2);
                fb += __shfl_xor_sync(0xffffffffu, fb, 2);
                const float vals[2] = {fa, fb};
                const int idx[2] = {t == 0 ? g : -1, t == 0 ? g + 8 : -1};
                if (!reduce_and_emit<Nvfp4Mma>(c, grp, w, cg, vals, idx, yt, y, c.r0 + jst * ROWS)) return;
            }
            layer_done(c, l);
        }
    }
};

// dp4a consumer of the same format: one warp per row of a stage, the arithmetic of nvfp4_gemv<1,1>
// (I = dp4a(pos) - dp4a(neg) per packed word, lane l owns the words l, l + 32, ..).
template <int STAGES_, int NACT_, bool DUMP>
struct Nvfp4Dp4a {
    using Params = Nvfp4Params;
    static constexpr int M = 1, STAGES = STAGES_, NGROUPS = 1, NACT = NACT_;
    static constexpr bool ACT_IN_STAGE = false;
    static constexpr int K = 5120, KITER = 5, NB = K / 16, CW = 12, ROWS = CW;
    static constexpr int ROWB = K / 2, SCB = NB, PITCH = ROWB;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB, STAGE = OFF_ACT;
    static constexpr int ACT = K + NB * 4;
    static constexpr int RED = 0, EXTRA = 1024;
    static constexpr int NPROD = 1;
    static constexpr int kThreads = (CW + 2) * 32;

    __device__ static void init_extra(const Params& pp, uint8_t* extra) { nvfp4_init_lut(pp.gscale, extra); }
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) { nvfp4_copy_act(pp.s, l, dst, bar); }

    __device__ static void consume(const Cta& c, const Params& pp, int, int w) {
        const StreamParams& p = pp.s;
        const float* lut = reinterpret_cast<const float*>(c.extra);
        const int lane = c.lane;
        int cc = 0;
        for (int l = 0; l < p.nlayers; l++) {
            if (!layer_enter<Nvfp4Dp4a>(c, l)) return;
            const uint8_t* ab = c.act + (size_t)(l % NACT) * ACT;
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + p.row_base;
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
            for (int j = 0; j < c.nst; j++, cc++) {
                const int s = cc % STAGES;
                if (!stage_wait<Nvfp4Dp4a>(c, cc)) return;
                const int row = c.r0 + j * CW + w;
                const bool live = row < c.r1;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                float acc = 0.f;
                if (live) {
                    const uint4* wrow = reinterpret_cast<const uint4*>(st + (size_t)w * ROWB);
                    const uint8_t* srow = st + STAGE_W + (size_t)w * SCB;
                    uint4 wv[KITER];
                    uint32_t sb[KITER];
#pragma unroll
                    for (int it = 0; it < KITER; it++) {
                        wv[it] = wrow[it * 32 + lane];
                        sb[it] = *reinterpret_cast<const unsigned short*>(srow + ((it * 128 + lane * 4) >> 1));
                    }
#pragma unroll
                    for (int it = 0; it < KITER; it++) {
                        int i0 = dot8_e2m1(wv[it].x, a0[it].x, a0[it].y, 0);
                        i0 = dot8_e2m1(wv[it].y, a0[it].z, a0[it].w, i0);
                        int i1 = dot8_e2m1(wv[it].z, a1[it].x, a1[it].y, 0);
                        i1 = dot8_e2m1(wv[it].w, a1[it].z, a1[it].w, i1);
                        acc = fmaf((float)i0, lut[sb[it] & 0xFFu] * asc[it].x, acc);
                        acc = fmaf((float)i1, lut[(sb[it] >> 8) & 0xFFu] * asc[it].y, acc);
                        if (DUMP) {
                            int* d = p.iacc + ((size_t)l * p.rows + row) * NB + ((it * 128 + lane * 4) >> 1);
                            d[0] = i0;
                            d[1] = i1;
                        }
                    }
                }
                consumed(acc);                                  // release only after the loaded data has been used
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                if (j == 0) act_release<Nvfp4Dp4a>(c, l);
                if (!live) continue;
                acc = warp_sum(acc);
                if (lane == 0) emit<1>(c, yt, y, row, 0, acc);
            }
            layer_done(c, l);
        }
    }
};

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

struct W4a16Params {
    StreamParams s;                    // layers[].wq offset-binary codes, layers[].ws bf16 scales [rows][K/128]
    const uint32_t* frags;             // [nlayers][40 * 192] B fragments of the activations
};

//   NGROUPS consumer groups that take the stages in turn (2: a group has two stage times for its own stage)
//   BREG    a warp keeps the B fragments of its blocks in registers for the whole layer (80 registers: one group only);
//           otherwise they are read from the layer's tile with every stage
//   ROT_    whole stages are dealt out to the CTAs, from a position that moves with the layer (stream_common.cuh: var_rows)
template <int STAGES_, int NGROUPS_, int NACT_, bool BREG, bool ROT_ = false>
struct W4A16Mma {
    using Params = W4a16Params;
    static constexpr int M = 1, STAGES = STAGES_, NGROUPS = NGROUPS_, NACT = NACT_;
    static constexpr bool ACT_IN_STAGE = false, ROT = ROT_;
    static_assert(!ROT || !BREG, "moving row ranges: no fragments held over a layer");
    static constexpr int K = 5120, NG = 40, CW = 8, GPW = NG / CW, ROWS = 16;
    static constexpr int ROWB = K / 2, SCB = NG * 2, PITCH = ROWB;
    static constexpr int STAGE_W = ROWS * PITCH, OFF_ACT = STAGE_W + ROWS * SCB, STAGE = OFF_ACT;
    static constexpr int ACT = NG * 192 * 4;             // fragment array of one layer
    static constexpr int RED = CW * ROWS, EXTRA = 0;
    static constexpr int NPROD = 1;
    static constexpr int kThreads = (NGROUPS * CW + 2) * 32;
    static_assert(!BREG || NGROUPS == 1, "fragments in registers leave no room for a second group");

    __device__ static void init_extra(const Params&, uint8_t*) {}
    __device__ static void copy_act(const Params& pp, int l, uint8_t* dst, uint64_t* bar) {
        bulk_g2s(dst, pp.frags + (size_t)l * (NG * 192), ACT, bar);
    }
    // B fragments of block b for this lane: {b0,b1 of (q,0), b0,b1 of (q,1)}, q = 0..3
    __device__ static __forceinline__ uint4 frag(const uint32_t* ft, int b, int g, int t, int q) {
        if (g >= 3) return make_uint4(0, 0, 0, 0);
        return reinterpret_cast<const uint4*>(ft + ((size_t)(b * 3 + g) * 4 + t) * 16)[q];
    }

    __device__ static void consume(const Cta& cta, const Params& pp, int grp, int w) {
        Cta c = cta;                                     // (rows and stages of the CTA follow the layer when ROT)
        const StreamParams& p = pp.s;
        const int lane = c.lane, g = lane >> 2, t = lane & 3;
        int cg = 0;                                      // stages this group has taken so far
        int c0 = 0;                                      // stages of the layers before this one
        for (int l = 0; l < p.nlayers; c0 += c.nst, l++) {
            set_geom<W4A16Mma>(c, l);
            const int jf = ((grp - c0) % NGROUPS + NGROUPS) % NGROUPS;     // this group's first stage of the layer
            if (!layer_enter<W4A16Mma>(c, l)) return;
            const uint32_t* ft = reinterpret_cast<const uint32_t*>(c.act + (size_t)(l % NACT) * ACT);
            float* yt = c.ytile + (l % kYBufs) * kOutCap;
            float* y = get_layer(p, l).y + p.row_base;
            uint4 bf[BREG ? GPW : 1][4];
            bool held = false;                           // the tile has not been released yet
            if (BREG) {
#pragma unroll
                for (int j = 0; j < GPW; j++)
#pragma unroll
                    for (int q = 0; q < 4; q++) bf[j][q] = frag(ft, j * CW + w, g, t, q);
                held = true;
            }
            for (int jst = jf; jst < c.nst; jst += NGROUPS, cg++) {
                const int cc0 = c0 + jst, s = cc0 % STAGES;
                if (!stage_wait<W4A16Mma>(c, cc0)) return;
                const uint8_t* st = c.ring + (size_t)s * STAGE;
                uint4 xa[GPW], xb[GPW];
                float swa[GPW], swb[GPW];
#pragma unroll
                for (int j = 0; j < GPW; j++) {
                    const int b = j * CW + w;
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
                        const uint4 f = BREG ? bf[j][q] : frag(ft, j * CW + w, g, t, q);
                        const uint32_t la = wav[q] & 0x0F0F0F0Fu, ha = (wav[q] >> 4) & 0x0F0F0F0Fu;
                        const uint32_t lb = wbv[q] & 0x0F0F0F0Fu, hb = (wbv[q] >> 4) & 0x0F0F0F0Fu;
                        const uint32_t m = 0x43434343u;
                        mma_bf16(cc, bf16x2_sub136(prmt(la, m, 0x5140u)), bf16x2_sub136(prmt(lb, m, 0x5140u)),
                                 bf16x2_sub136(prmt(la, m, 0x5342u)), bf16x2_sub136(prmt(lb, m, 0x5342u)), f.x, f.y);
                        mma_bf16(cc, bf16x2_sub136(prmt(ha, m, 0x5140u)), bf16x2_sub136(prmt(hb, m, 0x5140u)),
                                 bf16x2_sub136(prmt(ha, m, 0x5342u)), bf16x2_sub136(prmt(hb, m, 0x5342u)), f.z, f.w);
                    }
                    // columns 0, 1 (lane t = 0) and 2 (lane t = 1) hold the three terms: smallest first
                    const float va = __shfl_down_sync(0xffffffffu, cc[0], 1), vb = __shfl_down_sync(0xffffffffu, cc[2], 1);
                    fa += swa[j] * ((va + cc[1]) + cc[0]);
                    fb += swb[j] * ((vb + cc[3]) + cc[2]);
                }
                consumed(fa + fb);                              // release only after the loaded data has been used
                __syncwarp();
                if (lane == 0) mbar_arrive(&c.bars->empty[s]);
                if (BREG && held) {
                    act_release<W4A16Mma>(c, l);
                    held = false;
                }
                const float vals[2] = {fa, fb};
                const int idx[2] = {t == 0 ? g : -1, t == 0 ? g + 8 : -1};
                if (!reduce_and_emit<W4A16Mma>(c, grp, w, cg, vals, idx, yt, y, c.r0 + jst * ROWS)) return;
            }
            if (!BREG || held) act_release<W4A16Mma>(c, l);
            layer_done(c, l);
        }
    }
};

// ------------------------------------------------------------------------------------
// stream_flag_wait(flags, nlayers, target, status, spins): the acquire side of the completion counters.
// One thread per layer waits until flags[layer] >= target (every CTA of every contributing GPU has added
// its one), at most `spins` polls of about a microsecond each; a counter that does not get there in time sets
// *status to 9 and the kernel returns, so a consumer that is launched behind it can check the word and a
// missing producer costs a bounded wait, not a hang.  It must not share a GPU with a stream kernel that it
// waits for unless that kernel was launched first on another stream and is resident.
__global__ void __launch_bounds__(128)
stream_flag_wait_kernel(const unsigned* flags, int nlayers, unsigned target, int* status, int spins) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= nlayers) return;
    const volatile unsigned* f = flags + l;
    for (int i = 0; i < spins; i++) {
        unsigned v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v >= target) return;
        __nanosleep(1000);
    }
    atomicCAS(status, 0, 9);
}

// ------------------------------------------------------------------------------------ host side
template <class P>
int run_policy(const char* kn, const LaunchCtx& c, const typename P::Params& pp) {
    constexpr size_t smem = smem_bytes<P>();
    static_assert(smem <= 227 * 1024, "shared memory");
    static_assert(P::STAGES <= kMaxStages && P::NACT <= kMaxStages && P::NGROUPS <= 2, "barrier block");
    auto kern = stream_kernel<P>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    int grid = c.sm_count;
    if (grid > pp.s.rows) grid = pp.s.rows;
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(P::kThreads), smem, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

int env_or(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

// The arguments every stream kernel starts with: (layers, nlayers, rows, K, row_base, npeers, peer_delta, status)
//   layers      device array of nlayers x {wq, ws, x, y} pointers (32 bytes each), filled by
//               fm_stream_table (which range-checks every pointer in it)
//   rows        weight rows held by this GPU (N, or N / number of GPUs)
//   row_base    first output index of this GPU's rows inside each layer's y
//   npeers      0, or the number of other copies of y that also receive the rows (other GPUs'
//               buffers and/or a pinned host buffer: up to 8);
//   peer_delta  device array of npeers signed byte offsets (receiver's y address - local y address),
//               filled by fm_stream_peers
//   status      device int, must be 0 before the launch; non-zero afterwards = a bounded
//               wait ran out (codes in stream_common.cuh)
// and the one they all end with:
//   flags       0, or device array of nlayers u32 counters inside the window that fm_stream_peers
//               validated (so that every receiver has a copy at the same offset): each CTA adds 1 to
//               flags[layer] on every receiver once its rows of the layer are visible there.  The counters
//               are not cleared by the kernel.  Needs at most 512 y values per CTA and layer.
// Returns 1 when there is nothing to do.
int parse_common(const char* kn, const LaunchCtx& c, const uint64_t* a, uint64_t flags_arg, StreamParams& p, int M) {
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.nlayers = arg_i32(a[1]);
    p.rows = arg_i32(a[2]);
    p.K = arg_i32(a[3]);
    p.row_base = arg_i32(a[4]);
    p.npeers = arg_i32(a[5]);
    p.peer_delta = arg_ptr<const long long>(a[6]);
    p.status = arg_ptr<int>(a[7]);
    p.flags = arg_ptr<unsigned>(flags_arg);
    p.M = M;
    p.wait_hint_ns = (uint32_t)env_or("FM_STREAM_HINT_NS", 0);
    FM_REQUIRE(p.K == 5120, kn, "K=%d: the fused stream is built for K = 5120 only; launch the per-layer kernels", p.K);
    FM_REQUIRE(p.nlayers >= 0 && p.rows > 0 && p.row_base >= 0 && p.npeers >= 0 && p.npeers <= 8, kn,
               "bad nlayers/rows/row_base/npeers");
    if (p.nlayers == 0) return 1;
    FM_REQUIRE(aligned(p.layers, 8) && aligned(p.status, 4), kn, "misaligned layer table or status");
    FM_RANGE(p.layers, (size_t)p.nlayers * sizeof(StreamLayer), kn, "layers");
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    if (p.flags) {
        const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
        FM_REQUIRE(aligned(p.flags, 4), kn, "misaligned flags");
        FM_RANGE(p.flags, (size_t)p.nlayers * 4, kn, "flags");
        FM_REQUIRE((long long)(((p.rows + 15) / 16 + grid - 1) / grid * 16) * M <= kOutCap, kn,
                   "completion counters need at most %d y values per CTA and layer (rows=%d on %d CTAs, M=%d)", kOutCap,
                   p.rows, grid, M);
        FM_REQUIRE(p.npeers == 0 || peer_window_ok(p.peer_delta, p.npeers, p.flags, (size_t)p.nlayers * 4), kn,
                   "the flags array must lie inside the window that fm_stream_peers validated for these offsets");
    }
    return 0;
}

// the default W4A8 schedule deals out whole 16-row stages (instead of rows / grid) when a CTA gets three or more per layer
static bool whole_stages(int rows, int grid) { return (rows + 15) / 16 >= 3 * grid; }

// w4a8_decode_stream(common..., ae, ao, asc, asu, flags)
//   ae, ao, asc, asu   outputs of quant_act launched with grid y = nlayers over x [nlayers][K]:
//               int8 codes [nlayers][K/2] twice, f32 scales and int32 sums [nlayers][K/128]
// w4a4_decode_stream(common..., aq, asc, flags): the same with the outputs of quant_act4 (grid y = nlayers):
//   packed nibbles [nlayers][K/2], scales [nlayers][K/32].
// w4a8_decode_stream_iacc / w4a4_decode_stream_iacc(..., flags, iacc): the same kernels with the integer
//   accumulators stored as well, iacc int32 [nlayers][rows][K/128 or K/32].
// grid and work-group arguments are ignored (persistent: one CTA per SM).
// $FM_STREAM_CFG selects another schedule of w4a8_decode_stream than the default (see the switch below).
template <bool A4, bool DUMP>
int launch_w4_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = A4 ? (DUMP ? "w4a4_decode_stream_iacc" : "w4a4_decode_stream") : (DUMP ? "w4a8_decode_stream_iacc" : "w4a8_decode_stream");
    PlainParams pp = {};
    StreamParams& p = pp.s;
    const int nact = A4 ? 2 : 4;                         // activation arrays
    const int rc = parse_common(kn, c, a, a[8 + nact], p, 1);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ystride = 0;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    if (A4) {
        p.asc = arg_ptr<const uint8_t>(a[9]);
    } else {
        p.ao = arg_ptr<const uint8_t>(a[9]);
        p.asc = arg_ptr<const uint8_t>(a[10]);
        p.asu = arg_ptr<const uint8_t>(a[11]);
    }
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d "
               "(or was overwritten, or a buffer it points into was freed since), or the peer offsets do not come from "
               "fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.asc, 16) && (A4 || (aligned(p.ao, 16) && aligned(p.asu, 16))), kn,
               "the activation code arrays must be 16-byte aligned");
    FM_RANGE(p.ae, (size_t)p.nlayers * (p.K / 2), kn, A4 ? "aq" : "ae");
    FM_RANGE(p.asc, (size_t)p.nlayers * (p.K / (A4 ? 32 : 128)) * 4, kn, "asc");
    if (!A4) {
        FM_RANGE(p.ao, (size_t)p.nlayers * (p.K / 2), kn, "ao");
        FM_RANGE(p.asu, (size_t)p.nlayers * (p.K / 128) * 4, kn, "asu");
    }
    const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
    const int nst = ((p.rows + grid - 1) / grid + 15) / 16;      // stages per layer of the busiest CTA
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[9 + nact]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, (size_t)p.nlayers * p.rows * (p.K / (A4 ? 32 : 128)) * 4, kn, "iacc");
        if (A4) return env_or("FM_STREAM_CFG", 3) != 1 ? run_policy<W4A4Mma<4, 2, true>>(kn, c, pp)
                                                       : run_policy<W4Dp4a<true, 5, 2, true>>(kn, c, pp);
        return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, true>>(kn, c, pp);
    }
    if (A4) {
        // tensor-core consumer, two groups; $FM_STREAM_CFG=1 keeps the dp4a consumer
        if (env_or("FM_STREAM_CFG", 3) != 1) return run_policy<W4A4Mma<4, 2, false, 2>>(kn, c, pp);
        return nst >= 3 ? run_policy<W4Dp4a<true, 5, 2, false>>(kn, c, pp) : run_policy<W4Dp4a<true, 4, 5, false>>(kn, c, pp);
    }
    // Default: the token's codes travel inside every stage and two groups of eight warps take the stages in turn.
    // Measured on one B200 (400 layers, ms per token, 20-step burst / one-second run): 17408 rows 2.62 / 3.07 against
    // 3.04 / 3.35 for one group with the fragments in registers (0); 2176 rows — the shard of eight GPUs, one stage per
    // CTA and layer — 0.384 / 0.442 against 0.496 / 0.507.  The stages go round two producer lanes (one lane: 1 % slower
    // on the shard shapes, 1.6 % in the one-second run at 17408 rows).  The other numbers are kept for comparison.
    switch (env_or("FM_STREAM_CFG", -1)) {
        case 0: return run_policy<W4A8Mma<1, 5, 1, false, 2, true, 0, false>>(kn, c, pp);    // one group, fragments in registers
        case 1: return run_policy<W4Dp4a<false, 5, 2, false>>(kn, c, pp);                    // dp4a
        case 2: return run_policy<W4A8Mma<1, 4, 1, false, 5, true, 0, false>>(kn, c, pp);    // deeper ring of code tiles
        case 4: return run_policy<W4A8Mma<1, 4, 1, true, 1, false, 0, false>>(kn, c, pp);    // codes inside every stage, one group
        case 7: return run_policy<W4A8Mma<1, 4, 1, false, 2, true, 64, false>>(kn, c, pp);   // padded row pitch (no bank conflicts): slower
        case 3: return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false>>(kn, c, pp);    // one producer lane, rows / grid per CTA
        case 5: return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false, 2>>(kn, c, pp); // two producer lanes, rows / grid per CTA
        case 6: return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false, 2, false, true>>(kn, c, pp);   // whole stages per CTA
        default:
            // Whole stages per CTA pay when a CTA has three or more per layer (17408 rows: 2.59 against 2.64 ms per
            // token, 8704 rows: 1.29 against 1.31); with one stage per CTA and layer — the shard of eight GPUs — a
            // full stage on 136 CTAs is slower than 14.7 rows on each of 148 (0.40 against 0.36 ms).
            if (whole_stages(p.rows, grid)) return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false, 2, false, true>>(kn, c, pp);
            return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false, 2>>(kn, c, pp);
    }
}

// w4a8_stream_read_ceiling(common..., ae, ao, asc, asu, flags): the arguments of w4a8_decode_stream; copies what that
// kernel copies and computes nothing (y is not written, flags are not counted).
int launch_w4a8_read_ceiling(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "w4a8_stream_read_ceiling";
    PlainParams pp = {};
    StreamParams& p = pp.s;
    const int rc = parse_common(kn, c, a, a[12], p, 1);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    p.asu = arg_ptr<const uint8_t>(a[11]);
    p.npeers = 0;
    p.flags = nullptr;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, nullptr, 0), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d (or was "
               "overwritten, or a buffer it points into was freed since)", (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.ao, 16) && aligned(p.asc, 16) && aligned(p.asu, 16), kn,
               "the activation code arrays must be 16-byte aligned");
    FM_RANGE(p.ae, (size_t)p.nlayers * (p.K / 2), kn, "ae");
    FM_RANGE(p.ao, (size_t)p.nlayers * (p.K / 2), kn, "ao");
    FM_RANGE(p.asc, (size_t)p.nlayers * (p.K / 128) * 4, kn, "asc");
    FM_RANGE(p.asu, (size_t)p.nlayers * (p.K / 128) * 4, kn, "asu");
    const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
    const int cfg = env_or("FM_STREAM_CFG", -1);
    if (cfg == 5 || (cfg != 6 && !whole_stages(p.rows, grid))) return run_policy<W4A8ReadCeiling<4, 2>>(kn, c, pp);
    return run_policy<W4A8ReadCeiling<4, 2, true>>(kn, c, pp);
}

// w4a8_layers_stream(layers, shapes, nlayers, npeers, peer_delta, status, flags): W4A8, one token, layers of different
// shapes in one launch.  `layers` / `shapes` are the two device arrays filled by fm_stream_table_var (a layer = 5120 k of
// a set of rows; longer rows are consecutive layers that add to the same y); npeers, peer_delta, status and flags as for
// the other stream kernels (flags: one counter per table entry, each reaching min(SM count, rows of the largest layer)).
// Every CTA takes an equal share of the 16-row stages of every layer (stream_common.cuh: var_rows).
int launch_w4a8_layers_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "w4a8_layers_stream";
    PlainParams pp = {};
    StreamParams& p = pp.s;
    p.layers = arg_ptr<const StreamLayer>(a[0]);
    p.var = arg_ptr<const VarLayer>(a[1]);
    p.nlayers = arg_i32(a[2]);
    p.npeers = arg_i32(a[3]);
    p.peer_delta = arg_ptr<const long long>(a[4]);
    p.status = arg_ptr<int>(a[5]);
    p.flags = arg_ptr<unsigned>(a[6]);
    p.K = 5120;
    p.M = 1;
    p.ystride = 0;
    p.wait_hint_ns = (uint32_t)env_or("FM_STREAM_HINT_NS", 0);
    FM_REQUIRE(p.nlayers >= 0 && p.npeers >= 0 && p.npeers <= 8, kn, "bad nlayers / npeers");
    if (p.nlayers == 0) return FM_OK;
    FM_REQUIRE(aligned(p.status, 4), kn, "misaligned status");
    FM_RANGE(p.status, 4, kn, "status");
    if (p.npeers) FM_RANGE(p.peer_delta, (size_t)p.npeers * 8, kn, "peer_delta");
    int min_rows = 0, max_rows = 0;
    FM_REQUIRE(stream_var_ok(p.layers, p.var, p.nlayers, p.peer_delta, p.npeers, &min_rows, &max_rows, &p.chunk_maps), kn,
               "the layer table at %p and the shapes at %p were not filled by fm_stream_table_var for at least %d layers (or were "
               "overwritten, or a buffer they point into was freed since), or the peer offsets do not come from fm_stream_peers "
               "for its outputs", (const void*)p.layers, (const void*)p.var, p.nlayers);
    p.rows = max_rows;
    // one CTA per SM unless even the largest layer has fewer rows; a CTA without rows in a small layer still takes part
    // in the layer's hand-overs (and counts in its completion counter)
    const int grid = c.sm_count < max_rows ? c.sm_count : max_rows;
    (void)min_rows;
    const int cta_rows = ((max_rows + 15) / 16 + grid - 1) / grid * 16;      // whole 16-row stages are dealt out
    FM_REQUIRE(cta_rows <= kOutCap, kn,
               "a CTA would own %d rows of the largest layer (%d rows on %d CTAs); the output tile holds %d", cta_rows,
               max_rows, grid, kOutCap);
    if (p.flags) {
        FM_REQUIRE(aligned(p.flags, 4), kn, "misaligned flags");
        FM_RANGE(p.flags, (size_t)p.nlayers * 4, kn, "flags");
        FM_REQUIRE(p.npeers == 0 || peer_window_ok(p.peer_delta, p.npeers, p.flags, (size_t)p.nlayers * 4), kn,
                   "the flags array must lie inside the window that fm_stream_peers validated for these offsets");
    }
    using P = W4A8Mma<1, 4, 2, true, 1, false, 0, false, 2, true>;
    constexpr size_t smem = smem_bytes<P>();
    static_assert(smem <= 227 * 1024, "shared memory");
    auto kern = stream_kernel<P>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(kn, e);
        configured = true;
    }
    cudaError_t e = launch_kernel(kern, dim3(grid), dim3(P::kThreads), smem, c.stream, pdl_enabled(), pp);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// w4a8_decode_stream_m(common..., ae, ao, asc, asu, M, ystride, flags): M = 2..4 tokens per layer.  The code arrays
// hold [nlayers * M] tokens (one 2-D quant_act launch with grid y = nlayers * M over x[nlayers][M][K]); y of a layer is
// token-major, y[token * ystride + row_base + row].  The layer table must have been validated by fm_stream_table with
// row_base + (M - 1) * ystride as its row_base argument, which is what makes every token's rows lie inside the checked
// footprint of y.  w4a8_decode_stream_m_iacc(..., flags, iacc): iacc int32 [nlayers][M][rows][K/128].
template <bool DUMP>
int launch_w4a8_stream_m(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = DUMP ? "w4a8_decode_stream_m_iacc" : "w4a8_decode_stream_m";
    PlainParams pp = {};
    StreamParams& p = pp.s;
    const int M = arg_i32(a[12]);
    FM_REQUIRE(M >= 2 && M <= 4, kn, "M=%d: this kernel takes 2..4 tokens (w4a8_decode_stream takes one)", M);
    const int rc = parse_common(kn, c, a, a[14], p, M);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    p.asu = arg_ptr<const uint8_t>(a[11]);
    p.ystride = arg_i32(a[13]);
    FM_REQUIRE(p.ystride >= p.row_base + p.rows && (long long)(p.M - 1) * p.ystride + p.row_base < (1LL << 31), kn,
               "ystride=%d must be at least row_base + rows = %d", p.ystride, p.row_base + p.rows);
    const int vbase = p.row_base + (p.M - 1) * p.ystride;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, vbase, p.peer_delta, p.npeers, true), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d and the row_base "
               "argument row_base + (M - 1) * ystride = %d (or was overwritten, or a buffer it points into was freed since), "
               "or the peer offsets do not come from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers,
               p.rows, p.K, vbase);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.asc, 16) && aligned(p.ao, 16) && aligned(p.asu, 16), kn,
               "the activation code arrays must be 16-byte aligned");
    const size_t tokens = (size_t)p.nlayers * p.M;
    FM_RANGE(p.ae, tokens * (p.K / 2), kn, "ae");
    FM_RANGE(p.ao, tokens * (p.K / 2), kn, "ao");
    FM_RANGE(p.asc, tokens * (p.K / 128) * 4, kn, "asc");
    FM_RANGE(p.asu, tokens * (p.K / 128) * 4, kn, "asu");
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[15]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, tokens * p.rows * (p.K / 128) * 4, kn, "iacc");
    }
    // Default: two consumer groups that read the B fragments from the layer's tile.  Measured per layer (64 layers per
    // launch, burst): 7.3 / 8.3 / 8.1 us at M = 2 / 3 / 4 against 7.8 / 9.1 / 9.0 for one group with the fragments in
    // registers ($FM_STREAM_M_CFG=0, and the kernel the accumulator dump runs).
    const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
    if (!DUMP && env_or("FM_STREAM_M_CFG", 1) == 1 && whole_stages(p.rows, grid)) {
        switch (p.M) {                                   // + whole stages per CTA
            case 2: return run_policy<W4A8Mma<2, 4, 2, false, 2, false, 0, false, 1, false, true>>(kn, c, pp);
            case 3: return run_policy<W4A8Mma<3, 4, 2, false, 2, false, 0, false, 1, false, true>>(kn, c, pp);
            default: return run_policy<W4A8Mma<4, 4, 2, false, 2, false, 0, false, 1, false, true>>(kn, c, pp);
        }
    }
    if (!DUMP && env_or("FM_STREAM_M_CFG", 1) != 0) {    // (5: rows / grid per CTA whatever the row count)
        switch (p.M) {
            case 2: return run_policy<W4A8Mma<2, 4, 2, false, 2, false, 0, false>>(kn, c, pp);
            case 3: return run_policy<W4A8Mma<3, 4, 2, false, 2, false, 0, false>>(kn, c, pp);
            default: return run_policy<W4A8Mma<4, 4, 2, false, 2, false, 0, false>>(kn, c, pp);
        }
    }
    switch (p.M) {
        case 2: return run_policy<W4A8Mma<2, 4, 1, false, 2, true, 0, DUMP>>(kn, c, pp);
        case 3: return run_policy<W4A8Mma<3, 4, 1, false, 2, true, 0, DUMP>>(kn, c, pp);
        default: return run_policy<W4A8Mma<4, 4, 1, false, 2, true, 0, DUMP>>(kn, c, pp);
    }
}

// w4a4_decode_stream_m(common..., aq, asc, M, ystride, flags): M = 2..4 tokens per layer on the W4A4 tensor-core
// consumer.  aq / asc hold [nlayers * M] tokens (one 2-D quant_act4 launch with grid y = nlayers * M over
// x[nlayers][M][K]); y and the table's row_base argument as for w4a8_decode_stream_m.
// w4a4_decode_stream_m_iacc(..., flags, iacc): iacc int32 [nlayers][M][rows][K/32].
template <bool DUMP>
int launch_w4a4_stream_m(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = DUMP ? "w4a4_decode_stream_m_iacc" : "w4a4_decode_stream_m";
    PlainParams pp = {};
    StreamParams& p = pp.s;
    const int M = arg_i32(a[10]);
    FM_REQUIRE(M >= 2 && M <= 4, kn, "M=%d: this kernel takes 2..4 tokens (w4a4_decode_stream takes one)", M);
    const int rc = parse_common(kn, c, a, a[12], p, M);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.asc = arg_ptr<const uint8_t>(a[9]);
    p.ystride = arg_i32(a[11]);
    FM_REQUIRE(p.ystride >= p.row_base + p.rows && (long long)(p.M - 1) * p.ystride + p.row_base < (1LL << 31), kn,
               "ystride=%d must be at least row_base + rows = %d", p.ystride, p.row_base + p.rows);
    const int vbase = p.row_base + (p.M - 1) * p.ystride;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, vbase, p.peer_delta, p.npeers, true), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d and the row_base "
               "argument row_base + (M - 1) * ystride = %d (or was overwritten, or a buffer it points into was freed since), "
               "or the peer offsets do not come from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers,
               p.rows, p.K, vbase);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.asc, 16), kn, "the activation code arrays must be 16-byte aligned");
    const size_t tokens = (size_t)p.nlayers * p.M;
    FM_RANGE(p.ae, tokens * (p.K / 2), kn, "aq");
    FM_RANGE(p.asc, tokens * (p.K / 32) * 4, kn, "asc");
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[13]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, tokens * p.rows * (p.K / 32) * 4, kn, "iacc");
    }
    // four stages where they fit beside the tokens' codes (3200 bytes per token and stage), three at M = 4
    const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
    if (!DUMP && whole_stages(p.rows, grid) && env_or("FM_STREAM_M_CFG", 1) != 5) {
        switch (p.M) {
            case 2: return run_policy<W4A4Mma<4, 2, false, 2, 2, true>>(kn, c, pp);
            case 3: return run_policy<W4A4Mma<4, 2, false, 2, 3, true>>(kn, c, pp);
            default: return run_policy<W4A4Mma<3, 2, false, 1, 4, true>>(kn, c, pp);
        }
    }
    switch (p.M) {
        case 2: return run_policy<W4A4Mma<4, 2, DUMP, 2, 2>>(kn, c, pp);
        case 3: return run_policy<W4A4Mma<4, 2, DUMP, 2, 3>>(kn, c, pp);
        default: return run_policy<W4A4Mma<3, 2, DUMP, 1, 4>>(kn, c, pp);
    }
}

// nvfp4_decode_stream(common..., qa, qb, sc, gscale, flags): the layer table's ws entries are the E4M3 block scales
// [rows][K/16] (the table must have been validated with room for them: fm_stream_table records how many bytes follow
// every ws pointer inside its allocation); qa / qb / sc are nvfp4_quant_act's outputs for all layers: [nlayers][K/2],
// [nlayers][K/2], [nlayers][K/16].  nvfp4_decode_stream_iacc(..., flags, iacc): iacc int32 [nlayers][rows][K/16].
// $FM_NVFP4_CFG=1 selects the dp4a consumer, 0 / 2 the mma.sync consumer (one / two groups), for the run and for the dump.
template <bool DUMP>
int launch_nvfp4_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = DUMP ? "nvfp4_decode_stream_iacc" : "nvfp4_decode_stream";
    Nvfp4Params pp = {};
    StreamParams& p = pp.s;
    const int rc = parse_common(kn, c, a, a[12], p, 1);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    pp.gscale = arg_f32(a[11]);
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers, false,
                               (size_t)p.rows * (p.K / 16)), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d (or was "
               "overwritten, or a buffer it points into was freed since), a ws entry has fewer than rows*K/16 bytes behind it, "
               "or the peer offsets do not come from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers,
               p.rows, p.K, p.row_base);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.ao, 16) && aligned(p.asc, 16), kn, "the activation code arrays must be 16-byte aligned");
    FM_RANGE(p.ae, (size_t)p.nlayers * (p.K / 2), kn, "qa");
    FM_RANGE(p.ao, (size_t)p.nlayers * (p.K / 2), kn, "qb");
    FM_RANGE(p.asc, (size_t)p.nlayers * (p.K / 16) * 4, kn, "sc");
    // Default (3): the tcgen05 consumer of nvfp4_tc_stream.cu — the codes go from HBM to the MMA without an instruction.
    // Measured per 17408 x 5120 layer (64 layers per launch, burst): dp4a (1) 10.1 us, mma.sync consumer 10.2 (two
    // groups, 2) - 10.9 us (one group, 0): those three are bound by the integer pipe (PRMT decode).
    const bool forced = getenv("FM_NVFP4_CFG") != nullptr;
    int cfg = env_or("FM_NVFP4_CFG", 3);
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[13]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, (size_t)p.nlayers * p.rows * (p.K / 16) * 4, kn, "iacc");
    }
    if (cfg == 3) {
        const int rc3 = nvfp4_tc_stream(kn, c, p, pp.gscale, DUMP);
        if (rc3 <= 0) return rc3;
        FM_REQUIRE(!forced, kn, "FM_NVFP4_CFG=3: the tcgen05 consumer cannot take this launch (the table has no tensor maps: the driver "
                   "refused the encoding; or the workspace is too small)");
        cfg = 1;                                             // no tensor maps for this table: the dp4a consumer
    }
    if (DUMP) return cfg == 1 ? run_policy<Nvfp4Dp4a<5, 2, true>>(kn, c, pp) : run_policy<Nvfp4Mma<4, 1, 2, true>>(kn, c, pp);
    switch (cfg) {
        case 0: return run_policy<Nvfp4Mma<4, 1, 2, false>>(kn, c, pp);      // mma.sync, one consumer group
        case 2: return run_policy<Nvfp4Mma<4, 2, 2, false>>(kn, c, pp);      // mma.sync, two consumer groups
        default: return run_policy<Nvfp4Dp4a<5, 2, false>>(kn, c, pp);
    }
}

// nvfp4_decode_stream_m(common..., qa, qb, sc, gscale, M, ystride, flags): M = 2..4 tokens per layer on the tcgen05
// consumer (a token is 12 more columns of B; the weights are streamed once).  The code arrays hold [nlayers * M] tokens
// (one 2-D nvfp4_quant_act launch with grid y = nlayers * M over x[nlayers][M][K]); y of a layer is token-major,
// y[token * ystride + row_base + row]; the table must have been validated with row_base + (M - 1) * ystride as its
// row_base argument, as for w4a8_decode_stream_m.  nvfp4_decode_stream_m_iacc(..., flags, iacc): iacc int32
// [nlayers][M][rows][K/16].  There is no other consumer behind this entry: -4 when the table has no tensor maps.
template <bool DUMP>
int launch_nvfp4_stream_m(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = DUMP ? "nvfp4_decode_stream_m_iacc" : "nvfp4_decode_stream_m";
    Nvfp4Params pp = {};
    StreamParams& p = pp.s;
    const int M = arg_i32(a[12]);
    FM_REQUIRE(M >= 2 && M <= 4, kn, "M=%d: this kernel takes 2..4 tokens (nvfp4_decode_stream takes one)", M);
    const int rc = parse_common(kn, c, a, a[14], p, M);
    if (rc) return rc < 0 ? rc : FM_OK;
    p.ae = arg_ptr<const uint8_t>(a[8]);
    p.ao = arg_ptr<const uint8_t>(a[9]);
    p.asc = arg_ptr<const uint8_t>(a[10]);
    pp.gscale = arg_f32(a[11]);
    p.ystride = arg_i32(a[13]);
    FM_REQUIRE(p.ystride >= p.row_base + p.rows && (long long)(p.M - 1) * p.ystride + p.row_base < (1LL << 31), kn,
               "ystride=%d must be at least row_base + rows = %d", p.ystride, p.row_base + p.rows);
    const int vbase = p.row_base + (p.M - 1) * p.ystride;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, vbase, p.peer_delta, p.npeers, true,
                               (size_t)p.rows * (p.K / 16)), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d and the row_base argument "
               "row_base + (M - 1) * ystride = %d (or was overwritten, or a buffer it points into was freed since), a ws entry has "
               "fewer than rows*K/16 bytes behind it, or the peer offsets do not come from fm_stream_peers for its outputs",
               (const void*)p.layers, p.nlayers, p.rows, p.K, vbase);
    FM_REQUIRE(aligned(p.ae, 16) && aligned(p.ao, 16) && aligned(p.asc, 16), kn, "the activation code arrays must be 16-byte aligned");
    const size_t tokens = (size_t)p.nlayers * p.M;
    FM_RANGE(p.ae, tokens * (p.K / 2), kn, "qa");
    FM_RANGE(p.ao, tokens * (p.K / 2), kn, "qb");
    FM_RANGE(p.asc, tokens * (p.K / 16) * 4, kn, "sc");
    if (DUMP) {
        p.iacc = arg_ptr<int>(a[15]);
        FM_REQUIRE(aligned(p.iacc, 4), kn, "misaligned accumulator dump");
        FM_RANGE(p.iacc, tokens * p.rows * (p.K / 16) * 4, kn, "iacc");
    }
    const int rc3 = nvfp4_tc_stream(kn, c, p, pp.gscale, DUMP);
    FM_REQUIRE(rc3 <= 0, kn, "the tcgen05 consumer cannot take this launch (the table has no tensor maps, K is not a multiple of "
               "1024, or the workspace is too small)");
    return rc3;
}

// w4a16_decode_stream(common..., flags): the table's x entries (fp32 activations [K] per layer) are read here —
// fm_stream_table must have seen a valid x for every layer —, wq are compressed-tensors codes, ws bf16 scales.
// Launches the split kernel (grid y = layer) into the engine workspace (30 720 bytes per layer), then the stream kernel.
int launch_w4a16_stream(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "w4a16_decode_stream";
    W4a16Params pp = {};
    StreamParams& p = pp.s;
    const int rc = parse_common(kn, c, a, a[8], p, 1);
    if (rc) return rc < 0 ? rc : FM_OK;
    FM_REQUIRE(stream_table_ok(p.layers, p.nlayers, p.rows, p.K, p.row_base, p.peer_delta, p.npeers, false, 0, true), kn,
               "the layer table at %p was not filled by fm_stream_table for nlayers=%d rows=%d K=%d row_base=%d (or was "
               "overwritten, or a buffer it points into was freed since), an x entry is missing, or the peer offsets do not "
               "come from fm_stream_peers for its outputs", (const void*)p.layers, p.nlayers, p.rows, p.K, p.row_base);
    constexpr int NG = 40;
    uint32_t* frags = static_cast<uint32_t*>(engine_scratch((size_t)p.nlayers * NG * 192 * 4));
    FM_REQUIRE(frags != nullptr, kn, "the engine workspace cannot hold %d x 30720 bytes here (FM_SCRATCH_MB, or a first use "
               "inside a graph capture)", p.nlayers);
    pp.frags = frags;
    cudaError_t e = launch_kernel(w4a16_split_layers_kernel, dim3((NG * 192 + 255) / 256, p.nlayers), dim3(256), 0, c.stream,
                                  pdl_enabled(), p.layers, frags, (uint32_t)NG);
    if (e != cudaSuccess) return cuda_fail(kn, e);
    after_launch(kn);
    // Two consumer groups reading the fragments from the layer's tile; $FM_W4A16_CFG=0: one group with the fragments
    // of the layer in registers.
    if (env_or("FM_W4A16_CFG", 1) == 0) return run_policy<W4A16Mma<3, 1, 2, true>>(kn, c, pp);
    const int grid = c.sm_count < p.rows ? c.sm_count : p.rows;
    if (whole_stages(p.rows, grid) && env_or("FM_W4A16_CFG", 1) != 5) return run_policy<W4A16Mma<3, 2, 2, false, true>>(kn, c, pp);
    return run_policy<W4A16Mma<3, 2, 2, false>>(kn, c, pp);
}

// stream_flag_wait(flags, nlayers, target, status, spins)
int launch_flag_wait(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "stream_flag_wait";
    const unsigned* flags = arg_ptr<const unsigned>(a[0]);
    const int nlayers = arg_i32(a[1]);
    const unsigned target = arg_u32(a[2]);
    int* status = arg_ptr<int>(a[3]);
    const int spins = arg_i32(a[4]);
    FM_REQUIRE(nlayers > 0 && spins > 0 && spins <= (1 << 21), kn, "nlayers=%d spins=%d: spins must be 1..2097152 (about two seconds)", nlayers, spins);
    FM_REQUIRE(aligned(flags, 4) && aligned(status, 4), kn, "misaligned flags or status");
    FM_RANGE(flags, (size_t)nlayers * 4, kn, "flags");
    FM_RANGE(status, 4, kn, "status");
    cudaError_t e = launch_kernel(stream_flag_wait_kernel, dim3((nlayers + 127) / 128), dim3(128), 0, c.stream, false, flags,
                                  nlayers, target, status, spins);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kStream[] = {
    {"w4a8_decode_stream", 13, launch_w4_stream<false, false>, "piiiiippppppp"},
    {"w4a4_decode_stream", 11, launch_w4_stream<true, false>, "piiiiippppp"},
    {"w4a8_decode_stream_m", 15, launch_w4a8_stream_m<false>, "piiiiippppppiip"},
    {"w4a4_decode_stream_m", 13, launch_w4a4_stream_m<false>, "piiiiippppiip"},
    {"nvfp4_decode_stream", 13, launch_nvfp4_stream<false>, "piiiiipppppfp"},
    {"w4a16_decode_stream", 9, launch_w4a16_stream, "piiiiippp"},
    {"w4a8_decode_stream_iacc", 14, launch_w4_stream<false, true>, "piiiiipppppppp"},
    {"w4a4_decode_stream_iacc", 12, launch_w4_stream<true, true>, "piiiiipppppp"},
    {"w4a8_decode_stream_m_iacc", 16, launch_w4a8_stream_m<true>, "piiiiippppppiipp"},
    {"w4a4_decode_stream_m_iacc", 14, launch_w4a4_stream_m<true>, "piiiiippppiipp"},
    {"nvfp4_decode_stream_iacc", 14, launch_nvfp4_stream<true>, "piiiiipppppfpp"},
    {"stream_flag_wait", 5, launch_flag_wait, "piipi"},
    {"w4a8_stream_read_ceiling", 13, launch_w4a8_read_ceiling, "piiiiippppppp"},
    {"nvfp4_decode_stream_m", 15, launch_nvfp4_stream_m<false>, "piiiiipppppfiip"},
    {"nvfp4_decode_stream_m_iacc", 16, launch_nvfp4_stream_m<true>, "piiiiipppppfiipp"},
    {"w4a8_layers_stream", 7, launch_w4a8_layers_stream, "ppiippp"},
};

// Status word of the ring kernels when they are launched by name for a single layer (those entries have
// no status argument): 0, or the code of the first bounded wait that ran out.  Read and cleared by fm_stream_status().
__device__ int g_stream_status;

int* byname_status() {
    static int* ptr = nullptr;
    if (!ptr && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_stream_status) != cudaSuccess) {
        cudaGetLastError();
        ptr = nullptr;
    }
    return ptr;
}

void one_layer(StreamParams& p, const void* wq, const void* ws, float* y, int rows, int M, int ystride) {
    p.layers = nullptr;
    p.one.wq = static_cast<const uint8_t*>(wq);
    p.one.ws = static_cast<const uint8_t*>(ws);
    p.one.x = nullptr;
    p.one.y = y;
    p.nlayers = 1;
    p.rows = rows;
    p.K = 5120;
    p.row_base = 0;
    p.npeers = 0;
    p.M = M;
    p.ystride = ystride;
    p.status = byname_status();
}

}  // namespace

// ---- single-layer launches of the ring kernels for the by-name GEMV entries (K = 5120, 16-byte aligned operands;
// the callers have range-checked every pointer).  y is token-major with `ystride` floats between tokens.
int stream_gemv_w4a8(const LaunchCtx& c, const char* kn, const void* wq, const void* ws, const void* ae, const void* ao,
                     const void* asc, const void* asu, float* y, int M, int ystride, int rows, int* iacc) {
    PlainParams pp = {};
    one_layer(pp.s, wq, ws, y, rows, M, ystride);
    FM_REQUIRE(pp.s.status != nullptr, kn, "the status word of the ring kernels is not addressable");
    pp.s.ae = static_cast<const uint8_t*>(ae);
    pp.s.ao = static_cast<const uint8_t*>(ao);
    pp.s.asc = static_cast<const uint8_t*>(asc);
    pp.s.asu = static_cast<const uint8_t*>(asu);
    pp.s.iacc = iacc;
    if (iacc) {
        switch (M) {
            case 1: return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, true>>(kn, c, pp);
            case 2: return run_policy<W4A8Mma<2, 4, 1, false, 2, true, 0, true>>(kn, c, pp);
            case 3: return run_policy<W4A8Mma<3, 4, 1, false, 2, true, 0, true>>(kn, c, pp);
            default: return run_policy<W4A8Mma<4, 4, 1, false, 2, true, 0, true>>(kn, c, pp);
        }
    }
    switch (M) {
        case 1: return run_policy<W4A8Mma<1, 4, 2, true, 1, false, 0, false>>(kn, c, pp);
        case 2: return run_policy<W4A8Mma<2, 4, 1, false, 2, true, 0, false>>(kn, c, pp);
        case 3: return run_policy<W4A8Mma<3, 4, 1, false, 2, true, 0, false>>(kn, c, pp);
        default: return run_policy<W4A8Mma<4, 4, 1, false, 2, true, 0, false>>(kn, c, pp);
    }
}

// The same for gemv_w4a4<2..4> and its r2 names: aq [M][K/2] packed nibbles, asc [M][K/32]; iacc [M][rows][K/32].
int stream_gemv_w4a4(const LaunchCtx& c, const char* kn, const void* wq, const void* ws, const void* aq, const void* asc,
                     float* y, int M, int ystride, int rows, int* iacc) {
    PlainParams pp = {};
    one_layer(pp.s, wq, ws, y, rows, M, ystride);
    FM_REQUIRE(pp.s.status != nullptr, kn, "the status word of the ring kernels is not addressable");
    FM_REQUIRE(M >= 2 && M <= 4, kn, "M=%d: the ring takes 2..4 tokens here", M);
    pp.s.ae = static_cast<const uint8_t*>(aq);
    pp.s.asc = static_cast<const uint8_t*>(asc);
    pp.s.iacc = iacc;
    if (iacc) {
        switch (M) {
            case 2: return run_policy<W4A4Mma<4, 2, true, 2, 2>>(kn, c, pp);
            case 3: return run_policy<W4A4Mma<4, 2, true, 2, 3>>(kn, c, pp);
            default: return run_policy<W4A4Mma<3, 2, true, 1, 4>>(kn, c, pp);
        }
    }
    switch (M) {
        case 2: return run_policy<W4A4Mma<4, 2, false, 2, 2>>(kn, c, pp);
        case 3: return run_policy<W4A4Mma<4, 2, false, 2, 3>>(kn, c, pp);
        default: return run_policy<W4A4Mma<3, 2, false, 1, 4>>(kn, c, pp);
    }
}

int stream_read_status(cudaStream_t stream) {
    int v = 0, zero = 0;
    if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
    return v;
}

const KernelEntry* stream_kernels(int* n) {
    *n = (int)(sizeof(kStream) / sizeof(kStream[0]));
    return kStream;
}

}  // namespace fm
