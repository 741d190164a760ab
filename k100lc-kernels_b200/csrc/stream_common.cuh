// Shared skeleton of the multi-layer decode stream kernels (decode_stream.cu): one persistent launch
// walks a stack of independent layers, CTA c owning the same contiguous row range of every layer.
//
//   producer warp (one lane)   issues 1-D bulk async copies (cp.async.bulk, never multicast) of ROWS weight
//                              rows + their scales into a ring of shared-memory stages, completion counted
//                              on an mbarrier per stage, and the token's activation codes of each layer
//                              either into a small ring of tiles of their own or into every stage;
//   consumer warps             one or two groups that take the stages in turn; what a group does with a
//                              stage is the policy (dp4a or mma.sync arithmetic of one quantisation format);
//   writer warp                collects nothing itself: the consumers put a CTA's y values of a layer into a
//                              shared-memory tile and the writer stores it once per layer, coalesced, to the
//                              local y and to every additional receiver (other GPUs' y over NVLink peer
//                              mappings, a pinned host buffer), then bumps the layer's completion counter
//                              on every receiver.
//
// Every wait on an mbarrier is bounded.  A wait that runs out records its code in *status, raises a
// CTA-wide abort flag that every other wait polls, and all roles fall through to a common exit: the
// producer first waits (bounded again) for the copies it has already issued, so that no bulk copy is
// still landing in this CTA's shared memory when the CTA gives it up.
#pragma once
#include "stage_split.h"
#include <stdint.h>

#include <type_traits>

#include "device_utils.cuh"

namespace fm {
namespace stream {

constexpr int kSpinLimit = 1 << 20;    // try_wait rounds (each may sleep up to the suspend hint) before a wait gives up
constexpr int kOutCap = 512;           // y values of one layer that a CTA collects in shared memory (else stored one by one)
constexpr int kMaxStages = 8;
constexpr int kYBufs = 4;              // output tiles of a CTA: the writer may lag the consumers by up to three layers
constexpr int kHeader = 512;           // bytes reserved for the barriers at the start of the dynamic shared memory

struct StreamLayer {                   // one entry of the device-side layer table (32 bytes)
    const uint8_t* wq;                 // [rows][K/2] packed 4-bit codes
    const uint8_t* ws;                 // [rows][..] weight scales (f16 / bf16 per 128, or E4M3 per 16)
    const float* x;                    // [K] fp32 activations of this layer (read by the W4A16 kernel only)
    float* y;                          // [>= row_base + rows] fp32 output of this layer
};

// Per-layer shape of a table whose layers differ (the policies that declare VAR).  A layer here is 5120 k of a set of
// weight rows: a weight matrix with longer rows is several such layers over the same rows, the second and later ones
// adding to y (`accumulate`); rows may be `wpitch` bytes apart with `wbytes` valid bytes in this chunk.
struct VarLayer {                      // 64 bytes
    const uint8_t *ae, *ao, *asc, *asu;   // the token's codes of this chunk: 2560 + 2560 bytes, 40 scales, 40 sums (zero behind the row's K)
    int rows;                          // weight rows of this layer
    int wpitch, spitch;                // bytes between the rows of wq / ws
    int wbytes, sbytes;                // valid bytes of a row of wq / ws in this chunk (2560 / 80 for a full chunk)
    int accumulate;                    // 0: y = value; 1: y += value
    int row_base;                      // first output index of these rows inside the layer's y
    int chunk;                         // which 5120 k of the row this layer is (its wq / ws point at that chunk of row 0)
};

struct StreamParams {
    const StreamLayer* layers;         // device table, or nullptr: the single layer `one`
    const VarLayer* var;               // per-layer shapes (VAR policies), else nullptr: `rows` and `row_base` below for all
    const void* chunk_maps;            // VAR: two TMA maps (128 bytes each: weights, scales) per layer that is a chunk of longer rows, or nullptr
    const uint8_t *ae, *ao, *asc, *asu;   // activation-quantiser outputs of all layers (meaning depends on the format)
    int nlayers, rows, K, row_base;
    int npeers;                        // additional receivers of y (0 on one GPU)
    const long long* peer_delta;       // [npeers] byte offset from a local y address to the receiver's copy
    int* status;                       // 0 ok, else the code of the first wait that ran out
    int M, ystride;                    // tokens per layer and floats between their outputs (token-major y)
    int* iacc;                         // accumulator dump (parity tests): [nlayers][M][rows][units per row]
    unsigned* flags;                   // optional [nlayers] completion counters, +1 per CTA and layer on every receiver
    uint32_t wait_hint_ns;             // suspend-time hint of the barrier waits (0: none)
    StreamLayer one;
};

__device__ __forceinline__ StreamLayer get_layer(const StreamParams& p, int l) { return p.layers ? p.layers[l] : p.one; }

struct Bars {
    uint64_t full[kMaxStages];         // a stage's bytes have landed
    uint64_t empty[kMaxStages];        // its consumers have used them
    uint64_t act_ready[kMaxStages];    // a layer's activation tile has landed (tiles of their own only)
    uint64_t act_free[kMaxStages];     // every consumer warp is done with it
    uint64_t red_full[4], red_free[4]; // partial-sum tiles of the tensor-core consumers (two per group)
    uint64_t ydone[kYBufs], yfree[kYBufs];   // output tile complete / written out
    volatile int abort;
    uint32_t seen[kMaxStages];         // fills of a slot that some consumer has seen land (stage_wait)
};
static_assert(sizeof(Bars) <= kHeader, "barrier block");

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
// one round of waiting: with a hint the thread may sleep up to that many nanoseconds inside the instruction
// instead of spinning through the issue slots
__device__ __forceinline__ bool mbar_try_wait(uint64_t* b, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    if (hint_ns)
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_u32(b)), "r"(parity), "r"(hint_ns) : "memory");
    else
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(smem_u32(b)), "r"(parity) : "memory");
    return ok != 0;
}
// Pins a value in program order: volatile statements are not reordered with each other, so an
// mbarrier.arrive that follows cannot be scheduled ahead of the arithmetic that produced `v`
// (and with it ahead of the shared-memory loads that arithmetic consumed).
__device__ __forceinline__ void consumed(float v) { asm volatile("" ::"f"(v) : "memory"); }
// tiled TMA copies (never multicast) global -> this CTA's shared memory
__device__ __forceinline__ void tma_g2s_3d(void* dst, const void* map, int x, int y, int z, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_g2s_2d(void* dst, const void* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// 1-D bulk async copy global -> this CTA's shared memory
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// What every role of a CTA needs.
struct Cta {
    const StreamParams* p;
    Bars* bars;
    uint8_t* ring;
    uint8_t* act;
    float* red;
    float* ytile;
    uint8_t* extra;
    int warp, lane;
    int r0, r1, nst;                   // this CTA's rows [r0, r1) of every layer = nst stages
    bool tiled;                        // its y values of a layer fit the output tile
    uint32_t hint;
};

// bounded wait that also gives up when another role has raised the abort flag
__device__ __forceinline__ bool cta_wait(const Cta& c, uint64_t* bar, uint32_t parity, int code) {
    for (int i = 0; i < kSpinLimit; i++) {
        if (mbar_try_wait(bar, parity, c.hint)) return true;
        if ((i & 7) == 7 && c.bars->abort) return false;
    }
    c.bars->abort = 1;
    atomicCAS(c.p->status, 0, code);
    return false;
}
// A consumer group waits until stage `cc` (counted over the whole launch) has landed in its ring slot.  A parity wait
// tells "this fill has landed" from "the fill before it has not landed yet" only for a waiter that knows that the fill
// before has landed.  The groups take the stages in turn, so when STAGES is not a multiple of NGROUPS the fill before
// was another group's: whoever sees a fill land writes its number beside the barrier, and a group reads that number
// before it trusts the parity (the fill it waits for cannot be issued before that group released the slot, so this
// adds no dependence).
template <class P>
__device__ __forceinline__ bool stage_wait(const Cta& c, int cc) {
    const int s = cc % P::STAGES, ph = cc / P::STAGES;
    constexpr bool kShared = P::STAGES % P::NGROUPS != 0;
    if constexpr (kShared) {
        const uint32_t addr = smem_u32(&c.bars->seen[s]);
        for (int i = 0; ph > 0; i++) {
            uint32_t v;
            asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
            if (v >= (uint32_t)ph) break;
            if ((i & 7) == 7 && c.bars->abort) return false;
            if (i >= kSpinLimit) {
                c.bars->abort = 1;
                atomicCAS(c.p->status, 0, 3);
                return false;
            }
        }
    }
    if (!cta_wait(c, &c.bars->full[s], ph & 1, 3)) return false;
    if constexpr (kShared) {
        if (c.lane == 0 && c.warp % P::CW == 0)            // one warp of the group speaks for it
            asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&c.bars->seen[s])), "r"((uint32_t)ph + 1u) : "memory");
    }
    return true;
}
// the same without a report: used on the way out, for copies that are still in flight
__device__ __forceinline__ void quiet_wait(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < kSpinLimit && !mbar_try_wait(bar, parity, 1000u); i++) {}
}

// Status codes: 1 ring slot not freed (producer), 2 activation tile not landed, 3 stage not landed,
// 4 activation tile not freed, 5 / 6 partial-sum tile, 7 output tile not written, 8 output tile not complete.

// A policy may declare `static constexpr bool VAR = true`: the layers of its table have shapes of their own
// (StreamParams::var), and every role recomputes this CTA's rows and stages at the start of each layer.
template <class P, class = void> struct is_var : std::false_type {};
template <class P> struct is_var<P, std::void_t<decltype(P::VAR)>> : std::bool_constant<P::VAR> {};

// Rows of a layer with a shape of its own that this CTA takes.  Whole stages are dealt out, not rows: with rows / grid
// a CTA's last stage of every layer is a partial one, and a stage costs its hand-overs however few rows it holds
// (5120 rows on 148 CTAs: 2.16 stages per CTA instead of three).  The CTAs that get one stage more than the others
// start at a position that moves with the weight matrix (`first`: the table index of its first chunk, so that all
// chunks of a matrix — which add to the same y — are split alike), which spreads those stages evenly over the launch.
template <int ROWS>
__device__ __forceinline__ void var_rows(int rows, int first, int& r0, int& r1) {
    stage_split(rows, first, (int)gridDim.x, (int)blockIdx.x, ROWS, &r0, &r1);     // stage_split.h
}
// A policy may also declare `static constexpr bool ROT = true`: all layers have the table's one shape, and the CTA's
// rows are dealt out per layer as above (the position moves with the layer).
template <class P, class = void> struct is_rot : std::false_type {};
template <class P> struct is_rot<P, std::void_t<decltype(P::ROT)>> : std::bool_constant<P::ROT> {};
template <class P>
__device__ __forceinline__ void set_geom(Cta& c, int l) {
    if constexpr (is_var<P>::value) {
        const VarLayer& v = c.p->var[l];
        var_rows<P::ROWS>(v.rows, l - v.chunk, c.r0, c.r1);
        c.nst = (c.r1 - c.r0 + P::ROWS - 1) / P::ROWS;
    } else if constexpr (is_rot<P>::value) {
        var_rows<P::ROWS>(c.p->rows, l, c.r0, c.r1);
        c.nst = (c.r1 - c.r0 + P::ROWS - 1) / P::ROWS;
    }
}

// ---- producer ------------------------------------------------------------------------------
// P supplies: ROWS, STAGES, PITCH, ROWB, SCB, STAGE_W, STAGE, ACT, NACT, ACT_IN_STAGE, OFF_ACT and
// copy_act(pp, layer, dst, bar), which issues bulk copies of exactly ACT bytes.
// `pl` of P::NPROD producer lanes: with the codes inside every stage a stage is self-contained, and the stages can go
// round several lanes (each is a chain of a barrier wait and half a dozen copy instructions per stage, which paces
// the ring when a CTA has a single small stage per layer).
template <class P>
__device__ __forceinline__ void run_producer(const Cta& cta, const typename P::Params& pp, int pl) {
    Cta c = cta;                       // rows and stages of this CTA change with the layer when the shapes do
    const StreamParams& p = *c.p;
    Bars* B = c.bars;
    static_assert(P::NPROD == 1 || P::ACT_IN_STAGE, "several producer lanes need self-contained stages");
    // a ring slot belongs to one lane: a lane that met a slot only every other round could not tell its phases apart
    static_assert(P::STAGES % P::NPROD == 0, "the producer lanes must divide the ring");
    int issued = 0, acts = 0;          // stages armed by any lane up to this lane's last one / activation tiles armed
    bool ok = true;
    auto copy_tile = [&](int l) -> bool {          // layer l's codes -> tile l % NACT
        const int b = l % P::NACT;
        if (l >= P::NACT && !cta_wait(c, &B->act_free[b], ((l / P::NACT) & 1) ^ 1, 4)) return false;
        mbar_expect_tx(&B->act_ready[b], P::ACT);
        P::copy_act(pp, l, c.act + (size_t)b * P::ACT, &B->act_ready[b]);
        acts = l + 1;
        return true;
    };
    // A layer's codes are copied right before its first stage, into tile l % NACT: that tile was last used
    // by layer l - NACT, and the ring keeps the consumers at most STAGES stages behind, so with
    // NACT > STAGES / (stages per layer) + 1 tiles the copy never waits for them (the launcher picks NACT).
    // The table entries of the next two layers are requested ahead of their use: with one stage per layer (a
    // row shard of eight GPUs) a dependent 32-byte load per layer would otherwise cost this thread a trip to
    // L2 — most of a stage time — before it can issue anything.
    int cc = 0;
    VarLayer vnext = {};
    if constexpr (is_var<P>::value) vnext = p.var[0];
    StreamLayer lay = get_layer(p, 0), lay1 = get_layer(p, min(1, p.nlayers - 1)), lay2;
    for (int l = 0; ok && l < p.nlayers; l++, lay = lay1, lay1 = lay2) {
        lay2 = get_layer(p, min(l + 2, p.nlayers - 1));
        VarLayer vl = {};
        if constexpr (is_var<P>::value) {                  // this layer's shape was requested a layer ago
            vl = vnext;
            vnext = p.var[min(l + 1, p.nlayers - 1)];
            var_rows<P::ROWS>(vl.rows, l - vl.chunk, c.r0, c.r1);
            c.nst = (c.r1 - c.r0 + P::ROWS - 1) / P::ROWS;
        } else if constexpr (is_rot<P>::value) {
            set_geom<P>(c, l);
        }
        if (!P::ACT_IN_STAGE && !copy_tile(l)) { ok = false; break; }
        for (int j = 0; j < c.nst; j++, cc++) {
            if (P::NPROD > 1 && cc % P::NPROD != pl) continue;
            const int s = cc % P::STAGES;
            if (cc >= P::STAGES && !cta_wait(c, &B->empty[s], ((cc / P::STAGES) & 1) ^ 1, 1)) { ok = false; break; }
            const int row = c.r0 + j * P::ROWS;
            const int nr = min(P::ROWS, c.r1 - row);
            uint8_t* dst = c.ring + (size_t)s * P::STAGE;
            if constexpr (is_var<P>::value) {
                // rows may be further apart than a chunk is wide, and the last chunk of a row may be short: the rest of
                // the stage keeps what it held (finite numbers: the ring is cleared at the start), and the token's codes
                // behind the row's K are zero
                const bool strided = vl.wpitch != P::ROWB || vl.spitch != P::SCB;
                if (strided && nr == P::ROWS && p.chunk_maps) {
                    // a chunk of 16 longer rows: one box copy for the weights (pieces of the rows past their end read
                    // as zero), one for the scales
                    const uint8_t* maps = static_cast<const uint8_t*>(p.chunk_maps) + (size_t)l * 256;
                    mbar_expect_tx(&B->full[s], (uint32_t)(P::ROWS * (P::ROWB + P::SCB)) + P::ACT);
                    tma_g2s_3d(dst, maps, 0, vl.chunk * 5, row, &B->full[s]);
                    tma_g2s_2d(dst + P::STAGE_W, maps + 128, vl.chunk * 20, row, &B->full[s]);
                    P::copy_act(pp, l, dst + P::OFF_ACT, &B->full[s]);
                    issued = cc + 1;
                    continue;
                }
                mbar_expect_tx(&B->full[s], (uint32_t)(nr * (vl.wbytes + vl.sbytes)) + P::ACT);
                if (vl.wpitch == P::ROWB && vl.wbytes == P::ROWB) {
                    bulk_g2s(dst, lay.wq + (size_t)row * P::ROWB, (uint32_t)(nr * P::ROWB), &B->full[s]);
                } else {
                    for (int r = 0; r < nr; r++)
                        bulk_g2s(dst + (size_t)r * P::PITCH, lay.wq + (size_t)(row + r) * vl.wpitch, (uint32_t)vl.wbytes, &B->full[s]);
                }
                if (vl.spitch == P::SCB && vl.sbytes == P::SCB) {
                    bulk_g2s(dst + P::STAGE_W, lay.ws + (size_t)row * P::SCB, (uint32_t)(nr * P::SCB), &B->full[s]);
                } else {
                    for (int r = 0; r < nr; r++)
                        bulk_g2s(dst + P::STAGE_W + r * P::SCB, lay.ws + (size_t)(row + r) * vl.spitch, (uint32_t)vl.sbytes, &B->full[s]);
                }
                P::copy_act(pp, l, dst + P::OFF_ACT, &B->full[s]);
                issued = cc + 1;
                continue;
            }
            mbar_expect_tx(&B->full[s], (uint32_t)(nr * (P::ROWB + P::SCB)) + (P::ACT_IN_STAGE ? P::ACT : 0));
            if (P::PITCH == P::ROWB) {
                bulk_g2s(dst, lay.wq + (size_t)row * P::ROWB, (uint32_t)(nr * P::ROWB), &B->full[s]);
            } else {                                   // padded pitch: one copy per row
                for (int r = 0; r < nr; r++)
                    bulk_g2s(dst + (size_t)r * P::PITCH, lay.wq + (size_t)(row + r) * P::ROWB, P::ROWB, &B->full[s]);
            }
            bulk_g2s(dst + P::STAGE_W, lay.ws + (size_t)row * P::SCB, (uint32_t)(nr * P::SCB), &B->full[s]);
            if (P::ACT_IN_STAGE) P::copy_act(pp, l, dst + P::OFF_ACT, &B->full[s]);
            issued = cc + 1;
        }
    }
    if (!ok) {
        // leaving early: what was issued must have landed before the CTA's shared memory is given up
        for (int j = issued > P::STAGES ? issued - P::STAGES : 0; j < issued; j++)
            if (j % P::NPROD == pl) quiet_wait(&B->full[j % P::STAGES], (j / P::STAGES) & 1);
        if (!P::ACT_IN_STAGE)
            for (int l = acts > P::NACT ? acts - P::NACT : 0; l < acts; l++)
                quiet_wait(&B->act_ready[l % P::NACT], (l / P::NACT) & 1);
    }
}

// ---- writer --------------------------------------------------------------------------------
// tile layout [row][token]; y of a layer is token-major: y[token * ystride + row].  `delta` are the receivers' byte
// offsets, held in registers: read from global memory inside the loop they cost a dependent load per receiver and
// layer, which is more than a stage time when a CTA has one stage per layer.
// `add`: the tile is added to what y holds (the later chunks of a row that is longer than a layer's 5120 k; the same
// lane wrote that value, in program order, when it handled the chunk before).
template <int M>
__device__ __forceinline__ void write_out(const StreamParams& p, const float* tile, float* y, int n, int lane,
                                          const long long (&delta)[8], bool add = false) {
    for (int i = lane; i < n * M; i += 32) {
        const int tok = M == 1 ? 0 : i / n, row = M == 1 ? i : i - tok * n;      // token-major walk: coalesced stores
        float* dst = y + (size_t)tok * p.ystride + row;
        const float v = add ? *dst + tile[row * M + tok] : tile[row * M + tok];
        *dst = v;
#pragma unroll
        for (int q = 0; q < 8; q++)
            if (q < p.npeers) *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + delta[q]) = v;
    }
}

template <class P>
__device__ __forceinline__ void run_writer(const Cta& cta) {
    Cta c = cta;
    const StreamParams& p = *c.p;
    if (!c.tiled) return;
    long long delta[8];
#pragma unroll
    for (int q = 0; q < 8; q++) delta[q] = q < p.npeers ? p.peer_delta[q] : 0;
    float* y_next = get_layer(p, 0).y;                   // requested a layer ahead (see the producer)
    for (int l = 0; l < p.nlayers; l++) {
        float* y_l = y_next;
        y_next = get_layer(p, min(l + 1, p.nlayers - 1)).y;
        const int b = l % kYBufs;
        set_geom<P>(c, l);
        int row_base = p.row_base;
        bool add = false;
        if constexpr (is_var<P>::value) {
            row_base = p.var[l].row_base;
            add = p.var[l].accumulate != 0;
        }
        if (!cta_wait(c, &c.bars->ydone[b], (l / kYBufs) & 1, 8)) return;
        write_out<P::M>(p, c.ytile + b * kOutCap, y_l + row_base + c.r0, c.r1 - c.r0, c.lane, delta, add);
        __syncwarp();
        if (c.lane == 0) mbar_arrive(&c.bars->yfree[b]);
        if (p.flags) {
            // the rows are visible everywhere before the counter of the layer moves: receiver 0 is
            // this GPU, receiver q > 0 the q-th additional copy
            __threadfence_system();
            __syncwarp();
            if (c.lane <= p.npeers) {
                unsigned* f = p.flags + l;
                if (c.lane > 0) f = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(f) + p.peer_delta[c.lane - 1]);
                asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(f) : "memory");
            }
        }
    }
    if (p.npeers) __threadfence_system();
}

// ---- consumer side of the layer protocol -----------------------------------------------------
// before the first stage of layer l that a warp works on
template <class P>
__device__ __forceinline__ bool layer_enter(const Cta& c, int l) {
    if (c.tiled && l >= kYBufs && !cta_wait(c, &c.bars->yfree[l % kYBufs], ((l / kYBufs) & 1) ^ 1, 7)) return false;
    if (!P::ACT_IN_STAGE && !cta_wait(c, &c.bars->act_ready[l % P::NACT], (l / P::NACT) & 1, 2)) return false;
    return true;
}
// the activation tile of layer l is no longer needed by this warp
template <class P>
__device__ __forceinline__ void act_release(const Cta& c, int l) {
    if (!P::ACT_IN_STAGE && c.lane == 0) mbar_arrive(&c.bars->act_free[l % P::NACT]);
}
// this warp has put its last y value of layer l into the tile
__device__ __forceinline__ void layer_done(const Cta& c, int l) {
    if (c.tiled) {
        __syncwarp();
        if (c.lane == 0) mbar_arrive(&c.bars->ydone[l % kYBufs]);
    }
}
// one y value: into the layer's tile `yt`, or (too many rows per CTA for the tile) straight to every receiver
template <int M>
__device__ __forceinline__ void emit(const Cta& c, float* yt, float* y, int row, int tok, float v) {
    const StreamParams& p = *c.p;
    if (c.tiled) {
        yt[(row - c.r0) * M + tok] = v;
    } else {
        float* dst = y + (size_t)tok * p.ystride + row;
        *dst = v;
        for (int q = 0; q < p.npeers; q++)
            *reinterpret_cast<float*>(reinterpret_cast<char*>(dst) + p.peer_delta[q]) = v;
    }
}

// A policy may declare `static constexpr bool NO_OUTPUT = true`: its consumers produce no y (the read-ceiling probe),
// so there is no output tile and the writer has nothing to do.
template <class P, class = void> struct no_output : std::false_type {};
template <class P> struct no_output<P, std::void_t<decltype(P::NO_OUTPUT)>> : std::bool_constant<P::NO_OUTPUT> {};

// ---- the kernel ------------------------------------------------------------------------------
// P supplies the geometry constants, Params (with a StreamParams member `s`), init_extra() and
// consume(cta, params, group, warp_in_group).
template <class P>
__global__ void __launch_bounds__(P::kThreads, 1)
stream_kernel(const typename P::Params pp) {
    const StreamParams& p = pp.s;
    extern __shared__ __align__(128) uint8_t smem[];
    Cta c;
    c.p = &p;
    c.bars = reinterpret_cast<Bars*>(smem);
    c.ring = smem + kHeader;
    c.act = c.ring + (size_t)P::STAGES * P::STAGE;
    c.red = reinterpret_cast<float*>(c.act + (P::ACT_IN_STAGE ? 0 : P::NACT * P::ACT));
    c.ytile = c.red + P::NGROUPS * 2 * P::RED;
    c.extra = reinterpret_cast<uint8_t*>(c.ytile + kYBufs * kOutCap);
    c.warp = threadIdx.x >> 5;
    c.lane = threadIdx.x & 31;
    c.hint = p.wait_hint_ns;
    constexpr int CW = P::CW, NCW = P::NGROUPS * CW;
    if (threadIdx.x == 0) {
        for (int s = 0; s < P::STAGES; s++) {
            mbar_init(&c.bars->full[s], 1);
            mbar_init(&c.bars->empty[s], CW);
        }
        for (int b = 0; b < P::NACT; b++) {
            mbar_init(&c.bars->act_ready[b], 1);
            mbar_init(&c.bars->act_free[b], NCW);
        }
        for (int b = 0; b < 4; b++) {
            mbar_init(&c.bars->red_full[b], CW);
            mbar_init(&c.bars->red_free[b], 1);
        }
        for (int b = 0; b < kYBufs; b++) {
            mbar_init(&c.bars->ydone[b], NCW);
            mbar_init(&c.bars->yfree[b], 1);
        }
        c.bars->abort = 0;
        for (int s = 0; s < P::STAGES; s++) c.bars->seen[s] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    P::init_extra(pp, c.extra);
    if constexpr (is_var<P>::value) {
        // a short chunk leaves the rest of its rows in the stage as it was: make sure that is never an uninitialised
        // bit pattern (a NaN scale times a zero activation scale would still be a NaN)
        for (int i = threadIdx.x; i < P::STAGES * P::STAGE / 16; i += blockDim.x)
            reinterpret_cast<uint4*>(c.ring)[i] = make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_wait();                                          // the codes come from the preceding quantiser launch

    c.r0 = (int)((long long)p.rows * blockIdx.x / gridDim.x);
    c.r1 = (int)((long long)p.rows * (blockIdx.x + 1) / gridDim.x);
    c.nst = (c.r1 - c.r0 + P::ROWS - 1) / P::ROWS;
    c.tiled = !no_output<P>::value && (is_var<P>::value || (c.r1 - c.r0) * P::M <= kOutCap);   // (the launcher of a VAR policy checks the tile)
    if constexpr (is_rot<P>::value) {                    // the most rows a layer can give this CTA
        const int most = ((p.rows + P::ROWS - 1) / P::ROWS + (int)gridDim.x - 1) / (int)gridDim.x * P::ROWS;
        c.tiled = !no_output<P>::value && most * P::M <= kOutCap;
    }

    if (c.warp >= NCW && c.warp < NCW + P::NPROD) {
        if (c.lane == 0) run_producer<P>(c, pp, c.warp - NCW);
    } else if (c.warp == NCW + P::NPROD) {
        run_writer<P>(c);
    } else {
        P::consume(c, pp, c.warp / CW, c.warp % CW);
        if (p.npeers && !c.tiled) __threadfence_system();    // direct peer stores are visible before the kernel ends
    }
    // common exit: nobody leaves while a copy issued by the producer may still be landing
    __syncthreads();
}

template <class P>
constexpr size_t smem_bytes() {
    return (size_t)kHeader + (size_t)P::STAGES * P::STAGE + (P::ACT_IN_STAGE ? 0 : (size_t)P::NACT * P::ACT) +
           (size_t)P::NGROUPS * 2 * P::RED * 4 + (size_t)kYBufs * kOutCap * 4 + P::EXTRA;
}

}  // namespace stream
}  // namespace fm
