// Small device-side building blocks shared by the kernel files (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fm {

// 128-bit streaming load of read-once data: read-only path, no L1 allocation.
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const void* p) {
    unsigned short v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// signed 8-bit x 4 dot product with int32 accumulate
__device__ __forceinline__ int dot4(uint32_t a, uint32_t b, int c) {
    return __dp4a(static_cast<int>(a), static_cast<int>(b), c);
}

// unsigned 8-bit (a) x signed 8-bit (b) x 4 dot product with int32 accumulate
__device__ __forceinline__ int dot4_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// sum over the 32 int4 weights of one 16-byte word of (nibble ^ 8) * q, where e / o hold
// the int8 activations of the even / odd k positions.  Low nibbles become bytes u (one
// LOP3: mask and flip the sign bit); high nibbles stay in place as unsigned bytes 16*u
// (one LOP3) and go through the unsigned-by-signed dp4a, so no shift is needed per word;
// their sum is a multiple of 16 and is scaled back exactly at the end.
__device__ __forceinline__ int dot32_u(const uint4& w, const uint4& e, const uint4& o) {
    int lo = 0, hi = 0;
    lo = dot4((w.x & 0x0F0F0F0Fu) ^ 0x08080808u, e.x, lo);
    hi = dot4_us((w.x & 0xF0F0F0F0u) ^ 0x80808080u, o.x, hi);
    lo = dot4((w.y & 0x0F0F0F0Fu) ^ 0x08080808u, e.y, lo);
    hi = dot4_us((w.y & 0xF0F0F0F0u) ^ 0x80808080u, o.y, hi);
    lo = dot4((w.z & 0x0F0F0F0Fu) ^ 0x08080808u, e.z, lo);
    hi = dot4_us((w.z & 0xF0F0F0F0u) ^ 0x80808080u, o.z, hi);
    lo = dot4((w.w & 0x0F0F0F0Fu) ^ 0x08080808u, e.w, lo);
    hi = dot4_us((w.w & 0xF0F0F0F0u) ^ 0x80808080u, o.w, hi);
    return lo + (hi >> 4);
}

// generic byte permute; selector nibble bit 3 replicates the sign bit of the
// selected byte (used as a "zero unless" switch with tables whose bytes are < 0x80)
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// ---- NVFP4: E2M1 weights (2 * magnitude in an 8-byte table, the packed word is the PRMT selector)
// and E4M3 block scales
constexpr uint32_t kTabLo = 0x03020100u;     // 2*E2M1 magnitude of index 0..3
constexpr uint32_t kTabHi = 0x0C080604u;     // index 4..7
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    const float mag = e == 0 ? ldexpf((float)m, -9) : ldexpf((float)(8u + m), (int)e - 10);
    return (b & 0x80u) ? -mag : mag;
}

// integer dot of 8 E2M1 codes (one packed word) with 8 int8 activations in natural order
__device__ __forceinline__ int dot8_e2m1(uint32_t w, uint32_t a_lo, uint32_t a_hi, int acc) {
    const uint32_t n = w ^ 0x88888888u;
    acc = dot4(prmt(kTabLo, kTabHi, w), a_lo, acc);
    acc = dot4(prmt(kTabLo, kTabHi, w >> 16), a_hi, acc);
    int neg = dot4(prmt(kTabLo, kTabHi, n), a_lo, 0);
    neg = dot4(prmt(kTabLo, kTabHi, n >> 16), a_hi, neg);
    return acc - neg;
}

// ---- W4A16 on the tensor cores: offset-binary int4 codes as bf16 pairs, fp32 activations as three bf16 terms
__device__ __forceinline__ uint32_t bf16x2_sub136(uint32_t v) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(v), "r"(0x43084308u));     // 136.0 twice
    return d;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// term `which` (0, 1, 2) of the three-way bf16 split of x, as the upper 16 bits of a float
__device__ __forceinline__ uint32_t bf16_term(float x, int which) {
    float r = x;
    uint32_t t = 0;
    for (int i = 0; i <= which; i++) {
        t = __float_as_uint(__bfloat162float(__float2bfloat16_rn(r))) >> 16;
        r -= __uint_as_float(t << 16);
    }
    return t;
}

// A CTA has one warp per block index of a group of eight adjacent blocks (512 contiguous bytes of
// every row) and walks 16-row units; the loads of the next two units are in flight while the
// current two are multiplied (HBM latency under load is several microseconds — a warp that
// loads, waits and then computes leaves the memory system idle half of the time).

// Programmatic dependent launch: wait until the preceding kernel on the stream
// has completed and its writes are visible / allow the next kernel to start.
// Both are no-ops when the kernel was launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Four int4 nibbles that sit in the low nibble of each byte -> four signed bytes.
// (x & 0x08)*30 = 0xF0 exactly when the nibble is negative; no carry crosses a byte.
__device__ __forceinline__ uint32_t sext_nibbles(uint32_t x) { return x | ((x & 0x08080808u) * 30u); }

// absmax scale and round-half-even quantisation, bit-identical to
// s = amax > 0 ? amax / qmax : 1 ; q = clip(rint(x / s)) evaluated in IEEE fp32
__device__ __forceinline__ float absmax_scale(float amax, float qmax) {
    return amax > 0.f ? __fdiv_rn(amax, qmax) : 1.f;
}
__device__ __forceinline__ int quant_rne(float x, float s, int lo, int hi) {
    int q = __float2int_rn(__fdiv_rn(x, s));
    return min(max(q, lo), hi);
}

}  // namespace fm
