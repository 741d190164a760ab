// Activation quantisers: fused absmax + round kernels.
//
//   quant_act          int8, group 128   (reference kernels/gemv_w4a8_core.h:34-66)
//   quant_act4         int4, group 32    (reference kernels/gemv_w4a4_core.h:26-45)
//   nvfp4_quant_act    int8, block 16    (reference kernels/asm/k_nvfp4/001_*.s,
//                                         oracle tools/selftest_all.py:1049-1059)
//   quant_rows_fast_k / quant_rows_k     int4 rows for the prefill GEMM
//                                        (reference tools/gen_quant_fast.py:61-184)
//   quant_rows_a8_k    int8 rows for the W4A8 prefill GEMM (catalog entry of the
//                      reference, never verified there; arithmetic = quant_act)
//
// All of them compute s = amax/qmax with a correctly rounded fp32 division and
// q = clip(rint(x / s)) with a correctly rounded division and round-half-even, so
// the outputs are bit-identical to the NumPy oracle.  One thread owns four (or
// eight) consecutive elements, loaded as 128-bit words; the group maximum and sum
// travel over 2..5 warp shuffles.  These kernels touch a few KB per token and
// are launch-latency bound; the prefill row quantisers stream M*K*4 bytes and are
// HBM bound.
#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

// ---------------------------------------------------------------- quant_act
// One warp per (token, 128-group): lane l owns elements 4l..4l+3.
__global__ void __launch_bounds__(128)
quant_act_kernel(const float* __restrict__ x, int8_t* __restrict__ ae, int8_t* __restrict__ ao,
                 float* __restrict__ asc, int* __restrict__ asu, int K, int ngroups_run, int tokens) {
    pdl_wait();
    const int warp = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int ng = K >> 7;
    if (warp >= ngroups_run * tokens) return;
    const int m = warp / ngroups_run, g = warp - m * ngroups_run;
    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)g * 128 + lane * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = absmax_scale(amax, 127.f);
    const int q0 = quant_rne(v.x, s, -128, 127), q1 = quant_rne(v.y, s, -128, 127);
    const int q2 = quant_rne(v.z, s, -128, 127), q3 = quant_rne(v.w, s, -128, 127);
    const size_t half = (size_t)m * (K >> 1) + (size_t)g * 64 + lane * 2;
    *reinterpret_cast<char2*>(ae + half) = make_char2((signed char)q0, (signed char)q2);
    *reinterpret_cast<char2*>(ao + half) = make_char2((signed char)q1, (signed char)q3);
    const int sum = warp_sum(q0 + q1 + q2 + q3);
    if (lane == 0) {
        asc[(size_t)m * ng + g] = s;
        asu[(size_t)m * ng + g] = sum;
    }
    pdl_launch_dependents();
}

// --------------------------------------------------------------- quant_act4
// One thread owns 8 consecutive elements (one output u32); 4 threads per 32-group.
__global__ void __launch_bounds__(128)
quant_act4_kernel(const float* __restrict__ x, uint8_t* __restrict__ aq, float* __restrict__ asc,
                  int K, int ngroups_run, int tokens) {
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_tok = ngroups_run * 4;
    const bool live = t < per_tok * tokens;
    const int tc = live ? t : 0;
    const int m = tc / per_tok, w = tc - m * per_tok;          // w = word index inside the token
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)w * 8);
    const float4 a = src[0], b = src[1];
    float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                       fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!live) return;
    const float s = absmax_scale(amax, 7.f);
    const float e[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; j++) word |= (uint32_t)(quant_rne(e[j], s, -8, 7) & 0xF) << (4 * j);
    *reinterpret_cast<uint32_t*>(aq + (size_t)m * (K >> 1) + (size_t)w * 4) = word;
    if ((w & 3) == 0) asc[(size_t)m * (K >> 5) + (w >> 2)] = s;
    pdl_launch_dependents();
}

// ---------------------------------------------------------- nvfp4_quant_act
// One thread owns 4 consecutive elements; 4 threads per 16-block.
__global__ void __launch_bounds__(128)
nvfp4_quant_act_kernel(const float* __restrict__ x, int8_t* __restrict__ a, int8_t* __restrict__ b,
                       float* __restrict__ scale, int K, int nblocks_run, int tokens) {
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const int per_tok = nblocks_run * 4;
    const bool live = t < per_tok * tokens;
    const int tc = live ? t : 0;
    const int m = tc / per_tok, c = tc - m * per_tok;          // c = 4-element chunk index
    const float4 v = *reinterpret_cast<const float4*>(x + (size_t)m * K + (size_t)c * 4);
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (!live) return;
    const float s = absmax_scale(amax, 127.f);
    const int q0 = quant_rne(v.x, s, -128, 127), q1 = quant_rne(v.y, s, -128, 127);
    const int q2 = quant_rne(v.z, s, -128, 127), q3 = quant_rne(v.w, s, -128, 127);
    const size_t half = (size_t)m * (K >> 1) + (size_t)c * 2;
    *reinterpret_cast<char2*>(a + half) = make_char2((signed char)q0, (signed char)q2);
    *reinterpret_cast<char2*>(b + half) = make_char2((signed char)q1, (signed char)q3);
    if ((c & 3) == 0) scale[(size_t)m * (K >> 4) + (c >> 2)] = s;
    pdl_launch_dependents();
}

// ------------------------------------------------------------- quant_rows_*
// One warp per (row, 128-group): lane l owns elements 4l..4l+3.
//   A4: int4 codes, eight per u32 (low nibble = lower k), scales group-first sc[g*rows+row]
//   A8: int8 codes, one byte per element, [rows][K], where every aligned run of 8
//       elements is stored as (k0,k2,k4,k6,k1,k3,k5,k7) — the order in which the
//       W4A8 prefill GEMM expands a packed weight word — plus group-first scales.
template <bool A8>
__global__ void __launch_bounds__(256)
quant_rows_kernel(uint32_t* __restrict__ q, float* __restrict__ sc,
                  const float* __restrict__ x, int K, int rows, int in_stride, int in_off, int ng) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const long long total = (long long)rows * ng;
    for (long long w = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); w < total;
         w += (long long)gridDim.x * wpb) {
        const int row = (int)(w / ng), g = (int)(w - (long long)row * ng);
        const float4 v = *reinterpret_cast<const float4*>(
            x + (size_t)row * in_stride + in_off + (size_t)g * 128 + lane * 4);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float qmax = A8 ? 127.f : 7.f;
        const int lo = A8 ? -128 : -8, hi = A8 ? 127 : 7;
        const float s = absmax_scale(amax, qmax);
        const int q0 = quant_rne(v.x, s, lo, hi), q1 = quant_rne(v.y, s, lo, hi);
        const int q2 = quant_rne(v.z, s, lo, hi), q3 = quant_rne(v.w, s, lo, hi);
        if (lane == 0) sc[(size_t)g * rows + row] = s;
        const size_t word = (size_t)row * (K >> 3) + (size_t)g * 16 + (lane >> 1);
        if (!A8) {
            uint32_t h = (q0 & 0xF) | ((q1 & 0xF) << 4) | ((q2 & 0xF) << 8) | ((q3 & 0xF) << 12);
            const uint32_t other = __shfl_down_sync(0xffffffffu, h, 1);
            if ((lane & 1) == 0) q[word] = h | (other << 16);
        } else {
            uint32_t he = (q0 & 0xFF) | ((q2 & 0xFF) << 8), ho = (q1 & 0xFF) | ((q3 & 0xFF) << 8);
            const uint32_t oe = __shfl_down_sync(0xffffffffu, he, 1);
            const uint32_t oo = __shfl_down_sync(0xffffffffu, ho, 1);
            if ((lane & 1) == 0)
                *reinterpret_cast<uint2*>(q + 2 * word) = make_uint2(he | (oe << 16), ho | (oo << 16));
        }
    }
    pdl_launch_dependents();
}

// ---------------------------------------------------------------- launchers
int launch_quant_act(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "quant_act";
    const float* x = arg_ptr<const float>(a[0]);
    int8_t* ae = arg_ptr<int8_t>(a[1]);
    int8_t* ao = arg_ptr<int8_t>(a[2]);
    float* asc = arg_ptr<float>(a[3]);
    int* asu = arg_ptr<int>(a[4]);
    const int K = arg_i32(a[6]);                      // a[5] = M is unused by the reference kernel too
    FM_REQUIRE(K > 0 && K % 128 == 0, kn, "K=%d must be a positive multiple of 128", K);
    const int ng = K / 128;
    const int run = (int)(c.gx < (uint32_t)ng ? c.gx : (uint32_t)ng);   // groups = min(grid, K/128)
    const int tokens = (int)c.gy;
    if (run == 0 || tokens == 0) return FM_OK;
    FM_REQUIRE(aligned(x, 16) && aligned(ae, 2) && aligned(ao, 2) && aligned(asc, 4) && aligned(asu, 4), kn,
               "misaligned pointer (x needs 16 bytes, ae/ao 2, asc/asu 4)");
    FM_RANGE(x, (size_t)(tokens - 1) * K * 4 + (size_t)run * 512, kn, "x");
    FM_RANGE(ae, (size_t)(tokens - 1) * (K / 2) + (size_t)run * 64, kn, "ae");
    FM_RANGE(ao, (size_t)(tokens - 1) * (K / 2) + (size_t)run * 64, kn, "ao");
    FM_RANGE(asc, ((size_t)(tokens - 1) * ng + run) * 4, kn, "asc");
    FM_RANGE(asu, ((size_t)(tokens - 1) * ng + run) * 4, kn, "asu");
    const int warps = run * tokens;
    cudaError_t e = launch_kernel(quant_act_kernel, dim3((warps + 3) / 4), dim3(128), 0, c.stream, pdl_enabled(),
                                  x, ae, ao, asc, asu, K, run, tokens);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

int launch_quant_act4(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "quant_act4";
    const float* x = arg_ptr<const float>(a[0]);
    uint8_t* aq = arg_ptr<uint8_t>(a[1]);
    float* asc = arg_ptr<float>(a[2]);
    const int K = arg_i32(a[4]);
    FM_REQUIRE(K > 0 && K % 32 == 0, kn, "K=%d must be a positive multiple of 32", K);
    const int ng = K / 32;
    const int run = (int)(c.gx < (uint32_t)ng ? c.gx : (uint32_t)ng);
    const int tokens = (int)c.gy;
    if (run == 0 || tokens == 0) return FM_OK;
    FM_REQUIRE(aligned(x, 16) && aligned(aq, 4) && aligned(asc, 4), kn,
               "misaligned pointer (x needs 16 bytes, aq 4, asc 4)");
    FM_RANGE(x, (size_t)(tokens - 1) * K * 4 + (size_t)run * 128, kn, "x");
    FM_RANGE(aq, (size_t)(tokens - 1) * (K / 2) + (size_t)run * 16, kn, "aq");
    FM_RANGE(asc, ((size_t)(tokens - 1) * ng + run) * 4, kn, "asc");
    const int threads = run * 4 * tokens;
    cudaError_t e = launch_kernel(quant_act4_kernel, dim3((threads + 127) / 128), dim3(128), 0, c.stream,
                                  pdl_enabled(), x, aq, asc, K, run, tokens);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

int launch_nvfp4_quant_act(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "nvfp4_quant_act";
    const float* x = arg_ptr<const float>(a[0]);
    int8_t* qa = arg_ptr<int8_t>(a[1]);
    int8_t* qb = arg_ptr<int8_t>(a[2]);
    float* sc = arg_ptr<float>(a[3]);
    const int K = arg_i32(a[5]);
    FM_REQUIRE(K > 0 && K % 16 == 0, kn, "K=%d must be a positive multiple of 16", K);
    const int nb = K / 16;
    const int run = (int)(c.gx < (uint32_t)nb ? c.gx : (uint32_t)nb);
    const int tokens = (int)c.gy;
    if (run == 0 || tokens == 0) return FM_OK;
    FM_REQUIRE(aligned(x, 16) && aligned(qa, 2) && aligned(qb, 2) && aligned(sc, 4), kn,
               "misaligned pointer (x needs 16 bytes, a/b 2, scale 4)");
    FM_RANGE(x, (size_t)(tokens - 1) * K * 4 + (size_t)run * 64, kn, "x");
    FM_RANGE(qa, (size_t)(tokens - 1) * (K / 2) + (size_t)run * 8, kn, "a");
    FM_RANGE(qb, (size_t)(tokens - 1) * (K / 2) + (size_t)run * 8, kn, "b");
    FM_RANGE(sc, ((size_t)(tokens - 1) * nb + run) * 4, kn, "scale");
    const int threads = run * 4 * tokens;
    cudaError_t e = launch_kernel(nvfp4_quant_act_kernel, dim3((threads + 127) / 128), dim3(128), 0, c.stream,
                                  pdl_enabled(), x, qa, qb, sc, K, run, tokens);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// (q, sc, x, K, G, rows, in_stride, in_off[, NG]); grid = rows.
template <bool FAST>
int launch_quant_rows(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = FAST ? "quant_rows_fast_k" : "quant_rows_k";
    uint32_t* q = arg_ptr<uint32_t>(a[0]);
    float* sc = arg_ptr<float>(a[1]);
    const float* x = arg_ptr<const float>(a[2]);
    const int K = arg_i32(a[3]), G = arg_i32(a[4]), rows = arg_i32(a[5]);
    const int in_stride = arg_i32(a[6]), in_off = arg_i32(a[7]);
    FM_REQUIRE(G == 128, kn, "G=%d: only the group size 128 of the W4 GEMM is built", G);
    FM_REQUIRE(K > 0 && K % 128 == 0 && rows >= 0, kn, "K=%d must be a positive multiple of 128", K);
    const int ng = K / G;
    if (FAST) FM_REQUIRE(arg_i32(a[8]) == ng, kn, "NG=%d does not equal K/G=%d", arg_i32(a[8]), ng);
    else FM_REQUIRE((int)c.wx == ng, kn, "work-group size %u must equal K/G=%d", c.wx, ng);
    FM_REQUIRE(in_stride >= 0 && in_off >= 0 && in_stride % 4 == 0 && in_off % 4 == 0, kn,
               "in_stride/in_off must be non-negative multiples of 4 elements");
    FM_REQUIRE((int)c.gx >= rows, kn, "grid=%u covers only part of rows=%d; launch with grid = rows", c.gx, rows);
    if (rows == 0) return FM_OK;
    FM_REQUIRE(aligned(x, 16) && aligned(q, 4) && aligned(sc, 4), kn, "misaligned pointer");
    FM_RANGE(x, ((size_t)(rows - 1) * in_stride + in_off + K) * 4, kn, "x");
    FM_RANGE(q, (size_t)rows * (K / 8) * 4, kn, "q");
    FM_RANGE(sc, (size_t)ng * rows * 4, kn, "sc");
    long long blocks = ((long long)rows * ng + 7) / 8;
    const long long cap = (long long)c.sm_count * 16;
    if (blocks > cap) blocks = cap;
    cudaError_t e = launch_kernel(quant_rows_kernel<false>, dim3((unsigned)blocks), dim3(256), 0, c.stream,
                                  pdl_enabled(), q, sc, x, K, rows, in_stride, in_off, ng);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// quant_rows_a8_k (q, reserved, sc, reserved, x, K, G, rows, in_stride, in_off); grid = rows.
// The reference catalogues a kernel of this name and argument shape but never verified or
// used it; the output layout is the one described above quant_rows_kernel.
int launch_quant_rows_a8(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "quant_rows_a8_k";
    uint32_t* q = arg_ptr<uint32_t>(a[0]);
    float* sc = arg_ptr<float>(a[2]);
    const float* x = arg_ptr<const float>(a[4]);
    const int K = arg_i32(a[5]), G = arg_i32(a[6]), rows = arg_i32(a[7]);
    const int in_stride = arg_i32(a[8]), in_off = arg_i32(a[9]);
    FM_REQUIRE(G == 128, kn, "G=%d: only the group size 128 of the W4 GEMM is built", G);
    FM_REQUIRE(K > 0 && K % 128 == 0 && rows >= 0, kn, "K=%d must be a positive multiple of 128", K);
    FM_REQUIRE(in_stride >= 0 && in_off >= 0 && in_stride % 4 == 0 && in_off % 4 == 0, kn,
               "in_stride/in_off must be non-negative multiples of 4 elements");
    FM_REQUIRE((int)c.gx >= rows, kn, "grid=%u covers only part of rows=%d; launch with grid = rows", c.gx, rows);
    if (rows == 0) return FM_OK;
    const int ng = K / G;
    FM_REQUIRE(aligned(x, 16) && aligned(q, 8) && aligned(sc, 4), kn, "misaligned pointer");
    FM_RANGE(x, ((size_t)(rows - 1) * in_stride + in_off + K) * 4, kn, "x");
    FM_RANGE(q, (size_t)rows * K, kn, "q");
    FM_RANGE(sc, (size_t)ng * rows * 4, kn, "sc");
    long long blocks = ((long long)rows * ng + 7) / 8;
    const long long cap = (long long)c.sm_count * 16;
    if (blocks > cap) blocks = cap;
    cudaError_t e = launch_kernel(quant_rows_kernel<true>, dim3((unsigned)blocks), dim3(256), 0, c.stream,
                                  pdl_enabled(), q, sc, x, K, rows, in_stride, in_off, ng);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kQuant[] = {
    {"quant_act", 7, launch_quant_act, "pppppii"},
    {"quant_act4", 5, launch_quant_act4, "pppii"},
    {"nvfp4_quant_act", 6, launch_nvfp4_quant_act, "ppppii"},
    {"quant_rows_fast_k", 9, launch_quant_rows<true>, "pppiiiiii"},
    {"quant_rows_k", 8, launch_quant_rows<false>, "pppiiiii"},
    {"quant_rows_a8_k", 10, launch_quant_rows_a8, "pppppiiiii"},
};

}  // namespace

cudaError_t quant_act_raw(const float* x, int8_t* ae, int8_t* ao, float* asc, int* asu, int K, int tokens,
                          cudaStream_t stream) {
    const int groups = K / 128;
    const int warps = groups * tokens;
    quant_act_kernel<<<(warps + 3) / 4, 128, 0, stream>>>(x, ae, ao, asc, asu, K, groups, tokens);
    return cudaGetLastError();
}

const KernelEntry* quant_kernels(int* n) {
    *n = (int)(sizeof(kQuant) / sizeof(kQuant[0]));
    return kQuant;
}

}  // namespace fm
