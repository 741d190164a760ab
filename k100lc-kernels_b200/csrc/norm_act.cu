// The operators either side of a streamed linear layer, fused with its activation quantiser.
//
//   rmsnorm_k(y, x, w, dim, eps, flag) / rmsnorm_fast_k / rmsnorm_deep_k(y, x, w, dim, eps)
//                         y = x * rsqrt(mean(x^2) + eps) * w        (reference python/k100lc_kernels/model.py:480-524,
//                                                                    tools/selftest_all.py:266-300)
//   silu_mul_k(y, gate, up, n)   y = gate / (1 + exp(-gate)) * up   (reference model.py:527-544, selftest_all.py:214-223)
//   rmsnorm_quant_k(ae, ao, sc, asum, x, w, dim, eps)               (reference tools/gen_rmsnorm_quant.py:16-33)
//                         the norm and quant_act in one kernel: the normalised row never goes to memory,
//                         the outputs are quant_act's (even / odd int8 streams, group scales, group sums)
//   silu_mul_quant_k(ae, ao, sc, asum, gate, up, K)   extension: silu(gate) * up and quant_act in one kernel —
//                         the input of a W4A8 down projection (the reference fuses the gate into its f32 GEMV,
//                         model.py:1262-1266; with int8 activations the fusion point is the quantiser)
//
// One CTA per row.  The mean of squares is accumulated in double precision (the squares of fp32 values are
// exact there and the order of the additions stops mattering at fp32 resolution), rs = float(1 / sqrt(ms + eps)),
// y = (x * rs) * w with both products rounded to fp32 — the arithmetic of the reference's own checker
// (gen_rmsnorm_quant.py:288-296), so the quantised outputs can be compared bit for bit.
#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int kThreads = 256;

// sum over the CTA of a per-thread double; every thread gets the total
__device__ __forceinline__ double block_sum(double v, double* slots) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) slots[warp] = v;
    __syncthreads();
    double t = 0.0;
#pragma unroll
    for (int i = 0; i < kThreads / 32; i++) t += slots[i];       // fixed order: the same bits in every thread
    return t;
}

__device__ __forceinline__ float row_rs(const float* __restrict__ x, int dim, float eps, double* slots) {
    double ss = 0.0;
    for (int i = threadIdx.x * 4; i < dim; i += kThreads * 4) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
    }
    const double ms = block_sum(ss, slots) / (double)dim;
    return (float)(1.0 / sqrt(ms + (double)eps));
}

__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ w, int dim, float eps) {
    __shared__ double slots[kThreads / 32];
    pdl_wait();
    const float* xr = x + (size_t)blockIdx.x * dim;
    float* yr = y + (size_t)blockIdx.x * dim;
    const float rs = row_rs(xr, dim, eps, slots);
    for (int i = threadIdx.x * 4; i < dim; i += kThreads * 4) {
        const float4 v = *reinterpret_cast<const float4*>(xr + i), g = *reinterpret_cast<const float4*>(w + i);
        *reinterpret_cast<float4*>(yr + i) = make_float4((v.x * rs) * g.x, (v.y * rs) * g.y, (v.z * rs) * g.z, (v.w * rs) * g.w);
    }
    pdl_launch_dependents();
}

__device__ __forceinline__ float silu(float g) { return __fdiv_rn(g, 1.0f + expf(-g)); }

__global__ void __launch_bounds__(kThreads)
silu_mul_kernel(float* __restrict__ y, const float* __restrict__ gate, const float* __restrict__ up, int n) {
    pdl_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) y[i] = silu(gate[i]) * up[i];
    pdl_launch_dependents();
}

// quant_act's arithmetic on the four values of a lane (one warp = one 128-group): reference
// kernels/gemv_w4a8_core.h:34-66
__device__ __forceinline__ void quant_group(const float (&v)[4], int8_t* ae, int8_t* ao, float* sc, int* asum, size_t half, size_t gi) {
    const int lane = threadIdx.x & 31;
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float s = absmax_scale(amax, 127.f);
    const int q0 = quant_rne(v[0], s, -128, 127), q1 = quant_rne(v[1], s, -128, 127);
    const int q2 = quant_rne(v[2], s, -128, 127), q3 = quant_rne(v[3], s, -128, 127);
    *reinterpret_cast<char2*>(ae + half + lane * 2) = make_char2((signed char)q0, (signed char)q2);
    *reinterpret_cast<char2*>(ao + half + lane * 2) = make_char2((signed char)q1, (signed char)q3);
    const int sum = warp_sum(q0 + q1 + q2 + q3);
    if (lane == 0) {
        sc[gi] = s;
        asum[gi] = sum;
    }
}

__global__ void __launch_bounds__(kThreads)
rmsnorm_quant_kernel(int8_t* __restrict__ ae, int8_t* __restrict__ ao, float* __restrict__ sc, int* __restrict__ asum,
                     const float* __restrict__ x, const float* __restrict__ w, int dim, float eps) {
    __shared__ double slots[kThreads / 32];
    pdl_wait();
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, ng = dim >> 7;
    const float* xr = x + (size_t)row * dim;
    const float rs = row_rs(xr, dim, eps, slots);
    for (int g = warp; g < ng; g += kThreads / 32) {                 // one warp per 128-group
        const float4 v = *reinterpret_cast<const float4*>(xr + g * 128 + lane * 4);
        const float4 k = *reinterpret_cast<const float4*>(w + g * 128 + lane * 4);
        const float y[4] = {(v.x * rs) * k.x, (v.y * rs) * k.y, (v.z * rs) * k.z, (v.w * rs) * k.w};
        quant_group(y, ae, ao, sc, asum, (size_t)row * (dim >> 1) + (size_t)g * 64, (size_t)row * ng + g);
    }
    pdl_launch_dependents();
}

__global__ void __launch_bounds__(kThreads)
silu_mul_quant_kernel(int8_t* __restrict__ ae, int8_t* __restrict__ ao, float* __restrict__ sc, int* __restrict__ asum,
                      const float* __restrict__ gate, const float* __restrict__ up, int K) {
    pdl_wait();
    const int row = blockIdx.y, lane = threadIdx.x & 31, ng = K >> 7;
    const int g = blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    if (g < ng) {
        const float4 a = *reinterpret_cast<const float4*>(gate + (size_t)row * K + g * 128 + lane * 4);
        const float4 b = *reinterpret_cast<const float4*>(up + (size_t)row * K + g * 128 + lane * 4);
        const float y[4] = {silu(a.x) * b.x, silu(a.y) * b.y, silu(a.z) * b.z, silu(a.w) * b.w};
        quant_group(y, ae, ao, sc, asum, (size_t)row * (K >> 1) + (size_t)g * 64, (size_t)row * ng + g);
    }
    pdl_launch_dependents();
}

// ------------------------------------------------------------------------- host side
// rows come from the grid, as on the reference (grid = rows, work-group = 64)
template <bool HAS_FLAG>
int launch_rmsnorm(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = HAS_FLAG ? "rmsnorm_k" : "rmsnorm_fast_k";
    float* y = arg_ptr<float>(a[0]);
    const float* x = arg_ptr<const float>(a[1]);
    const float* w = arg_ptr<const float>(a[2]);
    const int dim = arg_i32(a[3]);
    const float eps = arg_f32(a[4]);
    FM_REQUIRE(!HAS_FLAG || arg_i32(a[5]) == 0, kn, "flag=%d: only the standard RMSNorm (flag 0) is built", arg_i32(a[5]));
    FM_REQUIRE(c.gy == 1 && dim > 0 && dim % 4 == 0, kn, "dim=%d must be a positive multiple of 4 on a 1-D grid", dim);
    const int rows = (int)c.gx;
    if (rows == 0) return FM_OK;
    FM_REQUIRE(aligned(y, 16) && aligned(x, 16) && aligned(w, 16), kn, "x, w and y must be 16-byte aligned");
    FM_RANGE(x, (size_t)rows * dim * 4, kn, "x");
    FM_RANGE(y, (size_t)rows * dim * 4, kn, "y");
    FM_RANGE(w, (size_t)dim * 4, kn, "w");
    cudaError_t e = launch_kernel(rmsnorm_kernel, dim3(rows), dim3(kThreads), 0, c.stream, pdl_enabled(), y, x, w, dim, eps);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

int launch_silu_mul(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "silu_mul_k";
    float* y = arg_ptr<float>(a[0]);
    const float* gate = arg_ptr<const float>(a[1]);
    const float* up = arg_ptr<const float>(a[2]);
    const int n = arg_i32(a[3]);
    FM_REQUIRE(n >= 0 && aligned(y, 4) && aligned(gate, 4) && aligned(up, 4), kn, "bad n or misaligned pointer");
    const long long covered = (long long)c.gx * c.wx;              // elements the caller's grid covers
    const int run = (int)(covered < n ? covered : n);
    if (run == 0) return FM_OK;
    FM_RANGE(y, (size_t)run * 4, kn, "y");
    FM_RANGE(gate, (size_t)run * 4, kn, "gate");
    FM_RANGE(up, (size_t)run * 4, kn, "up");
    int blocks = (run + kThreads - 1) / kThreads;
    if (blocks > c.sm_count * 8) blocks = c.sm_count * 8;
    cudaError_t e = launch_kernel(silu_mul_kernel, dim3(blocks), dim3(kThreads), 0, c.stream, pdl_enabled(), y, gate, up, run);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

struct QuantOut {
    int8_t *ae, *ao;
    float* sc;
    int* asum;
};
int check_quant_out(const char* kn, const uint64_t* a, QuantOut& q, int rows, int K) {
    q.ae = arg_ptr<int8_t>(a[0]);
    q.ao = arg_ptr<int8_t>(a[1]);
    q.sc = arg_ptr<float>(a[2]);
    q.asum = arg_ptr<int>(a[3]);
    FM_REQUIRE(K > 0 && K % 128 == 0, kn, "K=%d must be a positive multiple of 128", K);
    FM_REQUIRE(aligned(q.ae, 2) && aligned(q.ao, 2) && aligned(q.sc, 4) && aligned(q.asum, 4), kn, "misaligned output");
    FM_RANGE(q.ae, (size_t)rows * (K / 2), kn, "ae");
    FM_RANGE(q.ao, (size_t)rows * (K / 2), kn, "ao");
    FM_RANGE(q.sc, (size_t)rows * (K / 128) * 4, kn, "sc");
    FM_RANGE(q.asum, (size_t)rows * (K / 128) * 4, kn, "asum");
    return FM_OK;
}

// rmsnorm_quant_k(ae, ao, sc, asum, x, w, dim, eps): grid = rows
int launch_rmsnorm_quant(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "rmsnorm_quant_k";
    const float* x = arg_ptr<const float>(a[4]);
    const float* w = arg_ptr<const float>(a[5]);
    const int dim = arg_i32(a[6]);
    const float eps = arg_f32(a[7]);
    const int rows = (int)c.gx;
    FM_REQUIRE(c.gy == 1, kn, "1-D grid of rows expected");
    if (rows == 0) return FM_OK;
    QuantOut q;
    const int rc = check_quant_out(kn, a, q, rows, dim);
    if (rc) return rc;
    FM_REQUIRE(aligned(x, 16) && aligned(w, 16), kn, "x and w must be 16-byte aligned");
    FM_RANGE(x, (size_t)rows * dim * 4, kn, "x");
    FM_RANGE(w, (size_t)dim * 4, kn, "w");
    cudaError_t e = launch_kernel(rmsnorm_quant_kernel, dim3(rows), dim3(kThreads), 0, c.stream, pdl_enabled(), q.ae, q.ao, q.sc,
                                  q.asum, x, w, dim, eps);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

// silu_mul_quant_k(ae, ao, sc, asum, gate, up, K): grid y = rows (grid x is ignored)
int launch_silu_mul_quant(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "silu_mul_quant_k";
    const float* gate = arg_ptr<const float>(a[4]);
    const float* up = arg_ptr<const float>(a[5]);
    const int K = arg_i32(a[6]);
    const int rows = (int)c.gy;
    if (rows == 0) return FM_OK;
    QuantOut q;
    const int rc = check_quant_out(kn, a, q, rows, K);
    if (rc) return rc;
    FM_REQUIRE(aligned(gate, 16) && aligned(up, 16), kn, "gate and up must be 16-byte aligned");
    FM_RANGE(gate, (size_t)rows * K * 4, kn, "gate");
    FM_RANGE(up, (size_t)rows * K * 4, kn, "up");
    const int ng = K / 128;
    cudaError_t e = launch_kernel(silu_mul_quant_kernel, dim3((ng + kThreads / 32 - 1) / (kThreads / 32), rows), dim3(kThreads), 0,
                                  c.stream, pdl_enabled(), q.ae, q.ao, q.sc, q.asum, gate, up, K);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kNormAct[] = {
    {"rmsnorm_k", 6, launch_rmsnorm<true>, "pppifi"},
    {"rmsnorm_fast_k", 5, launch_rmsnorm<false>, "pppif"},
    {"rmsnorm_deep_k", 5, launch_rmsnorm<false>, "pppif"},
    {"silu_mul_k", 4, launch_silu_mul, "pppi"},
    {"rmsnorm_quant_k", 8, launch_rmsnorm_quant, "ppppppif"},
    {"silu_mul_quant_k", 7, launch_silu_mul_quant, "ppppppi"},
};

}  // namespace

const KernelEntry* norm_act_kernels(int* n) {
    *n = (int)(sizeof(kNormAct) / sizeof(kNormAct[0]));
    return kNormAct;
}

}  // namespace fm
