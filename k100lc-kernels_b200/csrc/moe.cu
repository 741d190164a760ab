// Row gather and weighted combine around bucketed mixture-of-experts linear layers.
//
//   gather_rows_k(dst, src, idx, rows, dim)                 dst[r,:] = src[idx[r],:]
//   moe_combine_k(y, exp_out, w, n_exp, rows, dim)          y[r,:] = sum_e w[r,e] * exp_out[e,r,:]
//   moe_combine_gather_k(y, bucket, w, base, n_sel, rows, dim)   y[r,:] = sum_e w[r,e] * bucket[base[r,e],:]
//
// Reference: python/k100lc_kernels/model.py:582-720 (MoECombine, MoEExperts) and tools/selftest_all.py:450-489.
// The sums run over e in ascending order, product rounded first, as the reference's host loop does.
// One CTA per output row, 128-bit accesses.
#include "device_utils.cuh"
#include "fm_internal.h"

namespace fm {
namespace {

constexpr int kThreads = 128;

__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(float* __restrict__ dst, const float* __restrict__ src, const uint32_t* __restrict__ idx, int dim) {
    pdl_wait();
    const float4* s = reinterpret_cast<const float4*>(src + (size_t)idx[blockIdx.x] * dim);
    float4* d = reinterpret_cast<float4*>(dst + (size_t)blockIdx.x * dim);
    for (int i = threadIdx.x; i < dim / 4; i += kThreads) d[i] = s[i];
    pdl_launch_dependents();
}

// GATHER: the row of expert slot e is bucket[base[r,e]]; otherwise exp_out[e][r]
template <bool GATHER>
__global__ void __launch_bounds__(kThreads)
moe_combine_kernel(float* __restrict__ y, const float* __restrict__ src, const float* __restrict__ w,
                   const uint32_t* __restrict__ base, int n_sel, int rows, int dim) {
    pdl_wait();
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < dim / 4; i += kThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int e = 0; e < n_sel; e++) {
            const size_t row = GATHER ? (size_t)base[r * n_sel + e] : (size_t)e * rows + r;
            const float4 v = reinterpret_cast<const float4*>(src + row * dim)[i];
            const float we = w[r * n_sel + e];
            acc.x = __fadd_rn(acc.x, __fmul_rn(we, v.x));       // product rounded first, like the reference's host loop
            acc.y = __fadd_rn(acc.y, __fmul_rn(we, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(we, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(we, v.w));
        }
        reinterpret_cast<float4*>(y + (size_t)r * dim)[i] = acc;
    }
    pdl_launch_dependents();
}

int launch_gather_rows(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = "gather_rows_k";
    float* dst = arg_ptr<float>(a[0]);
    const float* src = arg_ptr<const float>(a[1]);
    const uint32_t* idx = arg_ptr<const uint32_t>(a[2]);
    const int rows = arg_i32(a[3]), dim = arg_i32(a[4]);
    FM_REQUIRE(rows >= 0 && dim > 0 && dim % 4 == 0, kn, "rows=%d dim=%d: dim must be a positive multiple of 4", rows, dim);
    const int run = (int)c.gx < rows ? (int)c.gx : rows;
    if (run == 0) return FM_OK;
    FM_REQUIRE(aligned(dst, 16) && aligned(src, 16) && aligned(idx, 4), kn, "misaligned pointer");
    FM_RANGE(dst, (size_t)run * dim * 4, kn, "dst");
    FM_RANGE(idx, (size_t)run * 4, kn, "idx");
    FM_RANGE(src, (size_t)dim * 4, kn, "src");          // the rows named by idx are the caller's responsibility beyond the first
    cudaError_t e = launch_kernel(gather_rows_kernel, dim3(run), dim3(kThreads), 0, c.stream, pdl_enabled(), dst, src, idx, dim);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

template <bool GATHER>
int launch_combine(const LaunchCtx& c, const uint64_t* a) {
    const char* kn = GATHER ? "moe_combine_gather_k" : "moe_combine_k";
    float* y = arg_ptr<float>(a[0]);
    const float* src = arg_ptr<const float>(a[1]);
    const float* w = arg_ptr<const float>(a[2]);
    const uint32_t* base = GATHER ? arg_ptr<const uint32_t>(a[3]) : nullptr;
    const int n_sel = arg_i32(a[GATHER ? 4 : 3]), rows = arg_i32(a[GATHER ? 5 : 4]), dim = arg_i32(a[GATHER ? 6 : 5]);
    FM_REQUIRE(rows >= 0 && n_sel > 0 && dim > 0 && dim % 4 == 0, kn, "rows=%d n=%d dim=%d: dim must be a positive multiple of 4", rows, n_sel, dim);
    const int run = (int)c.gx < rows ? (int)c.gx : rows;
    if (run == 0) return FM_OK;
    FM_REQUIRE(aligned(y, 16) && aligned(src, 16) && aligned(w, 4) && (!GATHER || aligned(base, 4)), kn, "misaligned pointer");
    FM_RANGE(y, (size_t)run * dim * 4, kn, "y");
    FM_RANGE(w, (size_t)run * n_sel * 4, kn, "weights");
    if (GATHER) FM_RANGE(base, (size_t)run * n_sel * 4, kn, "base");
    else FM_RANGE(src, (size_t)n_sel * rows * dim * 4, kn, "exp_out");
    cudaError_t e = launch_kernel(moe_combine_kernel<GATHER>, dim3(run), dim3(kThreads), 0, c.stream, pdl_enabled(), y, src, w, base,
                                  n_sel, rows, dim);
    return e == cudaSuccess ? after_launch(kn) : cuda_fail(kn, e);
}

const KernelEntry kMoe[] = {
    {"gather_rows_k", 5, launch_gather_rows, "pppii"},
    {"moe_combine_k", 6, launch_combine<false>, "pppiii"},
    {"moe_combine_gather_k", 7, launch_combine<true>, "ppppiii"},
};

}  // namespace

const KernelEntry* moe_kernels(int* n) {
    *n = (int)(sizeof(kMoe) / sizeof(kMoe[0]));
    return kMoe;
}

}  // namespace fm
