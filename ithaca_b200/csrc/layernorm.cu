// Layer norm with weight and bias, and the sum of two residual streams.
//
// y = (x - mean) / sqrt(var + eps) * w + b, var = mean((x - mean)^2): the mean first, then the mean of
// the squared deviations (no E[x^2] - E[x]^2), all in float.  One block per row; a row of up to 4096
// elements stays in the thread's registers between the passes.
//
// Two ways to deliver y:
//   * out[r, :] = y in the storage type asked for (the norm in front of a sublayer), or
//   * into[r, :] += mult * y in float (the norm behind a sublayer: the scaled result joins the residual
//     stream in the same kernel, so the sublayer's normed output is never written).
#include "common.cuh"

namespace {

constexpr int LN_THREADS = 256, LN_REG = 16;      // 256 * 16 = 4096 elements in registers

template <typename TO, bool IN_REGS>
__global__ void __launch_bounds__(LN_THREADS)
layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows_in, const float* __restrict__ w,
                 const float* __restrict__ b, TO* __restrict__ out, float* __restrict__ into, float mult, int d, float eps) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(rows_in);
    IK_AFTER_WAIT(into);
    ik_pdl_launch_dependents();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* a = x + (size_t)(rows_in ? rows_in[r] : r) * d;
    float xv[LN_REG];
    float s = 0.f;
    if (IN_REGS) {
        #pragma unroll
        for (int j = 0; j < LN_REG; j++) {
            const int i = threadIdx.x + j * LN_THREADS;
            xv[j] = i < d ? a[i] : 0.f;
            s += xv[j];
        }
    } else {
        for (int i = threadIdx.x; i < d; i += LN_THREADS) s += a[i];
    }
    const float mean = ik_block_sum<LN_THREADS>(s, red) / (float)d;
    float q = 0.f;
    if (IN_REGS) {
        #pragma unroll
        for (int j = 0; j < LN_REG; j++) {
            const int i = threadIdx.x + j * LN_THREADS;
            const float dv = i < d ? xv[j] - mean : 0.f;
            q = fmaf(dv, dv, q);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += LN_THREADS) { const float dv = a[i] - mean; q = fmaf(dv, dv, q); }
    }
    const float var = ik_block_sum<LN_THREADS>(q, red) / (float)d;
    const float inv = 1.0f / sqrtf(var + eps);
    auto deliver = [&](int i, float v) {
        const float y = (v - mean) * inv * w[i] + b[i];
        const size_t o = (size_t)r * d + i;
        if (into) into[o] = fmaf(mult, y, into[o]);
        else ik_st(out, o, y);
    };
    if (IN_REGS) {
        #pragma unroll
        for (int j = 0; j < LN_REG; j++) {
            const int i = threadIdx.x + j * LN_THREADS;
            if (i < d) deliver(i, xv[j]);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += LN_THREADS) deliver(i, a[i]);
    }
}

// y[i] += x[i] over n floats
__global__ void add_kernel(float* __restrict__ y, const float* __restrict__ x, size_t n) {
    ik_pdl_wait();
    IK_AFTER_WAIT(x);
    IK_AFTER_WAIT(y);
    ik_pdl_launch_dependents();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) y[i] += x[i];
}

}  // namespace

// out (storage type out_dtype) or into (float, += mult * y): exactly one of them is given.
IK_EXPORT int ik_layernorm(const float* x, const int* rows_in, const float* w, const float* b, void* out, int out_dtype,
                           float* into, float mult, int rows, int d, float eps, cudaStream_t stream) {
    if (rows < 0 || d <= 0 || (out == nullptr) == (into == nullptr)) return IK_BAD_ARGUMENT;
    if (rows == 0) return IK_OK;
    const bool regs = d <= LN_THREADS * LN_REG;
#define IK_LN(TO, R) IK_RETURN_IF_ERROR(ik_launch(layernorm_kernel<TO, R>, rows, LN_THREADS, 0, stream, x, rows_in, w, b, (TO*)out, into, mult, d, eps))
    if (into || out_dtype == IK_F32) { if (regs) IK_LN(float, true); else IK_LN(float, false); }
    else if (out_dtype == IK_BF16) { if (regs) IK_LN(__nv_bfloat16, true); else IK_LN(__nv_bfloat16, false); }
    else return IK_BAD_ARGUMENT;
#undef IK_LN
    IK_LAUNCH_STATUS();
}

IK_EXPORT int ik_add(float* y, const float* x, unsigned long long n, cudaStream_t stream) {
    if (n == 0) return IK_OK;
    const size_t want = (n + 255) / 256, cap = (size_t)ik_sm_count() * 16;
    IK_RETURN_IF_ERROR(ik_launch(add_kernel, (int)(want < cap ? want : cap), 256, 0, stream, y, x, (size_t)n));
    IK_LAUNCH_STATUS();
}
