// Small kernels of a layer whose branches all read ONE norm's output and are added to the stream together
// (x += s0 * a + s1 * f with a gain per feature on each branch), with a layer norm (mean taken off) as that norm,
// and the elementwise half of a gated feed-forward with a choice of activation.  All arithmetic is fp32; `dtype`
// is the type of the activations (0 = float32, 1 = bfloat16).  The residual stream is float32.
#include "common.cuh"

// A branch output at element i of row r: an activation-dtype tensor, or fp32 partial sums added in index order.
template <typename T>
__device__ __forceinline__ float branch_at(const T* y, const float* parts, int n_parts, long long part_stride, size_t at) {
    if (parts) {
        float acc = parts[at];
        for (int s = 1; s < n_parts; ++s) acc += parts[(size_t)s * part_stride + at];
        return acc;
    }
    return to_f32<T>(y[at]);
}

// ---------------------------------------------------------------------------
// v      = x[src] + (s0 * b0[src] + s1 * b1[src])      src = rows[r] or r; a branch may be absent
// x[src] = v                                            (update_x, without rows)
// out[r] = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w (+ bias)      activation dtype, or fp32 when out_f32
// One block per row; the row waits in shared memory between the passes.  The block size depends on H only, so a
// row's sums are added in the same order whatever the batch holds.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_layernorm_kernel(float* x, const T* y0, const float* p0, int n0, const float* s0, const T* y1,
                                     const float* p1, int n1, const float* s1, long long part_stride, const float* w,
                                     const float* bias, void* out, int out_f32, const int* rows, int H, float eps, int update_x) {
    extern __shared__ float row_smem[];   // [H]
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* xr = x + (size_t)src * H;
    const bool b0 = y0 != nullptr || p0 != nullptr, b1 = y1 != nullptr || p1 != nullptr;
    float sum = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = xr[i];
        if (b0 || b1) {
            const size_t at = (size_t)src * H + i;
            float add = 0.f;
            if (b0) add = __fmul_rn(s0[i], branch_at<T>(y0, p0, n0, part_stride, at));
            if (b1) add = __fadd_rn(add, __fmul_rn(s1[i], branch_at<T>(y1, p1, n1, part_stride, at)));
            v = __fadd_rn(v, add);
            if (update_x) xr[i] = v;
        }
        row_smem[i] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row_smem[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float o = __fmul_rn(__fmul_rn(row_smem[i] - mean, rstd), w[i]);
        if (bias) o = __fadd_rn(o, bias[i]);
        if (out_f32) ((float*)out)[(size_t)r * H + i] = o;
        else ((T*)out)[(size_t)r * H + i] = from_f32<T>(o);
    }
}

PYRE_API int pyre_add_layernorm(float* x, const void* y0, const float* p0, int n0, const float* s0, const void* y1,
                                const float* p1, int n1, const float* s1, long long part_stride, const float* weight,
                                const float* bias, void* out, int out_f32, const int* rows, int n_rows, int H, float eps, int update_x,
                                int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (size_t)H * sizeof(float) > 48 * 1024) return PYRE_ERR_UNSUPPORTED;
    if ((y0 && p0) || (y1 && p1) || ((y0 || p0) && !s0) || ((y1 || p1) && !s1)) return PYRE_ERR_BAD_ARG;
    if ((p0 && n0 < 1) || (p1 && n1 < 1)) return PYRE_ERR_BAD_ARG;
    const int threads = min(512, max(32, ((H / 4 + 31) / 32) * 32));
    const size_t smem = (size_t)H * sizeof(float);
    if (dtype == PYRE_BF16)
        pyre_launch(add_layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x, (const __nv_bfloat16*)y0, p0,
                    n0, s0, (const __nv_bfloat16*)y1, p1, n1, s1, part_stride, weight, bias, out, out_f32, rows, H, eps, update_x);
    else if (dtype == PYRE_F32)
        pyre_launch(add_layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, (const float*)y0, p0, n0, s0,
                    (const float*)y1, p1, n1, s1, part_stride, weight, bias, out, out_f32, rows, H, eps, update_x);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[r, i] = s0[i] * b0[r, i] + s1[i] * b1[r, i] in the activation dtype: the branches of such a layer as one
// plain tensor, for a consumer that knows nothing of them.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void scaled_sum_kernel(const T* y0, const float* p0, int n0, const float* s0, const T* y1, const float* p1,
                                  int n1, const float* s1, long long part_stride, T* out, size_t n, int H) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const bool b1 = y1 != nullptr || p1 != nullptr;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < n; at += stride) {
        const int i = (int)(at % H);
        float add = __fmul_rn(s0[i], branch_at<T>(y0, p0, n0, part_stride, at));
        if (b1) add = __fadd_rn(add, __fmul_rn(s1[i], branch_at<T>(y1, p1, n1, part_stride, at)));
        out[at] = from_f32<T>(add);
    }
}

PYRE_API int pyre_scaled_sum(const void* y0, const float* p0, int n0, const float* s0, const void* y1, const float* p1,
                             int n1, const float* s1, long long part_stride, void* out, int n_rows, int H, int dtype,
                             cudaStream_t stream) {
    if (n_rows <= 0 || H <= 0) return 0;
    if ((y0 == nullptr) == (p0 == nullptr) || !s0 || (y1 && p1) || ((y1 || p1) && !s1)) return PYRE_ERR_BAD_ARG;
    const size_t n = (size_t)n_rows * H;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll((long long)n, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(scaled_sum_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)y0, p0, n0, s0,
                    (const __nv_bfloat16*)y1, p1, n1, s1, part_stride, (__nv_bfloat16*)out, n, H);
    else if (dtype == PYRE_F32)
        pyre_launch(scaled_sum_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)y0, p0, n0, s0, (const float*)y1,
                    p1, n1, s1, part_stride, (float*)out, n, H);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[r, i] = act(gu[r, i]) * gu[r, I + i]: the elementwise half of a gated feed-forward whose product left
// [gates | ups] per row.  kind 0: silu, z / (1 + exp(-z)); kind 1: the tanh form of gelu,
// 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float gate_act(float z, int kind) {
    if (kind == 0) return z / (1.0f + expf(-z));
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(u));
}

template <typename T>
__global__ void act_mul_kernel(const T* gu, T* out, size_t n_rows, int I, int kind) {
    pdl_trigger();
    pdl_wait();
    const size_t total = n_rows * (size_t)I;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t r = idx / I;
        const int i = (int)(idx - r * I);
        const T* row = gu + r * (size_t)(2 * I);
        out[idx] = from_f32<T>(__fmul_rn(gate_act(to_f32<T>(row[i]), kind), to_f32<T>(row[I + i])));
    }
}

PYRE_API int pyre_act_mul(const void* gu, void* out, int n_rows, int I, int kind, int dtype, cudaStream_t stream) {
    if (n_rows <= 0 || I <= 0) return 0;
    if (kind != 0 && kind != 1) return PYRE_ERR_BAD_ARG;
    const long long total = (long long)n_rows * I;
    const int blocks = (int)min((long long)pyre_sm_count() * 16, ceil_div_ll(total, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(act_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                    (size_t)n_rows, I, kind);
    else if (dtype == PYRE_F32)
        pyre_launch(act_mul_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gu, (float*)out, (size_t)n_rows, I, kind);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
