// Small kernels of layers that are arranged otherwise than the pre-norm decoder block: a norm on a
// branch's OUTPUT that is added to the residual stream, the stream as activations, plain activation
// functions, per-head query/key norms with a partial rotation and the paged write for heads whose key and
// value sizes differ, and sigmoid gates on a mixer's output.  All arithmetic is fp32; `dtype` is the type
// of the activations and of the cache (0 = float32, 1 = bfloat16).  The residual stream is float32.
#include "common.cuh"

// ---------------------------------------------------------------------------
// out[i] = T(x[i]): the fp32 residual stream as the activations a branch reads.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void cast_rows_kernel(const float* x, T* out, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = from_f32<T>(x[i]);
}

PYRE_API int pyre_cast_rows(const float* x, void* out, long long n, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)min((long long)4096, ceil_div_ll(n, 256));
    if (dtype == PYRE_BF16) pyre_launch(cast_rows_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, x, (__nv_bfloat16*)out, (size_t)n);
    else if (dtype == PYRE_F32) pyre_launch(cast_rows_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (float*)out, (size_t)n);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Norm of a branch's output, added to the stream:
//   v      = y[r]  (activation dtype, or the sum of n_partials fp32 partial sums, added in index order)
//   x[r]  += (v * (1 / sqrt(mean(v^2) + eps))) * w
//   next[r] = T(x[r])   when `next` is given: what the following branch reads
// One block per row; the block size depends on H only, so a row's sum of squares is added in the same
// order whatever the batch holds.
// ---------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float branch_value(const T* yr, const float* pr, int n_partials, long long partial_stride, int i) {
    if (pr) {
        float acc = pr[i];
        for (int s = 1; s < n_partials; ++s) acc += pr[(size_t)s * partial_stride + i];
        return acc;
    }
    return to_f32<T>(yr[i]);
}

template <typename T>
__global__ void norm_add_kernel(float* x, const T* y, const float* partials, int n_partials, long long partial_stride,
                                const float* w, T* next, int H, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const T* yr = y ? y + (size_t)r * H : nullptr;
    const float* pr = partials ? partials + (size_t)r * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = branch_value<T>(yr, pr, n_partials, partial_stride, i);
        ss = fmaf(v, v, ss);
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);
    float* xr = x + (size_t)r * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = branch_value<T>(yr, pr, n_partials, partial_stride, i);
        const float s = xr[i] + __fmul_rn(__fmul_rn(v, rstd), w[i]);
        xr[i] = s;
        if (next) next[(size_t)r * H + i] = from_f32<T>(s);
    }
}

// The same for rows of H = 4 m elements: vectors of four, and a thread keeps its (at most KEEP) vectors of the branch
// output in registers between the sum of squares and the update, so the output is read once.  The sums are those
// of the scalar kernel in another order; a row's order depends on H alone.
template <typename T, int KEEP>
__global__ void norm_add_vec_kernel(float* x, const T* y, const float* partials, int n_partials, long long partial_stride,
                                    const float* w, T* next, int H, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const T* yr = y ? y + (size_t)r * H : nullptr;
    const float* pr = partials ? partials + (size_t)r * H : nullptr;
    Vec<float, 4> kept[KEEP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < H) {
            Vec<float, 4> v;
            if (pr) {
                v = load_vec<float, 4>(pr + i);
                for (int s = 1; s < n_partials; ++s) {
                    const Vec<float, 4> q = load_vec<float, 4>(pr + (size_t)s * partial_stride + i);
#pragma unroll
                    for (int k = 0; k < 4; ++k) v.v[k] += q.v[k];
                }
            } else {
                const Vec<T, 4> a = load_vec<T, 4>(yr + i);
#pragma unroll
                for (int k = 0; k < 4; ++k) v.v[k] = to_f32<T>(a.v[k]);
            }
            kept[j] = v;
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(v.v[k], v.v[k], ss);
        }
    }
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);
    float* xr = x + (size_t)r * H;
#pragma unroll
    for (int j = 0; j < KEEP; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < H) {
            Vec<float, 4> a = load_vec<float, 4>(xr + i);
            const Vec<float, 4> g = load_vec<float, 4>(w + i);
            Vec<T, 4> o;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                a.v[k] = a.v[k] + __fmul_rn(__fmul_rn(kept[j].v[k], rstd), g.v[k]);
                o.v[k] = from_f32<T>(a.v[k]);
            }
            store_vec<float, 4>(xr + i, a);
            if (next) store_vec<T, 4>(next + (size_t)r * H + i, o);
        }
    }
}

PYRE_API int pyre_norm_add(float* x, const void* y, const float* partials, int n_partials, long long partial_stride,
                           const float* weight, void* next, int n_rows, int H, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((y == nullptr) == (partials == nullptr)) return PYRE_ERR_BAD_ARG;
    if (partials && n_partials < 1) return PYRE_ERR_BAD_ARG;
    if (H % 4 == 0 && H <= 512 * 4 * 4 && partial_stride % 4 == 0 &&
        (((uintptr_t)x | (uintptr_t)partials | (uintptr_t)weight | (uintptr_t)y | (uintptr_t)next) & 15) == 0) {
        const int per = H / 4;
        const int threads = min(512, max(32, ((per + 31) / 32) * 32));
        const int per_thread = ceil_div(per, threads);
#define NA(TT, KP) pyre_launch(norm_add_vec_kernel<TT, KP>, dim3(n_rows), dim3(threads), 0, stream, x, (const TT*)y, partials, n_partials, partial_stride, weight, (TT*)next, H, eps)
#define NA_PICK(TT) do { if (per_thread <= 1) NA(TT, 1); else if (per_thread <= 2) NA(TT, 2); else NA(TT, 4); } while (0)
        if (dtype == PYRE_BF16) NA_PICK(__nv_bfloat16);
        else if (dtype == PYRE_F32) NA_PICK(float);
        else return PYRE_ERR_BAD_ARG;
#undef NA_PICK
#undef NA
        PYRE_LAUNCH_CHECK();
        return 0;
    }
    const int threads = min(512, max(32, ((H + 31) / 32) * 32));
    if (dtype == PYRE_BF16)
        pyre_launch(norm_add_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, x, (const __nv_bfloat16*)y, partials, n_partials, partial_stride, weight, (__nv_bfloat16*)next, H, eps);
    else if (dtype == PYRE_F32)
        pyre_launch(norm_add_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, x, (const float*)y, partials, n_partials, partial_stride, weight, (float*)next, H, eps);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[i] = act(in[i]);  kind 0: silu z / (1 + exp(-z));  kind 1: the tanh form of gelu,
// 0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float act_gelu_tanh(float z) {
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float act_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float act_relu2(float z) { return z > 0.f ? z * z : 0.f; }
__device__ __forceinline__ float act_any(float z, int kind) {
    return kind == 0 ? act_silu(z) : kind == 1 ? act_gelu_tanh(z) : kind == 2 ? act_relu2(z) : kind == 3 ? tanhf(z) : z;
}

template <typename T, int KIND>
__global__ void activation_kernel(const T* in, T* out, size_t n) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float z = to_f32<T>(in[i]);
        out[i] = from_f32<T>(KIND == 0 ? act_silu(z) : act_gelu_tanh(z));
    }
}

// the same in vectors of 16 bytes (n a multiple of VEC, both pointers aligned)
template <typename T, int KIND, int VEC>
__global__ void activation_vec_kernel(const T* in, T* out, size_t n_vec) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
        Vec<T, VEC> a = load_vec<T, VEC>(in + i * VEC), o;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float z = to_f32<T>(a.v[k]);
            o.v[k] = from_f32<T>(KIND == 0 ? act_silu(z) : act_gelu_tanh(z));
        }
        store_vec<T, VEC>(out + i * VEC, o);
    }
}

PYRE_API int pyre_activation(const void* in, void* out, long long n, int kind, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (kind != 0 && kind != 1) return PYRE_ERR_BAD_ARG;
    const int vec = dtype == PYRE_BF16 ? 8 : 4;
    const bool vector = n % vec == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const long long items = vector ? n / vec : n;
    const int blocks = (int)min((long long)148 * 16, ceil_div_ll(items, 256));
#define ACT(TT, K, V) do { if (vector) pyre_launch(activation_vec_kernel<TT, K, V>, dim3(blocks), dim3(256), 0, stream, (const TT*)in, (TT*)out, (size_t)items); \
                           else pyre_launch(activation_kernel<TT, K>, dim3(blocks), dim3(256), 0, stream, (const TT*)in, (TT*)out, (size_t)n); } while (0)
    if (dtype == PYRE_BF16) { if (kind == 0) ACT(__nv_bfloat16, 0, 8); else ACT(__nv_bfloat16, 1, 8); }
    else if (dtype == PYRE_F32) { if (kind == 0) ACT(float, 0, 4); else ACT(float, 1, 4); }
    else return PYRE_ERR_BAD_ARG;
#undef ACT
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Per-head norm of queries and keys, rotation of the first `rot` dims, and the paged write, for heads
// whose query/key size dk and value size dv differ from the cache's row size D (>= both; the rest of a
// row is zero, so that a kernel that works on D-wide heads sees the same scores and outputs).
//   proj [T, row_stride]: the token's projections; queries at column q_col (nh heads of dk), keys at
//         k_col (nkv heads of dk), values at v_col (nkv heads of dv); k_col < 0: no keys or values (a layer
//         that reads another layer's cache)
//   q_w, k_w [dk] fp32 or null: the weight of the RMS norm over a head's dk dims (shared by all heads),
//         n = (v * (1 / sqrt(mean(v^2) + eps))) * w; null: no norm
//   rotation (pairs (j, j + rot / 2), j < rot / 2, after the norm):
//         out[j] = n[j] cos[j] - n[j + rot/2] sin[j];  out[j + rot/2] = n[j + rot/2] cos[j] + n[j] sin[j]
//   vcos_t, vsin_t [T, dv / 2] or null: the VALUES are turned too, over all their dv dims (pairs (m, m + dv / 2)),
//         by tables of their own, and cached so; whoever reads them turns the weighted sum back (head_gate below)
//   q_out [T, nh, D]; cache: one layer [page][2][nkv][page_size][D]; slot_mapping[t] < 0: store nothing
// One warp per (token, head); the sum of squares is a warp reduction whose order depends on dk only.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void qk_norm_rope_write_kernel(const T* proj, long long row_stride, int q_col, int k_col, int v_col,
                                          const float* q_w, const float* k_w, float eps, const float* cos_t,
                                          const float* sin_t, const float* vcos_t, const float* vsin_t, T* q_out, T* cache,
                                          const int* slot_mapping, int n_tokens, int nh, int nkv, int dk, int dv, int D,
                                          int rot, int page_size, long long n_pages, int* err_flag) {
    extern __shared__ float head_smem[];   // [warps][D]
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int per_token = nh + (k_col >= 0 ? 2 * nkv : 0);
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)n_tokens * per_token) return;
    const int t = (int)(item / per_token), h = (int)(item - (long long)t * per_token);
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    const T* in = proj + (size_t)t * row_stride;
    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * nh + h) * D;
    } else {
        const int slot = (cache && slot_mapping) ? pyre_checked_slot(slot_mapping[t], n_pages, page_size, err_flag) : -1;
        if (slot < 0) return;
        const int page = slot / page_size, off = slot - page * page_size;
        const int kvh = is_k ? h - nh : h - nh - nkv;
        dst = cache + ((((size_t)page * 2 + (is_k ? 0 : 1)) * nkv + kvh) * page_size + off) * D;
    }
    if (!is_q && !is_k) {      // a value head: copied (or turned by its own tables), the rest of the row zero
        const T* src = in + v_col + (size_t)(h - nh - nkv) * dv;
        if (vcos_t) {
            const int vh = dv / 2;
            const float* ct = vcos_t + (size_t)t * vh;
            const float* st = vsin_t + (size_t)t * vh;
            for (int d = lane; d < D; d += 32) {
                float o = 0.f;
                if (d < vh) o = __fadd_rn(__fmul_rn(to_f32<T>(src[d]), ct[d]), __fmul_rn(-to_f32<T>(src[d + vh]), st[d]));
                else if (d < 2 * vh) o = __fadd_rn(__fmul_rn(to_f32<T>(src[d]), ct[d - vh]), __fmul_rn(to_f32<T>(src[d - vh]), st[d - vh]));
                else if (d < dv) o = to_f32<T>(src[d]);
                dst[d] = from_f32<T>(o);
            }
            return;
        }
        for (int d = lane; d < D; d += 32) dst[d] = d < dv ? src[d] : from_f32<T>(0.f);
        return;
    }
    const T* src = in + (is_q ? q_col + (size_t)h * dk : k_col + (size_t)(h - nh) * dk);
    const float* w = is_q ? q_w : k_w;
    float* n = head_smem + warp * D;
    float ss = 0.f;
    for (int d = lane; d < dk; d += 32) {
        const float v = to_f32<T>(src[d]);
        n[d] = v;
        ss = fmaf(v, v, ss);
    }
    if (w) {
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)dk + eps);
        for (int d = lane; d < dk; d += 32) n[d] = __fmul_rn(__fmul_rn(n[d], rstd), w[d]);
    }
    __syncwarp();
    const int half = rot / 2;
    const float* ct = cos_t ? cos_t + (size_t)t * half : nullptr;
    const float* st = sin_t ? sin_t + (size_t)t * half : nullptr;
    for (int d = lane; d < D; d += 32) {
        float o = 0.f;
        if (d < half) o = __fadd_rn(__fmul_rn(n[d], ct[d]), __fmul_rn(-n[d + half], st[d]));
        else if (d < rot) o = __fadd_rn(__fmul_rn(n[d], ct[d - half]), __fmul_rn(n[d - half], st[d - half]));
        else if (d < dk) o = n[d];
        dst[d] = from_f32<T>(o);
    }
}

PYRE_API int pyre_qk_norm_rope_write(const void* proj, long long row_stride, int q_col, int k_col, int v_col,
                                     const float* q_w, const float* k_w, float eps, const float* cos_t, const float* sin_t,
                                     const float* vcos_t, const float* vsin_t, void* q_out, void* cache, const int* slot_mapping, int n_tokens, int nh, int nkv,
                                     int dk, int dv, int D, int rot, int page_size, int dtype, long long n_pages,
                                     int* err_flag, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dk <= 0 || dv <= 0 || D < dk || D < dv || rot < 0 || rot > dk || rot % 2 || page_size <= 0 || nh <= 0 || nkv <= 0)
        return PYRE_ERR_BAD_ARG;
    if (rot && (!cos_t || !sin_t)) return PYRE_ERR_BAD_ARG;
    if ((vcos_t == nullptr) != (vsin_t == nullptr) || (vcos_t && dv % 2)) return PYRE_ERR_BAD_ARG;
    if (k_col >= 0 && !cache) k_col = -1;
    const int warps = 4;
    const long long items = (long long)n_tokens * (nh + (k_col >= 0 ? 2 * nkv : 0));
    const int blocks = (int)ceil_div_ll(items, warps);
    const size_t smem = (size_t)warps * D * sizeof(float);
    if (dtype == PYRE_BF16)
        pyre_launch(qk_norm_rope_write_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)proj, row_stride, q_col, k_col, v_col, q_w, k_w, eps, cos_t, sin_t, vcos_t, vsin_t, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, slot_mapping, n_tokens, nh, nkv, dk, dv, D, rot, page_size, n_pages, err_flag);
    else if (dtype == PYRE_F32)
        pyre_launch(qk_norm_rope_write_kernel<float>, dim3(blocks), dim3(warps * 32), smem, stream, (const float*)proj, row_stride, q_col, k_col, v_col, q_w, k_w, eps, cos_t, sin_t, vcos_t, vsin_t, (float*)q_out, (float*)cache, slot_mapping, n_tokens, nh, nkv, dk, dv, D, rot, page_size, n_pages, err_flag);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// A sigmoid gate on a mixer's heads: out[t, h, j] = a[t, h, j] * sigmoid(gate[t, h, j]) for j < dv, where a
// head of `a` has a_dim >= dv columns (the rest is dropped) and the gate lies in the token's projection row
// at column g_col (g_col < 0: no gate, the heads are only narrowed to dv columns).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void sigmoid_gate_kernel(const T* a, int a_dim, const T* proj, long long row_stride, int g_col, T* out,
                                    int n_tokens, int nh, int dv) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)n_tokens * nh * dv, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t t = i / ((size_t)nh * dv);
        const int c = (int)(i - t * nh * dv), h = c / dv, j = c - h * dv;
        const float g = g_col >= 0 ? act_sigmoid(to_f32<T>(proj[t * row_stride + g_col + c])) : 1.0f;
        out[i] = from_f32<T>(to_f32<T>(a[(t * nh + h) * a_dim + j]) * g);
    }
}

// the same in vectors of VEC elements along a head (dv, a_dim, g_col and row_stride multiples of VEC, aligned pointers)
template <typename T, int VEC>
__global__ void sigmoid_gate_vec_kernel(const T* a, int a_dim, const T* proj, long long row_stride, int g_col, T* out,
                                        int n_tokens, int nh, int dv) {
    pdl_trigger();
    pdl_wait();
    const int per_head = dv / VEC;
    const size_t n = (size_t)n_tokens * nh * per_head, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t t = i / ((size_t)nh * per_head);
        const int c = (int)(i - t * nh * per_head), h = c / per_head, j = (c - h * per_head) * VEC;
        Vec<T, VEC> v = load_vec<T, VEC>(a + (t * nh + h) * a_dim + j), o;
        if (g_col >= 0) {
            const Vec<T, VEC> gt = load_vec<T, VEC>(proj + t * row_stride + g_col + h * dv + j);
#pragma unroll
            for (int k = 0; k < VEC; ++k) o.v[k] = from_f32<T>(to_f32<T>(v.v[k]) * act_sigmoid(to_f32<T>(gt.v[k])));
        } else {
            o = v;
        }
        store_vec<T, VEC>(out + (t * nh + h) * dv + j, o);
    }
}

PYRE_API int pyre_sigmoid_gate(const void* a, int a_dim, const void* proj, long long row_stride, int g_col, void* out,
                               int n_tokens, int nh, int dv, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (a_dim < dv || dv <= 0 || nh <= 0 || (g_col >= 0 && !proj)) return PYRE_ERR_BAD_ARG;
    {
        const int vec = dtype == PYRE_BF16 ? 8 : 4;
        if (dv % vec == 0 && a_dim % vec == 0 && (g_col < 0 || (g_col % vec == 0 && row_stride % vec == 0)) &&
            (((uintptr_t)a | (uintptr_t)out | (uintptr_t)proj) & 15) == 0 && (dtype == PYRE_BF16 || dtype == PYRE_F32)) {
            const long long items = (long long)n_tokens * nh * (dv / vec);
            const int blocks = (int)min((long long)148 * 16, ceil_div_ll(items, 256));
            if (dtype == PYRE_BF16)
                pyre_launch(sigmoid_gate_vec_kernel<__nv_bfloat16, 8>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, a_dim, (const __nv_bfloat16*)proj, row_stride, g_col, (__nv_bfloat16*)out, n_tokens, nh, dv);
            else
                pyre_launch(sigmoid_gate_vec_kernel<float, 4>, dim3(blocks), dim3(256), 0, stream, (const float*)a, a_dim, (const float*)proj, row_stride, g_col, (float*)out, n_tokens, nh, dv);
            PYRE_LAUNCH_CHECK();
            return 0;
        }
    }
    const long long n = (long long)n_tokens * nh * dv;
    const int blocks = (int)min((long long)4096, ceil_div_ll(n, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, a_dim, (const __nv_bfloat16*)proj, row_stride, g_col, (__nv_bfloat16*)out, n_tokens, nh, dv);
    else if (dtype == PYRE_F32)
        pyre_launch(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, a_dim, (const float*)proj, row_stride, g_col, (float*)out, n_tokens, nh, dv);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// RMS norm over a whole row of fp32 mixer outputs, times a sigmoid gate:
//   out[t, i] = T( ((o[t, i] * (1 / sqrt(mean(o[t]^2) + eps))) * w[i]) * sigmoid(gate[t, i]) )
// with the gate in the token's projection row at column g_col (g_col < 0: no gate).  One block per row.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_gate_kernel(const float* o, const float* w, const T* proj, long long row_stride, int g_col, T* out,
                                    int H, float eps) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const float* orow = o + (size_t)r * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) ss = fmaf(orow[i], orow[i], ss);
    const float total = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(total / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = __fmul_rn(__fmul_rn(orow[i], rstd), w[i]);
        if (g_col >= 0) v *= act_sigmoid(to_f32<T>(proj[(size_t)r * row_stride + g_col + i]));
        out[(size_t)r * H + i] = from_f32<T>(v);
    }
}

PYRE_API int pyre_rmsnorm_gate(const float* o, const float* weight, const void* proj, long long row_stride, int g_col,
                               void* out, int n_rows, int H, float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || (g_col >= 0 && !proj)) return PYRE_ERR_BAD_ARG;
    const int threads = min(512, max(32, ((H + 31) / 32) * 32));
    if (dtype == PYRE_BF16)
        pyre_launch(rmsnorm_gate_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, o, weight, (const __nv_bfloat16*)proj, row_stride, g_col, (__nv_bfloat16*)out, H, eps);
    else if (dtype == PYRE_F32)
        pyre_launch(rmsnorm_gate_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, o, weight, (const float*)proj, row_stride, g_col, (float*)out, H, eps);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[r, i] = act(in[r, i] + bias[i]) over rows of H entries (bias null: none); kind 0 silu, 1 gelu (tanh form),
// 2 the square of relu, 3 tanh, 4 none (the bias only).  fp32 arithmetic on the product's result.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void bias_act_kernel(const T* in, const float* bias, T* out, size_t n, int H, int kind) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float z = to_f32<T>(in[i]);
        if (bias) z += bias[i % (size_t)H];
        out[i] = from_f32<T>(act_any(z, kind));
    }
}

PYRE_API int pyre_bias_act(const void* in, const float* bias, void* out, long long n_rows, int H, int kind, int dtype,
                           cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0 || kind < 0 || kind > 4) return PYRE_ERR_BAD_ARG;
    const long long n = n_rows * H;
    const int blocks = (int)min((long long)148 * 16, ceil_div_ll(n, 256));
    if (dtype == PYRE_BF16) pyre_launch(bias_act_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)in, bias, (__nv_bfloat16*)out, (size_t)n, H, kind);
    else if (dtype == PYRE_F32) pyre_launch(bias_act_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)in, bias, (float*)out, (size_t)n, H, kind);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// x[r, i] += v[i] for every row of the fp32 stream: a vector that a model adds to all tokens at one place of
// its schedule.
// ---------------------------------------------------------------------------
__global__ void add_row_vector_kernel(float* x, const float* v, size_t n, int H) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] += v[i % (size_t)H];
}

PYRE_API int pyre_add_row_vector(float* x, const float* v, long long n_rows, int H, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (H <= 0) return PYRE_ERR_BAD_ARG;
    const long long n = n_rows * H;
    const int blocks = (int)min((long long)148 * 16, ceil_div_ll(n, 256));
    pyre_launch(add_row_vector_kernel, dim3(blocks), dim3(256), 0, stream, x, v, (size_t)n, H);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// A branch's output, gated and normed, as an fp32 update of the stream (not added here: it travels to the next
// norm's kernel as one fp32 part):
//   v[i]   = (y[r, i] + y_bias[i]) * sigmoid(g[r, i] + g_bias[i])      y: activation dtype, or the sum of n_partials
//                                                                      fp32 partial sums; g null: no gate
//   out[r] = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps) * w     center = 1 (a layer norm without bias)
//   out[r] = v / sqrt(mean(v^2) + eps) * w                              center = 0
// One block per row, the row kept in shared memory; the block size depends on H only, so a row's sums are added in
// the same order whatever the batch holds.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gated_norm_kernel(const T* y, const float* partials, int n_partials, long long partial_stride,
                                  const float* y_bias, const T* g, const float* g_bias, const float* w, const float* out_bias,
                                  float* out, int H, float eps, int center) {
    extern __shared__ float row_smem[];   // [H]
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x;
    const T* yr = y ? y + (size_t)r * H : nullptr;
    const float* pr = partials ? partials + (size_t)r * H : nullptr;
    float sum = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = branch_value<T>(yr, pr, n_partials, partial_stride, i);
        if (y_bias) v += y_bias[i];
        if (g) v *= act_sigmoid(to_f32<T>(g[(size_t)r * H + i]) + (g_bias ? g_bias[i] : 0.f));
        row_smem[i] = v;
        sum += v;
    }
    float mean = 0.f;
    if (center) mean = block_sum(sum, scratch) / (float)H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float d = row_smem[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float o = __fmul_rn(__fmul_rn(row_smem[i] - mean, rstd), w[i]);
        out[(size_t)r * H + i] = out_bias ? __fadd_rn(o, out_bias[i]) : o;
    }
}

PYRE_API int pyre_gated_norm(const void* y, const float* partials, int n_partials, long long partial_stride,
                             const float* y_bias, const void* gate, const float* gate_bias, const float* weight,
                             const float* out_bias, float* out, int n_rows, int H, float eps, int center, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if ((y == nullptr) == (partials == nullptr) || (partials && n_partials < 1) || H <= 0 || !weight || !out) return PYRE_ERR_BAD_ARG;
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 48 * 1024) return PYRE_ERR_UNSUPPORTED;
    const int threads = min(512, max(32, ((H / 4 + 31) / 32) * 32));
    if (dtype == PYRE_BF16)
        pyre_launch(gated_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, (const __nv_bfloat16*)y, partials, n_partials, partial_stride, y_bias, (const __nv_bfloat16*)gate, gate_bias, weight, out_bias, out, H, eps, center);
    else if (dtype == PYRE_F32)
        pyre_launch(gated_norm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, (const float*)y, partials, n_partials, partial_stride, y_bias, (const float*)gate, gate_bias, weight, out_bias, out, H, eps, center);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// One gate per HEAD on a mixer's output, after turning each head's sum of rotated values back:
//   u = a[t, h, :dv]                     a head of `a` has a_dim >= dv columns (the rest is dropped)
//   pairs (m, m + dv / 2) of u turn by MINUS the token's angle (cos, sin [T, dv / 2]; null: no turn)
//   out[t, h, j] = u[j] * sigmoid(proj[t, g_col + h])          g_col < 0: no gate
// ---------------------------------------------------------------------------
template <typename T>
__global__ void head_gate_kernel(const T* a, int a_dim, const T* proj, long long row_stride, int g_col, const float* cos_t,
                                 const float* sin_t, T* out, int n_tokens, int nh, int dv) {
    pdl_trigger();
    pdl_wait();
    const int vh = dv / 2;
    const size_t n = (size_t)n_tokens * nh * dv, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const size_t t = i / ((size_t)nh * dv);
        const int c = (int)(i - t * nh * dv), h = c / dv, j = c - h * dv;
        const T* head = a + (t * nh + h) * a_dim;
        float u = to_f32<T>(head[j]);
        if (cos_t) {
            if (j < vh) u = __fadd_rn(__fmul_rn(u, cos_t[t * vh + j]), __fmul_rn(to_f32<T>(head[j + vh]), sin_t[t * vh + j]));
            else if (j < 2 * vh) u = __fadd_rn(__fmul_rn(u, cos_t[t * vh + j - vh]), __fmul_rn(-to_f32<T>(head[j - vh]), sin_t[t * vh + j - vh]));
        }
        const float gt = g_col >= 0 ? act_sigmoid(to_f32<T>(proj[t * row_stride + g_col + h])) : 1.0f;
        out[i] = from_f32<T>(u * gt);
    }
}

PYRE_API int pyre_head_gate(const void* a, int a_dim, const void* proj, long long row_stride, int g_col, const float* cos_t,
                            const float* sin_t, void* out, int n_tokens, int nh, int dv, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (a_dim < dv || dv <= 0 || nh <= 0 || (g_col >= 0 && !proj) || (cos_t == nullptr) != (sin_t == nullptr) || (cos_t && dv % 2))
        return PYRE_ERR_BAD_ARG;
    const long long n = (long long)n_tokens * nh * dv;
    const int blocks = (int)min((long long)148 * 16, ceil_div_ll(n, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(head_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)a, a_dim, (const __nv_bfloat16*)proj, row_stride, g_col, cos_t, sin_t, (__nv_bfloat16*)out, n_tokens, nh, dv);
    else if (dtype == PYRE_F32)
        pyre_launch(head_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)a, a_dim, (const float*)proj, row_stride, g_col, cos_t, sin_t, (float*)out, n_tokens, nh, dv);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
