// Time mixing with a matrix state per head (an RWKV-style "wkv" mixer): the blend of each token's input with
// the previous token's, and the recurrence itself with its decay, bonus, per-head unit norm and gate.
// All arithmetic is fp32; `dtype` is the type of the activations (0 = float32, 1 = bfloat16).  A request's state
// slot holds, as floats, [heads][d][d] the matrices S and then [width] the last token's input of the mixer.
#include "common.cuh"

// ---------------------------------------------------------------------------
// out[s, t, i] = T( h[t, i] + (prev[t, i] - h[t, i]) * mu[s, i] )      s < n_mix blends of one token
//   prev[t] = h[t - 1] inside an entry of the step; for an entry's first token the vector kept in the request's
//   state slot (zeros for a new request).  One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void token_shift_mix_kernel(const T* h, const float* state, long long slot_stride, long long prev_off,
                                       const int* slots, const int* seq_of_token, const int* cu_seqlens, const float* mu,
                                       T* out, int n_tokens, int W, int n_mix) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int b = seq_of_token[t];
    const bool first = t == cu_seqlens[b];
    const float* kept = state + (size_t)slots[b] * slot_stride + prev_off;
    const T* cur = h + (size_t)t * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float x = to_f32<T>(cur[i]);
        const float p = first ? kept[i] : to_f32<T>(cur[i - W]);
        const float d = p - x;
        for (int s = 0; s < n_mix; ++s)
            out[((size_t)s * n_tokens + t) * W + i] = from_f32<T>(fmaf(d, mu[(size_t)s * W + i], x));
    }
}

PYRE_API int pyre_token_shift_mix(const void* h, const float* state, long long slot_stride, long long prev_off,
                                  const int* slots, const int* seq_of_token, const int* cu_seqlens, const float* mu, void* out,
                                  int n_tokens, int W, int n_mix, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (W <= 0 || n_mix <= 0 || !state || !slots || !seq_of_token || !cu_seqlens || prev_off < 0 || prev_off + W > slot_stride)
        return PYRE_ERR_BAD_ARG;
    const int threads = min(256, max(32, ((W + 31) / 32) * 32));
    if (dtype == PYRE_BF16)
        pyre_launch(token_shift_mix_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, (const __nv_bfloat16*)h, state, slot_stride, prev_off, slots, seq_of_token, cu_seqlens, mu, (__nv_bfloat16*)out, n_tokens, W, n_mix);
    else if (dtype == PYRE_F32)
        pyre_launch(token_shift_mix_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)h, state, slot_stride, prev_off, slots, seq_of_token, cu_seqlens, mu, (float*)out, n_tokens, W, n_mix);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The recurrence, token by token.  Per head, with r, k, v of d entries, the decay w = exp(-exp(dlog + w0)) per key
// channel and the bonus u:
//   o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])        the current token counts with the bonus only
//   S[i][j] = w_t[i] S[i][j] + k_t[i] v_t[j]
//   out[t, h d + j] = T( o_t[j] / sqrt(mean_j(o_t^2) + eps) * norm_w[h d + j] * silu(g[t, h d + j]) )
// One block per (head, entry); thread j keeps column j of S in registers and walks the entry's tokens in order,
// so a token's result does not depend on how the request was cut into steps or on what else the step holds.
// Block (0, b) also leaves the entry's last input row in the state slot for the next step's blend.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float wkv_silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T, int MAXD>
__global__ void __launch_bounds__(MAXD) wkv_scan_kernel(const T* r, const T* k, const T* v, const T* g, const float* dlog,
                                                        const float* w0, const float* u, const float* norm_w, float* state,
                                                        long long slot_stride, long long prev_off, const int* slots,
                                                        const int* cu_seqlens, const T* h, T* out, int H, int d, int W,
                                                        float eps) {
    __shared__ float sr[MAXD], sk[MAXD], sw[MAXD], su[MAXD];
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y, j = threadIdx.x;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    float* slot = state + (size_t)slots[b] * slot_stride;
    float* Sg = slot + (size_t)head * d * d;
    const bool own = j < d;
    const int col = head * d + j;
    float S[MAXD];
#pragma unroll
    for (int i = 0; i < MAXD; ++i) S[i] = (own && i < d) ? Sg[(size_t)i * d + j] : 0.f;
    if (own) su[j] = u[col];
    const float nw = own ? norm_w[col] : 0.f;
    const float wz = own ? w0[col] : 0.f;
    const size_t HD = (size_t)H * d;
    for (int t = t0; t < t1; ++t) {
        __syncthreads();      // the token before is done with sr / sk / sw
        float vj = 0.f;
        if (own) {
            sr[j] = to_f32<T>(r[t * HD + col]);
            sk[j] = to_f32<T>(k[t * HD + col]);
            sw[j] = expf(-expf(dlog[t * HD + col] + wz));
            vj = to_f32<T>(v[t * HD + col]);
        }
        __syncthreads();
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < MAXD; ++i) {
            if (i < d) {
                const float kv = sk[i] * vj;
                o = fmaf(sr[i], fmaf(su[i], kv, S[i]), o);
                S[i] = fmaf(sw[i], S[i], kv);
            }
        }
        const float ss = block_sum(own ? o * o : 0.f, scratch);
        if (own) {
            const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
            out[t * HD + col] = from_f32<T>(__fmul_rn(__fmul_rn(o, rstd), nw) * wkv_silu(to_f32<T>(g[t * HD + col])));
        }
    }
    if (own) {
#pragma unroll
        for (int i = 0; i < MAXD; ++i)
            if (i < d) Sg[(size_t)i * d + j] = S[i];
    }
    if (head == 0 && t1 > t0) {
        const T* last = h + (size_t)(t1 - 1) * W;
        for (int i = j; i < W; i += MAXD) slot[prev_off + i] = to_f32<T>(last[i]);
    }
}

PYRE_API int pyre_wkv_scan(const void* r, const void* k, const void* v, const void* g, const float* dlog, const float* w0,
                           const float* u, const float* norm_w, float* state, long long slot_stride, long long prev_off,
                           const int* slots, const int* cu_seqlens, const void* h, void* out, int n_tokens, int n_seqs, int H,
                           int d, int W, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || W <= 0 || !state || !slots || !cu_seqlens || prev_off < (long long)H * d * d || prev_off + W > slot_stride)
        return PYRE_ERR_BAD_ARG;
    if (d > 128) return PYRE_ERR_UNSUPPORTED;
    const dim3 grid(H, n_seqs);
#define WKV(TT, MD) pyre_launch(wkv_scan_kernel<TT, MD>, grid, dim3(MD), 0, stream, (const TT*)r, (const TT*)k, (const TT*)v, (const TT*)g, dlog, w0, u, norm_w, state, slot_stride, prev_off, slots, cu_seqlens, (const TT*)h, (TT*)out, H, d, W, eps)
#define WKV_PICK(TT) do { if (d <= 32) WKV(TT, 32); else if (d <= 64) WKV(TT, 64); else WKV(TT, 128); } while (0)
    if (dtype == PYRE_BF16) WKV_PICK(__nv_bfloat16);
    else if (dtype == PYRE_F32) WKV_PICK(float);
    else return PYRE_ERR_BAD_ARG;
#undef WKV_PICK
#undef WKV
    PYRE_LAUNCH_CHECK();
    return 0;
}
