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
// One CTA per (head, entry) holds the head's whole state in registers: a warp owns eight columns j, and its lanes
// split the rows four ways in groups of four (row = 16 g + 4 q + e), so r, k and the decays come from shared
// memory as conflict-free 16-byte loads and the four row groups of a column meet in two shuffles.  Tokens are
// staged through shared memory sixteen at a time (decays evaluated while staging, all threads at once); the sixteen
// tokens then run without a barrier, and their unit norm, gain and gate follow for all sixteen in parallel.  A
// token's arithmetic is the same wherever its chunk begins, so a result does not depend on how the request was cut
// into steps or on what else the step holds.  Block (0, b) also leaves the entry's last input row in the state
// slot for the next step's blend.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float wkv_silu(float z) { return z / (1.0f + expf(-z)); }

constexpr int WKV_CHUNK = 16;      // tokens staged at a time

// G: groups of 16 rows (d <= 16 G); a thread holds 4 G state elements of one column; ceil(d / 8) warps
template <typename T, int G>
__global__ void __launch_bounds__(G * 64) wkv_scan_kernel(const T* r, const T* k, const T* v, const T* g, const float* dlog,
                                                          const float* w0, const float* u, const float* norm_w, float* state,
                                                          long long slot_stride, long long prev_off, const int* slots,
                                                          const int* cu_seqlens, const T* h, T* out, int H, int d, int W,
                                                          float eps) {
    constexpr int DP = 16 * G;
    __shared__ __align__(16) float sr[WKV_CHUNK][DP];
    __shared__ __align__(16) float sk[WKV_CHUNK][DP];
    __shared__ __align__(16) float sw[WKV_CHUNK][DP];
    __shared__ float sv[WKV_CHUNK][DP];
    __shared__ float so[WKV_CHUNK][DP];
    pdl_trigger();
    pdl_wait();
    const int head = blockIdx.x, b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int jj = lane & 7, q = lane >> 3;
    const int col = warp * 8 + jj;
    const bool col_ok = col < d;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    float* slot = state + (size_t)slots[b] * slot_stride;
    float* Sg = slot + (size_t)head * d * d;
    const size_t HD = (size_t)H * d;
    const size_t base = (size_t)head * d;

    float S[4 * G], ub[4 * G];
#pragma unroll
    for (int gg = 0; gg < G; ++gg)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = 16 * gg + 4 * q + e;
            S[4 * gg + e] = (col_ok && i < d) ? Sg[(size_t)i * d + col] : 0.f;
            ub[4 * gg + e] = i < d ? u[base + i] : 0.f;
        }

    for (int c0 = t0; c0 < t1; c0 += WKV_CHUNK) {
        const int n = min(WKV_CHUNK, t1 - c0);
        __syncthreads();      // the chunk before is done with the staged rows and its outputs
        for (int e = threadIdx.x; e < n * DP; e += blockDim.x) {
            const int tt = e / DP, i = e - tt * DP;
            const size_t at = (size_t)(c0 + tt) * HD + base + i;
            const bool real = i < d;
            sr[tt][i] = real ? to_f32<T>(r[at]) : 0.f;
            sk[tt][i] = real ? to_f32<T>(k[at]) : 0.f;
            sv[tt][i] = real ? to_f32<T>(v[at]) : 0.f;
            sw[tt][i] = real ? expf(-expf(dlog[at] + w0[base + i])) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < n; ++tt) {
            const float vj = sv[tt][col];
            float acc = 0.f;
#pragma unroll
            for (int gg = 0; gg < G; ++gg) {
                const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt][16 * gg + 4 * q]);
                const float4 r4 = *reinterpret_cast<const float4*>(&sr[tt][16 * gg + 4 * q]);
                const float4 w4 = *reinterpret_cast<const float4*>(&sw[tt][16 * gg + 4 * q]);
                const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float kv = kk[e] * vj;
                    acc = fmaf(rr[e], fmaf(ub[4 * gg + e], kv, S[4 * gg + e]), acc);
                    S[4 * gg + e] = fmaf(ww[e], S[4 * gg + e], kv);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (q == 0) so[tt][col] = acc;
        }
        __syncthreads();
        // the chunk's tokens, one warp each: unit norm over the head, gain, gate
        for (int tt = warp; tt < n; tt += n_warps) {
            float ss = 0.f;
            for (int j = lane; j < d; j += 32) ss = fmaf(so[tt][j], so[tt][j], ss);
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
            const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
            const size_t at = (size_t)(c0 + tt) * HD + base;
            for (int j = lane; j < d; j += 32)
                out[at + j] = from_f32<T>(__fmul_rn(__fmul_rn(so[tt][j], rstd), norm_w[base + j]) * wkv_silu(to_f32<T>(g[at + j])));
        }
    }
    if (col_ok) {
#pragma unroll
        for (int gg = 0; gg < G; ++gg)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = 16 * gg + 4 * q + e;
                if (i < d) Sg[(size_t)i * d + col] = S[4 * gg + e];
            }
    }
    if (head == 0 && t1 > t0) {
        const T* last = h + (size_t)(t1 - 1) * W;
        for (int i = threadIdx.x; i < W; i += blockDim.x) slot[prev_off + i] = to_f32<T>(last[i]);
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
    const dim3 block(((d + 7) / 8) * 32);
#define WKV(TT, GG) pyre_launch(wkv_scan_kernel<TT, GG>, grid, block, 0, stream, (const TT*)r, (const TT*)k, (const TT*)v, (const TT*)g, dlog, w0, u, norm_w, state, slot_stride, prev_off, slots, cu_seqlens, (const TT*)h, (TT*)out, H, d, W, eps)
#define WKV_PICK(TT) do { if (d <= 16) WKV(TT, 1); else if (d <= 32) WKV(TT, 2); else if (d <= 48) WKV(TT, 3); else if (d <= 64) WKV(TT, 4); \
                          else if (d <= 96) WKV(TT, 6); else WKV(TT, 8); } while (0)
    if (dtype == PYRE_BF16) WKV_PICK(__nv_bfloat16);
    else if (dtype == PYRE_F32) WKV_PICK(float);
    else return PYRE_ERR_BAD_ARG;
#undef WKV_PICK
#undef WKV
    PYRE_LAUNCH_CHECK();
    return 0;
}
