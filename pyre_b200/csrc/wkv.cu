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
// ---------------------------------------------------------------------------
// The recurrence, token by token.  Per head, with r, k, v of d entries, the decay w = exp(-exp(dlog + w0)) per key
// channel and the bonus u:
//   o_t[j] = sum_i r_t[i] (S[i][j] + u[i] k_t[i] v_t[j])        the current token counts with the bonus only
//   S[i][j] = w_t[i] S[i][j] + k_t[i] v_t[j]
//   out[t, h d + j] = T( o_t[j] / sqrt(mean_j(o_t^2) + eps) * norm_w[h d + j] * silu(g[t, h d + j]) )
// A column j of S never meets another column, so the grid is (tiles of columns, heads, entries): a CTA of four warps
// (two for d <= 16) holds a [d, 32] tile of the head's state in registers.  A warp owns eight columns, and its lanes
// split the rows four ways in groups of four (row = 16 g + 4 q + e), so r, k and the decays come from shared memory
// as conflict-free 16-byte loads and the four row groups of a column meet in two shuffles.  Tokens are staged through
// shared memory sixteen at a time (decays evaluated while staging, all threads at once); the rows of the next
// sixteen are already on their way into registers while the staged ones run, so global latency shows once per
// entry, not once per chunk.  Four tokens run together where four are left, and their shuffles overlap.  The raw
// o goes to an fp32 scratch; the unit norm, gain and gate need the whole head and follow in wkv_finish_kernel.
// A token's arithmetic is the same wherever its chunk begins, so a result does not depend on how the request was
// cut into steps or on what else the step holds.  Block (0, 0, b) also leaves the entry's last input row in the
// state slot for the next step's blend.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float wkv_silu(float z) { return z / (1.0f + expf(-z)); }

constexpr int WKV_CHUNK = 16;      // tokens staged at a time

template <int G> struct WkvShape {
    static constexpr int DP = 16 * G;                       // rows, padded
    static constexpr int WARPS = G >= 2 ? 4 : 2;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int CT = WARPS * 8;                    // columns of a tile
    static constexpr int PER = WKV_CHUNK * DP / THREADS;    // staged (token, row) pairs per thread: 4 for G = 1, else 2 G
    static constexpr int PERV = WKV_CHUNK * CT / THREADS;   // staged (token, column) pairs per thread: 4
};

// U tokens from row tt of the staged chunk on
template <int G, int U>
__device__ __forceinline__ void wkv_tokens(float (&S)[4 * G], const float (&ub)[4 * G], const float (*sr)[16 * G],
                                           const float (*sk)[16 * G], const float (*sw)[16 * G], const float (*sv)[WkvShape<G>::CT],
                                           int tt, int q, int cw, bool store, float* o_at, size_t HD) {
    float acc[U];
#pragma unroll
    for (int x = 0; x < U; ++x) {
        const float vj = sv[tt + x][cw];
        float a = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) {
            const float4 k4 = *reinterpret_cast<const float4*>(&sk[tt + x][16 * gg + 4 * q]);
            const float4 r4 = *reinterpret_cast<const float4*>(&sr[tt + x][16 * gg + 4 * q]);
            const float4 w4 = *reinterpret_cast<const float4*>(&sw[tt + x][16 * gg + 4 * q]);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float kv = __fmul_rn(kk[e], vj);
                a = fmaf(rr[e], fmaf(ub[4 * gg + e], kv, S[4 * gg + e]), a);
                S[4 * gg + e] = fmaf(ww[e], S[4 * gg + e], kv);
            }
        }
        acc[x] = a;
    }
#pragma unroll
    for (int x = 0; x < U; ++x) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], 8);
#pragma unroll
    for (int x = 0; x < U; ++x) acc[x] += __shfl_xor_sync(0xffffffffu, acc[x], 16);
    if (store) {
#pragma unroll
        for (int x = 0; x < U; ++x) o_at[(size_t)(tt + x) * HD] = acc[x];
    }
}

template <typename T, int G>
__global__ void __launch_bounds__(WkvShape<G>::THREADS)
wkv_scan_kernel(const T* r, const T* k, const T* v, const float* dlog,
                const float* w0, const float* u, float* state, long long slot_stride,
                long long prev_off, const int* slots, const int* cu_seqlens,
                const T* h, float* o_raw, int H, int d, int W) {
    using Sh = WkvShape<G>;
    constexpr int DP = Sh::DP, THREADS = Sh::THREADS, CT = Sh::CT, PER = Sh::PER, PERV = Sh::PERV;
    __shared__ __align__(16) float sr[WKV_CHUNK][DP];
    __shared__ __align__(16) float sk[WKV_CHUNK][DP];
    __shared__ __align__(16) float sw[WKV_CHUNK][DP];
    __shared__ float sv[WKV_CHUNK][CT];
    __shared__ float sw0[DP];
    pdl_trigger();
    pdl_wait();
    const int tile = blockIdx.x, head = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int jj = lane & 7, q = lane >> 3;
    const int cw = warp * 8 + jj;             // column inside the tile
    const int col = tile * CT + cw;
    const bool col_ok = col < d;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    if (t1 <= t0) return;
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
    for (int i = tid; i < DP; i += THREADS) sw0[i] = i < d ? w0[base + i] : 0.f;

    // the rows of a chunk on their way from global memory to the staged arrays
    T pr[PER], pk[PER], pv[PERV];
    float pd[PER];
    auto fetch = [&](int c0) {
        const int n = min(WKV_CHUNK, t1 - c0);
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int e = p * THREADS + tid, tt = e / DP, i = e - tt * DP;
            const bool real = tt < n && i < d;
            const size_t at = (size_t)(c0 + tt) * HD + base + i;
            pr[p] = real ? r[at] : from_f32<T>(0.f);
            pk[p] = real ? k[at] : from_f32<T>(0.f);
            pd[p] = real ? dlog[at] : 0.f;
        }
#pragma unroll
        for (int p = 0; p < PERV; ++p) {
            const int e = p * THREADS + tid, tt = e / CT, c = e - tt * CT;
            const bool real = tt < n && tile * CT + c < d;
            pv[p] = real ? v[(size_t)(c0 + tt) * HD + base + tile * CT + c] : from_f32<T>(0.f);
        }
    };
    fetch(t0);

    for (int c0 = t0; c0 < t1; c0 += WKV_CHUNK) {
        const int n = min(WKV_CHUNK, t1 - c0);
        __syncthreads();      // the chunk before is done with the staged rows (and sw0 is written)
#pragma unroll
        for (int p = 0; p < PER; ++p) {
            const int e = p * THREADS + tid, tt = e / DP, i = e - tt * DP;
            const bool real = tt < n && i < d;
            sr[tt][i] = to_f32<T>(pr[p]);
            sk[tt][i] = to_f32<T>(pk[p]);
            sw[tt][i] = real ? expf(-expf(pd[p] + sw0[i])) : 0.f;
        }
#pragma unroll
        for (int p = 0; p < PERV; ++p) {
            const int e = p * THREADS + tid, tt = e / CT, c = e - tt * CT;
            sv[tt][c] = to_f32<T>(pv[p]);
        }
        __syncthreads();
        if (c0 + WKV_CHUNK < t1) fetch(c0 + WKV_CHUNK);
        float* o_at = o_raw + (size_t)c0 * HD + base + col;
        const bool store = col_ok && q == 0;
        int tt = 0;
        for (; tt + 4 <= n; tt += 4) wkv_tokens<G, 4>(S, ub, sr, sk, sw, sv, tt, q, cw, store, o_at, HD);
        for (; tt < n; ++tt) wkv_tokens<G, 1>(S, ub, sr, sk, sw, sv, tt, q, cw, store, o_at, HD);
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
    if (tile == 0 && head == 0) {
        const T* last = h + (size_t)(t1 - 1) * W;
        for (int i = tid; i < W; i += THREADS) slot[prev_off + i] = to_f32<T>(last[i]);
    }
}

// out[t, h d + j] = T( o[j] / sqrt(mean_j(o^2) + eps) * norm_w[h d + j] * silu(g[t, h d + j]) ), o the raw result of
// head h at token t: one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128) wkv_finish_kernel(const float* o_raw, const T* g,
                                                         const float* norm_w, T* out,
                                                         long long n_rows, int H, int d, float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int head = (int)(row % H);
    const size_t at = (size_t)row * d;          // (t H + head) d
    const size_t base = (size_t)head * d;
    float ss = 0.f;
    for (int j = lane; j < d; j += 32) { const float o = o_raw[at + j]; ss = fmaf(o, o, ss); }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
    const float rstd = 1.0f / sqrtf(ss / (float)d + eps);
    for (int j = lane; j < d; j += 32)
        out[at + j] = from_f32<T>(__fmul_rn(__fmul_rn(o_raw[at + j], rstd), norm_w[base + j]) * wkv_silu(to_f32<T>(g[at + j])));
}

// o_raw: fp32 scratch [n_tokens, H d]
PYRE_API int pyre_wkv_scan(const void* r, const void* k, const void* v, const void* g, const float* dlog, const float* w0,
                           const float* u, const float* norm_w, float* state, long long slot_stride, long long prev_off,
                           const int* slots, const int* cu_seqlens, const void* h, float* o_raw, void* out, int n_tokens,
                           int n_seqs, int H, int d, int W, float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || d <= 0 || W <= 0 || !state || !slots || !cu_seqlens || !o_raw || prev_off < (long long)H * d * d ||
        prev_off + W > slot_stride)
        return PYRE_ERR_BAD_ARG;
    if (d > 128 || n_seqs > 65535 || H > 65535) return PYRE_ERR_UNSUPPORTED;
    const long long n_rows = (long long)n_tokens * H;
    const dim3 fgrid((unsigned)((n_rows + 3) / 4));
#define WKV(TT, GG) do { \
        const dim3 grid((d + WkvShape<GG>::CT - 1) / WkvShape<GG>::CT, H, n_seqs); \
        pyre_launch(wkv_scan_kernel<TT, GG>, grid, dim3(WkvShape<GG>::THREADS), 0, stream, (const TT*)r, (const TT*)k, (const TT*)v, dlog, w0, u, state, slot_stride, prev_off, slots, cu_seqlens, (const TT*)h, o_raw, H, d, W); \
        PYRE_LAUNCH_CHECK(); \
        pyre_launch(wkv_finish_kernel<TT>, fgrid, dim3(128), 0, stream, (const float*)o_raw, (const TT*)g, norm_w, (TT*)out, n_rows, H, d, eps); \
    } while (0)
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
