// Kernels of mixers that carry a short history or a recurrent state per request, and the small steps around them:
//   * a short causal convolution per channel whose last inputs live in the request's state slot,
//   * the selective state-space recurrence (a matrix state per head, a step size per token and head),
//   * a unit norm over equal parts of a row with a gate before or after it,
//   * the combination of two softmax maps per head (a1 - lambda a2) with its unit norm,
//   * a rotation of the leading dims of heads that lie in a projection row, with a factor,
//   * a token's slice of a side table times gelu of a small projection, a shared branch added with one gate per
//     token, and a factor with a tanh cap on fp32 rows.
// All arithmetic is fp32; `dtype` is the type of the activations (0 = float32, 1 = bfloat16).
#include "common.cuh"

__device__ __forceinline__ float sm_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float sm_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sm_gelu_tanh(float z) {
    const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(u));
}
// log(1 + exp(z)) without a clamp; beyond 20 the sum is z itself in fp32
__device__ __forceinline__ float sm_softplus(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// ---------------------------------------------------------------------------
// x[i] = scale * x[i], then cap * tanh(x[i] / cap) where cap > 0.  fp32, in place.
// ---------------------------------------------------------------------------
__global__ void scale_cap_kernel(float* x, size_t n, float scale, float cap) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = __fmul_rn(x[i], scale);
        if (cap > 0.f) v = __fmul_rn(cap, tanhf(v / cap));
        x[i] = v;
    }
}

PYRE_API int pyre_scale_cap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll(n, 256));
    pyre_launch(scale_cap_kernel, dim3(blocks), dim3(256), 0, stream, x, (size_t)n, scale, cap);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Short causal convolution over time, per channel:
//   y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c])        j = 0 .. taps - 1, the last tap is the token's own
// u are `n_ch` columns of `in` from column `col`; inputs before an entry's first token come from the request's state
// slot, which holds the sequence's last taps - 1 inputs [taps - 1, n_ch] in fp32, oldest first, at `state_off` floats
// into the slot (zeros when the request begins: the zeros before a sequence's start).  The sum runs over j ascending
// whatever the cutting.  `silu` != 0: y = silu(.).  `in_bias` (fp32 [n_ch] or null) is added to every input as it is read
// from `in` (a projection's bias; the state holds inputs with it).  A second kernel moves the state on (after every read
// of the old one).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void short_conv_kernel(const T* in, long long row_stride, int col, const float* in_bias, const float* w, const float* bias,
                                  const float* state, long long slot_stride, long long state_off, const int* slots,
                                  const int* seq_of_token, const int* cu_seqlens, T* out, int n_tokens, int n_ch, int taps,
                                  int silu) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;                                  // a token per block row, the channels across threads and blockIdx.y
    const int b = seq_of_token[t];
    const int first = cu_seqlens[b];
    const float* hist = state + (size_t)slots[b] * slot_stride + state_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n_ch; c += gridDim.y * blockDim.x) {
        float acc = bias ? bias[c] : 0.f;
        const float ib = in_bias ? in_bias[c] : 0.f;
        for (int j = 0; j < taps; ++j) {
            const int local = t - first - (taps - 1) + j;      // index among the entry's tokens; negative: history
            const float u = local >= 0 ? __fadd_rn(to_f32<T>(in[(size_t)(first + local) * row_stride + col + c]), ib)
                                       : hist[(size_t)(taps - 1 + local) * n_ch + c];
            acc = fmaf(w[(size_t)c * taps + j], u, acc);
        }
        out[(size_t)t * n_ch + c] = from_f32<T>(silu ? sm_silu(acc) : acc);
    }
}

// The same for up to CONV_MAX_TAPS taps, a tile of CONV_TILE consecutive tokens per block: a thread walks its channel
// through the tile with the last inputs in registers, so every input and every tap is read once.  The window is filled
// anew where the tile or an entry begins (from the tokens before, or from the history).  Same sum, same order.
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_TILE = 8;

template <typename T>
__global__ void short_conv_tiled_kernel(const T* in, long long row_stride, int col, const float* in_bias, const float* w,
                                        const float* bias, const float* state, long long slot_stride, long long state_off,
                                        const int* slots, const int* seq_of_token, const int* cu_seqlens, T* out, int n_tokens,
                                        int n_ch, int taps, int silu) {
    pdl_trigger();
    pdl_wait();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= n_ch) return;
    const int t0 = blockIdx.x * CONV_TILE, t1 = min(t0 + CONV_TILE, n_tokens);
    float wt[CONV_MAX_TAPS], u[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        u[j] = 0.f;
    }
    const float b0 = bias ? bias[c] : 0.f, ib = in_bias ? in_bias[c] : 0.f;
    int entry = -1;
    for (int t = t0; t < t1; ++t) {
        const int b = seq_of_token[t];
        if (b != entry) {                                      // the window's first taps - 1 inputs: tokens before, or the history
            entry = b;
            const int first = cu_seqlens[b];
            const float* hist = state + (size_t)slots[b] * slot_stride + state_off;
#pragma unroll
            for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
                if (j < taps - 1) {
                    const int local = t - first - (taps - 1) + j;
                    u[j] = local >= 0 ? __fadd_rn(to_f32<T>(in[(size_t)(first + local) * row_stride + col + c]), ib)
                                      : hist[(size_t)(taps - 1 + local) * n_ch + c];
                }
            }
        }
        const float now = __fadd_rn(to_f32<T>(in[(size_t)t * row_stride + col + c]), ib);
        float acc = b0;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < taps) {
                const float v = j == taps - 1 ? now : u[j];
                acc = fmaf(wt[j], v, acc);
            }
        }
        out[(size_t)t * n_ch + c] = from_f32<T>(silu ? sm_silu(acc) : acc);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {          // the window moves on by one input
            if (j < taps - 1) u[j] = j == taps - 2 ? now : u[j + 1];
        }
    }
}

// The same for 2 to CONV_VEC_TAPS taps (a template parameter: no predicate per tap) where rows, columns and channel counts
// are multiples of a 16-byte vector: a thread walks 16 bytes of channels (eight bfloat16 or four float) through the tile, one
// vector load and one vector store per token.  Per channel the same sum in the same order.  The kernel was bound by the
// instructions it issues, not by memory: with bfloat16 results silu uses the fast exponential and reciprocal (their error is
// a thousandth of the result's rounding).
constexpr int CONV_VEC_TAPS = 4;

template <typename T> __device__ __forceinline__ float conv_silu(float z) { return sm_silu(z); }
template <> __device__ __forceinline__ float conv_silu<__nv_bfloat16>(float z) { return z * __frcp_rn(1.0f + __expf(-z)); }

template <typename T, int TAPS>
__global__ void short_conv_vec_kernel(const T* in, long long row_stride, int col, const float* in_bias, const float* w,
                                      const float* bias, const float* state, long long slot_stride, long long state_off,
                                      const int* slots, const int* seq_of_token, const int* cu_seqlens, T* out, int n_tokens,
                                      int n_ch, int silu) {
    constexpr int V = 16 / sizeof(T);
    pdl_trigger();
    pdl_wait();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    if (c >= n_ch) return;
    const int t0 = blockIdx.x * CONV_TILE, t1 = min(t0 + CONV_TILE, n_tokens);
    float wt[TAPS][V], u[TAPS - 1][V], b0[V], ib[V];
#pragma unroll
    for (int v = 0; v < V; ++v) {
        b0[v] = bias ? bias[c + v] : 0.f;
        ib[v] = in_bias ? in_bias[c + v] : 0.f;
#pragma unroll
        for (int j = 0; j < TAPS; ++j) wt[j][v] = w[(size_t)(c + v) * TAPS + j];
#pragma unroll
        for (int j = 0; j < TAPS - 1; ++j) u[j][v] = 0.f;
    }
    int entry = -1;
    const T* src = in + (size_t)t0 * row_stride + col + c;
    T* dst = out + (size_t)t0 * n_ch + c;
    for (int t = t0; t < t1; ++t, src += row_stride, dst += n_ch) {
        const int b = seq_of_token[t];
        if (b != entry) {                                      // the window's first taps - 1 inputs: tokens before, or the history
            entry = b;
            const int first = cu_seqlens[b];
            const float* hist = state + (size_t)slots[b] * slot_stride + state_off;
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) {
                const int local = t - first - (TAPS - 1) + j;
                if (local >= 0) {
                    const Vec<T, V> x = load_vec<T, V>(in + (size_t)(first + local) * row_stride + col + c);
#pragma unroll
                    for (int v = 0; v < V; ++v) u[j][v] = __fadd_rn(to_f32<T>(x.v[v]), ib[v]);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) u[j][v] = hist[(size_t)(TAPS - 1 + local) * n_ch + c + v];
                }
            }
        }
        const Vec<T, V> x = load_vec<T, V>(src);
        Vec<T, V> y;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const float now = __fadd_rn(to_f32<T>(x.v[v]), ib[v]);
            float acc = b0[v];
#pragma unroll
            for (int j = 0; j < TAPS - 1; ++j) acc = fmaf(wt[j][v], u[j][v], acc);
            acc = fmaf(wt[TAPS - 1][v], now, acc);
            y.v[v] = from_f32<T>(silu ? conv_silu<T>(acc) : acc);
#pragma unroll
            for (int j = 0; j + 1 < TAPS - 1; ++j) u[j][v] = u[j + 1][v];      // the window moves on by one input
            u[TAPS - 2][v] = now;
        }
        store_vec<T, V>(dst, y);
    }
}

template <typename T>
static void launch_conv_vec(int taps, dim3 grid, cudaStream_t stream, const void* in, long long row_stride, int col,
                            const float* in_bias, const float* w, const float* bias, const float* state, long long slot_stride,
                            long long state_off, const int* slots, const int* seq_of_token, const int* cu_seqlens, void* out,
                            int n_tokens, int n_ch, int silu) {
#define CONV_VEC_CASE(TAPS_)                                                                                                  \
    pyre_launch(short_conv_vec_kernel<T, TAPS_>, grid, dim3(64), 0, stream, (const T*)in, row_stride, col, in_bias, w, bias,  \
                state, slot_stride, state_off, slots, seq_of_token, cu_seqlens, (T*)out, n_tokens, n_ch, silu)
    if (taps == 2) CONV_VEC_CASE(2);
    else if (taps == 3) CONV_VEC_CASE(3);
    else CONV_VEC_CASE(4);
#undef CONV_VEC_CASE
}

// state[i] <- the sequence's input number (len - (taps - 1) + i) counted from the entry's first token; a negative
// number is an input the state already holds, at i + len.  One thread per (entry, channel), i ascending: what it
// reads lies above what it has written.
template <typename T>
__global__ void short_conv_state_kernel(const T* in, long long row_stride, int col, const float* in_bias, float* state, long long slot_stride,
                                        long long state_off, const int* slots, const int* cu_seqlens, int n_seqs, int n_ch,
                                        int taps) {
    pdl_trigger();
    pdl_wait();
    const int total = n_seqs * n_ch;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int b = i / n_ch, c = i - b * n_ch;
        const int first = cu_seqlens[b], len = cu_seqlens[b + 1] - first;
        if (len <= 0) continue;
        float* hist = state + (size_t)slots[b] * slot_stride + state_off;
        const float ib = in_bias ? in_bias[c] : 0.f;
        for (int k = 0; k < taps - 1; ++k) {
            const int local = len - (taps - 1) + k;
            hist[(size_t)k * n_ch + c] = local >= 0 ? __fadd_rn(to_f32<T>(in[(size_t)(first + local) * row_stride + col + c]), ib)
                                                    : hist[(size_t)(k + len) * n_ch + c];
        }
    }
}

PYRE_API int pyre_short_conv(const void* in, long long row_stride, int col, const float* in_bias, const float* w, const float* bias, float* state,
                             long long slot_stride, long long state_off, const int* slots, const int* seq_of_token,
                             const int* cu_seqlens, void* out, int n_tokens, int n_seqs, int n_ch, int taps, int silu, int dtype,
                             cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (n_ch <= 0 || taps < 1 || col < 0 || !w || !state || !slots || !seq_of_token || !cu_seqlens) return PYRE_ERR_BAD_ARG;
    const dim3 blocks(n_tokens, min(ceil_div(n_ch, 256), 64));
    const int sblocks = (int)min((long long)pyre_sm_count() * 4, ceil_div_ll((long long)n_seqs * n_ch, 128));
    // prompt portions walk tiles of tokens; steps of single tokens (every token another entry) keep a thread per element
    const bool tiled = taps <= CONV_MAX_TAPS && n_tokens >= 8 * n_seqs;
    const dim3 tiles(ceil_div(n_tokens, CONV_TILE), ceil_div(n_ch, 128));
    // 16 bytes of channels per thread where everything is a multiple of a vector
    const int vlen = dtype == PYRE_BF16 ? 8 : 4;
    const bool vec = tiled && taps >= 2 && taps <= CONV_VEC_TAPS && n_ch % vlen == 0 && col % vlen == 0 && row_stride % vlen == 0 &&
                     (((uintptr_t)in | (uintptr_t)out) & 15) == 0;
    const dim3 vtiles(ceil_div(n_tokens, CONV_TILE), ceil_div(n_ch / vlen, 64));
    if (dtype == PYRE_BF16) {
        if (vec)
            launch_conv_vec<__nv_bfloat16>(taps, vtiles, stream, in, row_stride, col, in_bias, w, bias, (const float*)state, slot_stride,
                                           state_off, slots, seq_of_token, cu_seqlens, out, n_tokens, n_ch, silu);
        else if (tiled)
            pyre_launch(short_conv_tiled_kernel<__nv_bfloat16>, tiles, dim3(128), 0, stream, (const __nv_bfloat16*)in, row_stride, col,
                        in_bias, w, bias, (const float*)state, slot_stride, state_off, slots, seq_of_token, cu_seqlens,
                        (__nv_bfloat16*)out, n_tokens, n_ch, taps, silu);
        else
        pyre_launch(short_conv_kernel<__nv_bfloat16>, blocks, dim3(256), 0, stream, (const __nv_bfloat16*)in, row_stride, col, in_bias, w,
                    bias, (const float*)state, slot_stride, state_off, slots, seq_of_token, cu_seqlens, (__nv_bfloat16*)out, n_tokens,
                    n_ch, taps, silu);
        PYRE_LAUNCH_CHECK();
        if (taps > 1)
            pyre_launch(short_conv_state_kernel<__nv_bfloat16>, dim3(sblocks), dim3(128), 0, stream, (const __nv_bfloat16*)in, row_stride,
                        col, in_bias, state, slot_stride, state_off, slots, cu_seqlens, n_seqs, n_ch, taps);
    } else if (dtype == PYRE_F32) {
        if (vec)
            launch_conv_vec<float>(taps, vtiles, stream, in, row_stride, col, in_bias, w, bias, (const float*)state, slot_stride,
                                   state_off, slots, seq_of_token, cu_seqlens, out, n_tokens, n_ch, silu);
        else if (tiled)
            pyre_launch(short_conv_tiled_kernel<float>, tiles, dim3(128), 0, stream, (const float*)in, row_stride, col, in_bias, w, bias,
                        (const float*)state, slot_stride, state_off, slots, seq_of_token, cu_seqlens, (float*)out, n_tokens, n_ch,
                        taps, silu);
        else
        pyre_launch(short_conv_kernel<float>, blocks, dim3(256), 0, stream, (const float*)in, row_stride, col, in_bias, w, bias,
                    (const float*)state, slot_stride, state_off, slots, seq_of_token, cu_seqlens, (float*)out, n_tokens, n_ch, taps,
                    silu);
        PYRE_LAUNCH_CHECK();
        if (taps > 1)
            pyre_launch(short_conv_state_kernel<float>, dim3(sblocks), dim3(128), 0, stream, (const float*)in, row_stride, col, in_bias, state,
                        slot_stride, state_off, slots, cu_seqlens, n_seqs, n_ch, taps);
    } else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The selective state-space recurrence.  Per head h (group g = h / (H / G)), with x_t [P], B_t and C_t [N] columns of
// `xbc` (x at column 0, B at H P, C at H P + G N) and the raw step size a column of `proj`:
//   dt  = softplus(raw + dt_bias[h])                 decay = exp(-exp(A_log[h]) * dt)
//   S_t = decay * S_(t-1) + dt * B_t x_t^T           S [N, P] fp32, in the request's state slot
//   y_t = S_t^T C_t + D[h] x_t                       fp32 [T, H P]
// A column of S never meets another column, so the grid is (tiles of 32 columns, heads, entries).  A CTA keeps its
// [N, 32] tile in registers for the whole entry: a warp owns 32 / RG columns, its lanes split the rows RG ways (lane
// group r has the NR rows from r * NR, which it reads from shared memory as 16-byte vectors; rows beyond N are padding
// whose B is zero), and a column's partial sums meet in log2(RG) shuffles.  RG = 4 (four warps, eight
// columns each): a row segment of a warp's state is a whole 32-byte sector, for steps of single tokens, where reading
// and writing the state is the work.  RG = 16 (sixteen warps, two columns each): a quarter of the rows per thread and
// four times the warps, for prompt portions, where the token loop's latency is the work.  Tokens are staged through
// shared memory sixteen at a time (B, C, x, dt and the decay, evaluated while staging); a token's arithmetic does not
// depend on where a chunk begins, so with one RG results are bit-identical under cutting and batching.
// ---------------------------------------------------------------------------
constexpr int SSM_COLS = 32;      // columns of a CTA
constexpr int SSM_STAGE = 16;     // tokens staged at a time

template <typename T, int NR, int RG>     // NR: rows per thread, N <= RG * NR =: NP, the rows with padding
__global__ void __launch_bounds__(SSM_COLS * RG)
ssm_scan_kernel(const T* xbc, long long xbc_stride, const T* proj, long long proj_stride, int dt_col, const float* dt_bias,
                const float* A_log, const float* D, float* state, long long slot_stride, const int* slots,
                const int* cu_seqlens, float* y, int H, int G, int P, int N) {
    extern __shared__ __align__(16) float ssm_smem[];   // [STAGE][2 NP] B | C (zeros beyond N), [STAGE][COLS] x, [STAGE] dt, [STAGE] decay
    pdl_trigger();
    pdl_wait();
    constexpr int NP = NR * RG, THREADS = SSM_COLS * RG, CPW = 32 / RG;      // CPW: columns of a warp
    constexpr int XR = SSM_STAGE * SSM_COLS / THREADS;                       // x values per thread and chunk
    constexpr bool PREFETCH = RG > 4;                                        // the variant for prompt portions
    const int tile = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int first = cu_seqlens[b], len = cu_seqlens[b + 1] - first;
    if (len <= 0) return;
    const int g = h / (H / G);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rg = lane / CPW;                                 // which share of the rows: rows rg * NR .. rg * NR + NR - 1
    const int jc = warp * CPW + (lane % CPW);                  // column inside the tile
    const int j = tile * SSM_COLS + jc;
    const bool live = j < P;
    float* bc_s = ssm_smem;
    float* x_s = bc_s + SSM_STAGE * 2 * NP;
    float* dt_s = x_s + SSM_STAGE * SSM_COLS;
    float* dec_s = dt_s + SSM_STAGE;
    float* S = state + (size_t)slots[b] * slot_stride + ((size_t)h * N) * P;
    float s[NR];                                               // a padded row stays zero: its B is zero
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int n = rg * NR + i;
        s[i] = (live && n < N) ? S[(size_t)n * P + j] : 0.f;
    }
    const float a = expf(A_log[h]), bias = dt_bias[h], d_skip = D[h];
    const int b_col = H * P + g * N, c_col = H * P + G * N + g * N;
    // Element e of a chunk's [tokens][B | C] belongs to thread e mod THREADS (NR of them per thread), likewise its
    // [tokens][columns] of x (XR per thread); thread t < tokens has the token's raw step size.
    auto load_bc = [&](int base, int n_tok, int k) -> float {
        const int i = threadIdx.x + k * THREADS;
        const int tt = i / (2 * NP), e = i % (2 * NP), at = e % NP;            // powers of two
        // where row n lies in a token's staged B (and C): lane group r reads its NR rows as vectors of V = min(NR, 4),
        // and the groups' k-th vectors lie side by side (no two lanes of a load share a bank): [NR / V][RG][V]
        constexpr int V = NR < 4 ? NR : 4;
        const int n = ((at / V) % RG) * NR + (at / (V * RG)) * V + at % V;
        if (tt >= n_tok || n >= N) return 0.f;
        return to_f32<T>(xbc[(size_t)(first + base + tt) * xbc_stride + (e < NP ? b_col : c_col) + n]);
    };
    auto load_x = [&](int base, int n_tok, int k) -> float {
        const int i = threadIdx.x + k * THREADS;
        const int tt = i / SSM_COLS, col = tile * SSM_COLS + i % SSM_COLS;
        return (tt < n_tok && col < P) ? to_f32<T>(xbc[(size_t)(first + base + tt) * xbc_stride + h * P + col]) : 0.f;
    };
    auto load_dt = [&](int base, int n_tok) -> float {
        return (int)threadIdx.x < n_tok ? to_f32<T>(proj[(size_t)(first + base + threadIdx.x) * proj_stride + dt_col + h]) : 0.f;
    };
    // With PREFETCH the next sixteen tokens are on their way into registers while the staged ones run.
    float pre_bc[PREFETCH ? NR : 1], pre_x[PREFETCH ? XR : 1], pre_dt = 0.f;
    if (PREFETCH) {
        const int n0 = min(SSM_STAGE, len);
#pragma unroll
        for (int k = 0; k < NR; ++k) pre_bc[PREFETCH ? k : 0] = load_bc(0, n0, k);
#pragma unroll
        for (int k = 0; k < XR; ++k) pre_x[PREFETCH ? k : 0] = load_x(0, n0, k);
        pre_dt = load_dt(0, n0);
    }
    for (int base = 0; base < len; base += SSM_STAGE) {
        const int n_tok = min(SSM_STAGE, len - base);
        __syncthreads();      // the chunk before has been consumed
#pragma unroll
        for (int k = 0; k < NR; ++k)
            if (PREFETCH || k * THREADS < n_tok * 2 * NP)
                bc_s[threadIdx.x + k * THREADS] = PREFETCH ? pre_bc[PREFETCH ? k : 0] : load_bc(base, n_tok, k);
#pragma unroll
        for (int k = 0; k < XR; ++k)
            if (PREFETCH || k * THREADS < n_tok * SSM_COLS)
                x_s[threadIdx.x + k * THREADS] = PREFETCH ? pre_x[PREFETCH ? k : 0] : load_x(base, n_tok, k);
        if ((int)threadIdx.x < n_tok) {
            const float dt = sm_softplus(__fadd_rn(PREFETCH ? pre_dt : load_dt(base, n_tok), bias));
            dt_s[threadIdx.x] = dt;
            dec_s[threadIdx.x] = expf(-__fmul_rn(a, dt));
        }
        __syncthreads();
        if (PREFETCH && base + SSM_STAGE < len) {
            const int n1 = min(SSM_STAGE, len - base - SSM_STAGE);
#pragma unroll
            for (int k = 0; k < NR; ++k) pre_bc[PREFETCH ? k : 0] = load_bc(base + SSM_STAGE, n1, k);
#pragma unroll
            for (int k = 0; k < XR; ++k) pre_x[PREFETCH ? k : 0] = load_x(base + SSM_STAGE, n1, k);
            pre_dt = load_dt(base + SSM_STAGE, n1);
        }
        float* yo = y + (size_t)(first + base) * ((size_t)H * P) + (size_t)h * P + j;
        // one token: the state moves on and the thread's share of y_t comes back
        auto token = [&](int tt) -> float {
            constexpr int V = NR < 4 ? NR : 4;
            const float* Bt = bc_s + tt * 2 * NP + rg * V;     // vector k of this lane group at k * RG * V
            const float* Ct = Bt + NP;
            const float dx = __fmul_rn(dt_s[tt], x_s[tt * SSM_COLS + jc]), dec = dec_s[tt];
            float bv[NR], cv[NR];
            if (NR % 4 == 0) {
#pragma unroll
                for (int i = 0; i < NR; i += 4) {
                    *reinterpret_cast<float4*>(bv + i) = *reinterpret_cast<const float4*>(Bt + i * RG);
                    *reinterpret_cast<float4*>(cv + i) = *reinterpret_cast<const float4*>(Ct + i * RG);
                }
            } else {
#pragma unroll
                for (int i = 0; i < NR; i += 2) {
                    *reinterpret_cast<float2*>(bv + i) = *reinterpret_cast<const float2*>(Bt + i * RG);
                    *reinterpret_cast<float2*>(cv + i) = *reinterpret_cast<const float2*>(Ct + i * RG);
                }
            }
            float acc0 = 0.f, acc1 = 0.f;                      // two chains: rows of even and of odd i
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                s[i] = fmaf(dec, s[i], __fmul_rn(dx, bv[i]));
                if (i & 1) acc1 = fmaf(s[i], cv[i], acc1);
                else acc0 = fmaf(s[i], cv[i], acc0);
            }
            return acc0 + acc1;
        };
        // a column's shares meet across the lane groups; lane group 0 writes y_t
        auto finish = [&](int tt, float acc) {
#pragma unroll
            for (int o = CPW; o < 32; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (live && rg == 0) yo[(size_t)tt * ((size_t)H * P)] = fmaf(d_skip, x_s[tt * SSM_COLS + jc], acc);
        };
        if (PREFETCH && n_tok == SSM_STAGE) {
            // a whole chunk: the sixteen tokens' shares wait in registers and meet after the loop, so that the shuffles
            // of one token do not stand in the way of the next token's state (same sums, same order)
            float part[SSM_STAGE];
#pragma unroll
            for (int tt = 0; tt < SSM_STAGE; ++tt) part[tt] = token(tt);
#pragma unroll
            for (int tt = 0; tt < SSM_STAGE; ++tt) finish(tt, part[tt]);
        } else {
            for (int tt = 0; tt < n_tok; ++tt) finish(tt, token(tt));
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int n = rg * NR + i;
            if (n < N) S[(size_t)n * P + j] = s[i];
        }
    }
}

template <typename T, int NR, int RG>
static int launch_ssm_as(const void* xbc, long long xbc_stride, const void* proj, long long proj_stride, int dt_col,
                         const float* dt_bias, const float* A_log, const float* D, float* state, long long slot_stride,
                         const int* slots, const int* cu_seqlens, float* y, int n_seqs, int H, int G, int P, int N, cudaStream_t stream) {
    const dim3 grid(ceil_div(P, SSM_COLS), H, n_seqs);
    const size_t smem = ((size_t)SSM_STAGE * 2 * NR * RG + SSM_STAGE * SSM_COLS + 2 * SSM_STAGE) * sizeof(float);
    pyre_launch(ssm_scan_kernel<T, NR, RG>, grid, dim3(SSM_COLS * RG), smem, stream, (const T*)xbc, xbc_stride, (const T*)proj,
                proj_stride, dt_col, dt_bias, A_log, D, state, slot_stride, slots, cu_seqlens, y, H, G, P, N);
    PYRE_LAUNCH_CHECK();
    return 0;
}

template <typename T>
static int launch_ssm(bool wide, const void* xbc, long long xbc_stride, const void* proj, long long proj_stride, int dt_col,
                      const float* dt_bias, const float* A_log, const float* D, float* state, long long slot_stride,
                      const int* slots, const int* cu_seqlens, float* y, int n_seqs, int H, int G, int P, int N, cudaStream_t stream) {
#define SSM_ARGS xbc, xbc_stride, proj, proj_stride, dt_col, dt_bias, A_log, D, state, slot_stride, slots, cu_seqlens, y, n_seqs, H, G, P, N, stream
    if (wide) {
        if (N <= 32) return launch_ssm_as<T, 2, 16>(SSM_ARGS);
        if (N <= 64) return launch_ssm_as<T, 4, 16>(SSM_ARGS);
        if (N <= 128) return launch_ssm_as<T, 8, 16>(SSM_ARGS);
        return launch_ssm_as<T, 16, 16>(SSM_ARGS);
    }
    if (N <= 32) return launch_ssm_as<T, 8, 4>(SSM_ARGS);
    if (N <= 64) return launch_ssm_as<T, 16, 4>(SSM_ARGS);
    if (N <= 128) return launch_ssm_as<T, 32, 4>(SSM_ARGS);
    return launch_ssm_as<T, 64, 4>(SSM_ARGS);
#undef SSM_ARGS
}

// `wide` != 0: the variant for prompt portions (sixteen warps per tile); 0: the one for steps of single tokens.
PYRE_API int pyre_ssm_scan(const void* xbc, long long xbc_stride, const void* proj, long long proj_stride, int dt_col,
                           const float* dt_bias, const float* A_log, const float* D, float* state, long long slot_stride,
                           const int* slots, const int* cu_seqlens, float* y, int n_tokens, int n_seqs, int H, int G, int P, int N,
                           int wide, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || P <= 0 || N <= 0 || dt_col < 0 || !state || !slots || !cu_seqlens || !y) return PYRE_ERR_BAD_ARG;
    if (N > 256) return PYRE_ERR_UNSUPPORTED;      // the staged tokens of a state that large would not fit 48 KB of shared memory either
    if (dtype == PYRE_BF16)
        return launch_ssm<__nv_bfloat16>(wide != 0, xbc, xbc_stride, proj, proj_stride, dt_col, dt_bias, A_log, D, state, slot_stride,
                                         slots, cu_seqlens, y, n_seqs, H, G, P, N, stream);
    if (dtype == PYRE_F32)
        return launch_ssm<float>(wide != 0, xbc, xbc_stride, proj, proj_stride, dt_col, dt_bias, A_log, D, state, slot_stride, slots,
                                 cu_seqlens, y, n_seqs, H, G, P, N, stream);
    return PYRE_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------
// A unit norm over each of `groups` equal parts of a row, with a gate:
//   gate_first:  v = y * act(gate);  out = v / sqrt(mean(v^2) + eps) * w * post
//   else:        v = y;              out = v / sqrt(mean(v^2) + eps) * w * post * act(gate)
// y fp32 [T, W]; the gate are W columns of `proj` from g_col (g_col < 0: none); act: 1 silu, 2 sigmoid; w fp32 [W] or
// null (no gain).  One block per (token, part); the block size depends on the part's size only.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void group_norm_gate_kernel(const float* y, const T* proj, long long proj_stride, int g_col, int act,
                                       int gate_first, const float* w, float post, T* out, int W, int gs, float eps) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y;
    const float* yr = y + (size_t)t * W + (size_t)part * gs;
    const T* gr = g_col >= 0 ? proj + (size_t)t * proj_stride + g_col + (size_t)part * gs : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float v = yr[i];
        if (gr && gate_first) {
            const float z = to_f32<T>(gr[i]);
            v = __fmul_rn(v, act == 1 ? sm_silu(z) : sm_sigmoid(z));
        }
        ss = fmaf(v, v, ss);
    }
    const float rstd = 1.0f / sqrtf(block_sum(ss, scratch) / (float)gs + eps);
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float v = yr[i];
        float gate = 1.f;
        if (gr) {
            const float z = to_f32<T>(gr[i]);
            gate = act == 1 ? sm_silu(z) : sm_sigmoid(z);
        }
        if (gr && gate_first) v = __fmul_rn(v, gate);
        float o = __fmul_rn(v, rstd);
        if (w) o = __fmul_rn(o, w[(size_t)part * gs + i]);
        if (post != 1.0f) o = __fmul_rn(o, post);
        if (gr && !gate_first) o = __fmul_rn(o, gate);
        out[(size_t)t * W + (size_t)part * gs + i] = from_f32<T>(o);
    }
}

PYRE_API int pyre_group_norm_gate(const float* y, const void* proj, long long proj_stride, int g_col, int act, int gate_first,
                                  const float* w, float post, void* out, int n_tokens, int W, int groups, float eps, int dtype,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (W <= 0 || groups <= 0 || W % groups || (g_col >= 0 && (!proj || (act != 1 && act != 2)))) return PYRE_ERR_BAD_ARG;
    const int gs = W / groups;
    const int threads = min(256, max(32, ((gs / 4 + 31) / 32) * 32));
    const dim3 grid(n_tokens, groups);
    if (dtype == PYRE_BF16)
        pyre_launch(group_norm_gate_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, y, (const __nv_bfloat16*)proj, proj_stride,
                    g_col, act, gate_first, w, post, (__nv_bfloat16*)out, W, gs, eps);
    else if (dtype == PYRE_F32)
        pyre_launch(group_norm_gate_kernel<float>, grid, dim3(threads), 0, stream, y, (const float*)proj, proj_stride, g_col, act,
                    gate_first, w, post, (float*)out, W, gs, eps);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Two softmax maps per head over the same values: o = a1 - lambda a2, then o / sqrt(mean(o^2) + eps) * post over the
// head's dv values.  `a` [T, 2 H, a_dim] holds the maps' sums grouped by key/value head: for head h = g rep + r
// (rep = H / G) map m lies at row (g * 2 + m) * rep + r; a row has a_dim >= dv columns of which the first dv count.
// out [T, H dv] in the heads' own order.  One warp per (token, head).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void diff_combine_kernel(const T* a, int a_dim, float lambda, float post, T* out, int n_tokens, int H, int rep,
                                    int dv, float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (size_t)n_tokens * H) return;
    const size_t t = item / H;
    const int h = (int)(item - t * H), g = h / rep, r = h - g * rep;
    const T* a1 = a + (t * 2 * H + (size_t)(g * 2) * rep + r) * a_dim;
    const T* a2 = a + (t * 2 * H + (size_t)(g * 2 + 1) * rep + r) * a_dim;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) {
        const float o = __fsub_rn(to_f32<T>(a1[i]), __fmul_rn(lambda, to_f32<T>(a2[i])));
        ss = fmaf(o, o, ss);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)dv + eps);
    for (int i = lane; i < dv; i += 32) {
        const float o = __fsub_rn(to_f32<T>(a1[i]), __fmul_rn(lambda, to_f32<T>(a2[i])));
        out[(t * H + h) * dv + i] = from_f32<T>(__fmul_rn(__fmul_rn(o, rstd), post));
    }
}

PYRE_API int pyre_diff_combine(const void* a, int a_dim, float lambda, float post, void* out, int n_tokens, int H, int G, int dv,
                               float eps, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dv <= 0 || a_dim < dv) return PYRE_ERR_BAD_ARG;
    const long long items = (long long)n_tokens * H;
    const int blocks = (int)ceil_div_ll(items, 4);
    if (dtype == PYRE_BF16)
        pyre_launch(diff_combine_kernel<__nv_bfloat16>, dim3(blocks), dim3(128), 0, stream, (const __nv_bfloat16*)a, a_dim, lambda, post,
                    (__nv_bfloat16*)out, n_tokens, H, H / G, dv, eps);
    else if (dtype == PYRE_F32)
        pyre_launch(diff_combine_kernel<float>, dim3(blocks), dim3(128), 0, stream, (const float*)a, a_dim, lambda, post, (float*)out,
                    n_tokens, H, H / G, dv, eps);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Rotation of heads that lie in a projection row, in place: `nh` heads of `dim` columns from column `col`; the pairs
// (i, i + rot / 2), i < rot / 2, turn by the token's angle (cos, sin [T, rot / 2]); every column is then multiplied
// by `factor`.  One thread per (token, head, i) with i < dim - rot / 2: a pair, or a column that only gets the factor.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rotate_heads_kernel(T* proj, long long row_stride, int col, const float* cos_t, const float* sin_t,
                                    int n_tokens, int nh, int dim, int rot, float factor) {
    pdl_trigger();
    pdl_wait();
    const int half = rot / 2, per_head = dim - half;
    const size_t total = (size_t)n_tokens * nh * per_head, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const size_t t = idx / ((size_t)nh * per_head);
        const int rem = (int)(idx - t * nh * per_head), h = rem / per_head, i = rem - h * per_head;
        T* head = proj + t * row_stride + col + (size_t)h * dim;
        if (i < half) {
            const float u = to_f32<T>(head[i]), v = to_f32<T>(head[i + half]);
            const float c = cos_t[t * half + i], s = sin_t[t * half + i];
            head[i] = from_f32<T>(__fmul_rn(__fsub_rn(__fmul_rn(u, c), __fmul_rn(v, s)), factor));
            head[i + half] = from_f32<T>(__fmul_rn(__fadd_rn(__fmul_rn(v, c), __fmul_rn(u, s)), factor));
        } else if (factor != 1.0f) {
            head[i + half] = from_f32<T>(__fmul_rn(to_f32<T>(head[i + half]), factor));
        }
    }
}

PYRE_API int pyre_rotate_heads(void* proj, long long row_stride, int col, const float* cos_t, const float* sin_t, int n_tokens,
                               int nh, int dim, int rot, float factor, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (nh <= 0 || dim <= 0 || rot < 0 || rot % 2 || rot > dim || col < 0 || (rot && (!cos_t || !sin_t))) return PYRE_ERR_BAD_ARG;
    const long long total = (long long)n_tokens * nh * (dim - rot / 2);
    const int blocks = (int)min((long long)pyre_sm_count() * 16, ceil_div_ll(total, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(rotate_heads_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)proj, row_stride, col, cos_t,
                    sin_t, n_tokens, nh, dim, rot, factor);
    else if (dtype == PYRE_F32)
        pyre_launch(rotate_heads_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)proj, row_stride, col, cos_t, sin_t, n_tokens,
                    nh, dim, rot, factor);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[t, j] = gelu_tanh(pre[t, j]) * table[token[t], col + j], j < dim: a token's slice of a side table, gated.
// A token id outside the table raises the error word (1) and reads row 0.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void side_gate_kernel(const T* pre, const T* table, long long table_stride, int col, const int* tokens, int vocab,
                                 T* out, int n_tokens, int dim, int* err) {
    pdl_trigger();
    pdl_wait();
    const size_t total = (size_t)n_tokens * dim, stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t t = i / dim;
        const int j = (int)(i - t * dim);
        int id = tokens[t];
        if (id < 0 || id >= vocab) {
            if (err) atomicExch(err, 1);
            id = 0;
        }
        const float e = to_f32<T>(table[(size_t)id * table_stride + col + j]);
        out[i] = from_f32<T>(__fmul_rn(sm_gelu_tanh(to_f32<T>(pre[i])), e));
    }
}

PYRE_API int pyre_side_gate(const void* pre, const void* table, long long table_stride, int col, const int* tokens, int vocab,
                            void* out, int n_tokens, int dim, int dtype, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || col < 0 || vocab <= 0 || col + dim > table_stride) return PYRE_ERR_BAD_ARG;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll((long long)n_tokens * dim, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(side_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)pre,
                    (const __nv_bfloat16*)table, table_stride, col, tokens, vocab, (__nv_bfloat16*)out, n_tokens, dim, err);
    else if (dtype == PYRE_F32)
        pyre_launch(side_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)pre, (const float*)table, table_stride,
                    col, tokens, vocab, (float*)out, n_tokens, dim, err);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// acc[t, :] += sigmoid(w . h[t, :]) * y[t, :]: a branch that every token takes, let in by ONE gate per token.
// acc fp32 [T, W]; h, y activations [T, K] / [T, W]; w fp32 [K].  One block per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void token_gate_add_kernel(float* acc, const T* h, const float* w, const T* y, int K, int W) {
    __shared__ float scratch[33];
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    float dot = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) dot = fmaf(to_f32<T>(h[(size_t)t * K + i]), w[i], dot);
    const float gate = sm_sigmoid(block_sum(dot, scratch));
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const size_t at = (size_t)t * W + i;
        acc[at] = fmaf(gate, to_f32<T>(y[at]), acc[at]);
    }
}

PYRE_API int pyre_token_gate_add(float* acc, const void* h, const float* w, const void* y, int n_tokens, int K, int W, int dtype,
                                 cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (K <= 0 || W <= 0 || !acc || !h || !w || !y) return PYRE_ERR_BAD_ARG;
    const int threads = min(256, max(32, ((K / 4 + 31) / 32) * 32));
    if (dtype == PYRE_BF16)
        pyre_launch(token_gate_add_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, acc, (const __nv_bfloat16*)h, w,
                    (const __nv_bfloat16*)y, K, W);
    else if (dtype == PYRE_F32)
        pyre_launch(token_gate_add_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, acc, (const float*)h, w, (const float*)y, K, W);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
