// Products with one weight matrix per GROUP, and the small kernels of a routed feed-forward around them.
//
//   out[dst(p), g-th slice] = x[src(p), g-th slice] . w[g]^T        w[g] is [N, K] (a linear layer's layout)
//
// Two ways to say which rows belong to a group:
//   * every group takes all M rows (a product per HEAD: x and out hold the heads side by side in a row, each
//     group reads its own K columns and writes its own N columns);
//   * the rows are sorted by group, group g owning the sorted places offsets[g] .. offsets[g + 1] (a product per
//     EXPERT of a routed feed-forward: `src` gathers a place's input row, `dst` says where its result goes).
//
// One CTA computes a 64 x 64 tile of a group's result (128 x 128 for bfloat16 groups of many rows).  float32: FFMA, one chain per output element over k in
// ascending order, so a row's result does not depend on which other rows share its tile or its launch.
// bfloat16 operands: the same tiles on the tensor cores (mma.sync m16n8k16, fp32 accumulators).
// `dtype`: type of x and w (0 = float32, 1 = bfloat16); `out_f32`: the result stays fp32, else it is rounded to dtype.
#include "common.cuh"

struct GroupedArgs {
    const void* x;
    long long x_row_stride, x_group_stride;   // in elements
    const void* w;
    long long w_group_stride;                 // in elements; rows of w[g] are K apart
    void* out;
    long long out_row_stride, out_group_stride;
    const int* offsets;   // [G + 1] sorted places per group, or null: every group takes rows 0 .. M - 1
    const int* src;       // [places] input row of a sorted place, or null: the place itself
    const int* dst;       // [places] output row of a sorted place, or null: the place itself
    int M, N, K, G;
    int out_f32;
};

constexpr int GB_M = 64, GB_N = 64, GB_K = 16;

// Which (group, first place, places) a CTA works on; false: nothing to do.
template <int TILE_M = 64>
__device__ __forceinline__ bool grouped_tile(const GroupedArgs& a, int& g, int& first, int& count) {
    constexpr int GB_M = TILE_M;
    if (!a.offsets) {
        g = blockIdx.z;
        first = blockIdx.x * GB_M;
        count = min(GB_M, a.M - first);
        return count > 0;
    }
    __shared__ int found[3];
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, gg = 0;
        found[0] = -1;
        for (; gg < a.G; ++gg) {
            const int lo = a.offsets[gg], n = a.offsets[gg + 1] - lo;
            const int tiles = (n + GB_M - 1) / GB_M;
            if (tile < tiles) {
                found[0] = gg;
                found[1] = lo + tile * GB_M;
                found[2] = min(GB_M, n - tile * GB_M);
                break;
            }
            tile -= tiles;
        }
    }
    __syncthreads();
    g = found[0];
    first = found[1];
    count = found[2];
    return g >= 0;
}

template <typename T>
__global__ void __launch_bounds__(256) grouped_linear_kernel(GroupedArgs a) {
    __shared__ float xs[GB_K][GB_M + 4];
    __shared__ float ws[GB_K][GB_N + 4];
    __shared__ int src_row[GB_M], dst_row[GB_M];
    pdl_trigger();
    pdl_wait();
    int g, first, count;
    if (!grouped_tile(a, g, first, count)) return;
    const int n0 = blockIdx.y * GB_N;
    if (threadIdx.x < GB_M) {
        const int p = first + threadIdx.x;
        const bool live = (int)threadIdx.x < count;
        src_row[threadIdx.x] = live ? (a.src ? a.src[p] : p) : -1;
        dst_row[threadIdx.x] = live ? (a.dst ? a.dst[p] : p) : -1;
    }
    __syncthreads();
    const T* x = (const T*)a.x + (size_t)g * a.x_group_stride;
    const T* w = (const T*)a.w + (size_t)g * a.w_group_stride;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // loads: 64 rows x 16 k per operand = 1024 elements, four per thread: row = idx / 16, k = idx % 16
    for (int k0 = 0; k0 < a.K; k0 += GB_K) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = threadIdx.x + u * 256;
            const int r = idx >> 4, k = idx & 15;
            const int sr = src_row[r];
            xs[k][r] = (sr >= 0 && k0 + k < a.K) ? to_f32<T>(x[(size_t)sr * a.x_row_stride + k0 + k]) : 0.f;
            ws[k][r] = (n0 + r < a.N && k0 + k < a.K) ? to_f32<T>(w[(size_t)(n0 + r) * a.K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GB_K; ++k) {
            float xv[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) xv[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xv[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int dr = dst_row[ty * 4 + i];
        if (dr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            const size_t at = (size_t)dr * a.out_row_stride + (size_t)g * a.out_group_stride + n;
            if (a.out_f32) ((float*)a.out)[at] = acc[i][j];
            else ((T*)a.out)[at] = from_f32<T>(acc[i][j]);
        }
    }
}

// ---------------------------------------------------------------------------
// bfloat16 on the tensor cores: the same 64 x 64 tile, K in steps of 32 through shared memory, four warps of
// 32 x 32 each (2 x 4 MMAs of m16n8k16 per k-step of 16).  Needs K % 8 == 0 and 16-byte aligned rows of x and w.
// ---------------------------------------------------------------------------
constexpr int GT_K = 32, GT_LD = GT_K + 8;   // padded rows: 80 bytes, conflict-free for ldmatrix

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128) grouped_linear_mma_kernel(GroupedArgs a) {
    __shared__ __align__(16) __nv_bfloat16 xs[2][GB_M][GT_LD];
    __shared__ __align__(16) __nv_bfloat16 ws[2][GB_N][GT_LD];
    __shared__ int src_row[GB_M], dst_row[GB_M];
    pdl_trigger();
    pdl_wait();
    int g, first, count;
    if (!grouped_tile(a, g, first, count)) return;
    const int n0 = blockIdx.y * GB_N;
    if (threadIdx.x < GB_M) {
        const int p = first + threadIdx.x;
        const bool live = (int)threadIdx.x < count;
        src_row[threadIdx.x] = live ? (a.src ? a.src[p] : p) : -1;
        dst_row[threadIdx.x] = live ? (a.dst ? a.dst[p] : p) : -1;
    }
    __syncthreads();
    const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + (size_t)g * a.x_group_stride;
    const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)g * a.w_group_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    // a stage: 64 rows x 32 k of each operand = 256 vectors of 8 per operand, two per thread and operand
    auto load_stage = [&](int st, int k0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int idx = threadIdx.x + u * 128;
            const int r = idx >> 2, k = (idx & 3) * 8;
            const int sr = src_row[r];
            uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
            if (sr >= 0 && k0 + k < a.K) xv = *reinterpret_cast<const uint4*>(x + (size_t)sr * a.x_row_stride + k0 + k);
            if (n0 + r < a.N && k0 + k < a.K) wv = *reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * a.K + k0 + k);
            *reinterpret_cast<uint4*>(&xs[st][r][k]) = xv;
            *reinterpret_cast<uint4*>(&ws[st][r][k]) = wv;
        }
    };
    const int n_steps = (a.K + GT_K - 1) / GT_K;
    load_stage(0, 0);
    __syncthreads();
    for (int s = 0; s < n_steps; ++s) {
        const int st = s & 1;
        if (s + 1 < n_steps) load_stage(st ^ 1, (s + 1) * GT_K);
#pragma unroll
        for (int kk = 0; kk < GT_K; kk += 16) {
            uint32_t af[2][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(af[i], &xs[st][wm + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int j = 0; j < 2; ++j)   // 16 n-rows per ldmatrix: two 8-wide n tiles, both k halves
                ldmatrix_x4(bf[j], &ws[st][wn + j * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int dr = dst_row[wm + i * 16 + (lane >> 2) + half * 8];
            if (dr < 0) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn + j * 8 + (lane & 3) * 2 + e;
                    if (n >= a.N) continue;
                    const size_t at = (size_t)dr * a.out_row_stride + (size_t)g * a.out_group_stride + n;
                    const float v = acc[i][j][half * 2 + e];
                    if (a.out_f32) ((float*)a.out)[at] = v;
                    else ((__nv_bfloat16*)a.out)[at] = __float2bfloat16_rn(v);
                }
        }
}

// ---------------------------------------------------------------------------
// The same product for groups of many rows: 128 x 128 tiles, eight warps of 64 x 32 each (16 MMAs per four A and two B
// fragment loads), K in steps of 32 through two buffers filled by cp.async while the other is multiplied.
// ---------------------------------------------------------------------------
constexpr int GL_M = 128, GL_N = 128;

__global__ void __launch_bounds__(256) grouped_linear_mma_large_kernel(GroupedArgs a) {
    __shared__ __align__(16) __nv_bfloat16 xs[2][GL_M][GT_LD];
    __shared__ __align__(16) __nv_bfloat16 ws[2][GL_N][GT_LD];
    __shared__ int src_row[GL_M], dst_row[GL_M];
    pdl_trigger();
    pdl_wait();
    int g, first, count;
    if (!grouped_tile<GL_M>(a, g, first, count)) return;
    const int n0 = blockIdx.y * GL_N;
    if (threadIdx.x < GL_M) {
        const int p = first + threadIdx.x;
        const bool live = (int)threadIdx.x < count;
        src_row[threadIdx.x] = live ? (a.src ? a.src[p] : p) : -1;
        dst_row[threadIdx.x] = live ? (a.dst ? a.dst[p] : p) : -1;
    }
    __syncthreads();
    const __nv_bfloat16* x = (const __nv_bfloat16*)a.x + (size_t)g * a.x_group_stride;
    const __nv_bfloat16* w = (const __nv_bfloat16*)a.w + (size_t)g * a.w_group_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
    float acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    // a stage: 128 rows x 32 k of each operand = 512 pieces of 16 bytes per operand, two per thread and operand
    auto load_stage = [&](int st, int k0) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int idx = threadIdx.x + u * 256;
            const int r = idx >> 2, k = (idx & 3) * 8;
            const int sr = src_row[r];
            __nv_bfloat16* xd = &xs[st][r][k];
            __nv_bfloat16* wd = &ws[st][r][k];
            if (sr >= 0 && k0 + k < a.K) {
                const uint32_t d = (uint32_t)__cvta_generic_to_shared(xd);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(x + (size_t)sr * a.x_row_stride + k0 + k));
            } else {
                *reinterpret_cast<uint4*>(xd) = make_uint4(0, 0, 0, 0);
            }
            if (n0 + r < a.N && k0 + k < a.K) {
                const uint32_t d = (uint32_t)__cvta_generic_to_shared(wd);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(w + (size_t)(n0 + r) * a.K + k0 + k));
            } else {
                *reinterpret_cast<uint4*>(wd) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::);
    };
    const int n_steps = (a.K + GT_K - 1) / GT_K;
    load_stage(0, 0);
    for (int s = 0; s < n_steps; ++s) {
        const int st = s & 1;
        if (s + 1 < n_steps) {
            load_stage(st ^ 1, (s + 1) * GT_K);
            asm volatile("cp.async.wait_group 1;" ::);
        } else {
            asm volatile("cp.async.wait_group 0;" ::);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GT_K; kk += 16) {
            uint32_t af[4][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                ldmatrix_x4(af[i], &xs[st][wm + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
            for (int j = 0; j < 2; ++j)
                ldmatrix_x4(bf[j], &ws[st][wn + j * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
        }
        __syncthreads();      // the buffer is filled again two steps on
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int dr = dst_row[wm + i * 16 + (lane >> 2) + half * 8];
            if (dr < 0) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + (lane & 3) * 2;
                const size_t at = (size_t)dr * a.out_row_stride + (size_t)g * a.out_group_stride + n;
                const float v0 = acc[i][j][half * 2], v1 = acc[i][j][half * 2 + 1];
                if (a.out_f32) {
                    if (n < a.N) ((float*)a.out)[at] = v0;
                    if (n + 1 < a.N) ((float*)a.out)[at + 1] = v1;
                } else {
                    if (n < a.N) ((__nv_bfloat16*)a.out)[at] = __float2bfloat16_rn(v0);
                    if (n + 1 < a.N) ((__nv_bfloat16*)a.out)[at + 1] = __float2bfloat16_rn(v1);
                }
            }
        }
}

// places: an upper bound of the sorted places (the host does not know the groups' sizes); with offsets == null it is unused
PYRE_API int pyre_grouped_linear(const void* x, long long x_row_stride, long long x_group_stride, const void* w,
                                 long long w_group_stride, void* out, long long out_row_stride, long long out_group_stride,
                                 const int* offsets, const int* src, const int* dst, int M, int N, int K, int G, int places,
                                 int out_f32, int dtype, int use_mma, cudaStream_t stream) {
    if (N <= 0 || K <= 0 || G <= 0) return PYRE_ERR_BAD_ARG;
    GroupedArgs a{x, x_row_stride, x_group_stride, w, w_group_stride, out, out_row_stride, out_group_stride,
                  offsets, src, dst, M, N, K, G, out_f32};
    dim3 grid;
    if (offsets) {
        if (places <= 0) return 0;
        grid = dim3(ceil_div(places, GB_M) + G, ceil_div(N, GB_N), 1);
    } else {
        if (M <= 0) return 0;
        grid = dim3(ceil_div(M, GB_M), ceil_div(N, GB_N), G);
    }
    if (dtype == PYRE_BF16 && use_mma) {
        if (K % 8 || x_row_stride % 8 || x_group_stride % 8 || w_group_stride % 8 || (((uintptr_t)x | (uintptr_t)w) & 15))
            return PYRE_ERR_UNSUPPORTED;
        // groups of about a hundred rows or more (a prompt portion's heads or experts): the large tiles
        const long long rows_per_group = offsets ? (long long)places / G : M;
        if (rows_per_group >= 96) {
            const dim3 big = offsets ? dim3(ceil_div(places, GL_M) + G, ceil_div(N, GL_N), 1) : dim3(ceil_div(M, GL_M), ceil_div(N, GL_N), G);
            pyre_launch(grouped_linear_mma_large_kernel, big, dim3(256), 0, stream, a);
        } else {
            pyre_launch(grouped_linear_mma_kernel, grid, dim3(128), 0, stream, a);
        }
    } else if (dtype == PYRE_BF16) pyre_launch(grouped_linear_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, a);
    else if (dtype == PYRE_F32) pyre_launch(grouped_linear_kernel<float>, grid, dim3(256), 0, stream, a);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The router of a routed feed-forward.  Per token: logits z = W h over all `n_out` router outputs in fp32 (W fp32
// [n_out, H]; h in the activation dtype), scores s = softmax(z), choice scores s + correction; the `top` outputs
// with the largest choice scores are chosen (the lowest index wins a tie), and each chosen output's weight is its
// plain score s times `scale` (not renormalised).  `sigmoid` != 0: the scores are s = sigmoid(z), each output by itself,
// instead of the softmax.  `bias` (fp32 [n_out] or null) is added to the logits before anything else.  `renorm` != 0: the
// chosen outputs' weights are divided by their sum (with softmax scores: the softmax over the chosen logits alone).
// One block per token, one warp per output in turn.
//   idx_out [T, top] int32, weight_out [T, top] fp32
// ---------------------------------------------------------------------------
template <typename T>
__global__ void route_kernel(const T* h, const float* w, const float* correction, const float* bias, int* idx_out,
                             float* weight_out, int H, int n_out, int top, float scale, int sigmoid, int renorm) {
    extern __shared__ float z_smem[];   // [n_out] logits, then scores; [n_out] choice scores
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const T* hr = h + (size_t)t * H;
    float* z = z_smem;
    float* choice = z_smem + n_out;
    // which columns a lane adds depends on H and the pointers' alignment only, never on the batch
    const bool vec = H % 128 == 0 && (((uintptr_t)hr | (uintptr_t)w) & 15) == 0;
    for (int e = warp; e < n_out; e += warps) {
        const float* wr = w + (size_t)e * H;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (vec) {
            for (int i = lane * 4; i < H; i += 128) {
                const Vec<T, 4> hv = load_vec<T, 4>(hr + i);
                const Vec<float, 4> wv = load_vec<float, 4>(wr + i);
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[k] = fmaf(to_f32<T>(hv.v[k]), wv.v[k], acc[k]);
            }
        } else {
            for (int i = lane; i < H; i += 32) acc[0] = fmaf(to_f32<T>(hr[i]), wr[i], acc[0]);
        }
        const float sum = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
        if (lane == 0) z[e] = bias ? __fadd_rn(sum, bias[e]) : sum;
    }
    __syncthreads();
    if (warp == 0) {
        float sum = 1.f;
        if (sigmoid) {
            for (int e = lane; e < n_out; e += 32) z[e] = 1.0f / (1.0f + expf(-z[e]));
        } else {
            float mx = -INFINITY;
            for (int e = lane; e < n_out; e += 32) mx = fmaxf(mx, z[e]);
            mx = warp_max(mx);
            sum = 0.f;
            for (int e = lane; e < n_out; e += 32) {
                const float p = expf(z[e] - mx);
                z[e] = p;
                sum += p;
            }
            sum = warp_sum(sum);
        }
        __syncwarp();
        for (int e = lane; e < n_out; e += 32) {
            const float s = sigmoid ? z[e] : z[e] / sum;
            z[e] = s;
            choice[e] = s + (correction ? correction[e] : 0.f);
        }
        __syncwarp();
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int e = lane; e < n_out; e += 32) {
                const float c = choice[e];
                if (c > best) { best = c; at = e; }      // ascending e within a lane: the lowest index of equals stays
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (lane == 0) {
                idx_out[(size_t)t * top + k] = at;
                weight_out[(size_t)t * top + k] = z[at] * scale;
                choice[at] = -INFINITY;
            }
            __syncwarp();
        }
        if (renorm && lane == 0) {
            float total = 0.f;
            for (int k = 0; k < top; ++k) total += weight_out[(size_t)t * top + k];
            for (int k = 0; k < top; ++k) weight_out[(size_t)t * top + k] = weight_out[(size_t)t * top + k] / total;
        }
    }
}

PYRE_API int pyre_route(const void* h, const float* w, const float* correction, const float* bias, int* idx_out, float* weight_out,
                        int n_tokens, int H, int n_out, int top, float scale, int sigmoid, int renorm, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || n_out <= 0 || top <= 0 || top > n_out) return PYRE_ERR_BAD_ARG;
    const size_t smem = (size_t)2 * n_out * sizeof(float);
    if (smem > 48 * 1024) return PYRE_ERR_UNSUPPORTED;
    const int threads = n_tokens >= 512 ? 256 : 1024;      // few tokens: more warps per token's outputs
    if (dtype == PYRE_BF16)
        pyre_launch(route_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), smem, stream, (const __nv_bfloat16*)h, w, correction,
                    bias, idx_out, weight_out, H, n_out, top, scale, sigmoid, renorm);
    else if (dtype == PYRE_F32)
        pyre_launch(route_kernel<float>, dim3(n_tokens), dim3(threads), smem, stream, (const float*)h, w, correction, bias, idx_out,
                    weight_out, H, n_out, top, scale, sigmoid, renorm);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Sorting the (token, choice) pairs by expert.  idx [pairs] holds each pair's chosen output; outputs from
// `n_experts` on have no weights (their result is the input itself) and get no place.
//   offsets [n_experts + 1]   first sorted place of every expert
//   place_of [pairs]          the pair's sorted place, or -1
//   src [pairs]               for a sorted place, the token whose row it reads (pair / top)
// One block; the places inside an expert's range are handed out by atomic counters (any order: a place's result
// does not depend on its neighbours).
// ---------------------------------------------------------------------------
__global__ void group_pairs_kernel(const int* idx, int n_pairs, int top, int n_experts, int* offsets, int* place_of, int* src) {
    extern __shared__ int counts[];   // [n_experts] counts, then cursors
    pdl_trigger();
    pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        if (e >= 0 && e < n_experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = counts[e];
            offsets[e] = run;
            counts[e] = run;
            run += n;
        }
        offsets[n_experts] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = idx[p];
        int place = -1;
        if (e >= 0 && e < n_experts) {
            place = atomicAdd(&counts[e], 1);
            src[place] = p / top;
        }
        place_of[p] = place;
    }
}

PYRE_API int pyre_group_pairs(const int* idx, int n_pairs, int top, int n_experts, int* offsets, int* place_of, int* src,
                              cudaStream_t stream) {
    if (n_experts <= 0 || top <= 0) return PYRE_ERR_BAD_ARG;
    if ((size_t)n_experts * sizeof(int) > 48 * 1024) return PYRE_ERR_UNSUPPORTED;
    pyre_launch(group_pairs_kernel, dim3(1), dim3(1024), (size_t)n_experts * sizeof(int), stream, idx, n_pairs, top, n_experts,
                offsets, place_of, src);
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// out[t] = sum_k weight[t, k] * (y[place_of[t, k]]  or, for an output without weights,  h[t]), k ascending, fp32.
//   y [places, H] fp32 results of the experts' last product; h [T, H] the feed-forward's input
// ---------------------------------------------------------------------------
template <typename T>
__global__ void combine_pairs_kernel(const float* y, const T* h, const int* place_of, const float* weight, float* out,
                                     size_t total, int H, int top) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += stride) {
        const size_t t = at / H;
        const int i = (int)(at - t * H);
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int place = place_of[t * top + k];
            const float v = place >= 0 ? y[(size_t)place * H + i] : to_f32<T>(h[at]);
            acc = fmaf(weight[t * top + k], v, acc);
        }
        out[at] = acc;
    }
}

PYRE_API int pyre_combine_pairs(const float* y, const void* h, const int* place_of, const float* weight, float* out,
                                int n_tokens, int H, int top, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0) return 0;
    const size_t total = (size_t)n_tokens * H;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll((long long)total, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(combine_pairs_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, y, (const __nv_bfloat16*)h, place_of,
                    weight, out, total, H, top);
    else if (dtype == PYRE_F32)
        pyre_launch(combine_pairs_kernel<float>, dim3(blocks), dim3(256), 0, stream, y, (const float*)h, place_of, weight, out,
                    total, H, top);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// The experts' inputs of a routed feed-forward whose weights multiply what an expert READS:
//   out[place_of[t, k]] = T( weight[t, k] * h[t] )      for every pair with a place (place_of >= 0)
// out [places, H] in the order of the sorted places, so the products that follow read it without a gather.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void scale_to_places_kernel(const T* h, const int* place_of, const float* weight, T* out, size_t total, int H, int top) {
    pdl_trigger();
    pdl_wait();
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += stride) {
        const size_t pair = at / H;
        const int i = (int)(at - pair * H);
        const int place = place_of[pair];
        if (place >= 0) out[(size_t)place * H + i] = from_f32<T>(weight[pair] * to_f32<T>(h[(pair / top) * H + i]));
    }
}

PYRE_API int pyre_scale_to_places(const void* h, const int* place_of, const float* weight, void* out, int n_tokens, int H, int top,
                                  int dtype, cudaStream_t stream) {
    if (n_tokens <= 0 || H <= 0 || top <= 0) return 0;
    const size_t total = (size_t)n_tokens * top * H;
    const int blocks = (int)min((long long)pyre_sm_count() * 8, ceil_div_ll((long long)total, 256));
    if (dtype == PYRE_BF16)
        pyre_launch(scale_to_places_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (const __nv_bfloat16*)h, place_of, weight, (__nv_bfloat16*)out, total, H, top);
    else if (dtype == PYRE_F32)
        pyre_launch(scale_to_places_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)h, place_of, weight, (float*)out, total, H, top);
    else return PYRE_ERR_BAD_ARG;
    PYRE_LAUNCH_CHECK();
    return 0;
}
