// A mixture of experts as a feed-forward: routing, the plan of a step's work, and the experts' products.
//
//   route     scores s = sigmoid(z) of a token's router logits; with groups, the experts form equal groups of
//             neighbours, a group's score is the sum of its two largest scores and only experts of the best
//             ``keep`` groups may be chosen; the ``top`` largest scores are chosen (the lower index wins a
//             tie); their weights are s / (sum of the chosen s + 1e-20) * scale.  All 32-bit.
//   plan      the step's assignments (token, choice) sorted by expert, and the list of row tiles: every
//             expert's rows cut into tiles of MOE_TM, so that a grid of fixed size (an upper bound of tiles)
//             covers whatever the router chose without the host learning of it.
//   gate_up   for every tile: rows gathered from the tokens' inputs, times the expert's gate and up weights,
//             silu(gate) * up written in sorted order.
//   down      for every tile: those rows times the expert's down weights, times the assignment's weight,
//             written 32-bit at the assignment's own place [token, choice].
//   combine   out[t] = sum over a token's choices (in the order of the choices) + what is to be added.
// With many rows an expert (prompts, bfloat16) the plan instead starts every expert's rows on a tile of 128 of
// their own; the rows are gathered into that order, and gate_up and down are each ONE product with grouped
// weights on the 5th-generation tensor cores (gemm_tcgen05.cu), with the gated activation between them.
//
// A row's result does not depend on which tile it falls in or what else the tile holds: every output
// element sums over k in ascending order (the 32-bit kernels) or in the tensor cores' fixed order (the
// bfloat16 kernels), so the order in which the plan happens to list an expert's rows changes nothing.
#include "common.cuh"

#define MOE_TM 32          // rows of a tile

// ---------------------------------------------------------------------------
// Routing: one warp a token.
// ---------------------------------------------------------------------------
struct RouteArgs {
    const float* logits;      // [T, E]
    int* ids;                 // [T, top]
    float* weights;           // [T, top]
    int T, E, top, groups, keep;
    float scale;
    const float* bias;        // [E] or null: added to the logits
    int softmax_chosen;       // 1: the largest LOGITS are chosen and weighted by the softmax over the chosen logits alone
                              // (times scale; one group); 0: sigmoid scores as above
};

// a token's score for expert e from its logit
__device__ __forceinline__ float moe_score(const RouteArgs& a, float z, int e) {
    if (a.bias) z += a.bias[e];
    return a.softmax_chosen ? z : 1.0f / (1.0f + expf(-z));
}

// the largest value among sc[e], e = first + lane, first + lane + 32, ... < last, and its (lowest) index
__device__ __forceinline__ void moe_argmax(const float* sc, int first, int last, int lane, float& best, int& at) {
    best = -INFINITY;
    at = 0x7fffffff;
    for (int e = first + lane; e < last; e += 32) {
        const float v = sc[e];
        if (v > best) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
}

__device__ __forceinline__ void moe_choose(const RouteArgs& a, float* sc, float* gsc, int t, int lane) {
    if (a.groups > 1 && a.keep < a.groups) {
        const int per = a.E / a.groups;
        for (int g = 0; g < a.groups; ++g) {
            float b1, b2 = 0.f;
            int i1, i2;
            moe_argmax(sc, g * per, (g + 1) * per, lane, b1, i1);
            if (per > 1) {
                const float keep1 = sc[i1];
                __syncwarp();
                if (lane == 0) sc[i1] = -INFINITY;
                __syncwarp();
                moe_argmax(sc, g * per, (g + 1) * per, lane, b2, i2);
                __syncwarp();
                if (lane == 0) sc[i1] = keep1;
                __syncwarp();
            }
            if (lane == 0) gsc[g] = b1 + b2;
        }
        __syncwarp();
        // the best groups stay; the others' experts drop out of the choice
        for (int k = 0; k < a.keep; ++k) {
            float b;
            int g;
            moe_argmax(gsc, 0, a.groups, lane, b, g);
            __syncwarp();
            if (lane == 0) gsc[g] = -INFINITY;             // marks a kept group
            __syncwarp();
        }
        for (int e = lane; e < a.E; e += 32)
            if (gsc[e / per] != -INFINITY) sc[e] = -1.0f;    // scores lie in (0, 1): -1 is never chosen before them
        __syncwarp();
    }
    if (a.softmax_chosen) {
        float first = 0.f, sum = 0.f;
        for (int k = 0; k < a.top; ++k) {
            float b;
            int e;
            moe_argmax(sc, 0, a.E, lane, b, e);
            if (k == 0) first = b;                           // the largest: the softmax is taken against it
            const float w = expf(b - first);
            sum += w;
            __syncwarp();
            if (lane == 0) {
                a.ids[(size_t)t * a.top + k] = e;
                a.weights[(size_t)t * a.top + k] = w;
                sc[e] = -INFINITY;
            }
            __syncwarp();
        }
        const float f = a.scale / sum;
        for (int k = lane; k < a.top; k += 32) a.weights[(size_t)t * a.top + k] *= f;
        return;
    }
    float sum = 0.f;
    for (int k = 0; k < a.top; ++k) {
        float b;
        int e;
        moe_argmax(sc, 0, a.E, lane, b, e);
        sum += b;
        __syncwarp();
        if (lane == 0) {
            a.ids[(size_t)t * a.top + k] = e;
            a.weights[(size_t)t * a.top + k] = b;
            sc[e] = -2.0f;
        }
        __syncwarp();
    }
    const float f = a.scale / (sum + 1e-20f);
    __syncwarp();
    for (int k = lane; k < a.top; k += 32) a.weights[(size_t)t * a.top + k] *= f;
}

__global__ void __launch_bounds__(128)
moe_route_kernel(RouteArgs a) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= a.T) return;
    float* sc = smem + (size_t)warp * (a.E + a.groups);      // [E] scores, then [groups] group scores
    float* gsc = sc + a.E;
    for (int e = lane; e < a.E; e += 32) sc[e] = moe_score(a, a.logits[(size_t)t * a.E + e], e);
    __syncwarp();
    moe_choose(a, sc, gsc, t, lane);
}

// The same with the router's product in front: a block a token.  Its four warps take the experts in turn,
// z_e = sum_k x[k] W[e, k] with the lanes striding over k and a butterfly sum, so a token's logits do not
// depend on what else is in the step; warp 0 then chooses as the kernel above does.
struct RouteFromArgs {
    const void* x;            // [T, K] activation type
    const float* w;           // [E, K] 32-bit
    int K;
    RouteArgs r;              // (logits unused)
};

template <typename TA>
__global__ void __launch_bounds__(128)
moe_route_from_kernel(RouteFromArgs f) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const RouteArgs& a = f.r;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    float* sc = smem;                        // [E] scores
    float* gsc = sc + a.E;                   // [groups] group scores
    float* xs = gsc + a.groups;              // [K] the token's input
    const TA* x = (const TA*)f.x + (size_t)t * f.K;
    for (int k = threadIdx.x; k < f.K; k += 128) xs[k] = gl_load(x + k);
    __syncthreads();
    for (int e = warp; e < a.E; e += 4) {
        const float* w = f.w + (size_t)e * f.K;
        float z = 0.f;
        for (int k = lane; k < f.K; k += 32) z = fmaf(xs[k], w[k], z);
        z = gl_warp_sum(z);
        if (lane == 0) sc[e] = moe_score(a, z, e);
    }
    __syncthreads();
    if (warp == 0) moe_choose(a, sc, gsc, t, lane);
}

GL_API int gl_moe_route_from(const RouteFromArgs* args, int x_dtype, cudaStream_t stream) {
    const RouteFromArgs& f = *args;
    const RouteArgs& a = f.r;
    if (a.T <= 0) return GL_OK;
    if (f.K <= 0 || a.E <= 0 || a.top <= 0 || a.top > a.E || a.groups <= 0 || a.E % a.groups || a.keep <= 0 || a.keep > a.groups) return GL_ERR_SHAPE;
    if ((long long)a.keep * (a.E / a.groups) < a.top || (a.softmax_chosen && a.groups != 1)) return GL_ERR_SHAPE;
    const size_t smem = (size_t)(a.E + a.groups + f.K) * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    int rc;
    if (x_dtype == GL_F32) rc = gl_launch(moe_route_from_kernel<float>, dim3(a.T), dim3(128), smem, stream, 1, f);
    else if (x_dtype == GL_BF16) rc = gl_launch(moe_route_from_kernel<__nv_bfloat16>, dim3(a.T), dim3(128), smem, stream, 1, f);
    else return GL_ERR_DTYPE;
    return rc == 0 ? GL_OK : GL_ERR_LAUNCH;
}

GL_API int gl_moe_route(const RouteArgs* args, cudaStream_t stream) {
    const RouteArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.E <= 0 || a.top <= 0 || a.top > a.E || a.groups <= 0 || a.E % a.groups || a.keep <= 0 || a.keep > a.groups) return GL_ERR_SHAPE;
    if ((long long)a.keep * (a.E / a.groups) < a.top || (a.softmax_chosen && a.groups != 1)) return GL_ERR_SHAPE;
    const size_t smem = 4 * (size_t)(a.E + a.groups) * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    return gl_launch(moe_route_kernel, dim3((a.T + 3) / 4), dim3(128), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// The plan: one block.
// ---------------------------------------------------------------------------
struct PlanArgs {
    const int* ids;           // [A] expert of every assignment (A = tokens * top)
    int* order;               // [A] assignments sorted by expert
    int* tile_expert;         // [max_tiles]
    int* tile_start;          // [max_tiles] first place in ``order``
    int* tile_rows;           // [max_tiles] rows of the tile (1..MOE_TM)
    int* n_tiles;             // [1]
    int A, E, max_tiles;
};

__global__ void __launch_bounds__(1024)
moe_plan_kernel(PlanArgs a) {
    extern __shared__ int ism[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    int* count = ism;                 // [E]
    int* start = count + a.E;         // [E] first place of the expert's rows, then the running cursor
    int* tile0 = start + a.E;         // [E] first tile of the expert
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < a.A; i += blockDim.x) {
        int e = a.ids[i];
        e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < a.E; ++e) {
            start[e] = at;
            tile0[e] = tiles;
            at += count[e];
            tiles += (count[e] + MOE_TM - 1) / MOE_TM;
        }
        *a.n_tiles = tiles < a.max_tiles ? tiles : a.max_tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
        const int n = (count[e] + MOE_TM - 1) / MOE_TM;
        for (int i = 0; i < n; ++i) {
            const int tile = tile0[e] + i;
            if (tile >= a.max_tiles) break;
            a.tile_expert[tile] = e;
            a.tile_start[tile] = start[e] + i * MOE_TM;
            a.tile_rows[tile] = min(MOE_TM, count[e] - i * MOE_TM);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.A; i += blockDim.x) {
        int e = a.ids[i];
        e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
        a.order[atomicAdd(&start[e], 1)] = i;
    }
}

GL_API int gl_moe_plan(const PlanArgs* args, cudaStream_t stream) {
    const PlanArgs& a = *args;
    if (a.A <= 0) return GL_OK;
    if (a.E <= 0 || a.max_tiles < (a.A + MOE_TM - 1) / MOE_TM + (a.E < a.A ? a.E : a.A)) return GL_ERR_SHAPE;
    const size_t smem = 3 * (size_t)a.E * sizeof(int);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    return gl_launch(moe_plan_kernel, dim3(1), dim3(1024), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// The plan for many rows an expert: every expert's rows start on a tile of ``tile_m`` rows of their own, so that
// the experts' products are ONE product with grouped weights (a tile of rows meets one expert's matrix).
// order[row] is the assignment at a padded row (-1: padding), place[assignment] its row, tile_expert[tile] the
// tile's expert (-1: not in use).
// ---------------------------------------------------------------------------
struct PadPlanArgs {
    const int* ids;           // [A]
    int* order;               // [max_tiles * tile_m]
    int* place;               // [A]
    int* tile_expert;         // [max_tiles]
    int A, E, max_tiles, tile_m;
};

__global__ void __launch_bounds__(1024)
moe_plan_padded_kernel(PadPlanArgs a) {
    extern __shared__ int ism[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    int* count = ism;                 // [E]
    int* start = count + a.E;         // [E] the expert's first row, then the running cursor
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) count[e] = 0;
    for (int i = threadIdx.x; i < a.max_tiles; i += blockDim.x) a.tile_expert[i] = -1;
    for (int i = threadIdx.x; i < a.max_tiles * a.tile_m; i += blockDim.x) a.order[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < a.A; i += blockDim.x) {
        int e = a.ids[i];
        e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
        atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tiles = 0;
        for (int e = 0; e < a.E; ++e) {
            start[e] = tiles * a.tile_m;
            const int n = (count[e] + a.tile_m - 1) / a.tile_m;
            for (int i = 0; i < n && tiles + i < a.max_tiles; ++i) a.tile_expert[tiles + i] = e;
            tiles += n;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.A; i += blockDim.x) {
        int e = a.ids[i];
        e = e < 0 ? 0 : (e >= a.E ? a.E - 1 : e);
        const int row = atomicAdd(&start[e], 1);
        if (row < a.max_tiles * a.tile_m) a.order[row] = i;
        a.place[i] = row;
    }
}

GL_API int gl_moe_plan_padded(const PadPlanArgs* args, cudaStream_t stream) {
    const PadPlanArgs& a = *args;
    if (a.A <= 0) return GL_OK;
    if (a.E <= 0 || a.tile_m <= 0 || a.max_tiles < (a.A + a.tile_m - 1) / a.tile_m + (a.E < a.A ? a.E : a.A)) return GL_ERR_SHAPE;
    const size_t smem = 2 * (size_t)a.E * sizeof(int);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    return gl_launch(moe_plan_padded_kernel, dim3(1), dim3(1024), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// rows of the padded, sorted input: xs[row] = x[order[row] / top], zeros where order[row] < 0; bfloat16, K % 8 == 0
__global__ void __launch_bounds__(128)
moe_gather_rows_kernel(const __nv_bfloat16* x, const int* order, __nv_bfloat16* xs, int K, int top) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int row = blockIdx.x;
    const int src = order[row];
    uint4* dst = (uint4*)(xs + (size_t)row * K);
    if (src < 0) {
        for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    const uint4* from = (const uint4*)(x + (size_t)(src / top) * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = from[i];
}

GL_API int gl_moe_gather_rows(const void* x, const int* order, void* xs, int rows, int K, int top, cudaStream_t stream) {
    if (rows <= 0) return GL_OK;
    if (K <= 0 || K % 8 || top <= 0) return GL_ERR_SHAPE;
    return gl_launch(moe_gather_rows_kernel, dim3(rows), dim3(128), 0, stream, 1, (const __nv_bfloat16*)x, order,
                     (__nv_bfloat16*)xs, K, top) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// out[t, :] = sum_k weights[t, k] * y[place[t, k], :] (+ add[t, :]), in the order of the choices
__global__ void __launch_bounds__(256)
moe_combine_placed_kernel(const float* y, const int* place, const float* weights, const float* add, float* out,
                          long long n, int N, int top) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / N;
    const int c = (int)(i - t * N);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += weights[t * top + k] * y[(size_t)place[t * top + k] * N + c];
    out[i] = add ? add[i] + s : s;
}

GL_API int gl_moe_combine_placed(const float* y, const int* place, const float* weights, const float* add, float* out,
                                 int T, int N, int top, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (N <= 0 || top <= 0) return GL_ERR_SHAPE;
    const long long n = (long long)T * N;
    return gl_launch(moe_combine_placed_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, y, place, weights,
                     add, out, n, N, top) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// The experts' products, 32-bit FMA on CUDA cores for any element type (the 32-bit path, and what the
// tensor-core kernels are checked against).  A block: one tile of rows x MOE_TN columns.
// ---------------------------------------------------------------------------
struct ExpertArgs {
    const void* x;            // gate_up: [T, K] the tokens' inputs;  down: [A, K] rows in sorted order
    const void* w;            // gate_up: [E, 2N, K] (gate rows, then up rows);  down: [E, N, K]
    void* out;                // gate_up: [A, N] activation type, sorted order;  down: [A, N] 32-bit, by assignment
    const int* order;         // [A]
    const int* tile_expert;
    const int* tile_start;
    const int* tile_rows;
    const int* n_tiles;
    const float* weights;     // [A] by assignment (down)
    int A, N, K, top, max_tiles;
    int E;                    // experts (to choose a kernel by the rows an expert meets on average)
};

#define MOE_TN 64
#define MOE_BK 32

template <typename TA, typename TW, bool GATED>
__global__ void __launch_bounds__(256)
moe_expert_simt_kernel(ExpertArgs a) {
    __shared__ float As[MOE_BK][MOE_TM + 1];
    __shared__ float W0[MOE_BK][MOE_TN + 1];
    __shared__ float W1[GATED ? MOE_BK : 1][MOE_TN + 1];
    __shared__ int rows[MOE_TM];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int tile = blockIdx.y;
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_expert[tile], start = a.tile_start[tile], nrows = a.tile_rows[tile];
    const int n0 = blockIdx.x * MOE_TN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    if (tid < MOE_TM) {
        // gate_up gathers a token's row; down reads the sorted rows themselves
        int r = -1;
        if (tid < nrows) r = GATED ? a.order[start + tid] / a.top : start + tid;
        rows[tid] = r;
    }
    __syncthreads();
    const TA* X = (const TA*)a.x;
    const TW* Wg = (const TW*)a.w + (size_t)e * (GATED ? 2 : 1) * a.N * a.K;
    const TW* Wu = Wg + (size_t)a.N * a.K;
    float acc0[2][4], acc1[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc0[i][j] = acc1[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += MOE_BK) {
#pragma unroll
        for (int i = 0; i < (MOE_TM * MOE_BK) / 256; ++i) {
            const int el = tid + i * 256, r = el / MOE_BK, c = el % MOE_BK;
            const int k = k0 + c, src = rows[r];
            As[c][r] = (src >= 0 && k < a.K) ? gl_load(X + (size_t)src * a.K + k) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < (MOE_TN * MOE_BK) / 256; ++i) {
            const int el = tid + i * 256, r = el / MOE_BK, c = el % MOE_BK;
            const int k = k0 + c, n = n0 + r;
            const bool ok = n < a.N && k < a.K;
            W0[c][r] = ok ? gl_load(Wg + (size_t)n * a.K + k) : 0.f;
            if (GATED) W1[c][r] = ok ? gl_load(Wu + (size_t)n * a.K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float av[2], w0[4], w1[4];
#pragma unroll
            for (int i = 0; i < 2; ++i) av[i] = As[kk][ty * 2 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                w0[j] = W0[kk][tx * 4 + j];
                if (GATED) w1[j] = W1[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc0[i][j] = fmaf(av[i], w0[j], acc0[i][j]);
                    if (GATED) acc1[i][j] = fmaf(av[i], w1[j], acc1[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = ty * 2 + i;
        if (r >= nrows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= a.N) continue;
            if (GATED) {
                const float g = acc0[i][j];
                gl_store((TA*)a.out + (size_t)(start + r) * a.N + n, g / (1.0f + expf(-g)) * acc1[i][j]);
            } else {
                const int asg = a.order[start + r];
                ((float*)a.out)[(size_t)asg * a.N + n] = acc0[i][j] * a.weights[asg];
            }
        }
    }
}

template <bool GATED>
static int launch_expert_simt(const ExpertArgs& a, int x_dtype, int w_dtype, cudaStream_t stream) {
    const dim3 grid((a.N + MOE_TN - 1) / MOE_TN, a.max_tiles);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    if (x_dtype == GL_F32 && w_dtype == GL_F32)
        return gl_launch(moe_expert_simt_kernel<float, float, GATED>, grid, dim3(256), 0, stream, 1, a);
    if (x_dtype == GL_BF16 && w_dtype == GL_BF16)
        return gl_launch(moe_expert_simt_kernel<__nv_bfloat16, __nv_bfloat16, GATED>, grid, dim3(256), 0, stream, 1, a);
    if (x_dtype == GL_F32 && w_dtype == GL_BF16)
        return gl_launch(moe_expert_simt_kernel<float, __nv_bfloat16, GATED>, grid, dim3(256), 0, stream, 1, a);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// The same products for bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulators).  A block of four
// warps takes one tile of 32 rows x 64 columns; warp w owns columns 16w..16w+15 for both 16-row halves.  The
// rows' inputs and the weights' k-slices go through shared memory (16-byte loads, rows padded by 16 bytes so
// that the fragments' 4-byte reads fall in distinct banks).
// ---------------------------------------------------------------------------
#define MT_BK 64
#define MT_PITCH (MT_BK + 8)

__device__ __forceinline__ void moe_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_expert_tc_kernel(ExpertArgs a) {
    __shared__ __align__(16) __nv_bfloat16 As[MOE_TM][MT_PITCH];
    __shared__ __align__(16) __nv_bfloat16 W0[MOE_TN][MT_PITCH];
    __shared__ __align__(16) __nv_bfloat16 W1[GATED ? MOE_TN : 1][MT_PITCH];
    __shared__ int rows[MOE_TM];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int tile = blockIdx.y;
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_expert[tile], start = a.tile_start[tile], nrows = a.tile_rows[tile];
    const int n0 = blockIdx.x * MOE_TN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = lane >> 2, tq = lane & 3;
    if (tid < MOE_TM) {
        int r = -1;
        if (tid < nrows) r = GATED ? a.order[start + tid] / a.top : start + tid;
        rows[tid] = r;
    }
    __syncthreads();
    const __nv_bfloat16* X = (const __nv_bfloat16*)a.x;
    const __nv_bfloat16* Wg = (const __nv_bfloat16*)a.w + (size_t)e * (GATED ? 2 : 1) * a.N * a.K;
    const __nv_bfloat16* Wu = Wg + (size_t)a.N * a.K;
    float acc0[2][2][4], acc1[2][2][4];      // [row half][8-column block][fragment]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int f = 0; f < 4; ++f) acc0[i][j][f] = acc1[i][j][f] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const int halves = nrows > 16 ? 2 : 1;
    for (int k0 = 0; k0 < a.K; k0 += MT_BK) {
        // K is a multiple of 8: a 16-byte piece lies wholly inside a row or wholly outside
        for (int el = tid; el < MOE_TM * (MT_BK / 8); el += 128) {
            const int r = el / (MT_BK / 8), c = (el % (MT_BK / 8)) * 8;
            const int src = rows[r];
            *(uint4*)&As[r][c] = (src >= 0 && k0 + c < a.K) ? *(const uint4*)(X + (size_t)src * a.K + k0 + c) : zero;
        }
        for (int el = tid; el < MOE_TN * (MT_BK / 8); el += 128) {
            const int r = el / (MT_BK / 8), c = (el % (MT_BK / 8)) * 8;
            const bool ok = n0 + r < a.N && k0 + c < a.K;
            *(uint4*)&W0[r][c] = ok ? *(const uint4*)(Wg + (size_t)(n0 + r) * a.K + k0 + c) : zero;
            if (GATED) *(uint4*)&W1[r][c] = ok ? *(const uint4*)(Wu + (size_t)(n0 + r) * a.K + k0 + c) : zero;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MT_BK; kk += 16) {
            unsigned bf0[2][2], bf1[2][2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int n = warp * 16 + j * 8 + grp;
                bf0[j][0] = *(const unsigned*)&W0[n][kk + 2 * tq];
                bf0[j][1] = *(const unsigned*)&W0[n][kk + 8 + 2 * tq];
                if (GATED) {
                    bf1[j][0] = *(const unsigned*)&W1[n][kk + 2 * tq];
                    bf1[j][1] = *(const unsigned*)&W1[n][kk + 8 + 2 * tq];
                }
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (i >= halves) break;
                unsigned af[4];
                af[0] = *(const unsigned*)&As[i * 16 + grp][kk + 2 * tq];
                af[1] = *(const unsigned*)&As[i * 16 + grp + 8][kk + 2 * tq];
                af[2] = *(const unsigned*)&As[i * 16 + grp][kk + 8 + 2 * tq];
                af[3] = *(const unsigned*)&As[i * 16 + grp + 8][kk + 8 + 2 * tq];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    moe_mma(acc0[i][j], af, bf0[j][0], bf0[j][1]);
                    if (GATED) moe_mma(acc1[i][j], af, bf1[j][0], bf1[j][1]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int f = 0; f < 4; ++f) {
                const int r = i * 16 + grp + (f >> 1) * 8;
                const int n = n0 + warp * 16 + j * 8 + 2 * tq + (f & 1);
                if (r >= nrows || n >= a.N) continue;
                if (GATED) {
                    const float g = acc0[i][j][f];
                    ((__nv_bfloat16*)a.out)[(size_t)(start + r) * a.N + n] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * acc1[i][j][f]);
                } else {
                    const int asg = a.order[start + r];
                    ((float*)a.out)[(size_t)asg * a.N + n] = acc0[i][j][f] * a.weights[asg];
                }
            }
}

// ---------------------------------------------------------------------------
// Few rows an expert (single tokens of a few sequences): the products are a stream of the chosen experts'
// weights, every weight row met by one to a few input rows.  A warp owns an output column: its lanes stride
// over k with 16-byte loads of the weight row (gate and up rows together), the tile's input rows wait in shared
// memory (eight at a time, 2,048 columns at a time), and a butterfly sum ends each row's dot product.  32-bit
// accumulation in a fixed order; bfloat16 operands, K a multiple of 8.
// ---------------------------------------------------------------------------
#define MV_ROWS 8
#define MV_KCH 2048
#define MV_COLS 8

template <bool GATED>
__global__ void __launch_bounds__(128)
moe_expert_rows_kernel(ExpertArgs a) {
    __shared__ __align__(16) __nv_bfloat16 xs[MV_ROWS][MV_KCH];
    __shared__ int rows[MOE_TM];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int tile = blockIdx.y;
    if (tile >= *a.n_tiles) return;
    const int e = a.tile_expert[tile], start = a.tile_start[tile], nrows = a.tile_rows[tile];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < MOE_TM) rows[tid] = tid < nrows ? (GATED ? a.order[start + tid] / a.top : start + tid) : -1;
    __syncthreads();
    const __nv_bfloat16* X = (const __nv_bfloat16*)a.x;
    const __nv_bfloat16* Wg = (const __nv_bfloat16*)a.w + (size_t)e * (GATED ? 2 : 1) * a.N * a.K;
    const __nv_bfloat16* Wu = Wg + (size_t)a.N * a.K;
    const int n_first = blockIdx.x * MV_COLS;
    for (int r0 = 0; r0 < nrows; r0 += MV_ROWS) {
        const int nr = min(MV_ROWS, nrows - r0);
        float accg[MV_COLS / 4][MV_ROWS], accu[MV_COLS / 4][MV_ROWS];
#pragma unroll
        for (int c = 0; c < MV_COLS / 4; ++c)
#pragma unroll
            for (int r = 0; r < MV_ROWS; ++r) accg[c][r] = accu[c][r] = 0.f;
        for (int k0 = 0; k0 < a.K; k0 += MV_KCH) {
            const int kn = min(MV_KCH, a.K - k0);
            __syncthreads();
            for (int el = tid; el < nr * (kn / 8); el += 128) {
                const int r = el / (kn / 8), c = (el - r * (kn / 8)) * 8;
                *(uint4*)&xs[r][c] = *(const uint4*)(X + (size_t)rows[r0 + r] * a.K + k0 + c);
            }
            __syncthreads();
#pragma unroll
            for (int c = 0; c < MV_COLS / 4; ++c) {
                const int n = n_first + warp + 4 * c;
                if (n >= a.N) continue;
                const __nv_bfloat16* wg = Wg + (size_t)n * a.K + k0;
                const __nv_bfloat16* wu = Wu + (size_t)n * a.K + k0;
#pragma unroll 2
                for (int k = lane * 8; k < kn; k += 256) {
                    const uint4 rg = *(const uint4*)(wg + k);
                    uint4 ru = make_uint4(0, 0, 0, 0);
                    if (GATED) ru = *(const uint4*)(wu + k);
                    const __nv_bfloat162* pg = (const __nv_bfloat162*)&rg;
                    const __nv_bfloat162* pu = (const __nv_bfloat162*)&ru;
                    float g[8], u[8];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 fg = __bfloat1622float2(pg[i]);
                        g[2 * i] = fg.x; g[2 * i + 1] = fg.y;
                        if (GATED) {
                            const float2 fu = __bfloat1622float2(pu[i]);
                            u[2 * i] = fu.x; u[2 * i + 1] = fu.y;
                        }
                    }
#pragma unroll
                    for (int r = 0; r < MV_ROWS; ++r) {
                        if (r >= nr) break;
                        const uint4 rx = *(const uint4*)&xs[r][k];
                        const __nv_bfloat162* px = (const __nv_bfloat162*)&rx;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 fx = __bfloat1622float2(px[i]);
                            accg[c][r] = fmaf(fx.x, g[2 * i], accg[c][r]);
                            accg[c][r] = fmaf(fx.y, g[2 * i + 1], accg[c][r]);
                            if (GATED) {
                                accu[c][r] = fmaf(fx.x, u[2 * i], accu[c][r]);
                                accu[c][r] = fmaf(fx.y, u[2 * i + 1], accu[c][r]);
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int c = 0; c < MV_COLS / 4; ++c) {
            const int n = n_first + warp + 4 * c;
#pragma unroll
            for (int r = 0; r < MV_ROWS; ++r) {
                if (r >= nr) break;
                const float g = gl_warp_sum(accg[c][r]);
                const float u = GATED ? gl_warp_sum(accu[c][r]) : 0.f;
                if (lane != 0 || n >= a.N) continue;
                if (GATED) {
                    ((__nv_bfloat16*)a.out)[(size_t)(start + r0 + r) * a.N + n] = __float2bfloat16_rn(g / (1.0f + __expf(-g)) * u);
                } else {
                    const int asg = a.order[start + r0 + r];
                    ((float*)a.out)[(size_t)asg * a.N + n] = g * a.weights[asg];
                }
            }
        }
    }
}

// how many assignments an expert meets on average before the tiles of rows go to the tensor cores
#define MV_MAX_ROWS_PER_EXPERT 4

template <bool GATED>
static int launch_expert(const ExpertArgs& a, int x_dtype, int w_dtype, cudaStream_t stream) {
    if (a.A <= 0 || a.max_tiles <= 0) return GL_OK;
    if (a.N <= 0 || a.K <= 0 || a.top <= 0) return GL_ERR_SHAPE;
    if (x_dtype == GL_BF16 && w_dtype == GL_BF16 && a.K % 8 == 0 && a.A <= MV_MAX_ROWS_PER_EXPERT * a.E) {
        const dim3 grid((a.N + MV_COLS - 1) / MV_COLS, a.max_tiles);
        if (grid.y > 65535) return GL_ERR_SHAPE;
        return gl_launch(moe_expert_rows_kernel<GATED>, grid, dim3(128), 0, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
    }
    if (x_dtype == GL_BF16 && w_dtype == GL_BF16 && a.K % 8 == 0) {
        const dim3 grid((a.N + MOE_TN - 1) / MOE_TN, a.max_tiles);
        if (grid.y > 65535) return GL_ERR_SHAPE;
        return gl_launch(moe_expert_tc_kernel<GATED>, grid, dim3(128), 0, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
    }
    return launch_expert_simt<GATED>(a, x_dtype, w_dtype, stream) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

GL_API int gl_moe_gate_up(const ExpertArgs* args, int x_dtype, int w_dtype, cudaStream_t stream) {
    return launch_expert<true>(*args, x_dtype, w_dtype, stream);
}

GL_API int gl_moe_down(const ExpertArgs* args, int x_dtype, int w_dtype, cudaStream_t stream) {
    return launch_expert<false>(*args, x_dtype, w_dtype, stream);
}

// the same two on the CUDA cores whatever the types (what the tensor-core kernels are checked against)
GL_API int gl_moe_gate_up_simt(const ExpertArgs* args, int x_dtype, int w_dtype, cudaStream_t stream) {
    if (args->A <= 0 || args->max_tiles <= 0) return GL_OK;
    return launch_expert_simt<true>(*args, x_dtype, w_dtype, stream) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

GL_API int gl_moe_down_simt(const ExpertArgs* args, int x_dtype, int w_dtype, cudaStream_t stream) {
    if (args->A <= 0 || args->max_tiles <= 0) return GL_OK;
    return launch_expert_simt<false>(*args, x_dtype, w_dtype, stream) == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// out[t, :] = sum_k y[t, k, :] (+ add[t, :]); out may be add itself.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* y, const float* add, float* out, long long n, int N, int top) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const long long t = i / N;
    const int c = (int)(i - t * N);
    float s = 0.f;
    for (int k = 0; k < top; ++k) s += y[((size_t)t * top + k) * N + c];
    out[i] = add ? add[i] + s : s;
}

GL_API int gl_moe_combine(const float* y, const float* add, float* out, int T, int N, int top, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (N <= 0 || top <= 0) return GL_ERR_SHAPE;
    const long long n = (long long)T * N;
    return gl_launch(moe_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, y, add, out, n, N, top) == 0
               ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// Routing without a router: a table [vocab, top] names every token id's experts, each with weight 1 / top.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_route_table_kernel(const int* tokens, const int* __restrict__ table, int* ids, float* weights, int n, int top, int vocab, int E) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int t = i / top, k = i - t * top;
    const int tok = gl_checked(tokens[t], vocab, GL_BAD_TOKEN);
    ids[i] = gl_checked(table[(size_t)tok * top + k], E, GL_BAD_ROW);
    weights[i] = 1.0f / (float)top;
}

GL_API int gl_moe_route_table(const int* tokens, const int* table, int* ids, float* weights, int T, int top, int vocab, int E,
                              cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (top <= 0 || vocab <= 0 || E <= 0) return GL_ERR_SHAPE;
    const int n = T * top;
    return gl_launch(moe_route_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 1, tokens, table, ids,
                     weights, n, top, vocab, E);
}
