// Attention through a latent: what stands between the products of a mixer whose keys and values are read out of
// a small vector c per position.
//
// Such a mixer never has to build a position's keys and values.  With k_h(j) = U_h c(j) and v_h(j) = V_h c(j),
//     q_h . k_h(j) = (U_h^T q_h) . c(j),        sum_j p(j) v_h(j) = V_h (sum_j p(j) c(j)),
// so the cache holds one row [c | shared rotated key part] per position, every head's query becomes a row
// [U_h^T q_h | its rotated part] of the same length, attention runs as many query heads on one key head whose
// values are the row's first columns, and V_h is applied to a head's result afterwards.
//
//   gl_latent_prepare   a token's down projections [query latent | c | rotated key part | ...]: both latents
//                       RMS-normed with a weight, the key part rotated; the query latent written out, the row
//                       [c | key part] written to the token's place in the cache (the values are its first columns;
//                       a cache that keeps values of its own gets c once more).
//   gl_head_linear      out[t, h, :] = W_h x[t, h, :] per head (strided rows on both sides), optionally followed by
//                       a rotated copy of the columns behind x[t, h, :K] (the query's rotated part) and optionally
//                       times sigmoid(gate[t, h]) (an output gate per head).
// Norms, rotation, gates and all sums are 32-bit; one block a token in the first kernel, tiles of 64 x 64 with sums
// over k in ascending order in the second.
#include "common.cuh"

struct LatentPrepareArgs {
    const void* proj;         // [T, ld] activation type: query latent (q_rank), c (kv_rank), key part (rot), then others
    void* cq_out;             // [T, q_rank] activation type: the normed query latent
    void* k_cache;            // [pages, 1, GL_PAGE, kv_rank + rot] cache type
    void* v_cache;            // [pages, 1, GL_PAGE, kv_rank] cache type, or null: the values are read from the key rows
    const float* cosv;        // [T, rot / 2] or null
    const float* sinv;
    const float* q_gamma;     // [q_rank]
    const float* kv_gamma;    // [kv_rank]
    const int* tok_seq;
    const int* tok_pos;
    const int* pages;         // [B, max_pages]
    int T, ld, q_rank, kv_rank, rot, max_pages, n_pages, interleaved, write_kv;
    float eps;
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(LatentPrepareArgs a) {
    extern __shared__ float smem[];
    __shared__ float red[2][8];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int t = blockIdx.x;
    const int n = a.q_rank + a.kv_rank + a.rot;
    const TA* row = (const TA*)a.proj + (size_t)t * a.ld;
    float* v = smem;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = gl_load(row + i);
        v[i] = x;
        if (i < a.q_rank) sq = fmaf(x, x, sq);
        else if (i < a.q_rank + a.kv_rank) sk = fmaf(x, x, sk);
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    sq = gl_warp_sum(sq);
    sk = gl_warp_sum(sk);
    if (lane == 0) { red[0][w] = sq; red[1][w] = sk; }
    __syncthreads();
    float tq = 0.f, tk = 0.f;
    for (int i = 0; i < nw; ++i) { tq += red[0][i]; tk += red[1][i]; }       // the same order in every thread
    const float inv_q = a.q_rank > 0 ? 1.0f / sqrtf(tq / (float)a.q_rank + a.eps) : 0.f;
    const float inv_k = 1.0f / sqrtf(tk / (float)a.kv_rank + a.eps);
    TA* cq = (TA*)a.cq_out + (size_t)t * a.q_rank;
    for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) gl_store(cq + i, v[i] * inv_q * a.q_gamma[i]);
    if (!a.write_kv) return;
    const int pos = a.tok_pos[t];
    const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
    const int page = gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
    const int wide = a.kv_rank + a.rot;
    TC* kr = (TC*)a.k_cache + ((size_t)page * GL_PAGE + (pos % GL_PAGE)) * wide;
    TC* vr = (TC*)a.v_cache + ((size_t)page * GL_PAGE + (pos % GL_PAGE)) * a.kv_rank;
    const float* c = v + a.q_rank;
    for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) {
        const float y = c[i] * inv_k * a.kv_gamma[i];
        gl_store(kr + i, y);
        if (a.v_cache) gl_store(vr + i, y);
    }
    const float* kp = c + a.kv_rank;
    const int half = a.rot / 2;
    if (a.cosv) {
        const float* cs = a.cosv + (size_t)t * half;
        const float* sn = a.sinv + (size_t)t * half;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int i0 = a.interleaved ? 2 * i : i, i1 = a.interleaved ? 2 * i + 1 : i + half;
            const float u = kp[i0], x = kp[i1];
            gl_store(kr + a.kv_rank + i0, u * cs[i] - x * sn[i]);
            gl_store(kr + a.kv_rank + i1, x * cs[i] + u * sn[i]);
        }
    } else {
        for (int i = threadIdx.x; i < a.rot; i += blockDim.x) gl_store(kr + a.kv_rank + i, kp[i]);
    }
}

GL_API int gl_latent_prepare(const LatentPrepareArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const LatentPrepareArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.q_rank < 0 || a.kv_rank <= 0 || a.rot < 0 || a.rot % 2 || a.ld < a.q_rank + a.kv_rank + a.rot) return GL_ERR_SHAPE;
    const size_t smem = (size_t)(a.q_rank + a.kv_rank + a.rot) * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    if (act_dtype != cache_dtype) return GL_ERR_DTYPE;
    const dim3 g((unsigned)a.T), b(256);
    int rc;
    if (act_dtype == GL_F32) rc = gl_launch(latent_prepare_kernel<float, float>, g, b, smem, stream, 1, a);
    else if (act_dtype == GL_BF16) rc = gl_launch(latent_prepare_kernel<__nv_bfloat16, __nv_bfloat16>, g, b, smem, stream, 1, a);
    else return GL_ERR_DTYPE;
    return rc == 0 ? GL_OK : GL_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// A product per head.
// ---------------------------------------------------------------------------
struct HeadLinearArgs {
    const void* x;            // activation type; head h of token t starts at x[t * x_row + h * x_head + x_off]
    const void* w;            // [H, N, K] weight type
    void* out;                // activation type; head h of token t starts at out[t * o_row + h * o_head + o_off]
    const void* gate;         // activation type or null: gate[t * g_row + g_off + h], the result times its sigmoid
    const float* cosv;        // [T, tail / 2] or null
    const float* sinv;
    int T, H, N, K;
    int x_row, x_head, x_off, o_row, o_head, o_off, g_row, g_off;
    int tail;                 // columns behind the K of x that are copied behind the N of out, rotated by the
                              // token's angles when cosv is given (tail even then)
    int interleaved;          // the rotation pairs column 2i with 2i+1 (else i with i + tail/2)
};

#define HL_BM 64
#define HL_BN 64
#define HL_BK 16

template <typename TA, typename TW>
__global__ void __launch_bounds__(256)
head_linear_kernel(HeadLinearArgs g) {
    __shared__ float As[HL_BK][HL_BM + 4];
    __shared__ float Ws[HL_BK][HL_BN + 4];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int h = blockIdx.z;
    const TA* X = (const TA*)g.x + (size_t)h * g.x_head + g.x_off;
    const TW* W = (const TW*)g.w + (size_t)h * g.N * g.K;
    TA* O = (TA*)g.out + (size_t)h * g.o_head + g.o_off;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN;
    if (blockIdx.x == 0 && g.tail > 0) {
        // the columns behind the product's input go behind its output, rotated
        const int half = g.tail / 2;
        if (g.cosv) {
            for (int e = tid; e < HL_BM * half; e += 256) {
                const int r = e / half, i = e - r * half, m = m0 + r;
                if (m >= g.T) break;
                const int i0 = g.interleaved ? 2 * i : i, i1 = g.interleaved ? 2 * i + 1 : i + half;
                const TA* src = X + (size_t)m * g.x_row + g.K;
                const float c = g.cosv[(size_t)m * half + i], s = g.sinv[(size_t)m * half + i];
                const float u = gl_load(src + i0), x = gl_load(src + i1);
                gl_store(O + (size_t)m * g.o_row + g.N + i0, u * c - x * s);
                gl_store(O + (size_t)m * g.o_row + g.N + i1, x * c + u * s);
            }
        } else {
            for (int e = tid; e < HL_BM * g.tail; e += 256) {
                const int r = e / g.tail, i = e - r * g.tail, m = m0 + r;
                if (m >= g.T) break;
                gl_store(O + (size_t)m * g.o_row + g.N + i, gl_load(X + (size_t)m * g.x_row + g.K + i));
            }
        }
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < g.K; k0 += HL_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256, r = e >> 4, c = e & 15;
            const int k = k0 + c;
            float va = 0.f, vw = 0.f;
            if (k < g.K) {
                if (m0 + r < g.T) va = gl_load(X + (size_t)(m0 + r) * g.x_row + k);
                if (n0 + r < g.N) vw = gl_load(W + (size_t)(n0 + r) * g.K + k);
            }
            As[c][r] = va;
            Ws[c][r] = vw;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HL_BK; ++kk) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= g.T) continue;
        float mul = 1.0f;
        if (g.gate) mul = 1.0f / (1.0f + expf(-gl_load((const TA*)g.gate + (size_t)m * g.g_row + g.g_off + h)));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < g.N) gl_store(O + (size_t)m * g.o_row + n, acc[i][j] * mul);
        }
    }
}

GL_API int gl_head_linear(const HeadLinearArgs* args, int act_dtype, int w_dtype, cudaStream_t stream) {
    const HeadLinearArgs& g = *args;
    if (g.T <= 0 || g.H <= 0) return GL_OK;
    if (g.N <= 0 || g.K <= 0 || g.tail < 0 || (g.cosv && g.tail % 2) || g.H > 65535) return GL_ERR_SHAPE;
    const dim3 grid((g.N + HL_BN - 1) / HL_BN, (g.T + HL_BM - 1) / HL_BM, g.H);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    int rc;
    if (act_dtype == GL_F32 && w_dtype == GL_F32) rc = gl_launch(head_linear_kernel<float, float>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_BF16 && w_dtype == GL_BF16)
        rc = gl_launch(head_linear_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_BF16 && w_dtype == GL_F32) rc = gl_launch(head_linear_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_F32 && w_dtype == GL_BF16) rc = gl_launch(head_linear_kernel<float, __nv_bfloat16>, grid, dim3(256), 0, stream, 1, g);
    else return GL_ERR_DTYPE;
    return rc == 0 ? GL_OK : GL_ERR_LAUNCH;
}
