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
// Norms, rotation, gates and all sums are 32-bit; one block a token in the first kernel, tiles of 64 x 64 in the
// second: on the CUDA cores with sums over k in ascending order (the 32-bit path, and sizes the other form does not
// take), on the tensor cores for bfloat16 in whole 16-byte pieces.
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

// The same product on the tensor cores for bfloat16 operands in whole 16-byte pieces: a block takes 64 tokens x 64
// outputs of a head, each of its 4 warps 16 tokens; K passes through shared memory 64 at a time (padded rows, so
// that the eight rows of an ldmatrix fall on different banks); mma.sync.m16n8k16 with 32-bit sums; the gate and the
// rounding in the epilogue.
#define HT_BK 64
#define HT_ROW (HT_BK * 2 + 16)

__device__ __forceinline__ void ht_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ht_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
head_linear_tc_kernel(HeadLinearArgs g) {
    __shared__ __align__(16) unsigned char sA[64 * HT_ROW];
    __shared__ __align__(16) unsigned char sW[64 * HT_ROW];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int h = blockIdx.z;
    const __nv_bfloat16* X = (const __nv_bfloat16*)g.x + (size_t)h * g.x_head + g.x_off;
    const __nv_bfloat16* W = (const __nv_bfloat16*)g.w + (size_t)h * g.N * g.K;
    __nv_bfloat16* O = (__nv_bfloat16*)g.out + (size_t)h * g.o_head + g.o_off;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = lane >> 2, t = lane & 3;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    if (blockIdx.x == 0 && g.tail > 0) {
        const int half = g.tail / 2;
        if (g.cosv) {
            for (int e = tid; e < 64 * half; e += 128) {
                const int r = e / half, i = e - r * half, m = m0 + r;
                if (m >= g.T) break;
                const int i0 = g.interleaved ? 2 * i : i, i1 = g.interleaved ? 2 * i + 1 : i + half;
                const __nv_bfloat16* src = X + (size_t)m * g.x_row + g.K;
                const float c = g.cosv[(size_t)m * half + i], s = g.sinv[(size_t)m * half + i];
                const float u = gl_load(src + i0), x = gl_load(src + i1);
                gl_store(O + (size_t)m * g.o_row + g.N + i0, u * c - x * s);
                gl_store(O + (size_t)m * g.o_row + g.N + i1, x * c + u * s);
            }
        } else {
            for (int e = tid; e < 64 * g.tail; e += 128) {
                const int r = e / g.tail, i = e - r * g.tail, m = m0 + r;
                if (m >= g.T) break;
                O[(size_t)m * g.o_row + g.N + i] = X[(size_t)m * g.x_row + g.K + i];
            }
        }
    }
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
    const unsigned a_base = (unsigned)__cvta_generic_to_shared(sA), w_base = (unsigned)__cvta_generic_to_shared(sW);
    for (int k0 = 0; k0 < g.K; k0 += HT_BK) {
        const int kc = min(HT_BK, g.K - k0);
        for (int i = tid; i < 64 * 8; i += 128) {
            const int r = i >> 3, c = i & 7;
            uint4 va = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
            if (c * 8 < kc) {
                if (m0 + r < g.T) va = *(const uint4*)(X + (size_t)(m0 + r) * g.x_row + k0 + c * 8);
                if (n0 + r < g.N) vw = *(const uint4*)(W + (size_t)(n0 + r) * g.K + k0 + c * 8);
            }
            *(uint4*)(sA + r * HT_ROW + c * 16) = va;
            *(uint4*)(sW + r * HT_ROW + c * 16) = vw;
        }
        __syncthreads();
        for (int kk = 0; kk < kc / 16; ++kk) {
            unsigned af[4];
            ht_ldm4(a_base + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * HT_ROW + (kk * 2 + (lane >> 4)) * 16,
                    af[0], af[1], af[2], af[3]);
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                unsigned b0, b1, b2, b3;
                ht_ldm4(w_base + (j * 8 + ((lane >> 4) & 1) * 8 + (lane & 7)) * HT_ROW + (kk * 2 + ((lane >> 3) & 1)) * 16,
                        b0, b1, b2, b3);
                ht_mma(acc[j], af, b0, b1);
                ht_mma(acc[j + 1], af, b2, b3);
            }
        }
        __syncthreads();
    }
    const int r_lo = m0 + warp * 16 + grp, r_hi = r_lo + 8;
    float mul_lo = 1.0f, mul_hi = 1.0f;
    if (g.gate) {
        const __nv_bfloat16* G = (const __nv_bfloat16*)g.gate;
        if (r_lo < g.T) mul_lo = 1.0f / (1.0f + expf(-gl_load(G + (size_t)r_lo * g.g_row + g.g_off + h)));
        if (r_hi < g.T) mul_hi = 1.0f / (1.0f + expf(-gl_load(G + (size_t)r_hi * g.g_row + g.g_off + h)));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int n = n0 + j * 8 + 2 * t;
        if (n >= g.N) continue;
        if (r_lo < g.T)
            *(__nv_bfloat162*)(O + (size_t)r_lo * g.o_row + n) = __floats2bfloat162_rn(acc[j][0] * mul_lo, acc[j][1] * mul_lo);
        if (r_hi < g.T)
            *(__nv_bfloat162*)(O + (size_t)r_hi * g.o_row + n) = __floats2bfloat162_rn(acc[j][2] * mul_hi, acc[j][3] * mul_hi);
    }
}

GL_API int gl_head_linear(const HeadLinearArgs* args, int act_dtype, int w_dtype, cudaStream_t stream) {
    const HeadLinearArgs& g = *args;
    if (g.T <= 0 || g.H <= 0) return GL_OK;
    if (g.N <= 0 || g.K <= 0 || g.tail < 0 || (g.cosv && g.tail % 2) || g.H > 65535) return GL_ERR_SHAPE;
    const dim3 grid((g.N + HL_BN - 1) / HL_BN, (g.T + HL_BM - 1) / HL_BM, g.H);
    if (grid.y > 65535) return GL_ERR_SHAPE;
    int rc;
    if (act_dtype == GL_BF16 && w_dtype == GL_BF16 && g.K % 16 == 0 && g.N % 8 == 0 && g.x_row % 8 == 0 && g.x_head % 8 == 0 &&
        g.x_off % 8 == 0 && g.o_row % 2 == 0 && g.o_head % 2 == 0 && g.o_off % 2 == 0 &&
        !(((uintptr_t)g.x | (uintptr_t)g.w) & 15) && !((uintptr_t)g.out & 3))
        return gl_launch(head_linear_tc_kernel, grid, dim3(128), 0, stream, 1, g) == 0 ? GL_OK : GL_ERR_LAUNCH;
    if (act_dtype == GL_F32 && w_dtype == GL_F32) rc = gl_launch(head_linear_kernel<float, float>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_BF16 && w_dtype == GL_BF16)
        rc = gl_launch(head_linear_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_BF16 && w_dtype == GL_F32) rc = gl_launch(head_linear_kernel<__nv_bfloat16, float>, grid, dim3(256), 0, stream, 1, g);
    else if (act_dtype == GL_F32 && w_dtype == GL_BF16) rc = gl_launch(head_linear_kernel<float, __nv_bfloat16>, grid, dim3(256), 0, stream, 1, g);
    else return GL_ERR_DTYPE;
    return rc == 0 ? GL_OK : GL_ERR_LAUNCH;
}
