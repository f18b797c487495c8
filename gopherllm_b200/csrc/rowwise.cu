// Row-wise kernels: embedding gather and normalisation.
//
// The residual stream is 32-bit in every mode; the norm writes the activation
// type of the mode (32-bit or bfloat16) that the matrix products read.
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding: out[t, :] = scale * table[tokens[t], :]          (model.go:2642-2651)
// ---------------------------------------------------------------------------
// (tokens, index, x below: what an earlier kernel of the step wrote is not declared restrict: loads through a
// const restrict pointer count as loads of memory nobody writes, which the compiler may move above the wait)
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* tokens,
                             float* __restrict__ out, int D, int V, float scale) {
    const int t = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    int tok = gl_checked(tokens[t], V, GL_BAD_TOKEN);
    // ids are checked on the host; a bad id must still not read outside the table
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    const TW* row = table + (size_t)tok * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] = gl_load(row + d) * scale;
}

GL_API int gl_embed(const void* table, int table_dtype, const int* tokens, float* out,
                    int T, int D, int V, float scale, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (D <= 0 || V <= 0) return GL_ERR_SHAPE;
    const int threads = D >= 1024 ? 256 : 128;
    if (table_dtype == GL_F32)
        return gl_launch(embed_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, (const float*)table, tokens, out, D, V, scale);
    if (table_dtype == GL_BF16)
        return gl_launch(embed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1,
                         (const __nv_bfloat16*)table, tokens, out, D, V, scale);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Embedding plus a hashed embedding of the pair (token before, token):
//   out[t, :] = scale * table[tok, :] + pair_table[(prev * mul_prev + tok * mul_cur) mod buckets, :],
// a sequence's first token (position 0) taking row ``buckets``, the table's last.  The token before a
// run's first token is the sequence's state: one int32 per slot (``last_token``, row pitch ``stride``),
// read by the block of the run's first token, which then stores the run's last token there.
// ---------------------------------------------------------------------------
struct EmbedPairArgs {
    const void* table;        // [V, D]
    const void* pair_table;   // [buckets + 1, D], same element type
    const int* tokens;        // [T]
    const int* tok_seq;       // [T]
    const int* tok_pos;       // [T]
    const int* seq_slot;      // [B]
    const int* seq_qstart;    // [B]
    const int* seq_qlen;      // [B]
    int* last_token;          // [slots, stride]
    float* out;               // [T, D]
    int T, D, V, buckets, stride;
    long long mul_prev, mul_cur;
    float scale;
};

template <typename TW>
__global__ void embed_pair_kernel(EmbedPairArgs a) {
    const int t = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    int tok = gl_checked(a.tokens[t], a.V, GL_BAD_TOKEN);
    tok = tok < 0 ? 0 : (tok >= a.V ? a.V - 1 : tok);
    const int b = a.tok_seq[t];
    const int qstart = a.seq_qstart[b];
    const bool first = t == qstart;
    int* state = a.last_token + (size_t)a.seq_slot[b] * a.stride;
    const int prev = first ? *state : a.tokens[t - 1];
    long long row = a.buckets;
    if (a.tok_pos[t] > 0) {
        row = ((long long)prev * a.mul_prev + (long long)tok * a.mul_cur) % a.buckets;
        if (row < 0) row += a.buckets;
    }
    const TW* e = (const TW*)a.table + (size_t)tok * a.D;
    const TW* p = (const TW*)a.pair_table + (size_t)row * a.D;
    float* o = a.out + (size_t)t * a.D;
    for (int d = threadIdx.x; d < a.D; d += blockDim.x) o[d] = fmaf(gl_load(e + d), a.scale, gl_load(p + d));
    if (first) {
        __syncthreads();                              // every thread has read the state
        if (threadIdx.x == 0) *state = a.tokens[qstart + a.seq_qlen[b] - 1];
    }
}

GL_API int gl_embed_pair(const EmbedPairArgs* args, int table_dtype, cudaStream_t stream) {
    const EmbedPairArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.D <= 0 || a.V <= 0 || a.buckets <= 0 || a.stride <= 0) return GL_ERR_SHAPE;
    const int threads = a.D >= 1024 ? 256 : 128;
    if (table_dtype == GL_F32) return gl_launch(embed_pair_kernel<float>, dim3(a.T), dim3(threads), 0, stream, 1, a);
    if (table_dtype == GL_BF16) return gl_launch(embed_pair_kernel<__nv_bfloat16>, dim3(a.T), dim3(threads), 0, stream, 1, a);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// A second table added onto the residual stream: out[t, :] += table[index[t], :].  Learned
// absolute positions are added once, before the first layer (model.go:2648-2651).
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void add_rows_kernel(const TW* __restrict__ table, const int* index,
                                float* __restrict__ out, int D, int N) {
    const int t = blockIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    int i = gl_checked(index[t], N, GL_BAD_ROW);
    i = i < 0 ? 0 : (i >= N ? N - 1 : i);        // checked on the host; never read outside the table
    const TW* row = table + (size_t)i * D;
    float* o = out + (size_t)t * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) o[d] += gl_load(row + d);
}

GL_API int gl_add_rows(const void* table, int table_dtype, const int* index, float* out,
                       int T, int D, int N, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (D <= 0 || N <= 0) return GL_ERR_SHAPE;
    const int threads = D >= 1024 ? 256 : 128;
    if (table_dtype == GL_F32)
        return gl_launch(add_rows_kernel<float>, dim3(T), dim3(threads), 0, stream, 1, (const float*)table, index, out, D, N);
    if (table_dtype == GL_BF16)
        return gl_launch(add_rows_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, 1,
                         (const __nv_bfloat16*)table, index, out, D, N);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Logits in place: x <- x * scale, then x <- cap * tanh(x / cap) if cap > 0 (the reference's
// LogitScale and final soft cap, model.go:2555-2564).  32-bit throughout.
// ---------------------------------------------------------------------------
__global__ void scale_softcap_kernel(float* __restrict__ x, size_t n, float scale, float cap) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

GL_API int gl_scale_softcap(float* x, long long n, float scale, float cap, cudaStream_t stream) {
    if (n <= 0) return GL_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want > 4096 ? 4096 : want);
    return gl_launch(scale_softcap_kernel, dim3(blocks), dim3(threads), 0, stream, 1, x, (size_t)n, scale, cap);
}

// ---------------------------------------------------------------------------
// Normalisation of selected rows of a 32-bit matrix.
//   layernorm: mean, biased variance over the row, y = (x-mean)*rsqrt(var+eps)*g + b
//              (bert.go:748-776; the reference takes 1/sqrt in 64-bit, so does this)
//   rmsnorm:   y = x * rsqrt(mean(x^2)+eps) * g            (model.go:2949-2981)
// rows == nullptr: row r of the output comes from row r of x; else from x[rows[r]].
// ---------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = gl_warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];   // same order in every thread
    return s;
}

// NV: values of the row each thread keeps in registers (the row is read once when it fits)
template <typename TO, int NV>
__global__ void norm_kernel(const float* x, const int* __restrict__ rows,
                            const float* __restrict__ gamma, const float* __restrict__ beta,
                            TO* __restrict__ out, int D, float eps, int rms) {
    __shared__ float red[32];
    __shared__ float s_inv;
    const int r = blockIdx.x;
    gl_grid_launch_dependents();
    // The norm's own vectors do not depend on the kernel before this one: they are asked for before this
    // kernel waits for it.  In a decode step they are cold (a layer's vectors are read once a step, with
    // gigabytes in between), and fetched at the end their trip to memory would stand between two products.
    float gv[NV > 0 ? NV : 1], bv[NV > 0 ? NV : 1];
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            gv[i] = d < D ? gamma[d] : 0.f;
            bv[i] = (d < D && beta) ? beta[d] : 0.f;
        }
    }
    gl_grid_wait();
    // (x is what the kernel before this one wrote: it is read with loads that the compiler may not move
    // above the wait.  Declared const and restrict, a pointer's loads count as loads of memory that nobody
    // writes, and those may be issued together with the loads above.)
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    TO* o = out + (size_t)r * D;
    float v[NV > 0 ? NV : 1];
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            v[i] = d < D ? __ldcg(xr + d) : 0.f;
        }
    }
    float mean = 0.f;
    if (!rms) {
        float s = 0.f;
        if (NV > 0) {
#pragma unroll
            for (int i = 0; i < NV; ++i) s += v[i];
        } else {
            for (int d = threadIdx.x; d < D; d += blockDim.x) s += __ldcg(xr + d);
        }
        mean = block_sum(s, red) / (float)D;
    }
    float q = 0.f;
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float c = (threadIdx.x + i * blockDim.x < D) ? v[i] - mean : 0.f;
            q += c * c;
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) { const float c = __ldcg(xr + d) - mean; q += c * c; }
    }
    const float var = block_sum(q, red) / (float)D;
    // one thread takes the reciprocal square root in 64-bit, as the reference does (bert.go:764)
    if (threadIdx.x == 0) s_inv = (float)(1.0 / sqrt((double)(var + eps)));
    __syncthreads();
    const float inv = s_inv;
    if (NV > 0) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int d = threadIdx.x + i * blockDim.x;
            if (d < D) gl_store(o + d, (v[i] - mean) * inv * gv[i] + bv[i]);
        }
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float y = (__ldcg(xr + d) - mean) * inv * gamma[d];
            if (beta) y += beta[d];
            gl_store(o + d, y);
        }
    }
}

// One warp per row, for many rows: the row lives in registers as NV4 float4 per lane, the
// statistics need warp shuffles only, loads and stores are 16 bytes (D a multiple of 4).
template <typename TO, int NV4>
__global__ void __launch_bounds__(256)
norm_warp_kernel(const float* x, const int* __restrict__ rows, const float* __restrict__ gamma,
                 const float* __restrict__ beta, TO* __restrict__ out, int R, int D, float eps, int rms) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    const float4* xr = (const float4*)(x + (size_t)(rows ? rows[r] : r) * D);
    const int n4 = D >> 2;
    float4 v[NV4];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int k = lane + 32 * i;
        v[i] = k < n4 ? xr[k] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
    const float mean = rms ? 0.f : gl_warp_sum(s) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        if (lane + 32 * i < n4) {
            const float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
            q += (a * a + b * b) + (c * c + d * d);
        }
    }
    const float var = gl_warp_sum(q) / (float)D;
    float inv = 0.f;
    if (lane == 0) inv = (float)(1.0 / sqrt((double)(var + eps)));
    inv = __shfl_sync(0xffffffffu, inv, 0);
    const float4* g4 = (const float4*)gamma;
    const float4* b4 = (const float4*)beta;
#pragma unroll
    for (int i = 0; i < NV4; ++i) {
        const int k = lane + 32 * i;
        if (k < n4) {
            const float4 g = g4[k];
            float4 y;
            y.x = (v[i].x - mean) * inv * g.x; y.y = (v[i].y - mean) * inv * g.y;
            y.z = (v[i].z - mean) * inv * g.z; y.w = (v[i].w - mean) * inv * g.w;
            if (beta) { const float4 b = b4[k]; y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w; }
            if constexpr (sizeof(TO) == 4) {
                ((float4*)(out + (size_t)r * D))[k] = y;
            } else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(y.x, y.y), p1 = __floats2bfloat162_rn(y.z, y.w);
                uint2 pk;
                pk.x = *(unsigned*)&p0; pk.y = *(unsigned*)&p1;
                ((uint2*)(out + (size_t)r * D))[k] = pk;
            }
        }
    }
}

template <typename TO, int NV4>
static int launch_norm_warp(const float* x, const int* rows, const float* gamma, const float* beta, TO* out,
                            int R, int D, float eps, int rms, cudaStream_t stream) {
    return gl_launch(norm_warp_kernel<TO, NV4>, dim3((R + 7) / 8), dim3(256), 0, stream, 1, x, rows, gamma, beta, out, R, D, eps, rms);
}

template <typename TO>
static int launch_norm(const float* x, const int* rows, const float* gamma, const float* beta, TO* out,
                       int R, int D, float eps, int rms, cudaStream_t stream) {
    const bool vec = D % 4 == 0 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)gamma | (uintptr_t)beta) & 15);
    // (the 32-bit path keeps one kernel for every row count, so that a row's result never depends
    // on how many rows come with it)
    if (sizeof(TO) == 2 && R >= 256 && vec && D <= 4096) {
        const int n = (D / 4 + 31) / 32;
        if (n <= 4) return launch_norm_warp<TO, 4>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 8) return launch_norm_warp<TO, 8>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 16) return launch_norm_warp<TO, 16>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        if (n <= 24) return launch_norm_warp<TO, 24>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
        return launch_norm_warp<TO, 32>(x, rows, gamma, beta, out, R, D, eps, rms, stream);
    }
    const int threads = D >= 2048 ? 512 : (D >= 512 ? 256 : 128);
    const int per = (D + threads - 1) / threads;
    if (per <= 2) return gl_launch(norm_kernel<TO, 2>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 4) return gl_launch(norm_kernel<TO, 4>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 8) return gl_launch(norm_kernel<TO, 8>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    if (per <= 16) return gl_launch(norm_kernel<TO, 16>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
    return gl_launch(norm_kernel<TO, 0>, dim3(R), dim3(threads), 0, stream, 1, x, rows, gamma, beta, out, D, eps, rms);
}

GL_API int gl_norm(const float* x, const int* rows, const float* gamma, const float* beta,
                   void* out, int out_dtype, int R, int D, float eps, int rms,
                   cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0) return GL_ERR_SHAPE;
    if (out_dtype == GL_F32) return launch_norm<float>(x, rows, gamma, beta, (float*)out, R, D, eps, rms, stream);
    if (out_dtype == GL_BF16) return launch_norm<__nv_bfloat16>(x, rows, gamma, beta, (__nv_bfloat16*)out, R, D, eps, rms, stream);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Feeding a decode step's choices back on the device: the sampled token becomes
// the next input, positions and cached lengths move on by one, and the choice is
// appended to a history so that several steps can run without the host.
// ---------------------------------------------------------------------------
__global__ void advance_kernel(int* tokens, int* tok_pos, int* seq_ctx, const int* sampled,
                               int* history, int* counter, int B, int max_steps) {
    const int b = threadIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int i = counter[0];
    if (b < B) {
        const int t = sampled[b];
        if (i < max_steps) history[(size_t)i * B + b] = t;
        tokens[b] = t;
        tok_pos[b] += 1;
        seq_ctx[b] += 1;
    }
    __syncthreads();
    if (b == 0) counter[0] = i + 1;
}

GL_API int gl_advance_decode(int* tokens, int* tok_pos, int* seq_ctx, const int* sampled,
                             int* history, int* counter, int B, int max_steps, cudaStream_t stream) {
    if (B <= 0) return GL_OK;
    if (B > 1024) return GL_ERR_SHAPE;
    return gl_launch(advance_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, stream, 1, tokens, tok_pos, seq_ctx, sampled,
                     history, counter, B, max_steps);
}

// ---------------------------------------------------------------------------
// Gated feed-forward, between its products: out[t, j] = act(gu[t, j]) * gu[t, F + j], where a row
// of gu holds the gate's F columns and then the up projection's.  32-bit arithmetic, one rounding.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
gated_act_kernel(const TA* gu, TA* __restrict__ out, long long n, int F, int act) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F;
        const int j = (int)(i - t * F);
        const TA* row = gu + (size_t)t * 2 * F;
        const float g = gl_load(row + j), u = gl_load(row + F + j);
        gl_store(out + i, gl_activate<true>(g, act) * u);
    }
}

// bfloat16 rows whose halves are whole 16-byte units: eight columns a thread, 16-byte loads and stores
__global__ void __launch_bounds__(256)
gated_act_bf16x8_kernel(const __nv_bfloat16* gu, __nv_bfloat16* __restrict__ out, long long n8, int F8, int act) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F8;
        const int j = (int)(i - t * F8);
        const uint4* row = (const uint4*)(gu + (size_t)t * 16 * F8);
        const uint4 g = row[j], u = row[F8 + j];
        const __nv_bfloat162* g2 = (const __nv_bfloat162*)&g;
        const __nv_bfloat162* u2 = (const __nv_bfloat162*)&u;
        uint4 o;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&o;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gf = __bfloat1622float2(g2[e]), uf = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(gl_activate<true>(gf.x, act) * uf.x, gl_activate<true>(gf.y, act) * uf.y);
        }
        ((uint4*)out)[i] = o;
    }
}

GL_API int gl_gated_act(const void* gu, void* out, int T, int F, int act, int act_dtype, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (F <= 0) return GL_ERR_SHAPE;
    const long long n = (long long)T * F;
    if (act_dtype == GL_BF16 && F % 8 == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15)) {
        const long long n8 = n / 8, want8 = (n8 + 255) / 256;
        return gl_launch(gated_act_bf16x8_kernel, dim3((unsigned)(want8 > 8192 ? 8192 : want8)), dim3(256), 0, stream, 1,
                         (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n8, F / 8, act);
    }
    const long long want = (n + 255) / 256;
    const dim3 grid((unsigned)(want > 8192 ? 8192 : want));
    if (act_dtype == GL_F32)
        return gl_launch(gated_act_kernel<float>, grid, dim3(256), 0, stream, 1, (const float*)gu, (float*)out, n, F, act);
    if (act_dtype == GL_BF16)
        return gl_launch(gated_act_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, (const __nv_bfloat16*)gu,
                         (__nv_bfloat16*)out, n, F, act);
    return GL_ERR_DTYPE;
}

// The same between the products of a gated feed-forward whose first product carries more columns: rows of ld
// columns, the gate's F from column 0 and the up projection's F behind them; with row_gate >= 0 column
// row_gate holds one more number a row, and the row's result is multiplied by its sigmoid (a feed-forward that is
// added with a learned share per token: the share is applied before the last product, which is linear).
template <typename TA>
__global__ void __launch_bounds__(256)
gated_act_rows_kernel(const TA* gu, TA* __restrict__ out, long long n, int F, int ld, int row_gate, int act) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F;
        const int j = (int)(i - t * F);
        const TA* row = gu + (size_t)t * ld;
        const float g = gl_load(row + j), u = gl_load(row + F + j);
        float y = gl_activate<true>(g, act) * u;
        if (row_gate >= 0) y *= 1.0f / (1.0f + expf(-gl_load(row + row_gate)));
        gl_store(out + i, y);
    }
}

// bfloat16 rows whose halves and whose length are whole 16-byte units: eight columns a thread
__global__ void __launch_bounds__(256)
gated_act_rows_bf16x8_kernel(const __nv_bfloat16* gu, __nv_bfloat16* __restrict__ out, long long n8, int F8, int ld, int row_gate, int act) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F8;
        const int j = (int)(i - t * F8);
        const __nv_bfloat16* rowp = gu + (size_t)t * ld;
        const uint4* row = (const uint4*)rowp;
        const uint4 g = row[j], u = row[F8 + j];
        const float share = row_gate >= 0 ? 1.0f / (1.0f + expf(-__bfloat162float(rowp[row_gate]))) : 1.0f;
        const __nv_bfloat162* g2 = (const __nv_bfloat162*)&g;
        const __nv_bfloat162* u2 = (const __nv_bfloat162*)&u;
        uint4 o;
        __nv_bfloat162* o2 = (__nv_bfloat162*)&o;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 gf = __bfloat1622float2(g2[e]), uf = __bfloat1622float2(u2[e]);
            o2[e] = __floats2bfloat162_rn(gl_activate<true>(gf.x, act) * uf.x * share, gl_activate<true>(gf.y, act) * uf.y * share);
        }
        ((uint4*)out)[i] = o;
    }
}

GL_API int gl_gated_act_rows(const void* gu, void* out, int T, int F, int ld, int row_gate, int act, int act_dtype,
                             cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (F <= 0 || ld < 2 * F || row_gate >= ld) return GL_ERR_SHAPE;
    const long long n = (long long)T * F;
    if (act_dtype == GL_BF16 && F % 8 == 0 && ld % 8 == 0 && !(((uintptr_t)gu | (uintptr_t)out) & 15)) {
        const long long n8 = n / 8, want8 = (n8 + 255) / 256;
        return gl_launch(gated_act_rows_bf16x8_kernel, dim3((unsigned)(want8 > 8192 ? 8192 : want8)), dim3(256), 0, stream, 1,
                         (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, n8, F / 8, ld, row_gate, act);
    }
    const long long want = (n + 255) / 256;
    const dim3 grid((unsigned)(want > 8192 ? 8192 : want));
    if (act_dtype == GL_F32)
        return gl_launch(gated_act_rows_kernel<float>, grid, dim3(256), 0, stream, 1, (const float*)gu, (float*)out, n, F, ld,
                         row_gate, act);
    if (act_dtype == GL_BF16)
        return gl_launch(gated_act_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, (const __nv_bfloat16*)gu,
                         (__nv_bfloat16*)out, n, F, ld, row_gate, act);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// An activation with two learned numbers, in place: above zero the parabola up * z^2 + z / 2, at and below zero
// down * (e^z - 1 - z) + z / 2 (the same slope on both sides of zero).  32-bit arithmetic, one rounding.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void __launch_bounds__(256)
xielu_kernel(TA* x, long long n, float up, float down) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float z = gl_load(x + i);
        const float y = z > 0.f ? fmaf(up * z, z, 0.5f * z) : fmaf(down, expm1f(z) - z, 0.5f * z);
        gl_store(x + i, y);
    }
}

// bfloat16 in whole 16-byte units: eight numbers a thread
__global__ void __launch_bounds__(256)
xielu_bf16x8_kernel(uint4* x, long long n8, float up, float down) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        uint4 raw = x[i];
        __nv_bfloat162* p2 = (__nv_bfloat162*)&raw;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 z = __bfloat1622float2(p2[e]);
            const float y0 = z.x > 0.f ? fmaf(up * z.x, z.x, 0.5f * z.x) : fmaf(down, expm1f(z.x) - z.x, 0.5f * z.x);
            const float y1 = z.y > 0.f ? fmaf(up * z.y, z.y, 0.5f * z.y) : fmaf(down, expm1f(z.y) - z.y, 0.5f * z.y);
            p2[e] = __floats2bfloat162_rn(y0, y1);
        }
        x[i] = raw;
    }
}

GL_API int gl_xielu(void* x, long long n, float up, float down, int act_dtype, cudaStream_t stream) {
    if (n <= 0) return GL_OK;
    if (act_dtype == GL_BF16 && n % 8 == 0 && !((uintptr_t)x & 15)) {
        const long long n8 = n / 8, want8 = (n8 + 255) / 256;
        return gl_launch(xielu_bf16x8_kernel, dim3((unsigned)(want8 > 16384 ? 16384 : want8)), dim3(256), 0, stream, 1, (uint4*)x, n8,
                         up, down);
    }
    const long long want = (n + 255) / 256;
    const dim3 grid((unsigned)(want > 8192 ? 8192 : want));
    if (act_dtype == GL_F32) return gl_launch(xielu_kernel<float>, grid, dim3(256), 0, stream, 1, (float*)x, n, up, down);
    if (act_dtype == GL_BF16) return gl_launch(xielu_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, 1, (__nv_bfloat16*)x, n, up, down);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Entering a pass of a looped range of layers: x[t, :] += base[t, :] + table[row, :]
// (base, the stream as it left the embedding, may be absent; table: one learned vector per pass).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
enter_pass_kernel(float* x, const float* base, const float* __restrict__ table, long long n, int D, int row) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (base) v += base[i];
        if (table) v += table[(size_t)row * D + (int)(i % D)];
        x[i] = v;
    }
}

GL_API int gl_enter_pass(float* x, const float* base, const float* table, int T, int D, int row, cudaStream_t stream) {
    if (T <= 0) return GL_OK;
    if (D <= 0 || row < 0) return GL_ERR_SHAPE;
    const long long n = (long long)T * D;
    const long long want = (n + 255) / 256;
    return gl_launch(enter_pass_kernel, dim3((unsigned)(want > 8192 ? 8192 : want)), dim3(256), 0, stream, 1, x, base, table, n, D, row);
}

// ---------------------------------------------------------------------------
// A branch's output normalised over the width and added: 
//   out[t, :] = alpha * a[t, :] / sqrt(mean(a[t, :]^2) + eps) * w [+ the same of a second branch a2, w2]
//               + add0[t, :] + add1[t, :] + add2[t, :]
// (32-bit rows; the adds may be absent; out may be one of them).  One block per row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rms_scale_add_kernel(const float* a, const float* __restrict__ w, const float* a2, const float* __restrict__ w2,
                     const float* add0, const float* add1, const float* add2,
                     float* out, int R, int D, float eps, float alpha) {
    __shared__ float red[16];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int r = blockIdx.x;
    const float* src = a + (size_t)r * D;
    const float* src2 = a2 ? a2 + (size_t)r * D : nullptr;
    float q = 0.f, q2 = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = src[d];
        q += v * v;
        if (src2) { const float u = src2[d]; q2 += u * u; }
    }
    q = gl_warp_sum(q);
    q2 = gl_warp_sum(q2);
    const int nw = blockDim.x >> 5;
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = q; red[8 + (threadIdx.x >> 5)] = q2; }
    __syncthreads();
    float tot = 0.f, tot2 = 0.f;
    for (int i = 0; i < nw; ++i) { tot += red[i]; tot2 += red[8 + i]; }      // same order in every thread
    const float inv = alpha / sqrtf(tot / (float)D + eps);
    const float inv2 = alpha / sqrtf(tot2 / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float y = src[d] * inv * w[d];
        if (src2) y += src2[d] * inv2 * w2[d];
        const size_t i = (size_t)r * D + d;
        if (add0) y += add0[i];
        if (add1) y += add1[i];
        if (add2) y += add2[i];
        out[i] = y;
    }
}

// a2, w2: a second branch normalised the same way and added (may be absent)
GL_API int gl_rms_scale_add(const float* a, const float* w, const float* a2, const float* w2,
                            const float* add0, const float* add1, const float* add2,
                            float* out, int R, int D, float eps, float alpha, cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0 || (a2 && !w2)) return GL_ERR_SHAPE;
    const int threads = D >= 2048 ? 256 : (D >= 512 ? 128 : 64);
    return gl_launch(rms_scale_add_kernel, dim3((unsigned)R), dim3(threads), 0, stream, 1, a, w, a2, w2, add0, add1, add2, out, R, D, eps, alpha);
}

// ---------------------------------------------------------------------------
// Two RMS norms of the same 32-bit rows (a layer whose branches each have a norm of their own): the row is
// read and its mean square taken once, out1 = x * inv * g1, out2 = x * inv * g2.  A warp a row for many
// rows, a block a row for few.
// ---------------------------------------------------------------------------
template <typename TO, int WARP_ROWS>
__global__ void __launch_bounds__(256)
rms_norm_pair_kernel(const float* x, const float* __restrict__ g1, const float* __restrict__ g2,
                     TO* __restrict__ out1, TO* __restrict__ out2, int R, int D, float eps) {
    __shared__ float red[8];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = WARP_ROWS ? blockIdx.x * (blockDim.x >> 5) + warp : blockIdx.x;
    if (WARP_ROWS && r >= R) return;
    const float* src = x + (size_t)r * D;
    const int first = WARP_ROWS ? lane : threadIdx.x, step = WARP_ROWS ? 32 : blockDim.x;
    float q = 0.f;
    for (int d = first; d < D; d += step) { const float v = src[d]; q += v * v; }
    q = gl_warp_sum(q);
    if (!WARP_ROWS) {
        if (lane == 0) red[warp] = q;
        __syncthreads();
        q = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) q += red[i];      // same order in every thread
    }
    // one thread of the row takes the reciprocal square root in 64-bit, as the single norm does
    float inv = 0.f;
    if (WARP_ROWS) {
        if (lane == 0) inv = (float)(1.0 / sqrt((double)(q / (float)D + eps)));
        inv = __shfl_sync(0xffffffffu, inv, 0);
    } else {
        __syncthreads();
        if (threadIdx.x == 0) red[0] = (float)(1.0 / sqrt((double)(q / (float)D + eps)));
        __syncthreads();
        inv = red[0];
    }
    for (int d = first; d < D; d += step) {
        const float v = src[d] * inv;
        gl_store(out1 + (size_t)r * D + d, v * g1[d]);
        gl_store(out2 + (size_t)r * D + d, v * g2[d]);
    }
}

GL_API int gl_rms_norm_pair(const float* x, const float* g1, const float* g2, void* out1, void* out2, int out_dtype,
                            int R, int D, float eps, cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0) return GL_ERR_SHAPE;
    if (R >= 64) {
        const dim3 grid((unsigned)((R + 7) / 8));
        if (out_dtype == GL_F32) return gl_launch(rms_norm_pair_kernel<float, 1>, grid, dim3(256), 0, stream, 1, x, g1, g2, (float*)out1, (float*)out2, R, D, eps);
        if (out_dtype == GL_BF16) return gl_launch(rms_norm_pair_kernel<__nv_bfloat16, 1>, grid, dim3(256), 0, stream, 1, x, g1, g2, (__nv_bfloat16*)out1, (__nv_bfloat16*)out2, R, D, eps);
        return GL_ERR_DTYPE;
    }
    const int threads = D >= 2048 ? 256 : (D >= 512 ? 128 : 64);
    if (out_dtype == GL_F32) return gl_launch(rms_norm_pair_kernel<float, 0>, dim3((unsigned)R), dim3(threads), 0, stream, 1, x, g1, g2, (float*)out1, (float*)out2, R, D, eps);
    if (out_dtype == GL_BF16) return gl_launch(rms_norm_pair_kernel<__nv_bfloat16, 0>, dim3((unsigned)R), dim3(threads), 0, stream, 1, x, g1, g2, (__nv_bfloat16*)out1, (__nv_bfloat16*)out2, R, D, eps);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// The 32-bit residual stream rounded to the activation type, for sublayers that read the stream itself
// (a layer that norms what a sublayer returns, not what it reads).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
round_rows_kernel(const float* x, __nv_bfloat16* __restrict__ out, long long n2) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n2; i += (long long)gridDim.x * blockDim.x) {
        const float2 v = ((const float2*)x)[i];
        ((__nv_bfloat162*)out)[i] = __floats2bfloat162_rn(v.x, v.y);
    }
}

GL_API int gl_round_rows(const float* x, void* out, long long n, cudaStream_t stream) {
    if (n <= 0) return GL_OK;
    if (n % 2 || (((uintptr_t)x) & 7) || (((uintptr_t)out) & 3)) return GL_ERR_ALIGN;
    const long long want = (n / 2 + 255) / 256;
    return gl_launch(round_rows_kernel, dim3((unsigned)(want > 8192 ? 8192 : want)), dim3(256), 0, stream, 1, x,
                     (__nv_bfloat16*)out, n / 2);
}

// ---------------------------------------------------------------------------
// A sublayer's output normed and added onto the stream it was computed from:
//   y = sa * a [+ sb * b];   out[t, :] = add[t, :] + y / sqrt(mean(y^2) + eps) * w
// (32-bit rows; b may be absent: two branches of a sublayer are summed with their scales before the norm;
// out may be add).  ``rounded``, if given, also receives out in bfloat16: the next sublayer's input.
// One block per row; the row stays in shared memory between the two passes.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
post_norm_add_kernel(const float* a, const float* b, const float* __restrict__ w, const float* add, float* out,
                     __nv_bfloat16* rounded, int D, float eps, float sa, float sb) {
    extern __shared__ float row[];
    __shared__ float red[8];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const size_t base = (size_t)blockIdx.x * D;
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float y = sa * a[base + d];
        if (b) y = fmaf(sb, b[base + d], y);
        row[d] = y;
        q = fmaf(y, y, q);
    }
    q = gl_warp_sum(q);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];          // same order in every thread
    const float inv = 1.0f / sqrtf(tot / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float y = add[base + d] + row[d] * inv * w[d];
        out[base + d] = y;
        if (rounded) rounded[base + d] = __float2bfloat16_rn(y);
    }
}

GL_API int gl_post_norm_add(const float* a, const float* b, const float* w, const float* add, float* out, void* rounded,
                            int R, int D, float eps, float sa, float sb, cudaStream_t stream) {
    if (R <= 0) return GL_OK;
    if (D <= 0 || !a || !w || !add || !out) return GL_ERR_SHAPE;
    const size_t smem = (size_t)D * sizeof(float);
    if (smem > 48 * 1024) return GL_ERR_SMEM;
    const int threads = D >= 2048 ? 256 : (D >= 512 ? 128 : 64);
    return gl_launch(post_norm_add_kernel, dim3((unsigned)R), dim3(threads), smem, stream, 1, a, b, w, add, out,
                     (__nv_bfloat16*)rounded, D, eps, sa, sb);
}

// ---------------------------------------------------------------------------
// out = sa * a + sb * b [+ add0] [+ add1], 32-bit: two branches summed with a factor each.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
scaled_sum_kernel(const float* a, const float* b, const float* add0, const float* add1, float* out, long long n, float sa, float sb) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float y = fmaf(sb, b[i], sa * a[i]);
        if (add0) y += add0[i];
        if (add1) y += add1[i];
        out[i] = y;
    }
}

GL_API int gl_scaled_sum(const float* a, const float* b, const float* add0, const float* add1, float* out, long long n,
                         float sa, float sb, cudaStream_t stream) {
    if (n <= 0) return GL_OK;
    const long long want = (n + 255) / 256;
    return gl_launch(scaled_sum_kernel, dim3((unsigned)(want > 8192 ? 8192 : want)), dim3(256), 0, stream, 1, a, b, add0, add1,
                     out, n, sa, sb);
}
