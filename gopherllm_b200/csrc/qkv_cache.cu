// What happens between the QKV product and attention, in one pass over the
// projected rows: optional per-head norm of q and k, rotary position encoding,
// the query scale, and the write of k and v into the paged cache.
//
// Order as in the reference: bias (already in the product's epilogue), head
// norm, rotation, then the query scale (model.go:2677-2706, forward_batch.go:446-469);
// keys are cached rotated and unscaled (model.go:1466-1487).
#include "common.cuh"

// cos/sin of angle float(pos) * inv_freq[i]; the product is taken in 32-bit and
// the functions in 64-bit, as the reference does (model.go:3041-3046).
__global__ void rope_table_kernel(const int* pos, const float* __restrict__ inv_freq,
                                  float* __restrict__ cosv, float* __restrict__ sinv, int T, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    if (i >= T * half) return;
    const int t = i / half, p = i % half;
    const float a = (float)pos[t] * inv_freq[p];
    double s, c;
    sincos((double)a, &s, &c);
    cosv[i] = (float)c;
    sinv[i] = (float)s;
}

GL_API int gl_rope_table(const int* pos, const float* inv_freq, float* cosv, float* sinv,
                         int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return GL_OK;
    const int n = T * half;
    return gl_launch(rope_table_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, pos, inv_freq, cosv, sinv, T, half);
}

// The same tables from 64-bit frequencies: the angle pos * freq is a 64-bit product, so a table entry is
// the correctly rounded cosine of the exact angle whatever the position.
__global__ void rope_table64_kernel(const int* pos, const double* __restrict__ freq,
                                    float* __restrict__ cosv, float* __restrict__ sinv, int T, int half) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    gl_grid_launch_dependents();
    gl_grid_wait();
    if (i >= T * half) return;
    const int t = i / half, p = i % half;
    double s, c;
    sincos((double)pos[t] * freq[p], &s, &c);
    cosv[i] = (float)c;
    sinv[i] = (float)s;
}

GL_API int gl_rope_table64(const int* pos, const double* freq, float* cosv, float* sinv,
                           int T, int half, cudaStream_t stream) {
    if (T <= 0 || half <= 0) return GL_OK;
    const int n = T * half;
    return gl_launch(rope_table64_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, 1, pos, freq, cosv, sinv, T, half);
}

struct QkvCacheArgs {
    const void* qkv;          // [T, (nH + 2 nKV) * hd], activation type
    void* q_out;              // [T, nH * hd], activation type
    void* k_cache;            // this cache entry's keys   [pages, nKV, GL_PAGE, hd], cache type
    void* v_cache;            // this cache entry's values
    const float* cosv;        // [T, half] or null
    const float* sinv;
    const float* q_gamma;     // [hd] or null: per-head norm of q
    const float* q_beta;      // [hd] or null
    const float* k_gamma;
    const float* k_beta;
    const int* tok_seq;       // [T] sequence of each token
    const int* tok_pos;       // [T] absolute position of each token
    const int* pages;         // [B, max_pages] page ids of each sequence
    int T, nH, nKV, hd, half, max_pages;
    int interleaved, norm_rms, write_kv;
    float eps, q_scale;
    int n_pages;              // pages of the cache entry (read by builds that check indices; 0: unknown)
};

template <typename TA, typename TC>
__global__ void qkv_cache_kernel(QkvCacheArgs a) {
    extern __shared__ float smem[];
    gl_grid_launch_dependents();
    gl_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = a.nH + 2 * a.nKV;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long long)a.T * heads) return;
    const int t = (int)(item / heads), j = (int)(item % heads);
    const int kind = j < a.nH ? 0 : (j < a.nH + a.nKV ? 1 : 2);   // q, k, v
    if (kind != 0 && !a.write_kv) return;
    const int hd = a.hd;
    float* v = smem + warp * hd;
    const TA* src = (const TA*)a.qkv + (size_t)t * heads * hd + (size_t)j * hd;
    for (int d = lane; d < hd; d += 32) v[d] = gl_load(src + d);
    __syncwarp();

    const float* gamma = kind == 0 ? a.q_gamma : a.k_gamma;
    const float* beta = kind == 0 ? a.q_beta : a.k_beta;
    if (kind != 2 && gamma) {
        float mean = 0.f;
        if (!a.norm_rms) {
            float s = 0.f;
            for (int d = lane; d < hd; d += 32) s += v[d];
            mean = gl_warp_sum(s) / (float)hd;
        }
        float q = 0.f;
        for (int d = lane; d < hd; d += 32) { const float c = v[d] - mean; q += c * c; }
        const float var = gl_warp_sum(q) / (float)hd;
        const float inv = (float)(1.0 / sqrt((double)(var + a.eps)));
        for (int d = lane; d < hd; d += 32) {
            float y = (v[d] - mean) * inv * gamma[d];
            if (beta) y += beta[d];
            v[d] = y;
        }
        __syncwarp();
    }
    if (kind != 2 && a.half > 0 && a.cosv) {
        const float* cs = a.cosv + (size_t)t * a.half;
        const float* sn = a.sinv + (size_t)t * a.half;
        for (int i = lane; i < a.half; i += 32) {
            const int i0 = a.interleaved ? 2 * i : i;
            const int i1 = a.interleaved ? 2 * i + 1 : i + a.half;
            const float c = cs[i], s = sn[i];
            const float u = v[i0], w = v[i1];
            v[i0] = u * c - w * s;
            v[i1] = u * s + w * c;
        }
        __syncwarp();
    }
    if (kind == 0) {
        TA* dst = (TA*)a.q_out + (size_t)t * a.nH * hd + (size_t)j * hd;
        for (int d = lane; d < hd; d += 32) gl_store(dst + d, v[d] * a.q_scale);
    } else {
        const int head = kind == 1 ? j - a.nH : j - a.nH - a.nKV;
        const int pos = a.tok_pos[t];
        const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
        const int page = gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
        TC* base = (TC*)(kind == 1 ? a.k_cache : a.v_cache);
        TC* dst = base + (((size_t)page * a.nKV + head) * GL_PAGE + (pos % GL_PAGE)) * hd;
        for (int d = lane; d < hd; d += 32) gl_store(dst + d, v[d]);
    }
}

// The same for bfloat16 rows and cache without a head norm, one 16-byte chunk (8 dims) of a head at a
// time: the chunk and, inside the rotary part, its partner chunk are loaded with 16-byte loads and the
// result leaves with one 16-byte store.  One block per token, its threads over the token's chunks: what
// depends on the token alone (position, page, angle rows) is looked up once, and a chunk's place costs
// one 32-bit division (a flat index over all tokens cost three 64-bit ones a chunk and made the kernel
// instruction-bound).  Needs the head size and the rotary half to be multiples of 8 and split-half pairing.
__global__ void __launch_bounds__(256)
qkv_cache_bf16_kernel(QkvCacheArgs a) {
    gl_grid_launch_dependents();
    gl_grid_wait();
    const unsigned chunks = a.hd >> 3, heads = a.nH + 2 * a.nKV;
    const unsigned hc = a.half >> 3;                          // chunks in one half of the rotary part
    const int t = blockIdx.x;
    const unsigned n = (a.write_kv ? heads : (unsigned)a.nH) * chunks;
    const __nv_bfloat16* row = (const __nv_bfloat16*)a.qkv + (size_t)t * heads * a.hd;
    const float* cs_row = a.cosv ? a.cosv + (size_t)t * a.half : nullptr;
    const float* sn_row = a.sinv ? a.sinv + (size_t)t * a.half : nullptr;
    const int pos = a.tok_pos[t];
    const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
    const size_t cache_row = a.write_kv
        ? ((size_t)gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE)
           * a.nKV * GL_PAGE + (pos % GL_PAGE)) * a.hd : 0;
    for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
        const unsigned j = i / chunks, c = i - j * chunks;
        const int kind = j < (unsigned)a.nH ? 0 : (j < (unsigned)(a.nH + a.nKV) ? 1 : 2);
        const __nv_bfloat16* src = row + (size_t)j * a.hd;
        const uint4 raw = *(const uint4*)(src + c * 8);
        float v[8];
        {
            const __nv_bfloat162* p2 = (const __nv_bfloat162*)&raw;
#pragma unroll
            for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(p2[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
        }
        if (kind != 2 && cs_row && c < 2 * hc) {
            const bool low = c < hc;                             // this chunk holds u (first half) or w (second half)
            const uint4 praw = *(const uint4*)(src + (low ? c + hc : c - hc) * 8);
            const __nv_bfloat162* q2 = (const __nv_bfloat162*)&praw;
            const float* cs = cs_row + (low ? c : c - hc) * 8;
            const float* sn = sn_row + (low ? c : c - hc) * 8;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(q2[e]);
                const float pw[2] = {f.x, f.y};
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float co = cs[2 * e + k], si = sn[2 * e + k];
                    // u' = u cos - w sin ;  w' = u sin + w cos
                    v[2 * e + k] = low ? v[2 * e + k] * co - pw[k] * si : pw[k] * si + v[2 * e + k] * co;
                }
            }
        }
        const float sc = kind == 0 ? a.q_scale : 1.0f;
        uint4 out;
        {
            __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0] * sc, v[1] * sc), p1 = __floats2bfloat162_rn(v[2] * sc, v[3] * sc);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4] * sc, v[5] * sc), p3 = __floats2bfloat162_rn(v[6] * sc, v[7] * sc);
            out.x = *(unsigned*)&p0; out.y = *(unsigned*)&p1; out.z = *(unsigned*)&p2; out.w = *(unsigned*)&p3;
        }
        if (kind == 0) {
            *(uint4*)((__nv_bfloat16*)a.q_out + ((size_t)t * a.nH + j) * a.hd + c * 8) = out;
        } else {
            const unsigned head = kind == 1 ? j - a.nH : j - a.nH - a.nKV;
            __nv_bfloat16* base = (__nv_bfloat16*)(kind == 1 ? a.k_cache : a.v_cache);
            *(uint4*)(base + cache_row + (size_t)head * GL_PAGE * a.hd + c * 8) = out;
        }
    }
}

GL_API int gl_qkv_cache(const QkvCacheArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const QkvCacheArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.hd <= 0 || a.nH <= 0 || a.nKV <= 0 || 2 * a.half > a.hd) return GL_ERR_SHAPE;
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16 && !a.q_gamma && !a.k_gamma && !a.interleaved &&
        a.hd % 8 == 0 && a.half % 8 == 0 &&
        !(((uintptr_t)a.qkv | (uintptr_t)a.q_out | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache) & 15)) {
        return gl_launch(qkv_cache_bf16_kernel, dim3((unsigned)a.T), dim3(256), 0, stream, 1, a);
    }
    const int warps = 4;
    const long long items = (long long)a.T * (a.nH + 2 * a.nKV);
    const unsigned blocks = (unsigned)((items + warps - 1) / warps);
    const size_t smem = (size_t)warps * a.hd * sizeof(float);
    const dim3 g(blocks), b(warps * 32);
    if (act_dtype == GL_F32 && cache_dtype == GL_F32) return gl_launch(qkv_cache_kernel<float, float>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_BF16 && cache_dtype == GL_BF16)
        return gl_launch(qkv_cache_kernel<__nv_bfloat16, __nv_bfloat16>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_BF16 && cache_dtype == GL_F32) return gl_launch(qkv_cache_kernel<__nv_bfloat16, float>, g, b, smem, stream, 1, a);
    if (act_dtype == GL_F32 && cache_dtype == GL_BF16) return gl_launch(qkv_cache_kernel<float, __nv_bfloat16>, g, b, smem, stream, 1, a);
    return GL_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// The same step for a mixer that normalises queries and keys over the WHOLE projection (all heads of a
// token at once, root mean square, one weight per column) before the rotation, and whose values may
// have another size than its keys:
//   q <- q / sqrt(mean(q^2) + eps) * gq over nH*hd columns, k likewise over nKV*hd; rotation of the
//   first 2*half dims of every head; q * q_scale to q_out; k and v into the token's cache row.
// A query temperature that grows with the position may scale q as well:
//   q * (1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1))        (temp_every > 0)
// and a mixer that reads the keys and values another one wrote brings queries alone (q_only).  With head_unit
// every head of q and k is brought to unit root mean square after the rotation (no weight).
// One block per token; statistics, rotation and scale in 32-bit.
// ---------------------------------------------------------------------------
struct QkvRowNormArgs {
    const void* qkv;          // [T, ld] activation type: q (nH*hd), k (nKV*hd), v (nKV*vd) from column 0 on
    void* q_out;              // [T, nH*hd] activation type
    void* k_cache;            // [pages, nKV, GL_PAGE, hd] cache type
    void* v_cache;            // [pages, nKV, GL_PAGE, vd] cache type
    const float* cosv;        // [T, half] or null
    const float* sinv;
    const float* q_gamma;     // [nH*hd] or null (no norm)
    const float* k_gamma;     // [nKV*hd] or null
    const int* tok_seq;
    const int* tok_pos;
    const int* pages;         // [B, max_pages]
    int T, ld, nH, nKV, hd, vd, half, max_pages, interleaved, write_kv;
    float eps, q_scale;
    int n_pages;
    float temp_coef, temp_every;   // query temperature (temp_every <= 0: none)
    int q_only;                    // the rows hold queries alone; nothing is written to the cache
    int head_unit;                 // after the rotation every head of q and k is divided by its own root mean square
                                   // over hd (eps inside the root, no weight)
    const float* talk;             // [nH, nH] or null: a table that mixes the heads' SCORES before the softmax,
                                   // s'_h = sum_g talk[h, g] (q_g . k_c(g)).  The sum is taken on the queries: q_out
                                   // is then [T, nH, nKV*hd], head h holding, for every key head c, the sum of
                                   // talk[h, g] q_g over the query heads g of c, so that s'_h is ONE product of
                                   // that row with the position's key heads side by side
    int k_joined;                  // the key cache holds a position's heads side by side as one row:
                                   // [pages, 1, GL_PAGE, nKV*hd]
};

template <typename TA, typename TC>
__global__ void __launch_bounds__(512)
qkv_rownorm_cache_kernel(QkvRowNormArgs a) {
    extern __shared__ float smem[];
    __shared__ float red[16];
    gl_grid_launch_dependents();
    // the table that mixes the heads' scores is a weight: it comes into shared memory while the kernel before drains
    float* talk = smem + (size_t)(a.nH + a.nKV) * a.hd;
    if (a.talk)
        for (int i = threadIdx.x; i < a.nH * a.nH; i += blockDim.x) talk[i] = a.talk[i];
    gl_grid_wait();
    const int t = blockIdx.x;
    const int nq = a.nH * a.hd, nk = a.q_only ? 0 : a.nKV * a.hd, nv = a.q_only ? 0 : a.nKV * a.vd;
    const TA* row = (const TA*)a.qkv + (size_t)t * a.ld;
    float* v = smem;                                  // q then k, 32-bit
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const float x = gl_load(row + i);
        v[i] = x;
        if (i < nq) sq += x * x; else sk += x * x;
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    float inv_q = 1.f, inv_k = 1.f;
    {
        const int nw = blockDim.x >> 5;
        sq = gl_warp_sum(sq);
        if (lane == 0) red[w] = sq;
        __syncthreads();
        float tq = 0.f;
        for (int i = 0; i < nw; ++i) tq += red[i];           // same order in every thread
        __syncthreads();
        sk = gl_warp_sum(sk);
        if (lane == 0) red[w] = sk;
        __syncthreads();
        float tk = 0.f;
        for (int i = 0; i < nw; ++i) tk += red[i];
        if (a.q_gamma) inv_q = 1.0f / sqrtf(tq / (float)nq + a.eps);
        if (a.k_gamma) inv_k = 1.0f / sqrtf(tk / (float)nk + a.eps);
    }
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        if (i < nq) { if (a.q_gamma) v[i] = v[i] * inv_q * a.q_gamma[i]; }
        else if (a.k_gamma) v[i] = v[i] * inv_k * a.k_gamma[i - nq];
    }
    __syncthreads();
    if (a.half > 0 && a.cosv) {
        const float* cs = a.cosv + (size_t)t * a.half;
        const float* sn = a.sinv + (size_t)t * a.half;
        const int pairs = (a.nH + (a.q_only ? 0 : a.nKV)) * a.half;
        for (int e = threadIdx.x; e < pairs; e += blockDim.x) {
            const int head = e / a.half, i = e - head * a.half;
            float* hv = v + (size_t)head * a.hd;
            const int i0 = a.interleaved ? 2 * i : i;
            const int i1 = a.interleaved ? 2 * i + 1 : i + a.half;
            const float c = cs[i], s = sn[i];
            const float u = hv[i0], x = hv[i1];
            hv[i0] = u * c - x * s;
            hv[i1] = x * c + u * s;
        }
        __syncthreads();
    }
    if (a.head_unit) {
        const int heads = a.nH + (a.q_only ? 0 : a.nKV);
        for (int head = w; head < heads; head += (int)(blockDim.x >> 5)) {        // a warp a head
            float* hv = v + (size_t)head * a.hd;
            float q2 = 0.f;
            for (int d = lane; d < a.hd; d += 32) q2 = fmaf(hv[d], hv[d], q2);
            const float inv = 1.0f / sqrtf(gl_warp_sum(q2) / (float)a.hd + a.eps);
            for (int d = lane; d < a.hd; d += 32) hv[d] *= inv;
        }
        __syncthreads();
    }
    const int pos = a.tok_pos[t];
    float q_mul = a.q_scale;
    if (a.temp_every > 0.f)
        q_mul *= 1.0f + a.temp_coef * logf((float)floor((double)(pos + 1) / (double)a.temp_every) + 1.0f);
    if (a.talk) {
        // a thread a column (key head c, dim d) of the wide rows: the column's query heads' values stay in registers
        // while the heads of the result are walked; the table's entries are the same for all threads of a step
        const int wide = a.nKV * a.hd, per = a.nH / a.nKV;
        TA* qo = (TA*)a.q_out + (size_t)t * a.nH * wide;
        // where the block has more threads than the rows have columns, the heads of the result are shared out too
        int parts = (int)blockDim.x / wide;
        if (parts < 1 || a.nH % parts) parts = 1;
        const int heads_each = a.nH / parts;
        for (int item = threadIdx.x; item < wide * parts; item += blockDim.x) {
            const int part = item / wide, r = item - part * wide;
            const int c = r / a.hd, d = r - c * a.hd;
            const int h_first = part * heads_each, h_end = h_first + heads_each;
            if (per <= 8) {
                float qg[8];
#pragma unroll
                for (int g = 0; g < 8; ++g) qg[g] = g < per ? v[(size_t)(c * per + g) * a.hd + d] * q_mul : 0.f;
                for (int h = h_first; h < h_end; ++h) {
                    const float* row = talk + (size_t)h * a.nH + c * per;
                    float y = 0.f;
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        if (g < per) y = fmaf(row[g], qg[g], y);
                    gl_store(qo + (size_t)h * wide + r, y);
                }
            } else {
                for (int h = h_first; h < h_end; ++h) {
                    float y = 0.f;
                    for (int g = c * per; g < (c + 1) * per; ++g) y = fmaf(talk[h * a.nH + g], v[(size_t)g * a.hd + d], y);
                    gl_store(qo + (size_t)h * wide + r, y * q_mul);
                }
            }
        }
    } else {
        TA* qo = (TA*)a.q_out + (size_t)t * nq;
        for (int i = threadIdx.x; i < nq; i += blockDim.x) gl_store(qo + i, v[i] * q_mul);
    }
    if (!a.write_kv || a.q_only) return;
    const int slot = gl_checked(pos / GL_PAGE, a.max_pages, GL_BAD_POSITION);
    const int page = gl_checked(a.pages[(size_t)a.tok_seq[t] * a.max_pages + slot], a.n_pages > 0 ? a.n_pages : 0x7fffffff, GL_BAD_PAGE);
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int head = i / a.hd, d = i - head * a.hd;
        if (a.k_joined) gl_store((TC*)a.k_cache + ((size_t)page * GL_PAGE + (pos % GL_PAGE)) * nk + i, v[nq + i]);
        else gl_store((TC*)a.k_cache + (((size_t)page * a.nKV + head) * GL_PAGE + (pos % GL_PAGE)) * a.hd + d, v[nq + i]);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int head = i / a.vd, d = i - head * a.vd;
        gl_store((TC*)a.v_cache + (((size_t)page * a.nKV + head) * GL_PAGE + (pos % GL_PAGE)) * a.vd + d,
                 gl_load(row + nq + nk + i));
    }
}

GL_API int gl_qkv_rownorm_cache(const QkvRowNormArgs* args, int act_dtype, int cache_dtype, cudaStream_t stream) {
    const QkvRowNormArgs& a = *args;
    if (a.T <= 0) return GL_OK;
    if (a.hd <= 0 || a.vd <= 0 || a.nH <= 0 || a.nKV <= 0 || 2 * a.half > a.hd) return GL_ERR_SHAPE;
    const size_t smem = ((size_t)(a.nH + a.nKV) * a.hd + (a.talk ? (size_t)a.nH * a.nH : 0)) * sizeof(float);
    if (smem > 200 * 1024) return GL_ERR_SMEM;
    // few tokens: more threads a token, so that a row's loads are in flight together; a table on the queries: a thread
    // a column of the wide rows
    const dim3 g((unsigned)a.T), b(a.T <= 256 && (a.nH + a.nKV) * a.hd >= 2048 ? 512 : (a.talk && a.nKV * a.hd >= 256 ? 256 : 128));
    if (act_dtype != cache_dtype || (act_dtype != GL_F32 && act_dtype != GL_BF16)) return GL_ERR_DTYPE;
    if (smem > 48 * 1024) {                           // (many wide heads: a block may ask for more than the default)
        const cudaError_t e = act_dtype == GL_F32
            ? cudaFuncSetAttribute(qkv_rownorm_cache_kernel<float, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
            : cudaFuncSetAttribute(qkv_rownorm_cache_kernel<__nv_bfloat16, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
    }
    if (act_dtype == GL_F32) return gl_launch(qkv_rownorm_cache_kernel<float, float>, g, b, smem, stream, 1, a);
    return gl_launch(qkv_rownorm_cache_kernel<__nv_bfloat16, __nv_bfloat16>, g, b, smem, stream, 1, a);
}
