// Prompt attention for a mixer whose heads' softmax weights are mixed before they meet the values
// (see attention_mixed.cu): the pairs A[g, c](i) = sum_j p_g(i, j) v_c(j) on the tensor cores, bfloat16.
//
// A block takes 64 consecutive query rows of one pair (query head g, value head c) of one sequence; each
// of its 4 warps owns 16 rows.  Key pages of g's key head and value pages of head c (64 positions each)
// stream through shared memory with cp.async, two pages in flight.  Scores and the output are
// mma.sync.m16n8k16 products with 32-bit accumulators; the maximum, the sum, the weights and the
// rescaling of the running softmax are 32-bit, and the pair's result leaves in 32-bit for the mixing
// kernel.  Rows past a sequence's length are zero-filled on load.  Key and value sizes are compile-time
// constants (GL_HEAD_DIM, GL_VALUE_DIM), multiples of 16.
#include "common.cuh"

#ifndef GL_HEAD_DIM
#error "compile with -DGL_HEAD_DIM=<key size> [-DGL_VALUE_DIM=<value size>]"
#endif
#ifndef GL_VALUE_DIM
#define GL_VALUE_DIM GL_HEAD_DIM
#endif
static_assert(GL_HEAD_DIM % 16 == 0 && GL_HEAD_DIM >= 16 && GL_HEAD_DIM <= 256, "key size: 16..256 in steps of 16");
static_assert(GL_VALUE_DIM % 16 == 0 && GL_VALUE_DIM >= 16 && GL_VALUE_DIM <= 256, "value size: 16..256 in steps of 16");

#define AP_HD GL_HEAD_DIM
#define AP_VD GL_VALUE_DIM
#define AP_BM 64
#define AP_THREADS 128
#define AP_KS (AP_HD / 16)            // k-steps of the score product
#define AP_NT (AP_VD / 8)             // 8-wide column tiles of the output
#define AP_ROW (AP_HD * 2 + 16)       // padded row: 8 consecutive rows fall in distinct banks
#define AP_VROW (AP_VD * 2 + 16)
#define AP_TILE (64 * AP_ROW)
#define AP_VTILE (64 * AP_VROW)

struct PairsArgs {
    const void* q;            // [T, nH*hd] bf16, already scaled
    float* pairs;             // [T, nH, nVal, vd] 32-bit
    const void* k_cache;      // [pages, nKV, GL_PAGE, hd] bf16
    const void* v_cache;      // [pages, nKV, GL_PAGE, vd] bf16
    const int* seq_qstart;    // [B]
    const int* seq_qlen;      // [B]
    const int* seq_ctx;       // [B]
    const int* pages;         // [B, max_pages]
    int B, nH, nKV, nVal, max_pages, window, max_qlen;
    float score_scale;        // multiplies q . k
    float softcap;            // > 0: s <- softcap * tanh(s / softcap)
    const float* slopes;      // [nH] or null: s <- s - slope_h * (query position - key position)
    void* out;                // [T, nH*vd] bf16 or null: without a mixing table (nVal 1) the result goes here, rounded,
                              // and no second kernel has to read the 32-bit pairs again
    const float* sinks;       // [nH] or null: e^(sinks[h]) joins the softmax's denominator of head h
    int nVH;                  // heads of the value cache where they are more than the key heads (0: nKV); without a
                              // table, query head h then takes the values of head h / (nH / nVH)
};

__device__ __forceinline__ unsigned ap_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ap_cp16(unsigned dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void ap_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void ap_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }
__device__ __forceinline__ void ap_ldm4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_ldm4t(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ap_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// cap * tanh(x / cap) as cap * (1 - 2 / (e^(2x/cap) + 1)) with the hardware's exponential and reciprocal: off by
// a few 1e-7 of cap (1e-5 at a cap of 50), which is small against what bfloat16 queries and keys leave in a score
// (2^-9 of it), and a fifth of the instructions of tanhf; every score of a prompt passes here, and with tanhf the
// shaping was most of what the kernel issued.  (The 32-bit kernels keep tanhf.)
__device__ __forceinline__ float ap_softcap(float x, float cap, float two_over_cap) {
    const float e = __expf(x * two_over_cap);                 // inf for large x: the quotient is then 0
    return cap * (1.0f - __fdividef(2.0f, e + 1.0f));
}
__device__ __forceinline__ unsigned ap_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *(unsigned*)&v;
}

// rows [0, n_valid) of a page tile (or of the query tile) to padded shared memory; the rest is zero
template <int DIM>
__device__ __forceinline__ void ap_load_rows(unsigned dst, const __nv_bfloat16* src, size_t src_row_stride, int n_valid) {
    constexpr int CHUNKS = DIM / 8, ROW = DIM * 2 + 16;
    for (int i = threadIdx.x; i < 64 * CHUNKS; i += AP_THREADS) {
        const int r = i / CHUNKS, c = i - r * CHUNKS;
        const bool ok = r < n_valid;
        ap_cp16(dst + r * ROW + c * 16, ok ? (const void*)(src + (size_t)r * src_row_stride + c * 8) : (const void*)src,
                ok ? 16 : 0);
    }
}

__global__ void __launch_bounds__(AP_THREADS)
attn_pairs_tc_kernel(PairsArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const unsigned sQ = ap_smem(smem);
    const unsigned sK[2] = {sQ + AP_TILE, sQ + 2 * AP_TILE};
    const unsigned sV[2] = {sQ + 3 * AP_TILE, sQ + 3 * AP_TILE + AP_VTILE};
    gl_grid_wait();                                            // (a long kernel: the next one is not launched early)
    const int b = blockIdx.z;
    const int h = blockIdx.y / a.nVal;                         // query head
    const int g = h / (a.nH / a.nKV);                          // its key head
    const int nvh = a.nVH > 0 ? a.nVH : a.nKV;
    const int vh = a.nVal > 1 ? blockIdx.y - h * a.nVal : h / (a.nH / nvh);   // the pair's value head
    const int qlen = a.seq_qlen[b];
    const int n_qtiles = (qlen + AP_BM - 1) / AP_BM;
    const int qt = n_qtiles - 1 - (int)blockIdx.x;           // longest rows first
    if (qt < 0) return;
    const int ctx = a.seq_ctx[b], qstart = a.seq_qstart[b];
    const int q0 = qt * AP_BM;
    const int rows = min(AP_BM, qlen - q0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = lane >> 2, t = lane & 3;
    const int p_first = ctx + q0, p_last = ctx + q0 + rows - 1;
    const int lo_first = (a.window > 0 && p_first - a.window + 1 > 0) ? p_first - a.window + 1 : 0;
    const int page_begin = lo_first / GL_PAGE, page_end = p_last / GL_PAGE + 1;
    const int* pg = a.pages + (size_t)b * a.max_pages;
    const __nv_bfloat16* K = (const __nv_bfloat16*)a.k_cache;
    const __nv_bfloat16* V = (const __nv_bfloat16*)a.v_cache;
    const size_t head_off = (size_t)g * GL_PAGE * AP_HD, page_stride = (size_t)a.nKV * GL_PAGE * AP_HD;
    const size_t vhead_off = (size_t)vh * GL_PAGE * AP_VD, vpage_stride = (size_t)nvh * GL_PAGE * AP_VD;
    const int total = ctx + qlen;

    // the query tile, then the first page
    ap_load_rows<AP_HD>(sQ, (const __nv_bfloat16*)a.q + ((size_t)(qstart + q0) * a.nH + h) * AP_HD, (size_t)a.nH * AP_HD, rows);
    {
        const int nv = min(GL_PAGE, total - page_begin * GL_PAGE);
        ap_load_rows<AP_HD>(sK[0], K + (size_t)pg[page_begin] * page_stride + head_off, AP_HD, nv);
        ap_load_rows<AP_VD>(sV[0], V + (size_t)pg[page_begin] * vpage_stride + vhead_off, AP_VD, nv);
    }
    ap_commit();

    unsigned qf[AP_KS][4];
    float o[AP_NT][4];
#pragma unroll
    for (int i = 0; i < AP_NT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float LOG2E = 1.4426950408889634f;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    const bool shaped = a.score_scale != 1.0f || a.softcap > 0.f || a.slopes != nullptr;
    const float two_over_cap = a.softcap > 0.f ? 2.0f / a.softcap : 0.f;
    const int r_lo = warp * 16 + grp, r_hi = r_lo + 8;        // this thread's two rows inside the tile
    const int pos_lo = p_first + r_lo, pos_hi = p_first + r_hi;
    const int wlo_lo = (a.window > 0 && pos_lo - a.window + 1 > 0) ? pos_lo - a.window + 1 : 0;
    const int wlo_hi = (a.window > 0 && pos_hi - a.window + 1 > 0) ? pos_hi - a.window + 1 : 0;

    for (int p = page_begin; p < page_end; ++p) {
        const int st = (p - page_begin) & 1;
        if (p + 1 < page_end) {
            const int nv = min(GL_PAGE, total - (p + 1) * GL_PAGE);
            ap_load_rows<AP_HD>(sK[st ^ 1], K + (size_t)pg[p + 1] * page_stride + head_off, AP_HD, nv);
            ap_load_rows<AP_VD>(sV[st ^ 1], V + (size_t)pg[p + 1] * vpage_stride + vhead_off, AP_VD, nv);
        }
        ap_commit();
        ap_wait<1>();
        __syncthreads();
        if (p == page_begin) {
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
                const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int c = kk * 2 + (lane >> 4);
                ap_ldm4(sQ + r * AP_ROW + c * 16, qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
        }
        const int j0 = p * GL_PAGE;
        // a warp whose rows all lie before this page has nothing to do here (causal)
        const bool warp_active = j0 <= p_first + warp * 16 + 15;
        if (warp_active) {
            float s[8][4];
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < AP_KS; ++kk) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = j * 8 + ((lane >> 4) & 1) * 8 + (lane & 7);
                    const int c = kk * 2 + ((lane >> 3) & 1);
                    ap_ldm4(sK[st] + r * AP_ROW + c * 16, b0, b1, b2, b3);
                    ap_mma(s[j], qf[kk], b0, b1);
                    ap_mma(s[j + 1], qf[kk], b2, b3);
                }
            }
            if (shaped) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j0 + j * 8 + 2 * t + (e & 1);
                        float x = s[j][e] * a.score_scale;
                        if (a.softcap > 0.f) x = ap_softcap(x, a.softcap, two_over_cap);
                        s[j][e] = x - slope * (float)(((e < 2) ? pos_lo : pos_hi) - key);
                    }
                }
            }
            // mask: a row at position x sees keys max(0, x-window+1) .. x
            const bool need_mask = (j0 + GL_PAGE - 1 > p_first + warp * 16) || (a.window > 0 && j0 < wlo_hi + 8);
            if (need_mask) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int key = j0 + j * 8 + 2 * t + (e & 1);
                        const int pos = (e < 2) ? pos_lo : pos_hi;
                        const int wl = (e < 2) ? wlo_lo : wlo_hi;
                        if (key > pos || key < wl) s[j][e] = -INFINITY;
                    }
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            }
            float corr[2], mu[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float m_new = fmaxf(m_run[i], mx[i]);
                mu[i] = (m_new == -INFINITY) ? 0.f : m_new * LOG2E;
                corr[i] = exp2f(m_run[i] * LOG2E - mu[i]);       // m_run = -inf gives 0
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                s[j][0] = exp2f(s[j][0] * LOG2E - mu[0]);
                s[j][1] = exp2f(s[j][1] * LOG2E - mu[0]);
                s[j][2] = exp2f(s[j][2] * LOG2E - mu[1]);
                s[j][3] = exp2f(s[j][3] * LOG2E - mu[1]);
                l_run[0] += s[j][0] + s[j][1];
                l_run[1] += s[j][2] + s[j][3];
            }
#pragma unroll
            for (int i = 0; i < AP_NT; ++i) {
                o[i][0] *= corr[0]; o[i][1] *= corr[0];
                o[i][2] *= corr[1]; o[i][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                unsigned pa[4];
                pa[0] = ap_pack(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = ap_pack(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = ap_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = ap_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dn = 0; dn < AP_NT; dn += 2) {
                    unsigned b0, b1, b2, b3;
                    const int r = kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7);
                    const int c = dn + (lane >> 4);
                    ap_ldm4t(sV[st] + r * AP_VROW + c * 16, b0, b1, b2, b3);
                    ap_mma(o[dn], pa, b0, b1);
                    ap_mma(o[dn + 1], pa, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    ap_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    float inv_lo = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
    float inv_hi = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
    if (a.sinks) {
        // the sink joins the denominator once, against the larger of the row's maximum and itself
        const float sink = a.sinks[h];
        const float top_lo = fmaxf(m_run[0], sink), top_hi = fmaxf(m_run[1], sink);
        const float sc_lo = m_run[0] > -INFINITY ? expf(m_run[0] - top_lo) : 0.f;
        const float sc_hi = m_run[1] > -INFINITY ? expf(m_run[1] - top_hi) : 0.f;
        inv_lo = sc_lo / (l_run[0] * sc_lo + expf(sink - top_lo));
        inv_hi = sc_hi / (l_run[1] * sc_hi + expf(sink - top_hi));
    }
    const int slot = a.nVal > 1 ? vh : 0;
    if (a.out && a.nVal == 1) {
        __nv_bfloat16* O = (__nv_bfloat16*)a.out;
#pragma unroll
        for (int i = 0; i < AP_NT; ++i) {
            const int d = i * 8 + 2 * t;
            if (r_lo < rows)
                *(__nv_bfloat162*)(O + ((size_t)(qstart + q0 + r_lo) * a.nH + h) * AP_VD + d) =
                    __floats2bfloat162_rn(o[i][0] * inv_lo, o[i][1] * inv_lo);
            if (r_hi < rows)
                *(__nv_bfloat162*)(O + ((size_t)(qstart + q0 + r_hi) * a.nH + h) * AP_VD + d) =
                    __floats2bfloat162_rn(o[i][2] * inv_hi, o[i][3] * inv_hi);
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < AP_NT; ++i) {
        const int d = i * 8 + 2 * t;
        if (r_lo < rows)
            *(float2*)(a.pairs + (((size_t)(qstart + q0 + r_lo) * a.nH + h) * a.nVal + slot) * AP_VD + d) =
                make_float2(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (r_hi < rows)
            *(float2*)(a.pairs + (((size_t)(qstart + q0 + r_hi) * a.nH + h) * a.nVal + slot) * AP_VD + d) =
                make_float2(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

GL_API int gl_attention_pairs_tc_dims() { return AP_HD * 1000 + AP_VD; }

GL_API int gl_attention_pairs_tc(const PairsArgs* args, cudaStream_t stream) {
    const PairsArgs& a = *args;
    if (a.B <= 0 || a.max_qlen <= 0) return GL_OK;
    if (a.nH <= 0 || a.nKV <= 0 || a.nH % a.nKV || (a.nVal != 1 && a.nVal != a.nKV)) return GL_ERR_SHAPE;
    if (a.nVH < 0 || (a.nVH > 0 && (a.nH % a.nVH || (a.nVal != 1 && a.nVH != a.nKV)))) return GL_ERR_SHAPE;
    if (a.B > 65535 || a.nH * a.nVal > 65535) return GL_ERR_SHAPE;
    const size_t smem = 3 * (size_t)AP_TILE + 2 * (size_t)AP_VTILE;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_pairs_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return GL_ERR_SMEM;
        }
        configured = true;
    }
    dim3 grid((a.max_qlen + AP_BM - 1) / AP_BM, a.nH * a.nVal, a.B);
    return gl_launch(attn_pairs_tc_kernel, grid, dim3(AP_THREADS), smem, stream, 1, a) == 0 ? GL_OK : GL_ERR_LAUNCH;
}
