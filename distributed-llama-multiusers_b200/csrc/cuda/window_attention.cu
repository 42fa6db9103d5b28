// Grouped-query attention over a sliding window whose values ARE its keys: one projection k per token and key/value
// head; the key is k with rotary positions on its first `rope_dims` dimensions, the value is k as projected.
//     score_h(i, j) = cap( scale * q_h,i . rot(k_g,j) ),   cap(s) = softcap * tanh(s / softcap)   (softcap 0: none)
//     visible: 0 <= i - j < window                                                               (window 0: all j <= i)
//     out_h(i)      = sum_j softmax_j(score_h(i, .)) k_g,j              g = h / (heads / kv_heads)
// Only the first rope_dims dimensions differ between a key and its value, so the cache holds, per token and key/value
// head, ONE line  [ rot(k)[0 : dim] | k[0 : rope_dims] ]:  the key is the first `dim` entries, the value is the tail
// followed by entries rope_dims .. dim of the key.  (dim + rope_dims) instead of 2 dim numbers per token and head.
// Cache layout: [page][kv_head][page_size][dim + rope_dims], bf16 or f32; pages of a sequence from its block table.
//
// Rotary: interleaved pairs (2i, 2i + 1), angle = pos * freqs[i] formed in f64, cos and sin multiplied by rope_scale
// (frequency interpolation schemes that also scale the rotation's magnitude pass their factor here).
//
// Kernels: the cache writer; the per-row attention kernel (exact f32 arithmetic on either cache type; one CTA per
// (row, key/value head), all query heads of the group share each staged page; pages outside the window are never
// touched); the tensor-core kernel for prompt portions (bf16 cache) further down.
#include "mma_common.cuh"
#include "../../../include/dllama_b200.h"

#define WA_PAGE 32

// ------------------------------------------------------------------------------------------------
// cache writer
// ------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void __launch_bounds__(128) window_kv_write_kernel(DlWindowKvArgs a) {
    const int m = blockIdx.x;
    const int pos = a.pos[m], slot = a.slot[m];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / WA_PAGE];
    const int LD = a.dim + a.rope_dims, half = a.rope_dims / 2;
    for (int g = 0; g < a.kv_heads; ++g) {
        const float* in = a.k + (size_t)m * a.ld + (size_t)g * a.dim;
        CT* dst = (CT*)a.cache + (((size_t)page * a.kv_heads + g) * WA_PAGE + pos % WA_PAGE) * LD;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            double s, c;
            sincos((double)pos * a.freqs[i], &s, &c);
            const double u = in[2 * i], v = in[2 * i + 1], ms = a.rope_scale;
            st_f(dst + 2 * i, (float)((u * c - v * s) * ms));
            st_f(dst + 2 * i + 1, (float)((v * c + u * s) * ms));
        }
        for (int i = a.rope_dims + threadIdx.x; i < a.dim; i += blockDim.x) st_f(dst + i, in[i]);
        for (int i = threadIdx.x; i < a.rope_dims; i += blockDim.x) st_f(dst + a.dim + i, in[i]);
    }
}

extern "C" int dl_window_kv_write(const DlWindowKvArgs* args, int M, void* stream) {
    const DlWindowKvArgs& a = *args;
    if (a.rope_dims > a.dim || (a.rope_dims & 1) || a.page_size != WA_PAGE) { dl_set_error("dl_window_kv_write: bad rotary or page size"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.ctype == DL_T_BF16) window_kv_write_kernel<__nv_bfloat16><<<M, 128, 0, st>>>(a);
    else window_kv_write_kernel<float><<<M, 128, 0, st>>>(a);
    LAYER_CHECK_LAUNCH("dl_window_kv_write");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// per-row attention: one CTA per (row, key/value head)
// ------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void window_attention_kernel(DlWindowAttnArgs a) {
    extern __shared__ float sm[];
    const int m = blockIdx.x, g = blockIdx.y;
    const int rep = a.heads / a.kv_heads, D = a.dim, RD = a.rope_dims, LD = D + RD, LP = LD + 1;
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = sm;                                   // [rep][D]
    float* tile = q_s + (size_t)rep * D;               // [WA_PAGE][LD + 1]
    float* acc = tile + (size_t)WA_PAGE * LP;          // [rep][D]
    float* p_s = acc + (size_t)rep * D;                // [nw][WA_PAGE]
    float* ml = p_s + (size_t)nw * WA_PAGE;            // [rep][2]
    const int pos = a.pos[m], slot = a.slot[m];
    const int first = a.window > 0 ? max(0, pos - a.window + 1) : 0;      // oldest visible position
    for (int t = threadIdx.x; t < rep * D; t += blockDim.x) {
        q_s[t] = a.q[(size_t)m * a.ldq + (size_t)g * rep * D + t];
        acc[t] = 0.f;
    }
    for (int t = threadIdx.x; t < rep; t += blockDim.x) { ml[2 * t] = -INFINITY; ml[2 * t + 1] = 0.f; }
    for (int pg = first / WA_PAGE; pg <= pos / WA_PAGE; ++pg) {
        __syncthreads();
        const int page = a.block_table[(size_t)slot * a.max_pages + pg];
        const CT* src = (const CT*)a.cache + ((size_t)page * a.kv_heads + g) * WA_PAGE * LD;
        const int j_lo = max(0, first - pg * WA_PAGE), j_hi = min(WA_PAGE, pos + 1 - pg * WA_PAGE);   // visible lines [j_lo, j_hi)
        for (int i = threadIdx.x; i < WA_PAGE * LD; i += blockDim.x) {
            const int j = i / LD, d = i - j * LD;
            tile[j * LP + d] = (j >= j_lo && j < j_hi) ? ld_f(src + i) : 0.f;
        }
        __syncthreads();
        for (int h = warp; h < rep; h += nw) {
            const float* qh = q_s + (size_t)h * D;
            const float* row = tile + lane * LP;
            const bool vis = lane >= j_lo && lane < j_hi;
            float s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(qh[d], row[d], s);
            s *= a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            if (!vis) s = -INFINITY;
            const float m_old = ml[2 * h], m_new = fmaxf(m_old, warp_max(s));
            const float p = vis ? expf(s - m_new) : 0.f;
            const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            const float l_new = ml[2 * h + 1] * alpha + warp_sum(p);
            p_s[warp * WA_PAGE + lane] = p;
            __syncwarp();
            if (lane == 0) { ml[2 * h] = m_new; ml[2 * h + 1] = l_new; }
            float* ah = acc + (size_t)h * D;
            const float* ps = p_s + warp * WA_PAGE;
            for (int d = lane; d < D; d += 32) {
                const int col = d < RD ? D + d : d;              // the value's first entries sit behind the key
                float v = ah[d] * alpha;
                for (int j = j_lo; j < j_hi; ++j) v = fmaf(ps[j], tile[j * LP + col], v);
                ah[d] = v;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < rep * D; t += blockDim.x)
        a.out[(size_t)m * a.ldo + (size_t)g * rep * D + t] = acc[t] / ml[2 * (t / D) + 1];
}

static int window_args_ok(const DlWindowAttnArgs& a, const char* who) {
    if (a.heads < 1 || a.kv_heads < 1 || a.heads % a.kv_heads || a.dim < 1 || a.rope_dims > a.dim || a.window < 0 || a.page_size != WA_PAGE) {
        dl_set_error("%s: bad shape (heads %d / %d, dim %d, rotary %d, window %d, page %d)", who, a.heads, a.kv_heads, a.dim, a.rope_dims, a.window, a.page_size);
        return -1;
    }
    return 0;
}

extern "C" int dl_window_attention(const DlWindowAttnArgs* args, int M, void* stream) {
    const DlWindowAttnArgs& a = *args;
    if (window_args_ok(a, "dl_window_attention")) return -1;
    const int rep = a.heads / a.kv_heads, nw = rep < 8 ? rep : 8, LD = a.dim + a.rope_dims;
    const size_t smem = ((size_t)2 * rep * a.dim + (size_t)WA_PAGE * (LD + 1) + (size_t)nw * WA_PAGE + 2 * (size_t)rep) * sizeof(float);
    if (smem > 227 * 1024) { dl_set_error("dl_window_attention: %d heads per group x dim %d need %zu bytes of shared memory", rep, a.dim, smem); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(M, a.kv_heads);
    cudaError_t e;
    if (a.ctype == DL_T_BF16) {
        e = cudaFuncSetAttribute(window_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) window_attention_kernel<__nv_bfloat16><<<grid, nw * 32, smem, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(window_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) window_attention_kernel<float><<<grid, nw * 32, smem, st>>>(a);
    }
    if (e != cudaSuccess) { dl_set_error("dl_window_attention: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    LAYER_CHECK_LAUNCH("dl_window_attention");
    return 0;
}
