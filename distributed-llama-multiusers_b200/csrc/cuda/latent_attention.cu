// Latent attention: keys and values of all heads are up-projections of one small latent vector per token, plus one
// rotated key part that all heads share.  The cache holds, per token, [latent: rank | rotated key: rot] and nothing
// per head.  Attention runs in the latent space ("absorbed" form):
//     score_h(i, j) = scale * ( (U_k,h^T q_h,i) . c_j  +  qrot_h,i . krot_j )         softmax over j <= i
//     out_h(i)      = U_v,h ( sum_j p_h(i, j) c_j )
// so the per-head work against the cache is a dot product with, and a weighted sum of, the same rows for every head.
// The two per-head projections (U_k^T q before, U_v after) are batched dense products (dense.cu).
//
// Kernels here: the cache writer (RMS norm of the latent + rotary on the shared key part + paged store), rotary on
// a slice of each head of a row-major activation, and the attention itself over the paged latent cache, one CTA per
// query row with every head of the row sharing each page it stages in shared memory.  Softmax, norms and rotary
// angles are f32 (angles in f64); the cache is bf16 or f32.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

// rotate-half layout: dimension i pairs with i + dims/2; (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = pos * f_i
__device__ __forceinline__ void rot_pair(float u, float v, int pos, double f, float& ou, float& ov) {
    double s, c;
    sincos((double)pos * f, &s, &c);
    ou = (float)((double)u * c - (double)v * s);
    ov = (float)((double)v * c + (double)u * s);
}

// ------------------------------------------------------------------------------------------------
// cache writer: row m of kv = [rank latent | rot key part]
// ------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void __launch_bounds__(128) latent_kv_write_kernel(DlLatentKvArgs a) {
    __shared__ float red[32];
    const int m = blockIdx.x;
    const float* in = a.kv + (size_t)m * a.ld;
    const int pos = a.pos[m], slot = a.slot[m];
    const int page = a.block_table[(size_t)slot * a.max_pages + pos / a.page_size];
    const int D = a.rank + a.rot;
    CT* dst = (CT*)a.cache + ((size_t)page * a.page_size + pos % a.page_size) * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)a.rank + a.eps);
    for (int i = threadIdx.x; i < a.rank; i += blockDim.x) st_f(dst + i, in[i] * inv * a.norm_w[i]);
    const int half = a.rope_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float u, v;
        rot_pair(in[a.rank + i], in[a.rank + i + half], pos, a.freqs[i], u, v);
        st_f(dst + a.rank + i, u);
        st_f(dst + a.rank + i + half, v);
    }
    for (int i = a.rope_dims + threadIdx.x; i < a.rot; i += blockDim.x) st_f(dst + a.rank + i, in[a.rank + i]);
}

extern "C" int dl_latent_kv_write(const DlLatentKvArgs* args, int M, void* stream) {
    const DlLatentKvArgs& a = *args;
    if (a.rope_dims > a.rot || (a.rope_dims & 1)) { dl_set_error("dl_latent_kv_write: bad rotary size"); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    if (a.ctype == DL_T_BF16) latent_kv_write_kernel<__nv_bfloat16><<<M, 128, 0, st>>>(a);
    else latent_kv_write_kernel<float><<<M, 128, 0, st>>>(a);
    LAYER_CHECK_LAUNCH("dl_latent_kv_write");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// rotary on dims [offset, offset + rope_dims) of each head of x[M][n_heads][head_stride], in place
// ------------------------------------------------------------------------------------------------
__global__ void rope_rows_kernel(float* x, long long ld, int n_heads, int head_stride, int offset, int rope_dims,
                                 const double* __restrict__ freqs, const int* __restrict__ pos) {
    const int m = blockIdx.x, half = rope_dims / 2;
    const int p = pos[m];
    for (int t = threadIdx.x; t < n_heads * half; t += blockDim.x) {
        const int h = t / half, i = t % half;
        float* q = x + (size_t)m * ld + (size_t)h * head_stride + offset;
        float u, v;
        rot_pair(q[i], q[i + half], p, freqs[i], u, v);
        q[i] = u;
        q[i + half] = v;
    }
}

extern "C" int dl_rope_rows(float* x, long long ld, int M, int n_heads, int head_stride, int offset, int rope_dims,
                            const double* freqs, const int* pos, void* stream) {
    if ((rope_dims & 1) || offset + rope_dims > head_stride) { dl_set_error("dl_rope_rows: bad rotary size"); return -1; }
    rope_rows_kernel<<<M, 128, 0, (cudaStream_t)stream>>>(x, ld, n_heads, head_stride, offset, rope_dims, freqs, pos);
    LAYER_CHECK_LAUNCH("dl_rope_rows");
    return 0;
}

// ------------------------------------------------------------------------------------------------
// attention over the paged latent cache; one CTA per query row, one page (LA_TILE tokens) per step
// ------------------------------------------------------------------------------------------------
#define LA_TILE 32

template <typename CT>
__global__ void latent_attention_kernel(DlLatentAttnArgs a) {
    extern __shared__ float sm[];
    const int m = blockIdx.x;
    const int H = a.n_heads, R = a.rank, D = a.rank + a.rot, DP = D + 1;
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* q_s = sm;                                  // [H][D]   absorbed query | rotated query part
    float* tile = q_s + (size_t)H * D;                // [LA_TILE][D + 1]
    float* acc = tile + (size_t)LA_TILE * DP;         // [H][R]
    float* p_s = acc + (size_t)H * R;                 // [nw][LA_TILE]
    float* ml = p_s + (size_t)nw * LA_TILE;           // [H][2]   running maximum, running sum
    const int pos = a.pos[m], slot = a.slot[m];
    for (int t = threadIdx.x; t < H * D; t += blockDim.x) {
        const int h = t / D, d = t % D;
        q_s[t] = d < R ? a.q_lat[((size_t)m * H + h) * R + d]
                       : a.q[(size_t)m * a.ldq + (size_t)h * a.q_head_stride + a.q_rot_offset + (d - R)];
    }
    for (int t = threadIdx.x; t < H * R; t += blockDim.x) acc[t] = 0.f;
    for (int t = threadIdx.x; t < H; t += blockDim.x) { ml[2 * t] = -INFINITY; ml[2 * t + 1] = 0.f; }
    const int n_tiles = pos / LA_TILE + 1;
    for (int t = 0; t < n_tiles; ++t) {
        __syncthreads();                              // q_s / acc ready; previous tile consumed
        const int page = a.block_table[(size_t)slot * a.max_pages + t];
        const CT* src = (const CT*)a.cache + (size_t)page * LA_TILE * D;
        const int valid = min(LA_TILE, pos + 1 - t * LA_TILE);
        for (int i = threadIdx.x; i < LA_TILE * D; i += blockDim.x) {
            const int j = i / D, d = i % D;
            tile[j * DP + d] = j < valid ? ld_f(src + i) : 0.f;
        }
        __syncthreads();
        for (int h = warp; h < H; h += nw) {
            const float* qh = q_s + (size_t)h * D;
            const float* row = tile + lane * DP;
            float s = 0.f;
            for (int d = 0; d < D; ++d) s = fmaf(qh[d], row[d], s);
            s = lane < valid ? s * a.scale : -INFINITY;
            const float m_old = ml[2 * h], m_new = fmaxf(m_old, warp_max(s));
            const float p = lane < valid ? expf(s - m_new) : 0.f;
            const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            const float l_new = ml[2 * h + 1] * alpha + warp_sum(p);
            p_s[warp * LA_TILE + lane] = p;
            __syncwarp();
            if (lane == 0) { ml[2 * h] = m_new; ml[2 * h + 1] = l_new; }
            float* ah = acc + (size_t)h * R;
            const float* ps = p_s + warp * LA_TILE;
            for (int d = lane; d < R; d += 32) {
                float v = ah[d] * alpha;
                for (int j = 0; j < valid; ++j) v = fmaf(ps[j], tile[j * DP + d], v);
                ah[d] = v;
            }
            __syncwarp();
        }
    }
    __syncthreads();
    for (int t = threadIdx.x; t < H * R; t += blockDim.x) a.out[(size_t)m * H * R + t] = acc[t] / ml[2 * (t / R) + 1];
}

static size_t latent_attention_smem(int H, int rank, int rot, int nw) {
    const size_t D = (size_t)rank + rot;
    return ((size_t)H * D + (size_t)LA_TILE * (D + 1) + (size_t)H * rank + (size_t)nw * LA_TILE + 2 * (size_t)H) * sizeof(float);
}

extern "C" int dl_latent_attention(const DlLatentAttnArgs* args, int M, void* stream) {
    const DlLatentAttnArgs& a = *args;
    if (a.page_size != LA_TILE) { dl_set_error("dl_latent_attention: page size must be %d", LA_TILE); return -1; }
    const int nw = a.n_heads < 8 ? a.n_heads : 8;
    const size_t smem = latent_attention_smem(a.n_heads, a.rank, a.rot, nw);
    if (smem > 227 * 1024) { dl_set_error("dl_latent_attention: %d heads x rank %d need %zu bytes of shared memory", a.n_heads, a.rank, smem); return -1; }
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (a.ctype == DL_T_BF16) {
        e = cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) latent_attention_kernel<__nv_bfloat16><<<M, nw * 32, smem, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) latent_attention_kernel<float><<<M, nw * 32, smem, st>>>(a);
    }
    if (e != cudaSuccess) { dl_set_error("dl_latent_attention: shared memory attribute: %s", cudaGetErrorString(e)); return -(int)e; }
    LAYER_CHECK_LAUNCH("dl_latent_attention");
    return 0;
}
