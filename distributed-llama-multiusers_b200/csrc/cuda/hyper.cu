// Hyper-connections: the residual stream is kept in `streams` parallel copies x_1 .. x_S per token (row layout
// [S][dim]).  A sublayer reads one mixed vector and writes back into every copy:
//     read :  u   = sum_s w_in[s] x_s ;   h = u / sqrt(mean(u^2) + eps) * norm_w          (the sublayer's input)
//     write:  x_t <- sum_s mix[s][t] x_s  +  mult * w_out[t] * y       for all t at once, from the old copies
// With S = 1, mix = w_out = 1 this is the plain residual sum  x += mult * y.  Everything is f32.
//
// Kernels: the read (with an optional row gather: the model's last norm over the rows whose logits are wanted, where
// w_in = NULL means the plain sum of the copies), and the write fused with the read of the NEXT sublayer, so the
// copies are read once and written once per sublayer and the mixed vector never goes to memory.
// One CTA per row; a thread keeps its columns of u in registers between the sum of squares and the scaling.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

#define HC_THREADS 256
#define HC_CACHE 16                 // columns per thread kept in registers (dim <= 4096); wider rows recompute

template <int MAXS>
__global__ void __launch_bounds__(HC_THREADS) hc_step_kernel(DlHyperArgs a) {
    __shared__ float red[32];
    __shared__ float c_mix[MAXS * MAXS], c_out[MAXS], c_in[MAXS];
    const int m = blockIdx.x, S = a.streams, dim = a.dim;
    const bool write = a.y != nullptr, read = a.h != nullptr;
    if (threadIdx.x < S * S && write) c_mix[threadIdx.x] = a.mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (write) c_out[threadIdx.x] = a.mult * a.w_out[threadIdx.x];
        c_in[threadIdx.x] = a.w_in ? a.w_in[threadIdx.x] : 1.f;
    }
    __syncthreads();
    const int src = a.rows ? a.rows[m] : m;               // a gather never comes with a write
    float* x = a.x + (size_t)src * a.ldx;
    const float* y = write ? a.y + (size_t)m * a.ldy : nullptr;
    const bool cached = dim <= HC_THREADS * HC_CACHE;
    float u_keep[HC_CACHE];
    float ss = 0.f;
    // one column: the old copies in, the new copies out (a write), the mixed value of the (new) copies back
    auto column = [&](int i) -> float {
        float xs[MAXS];
#pragma unroll
        for (int s = 0; s < MAXS; ++s) xs[s] = s < S ? x[(size_t)s * dim + i] : 0.f;
        if (write) {
            const float yv = y[i];
            float xn[MAXS];
#pragma unroll
            for (int t = 0; t < MAXS; ++t) {
                xn[t] = 0.f;
                if (t < S) {
                    float v = 0.f;
#pragma unroll
                    for (int s = 0; s < MAXS; ++s)
                        if (s < S) v = fmaf(c_mix[s * S + t], xs[s], v);
                    xn[t] = fmaf(c_out[t], yv, v);
                    x[(size_t)t * dim + i] = xn[t];
                }
            }
#pragma unroll
            for (int s = 0; s < MAXS; ++s) xs[s] = xn[s];
        }
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
            if (s < S) u = fmaf(c_in[s], xs[s], u);
        return u;
    };
    if (cached) {
#pragma unroll
        for (int k = 0; k < HC_CACHE; ++k) {
            const int i = threadIdx.x + k * HC_THREADS;
            const float u = i < dim ? column(i) : 0.f;
            u_keep[k] = u;
            ss = fmaf(u, u, ss);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += HC_THREADS) {
            const float u = column(i);
            ss = fmaf(u, u, ss);
        }
    }
    if (!read) return;
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)dim + a.eps);
    float* h = a.h + (size_t)m * a.ldh;
    if (cached) {
#pragma unroll
        for (int k = 0; k < HC_CACHE; ++k) {
            const int i = threadIdx.x + k * HC_THREADS;
            if (i < dim) {
                const float t = u_keep[k] * inv;
                h[i] = a.norm_w ? t * a.norm_w[i] : t;
            }
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += HC_THREADS) {      // the copies are final by now: mix them again
            float u = 0.f;
            for (int s = 0; s < S; ++s) u = fmaf(c_in[s], x[(size_t)s * dim + i], u);
            const float t = u * inv;
            h[i] = a.norm_w ? t * a.norm_w[i] : t;
        }
    }
    if (a.u_out) {                                         // the mixed vector itself (tests, probes)
        float* uo = a.u_out + (size_t)m * dim;
        for (int i = threadIdx.x; i < dim; i += HC_THREADS) {
            float u = 0.f;
            for (int s = 0; s < S; ++s) u = fmaf(c_in[s], x[(size_t)s * dim + i], u);
            uo[i] = u;
        }
    }
}

// The same with four columns per thread and step (dim % 4 == 0, 16-byte aligned rows): all copies of a column group are
// loaded at once, so a decoding row is two or three dependent memory round trips instead of one per column.
#define HC_VEC_STREAMS 8            // copies the four-column kernel keeps in registers; more copies take the scalar kernel
#define HC_CACHE4 4                 // float4 groups per thread kept in registers (dim <= 4096)

__device__ __forceinline__ float4 f4_fma(float a, float4 x, float4 acc) {
    return make_float4(fmaf(a, x.x, acc.x), fmaf(a, x.y, acc.y), fmaf(a, x.z, acc.z), fmaf(a, x.w, acc.w));
}

__global__ void __launch_bounds__(HC_THREADS) hc_step_vec_kernel(DlHyperArgs a) {
    __shared__ float red[32];
    __shared__ float c_mix[HC_VEC_STREAMS * HC_VEC_STREAMS], c_out[HC_VEC_STREAMS], c_in[HC_VEC_STREAMS];
    const int m = blockIdx.x, S = a.streams, dim = a.dim, n4 = dim >> 2;
    const bool write = a.y != nullptr, read = a.h != nullptr;
    if (threadIdx.x < S * S && write) c_mix[threadIdx.x] = a.mix[threadIdx.x];
    if (threadIdx.x < S) {
        if (write) c_out[threadIdx.x] = a.mult * a.w_out[threadIdx.x];
        c_in[threadIdx.x] = a.w_in ? a.w_in[threadIdx.x] : 1.f;
    }
    __syncthreads();
    const int src = a.rows ? a.rows[m] : m;
    float4* x = reinterpret_cast<float4*>(a.x + (size_t)src * a.ldx);
    const float4* y = write ? reinterpret_cast<const float4*>(a.y + (size_t)m * a.ldy) : nullptr;
    float4 u_keep[HC_CACHE4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < HC_CACHE4; ++k) {
        const int i = threadIdx.x + k * HC_THREADS;
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            float4 xs[HC_VEC_STREAMS];
#pragma unroll
            for (int s = 0; s < HC_VEC_STREAMS; ++s) xs[s] = s < S ? x[(size_t)s * n4 + i] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (write) {
                const float4 yv = y[i];
                float4 xn[HC_VEC_STREAMS];
#pragma unroll
                for (int t = 0; t < HC_VEC_STREAMS; ++t) {
                    xn[t] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (t < S) {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (int s = 0; s < HC_VEC_STREAMS; ++s)
                            if (s < S) v = f4_fma(c_mix[s * S + t], xs[s], v);
                        xn[t] = f4_fma(c_out[t], yv, v);
                        x[(size_t)t * n4 + i] = xn[t];
                    }
                }
#pragma unroll
                for (int s = 0; s < HC_VEC_STREAMS; ++s) xs[s] = xn[s];
            }
#pragma unroll
            for (int s = 0; s < HC_VEC_STREAMS; ++s)
                if (s < S) u = f4_fma(c_in[s], xs[s], u);
        }
        u_keep[k] = u;
        ss = fmaf(u.x, u.x, fmaf(u.y, u.y, fmaf(u.z, u.z, fmaf(u.w, u.w, ss))));
    }
    if (!read) return;
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)dim + a.eps);
    float4* h = reinterpret_cast<float4*>(a.h + (size_t)m * a.ldh);
    const float4* nw = reinterpret_cast<const float4*>(a.norm_w);
#pragma unroll
    for (int k = 0; k < HC_CACHE4; ++k) {
        const int i = threadIdx.x + k * HC_THREADS;
        if (i < n4) {
            float4 t = make_float4(u_keep[k].x * inv, u_keep[k].y * inv, u_keep[k].z * inv, u_keep[k].w * inv);
            if (nw) { const float4 w = nw[i]; t.x *= w.x; t.y *= w.y; t.z *= w.z; t.w *= w.w; }
            h[i] = t;
            if (a.u_out) reinterpret_cast<float4*>(a.u_out + (size_t)m * dim)[i] = u_keep[k];
        }
    }
}

extern "C" int dl_hyper_step(const DlHyperArgs* args, void* stream) {
    const DlHyperArgs& a = *args;
    if (a.M < 1 || a.dim < 1 || a.streams < 1 || a.streams > DL_HC_MAX_STREAMS) {
        dl_set_error("dl_hyper_step: %d streams of %d (at most %d streams)", a.streams, a.dim, DL_HC_MAX_STREAMS);
        return -1;
    }
    if (a.y && (!a.mix || !a.w_out)) { dl_set_error("dl_hyper_step: a write needs mix and w_out"); return -1; }
    if (a.y && a.rows) { dl_set_error("dl_hyper_step: a row gather cannot come with a write"); return -1; }
    if (!a.y && !a.h) { dl_set_error("dl_hyper_step: nothing to do"); return -1; }
    const auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    const bool vec = a.streams <= HC_VEC_STREAMS && a.dim % 4 == 0 && a.dim <= 4 * HC_THREADS * HC_CACHE4 && a.ldx % 4 == 0 && al16(a.x) &&
                     (!a.y || (a.ldy % 4 == 0 && al16(a.y))) && (!a.h || (a.ldh % 4 == 0 && al16(a.h))) && al16(a.norm_w) && al16(a.u_out);
    if (vec) hc_step_vec_kernel<<<a.M, HC_THREADS, 0, (cudaStream_t)stream>>>(a);
    else if (a.streams <= 8) hc_step_kernel<8><<<a.M, HC_THREADS, 0, (cudaStream_t)stream>>>(a);
    else hc_step_kernel<DL_HC_MAX_STREAMS><<<a.M, HC_THREADS, 0, (cudaStream_t)stream>>>(a);
    LAYER_CHECK_LAUNCH("dl_hyper_step");
    return 0;
}
