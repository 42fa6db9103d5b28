// RMS normalisation in its variants, all in f32:  y = v / sqrt(mean(v^2) + eps) * scale
//   * scale = w  or  (1 + w)  (a weight stored around zero)  or 1 (no weight);
//   * the row may be normalised in `groups` equal parts, each by its own root mean square;
//   * v = x  or  x * silu(gate)  (a gate applied before the norm);
//   * the result is stored, or added to what y holds (a norm on a sublayer's output, summed into the residual stream);
//   * an optional row map gathers source rows (the final norm of the rows whose logits are wanted).
// One CTA per (row, group); groups of up to 4096 values stay in registers between the sum of squares and the scaling.
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

#define RN_THREADS 256
#define RN_CACHE 16                // values a thread keeps in registers between the two passes (groups of up to 4096)

__global__ void __launch_bounds__(RN_THREADS) rms_norm_kernel(DlNormArgs a) {
    __shared__ float red[32];
    const int m = blockIdx.x, g = blockIdx.y;
    const int src = a.rows ? a.rows[m] : m;
    const int gd = a.dim / a.groups;
    const float* x = a.x + (size_t)src * a.ldx + (size_t)g * gd;
    const float* gate = a.gate ? a.gate + (size_t)src * a.ld_gate + (size_t)g * gd : nullptr;
    const bool cached = gd <= RN_THREADS * RN_CACHE;
    float v[RN_CACHE];
    float ss = 0.f;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            float t = 0.f;
            if (i < gd) {
                t = x[i];
                if (gate) t *= silu_f(gate[i]);
            }
            v[k] = t;
            ss = fmaf(t, t, ss);
        }
    } else {
        for (int i = threadIdx.x; i < gd; i += RN_THREADS) {
            float t = x[i];
            if (gate) t *= silu_f(gate[i]);
            ss = fmaf(t, t, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)gd + a.eps);
    float* y = a.y + (size_t)m * a.ldy + (size_t)g * gd;
    const float* w = a.w ? a.w + (size_t)g * gd : nullptr;
    if (cached) {
#pragma unroll
        for (int k = 0; k < RN_CACHE; ++k) {
            const int i = threadIdx.x + k * RN_THREADS;
            if (i < gd) {
                float t = v[k] * inv;
                if (w) t *= a.plus_one ? 1.f + w[i] : w[i];
                y[i] = a.accumulate ? y[i] + t : t;
            }
        }
    } else {
        for (int i = threadIdx.x; i < gd; i += RN_THREADS) {
            float t = x[i];
            if (gate) t *= silu_f(gate[i]);
            t *= inv;
            if (w) t *= a.plus_one ? 1.f + w[i] : w[i];
            y[i] = a.accumulate ? y[i] + t : t;
        }
    }
}

extern "C" int dl_rms_norm(const DlNormArgs* args, void* stream) {
    const DlNormArgs& a = *args;
    if (a.M < 1 || a.dim < 1 || a.groups < 1 || a.dim % a.groups != 0) { dl_set_error("dl_rms_norm: bad shape"); return -1; }
    if (a.accumulate && (const float*)a.y == a.x) { dl_set_error("dl_rms_norm: accumulate needs y != x"); return -1; }
    dim3 grid(a.M, a.groups);
    rms_norm_kernel<<<grid, RN_THREADS, 0, (cudaStream_t)stream>>>(a);
    LAYER_CHECK_LAUNCH("dl_rms_norm");
    return 0;
}
