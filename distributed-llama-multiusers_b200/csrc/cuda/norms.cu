// RMS normalisation in its variants, all in f32:  y = v / sqrt(mean(v^2) + eps) * scale
//   * scale = w  or  (1 + w)  (a weight stored around zero)  or 1 (no weight);
//   * the row may be normalised in `groups` equal parts, each by its own root mean square;
//   * v = x  or  x * silu(gate)  (a gate applied before the norm);
//   * the result is stored, or added to what y holds (a norm on a sublayer's output, summed into the residual stream);
//   * an optional row map gathers source rows (the final norm of the rows whose logits are wanted).
// One CTA per (row, group).
#include "layer_common.cuh"
#include "../../../include/dllama_b200.h"

__global__ void __launch_bounds__(256) rms_norm_kernel(DlNormArgs a) {
    __shared__ float red[32];
    const int m = blockIdx.x, g = blockIdx.y;
    const int src = a.rows ? a.rows[m] : m;
    const int gd = a.dim / a.groups;
    const float* x = a.x + (size_t)src * a.ldx + (size_t)g * gd;
    const float* gate = a.gate ? a.gate + (size_t)src * a.ld_gate + (size_t)g * gd : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < gd; i += blockDim.x) {
        float v = x[i];
        if (gate) v *= silu_f(gate[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)gd + a.eps);
    float* y = a.y + (size_t)m * a.ldy + (size_t)g * gd;
    const float* w = a.w ? a.w + (size_t)g * gd : nullptr;
    for (int i = threadIdx.x; i < gd; i += blockDim.x) {
        float v = x[i];
        if (gate) v *= silu_f(gate[i]);
        v *= inv;
        if (w) v *= a.plus_one ? 1.f + w[i] : w[i];
        y[i] = a.accumulate ? y[i] + v : v;
    }
}

extern "C" int dl_rms_norm(const DlNormArgs* args, void* stream) {
    const DlNormArgs& a = *args;
    if (a.M < 1 || a.dim < 1 || a.groups < 1 || a.dim % a.groups != 0) { dl_set_error("dl_rms_norm: bad shape"); return -1; }
    if (a.accumulate && (const float*)a.y == a.x) { dl_set_error("dl_rms_norm: accumulate needs y != x"); return -1; }
    dim3 grid(a.M, a.groups);
    rms_norm_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    LAYER_CHECK_LAUNCH("dl_rms_norm");
    return 0;
}
