// RMS norm in groups, alone or behind a gated residual sum.
//
//   groups:  a row of d entries is cut into G equal consecutive parts; part g is divided by sqrt(mean(part²) + eps) of
//            its own, and the whole row is multiplied by the gain (gain index i mod gain_len: a gain as long as the row,
//            or one as long as a part that all parts share).  G = 1 is the ordinary RMS norm.
//   sum:     before the norm, v = alpha · x + s ⊙ b with
//              b  the branch's output: float32 [slices][n][d] added up in order, or the weighted sum of a token's expert
//                 rows  sum_j weight[t][j] · rows[row_of[t][j]]  (a negative row: the token's own input, `ident`),
//              s  = sigmoid(z + bias) per entry when gate logits z are given, else one.
//            Without a branch v = x.
//   stores:  the normed row goes back into x (float32, in place) and/or into `out` in its own type.
//
// Everything is float32.  A block per row: the row's v is staged in shared memory, then every group is summed by a fixed
// set of warps (a group's warps add their parts in a fixed order), so a row's result does not depend on what else is in
// the step.
#include "common.cuh"

namespace mlc {

struct GroupNormArgs {
    float* x;                   // [n] rows of d, stride x_stride; read, and written when write_x
    long long x_stride;
    int n, d, groups;
    const float* gain;
    int gain_len;
    float eps, alpha;
    const float* y;             // [slices][n][d] or null
    int slices;
    const float* rows;          // expert rows [.][d] or null
    const int* row_of;          // [n][top]
    const float* weights;       // [n][top]
    int top;
    const void* ident;          // [n][d] in ident_dtype, or null
    int ident_dtype;
    const float* z;             // gate logits, row stride z_stride, or null
    long long z_stride;
    const float* z_bias;        // [d] or null
    int write_x;
    void* out;                  // [n][d] or null
    int out_dtype;
};

__global__ void group_norm_kernel(GroupNormArgs a) {
    extern __shared__ float v[];                      // [d]
    __shared__ float part[32];
    const int t = blockIdx.x;
    const int d = a.d;
    const float* xr = a.x + (long long)t * a.x_stride;
    const bool has_branch = a.y != nullptr || a.rows != nullptr;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float val = xr[i];
        if (has_branch) {
            float b = 0.0f;
            if (a.y != nullptr) {
                for (int s = 0; s < a.slices; ++s) b += a.y[((long long)s * a.n + t) * d + i];
            } else {
                for (int j = 0; j < a.top; ++j) {
                    const int r = a.row_of[(long long)t * a.top + j];
                    float e;
                    if (r >= 0) e = a.rows[(long long)r * d + i];
                    else if (a.ident == nullptr) e = 0.0f;
                    else e = a.ident_dtype == MLC_DTYPE_F32 ? ((const float*)a.ident)[(long long)t * d + i]
                                                            : to_float(((const bf16*)a.ident)[(long long)t * d + i]);
                    b = fmaf(a.weights[(long long)t * a.top + j], e, b);
                }
            }
            if (a.z != nullptr) {
                const float zz = a.z[(long long)t * a.z_stride + i] + (a.z_bias != nullptr ? a.z_bias[i] : 0.0f);
                b *= 1.0f / (1.0f + expf(-zz));
            }
            val = fmaf(a.alpha, val, b);
        }
        v[i] = val;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int gsize = d / a.groups;
    int wpg = n_warps / a.groups;                     // warps that share a group
    if (wpg < 1) wpg = 1;
    while (wpg > 1 && (wpg - 1) * 32 >= gsize) --wpg; // no warp without entries
    const int at_once = n_warps / wpg;                // groups handled side by side
    const int sub = warp % wpg, team = warp / wpg;
    for (int g0 = 0; g0 < a.groups; g0 += at_once) {
        const int g = g0 + team;
        const bool live = team < at_once && g < a.groups;
        float ss = 0.0f;
        if (live)
            for (int j = sub * 32 + lane; j < gsize; j += wpg * 32) {
                const float e = v[g * gsize + j];
                ss = fmaf(e, e, ss);
            }
        ss = warp_sum(ss);
        __syncthreads();
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        if (live) {
            float total = 0.0f;
            for (int k = 0; k < wpg; ++k) total += part[team * wpg + k];
            const float f = 1.0f / sqrtf(total / (float)gsize + a.eps);
            for (int j = sub * 32 + lane; j < gsize; j += wpg * 32) {
                const int i = g * gsize + j;
                const float r = v[i] * f * a.gain[i % a.gain_len];
                if (a.write_x) a.x[(long long)t * a.x_stride + i] = r;
                if (a.out != nullptr) {
                    if (a.out_dtype == MLC_DTYPE_F32) ((float*)a.out)[(long long)t * d + i] = r;
                    else ((bf16*)a.out)[(long long)t * d + i] = from_float<bf16>(r);
                }
            }
        }
    }
}

// out = act(in), elementwise: 0 silu, 1 gelu (erf), 2 gelu with the tanh approximation.  float32 arithmetic.
template <typename TI, typename TO>
__global__ void activation_kernel(const TI* __restrict__ in, long long total, int kind, TO* __restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float z = to_float(in[i]);
    float r;
    if (kind == 0) r = z / (1.0f + expf(-z));
    else if (kind == 1) r = 0.5f * z * (1.0f + erff(z * 0.70710678118654752440f));
    else r = 0.5f * z * (1.0f + tanhf(0.79788456080286535588f * (z + 0.044715f * z * z * z)));
    out[i] = from_float<TO>(r);
}

}  // namespace mlc

using namespace mlc;

extern "C" int mlc_group_norm(float* x, long long x_stride, int n, int d, int groups, const float* gain, int gain_len, float eps,
                              float alpha, const float* y, int slices, const float* rows, const int* row_of,
                              const float* weights, int top, const void* ident, int ident_dtype, const float* z,
                              long long z_stride, const float* z_bias, int write_x, void* out, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || groups <= 0 || d % groups != 0 || gain_len <= 0 || d % gain_len != 0 || d > 12288) return MLC_ERR_BAD_SIZE;
    if (y != nullptr && slices < 1) return MLC_ERR_BAD_SIZE;
    if (rows != nullptr && (row_of == nullptr || weights == nullptr || top < 1)) return MLC_ERR_BAD_SIZE;
    if (out != nullptr && out_dtype != MLC_DTYPE_F32 && out_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    if (ident != nullptr && ident_dtype != MLC_DTYPE_F32 && ident_dtype != MLC_DTYPE_BF16) return MLC_ERR_BAD_DTYPE;
    GroupNormArgs a{x, x_stride, n, d, groups, gain, gain_len, eps, alpha, y, slices, rows, row_of, weights, top, ident,
                    ident_dtype, z, z_stride, z_bias, write_x, out, out_dtype};
    const int threads = d <= 256 ? 64 : (d <= 1024 ? 128 : 256);
    group_norm_kernel<<<n, threads, (size_t)d * sizeof(float), (cudaStream_t)stream>>>(a);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_activation(const void* in, int in_dtype, long long total, int kind, void* out, int out_dtype, void* stream) {
    if (total <= 0) return 0;
    if (kind < 0 || kind > 2) return MLC_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    const int code = in_dtype * 2 + out_dtype;
    switch (code) {
        case 0: activation_kernel<float, float><<<blocks, 256, 0, s>>>((const float*)in, total, kind, (float*)out); break;
        case 1: activation_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)in, total, kind, (bf16*)out); break;
        case 2: activation_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)in, total, kind, (float*)out); break;
        case 3: activation_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((const bf16*)in, total, kind, (bf16*)out); break;
        default: return MLC_ERR_BAD_DTYPE;
    }
    MLC_LAUNCH_CHECK();
    return 0;
}
