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
// the step.  Forms of the same arithmetic: `group_norm_rows_kernel` (rows of up to 4,096 entries in fours: the row stays in
// registers, see there), `group_norm_kernel<4, .>` moves four neighbouring entries per access (16-byte
// loads of every operand issued before any is used; rows, strides and parts that are multiples of four entries on
// 16-byte boundaries), `group_norm_kernel<1, .>` takes every other size one entry at a time.
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

// V entries of one operand at element offset `at`.
template <int V> struct Pack { float e[V]; };

template <int V>
__device__ __forceinline__ Pack<V> load_pack(const float* p, long long at) {
    Pack<V> r;
    if constexpr (V == 4) {
        const float4 q = *reinterpret_cast<const float4*>(p + at);
        r.e[0] = q.x; r.e[1] = q.y; r.e[2] = q.z; r.e[3] = q.w;
    } else {
        r.e[0] = p[at];
    }
    return r;
}

template <int V>
__device__ __forceinline__ Pack<V> load_pack_any(const void* p, int dtype, long long at) {
    if (dtype == MLC_DTYPE_F32) return load_pack<V>((const float*)p, at);
    Pack<V> r;
    if constexpr (V == 4) {
        const uint2 q = *reinterpret_cast<const uint2*>((const bf16*)p + at);
        const bf16* h = reinterpret_cast<const bf16*>(&q);
#pragma unroll
        for (int k = 0; k < 4; ++k) r.e[k] = to_float(h[k]);
    } else {
        r.e[0] = to_float(((const bf16*)p)[at]);
    }
    return r;
}

template <int V>
__device__ __forceinline__ void store_pack(const Pack<V>& r, float* xw, void* out, int out_dtype, long long x_at, long long out_at) {
    if constexpr (V == 4) {
        if (xw != nullptr) *reinterpret_cast<float4*>(xw + x_at) = make_float4(r.e[0], r.e[1], r.e[2], r.e[3]);
        if (out != nullptr) {
            if (out_dtype == MLC_DTYPE_F32) {
                *reinterpret_cast<float4*>((float*)out + out_at) = make_float4(r.e[0], r.e[1], r.e[2], r.e[3]);
            } else {
                uint2 q;
                bf16* h = reinterpret_cast<bf16*>(&q);
#pragma unroll
                for (int k = 0; k < 4; ++k) h[k] = from_float<bf16>(r.e[k]);
                *reinterpret_cast<uint2*>((bf16*)out + out_at) = q;
            }
        }
    } else {
        if (xw != nullptr) xw[x_at] = r.e[0];
        if (out != nullptr) {
            if (out_dtype == MLC_DTYPE_F32) ((float*)out)[out_at] = r.e[0];
            else ((bf16*)out)[out_at] = from_float<bf16>(r.e[0]);
        }
    }
}

constexpr int GN_MAX_TOP = 4;        // a token's expert rows loaded side by side; more are taken in rounds of this many

// Entries i .. i + V - 1 of row t before the norm: alpha · x + s ⊙ branch (x itself without a branch).
// EXPERTS: the branch is the weighted sum of expert rows (a form of its own: the rows held side by side cost registers
// that the other forms, which run far more often, then do not pay for with fewer rows in flight per SM).
template <int V, bool EXPERTS>
__device__ __forceinline__ Pack<V> summed_entries(const GroupNormArgs& a, const float* xr, int t, int i) {
    const int d = a.d;
    const bool has_branch = EXPERTS || a.y != nullptr;
    Pack<V> val = load_pack<V>(xr, i);
    if (has_branch) {
        Pack<V> b, zz, zb;
        const bool gated = a.z != nullptr;
        if (gated) {                               // the gate's operands first: their loads overlap the branch's
            zz = load_pack<V>(a.z, (long long)t * a.z_stride + i);
            if (a.z_bias != nullptr) zb = load_pack<V>(a.z_bias, i);
        }
#pragma unroll
        for (int k = 0; k < V; ++k) b.e[k] = 0.0f;
        if constexpr (!EXPERTS) {
            int s = 0;
            for (; s + 4 <= a.slices; s += 4) {    // four slices' loads in flight, added in slice order
                Pack<V> p[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) p[u] = load_pack<V>(a.y, ((long long)(s + u) * a.n + t) * d + i);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int k = 0; k < V; ++k) b.e[k] += p[u].e[k];
            }
            for (; s < a.slices; ++s) {
                const Pack<V> p = load_pack<V>(a.y, ((long long)s * a.n + t) * d + i);
#pragma unroll
                for (int k = 0; k < V; ++k) b.e[k] += p.e[k];
            }
        } else {
            for (int j0 = 0; j0 < a.top; j0 += GN_MAX_TOP) {
                Pack<V> p[GN_MAX_TOP];
                float w[GN_MAX_TOP];
#pragma unroll
                for (int u = 0; u < GN_MAX_TOP; ++u) {
                    const int j = j0 + u;
                    w[u] = 0.0f;
#pragma unroll
                    for (int k = 0; k < V; ++k) p[u].e[k] = 0.0f;
                    if (j < a.top) {
                        const int r = a.row_of[(long long)t * a.top + j];
                        w[u] = a.weights[(long long)t * a.top + j];
                        if (r >= 0) p[u] = load_pack<V>(a.rows, (long long)r * d + i);
                        else if (a.ident != nullptr) p[u] = load_pack_any<V>(a.ident, a.ident_dtype, (long long)t * d + i);
                    }
                }
#pragma unroll
                for (int u = 0; u < GN_MAX_TOP; ++u)
                    if (j0 + u < a.top)
#pragma unroll
                        for (int k = 0; k < V; ++k) b.e[k] = fmaf(w[u], p[u].e[k], b.e[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < V; ++k) {
            float bk = b.e[k];
            if (gated) bk *= 1.0f / (1.0f + expf(-(zz.e[k] + (a.z_bias != nullptr ? zb.e[k] : 0.0f))));
            val.e[k] = fmaf(a.alpha, val.e[k], bk);
        }
    }
    return val;
}

template <int V, bool EXPERTS>
__global__ void __launch_bounds__(512, 3) group_norm_kernel(GroupNormArgs a) {
    extern __shared__ __align__(16) float v[];        // [d]
    __shared__ float part[32];
    const int t = blockIdx.x;
    const int d = a.d;
    const float* xr = a.x + (long long)t * a.x_stride;
    for (int i = threadIdx.x * V; i < d; i += blockDim.x * V) {
        const Pack<V> val = summed_entries<V, EXPERTS>(a, xr, t, i);
#pragma unroll
        for (int k = 0; k < V; ++k) v[i + k] = val.e[k];
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int gsize = d / a.groups;
    int wpg = n_warps / a.groups;                     // warps that share a group
    if (wpg < 1) wpg = 1;
    while (wpg > 1 && (wpg - 1) * 32 * V >= gsize) --wpg; // no warp without entries
    const int at_once = n_warps / wpg;                // groups handled side by side
    const int sub = warp % wpg, team = warp / wpg;
    for (int g0 = 0; g0 < a.groups; g0 += at_once) {
        const int g = g0 + team;
        const bool live = team < at_once && g < a.groups;
        float ss = 0.0f;
        if (live)
            for (int j = (sub * 32 + lane) * V; j < gsize; j += wpg * 32 * V) {
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const float e = v[g * gsize + j + k];
                    ss = fmaf(e, e, ss);
                }
            }
        ss = warp_sum(ss);
        __syncthreads();
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        if (live) {
            float total = 0.0f;
            for (int k = 0; k < wpg; ++k) total += part[team * wpg + k];
            const float f = 1.0f / sqrtf(total / (float)gsize + a.eps);
            for (int j = (sub * 32 + lane) * V; j < gsize; j += wpg * 32 * V) {
                const int i = g * gsize + j;
                const Pack<V> gn = load_pack<V>(a.gain, i % a.gain_len);
                Pack<V> r;
#pragma unroll
                for (int k = 0; k < V; ++k) r.e[k] = v[i + k] * f * gn.e[k];
                store_pack<V>(r, a.write_x ? a.x : nullptr, a.out, a.out_dtype, (long long)t * a.x_stride + i, (long long)t * d + i);
            }
        }
    }
}

// The same norm with the row held in registers: thread th keeps the NP packs of four entries th, th + threads, ... of
// the row, so the row is read once and nothing but one sum of squares per pack goes through shared memory.  Warp w sums
// the packs of groups w, w + warps, ... (a lane a strided share in order, then the warp's tree), so a group's statistic is
// formed in an order that only the row's length and the number of groups fix.  Rows of up to 4 · NP · 512 entries.
template <int NP, bool EXPERTS>
__global__ void __launch_bounds__(512, 3) group_norm_rows_kernel(GroupNormArgs a) {
    extern __shared__ __align__(16) float v[];        // [d / 4] sums of squares of the packs, then [groups] factors
    const int t = blockIdx.x;
    const int d = a.d, packs = d >> 2;
    const float* xr = a.x + (long long)t * a.x_stride;
    Pack<4> val[NP];
#pragma unroll
    for (int u = 0; u < NP; ++u) {
        const int p = threadIdx.x + u * blockDim.x;
        if (p < packs) {
            val[u] = summed_entries<4, EXPERTS>(a, xr, t, p << 2);
            float ss = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) ss = fmaf(val[u].e[k], val[u].e[k], ss);
            v[p] = ss;
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int gsize = d / a.groups, ppg = gsize >> 2;
    float* factor = v + packs;
    for (int g = warp; g < a.groups; g += n_warps) {
        float ss = 0.0f;
        for (int j = lane; j < ppg; j += 32) ss += v[g * ppg + j];
        ss = warp_sum(ss);
        if (lane == 0) factor[g] = 1.0f / sqrtf(ss / (float)gsize + a.eps);
    }
    __syncthreads();
#pragma unroll
    for (int u = 0; u < NP; ++u) {
        const int p = threadIdx.x + u * blockDim.x;
        if (p < packs) {
            const int i = p << 2;
            const float f = factor[i / gsize];
            const Pack<4> gn = load_pack<4>(a.gain, i % a.gain_len);
            Pack<4> r;
#pragma unroll
            for (int k = 0; k < 4; ++k) r.e[k] = val[u].e[k] * f * gn.e[k];
            store_pack<4>(r, a.write_x ? a.x : nullptr, a.out, a.out_dtype, (long long)t * a.x_stride + i, (long long)t * d + i);
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
    const int gsize = d / groups;
    auto aligned = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const bool by_four = gsize % 4 == 0 && gain_len % 4 == 0 && x_stride % 4 == 0 && (z == nullptr || z_stride % 4 == 0) &&
                         aligned(x) && aligned(gain) && aligned(y) && aligned(rows) && aligned(ident) && aligned(z) &&
                         aligned(z_bias) && aligned(out);
    if (by_four && d <= 4096) {
        // the row in registers: one pack of four entries a thread up to 512 threads, two beyond
        const int packs = d / 4, np = packs <= 512 ? 1 : 2;
        int threads = (((packs + np - 1) / np + 31) / 32) * 32;
        threads = threads < 32 ? 32 : threads;
        const size_t shared = (size_t)(packs + groups) * sizeof(float);
        auto kernel = rows != nullptr ? (np == 1 ? group_norm_rows_kernel<1, true> : group_norm_rows_kernel<2, true>)
                                      : (np == 1 ? group_norm_rows_kernel<1, false> : group_norm_rows_kernel<2, false>);
        kernel<<<n, threads, shared, (cudaStream_t)stream>>>(a);
    } else if (by_four) {
        int threads = ((d / 4 + 31) / 32) * 32;        // a thread per four entries, up to 512 threads a row
        threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
        (rows != nullptr ? group_norm_kernel<4, true> : group_norm_kernel<4, false>)<<<n, threads, (size_t)d * sizeof(float), (cudaStream_t)stream>>>(a);
    } else {
        const int threads = d <= 256 ? 64 : (d <= 1024 ? 128 : 256);
        (rows != nullptr ? group_norm_kernel<1, true> : group_norm_kernel<1, false>)<<<n, threads, (size_t)d * sizeof(float), (cudaStream_t)stream>>>(a);
    }
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
