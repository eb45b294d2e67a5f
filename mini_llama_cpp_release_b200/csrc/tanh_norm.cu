// The elementwise "dynamic tanh" norm, gated units, and a sigmoid gate on rows.
//
// Dynamic tanh: T(v) = tanh(a · v) · w + b, with one stored number a, a gain w and a bias b per entry; no mean and no variance
// are taken, so every entry stands alone.  One kernel covers the ways a block uses it around the float32 residual stream x:
//
//   branch given:        x <- x + m · Tb(branch)         (Tb: the norm on the branch's output; m: one number; without Tb the
//                                                          branch is added as it is)
//   next norm given:     out = Tn(x)                     (in the engine's type: what the next part reads)
//
// both in one pass when both are given.  The branch is float32 [n][d], or slices of partial sums that are added in order, or
// the rows of a token's experts (sum over its choices j of rows[row_of[t][j]], in the order of its choices; a negative row
// adds nothing).  All arithmetic is float32.
//
// Gated units: out = act(g) · u over rows [g | u] (or interleaved g0, u0, g1, u1, ...), with act one of
//   0  silu:  g · sigmoid(g)
//   1  the tanh form of GELU: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g³)))
//   2  clamped: g' = min(g, limit), u' = clamp(u, -limit, limit); out = g' · sigmoid(alpha · g') · (u' + 1)
#include "common.cuh"

namespace mlc {

struct TanhNormArgs {
    float* x;                   // [n][d] the stream, updated in place when a branch is given
    const float* y;             // branch: [slices][n][d], or null
    int n_slices;
    long long slice_stride;
    const float* rows;          // expert rows [.][d], or null
    const int* row_of;          // [n][top]
    int top;
    const float* b_gain;        // the branch norm's gain and bias [d] (null: the branch joins as it is)
    const float* b_bias;
    float b_alpha;
    float mult;
    const float* n_gain;        // the next norm's gain and bias [d] (null: no output)
    const float* n_bias;
    float n_alpha;
    int d;
    long long total;            // n · d
};

// tanh for the norm.  EXACT: the library's tanhf (the float32 engine).  Otherwise 1 - 2 / (1 + e^2v) with the fast exponential
// and division, whose absolute error stays at float32's rounding of one (1e-7): for an engine whose products take 16-bit
// operands, where the norm's output is rounded to 16 bits and the stream it is added to is of the order of one.
template <bool EXACT>
__device__ __forceinline__ float tanh_of(float v) {
    if constexpr (EXACT) return tanhf(v);
    else return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * v));
}

template <bool EXACT>
__device__ __forceinline__ float tanh_norm_one(float v, float alpha, float gain, float bias) { return fmaf(tanh_of<EXACT>(alpha * v), gain, bias); }

__device__ __forceinline__ void load_vec(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_vec(const float* p, float (&v)[1]) { v[0] = *p; }
__device__ __forceinline__ void store_vec(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store_vec(float* p, const float (&v)[1]) { *p = v[0]; }
__device__ __forceinline__ void store_vec(bf16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const unsigned*>(&lo), *reinterpret_cast<const unsigned*>(&hi));
}
__device__ __forceinline__ void store_vec(bf16* p, const float (&v)[1]) { *p = __float2bfloat16_rn(v[0]); }

// VEC entries a thread (4: 16-byte accesses, for rows whose length is a multiple of four; 1: steps of few rows, where more
// threads with one entry each have all their loads in flight at once).  A branch's slices are added in the order of the slices.
template <typename TOut, int VEC, bool EXACT>
__global__ void __launch_bounds__(256)
tanh_norm_kernel(TanhNormArgs a, TOut* __restrict__ out) {
    grid_launch_dependents();
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= a.total) return;
    const long long t = idx / a.d;
    const int c = (int)(idx - t * a.d);
    // the norms' own numbers depend on no kernel before this one
    float bg[VEC], bb[VEC], ng[VEC], nb[VEC];
    if (a.b_gain != nullptr) { load_vec(a.b_gain + c, bg); load_vec(a.b_bias + c, bb); }
    if (a.n_gain != nullptr) { load_vec(a.n_gain + c, ng); load_vec(a.n_bias + c, nb); }
    grid_dependency_wait();
    float xv[VEC];
    load_vec(a.x + idx, xv);
    const bool has_branch = a.y != nullptr || a.rows != nullptr;
    if (has_branch) {
        float br[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) br[k] = 0.0f;
        if (a.y != nullptr) {
            int s = 0;
            for (; s + 4 <= a.n_slices; s += 4) {                    // four slices' loads in flight together, added in order
                float p0[VEC], p1[VEC], p2[VEC], p3[VEC];
                load_vec(a.y + (long long)s * a.slice_stride + idx, p0);
                load_vec(a.y + (long long)(s + 1) * a.slice_stride + idx, p1);
                load_vec(a.y + (long long)(s + 2) * a.slice_stride + idx, p2);
                load_vec(a.y + (long long)(s + 3) * a.slice_stride + idx, p3);
#pragma unroll
                for (int k = 0; k < VEC; ++k) br[k] = (((br[k] + p0[k]) + p1[k]) + p2[k]) + p3[k];
            }
            for (; s < a.n_slices; ++s) {
                float p0[VEC];
                load_vec(a.y + (long long)s * a.slice_stride + idx, p0);
#pragma unroll
                for (int k = 0; k < VEC; ++k) br[k] += p0[k];
            }
        } else {
            for (int j = 0; j < a.top; ++j) {
                const int r = a.row_of[t * a.top + j];
                if (r < 0) continue;
                float p0[VEC];
                load_vec(a.rows + (long long)r * a.d + c, p0);
#pragma unroll
                for (int k = 0; k < VEC; ++k) br[k] += p0[k];
            }
        }
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
            const float nbr = a.b_gain != nullptr ? tanh_norm_one<EXACT>(br[k], a.b_alpha, bg[k], bb[k]) : br[k];
            xv[k] = fmaf(a.mult, nbr, xv[k]);
        }
        store_vec(a.x + idx, xv);
    }
    if (a.n_gain != nullptr) {
        float o[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) o[k] = tanh_norm_one<EXACT>(xv[k], a.n_alpha, ng[k], nb[k]);
        store_vec(out + idx, o);
    }
}

__device__ __forceinline__ float glu_one(float g, float u, int kind, float limit, float alpha) {
    if (kind == 0) return g / (1.0f + expf(-g)) * u;
    if (kind == 1) {
        // 0.5 g (1 + tanh(w)) = g / (1 + exp(-2w)): the same function without the sum that cancels for negative w
        const float w = 0.7978845608028654f * (g + 0.044715f * g * g * g);
        return g / (1.0f + expf(-2.0f * w)) * u;
    }
    const float gc = fminf(g, limit), uc = fminf(fmaxf(u, -limit), limit);
    return gc / (1.0f + expf(-alpha * gc)) * (uc + 1.0f);
}

template <typename TIn, typename TOut>
__global__ void glu_kernel(const TIn* __restrict__ gu, int inter, long long total, int interleaved, int kind, float limit,
                           float alpha, TOut* __restrict__ out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long n = idx / inter;
    const int i = (int)(idx % inter);
    const TIn* row = gu + n * 2 * inter;
    const float g = to_float(interleaved ? row[2 * i] : row[i]);
    const float u = to_float(interleaved ? row[2 * i + 1] : row[inter + i]);
    out[idx] = from_float<TOut>(glu_one(g, u, kind, limit, alpha));
}

// o[t][c] <- o[t][c] · sigmoid(gate[t][gate_col + c]), gate float32 rows; heads of `vdim` entries sit in rows of `D` entries
// (D >= vdim: the entries beyond a head's own stay as they are)
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ o, const float* __restrict__ gate, long long gate_stride, int heads, int vdim,
                                    int D, long long total) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int width = heads * vdim;
    const long long t = idx / width;
    const int c = (int)(idx - t * width);
    const int h = c / vdim, i = c - h * vdim;
    const float z = gate[t * gate_stride + c];
    T* p = o + (t * heads + h) * D + i;
    *p = from_float<T>(to_float(*p) / (1.0f + expf(-z)));
}

}  // namespace mlc

using namespace mlc;

// x float32 [n][d].  Branch: y float32 (n_slices slices of n·d floats) or rows/row_of/top, or neither.  b_gain/b_bias null: the
// branch is added as it is.  n_gain null: nothing is written to out.  out: [n][d] of out_dtype.
extern "C" int mlc_tanh_norm(float* x, const float* y, int n_slices, const float* rows, const int* row_of, int top,
                             const float* b_gain, const float* b_bias, float b_alpha, float mult, const float* n_gain,
                             const float* n_bias, float n_alpha, int n, int d, void* out, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || (y != nullptr && n_slices < 1) || (rows != nullptr && (row_of == nullptr || top < 1))) return MLC_ERR_BAD_SIZE;
    if (y != nullptr && rows != nullptr) return MLC_ERR_UNSUPPORTED;
    if ((b_gain == nullptr) != (b_bias == nullptr) || (n_gain == nullptr) != (n_bias == nullptr)) return MLC_ERR_BAD_SIZE;
    if (n_gain != nullptr && out == nullptr) return MLC_ERR_BAD_SIZE;
    TanhNormArgs a{x, y, n_slices, (long long)n * d, rows, row_of, top, b_gain, b_bias, b_alpha, mult, n_gain, n_bias, n_alpha, d,
                   (long long)n * d};
    cudaStream_t s = (cudaStream_t)stream;
    // 16-byte accesses for rows whose length allows them, unless the step is so small that one entry a thread fills more SMs
    const bool vec = (d & 3) == 0 && a.total >= (1 << 18) &&
                     ((((uintptr_t)x) | ((uintptr_t)y) | ((uintptr_t)rows) | ((uintptr_t)b_gain) | ((uintptr_t)b_bias) |
                       ((uintptr_t)n_gain) | ((uintptr_t)n_bias) | ((uintptr_t)out)) & 15) == 0;
    const long long items = vec ? a.total / 4 : a.total;
    const dim3 grid((unsigned)((items + 255) / 256)), block(256);
    cudaError_t e;
    // a float32 output is the float32 engine: the library's tanh; 16 bits out: the fast form (see tanh_of)
    if (out_dtype == MLC_DTYPE_F32 && n_gain != nullptr)
        e = vec ? launch_pdl(tanh_norm_kernel<float, 4, true>, grid, block, 0, s, a, (float*)out)
                : launch_pdl(tanh_norm_kernel<float, 1, true>, grid, block, 0, s, a, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16 && n_gain != nullptr)
        e = vec ? launch_pdl(tanh_norm_kernel<bf16, 4, false>, grid, block, 0, s, a, (bf16*)out)
                : launch_pdl(tanh_norm_kernel<bf16, 1, false>, grid, block, 0, s, a, (bf16*)out);
    else if (n_gain == nullptr)          // no output: the stream's update alone, with the library's tanh
        e = vec ? launch_pdl(tanh_norm_kernel<float, 4, true>, grid, block, 0, s, a, (float*)nullptr)
                : launch_pdl(tanh_norm_kernel<float, 1, true>, grid, block, 0, s, a, (float*)nullptr);
    else
        return MLC_ERR_BAD_DTYPE;
    return e == cudaSuccess ? 0 : (int)e;
}

extern "C" int mlc_glu(const void* gate_up, int in_dtype, int n, int inter, int interleaved, int kind, float limit, float alpha,
                       void* out, int out_dtype, void* stream) {
    if (n <= 0) return 0;
    if (inter <= 0 || kind < 0 || kind > 2 || (kind == 2 && !(limit > 0.0f))) return MLC_ERR_BAD_SIZE;
    const long long total = (long long)n * inter;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == MLC_DTYPE_F32 && out_dtype == MLC_DTYPE_F32)
        glu_kernel<float, float><<<blocks, 256, 0, s>>>((const float*)gate_up, inter, total, interleaved, kind, limit, alpha, (float*)out);
    else if (in_dtype == MLC_DTYPE_F32 && out_dtype == MLC_DTYPE_BF16)
        glu_kernel<float, bf16><<<blocks, 256, 0, s>>>((const float*)gate_up, inter, total, interleaved, kind, limit, alpha, (bf16*)out);
    else if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_BF16)
        glu_kernel<bf16, bf16><<<blocks, 256, 0, s>>>((const bf16*)gate_up, inter, total, interleaved, kind, limit, alpha, (bf16*)out);
    else if (in_dtype == MLC_DTYPE_BF16 && out_dtype == MLC_DTYPE_F32)
        glu_kernel<bf16, float><<<blocks, 256, 0, s>>>((const bf16*)gate_up, inter, total, interleaved, kind, limit, alpha, (float*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_sigmoid_gate(void* o, int dtype, const float* gate, long long gate_stride, int n, int heads, int vdim, int D,
                                void* stream) {
    if (n <= 0) return 0;
    if (heads <= 0 || vdim <= 0 || D < vdim) return MLC_ERR_BAD_SIZE;
    const long long total = (long long)n * heads * vdim;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MLC_DTYPE_F32)
        sigmoid_gate_kernel<float><<<blocks, 256, 0, s>>>((float*)o, gate, gate_stride, heads, vdim, D, total);
    else if (dtype == MLC_DTYPE_BF16)
        sigmoid_gate_kernel<bf16><<<blocks, 256, 0, s>>>((bf16*)o, gate, gate_stride, heads, vdim, D, total);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}
