// Gated linear attention: a matrix memory per head with a decay per key channel.
//
//   a_t = sigmoid(z_t)^(1/tau) = exp(logsigmoid(z_t) / tau)              (per head and key channel, float32)
//   S_t = diag(a_t) S_{t-1} + k_t v_tᵀ,     o_t = S_tᵀ (q_t · dim^-1/2)   (S: [dim][vdim] per head, float32)
//
// The state starts at zero, lives in float32 and is carried per sequence in a slot's row; decays, their logarithms
// and everything else that enters the recurrence are float32 whatever the engine's type.
//
// Two kernels.  The first turns every decay logit into its decay in place, all tokens and channels at once.  The second
// walks: a block owns (sequence, head, 16 columns of S, a slab of its rows); a thread holds two columns x an eighth of
// the slab's rows (side by side) in registers.  Key channels do not meet until the output's sum over them, so the rows
// of S can be shared out over blocks: each row slab writes its partial outputs into a slice of its own, and whoever reads
// the outputs adds the slices up in order.  The host picks the slab so that a step has blocks enough to fill the GPU (a
// prompt of one sequence: narrow slabs; a decode step of many sequences: the whole head, one slice).  Tokens arrive sixteen at a time through shared memory while the next sixteen are on their way
// from memory into registers, and are walked four at a time: a row's state takes one multiply-add per token, and the
// four tokens' output sums, with their three shuffles each, are independent of one another and overlap; their results
// are stored behind the group.  The small blocks are many (heads x vdim / 16 per sequence), so that a prompt of one
// sequence still spreads over the GPU.  Tokens that are not there count as q = k = v = 0 with a
// decay of one.  State layout in a slot's row: [head][column][row] (a column's rows side by side).
#include "common.cuh"

namespace mlc {

constexpr int GLA_CHUNK = 16;      // tokens staged at a time
constexpr int GLA_COLS = 16;       // columns of S per block
constexpr int GLA_THREADS = 64;    // 8 pairs of columns x 8 groups of rows
constexpr int GLA_V_LOADS = GLA_CHUNK * GLA_COLS / GLA_THREADS;

struct GlaArgs {
    const float* qk;            // rows that hold q (at q_col) and k (at k_col)
    long long qk_stride;
    const float* vsrc;          // rows that hold v (at v_col); may be the same matrix
    long long v_stride;
    int q_col, k_col, v_col;
    const float* decay;         // [n][H*dim] decays
    float q_scale;
    float* state;               // [slots][H*vdim*dim]
    long long state_stride;
    const int* slots;
    const int* cu_seqlens;
    float* out;                 // [row slabs][n][H*vdim]
    long long out_slice;        // floats between the slices of two row slabs
    int H, dim, vdim;
    int col_slabs;
    // a state-space layer's use of the walk: `qk_share` heads in a row read the same q and k (head h reads group h / qk_share;
    // 1: every head its own), `head_decay` [n][H] is one decay per token and head for all of a head's rows (then `decay` is
    // not read), `v_scale` [n][H] multiplies the head's v as it is read.  Null: the ordinary forms.
    int qk_share;
    const float* head_decay;
    const float* v_scale;
};

// z <- sigmoid(z + bias)^(1/tau) = exp(logsigmoid(z + bias) / tau),  logsigmoid(x) = min(x, 0) - log1p(exp(-|x|))
__global__ void gla_decay_kernel(float* __restrict__ z, const float* __restrict__ bias, long long total, int width, float inv_tau) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const float x = z[idx] + (bias != nullptr ? bias[idx % width] : 0.0f);
    z[idx] = expf((fminf(x, 0.0f) - log1pf(expf(-fabsf(x)))) * inv_tau);
}

// The forget-gate form (the HGRN2 design): the
// decay of a key channel is a forget gate with a lower bound, and what is written through that channel is its complement:
//   f = l + (1 - l) · sigmoid(z_f + b),   S_t = diag(f_t) S_{t-1} + (1 - f_t) v_tᵀ,   o_t = S_tᵀ silu(z_q)
// which is the walk above with decay f, key 1 - f, query silu(z_q) and no scale.  This kernel makes the three from the
// rows of the input product: qk [n][2·HD] = [silu(z_q) | (1 - l) · sigmoid(-(z_f + b))], decay [n][HD] = f.  The key is formed as
// (1 - l)(1 - sigmoid), not as 1 - f: a gate close to one would leave 1 - f with few digits.
__global__ void forget_gates_kernel(const float* __restrict__ proj, long long stride, int q_col, int f_col,
                                    const float* __restrict__ f_bias, const float* __restrict__ lower, long long total, int width,
                                    float* __restrict__ qk, float* __restrict__ decay) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / width;
    const int c = (int)(idx - t * width);
    const float* row = proj + t * stride;
    const float zq = row[q_col + c];
    const float zf = row[f_col + c] + (f_bias != nullptr ? f_bias[c] : 0.0f);
    const float l = lower != nullptr ? lower[c] : 0.0f;
    const float e = expf(-fabsf(zf));                 // sigmoid(zf) and sigmoid(-zf) without overflow
    const float big = 1.0f / (1.0f + e), small = e / (1.0f + e);
    const float sig = zf >= 0.0f ? big : small, co = zf >= 0.0f ? small : big;
    qk[t * 2 * width + c] = zq / (1.0f + expf(-zq));
    qk[t * 2 * width + width + c] = (1.0f - l) * co;
    decay[idx] = l + (1.0f - l) * sig;
}

// ROWS floats from 8- or 16-byte aligned shared memory
template <int ROWS>
__device__ __forceinline__ void load_rows(const float* p, float (&v)[ROWS]) {
    if (ROWS == 2) {
        const float2 t = *reinterpret_cast<const float2*>(p);
        v[0] = t.x; v[1 % ROWS] = t.y;
    } else {
#pragma unroll
        for (int i4 = 0; i4 < ROWS / 4; ++i4) {
            const float4 t = reinterpret_cast<const float4*>(p)[i4];
            v[(4 * i4) % ROWS] = t.x; v[(4 * i4 + 1) % ROWS] = t.y; v[(4 * i4 + 2) % ROWS] = t.z; v[(4 * i4 + 3) % ROWS] = t.w;
        }
    }
}

template <int ROWS>       // rows of a column one thread holds, side by side: a block's slab has DP = 8 * ROWS rows
__global__ void __launch_bounds__(GLA_THREADS)
gla_walk_kernel(GlaArgs a) {
    constexpr int DP = 8 * ROWS;
    constexpr int U = GLA_CHUNK * DP / GLA_THREADS;  // q, k, decay logits a thread brings per chunk
    extern __shared__ __align__(16) float sh[];
    float* qs = sh;                                  // [CHUNK][DP] q · dim^-1/2
    float* ks = qs + GLA_CHUNK * DP;                 // [CHUNK][DP]
    float* as = ks + GLA_CHUNK * DP;                 // [CHUNK][DP] decays
    float* vs = as + GLA_CHUNK * DP;                 // [CHUNK][COLS]
    const int dim = a.dim, vdim = a.vdim;
    const int head = blockIdx.x, seq = blockIdx.y, col0 = (blockIdx.z % a.col_slabs) * GLA_COLS;
    const int slab = blockIdx.z / a.col_slabs, row0 = slab * DP;           // the block's rows of S: row0 .. row0 + DP - 1
    const int tid = threadIdx.x;
    const int r = tid & 7, cp = tid >> 3;
    const int col = col0 + 2 * cp;
    const int t0 = a.cu_seqlens[seq], t1 = a.cu_seqlens[seq + 1];
    float* S_base = a.state + (long long)a.slots[seq] * a.state_stride + (long long)head * vdim * dim;
    float S[2][ROWS];
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int row = row0 + r * ROWS + i;
            S[c][i] = (col + c < vdim && row < dim) ? S_base[(long long)(col + c) * dim + row] : 0.0f;
        }

    float rq[U], rk[U], ra[U], rv[GLA_V_LOADS];
    auto fetch = [&](int c0) {
        const int n_here = min(GLA_CHUNK, t1 - c0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = tid + u * GLA_THREADS;
            const int tt = idx / DP, d = idx % DP;
            rq[u] = rk[u] = 0.0f;
            ra[u] = 1.0f;                             // no token, or no such channel: a decay of one, q and k zero
            if (tt < n_here && row0 + d < dim) {
                const float* row = a.qk + (long long)(c0 + tt) * a.qk_stride + (head / a.qk_share) * dim + row0 + d;
                rq[u] = row[a.q_col];
                rk[u] = row[a.k_col];
                ra[u] = a.head_decay != nullptr ? a.head_decay[(long long)(c0 + tt) * a.H + head]
                                                : a.decay[(long long)(c0 + tt) * a.H * dim + head * dim + row0 + d];
            }
        }
#pragma unroll
        for (int u = 0; u < GLA_V_LOADS; ++u) {
            const int idx = tid + u * GLA_THREADS;
            const int tt = idx / GLA_COLS, cc = idx % GLA_COLS;
            rv[u] = (tt < n_here && col0 + cc < vdim) ? a.vsrc[(long long)(c0 + tt) * a.v_stride + a.v_col + head * vdim + col0 + cc] : 0.0f;
            if (a.v_scale != nullptr && tt < n_here) rv[u] *= a.v_scale[(long long)(c0 + tt) * a.H + head];
        }
    };
    if (t0 < t1) fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += GLA_CHUNK) {
        const int n_here = min(GLA_CHUNK, t1 - c0);
        __syncthreads();                              // the chunk before has been read
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = tid + u * GLA_THREADS;
            qs[idx] = rq[u] * a.q_scale;
            ks[idx] = rk[u];
            as[idx] = ra[u];
        }
#pragma unroll
        for (int u = 0; u < GLA_V_LOADS; ++u) vs[tid + u * GLA_THREADS] = rv[u];
        __syncthreads();
        if (c0 + GLA_CHUNK < t1) fetch(c0 + GLA_CHUNK);       // in flight while this chunk is walked
        // groups of four tokens (a single token, a decode step, is a group of one)
        const int group = n_here == 1 ? 1 : 4;
        for (int g0 = 0; g0 < n_here; g0 += group) {
            float res0[4], res1[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (u >= group) break;
                const int t = g0 + u;
                const float2 v2 = *reinterpret_cast<const float2*>(vs + t * GLA_COLS + 2 * cp);
                float qv[ROWS], kv[ROWS], av[ROWS];
                load_rows<ROWS>(qs + t * DP + r * ROWS, qv);
                load_rows<ROWS>(ks + t * DP + r * ROWS, kv);
                load_rows<ROWS>(as + t * DP + r * ROWS, av);
                float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
                for (int e = 0; e < ROWS; ++e) {
                    S[0][e] = fmaf(av[e], S[0][e], kv[e] * v2.x);
                    S[1][e] = fmaf(av[e], S[1][e], kv[e] * v2.y);
                    acc0 = fmaf(S[0][e], qv[e], acc0);
                    acc1 = fmaf(S[1][e], qv[e], acc1);
                }
                res0[u] = acc0;
                res1[u] = acc1;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (u >= group) break;
                res0[u] += __shfl_xor_sync(0xffffffffu, res0[u], 1); res1[u] += __shfl_xor_sync(0xffffffffu, res1[u], 1);
                res0[u] += __shfl_xor_sync(0xffffffffu, res0[u], 2); res1[u] += __shfl_xor_sync(0xffffffffu, res1[u], 2);
                res0[u] += __shfl_xor_sync(0xffffffffu, res0[u], 4); res1[u] += __shfl_xor_sync(0xffffffffu, res1[u], 4);
            }
            if (r == 0) {
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (u >= group || g0 + u >= n_here) break;
                    float* o = a.out + slab * a.out_slice + (long long)(c0 + g0 + u) * a.H * vdim + head * vdim + col;
                    if (col < vdim) o[0] = res0[u];
                    if (col + 1 < vdim) o[1] = res1[u];
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int row = row0 + r * ROWS + i;
            if (col + c < vdim && row < dim) S_base[(long long)(col + c) * dim + row] = S[c][i];
        }
}


// The state-space layer ("Mamba-2"; Dao and Gu, "Transformers are SSMs: Generalized Models and Efficient Algorithms Through
// Structured State Space Duality"): per head a state S [N][vdim] with one decay per token and head,
//   dt = softplus(z_dt + bias),   S_t = exp(-exp(A_log) · dt) S_{t-1} + dt · B_t x_tᵀ,   y_t = S_tᵀ C_t + D x_t
// which is the walk above with decay exp(-exp(A_log) dt) for all rows of a head, key B and query C of the head's group, value
// dt · x.  This kernel makes dt and the decay per (token, head), float32, with no clamp:
// softplus(v) = max(v, 0) + log1p(exp(-|v|)).
__global__ void state_space_steps_kernel(const float* __restrict__ proj, long long stride, int dt_col, const float* __restrict__ dt_bias,
                                         const float* __restrict__ A_log, long long total, int H, float* __restrict__ dt_out,
                                         float* __restrict__ decay_out) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long long t = idx / H;
    const int h = (int)(idx - t * H);
    const float v = proj[t * stride + dt_col + h] + dt_bias[h];
    const float dt = fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v)));
    dt_out[idx] = dt;
    decay_out[idx] = expf(-expf(A_log[h]) * dt);
}

// Behind the walk: y = (sum of the walk's slices + D_h · x) · silu(z); the row in `groups` equal parts, each divided by its own
// sqrt(mean(part²) + eps); times the gain; in the engine's type.  A block per token forms y into shared memory; then a warp takes parts in turn (a
// lane a strided share of the part, then the warp's tree: an order fixed by the sizes alone).
template <typename T>
__global__ void state_space_finish_kernel(const float* __restrict__ o, int slices, long long slice_stride,
                                          const float* __restrict__ xsrc, long long x_stride, const float* __restrict__ D,
                                          const float* __restrict__ z, long long z_stride, const float* __restrict__ gain, float eps,
                                          int H, int vdim, int groups, T* __restrict__ out) {
    const long long t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int inner = H * vdim, part = inner / groups;
    extern __shared__ float row[];                       // [inner]
    for (int c = threadIdx.x; c < inner; c += blockDim.x) {
        float y = 0.0f;
        for (int s = 0; s < slices; ++s) y += o[(long long)s * slice_stride + t * inner + c];
        y = fmaf(D[c / vdim], xsrc[t * x_stride + c], y);
        const float zz = z[t * z_stride + c];
        row[c] = y * (zz / (1.0f + expf(-zz)));
    }
    __syncthreads();
    for (int g = warp; g < groups; g += n_warps) {
        float ss = 0.0f;
        for (int i = lane; i < part; i += 32) ss += row[g * part + i] * row[g * part + i];
        ss = warp_sum(ss);
        const float f = 1.0f / sqrtf(ss / (float)part + eps);
        for (int i = lane; i < part; i += 32) {
            const int c = g * part + i;
            out[t * inner + c] = from_float<T>(row[c] * f * gain[c]);
        }
    }
}

template <int ROWS>
static int launch_gla(const GlaArgs& a, dim3 grid, cudaStream_t s) {
    constexpr int DP = 8 * ROWS;
    const size_t smem = (size_t)(3 * GLA_CHUNK * DP + GLA_CHUNK * GLA_COLS) * sizeof(float);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaError_t e = cudaFuncSetAttribute(gla_walk_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    gla_walk_kernel<ROWS><<<grid, GLA_THREADS, smem, s>>>(a);
    MLC_LAUNCH_CHECK();
    return 0;
}

}  // namespace mlc

using namespace mlc;

// Rows of S a thread holds (2, 4, 8, 16 or 32; a block's slab of rows is eight times that) for a step of these sizes: the
// whole head when the step's blocks fill the GPU anyway, else the widest slab that gives two blocks per SM, down to 16
// rows.  The outputs come in ceil(dim / (8 * rows)) slices.
extern "C" int mlc_gla_rows(int n_seqs, int H, int dim, int vdim, int n_sms) {
    int rows = 4;
    while (8 * rows < dim && rows < 32) rows *= 2;               // the whole head
    const long long base = (long long)n_seqs * H * ((vdim + GLA_COLS - 1) / GLA_COLS);
    while (rows > 2 && base * ((dim + 8 * rows - 1) / (8 * rows)) < 2LL * n_sms) rows /= 2;
    return rows;
}

// The walk alone, over decays that are already made: q and k (H x dim each) in the float32 rows `qk`, v (H x vdim) in the rows
// `v` (the same matrix or another), decay float32 [n][H*dim].
static int gla_walk(const float* qk, long long qk_stride, int q_col, int k_col, const float* v, long long v_stride, int v_col,
                    const float* decay, float q_scale, float* state, long long state_stride, const int* slots,
                    const int* cu_seqlens, int n_seqs, int n_tokens, int H, int dim, int vdim, int rows, float* out,
                    cudaStream_t s, int qk_share = 1, const float* head_decay = nullptr, const float* v_scale = nullptr) {
    if (H <= 0 || dim <= 0 || dim > 256 || vdim <= 0 || n_seqs > 65535 || qk_share < 1 || H % qk_share) return MLC_ERR_BAD_SIZE;
    if (rows != 2 && rows != 4 && rows != 8 && rows != 16 && rows != 32) return MLC_ERR_BAD_SIZE;
    const int col_slabs = (vdim + GLA_COLS - 1) / GLA_COLS, row_slabs = (dim + 8 * rows - 1) / (8 * rows);
    GlaArgs a{qk, qk_stride, v, v_stride, q_col, k_col, v_col, decay, q_scale, state, state_stride,
              slots, cu_seqlens, out, (long long)n_tokens * H * vdim, H, dim, vdim, col_slabs, qk_share, head_decay, v_scale};
    const dim3 grid(H, n_seqs, col_slabs * row_slabs);
    if (rows == 2) return launch_gla<2>(a, grid, s);
    if (rows == 4) return launch_gla<4>(a, grid, s);
    if (rows == 8) return launch_gla<8>(a, grid, s);
    if (rows == 16) return launch_gla<16>(a, grid, s);
    return launch_gla<32>(a, grid, s);
}

// proj: float32 rows (stride proj_stride) holding q (H x dim) at q_col, k (H x dim) at k_col, v (H x vdim) at v_col.
// z: float32 [n][H*dim] decay logits (overwritten with the decays), z_bias [H*dim] or null.  state: float32, a slot's row
// holds H*vdim*dim floats.  rows: what mlc_gla_rows gave.  out: float32 [ceil(dim / (8 * rows))][n][H*vdim], partial
// outputs to be added up.
extern "C" int mlc_gla(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, float* z,
                       const float* z_bias, float tau, float* state, long long state_stride, const int* slots,
                       const int* cu_seqlens, int n_seqs, int n_tokens, int H, int dim, int vdim, int rows, float* out,
                       void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H <= 0 || dim <= 0 || dim > 256 || vdim <= 0 || !(tau > 0.0f) || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    if (rows != 2 && rows != 4 && rows != 8 && rows != 16 && rows != 32) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_tokens * H * dim;
    gla_decay_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(z, z_bias, total, H * dim, 1.0f / tau);
    MLC_LAUNCH_CHECK();
    return gla_walk(proj, proj_stride, q_col, k_col, proj, proj_stride, v_col, z, 1.0f / sqrtf((float)dim), state, state_stride,
                    slots, cu_seqlens, n_seqs, n_tokens, H, dim, vdim, rows, out, s);
}

// The forget-gate form: proj float32 rows holding the query logits (H x dim) at q_col, the gate logits (H x dim) at f_col
// and v (H x vdim) at v_col; f_bias, lower [H*dim] or null (no bias; a lower bound of zero).  qk float32 [n][2*H*dim] and
// decay float32 [n][H*dim] are scratch that this call fills.  state, rows, out as in mlc_gla.
extern "C" int mlc_forget_gate_attention(const float* proj, long long proj_stride, int q_col, int f_col, int v_col,
                                         const float* f_bias, const float* lower, float* qk, float* decay, float* state,
                                         long long state_stride, const int* slots, const int* cu_seqlens, int n_seqs,
                                         int n_tokens, int H, int dim, int vdim, int rows, float* out, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H <= 0 || dim <= 0 || dim > 256 || vdim <= 0 || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int width = H * dim;
    const long long total = (long long)n_tokens * width;
    forget_gates_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(proj, proj_stride, q_col, f_col, f_bias, lower, total,
                                                                         width, qk, decay);
    MLC_LAUNCH_CHECK();
    return gla_walk(qk, 2LL * width, 0, width, proj, proj_stride, v_col, decay, 1.0f, state, state_stride, slots, cu_seqlens,
                    n_seqs, n_tokens, H, dim, vdim, rows, out, s);
}

// The state-space layer.  proj: float32 rows holding the gate z (H x vdim) at z_col and the step logits (H) at dt_col; xbc:
// float32 rows (what the convolution and its activation left) holding x (H x vdim) at column 0, B (G x N) at b_col and C
// (G x N) at c_col; head h reads group h / (H / G).  dt, decay: float32 [n][H] scratch that this call fills.  state: float32, a
// slot's row holds H*vdim*N floats ([head][column][row]).  rows: what mlc_gla_rows gave for (n_seqs, H, N, vdim).  walk: float32
// [ceil(N / (8 * rows))][n][H*vdim] scratch (the walk's partial outputs).  out [n][H*vdim] of out_dtype: the gated, normed y.
extern "C" int mlc_state_space(const float* proj, long long proj_stride, int z_col, int dt_col, const float* xbc, long long xbc_stride,
                               int b_col, int c_col, const float* dt_bias, const float* A_log, const float* D, const float* gain,
                               float eps, int norm_groups, float* dt, float* decay, float* state, long long state_stride,
                               const int* slots, const int* cu_seqlens, int n_seqs, int n_tokens, int H, int G, int N, int vdim,
                               int rows, float* walk, void* out, int out_dtype, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || N > 256 || vdim <= 0 || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    const int inner = H * vdim;
    if (norm_groups < 1 || inner % norm_groups || inner * sizeof(float) > 48 * 1024) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long total = (long long)n_tokens * H;
    state_space_steps_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(proj, proj_stride, dt_col, dt_bias, A_log, total, H, dt, decay);
    MLC_LAUNCH_CHECK();
    const int rc = gla_walk(xbc, xbc_stride, c_col, b_col, xbc, xbc_stride, 0, nullptr, 1.0f, state, state_stride, slots, cu_seqlens,
                            n_seqs, n_tokens, H, N, vdim, rows, walk, s, H / G, decay, dt);
    if (rc != 0) return rc;
    const int slices = (N + 8 * rows - 1) / (8 * rows);
    const int warps = inner >= 1024 ? 8 : 4;
    if (out_dtype == MLC_DTYPE_F32)
        state_space_finish_kernel<float><<<n_tokens, 32 * warps, inner * sizeof(float), s>>>(
            walk, slices, (long long)n_tokens * inner, xbc, xbc_stride, D, proj + z_col, proj_stride, gain, eps, H, vdim, norm_groups, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16)
        state_space_finish_kernel<bf16><<<n_tokens, 32 * warps, inner * sizeof(float), s>>>(
            walk, slices, (long long)n_tokens * inner, xbc, xbc_stride, D, proj + z_col, proj_stride, gain, eps, H, vdim, norm_groups, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}
