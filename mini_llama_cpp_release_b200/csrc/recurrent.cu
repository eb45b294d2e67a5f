// Mixers that keep a fixed-size state per sequence instead of keys and values: the short
// causal convolution over time, the gated delta rule, and the gated diagonal linear
// recurrence (real-gated LRU) with its block-diagonal gates.
//
// Everything that enters a recurrence is float32 here, in both engine modes: the inputs of
// the convolutions, the convolutions themselves, unit norms, decays, gates and the state.
// A step gives every sequence q_len >= 1 new tokens (cu_seqlens) and a slot; the state of a
// slot is read at the start of the step and left as it stands after the step's last token, so
// that the same kernels serve whole prompts, portions of prompts and single decoded tokens.
// No result depends on which other sequences run in the step.
#include "common.cuh"

namespace mlc {

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// gelu_tanh(z) = 0.5 z (1 + tanh(w)), w = sqrt(2/pi) (z + 0.044715 z³).  Since 1 + tanh(w) = 2 / (1 + exp(-2w)), it is
// formed as z / (1 + exp(-2w)): the sum 1 + tanh(w) would lose its digits where tanh(w) is close to -1.
__device__ __forceinline__ float gelu_tanh_f(float z) {
    const float w = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return z / (1.0f + expf(-2.0f * w));
}

// ------------------------------------------------------------------ causal convolution
// y_t[c] = bias[c] + sum_{j < taps} w[c][taps-1-j] · x_{t-j}[c], x before the sequence's first token being zero; an input
// bias, if given, is added to every real token's x first (it belongs to the projection that made x, not to the zeros).
// The last taps-1 inputs of a sequence are its state: state[slot][i][c] is the input at (length - (taps-1) + i).
// The terms are added in ascending j for every token, wherever its inputs come from.
struct ConvArgs {
    const float* x;             // [n_tokens] rows of x_stride floats; the C channels start at the pointer
    long long x_stride;
    const float* w;             // [C][taps]
    const float* bias;          // [C] or null
    const float* in_bias;       // [C] or null: added to x as it is read
    float* state;               // slot s: state + s * state_stride, [(taps-1)][C]
    long long state_stride;
    const int* slots;           // [n_seqs]
    const int* cu_seqlens;      // [n_seqs + 1]
    const int* tok_seq;         // [n_tokens]
    float* out;                 // [n_tokens] rows of out_stride floats
    long long out_stride;
    int C, taps, act;           // act 0: none, 1: silu
    int n_tokens, n_seqs;
};

__device__ __forceinline__ float conv_finish(float acc, int act) { return act == 1 ? acc * sigmoid_f(acc) : acc; }

// A block takes CONV_SUB tiles of CONV_TOKENS consecutive tokens x 256 channels, one after the other.  Where each token stands in its sequence is looked up
// once per block; the tile's inputs, with the taps-1 rows before it, are loaded in one sweep of independent loads into
// shared memory (a thread reads back only what it wrote itself); only a sequence's first taps-1 tokens reach for the
// state.  CONV_MAX_TAPS bounds the rows kept; longer filters take the plain kernel below.
constexpr int CONV_TOKENS = 16;
constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_SUB = 1;          // tiles a block walks one after the other (more than one was slower: 30 against 26 us
                                     // for 2,048 tokens x 3,072 channels; the kernel waits on latency, not on its look-up)

__global__ void __launch_bounds__(256)
conv_out_kernel(ConvArgs a) {
    __shared__ int t_of[CONV_SUB * CONV_TOKENS];
    __shared__ long long state_of[CONV_SUB * CONV_TOKENS];
    __shared__ float tile[CONV_TOKENS + CONV_MAX_TAPS - 1][256];
    const int block_tok0 = blockIdx.x * CONV_SUB * CONV_TOKENS, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (threadIdx.x < CONV_SUB * CONV_TOKENS) {
        const int token = block_tok0 + threadIdx.x;
        if (token < a.n_tokens) {
            const int seq = a.tok_seq[token];
            t_of[threadIdx.x] = token - a.cu_seqlens[seq];
            state_of[threadIdx.x] = (long long)a.slots[seq] * a.state_stride;
        }
    }
    __syncthreads();
    if (c >= a.C) return;
    const int halo = a.taps - 1;
    const float ib = a.in_bias != nullptr ? a.in_bias[c] : 0.0f;
    float w[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) w[j] = j < a.taps ? a.w[(long long)c * a.taps + a.taps - 1 - j] : 0.0f;
    const float b0 = a.bias != nullptr ? a.bias[c] : 0.0f;
    for (int sub = 0; sub < CONV_SUB; ++sub) {
        const int tok0 = block_tok0 + sub * CONV_TOKENS;
        if (tok0 >= a.n_tokens) break;
        const int n_here = min(CONV_TOKENS, a.n_tokens - tok0);
        float in[CONV_TOKENS + CONV_MAX_TAPS - 1];
#pragma unroll
        for (int r = 0; r < CONV_TOKENS + CONV_MAX_TAPS - 1; ++r) {      // every load of the tile in flight at once
            const int token = tok0 - halo + r;
            in[r] = (r < n_here + halo && token >= 0) ? a.x[(long long)token * a.x_stride + c] : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < CONV_TOKENS + CONV_MAX_TAPS - 1; ++r) tile[r][threadIdx.x] = in[r] + ib;   // a column of one's own
        for (int i = 0; i < n_here; ++i) {
            const int t = t_of[sub * CONV_TOKENS + i];
            float acc = b0;
            if (t >= halo) {
#pragma unroll
                for (int j = 0; j < CONV_MAX_TAPS; ++j)
                    if (j < a.taps) acc = fmaf(w[j], tile[i + halo - j][threadIdx.x], acc);
            } else {
                const float* st = a.state + state_of[sub * CONV_TOKENS + i];
                for (int j = 0; j < a.taps; ++j) {
                    const int src = t - j;
                    const float v = src >= 0 ? tile[i + halo - j][threadIdx.x] : st[(long long)(halo + src) * a.C + c];
                    acc = fmaf(a.w[(long long)c * a.taps + a.taps - 1 - j], v, acc);
                }
            }
            a.out[(long long)(tok0 + i) * a.out_stride + c] = conv_finish(acc, a.act);
        }
    }
}

// Any number of taps: a thread per (token, channel).
__global__ void conv_out_plain_kernel(ConvArgs a) {
    const int token = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const int seq = a.tok_seq[token];
    const int t = token - a.cu_seqlens[seq];
    const float* st = a.state + (long long)a.slots[seq] * a.state_stride;
    const float* w = a.w + (long long)c * a.taps;
    float acc = a.bias != nullptr ? a.bias[c] : 0.0f;
    const float ib = a.in_bias != nullptr ? a.in_bias[c] : 0.0f;
    for (int j = 0; j < a.taps; ++j) {
        const int src = t - j;
        const float v = src >= 0 ? a.x[(long long)(token - j) * a.x_stride + c] + ib : st[(long long)(a.taps - 1 + src) * a.C + c];
        acc = fmaf(w[a.taps - 1 - j], v, acc);
    }
    a.out[(long long)token * a.out_stride + c] = conv_finish(acc, a.act);
}

// After conv_out_kernel: the state becomes the last taps-1 inputs of the lengthened sequence.
__global__ void conv_state_kernel(ConvArgs a) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)a.n_seqs * a.C) return;
    const int seq = (int)(idx / a.C), c = (int)(idx % a.C);
    const int first = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - first;
    float* st = a.state + (long long)a.slots[seq] * a.state_stride;
    const float ib = a.in_bias != nullptr ? a.in_bias[c] : 0.0f;
    for (int i = 0; i < a.taps - 1; ++i) {            // ascending: what is read lies ahead of what was written
        const int src = q_len - (a.taps - 1) + i;
        st[(long long)i * a.C + c] = src >= 0 ? a.x[(long long)(first + src) * a.x_stride + c] + ib
                                              : st[(long long)(i + q_len) * a.C + c];
    }
}

// Every sequence brings one token (token b belongs to sequence b): output and state in one pass.
__global__ void conv_step_kernel(ConvArgs a) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)a.n_seqs * a.C) return;
    const int token = (int)(idx / a.C), c = (int)(idx % a.C);
    float* st = a.state + (long long)a.slots[token] * a.state_stride;
    const float* w = a.w + (long long)c * a.taps;
    const float cur = a.x[(long long)token * a.x_stride + c] + (a.in_bias != nullptr ? a.in_bias[c] : 0.0f);
    float acc = a.bias != nullptr ? a.bias[c] : 0.0f;
    acc = fmaf(w[a.taps - 1], cur, acc);
    for (int j = 1; j < a.taps; ++j) acc = fmaf(w[a.taps - 1 - j], st[(long long)(a.taps - 1 - j) * a.C + c], acc);
    for (int i = 0; i + 2 < a.taps; ++i) st[(long long)i * a.C + c] = st[(long long)(i + 1) * a.C + c];
    if (a.taps >= 2) st[(long long)(a.taps - 2) * a.C + c] = cur;
    a.out[(long long)token * a.out_stride + c] = conv_finish(acc, a.act);
}

// ------------------------------------------------------------------ gated delta rule
// Per head, with a state S [dim][vdim] and, for a token, unit vectors k and q (q also times dim^-1/2), a value row v,
// a decay g in (0, 1) and a step size beta in (0, 1):
//     S <- g·S;   u = beta·(v - Sᵀk);   S <- S + k uᵀ;   o = Sᵀq.
// Two kernels.  The first is parallel over tokens: per (token, head) the five numbers the recurrence needs beside the
// raw rows: g, beta, the factors fk = 1/sqrt(|k|² + 1e-6) and fq = dim^-1/2 / sqrt(|q|² + 1e-6) that make k and q unit
// vectors, and k·q of the unit vectors.  The second walks each sequence's tokens in order.  The columns of S never
// meet, so a block owns 32 of them for one (sequence, head); a warp owns 8, a lane two neighbouring columns and an
// eighth of their rows, in registers.  With the state before the token, S', and the raw rows k', q':
//     dk = fk·S'ᵀk',  dq = fq·S'ᵀq'   (two dot products per column that do not wait for each other)
//     u = beta·(v - g·dk),  o = g·dq + (k·q)·u,  S = g·S' + k' (fk·u)ᵀ.
// Tokens come in chunks of DR_CHUNK through two shared-memory buffers: while one chunk's steps run, the next
// chunk's rows and numbers are on their way (cp.async), and the steps touch global memory for the outputs only.
constexpr int DR_CHUNK = 16;
constexpr int DR_COLS = 32;
constexpr int DR_COEF = 5;      // g, beta, fk, fq, k·q

struct DeltaArgs {
    const float* qkv;           // rows of qkv_stride floats: q heads at q_col, k heads at k_col (G x dim each), v at v_col (H x vdim)
    long long qkv_stride;
    int q_col, k_col, v_col;
    const float* gates;         // rows of gates_stride floats: step-size logits at b_col (H), decay logits at a_col (H)
    long long gates_stride;
    int b_col, a_col;
    const float* A_log;         // [H]
    const float* dt_bias;       // [H]
    float* coef;                // [n_tokens][H][DR_COEF], written by the first kernel
    float* state;               // slot s: state + s * state_stride, [H][dim][vdim]
    long long state_stride;
    const int* slots;
    const int* cu_seqlens;
    float* out;                 // [n_tokens][H * vdim]
    int H, G, dim, vdim, n_tokens;
    float q_scale;              // dim^-1/2
    int vec4;                   // rows, columns and sizes allow 16-byte copies of q, k and v
};

__global__ void delta_prepare_kernel(DeltaArgs a) {
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)a.n_tokens * a.H) return;
    const int lane = threadIdx.x & 31;
    const int token = (int)(w / a.H), head = (int)(w % a.H);
    const int kv_head = head / (a.H / a.G);
    const float* row = a.qkv + (long long)token * a.qkv_stride + kv_head * a.dim;
    float sk = 0.0f, sq = 0.0f, skq = 0.0f;
    for (int i = lane; i < a.dim; i += 32) {
        const float kv = row[a.k_col + i], qv = row[a.q_col + i];
        sk = fmaf(kv, kv, sk);
        sq = fmaf(qv, qv, sq);
        skq = fmaf(kv, qv, skq);
    }
    sk = warp_sum(sk);
    sq = warp_sum(sq);
    skq = warp_sum(skq);
    if (lane == 0) {
        const float* gr = a.gates + (long long)token * a.gates_stride;
        const float fk = 1.0f / sqrtf(sk + 1e-6f), fq = a.q_scale / sqrtf(sq + 1e-6f);
        float* c = a.coef + w * DR_COEF;
        c[0] = expf(-expf(a.A_log[head]) * softplus_f(gr[a.a_col + head] + a.dt_bias[head]));
        c[1] = sigmoid_f(gr[a.b_col + head]);
        c[2] = fk;
        c[3] = fq;
        c[4] = skq * fk * fq;
    }
}

__device__ __forceinline__ void cp_async_f32x4(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

__device__ __forceinline__ void cp_async_f32(float* smem, const float* gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}

// Row part p of 8 holds rows p*NI .. p*NI + NI - 1.  In shared memory a k or q row keeps the parts NI + 4 floats apart, so
// that the 16-byte reads a warp makes at a time fall on different banks.
template <int NI>
struct DeltaSmem {
    static constexpr int ROW = 8 * (NI + 4);
    float k[DR_CHUNK][ROW];
    float q[DR_CHUNK][ROW];
    float v[DR_CHUNK][DR_COLS];
    float coef[DR_CHUNK][8];
};

template <int NI>
__global__ void __launch_bounds__(128)
delta_rule_kernel(DeltaArgs a) {
    static_assert(NI % 4 == 0, "rows per lane come in fours");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DeltaSmem<NI>* bufs = reinterpret_cast<DeltaSmem<NI>*>(smem_raw);

    const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * DR_COLS;
    const int kv_head = head / (a.H / a.G);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane >> 2;                               // 0..7: which rows
    const int col_in_block = warp * 8 + (lane & 3) * 2;       // this lane's two columns
    const int col = col0 + col_in_block;
    const bool ok0 = col < a.vdim, ok1 = col + 1 < a.vdim;
    const int first = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - first;
    float* S_glob = a.state + (long long)a.slots[seq] * a.state_stride + (long long)head * a.dim * a.vdim;

    float S0[NI], S1[NI];
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = part * NI + ii;
        S0[ii] = (ok0 && i < a.dim) ? S_glob[(long long)i * a.vdim + col] : 0.0f;
        S1[ii] = (ok1 && i < a.dim) ? S_glob[(long long)i * a.vdim + col + 1] : 0.0f;
    }

    // what a chunk brings: raw rows of q and k (zeros where dim ends), the block's columns of v, the tokens' five numbers
    auto fetch = [&](int t0, DeltaSmem<NI>& b) {
        const int n_t = min(DR_CHUNK, q_len - t0);
        for (int idx = tid; idx < DR_CHUNK * 8 * NI; idx += 128) {
            const int t = idx / (8 * NI), i = idx % (8 * NI);
            const int at = i + 4 * (i / NI);
            if (t < n_t && i < a.dim) {
                const float* row = a.qkv + (long long)(first + t0 + t) * a.qkv_stride + kv_head * a.dim + i;
                cp_async_f32(&b.k[t][at], row + a.k_col);
                cp_async_f32(&b.q[t][at], row + a.q_col);
            } else {
                b.k[t][at] = 0.0f;
                b.q[t][at] = 0.0f;
            }
        }
        for (int idx = tid; idx < DR_CHUNK * DR_COLS; idx += 128) {
            const int t = idx / DR_COLS, j = idx % DR_COLS;
            if (t < n_t && col0 + j < a.vdim)
                cp_async_f32(&b.v[t][j], a.qkv + (long long)(first + t0 + t) * a.qkv_stride + a.v_col + head * a.vdim + col0 + j);
            else
                b.v[t][j] = 0.0f;
        }
        if (tid < DR_CHUNK * DR_COEF) {
            const int t = tid / DR_COEF, e = tid % DR_COEF;
            if (t < n_t) cp_async_f32(&b.coef[t][e], a.coef + ((long long)(first + t0 + t) * a.H + head) * DR_COEF + e);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    fetch(0, bufs[0]);
    int cur = 0;
    for (int t0 = 0; t0 < q_len; t0 += DR_CHUNK, cur ^= 1) {
        const int n_t = min(DR_CHUNK, q_len - t0);
        DeltaSmem<NI>& b = bufs[cur];
        if (t0 + DR_CHUNK < q_len) {
            fetch(t0 + DR_CHUNK, bufs[cur ^ 1]);               // the other buffer's steps ended before the barrier below, last turn
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        for (int t = 0; t < n_t; ++t) {
            const float4* k4 = reinterpret_cast<const float4*>(&b.k[t][part * (NI + 4)]);
            const float4* q4 = reinterpret_cast<const float4*>(&b.q[t][part * (NI + 4)]);
            const float4 c03 = *reinterpret_cast<const float4*>(&b.coef[t][0]);      // g, beta, fk, fq
            const float kq = b.coef[t][4];
            const float2 vv = *reinterpret_cast<const float2*>(&b.v[t][col_in_block]);
            float kr[NI];
            float dk0[2] = {0.0f, 0.0f}, dk1[2] = {0.0f, 0.0f}, dq0[2] = {0.0f, 0.0f}, dq1[2] = {0.0f, 0.0f};
#pragma unroll
            for (int v = 0; v < NI / 4; ++v) {
                const float4 kk = k4[v], qq = q4[v];
                kr[4 * v] = kk.x; kr[4 * v + 1] = kk.y; kr[4 * v + 2] = kk.z; kr[4 * v + 3] = kk.w;
                dk0[0] = fmaf(S0[4 * v], kk.x, dk0[0]);     dk1[0] = fmaf(S1[4 * v], kk.x, dk1[0]);
                dq0[0] = fmaf(S0[4 * v], qq.x, dq0[0]);     dq1[0] = fmaf(S1[4 * v], qq.x, dq1[0]);
                dk0[1] = fmaf(S0[4 * v + 1], kk.y, dk0[1]); dk1[1] = fmaf(S1[4 * v + 1], kk.y, dk1[1]);
                dq0[1] = fmaf(S0[4 * v + 1], qq.y, dq0[1]); dq1[1] = fmaf(S1[4 * v + 1], qq.y, dq1[1]);
                dk0[0] = fmaf(S0[4 * v + 2], kk.z, dk0[0]); dk1[0] = fmaf(S1[4 * v + 2], kk.z, dk1[0]);
                dq0[0] = fmaf(S0[4 * v + 2], qq.z, dq0[0]); dq1[0] = fmaf(S1[4 * v + 2], qq.z, dq1[0]);
                dk0[1] = fmaf(S0[4 * v + 3], kk.w, dk0[1]); dk1[1] = fmaf(S1[4 * v + 3], kk.w, dk1[1]);
                dq0[1] = fmaf(S0[4 * v + 3], qq.w, dq0[1]); dq1[1] = fmaf(S1[4 * v + 3], qq.w, dq1[1]);
            }
            float sk0 = dk0[0] + dk0[1], sk1 = dk1[0] + dk1[1], sq0 = dq0[0] + dq0[1], sq1 = dq1[0] + dq1[1];
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
                sk0 += __shfl_xor_sync(0xffffffffu, sk0, o);
                sk1 += __shfl_xor_sync(0xffffffffu, sk1, o);
                sq0 += __shfl_xor_sync(0xffffffffu, sq0, o);
                sq1 += __shfl_xor_sync(0xffffffffu, sq1, o);
            }
            const float g = c03.x, beta = c03.y, fk = c03.z, fq = c03.w;
            const float u0 = beta * (vv.x - g * (fk * sk0)), u1 = beta * (vv.y - g * (fk * sk1));
            if (part == 0) {
                float* o = a.out + (long long)(first + t0 + t) * a.H * a.vdim + (long long)head * a.vdim + col;
                if (ok0) o[0] = fmaf(kq, u0, g * (fq * sq0));
                if (ok1) o[1] = fmaf(kq, u1, g * (fq * sq1));
            }
            const float w0 = fk * u0, w1 = fk * u1;
#pragma unroll
            for (int ii = 0; ii < NI; ++ii) {
                S0[ii] = fmaf(kr[ii], w0, g * S0[ii]);
                S1[ii] = fmaf(kr[ii], w1, g * S1[ii]);
            }
        }
        __syncthreads();                                       // this buffer may be written again from the next turn on
    }
#pragma unroll
    for (int ii = 0; ii < NI; ++ii) {
        const int i = part * NI + ii;
        if (ok0 && i < a.dim) S_glob[(long long)i * a.vdim + col] = S0[ii];
        if (ok1 && i < a.dim) S_glob[(long long)i * a.vdim + col + 1] = S1[ii];
    }
}

template <int NI>
static cudaError_t launch_delta_rule(const DeltaArgs& a, dim3 grid, cudaStream_t s) {
    const size_t smem = 2 * sizeof(DeltaSmem<NI>);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaError_t e = cudaFuncSetAttribute(delta_rule_kernel<NI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        raised = true;
    }
    delta_rule_kernel<NI><<<grid, 128, smem, s>>>(a);
    return cudaGetLastError();
}


// ------------------------------------------------------------------ gated delta rule, four tokens a round
// The walk above pays the latency of one round (shared-memory reads, products, shuffles, update) per token.  Four
// tokens can share a round: with S the state before the group, G_t the product of the group's decays up to token t,
// P_ts the product of the decays after s up to t, and k̂, q̂ the unit vectors,
//     u_t = beta_t (v_t − G_t Sᵀk̂_t − sum_{s<t} P_ts (k̂_s·k̂_t) u_s)
//     o_t = G_t Sᵀq̂_t + sum_{s<=t} P_ts (k̂_s·q̂_t) u_s
//     S  <- G_3 S + sum_t P_3t k̂_t u_tᵀ
// (the state after token t is G_t S + sum_{s<=t} P_ts k̂_s u_sᵀ, which put into the rule for token t+1 gives these).
// All eight products of a round with S (four with k, four with q) are independent, their shuffles overlap, and the u_t
// follow from each other by a few scalar operations.  The first kernel leaves, per (token, head), the sixteen numbers
// of a token's place in its group; a group's missing tokens at a sequence's end count as tokens that change nothing
// (beta = 0, decay 1).  Groups are counted from the sequence's first token of the step.
constexpr int DG = 4;            // tokens per round
constexpr int DG_COEF = 16;      // [0] G_t fk_t, [1] G_t fq_t, [2] beta_t, [3] P_3t fk_t, [4..6] P_ts k̂_s·k̂_t (s < t), [7] G_3, [8..11] P_ts k̂_s·q̂_t (s <= t)

// Records are kept per sequence with room for a last group's missing tokens: sequence b's token t is record
// cu_seqlens[b] + 3 b + t.
__global__ void __launch_bounds__(128)
delta_prepare_group_kernel(DeltaArgs a) {
    const int seq = blockIdx.z, group = blockIdx.x;
    const int head = blockIdx.y * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int first = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - first;
    if (group * DG >= q_len || head >= a.H) return;
    const int kv_head = head / (a.H / a.G);
    const int n_t = min(DG, q_len - group * DG);
    float nk[DG], nq[DG], kk[DG][DG], kq[DG][DG];
#pragma unroll
    for (int t = 0; t < DG; ++t) {
        nk[t] = nq[t] = 0.0f;
#pragma unroll
        for (int u = 0; u < DG; ++u) kk[t][u] = kq[t][u] = 0.0f;
    }
    for (int i = lane; i < a.dim; i += 32) {
        float kv[DG], qv[DG];
#pragma unroll
        for (int t = 0; t < DG; ++t) {
            const float* row = a.qkv + (long long)(first + group * DG + t) * a.qkv_stride + kv_head * a.dim + i;
            kv[t] = t < n_t ? row[a.k_col] : 0.0f;
            qv[t] = t < n_t ? row[a.q_col] : 0.0f;
        }
#pragma unroll
        for (int t = 0; t < DG; ++t) {
            nk[t] = fmaf(kv[t], kv[t], nk[t]);
            nq[t] = fmaf(qv[t], qv[t], nq[t]);
#pragma unroll
            for (int u = 0; u < DG; ++u) {
                if (u < t) kk[u][t] = fmaf(kv[u], kv[t], kk[u][t]);
                if (u <= t) kq[u][t] = fmaf(kv[u], qv[t], kq[u][t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < DG; ++t) {
        nk[t] = warp_sum(nk[t]);
        nq[t] = warp_sum(nq[t]);
#pragma unroll
        for (int u = 0; u < DG; ++u) {
            if (u < t) kk[u][t] = warp_sum(kk[u][t]);
            if (u <= t) kq[u][t] = warp_sum(kq[u][t]);
        }
    }
    float g[DG], beta[DG], fk[DG], fq[DG];
    const float neg_rate = -expf(a.A_log[head]), dt_bias = a.dt_bias[head];
#pragma unroll
    for (int t = 0; t < DG; ++t) {
        if (t < n_t) {
            const float* gr = a.gates + (long long)(first + group * DG + t) * a.gates_stride;
            g[t] = expf(neg_rate * softplus_f(gr[a.a_col + head] + dt_bias));
            beta[t] = sigmoid_f(gr[a.b_col + head]);
            fk[t] = 1.0f / sqrtf(nk[t] + 1e-6f);
            fq[t] = a.q_scale / sqrtf(nq[t] + 1e-6f);
        } else {
            g[t] = 1.0f;
            beta[t] = fk[t] = fq[t] = 0.0f;
        }
    }
    if (lane < DG) {
        const int t = lane;
        float P[DG];                                  // P[s] = product of g over s+1 .. t (1 for s = t)
        float run = 1.0f;
#pragma unroll
        for (int s = DG - 1; s >= 0; --s) {
            if (s <= t) {
                P[s] = run;
                run *= g[s];
            } else {
                P[s] = 0.0f;
            }
        }
        const float G_t = run;                       // g_0 .. g_t
        float after = 1.0f;                           // product of g over t+1 .. 3
        float G3 = 1.0f;
#pragma unroll
        for (int s = 0; s < DG; ++s) {
            G3 *= g[s];
            if (s > t) after *= g[s];
        }
        // select this lane's token's numbers without indexing registers by a variable
        float fk_t = 0.0f, fq_t = 0.0f, beta_t = 0.0f, A[DG], B[DG];
#pragma unroll
        for (int u = 0; u < DG; ++u) A[u] = B[u] = 0.0f;
#pragma unroll
        for (int tt = 0; tt < DG; ++tt) {
            if (tt == t) {
                fk_t = fk[tt];
                fq_t = fq[tt];
                beta_t = beta[tt];
#pragma unroll
                for (int u = 0; u < DG; ++u) {
                    if (u < tt) A[u] = P[u] * fk[u] * fk[tt] * kk[u][tt];
                    if (u <= tt) B[u] = P[u] * fk[u] * fq[tt] * kq[u][tt];
                }
            }
        }
        float* c = a.coef + ((long long)(first + 3 * seq + group * DG + t) * a.H + head) * DG_COEF;
        c[0] = G_t * fk_t;
        c[1] = G_t * fq_t;
        c[2] = beta_t;
        c[3] = after * fk_t;
        c[4] = A[0]; c[5] = A[1]; c[6] = A[2];
        c[7] = G3;
        c[8] = B[0]; c[9] = B[1]; c[10] = B[2]; c[11] = B[3];
    }
}

template <int NI>
struct DeltaGroupSmem {
    static constexpr int ROW = 8 * (NI + 4);
    float k[DR_CHUNK][ROW];
    float q[DR_CHUNK][ROW];
    float v[DR_CHUNK][DR_COLS];
    float coef[DR_CHUNK][DG_COEF];
};

template <int NI, int NC>
__global__ void __launch_bounds__(128)
delta_rule_group_kernel(DeltaArgs a) {
    static_assert(NI % 4 == 0 && DR_CHUNK % DG == 0, "rows per lane come in fours, groups do not straddle chunks");
    static_assert(NC == 1 || NC == 2, "a lane holds one column of S or two neighbouring ones");
    constexpr int COLS = 16 * NC;                               // columns of S per block
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DeltaGroupSmem<NI>* bufs = reinterpret_cast<DeltaGroupSmem<NI>*>(smem_raw);

    const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * COLS;
    const int kv_head = head / (a.H / a.G);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int part = lane >> 2;
    const int col_in_block = (warp * 4 + (lane & 3)) * NC;
    const int col = col0 + col_in_block;
    const int first = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - first;
    float* S_glob = a.state + (long long)a.slots[seq] * a.state_stride + (long long)head * a.dim * a.vdim;

    float S[NC][NI];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int ii = 0; ii < NI; ++ii) {
            const int i = part * NI + ii;
            S[c][ii] = (col + c < a.vdim && i < a.dim) ? S_glob[(long long)i * a.vdim + col + c] : 0.0f;
        }

    auto fetch = [&](int t0, DeltaGroupSmem<NI>& b) {
        const int n_t = min(DR_CHUNK, q_len - t0);
        const int n_rec = min(DR_CHUNK, (n_t + DG - 1) / DG * DG);       // a last group's missing tokens have records too
        if (a.vec4) {                                                      // 16 bytes a copy: a quarter of the copies
            for (int idx = tid; idx < DR_CHUNK * 2 * NI; idx += 128) {
                const int t = idx / (2 * NI), i = (idx % (2 * NI)) * 4;
                const int at = i + 4 * (i / NI);
                if (t < n_t && i < a.dim) {
                    const float* row = a.qkv + (long long)(first + t0 + t) * a.qkv_stride + kv_head * a.dim + i;
                    cp_async_f32x4(&b.k[t][at], row + a.k_col);
                    cp_async_f32x4(&b.q[t][at], row + a.q_col);
                } else {
                    *reinterpret_cast<float4*>(&b.k[t][at]) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    *reinterpret_cast<float4*>(&b.q[t][at]) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
            for (int idx = tid; idx < DR_CHUNK * COLS / 4; idx += 128) {
                const int t = idx / (COLS / 4), j = (idx % (COLS / 4)) * 4;
                if (t < n_t && col0 + j < a.vdim)
                    cp_async_f32x4(&b.v[t][j], a.qkv + (long long)(first + t0 + t) * a.qkv_stride + a.v_col + head * a.vdim + col0 + j);
                else
                    *reinterpret_cast<float4*>(&b.v[t][j]) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        } else {
            for (int idx = tid; idx < DR_CHUNK * 8 * NI; idx += 128) {
                const int t = idx / (8 * NI), i = idx % (8 * NI);
                const int at = i + 4 * (i / NI);
                if (t < n_t && i < a.dim) {
                    const float* row = a.qkv + (long long)(first + t0 + t) * a.qkv_stride + kv_head * a.dim + i;
                    cp_async_f32(&b.k[t][at], row + a.k_col);
                    cp_async_f32(&b.q[t][at], row + a.q_col);
                } else {
                    b.k[t][at] = 0.0f;
                    b.q[t][at] = 0.0f;
                }
            }
            for (int idx = tid; idx < DR_CHUNK * COLS; idx += 128) {
                const int t = idx / COLS, j = idx % COLS;
                if (t < n_t && col0 + j < a.vdim)
                    cp_async_f32(&b.v[t][j], a.qkv + (long long)(first + t0 + t) * a.qkv_stride + a.v_col + head * a.vdim + col0 + j);
                else
                    b.v[t][j] = 0.0f;
            }
        }
        for (int idx = tid; idx < DR_CHUNK * 3; idx += 128) {             // records are 64 bytes apart: always aligned
            const int t = idx / 3, e = (idx % 3) * 4;
            if (t < n_rec) cp_async_f32x4(&b.coef[t][e], a.coef + ((long long)(first + 3 * seq + t0 + t) * a.H + head) * DG_COEF + e);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    fetch(0, bufs[0]);
    int cur = 0;
    for (int t0 = 0; t0 < q_len; t0 += DR_CHUNK, cur ^= 1) {
        const int n_t = min(DR_CHUNK, q_len - t0);
        DeltaGroupSmem<NI>& b = bufs[cur];
        if (t0 + DR_CHUNK < q_len) {
            fetch(t0 + DR_CHUNK, bufs[cur ^ 1]);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();
        for (int g0 = 0; g0 < n_t; g0 += DG) {
            float kr[DG][NI];
            float dk[NC][DG], dq[NC][DG];
#pragma unroll
            for (int j = 0; j < DG; ++j) {
                const float4* k4 = reinterpret_cast<const float4*>(&b.k[g0 + j][part * (NI + 4)]);
                const float4* q4 = reinterpret_cast<const float4*>(&b.q[g0 + j][part * (NI + 4)]);
#pragma unroll
                for (int c = 0; c < NC; ++c) dk[c][j] = dq[c][j] = 0.0f;
#pragma unroll
                for (int v = 0; v < NI / 4; ++v) {
                    const float4 kk = k4[v], qq = q4[v];
                    kr[j][4 * v] = kk.x; kr[j][4 * v + 1] = kk.y; kr[j][4 * v + 2] = kk.z; kr[j][4 * v + 3] = kk.w;
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        dk[c][j] = fmaf(S[c][4 * v], kk.x, dk[c][j]);     dq[c][j] = fmaf(S[c][4 * v], qq.x, dq[c][j]);
                        dk[c][j] = fmaf(S[c][4 * v + 1], kk.y, dk[c][j]); dq[c][j] = fmaf(S[c][4 * v + 1], qq.y, dq[c][j]);
                        dk[c][j] = fmaf(S[c][4 * v + 2], kk.z, dk[c][j]); dq[c][j] = fmaf(S[c][4 * v + 2], qq.z, dq[c][j]);
                        dk[c][j] = fmaf(S[c][4 * v + 3], kk.w, dk[c][j]); dq[c][j] = fmaf(S[c][4 * v + 3], qq.w, dq[c][j]);
                    }
                }
            }
#pragma unroll
            for (int o = 4; o <= 16; o <<= 1) {
#pragma unroll
                for (int j = 0; j < DG; ++j)
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        dk[c][j] += __shfl_xor_sync(0xffffffffu, dk[c][j], o);
                        dq[c][j] += __shfl_xor_sync(0xffffffffu, dq[c][j], o);
                    }
            }
            float u[NC][DG], w[NC][DG];
            float G3 = 1.0f;
#pragma unroll
            for (int t = 0; t < DG; ++t) {
                const float4 c0 = *reinterpret_cast<const float4*>(&b.coef[g0 + t][0]);     // G fk, G fq, beta, P_3t fk
                const float4 c1 = *reinterpret_cast<const float4*>(&b.coef[g0 + t][4]);     // A[0..2], G_3
                const float4 c2 = *reinterpret_cast<const float4*>(&b.coef[g0 + t][8]);     // B[0..3]
                const float A[3] = {c1.x, c1.y, c1.z};
                const float B[4] = {c2.x, c2.y, c2.z, c2.w};
                G3 = c1.w;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    float r = b.v[g0 + t][col_in_block + c] - c0.x * dk[c][t];
                    float o = c0.y * dq[c][t];
#pragma unroll
                    for (int sidx = 0; sidx < DG; ++sidx) {
                        if (sidx < t) {
                            r = fmaf(-A[sidx], u[c][sidx], r);
                            o = fmaf(B[sidx], u[c][sidx], o);
                        }
                    }
                    u[c][t] = c0.z * r;
                    o = fmaf(B[t], u[c][t], o);
                    w[c][t] = c0.w * u[c][t];
                    if (part == 0 && g0 + t < n_t && col + c < a.vdim)
                        a.out[(long long)(first + t0 + g0 + t) * a.H * a.vdim + (long long)head * a.vdim + col + c] = o;
                }
            }
#pragma unroll
            for (int ii = 0; ii < NI; ++ii)
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    float sv = G3 * S[c][ii];
#pragma unroll
                    for (int t = 0; t < DG; ++t) sv = fmaf(kr[t][ii], w[c][t], sv);
                    S[c][ii] = sv;
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int ii = 0; ii < NI; ++ii) {
            const int i = part * NI + ii;
            if (col + c < a.vdim && i < a.dim) S_glob[(long long)i * a.vdim + col + c] = S[c][ii];
        }
}

// Two columns per lane (NC = 2): one column per lane and twice the blocks was measured too: 364 against 382 us for one
// 2,048-token sequence of 12 heads of 128 x 128, but 512 against 392 us for two sequences and 1,260 against 912 us for
// eight, since k and q are then read from shared memory twice as often.
template <int NI>
static cudaError_t launch_delta_rule_group(const DeltaArgs& a, dim3 grid, cudaStream_t s) {
    const size_t smem = 2 * sizeof(DeltaGroupSmem<NI>);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        cudaError_t e = cudaFuncSetAttribute(delta_rule_group_kernel<NI, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        raised = true;
    }
    delta_rule_group_kernel<NI, 2><<<dim3((a.vdim + 31) / 32, grid.y, grid.z), 128, smem, s>>>(a);
    return cudaGetLastError();
}

// ------------------------------------------------------------------ gated RMS norm of each head's output
// out[t][h][d] = o / sqrt(mean_d(o²) + eps) · w[d] · silu(gate[t][h][d]); a warp per (token, head).  o may come as
// n_slices partial sums [slice][t][h][d], slice_stride floats apart, that are added up in order as they are read.
template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, int n_slices, long long slice_stride,
                                     const float* __restrict__ gate, long long gate_stride,
                                     const float* __restrict__ w, float eps, long long n_rows, int H, int vdim,
                                     T* __restrict__ out) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int lane = threadIdx.x & 31;
    const long long token = row / H;
    const int head = (int)(row % H);
    const float* src0 = o + row * vdim;
    auto src_at = [&](int d) {
        float v = src0[d];
        for (int sl = 1; sl < n_slices; ++sl) v += src0[sl * slice_stride + d];
        return v;
    };
    const bool gated = gate != nullptr;               // no gate: the head norm alone
    const float* g = gated ? gate + token * gate_stride + (long long)head * vdim : src0;
    if (vdim <= 256) {                              // the row, its gates and gains in registers: every load issued at once
        float v[8], z[8], wv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int d = lane + 32 * k;
            v[k] = d < vdim ? src_at(d) : 0.0f;
            z[k] = d < vdim ? g[d] : 0.0f;
            wv[k] = d < vdim ? w[d] : 0.0f;
        }
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) ss = fmaf(v[k], v[k], ss);
        ss = warp_sum(ss);
        const float f = 1.0f / sqrtf(ss / (float)vdim + eps);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int d = lane + 32 * k;
            if (d < vdim) out[row * vdim + d] = from_float<T>(v[k] * f * wv[k] * (gated ? z[k] * sigmoid_f(z[k]) : 1.0f));
        }
        return;
    }
    float ss = 0.0f;
    for (int d = lane; d < vdim; d += 32) {
        const float v = src_at(d);
        ss += v * v;
    }
    ss = warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int d = lane; d < vdim; d += 32) {
        const float z = g[d];
        out[row * vdim + d] = from_float<T>(src_at(d) * f * w[d] * (gated ? z * sigmoid_f(z) : 1.0f));
    }
}

// ------------------------------------------------------------------ gates of the diagonal recurrence
// The channels are cut into B blocks of bw; in block b: r = sigmoid(Wr[b]·u_b + br), i = sigmoid(Wi[b]·u_b + bi),
// then per channel a = exp(-c·r·softplus(lam)) and drive = sqrt(1 - a²)·i·u.  What is stored is a - 1 = expm1(log a):
// slow channels have a within 1e-5 of one, where a float32 a is a decay that is wrong by up to a percent of 1 - a, and
// any bias of the exponential's last bit adds up over thousands of tokens; a - 1 keeps its digits.  Both products are float32
// multiply-adds, each output one accumulator over ascending k, so a token's gates do not depend on the batch.
// Tiles of 64 tokens x 64 channels, 4 x 4 per thread and gate.
struct GateArgs {
    const float* u;             // [n][W]
    const float* wr;            // [B][bw][bw] (out, in)
    const float* wi;
    const float* br;            // [W]
    const float* bi;            // [W]
    const float* lam;           // [W]
    float* a_out;               // [n][W]: a - 1
    float* drive_out;           // [n][W]
    int n, W, bw;
    float c;
};

__global__ void __launch_bounds__(256)
block_gates_kernel(GateArgs a) {
    __shared__ float Us[16][68];
    __shared__ float Rs[16][68];
    __shared__ float Is[16][68];
    const int tok0 = blockIdx.x * 64, out0 = blockIdx.y * 64, blk = blockIdx.z;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const float* wr = a.wr + (long long)blk * a.bw * a.bw;
    const float* wi = a.wi + (long long)blk * a.bw * a.bw;
    float ar[4][4], ai[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) ar[i][j] = ai[i][j] = 0.0f;
    const int lr = tid >> 2, lk = (tid & 3) * 4;          // the row (token or output channel) and first k this thread stages
    for (int k0 = 0; k0 < a.bw; k0 += 16) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const bool k_ok = k < a.bw;
            const int tok = tok0 + lr, oc = out0 + lr;
            Us[lk + e][lr] = (k_ok && tok < a.n) ? a.u[(long long)tok * a.W + blk * a.bw + k] : 0.0f;
            Rs[lk + e][lr] = (k_ok && oc < a.bw) ? wr[(long long)oc * a.bw + k] : 0.0f;
            Is[lk + e][lr] = (k_ok && oc < a.bw) ? wi[(long long)oc * a.bw + k] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float uv[4], rv[4], iv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) uv[i] = Us[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                rv[j] = Rs[k][tx * 4 + j];
                iv[j] = Is[k][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    ar[i][j] = fmaf(uv[i], rv[j], ar[i][j]);
                    ai[i][j] = fmaf(uv[i], iv[j], ai[i][j]);
                }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int tok = tok0 + ty * 4 + i;
        if (tok >= a.n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int oc = out0 + tx * 4 + j;
            if (oc >= a.bw) continue;
            const int ch = blk * a.bw + oc;
            const float r = sigmoid_f(ar[i][j] + a.br[ch]);
            const float gi = sigmoid_f(ai[i][j] + a.bi[ch]);
            const float log_a = -a.c * r * softplus_f(a.lam[ch]);
            const long long at = (long long)tok * a.W + ch;
            a.a_out[at] = expm1f(log_a);                  // a - 1: see the recurrence below
            // 1 - a² = -expm1(2 log a): formed from the logarithm, it keeps its digits where a is close to one
            a.drive_out[at] = sqrtf(-expm1f(2.0f * log_a)) * gi * a.u[at];
        }
    }
}

// ------------------------------------------------------------------ the diagonal recurrence itself
// S_t = a_t·S_{t-1} + drive_t per channel, formed as S + (a_t - 1)·S + drive_t from the stored a - 1;
// out_t = S_t · gelu_tanh(y_t + y_bias) · out_scale.  A thread per (sequence, channel) walks the sequence's tokens;
// the loads of four tokens are issued together.
template <typename T>
__global__ void linear_scan_kernel(const float* __restrict__ av, const float* __restrict__ drive, const float* __restrict__ y,
                                   long long y_stride, const float* __restrict__ y_bias, float* state, long long state_stride,
                                   const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int W, float out_scale,
                                   T* __restrict__ out) {
    const int seq = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= W) return;
    const int first = cu_seqlens[seq], last = cu_seqlens[seq + 1];
    float* st = state + (long long)slots[seq] * state_stride + c;
    float S = *st;
    const float yb = y_bias != nullptr ? y_bias[c] : 0.0f;
    int t = first;
    for (; t + 4 <= last; t += 4) {
        float a4[4], d4[4], y4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            a4[e] = av[(long long)(t + e) * W + c];
            d4[e] = drive[(long long)(t + e) * W + c];
            y4[e] = y[(long long)(t + e) * y_stride + c];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            S = fmaf(a4[e], S, S) + d4[e];
            out[(long long)(t + e) * W + c] = from_float<T>(S * gelu_tanh_f(y4[e] + yb) * out_scale);
        }
    }
    for (; t < last; ++t) {
        S = fmaf(av[(long long)t * W + c], S, S) + drive[(long long)t * W + c];
        out[(long long)t * W + c] = from_float<T>(S * gelu_tanh_f(y[(long long)t * y_stride + c] + yb) * out_scale);
    }
    *st = S;
}

// The same for long runs of tokens: 32 channels (a lane each) and SC_WARPS warps (1,024 threads) per block, the sequence's new tokens
// cut into SC_WARPS consecutive segments.  A warp first folds its segment into the pair (A, D) with
// S_end = A·S_begin + D; the pairs of the segments before it, applied in order to the sequence's state, give the
// state its segment starts from; then it walks its segment token by token as above.  Eight tokens' loads are issued
// together in both passes.
constexpr int SC_WARPS = 32;

template <typename T>
__global__ void __launch_bounds__(SC_WARPS * 32)
linear_scan_long_kernel(const float* __restrict__ av, const float* __restrict__ drive, const float* __restrict__ y,
                        long long y_stride, const float* __restrict__ y_bias, float* state, long long state_stride,
                        const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int W, float out_scale,
                        T* __restrict__ out) {
    __shared__ float As[SC_WARPS][32], Ds[SC_WARPS][32];
    const int seq = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + lane;
    const bool ok = c < W;
    const int first = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - first;
    const int per = (q_len + SC_WARPS - 1) / SC_WARPS;
    const int lo = first + min(q_len, warp * per), hi = first + min(q_len, (warp + 1) * per);
    float A = 1.0f, D = 0.0f;
    if (ok && warp + 1 < SC_WARPS) {
        int t = lo;
        for (; t + 8 <= hi; t += 8) {
            float a8[8], d8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a8[e] = av[(long long)(t + e) * W + c];
                d8[e] = drive[(long long)(t + e) * W + c];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                A = fmaf(a8[e], A, A);
                D = fmaf(a8[e], D, D) + d8[e];
            }
        }
        for (; t < hi; ++t) {
            const float at = av[(long long)t * W + c];
            A = fmaf(at, A, A);
            D = fmaf(at, D, D) + drive[(long long)t * W + c];
        }
    }
    As[warp][lane] = A;
    Ds[warp][lane] = D;
    __syncthreads();
    if (!ok) return;
    float* st = state + (long long)slots[seq] * state_stride + c;
    float S = *st;
    for (int u = 0; u < warp; ++u) S = fmaf(As[u][lane], S, Ds[u][lane]);
    const float yb = y_bias != nullptr ? y_bias[c] : 0.0f;
    int t = lo;
    for (; t + 8 <= hi; t += 8) {
        float a8[8], d8[8], y8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a8[e] = av[(long long)(t + e) * W + c];
            d8[e] = drive[(long long)(t + e) * W + c];
            y8[e] = y[(long long)(t + e) * y_stride + c];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            S = fmaf(a8[e], S, S) + d8[e];
            out[(long long)(t + e) * W + c] = from_float<T>(S * gelu_tanh_f(y8[e] + yb) * out_scale);
        }
    }
    for (; t < hi; ++t) {
        S = fmaf(av[(long long)t * W + c], S, S) + drive[(long long)t * W + c];
        out[(long long)t * W + c] = from_float<T>(S * gelu_tanh_f(y[(long long)t * y_stride + c] + yb) * out_scale);
    }
    if (warp == SC_WARPS - 1) *st = S;
}

// One token per sequence (token b belongs to sequence b): gates and recurrence in one kernel.  A block takes 32 channels
// of one gate block for up to GS_SEQS sequences; lane = channel, the eight warps share out the inner index and meet in
// shared memory.  The gate matrices come transposed, [block][in][out], so that a warp reads 32 neighbouring outputs of
// one input at a time.
constexpr int GS_SEQS = 8;

template <typename T>
__global__ void __launch_bounds__(256)
gates_scan_step_kernel(const float* __restrict__ u, const float* __restrict__ wr_t, const float* __restrict__ wi_t,
                       const float* __restrict__ br, const float* __restrict__ bi, const float* __restrict__ lam, float c,
                       const float* __restrict__ y, long long y_stride, const float* __restrict__ y_bias, float* state,
                       long long state_stride, const int* __restrict__ slots, int n_seqs, int W, int bw, float out_scale,
                       T* __restrict__ out) {
    extern __shared__ float gs_smem[];
    float* us = gs_smem;                                  // [GS_SEQS][bw]
    float* part = us + GS_SEQS * bw;                      // [8 warps][GS_SEQS][2][32]
    const int chunks = (bw + 31) / 32;
    const int blk = blockIdx.x / chunks, oc0 = (blockIdx.x % chunks) * 32;
    const int seq0 = blockIdx.y * GS_SEQS, n_here = min(GS_SEQS, n_seqs - seq0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int idx = threadIdx.x; idx < GS_SEQS * bw; idx += 256) {
        const int sq = idx / bw, k = idx % bw;
        us[idx] = sq < n_here ? u[(long long)(seq0 + sq) * W + blk * bw + k] : 0.0f;
    }
    __syncthreads();
    const int oc = oc0 + lane;
    float ar[GS_SEQS], ai[GS_SEQS];
#pragma unroll
    for (int sq = 0; sq < GS_SEQS; ++sq) ar[sq] = ai[sq] = 0.0f;
    if (oc < bw) {
        const int per = (bw + 7) / 8;
        const int k_end = min(bw, (warp + 1) * per);
        const float* pr = wr_t + (long long)blk * bw * bw + oc;
        const float* pi = wi_t + (long long)blk * bw * bw + oc;
#pragma unroll 4
        for (int k = warp * per; k < k_end; ++k) {
            const float r = pr[(long long)k * bw], i = pi[(long long)k * bw];
#pragma unroll
            for (int sq = 0; sq < GS_SEQS; ++sq) {
                const float uv = us[sq * bw + k];
                ar[sq] = fmaf(uv, r, ar[sq]);
                ai[sq] = fmaf(uv, i, ai[sq]);
            }
        }
    }
#pragma unroll
    for (int sq = 0; sq < GS_SEQS; ++sq) {
        part[((warp * GS_SEQS + sq) * 2 + 0) * 32 + lane] = ar[sq];
        part[((warp * GS_SEQS + sq) * 2 + 1) * 32 + lane] = ai[sq];
    }
    __syncthreads();
    // warp w finishes sequence w of the tile
    const int sq = warp;
    if (sq >= n_here || oc >= bw) return;
    float sr = 0.0f, si = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        sr += part[((w * GS_SEQS + sq) * 2 + 0) * 32 + lane];
        si += part[((w * GS_SEQS + sq) * 2 + 1) * 32 + lane];
    }
    const int ch = blk * bw + oc, token = seq0 + sq;
    const float r = sigmoid_f(sr + br[ch]), gi = sigmoid_f(si + bi[ch]);
    const float log_a = -c * r * softplus_f(lam[ch]);
    const float drive = sqrtf(-expm1f(2.0f * log_a)) * gi * us[sq * bw + oc];
    float* st = state + (long long)slots[token] * state_stride + ch;
    const float before = *st;
    const float S = fmaf(expm1f(log_a), before, before) + drive;
    *st = S;
    const float yb = y_bias != nullptr ? y_bias[ch] : 0.0f;
    out[(long long)token * W + ch] = from_float<T>(S * gelu_tanh_f(y[(long long)token * y_stride + ch] + yb) * out_scale);
}

}  // namespace mlc

using namespace mlc;

// x, out: float32 rows (strides in floats); w float32 [C][taps]; state float32, a slot's [(taps-1)][C] at
// state + slot * state_stride.  max_q_len == 1 (every sequence one token) runs output and state in one kernel.
extern "C" int mlc_causal_conv(const float* x, long long x_stride, const float* w, const float* bias, const float* in_bias,
                               int C, int taps, int act,
                               float* state, long long state_stride, const int* slots, const int* cu_seqlens,
                               const int* tok_seq, int n_seqs, int n_tokens, int max_q_len, float* out, long long out_stride,
                               void* stream) {
    if (n_tokens <= 0 || n_seqs <= 0) return 0;
    if (C <= 0 || taps < 1 || taps > 64 || (act != 0 && act != 1)) return MLC_ERR_BAD_SIZE;
    ConvArgs a{x, x_stride, w, bias, in_bias, state, state_stride, slots, cu_seqlens, tok_seq, out, out_stride, C, taps, act, n_tokens, n_seqs};
    cudaStream_t s = (cudaStream_t)stream;
    if (max_q_len == 1 && n_tokens == n_seqs) {
        conv_step_kernel<<<(unsigned)(((long long)n_seqs * C + 255) / 256), 256, 0, s>>>(a);
        MLC_LAUNCH_CHECK();
        return 0;
    }
    if ((C + 255) / 256 > 65535) return MLC_ERR_BAD_SIZE;
    if (taps <= CONV_MAX_TAPS)
        conv_out_kernel<<<dim3((n_tokens + CONV_SUB * CONV_TOKENS - 1) / (CONV_SUB * CONV_TOKENS), (C + 255) / 256), 256, 0, s>>>(a);
    else
        conv_out_plain_kernel<<<dim3(n_tokens, (C + 255) / 256), 256, 0, s>>>(a);
    MLC_LAUNCH_CHECK();
    if (taps > 1) {
        conv_state_kernel<<<(unsigned)(((long long)n_seqs * C + 255) / 256), 256, 0, s>>>(a);
        MLC_LAUNCH_CHECK();
    }
    return 0;
}

// coef: scratch of (n_tokens + 3 * n_seqs) * H * 16 floats.  max_q_len: the longest run of new tokens of any sequence.
extern "C" int mlc_gated_delta_rule(const float* qkv, long long qkv_stride, int q_col, int k_col, int v_col, const float* gates,
                                    long long gates_stride, int b_col, int a_col, const float* A_log, const float* dt_bias,
                                    float* coef, float* state, long long state_stride, const int* slots, const int* cu_seqlens,
                                    int n_seqs, int n_tokens, int max_q_len, int H, int G, int dim, int vdim, float* out,
                                    void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || dim <= 0 || dim > 256 || vdim <= 0 || n_seqs > 65535 || H > 65535) return MLC_ERR_BAD_SIZE;
    DeltaArgs a{qkv, qkv_stride, q_col, k_col, v_col, gates, gates_stride, b_col, a_col, A_log, dt_bias, coef, state, state_stride,
                slots, cu_seqlens, out, H, G, dim, vdim, n_tokens, 1.0f / sqrtf((float)dim), 0};
    a.vec4 = ((dim | vdim | q_col | k_col | v_col) % 4 == 0 && qkv_stride % 4 == 0 && ((uintptr_t)qkv | (uintptr_t)coef) % 16 == 0) ? 1 : 0;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((vdim + DR_COLS - 1) / DR_COLS, H, n_seqs);
    const int ni = (dim + 7) / 8;
    cudaError_t e;
    if (max_q_len >= DG && ni <= 16) {                    // runs of tokens: four a round (key sizes up to 128)
        const dim3 pgrid((max_q_len + DG - 1) / DG, (H + 3) / 4, n_seqs);
        if (pgrid.y > 65535) return MLC_ERR_BAD_SIZE;
        delta_prepare_group_kernel<<<pgrid, 128, 0, s>>>(a);
        MLC_LAUNCH_CHECK();
        if (ni <= 4) e = launch_delta_rule_group<4>(a, grid, s);
        else if (ni <= 8) e = launch_delta_rule_group<8>(a, grid, s);
        else if (ni <= 12) e = launch_delta_rule_group<12>(a, grid, s);
        else e = launch_delta_rule_group<16>(a, grid, s);
        return e == cudaSuccess ? 0 : (int)e;
    }
    delta_prepare_kernel<<<(unsigned)(((long long)n_tokens * H + 7) / 8), 256, 0, s>>>(a);
    MLC_LAUNCH_CHECK();
    if (ni <= 4) e = launch_delta_rule<4>(a, grid, s);
    else if (ni <= 8) e = launch_delta_rule<8>(a, grid, s);
    else if (ni <= 12) e = launch_delta_rule<12>(a, grid, s);
    else if (ni <= 16) e = launch_delta_rule<16>(a, grid, s);
    else if (ni <= 24) e = launch_delta_rule<24>(a, grid, s);
    else e = launch_delta_rule<32>(a, grid, s);
    if (e != cudaSuccess) return (int)e;
    return 0;
}

extern "C" int mlc_gated_rmsnorm(const float* o, int n_slices, const float* gate, long long gate_stride, const float* w, float eps,
                                 long long n_tokens, int H, int vdim, void* out, int out_dtype, void* stream) {
    if (n_tokens <= 0) return 0;
    if (H <= 0 || vdim <= 0 || n_slices < 1) return MLC_ERR_BAD_SIZE;
    const long long slice_stride = n_tokens * H * vdim;
    const long long n_rows = n_tokens * H;
    const unsigned blocks = (unsigned)((n_rows + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == MLC_DTYPE_F32)
        gated_rmsnorm_kernel<float><<<blocks, 128, 0, s>>>(o, n_slices, slice_stride, gate, gate_stride, w, eps, n_rows, H, vdim, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16)
        gated_rmsnorm_kernel<bf16><<<blocks, 128, 0, s>>>(o, n_slices, slice_stride, gate, gate_stride, w, eps, n_rows, H, vdim, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_block_gates(const float* u, const float* wr, const float* wi, const float* br, const float* bi,
                               const float* lam, int n, int W, int B, float c, float* a_out, float* drive_out, void* stream) {
    if (n <= 0) return 0;
    if (W <= 0 || B <= 0 || W % B != 0 || B > 65535) return MLC_ERR_BAD_SIZE;
    const int bw = W / B;
    GateArgs a{u, wr, wi, br, bi, lam, a_out, drive_out, n, W, bw, c};
    const dim3 grid((n + 63) / 64, (bw + 63) / 64, B);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    block_gates_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_linear_scan(const float* av, const float* drive, const float* y, long long y_stride, const float* y_bias,
                               float* state, long long state_stride, const int* slots, const int* cu_seqlens, int n_seqs, int W,
                               int max_q_len, float out_scale, void* out, int out_dtype, void* stream) {
    if (n_seqs <= 0) return 0;
    if (W <= 0 || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (max_q_len >= 4 * SC_WARPS) {                      // long runs of tokens: segments scanned side by side
        const dim3 grid((W + 31) / 32, n_seqs);
        if (out_dtype == MLC_DTYPE_F32)
            linear_scan_long_kernel<float><<<grid, SC_WARPS * 32, 0, s>>>(av, drive, y, y_stride, y_bias, state, state_stride, slots, cu_seqlens, W, out_scale, (float*)out);
        else if (out_dtype == MLC_DTYPE_BF16)
            linear_scan_long_kernel<bf16><<<grid, SC_WARPS * 32, 0, s>>>(av, drive, y, y_stride, y_bias, state, state_stride, slots, cu_seqlens, W, out_scale, (bf16*)out);
        else
            return MLC_ERR_BAD_DTYPE;
        MLC_LAUNCH_CHECK();
        return 0;
    }
    const dim3 grid((W + 127) / 128, n_seqs);
    if (out_dtype == MLC_DTYPE_F32)
        linear_scan_kernel<float><<<grid, 128, 0, s>>>(av, drive, y, y_stride, y_bias, state, state_stride, slots, cu_seqlens, W, out_scale, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16)
        linear_scan_kernel<bf16><<<grid, 128, 0, s>>>(av, drive, y, y_stride, y_bias, state, state_stride, slots, cu_seqlens, W, out_scale, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

// Gates and recurrence for a step in which every sequence brings one token: u float32 [n_seqs][W] (the convolution's
// output), wr_t / wi_t the gate matrices transposed to [B][in][out]; the state moves one token on.
extern "C" int mlc_gates_scan_step(const float* u, const float* wr_t, const float* wi_t, const float* br, const float* bi,
                                   const float* lam, float c, const float* y, long long y_stride, const float* y_bias,
                                   float* state, long long state_stride, const int* slots, int n_seqs, int W, int B,
                                   float out_scale, void* out, int out_dtype, void* stream) {
    if (n_seqs <= 0) return 0;
    if (W <= 0 || B <= 0 || W % B != 0) return MLC_ERR_BAD_SIZE;
    const int bw = W / B;
    const size_t smem = (size_t)(GS_SEQS * bw + 8 * GS_SEQS * 2 * 32) * sizeof(float);
    if (smem > 48 * 1024) return MLC_ERR_UNSUPPORTED;
    const dim3 grid(B * ((bw + 31) / 32), (n_seqs + GS_SEQS - 1) / GS_SEQS);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == MLC_DTYPE_F32)
        gates_scan_step_kernel<float><<<grid, 256, smem, s>>>(u, wr_t, wi_t, br, bi, lam, c, y, y_stride, y_bias, state, state_stride,
                                                              slots, n_seqs, W, bw, out_scale, (float*)out);
    else if (out_dtype == MLC_DTYPE_BF16)
        gates_scan_step_kernel<bf16><<<grid, 256, smem, s>>>(u, wr_t, wi_t, br, bi, lam, c, y, y_stride, y_bias, state, state_stride,
                                                             slots, n_seqs, W, bw, out_scale, (bf16*)out);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}
