// Mixture of experts: routing, the plan that sorts a step's (token, expert) pairs by expert, the product of every
// sorted row with its own expert's matrix, and the weighted sum back per token.
//
//   route      z = logits + bias (float32); the `top` largest of a token's E logits are chosen (the lower index wins a
//              tie) and weighted by the softmax over the chosen logits only.
//   plan       pairs (token, j-th choice) are ordered by expert, inside an expert by pair number; every expert's run
//              starts on a multiple of `tile` rows, the rows between runs are padding (source token -1).  Nothing
//              comes back to the host: the tables below are all a later kernel needs.
//                 row_of[pair]      the pair's row in the sorted order
//                 src_tok[row]      the token a row computes, -1 for padding
//                 tile_expert[t]    the expert of rows [t*tile, (t+1)*tile), -1 past the last run
//   grouped    out[row] = W[tile_expert[row / tile]] · x[src] with float32 accumulation, the K range walked in the
//              same order for every row, so a token's result does not depend on what else is in the step.
//   combine    y[token] = sum_j weight[token][j] · out[row_of[token][j]], j in the order of the choices.
#include "common.cuh"

namespace mlc {

constexpr int ROUTE_MAX_PER_LANE = 8;          // E <= 256

// A block of four warps per token.  With `w` given, `x` is the branch's input [n][K] (TX) and the logits are
// x · wᵀ + bias in float32 (w float32 [E][K]; `route_logits` below).  Without `w`, `x` holds the logits themselves, float32 [n][E].
// Warp 0 then chooses: lane l keeps logits l, l + 32, ...
// Router logits of token t into shared `logit[E]`: x · wᵀ + bias in float32 (w float32 [E][K]), R outputs a round, every
// thread a strided share of K, partial sums added within warps and then across them in a fixed order.  A round that has
// fewer than R outputs left reads its last row again in their place and drops those sums (no branch around the loads:
// all of a round's loads are in flight together).  All 128 threads of the block call it.
template <typename TX, int R>
__device__ __forceinline__ void route_logits_by(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                                int t, int E, int K, float (*part)[16], float* logit) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const TX* row = x + (long long)t * K;
    for (int e0 = 0; e0 < E; e0 += R) {
        float acc[R];
        const float* wr[R];
#pragma unroll
        for (int j = 0; j < R; ++j) {
            acc[j] = 0.0f;
            wr[j] = w + (long long)min(e0 + j, E - 1) * K;
        }
#pragma unroll 4
        for (int k = threadIdx.x; k < K; k += 128) {
            const float xv = to_float(row[k]);
#pragma unroll
            for (int j = 0; j < R; ++j) acc[j] = fmaf(xv, __ldg(wr[j] + k), acc[j]);
        }
#pragma unroll
        for (int j = 0; j < R; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0) part[warp][j] = v;
        }
        __syncthreads();
        if (threadIdx.x < R && e0 + threadIdx.x < E) {
            const int e = e0 + threadIdx.x;
            logit[e] = ((part[0][threadIdx.x] + part[1][threadIdx.x]) + (part[2][threadIdx.x] + part[3][threadIdx.x]))
                       + (bias != nullptr ? bias[e] : 0.0f);
        }
        __syncthreads();
    }
}

// The round's size is the smallest of 4, 8, 12 and 16 that takes all outputs at once, else 16.  An output's sum is formed
// in the same order whatever the round's size.
template <typename TX>
__device__ __forceinline__ void route_logits(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                                             int t, int E, int K, float (*part)[16], float* logit) {
    if (E <= 4) route_logits_by<TX, 4>(x, w, bias, t, E, K, part, logit);
    else if (E <= 8) route_logits_by<TX, 8>(x, w, bias, t, E, K, part, logit);
    else if (E <= 12) route_logits_by<TX, 12>(x, w, bias, t, E, K, part, logit);
    else route_logits_by<TX, 16>(x, w, bias, t, E, K, part, logit);
}

// PL: router outputs a lane of the choosing warp keeps (1 for up to 32 outputs, else 8).
template <typename TX, int PL>
__global__ void __launch_bounds__(128)
moe_route_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias, int n,
                 int E, int K, int top, int weighting, int* __restrict__ ids, float* __restrict__ weights) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float part[4][16];
    __shared__ float logit[32 * PL];
    if (w != nullptr) route_logits<TX>(x, w, bias, t, E, K, part, logit);
    if (warp != 0) return;
    float z[PL];
#pragma unroll
    for (int k = 0; k < PL; ++k) {
        const int e = lane + 32 * k;
        z[k] = -INFINITY;
        if (e < E) z[k] = w != nullptr ? logit[e] : reinterpret_cast<const float*>(x)[(long long)t * E + e] + (bias != nullptr ? bias[e] : 0.0f);
    }
    float mine = -INFINITY;          // lane j keeps the j-th chosen logit
    float first = 0.0f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int where = 0x7fffffff;
#pragma unroll
        for (int k = 0; k < PL; ++k) {
            const int e = lane + 32 * k;
            if (e < E && (z[k] > best || (z[k] == best && e < where))) {
                best = z[k];
                where = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, where, o);
            if (ob > best || (ob == best && ow < where)) {
                best = ob;
                where = ow;
            }
        }
        if (where != 0x7fffffff && (where & 31) == lane) {
#pragma unroll
            for (int k = 0; k < PL; ++k)
                if (k == (where >> 5)) z[k] = -INFINITY;
        }
        if (lane == j) mine = best;
        if (j == 0) first = best;                     // the largest: the softmax's reference point
        if (lane == 0) ids[(long long)t * top + j] = where == 0x7fffffff ? 0 : where;
    }
    if (weighting == 1) {
        // every chosen expert's own sigmoid score, as it is (the sigmoid rises with the logit, so the largest scores are the
        // largest logits)
        if (lane < top) weights[(long long)t * top + lane] = 1.0f / (1.0f + expf(-mine));
        return;
    }
    const float p = lane < top ? expf(mine - first) : 0.0f;
    const float sum = warp_sum(p);
    if (lane < top) weights[(long long)t * top + lane] = p / sum;
}

// Routing by scores of all experts.  s = softmax(z) over all E router outputs; an expert is *chosen* by s + correction
// (a stored per-expert term that steers the choice only) and *weighted* by s itself:
//   groups   the E outputs form G equal groups of neighbours; a group's score is its largest choice score, and only
//            experts of the `keep` best groups can be chosen (the others count as minus infinity);
//   choice   the `top` largest remaining choice scores (the lower index wins a tie);
//   weights  s of the chosen, divided by their sum + 1e-20, times `scale`.
// The last E - n_real outputs belong to identity experts (no matrices: the token's input itself); they are chosen and
// weighted like the others, and whoever sums the rows treats their ids apart.  A block of four warps per token forms the
// logits, warp 0 chooses.
template <typename TX, int PL>
__global__ void __launch_bounds__(128)
moe_route_scored_kernel(const TX* __restrict__ x, const float* __restrict__ w, const float* __restrict__ correction, int n,
                        int E, int K, int top, int G, int keep, float scale, int* __restrict__ ids,
                        float* __restrict__ weights) {
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ float part[4][16];
    __shared__ float logit[32 * PL];
    __shared__ float prob[32 * PL];
    __shared__ float gscore[32 * PL];
    route_logits<TX>(x, w, nullptr, t, E, K, part, logit);
    if (warp != 0) return;
    float z[PL], c[PL];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < PL; ++k) {
        const int e = lane + 32 * k;
        z[k] = e < E ? logit[e] : -INFINITY;
        m = fmaxf(m, z[k]);
    }
    m = warp_max(m);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < PL; ++k) {
        z[k] = lane + 32 * k < E ? expf(z[k] - m) : 0.0f;
        sum += z[k];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int k = 0; k < PL; ++k) {
        const int e = lane + 32 * k;
        z[k] = z[k] / sum;                            // the score s
        c[k] = e < E ? z[k] + (correction != nullptr ? correction[e] : 0.0f) : -INFINITY;
        if (e < E) {
            prob[e] = z[k];
            logit[e] = c[k];                          // the choice scores, for the groups
        }
    }
    __syncwarp();
    if (G > 1 && keep < G) {
        const int gs = E / G;
        for (int g = lane; g < G; g += 32) {
            float best = -INFINITY;
            for (int j = 0; j < gs; ++j) best = fmaxf(best, logit[g * gs + j]);
            gscore[g] = best;
        }
        __syncwarp();
        // the `keep` best groups, one a round (the lower index wins a tie); a kept group's score is replaced by +infinity
        for (int r = 0; r < keep; ++r) {
            float best = -INFINITY;
            int where = 0x7fffffff;
            for (int g = lane; g < G; g += 32) {
                const float v = gscore[g];
                if (v != INFINITY && (where == 0x7fffffff || v > best)) {
                    best = v;
                    where = g;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int ow = __shfl_xor_sync(0xffffffffu, where, o);
                if (ow != 0x7fffffff && (where == 0x7fffffff || ob > best || (ob == best && ow < where))) {
                    best = ob;
                    where = ow;
                }
            }
            if (lane == 0 && where != 0x7fffffff) gscore[where] = INFINITY;      // kept
            __syncwarp();
        }
#pragma unroll
        for (int k = 0; k < PL; ++k) {
            const int e = lane + 32 * k;
            if (e < E && gscore[e / gs] != INFINITY) c[k] = -INFINITY;
        }
    }
    float mine = 0.0f;                                // lane j keeps the score s of the j-th chosen expert
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int where = 0x7fffffff;
#pragma unroll
        for (int k = 0; k < PL; ++k) {
            const int e = lane + 32 * k;
            if (e < E && c[k] != -INFINITY && (where == 0x7fffffff || c[k] > best || (c[k] == best && e < where))) {
                best = c[k];
                where = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, where, o);
            if (ow != 0x7fffffff && (where == 0x7fffffff || ob > best || (ob == best && ow < where))) {
                best = ob;
                where = ow;
            }
        }
        if (where != 0x7fffffff && (where & 31) == lane) {
#pragma unroll
            for (int k = 0; k < PL; ++k)
                if (k == (where >> 5)) c[k] = -INFINITY;
        }
        if (where == 0x7fffffff) where = 0;
        if (lane == j) mine = prob[where];
        if (lane == 0) ids[(long long)t * top + j] = where;
    }
    const float total = warp_sum(lane < top ? mine : 0.0f);
    if (lane < top) weights[(long long)t * top + lane] = mine / (total + 1e-20f) * scale;
}

// One block of 32 warps.  Warp w takes the w-th stretch of the pairs.  Shared: cnt[w][e], the pairs of expert e in
// stretch w, turned into the row at which stretch w's pairs of expert e begin; inside a stretch the pairs of an expert
// keep their order (lanes that hold the same expert find each other with match.any), so an expert's rows are its pairs in
// pair order, whatever the number of warps.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_pairs, int top, int E, int tile, int max_rows, int* __restrict__ row_of,
                int* __restrict__ src_tok, int* __restrict__ tile_expert) {
    extern __shared__ int sh[];
    int* cnt = sh;                 // [32][E]
    int* start = sh + 32 * E;      // [E]: first row of the expert's run
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per = ((n_pairs + 31) / 32 + 31) / 32 * 32;            // pairs per stretch, a multiple of 32
    const int p_begin = min(n_pairs, warp * per), p_end = min(n_pairs, p_begin + per);
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) cnt[i] = 0;
    for (int r = threadIdx.x; r < max_rows; r += blockDim.x) src_tok[r] = -1;
    for (int t = threadIdx.x; t < max_rows / tile; t += blockDim.x) tile_expert[t] = -1;
    __syncthreads();
    // a pair whose id is E or more belongs to an expert without matrices (an identity expert): it takes no row, and its
    // row_of is -1
    for (int p0 = p_begin; p0 < p_end; p0 += 32) {
        const int p = p0 + lane;
        const bool have = p < p_end && ids[p] < E;
        const int e = have ? ids[p] : -1 - lane;                     // lanes without a pair match nobody
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (have && (same & ((1u << lane) - 1u)) == 0) cnt[warp * E + e] += __popc(same);      // the first lane of each expert
        __syncwarp();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            int c = 0;
            for (int w = 0; w < 32; ++w) {
                const int here = cnt[w * E + e];
                cnt[w * E + e] = at + c;
                c += here;
            }
            const int tiles = (c + tile - 1) / tile;
            for (int t = 0; t < tiles; ++t) tile_expert[at / tile + t] = e;
            at += tiles * tile;
        }
    }
    __syncthreads();
    for (int p0 = p_begin; p0 < p_end; p0 += 32) {
        const int p = p0 + lane;
        const bool have = p < p_end && ids[p] < E;
        if (p < p_end && !have) row_of[p] = -1;
        const int e = have ? ids[p] : -1 - lane;
        const unsigned same = __match_any_sync(0xffffffffu, e);
        if (have) {
            const int row = cnt[warp * E + e] + __popc(same & ((1u << lane) - 1u));
            row_of[p] = row;
            src_tok[row] = p / top;
        }
        __syncwarp();
        if (have && (same & ((1u << lane) - 1u)) == 0) cnt[warp * E + e] += __popc(same);
        __syncwarp();
    }
}

constexpr int GL_TILE = 64;        // rows and columns of a block's tile
constexpr int GL_K = 16;

// out[row][j] = sum_k x[src(row)][k] · W[expert][j][k].  W: [E][N][K].  A block: 64 rows x 64 columns, 256 threads,
// a thread 4 x 4.  `tile` (rows per expert run granule) is a multiple of 64, so a block's rows share an expert.
template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(const TX* __restrict__ x, const int* __restrict__ src_tok, const TW* __restrict__ w,
                      const int* __restrict__ tile_expert, int tile, int N, int K, TO* __restrict__ out) {
    const int row0 = blockIdx.y * GL_TILE;
    const int e = tile_expert[row0 / tile];
    if (e < 0) return;
    const int col0 = blockIdx.x * GL_TILE;
    __shared__ float xs[GL_K][GL_TILE + 1];
    __shared__ float ws[GL_K][GL_TILE + 1];
    __shared__ int src[GL_TILE];
    if (threadIdx.x < GL_TILE) src[threadIdx.x] = src_tok != nullptr ? src_tok[row0 + threadIdx.x] : row0 + threadIdx.x;
    __syncthreads();
    const TW* we = w + (long long)e * N * K;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += GL_K) {
        for (int idx = threadIdx.x; idx < GL_TILE * GL_K; idx += 256) {
            const int r = idx / GL_K, k = idx % GL_K;
            const int s = src[r];
            xs[k][r] = (s >= 0 && k0 + k < K) ? to_float(x[(long long)s * K + k0 + k]) : 0.0f;
            const int c = col0 + r;
            ws[k][r] = (c < N && k0 + k < K) ? to_float(we[(long long)c * K + k0 + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GL_K; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (src[r] < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = col0 + tx * 4 + j;
            if (c < N) out[(long long)(row0 + r) * N + c] = from_float<TO>(acc[i][j]);
        }
    }
}

// rows[r] = x[src_tok[r]] (zeros for padding), for products that want their operand dense
// With `weights` (and row_of, top) a row is multiplied, in float32, by the weight of the (token, choice) pair it stands for:
// the pair is the one of the row's token whose row_of names this row.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ src_tok, int d, T* __restrict__ rows,
                                  const float* __restrict__ weights, const int* __restrict__ row_of, int top) {
    const int r = blockIdx.x;
    const int s = src_tok[r];
    float w = 1.0f;
    if (weights != nullptr && s >= 0) {
        for (int j = 0; j < top; ++j)
            if (row_of[(long long)s * top + j] == r) w = weights[(long long)s * top + j];
    }
    if (weights == nullptr) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) rows[(long long)r * d + i] = s >= 0 ? x[(long long)s * d + i] : from_float<T>(0.0f);
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            rows[(long long)r * d + i] = from_float<T>(s >= 0 ? w * to_float(x[(long long)s * d + i]) : 0.0f);
    }
}

// A negative row stands for the token's own input, `ident` [n][d] (TI), if given; else it adds nothing.
template <typename TI>
__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ weights,
                                   const TI* __restrict__ ident, int top, int d, float* __restrict__ out) {
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < top; ++j) {
            const int r = row_of[(long long)t * top + j];
            const float e = r >= 0 ? y[(long long)r * d + i] : (ident != nullptr ? to_float(ident[(long long)t * d + i]) : 0.0f);
            acc = weights != nullptr ? fmaf(weights[(long long)t * top + j], e, acc) : acc + e;
        }
        out[(long long)t * d + i] = acc;
    }
}

// x[t][i] += s1[i] · sum_slices y1[.][t][i] (+ s2[i] · sum_slices y2[.][t][i]); a null factor is one.  VEC floats a thread.
template <int VEC>
__global__ void scaled_add_kernel(float* __restrict__ x, const float* __restrict__ y1, int slices1, const float* __restrict__ s1,
                                  const float* __restrict__ y2, int slices2, const float* __restrict__ s2, long long total, int d) {
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= total) return;
    const int i = (int)(idx % d);
    float a[VEC], b[VEC], v[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) a[e] = b[e] = 0.0f;
    if (VEC == 4) {
        for (int s = 0; s < slices1; ++s) {
            const float4 t = *reinterpret_cast<const float4*>(y1 + (long long)s * total + idx);
            a[0] += t.x; a[1 % VEC] += t.y; a[2 % VEC] += t.z; a[3 % VEC] += t.w;
        }
        if (y2 != nullptr)
            for (int s = 0; s < slices2; ++s) {
                const float4 t = *reinterpret_cast<const float4*>(y2 + (long long)s * total + idx);
                b[0] += t.x; b[1 % VEC] += t.y; b[2 % VEC] += t.z; b[3 % VEC] += t.w;
            }
        const float4 t = *reinterpret_cast<const float4*>(x + idx);
        v[0] = t.x; v[1 % VEC] = t.y; v[2 % VEC] = t.z; v[3 % VEC] = t.w;
    } else {
        for (int s = 0; s < slices1; ++s) a[0] += y1[(long long)s * total + idx];
        if (y2 != nullptr)
            for (int s = 0; s < slices2; ++s) b[0] += y2[(long long)s * total + idx];
        v[0] = x[idx];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        v[e] += s1 != nullptr ? s1[i + e] * a[e] : a[e];
        if (y2 != nullptr) v[e] += s2 != nullptr ? s2[i + e] * b[e] : b[e];
    }
    if (VEC == 4) *reinterpret_cast<float4*>(x + idx) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
    else x[idx] = v[0];
}

// x[t][i] += s1[i] · sum_slices y1[.][t][i] + s2[i] · sum_j weights[t][j] · rows[row_of[t][j]][i]: the block's addition with
// the weighted sum of a token's expert rows made on the way (j in the order of the choices; float32).
template <int VEC>
__global__ void scaled_add_experts_kernel(float* __restrict__ x, const float* __restrict__ y1, int slices1, const float* __restrict__ s1,
                                          const float* __restrict__ rows, const int* __restrict__ row_of,
                                          const float* __restrict__ weights, int top, const float* __restrict__ s2,
                                          long long total, int d) {
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= total) return;
    const long long t = idx / d;
    const int i = (int)(idx - t * d);
    float a[VEC], b[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) a[e] = b[e] = 0.0f;
    for (int s = 0; s < slices1; ++s) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) a[e] += y1[(long long)s * total + idx + e];
    }
    for (int j = 0; j < top; ++j) {
        const float wj = weights[t * top + j];
        const float* r = rows + (long long)row_of[t * top + j] * d + i;
#pragma unroll
        for (int e = 0; e < VEC; ++e) b[e] = fmaf(wj, r[e], b[e]);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e)
        x[idx + e] += (s1 != nullptr ? s1[i + e] * a[e] : a[e]) + (s2 != nullptr ? s2[i + e] * b[e] : b[e]);
}

}  // namespace mlc

using namespace mlc;

// x: with w, the branch's input [n][K] of x_dtype (w float32 [E][K]); without w, the logits float32 [n][E] (K unused).
// weighting 0: the softmax over the chosen logits; 1: the sigmoid of each chosen logit, not renormalised.
extern "C" int mlc_moe_route(const void* x, int x_dtype, const float* w, const float* bias, int n, int E, int K, int top,
                             int weighting, int* ids, float* weights, void* stream) {
    if (n <= 0) return 0;
    if (weighting != 0 && weighting != 1) return MLC_ERR_UNSUPPORTED;
    if (E <= 0 || E > 32 * ROUTE_MAX_PER_LANE || top <= 0 || top > 32 || top > E || (w != nullptr && K <= 0)) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (w == nullptr || x_dtype == MLC_DTYPE_F32)
        (E <= 32 ? moe_route_kernel<float, 1> : moe_route_kernel<float, ROUTE_MAX_PER_LANE>)<<<n, 128, 0, s>>>((const float*)x, w, bias, n, E, K, top, weighting, ids, weights);
    else if (x_dtype == MLC_DTYPE_BF16)
        (E <= 32 ? moe_route_kernel<bf16, 1> : moe_route_kernel<bf16, ROUTE_MAX_PER_LANE>)<<<n, 128, 0, s>>>((const bf16*)x, w, bias, n, E, K, top, weighting, ids, weights);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

// x: the branch's input [n][K] of x_dtype; w float32 [E][K]; correction float32 [E] or null.  G groups of which `keep` stay
// (G <= 1 or keep >= G: no grouping; E must be a multiple of G).
extern "C" int mlc_moe_route_scored(const void* x, int x_dtype, const float* w, const float* correction, int n, int E, int K,
                                    int top, int G, int keep, float scale, int* ids, float* weights, void* stream) {
    if (n <= 0) return 0;
    if (E <= 0 || E > 32 * ROUTE_MAX_PER_LANE || top <= 0 || top > 32 || top > E || K <= 0 || w == nullptr) return MLC_ERR_BAD_SIZE;
    if (G > 1 && (E % G != 0 || keep < 1)) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (x_dtype == MLC_DTYPE_F32)
        (E <= 32 ? moe_route_scored_kernel<float, 1> : moe_route_scored_kernel<float, ROUTE_MAX_PER_LANE>)<<<n, 128, 0, s>>>((const float*)x, w, correction, n, E, K, top, G, keep, scale, ids, weights);
    else if (x_dtype == MLC_DTYPE_BF16)
        (E <= 32 ? moe_route_scored_kernel<bf16, 1> : moe_route_scored_kernel<bf16, ROUTE_MAX_PER_LANE>)<<<n, 128, 0, s>>>((const bf16*)x, w, correction, n, E, K, top, G, keep, scale, ids, weights);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_moe_plan(const int* ids, int n_pairs, int top, int E, int tile, int max_rows, int* row_of, int* src_tok,
                            int* tile_expert, void* stream) {
    if (n_pairs <= 0) return 0;
    if (E <= 0 || E > 256 || tile <= 0 || max_rows % tile != 0 || top <= 0) return MLC_ERR_BAD_SIZE;
    // every expert's run, rounded up to whole tiles, must fit
    const long long most = (long long)n_pairs + (long long)(E < n_pairs ? E : n_pairs) * (tile - 1);     // only experts that were chosen have a run
    if ((long long)max_rows < most - most % tile) return MLC_ERR_BAD_SIZE;
    moe_plan_kernel<<<1, 1024, 33 * E * sizeof(int), (cudaStream_t)stream>>>(ids, n_pairs, top, E, tile, max_rows, row_of,
                                                                            src_tok, tile_expert);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_grouped_linear(const void* x, int x_dtype, const int* src_tok, const void* w, int w_dtype,
                                  const int* tile_expert, int tile, int max_rows, int N, int K, void* out, int out_dtype,
                                  void* stream) {
    if (max_rows <= 0) return 0;
    if (tile % GL_TILE != 0 || max_rows % tile != 0 || N <= 0 || K <= 0) return MLC_ERR_BAD_SIZE;
    const dim3 grid((N + GL_TILE - 1) / GL_TILE, max_rows / GL_TILE);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int code = x_dtype * 4 + w_dtype * 2 + out_dtype;
#define MLC_GL(TX, TW, TO) \
    grouped_linear_kernel<TX, TW, TO><<<grid, 256, 0, s>>>((const TX*)x, src_tok, (const TW*)w, tile_expert, tile, N, K, (TO*)out)
    switch (code) {
        case 0: MLC_GL(float, float, float); break;
        case 1: MLC_GL(float, float, bf16); break;
        case 2: MLC_GL(float, bf16, float); break;
        case 3: MLC_GL(float, bf16, bf16); break;
        case 4: MLC_GL(bf16, float, float); break;
        case 5: MLC_GL(bf16, float, bf16); break;
        case 6: MLC_GL(bf16, bf16, float); break;
        case 7: MLC_GL(bf16, bf16, bf16); break;
        default: return MLC_ERR_BAD_DTYPE;
    }
#undef MLC_GL
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_moe_gather(const void* x, int dtype, const int* src_tok, int max_rows, int d, void* rows, const float* weights,
                              const int* row_of, int top, void* stream) {
    if (max_rows <= 0) return 0;
    if (d <= 0 || (weights != nullptr && (row_of == nullptr || top < 1))) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = d >= 256 ? 256 : 64;
    if (dtype == MLC_DTYPE_F32)
        moe_gather_kernel<float><<<max_rows, threads, 0, s>>>((const float*)x, src_tok, d, (float*)rows, weights, row_of, top);
    else if (dtype == MLC_DTYPE_BF16)
        moe_gather_kernel<bf16><<<max_rows, threads, 0, s>>>((const bf16*)x, src_tok, d, (bf16*)rows, weights, row_of, top);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_moe_combine(const float* y, const int* row_of, const float* weights, const void* ident, int ident_dtype, int n,
                               int top, int d, float* out, void* stream) {
    if (n <= 0) return 0;
    if (top <= 0 || d <= 0) return MLC_ERR_BAD_SIZE;
    if (ident != nullptr && ident_dtype == MLC_DTYPE_BF16)
        moe_combine_kernel<bf16><<<n, d >= 256 ? 256 : 64, 0, (cudaStream_t)stream>>>(y, row_of, weights, (const bf16*)ident, top, d, out);
    else
        moe_combine_kernel<float><<<n, d >= 256 ? 256 : 64, 0, (cudaStream_t)stream>>>(y, row_of, weights, (const float*)ident, top, d, out);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_scaled_add(float* x, const float* y1, int slices1, const float* s1, const float* y2, int slices2,
                              const float* s2, long long n, int d, void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || y1 == nullptr || slices1 < 1 || (y2 != nullptr && slices2 < 1)) return MLC_ERR_BAD_SIZE;
    const long long total = n * d;
    const bool vec = (d & 3) == 0 && ((((uintptr_t)x) | ((uintptr_t)y1) | ((uintptr_t)y2)) & 15) == 0;
    if (vec)
        scaled_add_kernel<4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, y1, slices1, s1, y2, slices2,
                                                                                                    s2, total, d);
    else
        scaled_add_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, y1, slices1, s1, y2, slices2, s2,
                                                                                                total, d);
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_scaled_add_experts(float* x, const float* y1, int slices1, const float* s1, const float* rows,
                                      const int* row_of, const float* weights, int top, const float* s2, long long n, int d,
                                      void* stream) {
    if (n <= 0) return 0;
    if (d <= 0 || y1 == nullptr || slices1 < 1 || top < 1) return MLC_ERR_BAD_SIZE;
    const long long total = n * d;
    if ((d & 3) == 0)
        scaled_add_experts_kernel<4><<<(unsigned)((total / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            x, y1, slices1, s1, rows, row_of, weights, top, s2, total, d);
    else
        scaled_add_experts_kernel<1><<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            x, y1, slices1, s1, rows, row_of, weights, top, s2, total, d);
    MLC_LAUNCH_CHECK();
    return 0;
}
