// Latent attention: keys and values of all heads are expansions of one normed low-rank latent c per token, beside one
// rotated key part that the heads share.  Only [c | rotated part] is cached, one row per token, and attention runs
// on the cached rows themselves:
//
//   score_h(i, j) = (W_uk,hᵀ q_plain,h(i)) · c(j) + q_rot,h(i) · k_rot(j)         the key expansion moved to the query
//   out_h(i)      = W_uv,h (sum_j p_h(i, j) c(j))                                  the value expansion moved behind the sum
//
// which is attention with one key/value head of size rank + rot that every query head reads, values being the first
// `rank` entries of the key rows.  Two kernels here: `latent_prepare` (norm of the latent, rotation of the shared key
// part and of the queries' rotated parts, the cache write) and `head_project` (a small matrix product per head, for
// the two moved expansions), both with float32 arithmetic.
#include "common.cuh"

namespace mlc {

// A block per token.  proj row: q heads ([dim plain | rot rotated] each) at q_col, then [rank latent | rot] at kv_col.
// Cache row (kv head 0): [c · (rsqrt(mean c² + eps) · gain) | rotated key part | zeros up to D].
// q_out [n][H][D]: entries [rank, rank + rot) get the rotated query part, [rank + rot, D) zeros; [0, rank) is left to
// the projection that follows.  q_plain_out [n][H][dim] float32: the unrotated query parts, dense.
// `qsrc` (row stride `q_stride`) holds the query heads at q_col; it may be `proj` itself or another matrix (queries that
// come out of a product of their own, behind a query latent).  `interleaved`: the rotation pairs entry 2i with 2i + 1
// instead of i with i + rot/2; the table is the same, [position][pair] (cos, sin).
template <typename T>
__global__ void latent_prepare_kernel(const float* __restrict__ proj, long long stride, const float* __restrict__ qsrc,
                                      long long q_stride, int interleaved, int q_col, int kv_col,
                                      const float* __restrict__ gain, float eps, const int* __restrict__ positions,
                                      const int* __restrict__ tok_seq, const float2* __restrict__ rope, int rope_positions,
                                      int H, int dim, int rot, int rank, int D, T* __restrict__ q_out, int write_cache,
                                      PagedKV cache) {
    const int n = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const float* row = proj + (long long)n * stride;
    const int p = positions[n];
    const int half = rot >> 1;
    const float2* cs = (rope != nullptr && half > 0) ? rope + (long long)min(p, rope_positions - 1) * half : nullptr;
    for (int head = warp; head < H + 1; head += n_warps) {
        if (head < H) {
            const float* src = qsrc + (long long)n * q_stride + q_col + (long long)head * (dim + rot) + dim;
            T* dst = q_out + ((long long)n * H + head) * D + rank;
            for (int i = lane; i < D - rank; i += 32) {
                float v = 0.0f;
                if (i < rot) {
                    v = src[i];
                    if (cs != nullptr) {
                        const bool first = interleaved ? !(i & 1) : i < half;
                        const int j = interleaved ? i >> 1 : (i < half ? i : i - half);
                        const float w = src[interleaved ? i ^ 1 : (i < half ? i + half : i - half)];
                        const float2 t = cs[j];
                        v = first ? v * t.x - w * t.y : v * t.x + w * t.y;
                    }
                }
                dst[i] = from_float<T>(v);
            }
        } else if (write_cache) {
            const float* src = row + kv_col;
            T* dst = (T*)cache.k_pool + paged_offset(cache, tok_seq[n], p, 0);
            float ss = 0.0f;
            for (int i = lane; i < rank; i += 32) ss += src[i] * src[i];
            ss = warp_sum(ss);
            const float f = 1.0f / sqrtf(ss / (float)rank + eps);
            for (int i = lane; i < D; i += 32) {
                float v = 0.0f;
                if (i < rank) {
                    v = src[i] * f * gain[i];
                } else if (i < rank + rot) {
                    const int k = i - rank;
                    v = src[i];
                    if (cs != nullptr) {
                        const bool first = interleaved ? !(k & 1) : k < half;
                        const int j = interleaved ? k >> 1 : (k < half ? k : k - half);
                        const float w = src[rank + (interleaved ? k ^ 1 : (k < half ? k + half : k - half))];
                        const float2 t = cs[j];
                        v = first ? v * t.x - w * t.y : v * t.x + w * t.y;
                    }
                }
                dst[i] = from_float<T>(v);
            }
        }
    }
}

constexpr int HP_TILE = 64;
constexpr int HP_K = 16;

// out[t][h][j] = sum_d in[t][h][d] · W[h][d][j] for j < n_out, d < n_in; every operand by strides (in elements):
// in at t*in_st + h*in_sh + d, W at h*w_sh + d*w_sd + j*w_sj, out at t*out_st + h*out_sh + j.
template <typename TI, typename TW, typename TO>
__global__ void __launch_bounds__(256)
head_project_kernel(const TI* __restrict__ in, long long in_st, long long in_sh, const TW* __restrict__ w, long long w_sh,
                    long long w_sd, long long w_sj, TO* __restrict__ out, long long out_st, long long out_sh, int n, int n_in,
                    int n_out) {
    const int h = blockIdx.z;
    const int t0 = blockIdx.y * HP_TILE, j0 = blockIdx.x * HP_TILE;
    __shared__ float xs[HP_K][HP_TILE + 1];
    __shared__ float ws[HP_K][HP_TILE + 1];
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int d0 = 0; d0 < n_in; d0 += HP_K) {
        for (int idx = threadIdx.x; idx < HP_TILE * HP_K; idx += 256) {
            const int r = idx / HP_K, k = idx % HP_K;
            xs[k][r] = (t0 + r < n && d0 + k < n_in) ? to_float(in[(long long)(t0 + r) * in_st + h * in_sh + d0 + k]) : 0.0f;
            // W: walk it the way it lies in memory
            const int rr = w_sj == 1 ? idx % HP_TILE : r, kk = w_sj == 1 ? idx / HP_TILE : k;
            ws[kk][rr] = (j0 + rr < n_out && d0 + kk < n_in) ? to_float(w[h * w_sh + (long long)(d0 + kk) * w_sd + (long long)(j0 + rr) * w_sj]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < HP_K; ++k) {
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
        const int t = t0 + ty * 4 + i;
        if (t >= n) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = j0 + tx * 4 + j;
            if (c < n_out) out[(long long)t * out_st + h * out_sh + c] = from_float<TO>(acc[i][j]);
        }
    }
}

}  // namespace mlc

using namespace mlc;

extern "C" int mlc_latent_prepare(const float* proj, long long stride, const float* qsrc, long long q_stride, int interleaved,
                                  int q_col, int kv_col, const float* gain, float eps,
                                  const int* positions, const int* tok_seq, const void* rope_table, int rope_positions, int n,
                                  int H, int dim, int rot, int rank, int D, void* q_out, int dtype, int write_cache,
                                  void* k_pool, const int* page_table, long long entry_offset, int pages_per_seq,
                                  int page_size, void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || dim < 0 || rot < 0 || (rot & 1) || rank <= 0 || D < rank + rot) return MLC_ERR_BAD_SIZE;
    PagedKV c{k_pool, k_pool, page_table, entry_offset, pages_per_seq, page_size, 1, D};
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 32 * (H + 1 < 8 ? H + 1 : 8);
    if (dtype == MLC_DTYPE_F32)
        latent_prepare_kernel<float><<<n, threads, 0, s>>>(proj, stride, qsrc, q_stride, interleaved, q_col, kv_col, gain, eps, positions, tok_seq,
                                                           (const float2*)rope_table, rope_positions, H, dim, rot, rank, D,
                                                           (float*)q_out, write_cache, c);
    else if (dtype == MLC_DTYPE_BF16)
        latent_prepare_kernel<bf16><<<n, threads, 0, s>>>(proj, stride, qsrc, q_stride, interleaved, q_col, kv_col, gain, eps, positions, tok_seq,
                                                          (const float2*)rope_table, rope_positions, H, dim, rot, rank, D,
                                                          (bf16*)q_out, write_cache, c);
    else
        return MLC_ERR_BAD_DTYPE;
    MLC_LAUNCH_CHECK();
    return 0;
}

extern "C" int mlc_head_project(const void* in, int in_dtype, long long in_st, long long in_sh, const void* w, int w_dtype,
                                long long w_sh, long long w_sd, long long w_sj, void* out, int out_dtype, long long out_st,
                                long long out_sh, int n, int H, int n_in, int n_out, void* stream) {
    if (n <= 0) return 0;
    if (H <= 0 || H > 65535 || n_in <= 0 || n_out <= 0) return MLC_ERR_BAD_SIZE;
    const dim3 grid((n_out + HP_TILE - 1) / HP_TILE, (n + HP_TILE - 1) / HP_TILE, H);
    if (grid.y > 65535) return MLC_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int code = in_dtype * 4 + w_dtype * 2 + out_dtype;
#define MLC_HP(TI, TW, TO)                                                                                                  \
    head_project_kernel<TI, TW, TO><<<grid, 256, 0, s>>>((const TI*)in, in_st, in_sh, (const TW*)w, w_sh, w_sd, w_sj, (TO*)out, \
                                                         out_st, out_sh, n, n_in, n_out)
    switch (code) {
        case 0: MLC_HP(float, float, float); break;
        case 1: MLC_HP(float, float, bf16); break;
        case 2: MLC_HP(float, bf16, float); break;
        case 3: MLC_HP(float, bf16, bf16); break;
        case 4: MLC_HP(bf16, float, float); break;
        case 5: MLC_HP(bf16, float, bf16); break;
        case 6: MLC_HP(bf16, bf16, float); break;
        case 7: MLC_HP(bf16, bf16, bf16); break;
        default: return MLC_ERR_BAD_DTYPE;
    }
#undef MLC_HP
    MLC_LAUNCH_CHECK();
    return 0;
}
