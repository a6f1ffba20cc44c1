// What stands between a latent-attention layer's input projection and its attention.
//
// The projection's rows are [queries (q_width) | latent (rank) | gate logits (n_gate)], as the matrix
// product left them: S partial sums of 32-bit rows, or one row in the activations' type.  For every
// token of the step, one block
//   * adds the partial sums,
//   * normalises the latent: c = x * rsqrt(mean(x^2) + eps) * w (32-bit), and writes it to the token's
//     place in the paged cache ([pages][1][64][rank], the layer's only cached tensor),
//   * writes the queries in the activations' type when they arrived as partial sums (q_out absent: they
//     stay where they are),
//   * writes sigmoid(gate logit) per head in 32-bit.
// Padding tokens (slot -1) are skipped.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
// The sum of up to n_in partial sums `stride` apart, in their order, eight loads in flight at a time.
template <typename IT>
__device__ __forceinline__ float sum_parts(const IT* p, size_t stride, int n_in) {
    float v = 0.f;
    for (int s0 = 0; s0 < n_in; s0 += 8) {
        float d[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) d[j] = s0 + j < n_in ? to_f32(p[(size_t)(s0 + j) * stride]) : 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) v += d[j];
    }
    return v;
}

template <typename IT, typename AT, typename WT>
__global__ void __launch_bounds__(256)
latent_prep_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int q_width, int rank, int n_gate,
                   const WT* __restrict__ w, float eps, AT* __restrict__ q_out, int q_stride, float* __restrict__ gate_out,
                   AT* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                   const int* __restrict__ block_table, int max_pages) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float buf[];          // rank floats + 33
    float* red = buf + rank;
    const int t = blockIdx.x;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    const IT* row = in + (size_t)t * row_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
        const float v = sum_parts(row + q_width + i, in_stride, n_in);
        buf[i] = v;
        ss += v * v;
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)rank + eps);
    const int pos = positions[t];
    const int page = block_table[(size_t)slot * max_pages + pos / RB_PAGE];
    if (page >= 0) {
        AT* dst = cache + ((size_t)page * RB_PAGE + (pos % RB_PAGE)) * rank;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f32<AT>(buf[i] * inv * to_f32(w[i]));
    }
    if (q_out) {
        for (int i = threadIdx.x; i < q_width; i += blockDim.x) {
            q_out[(size_t)t * q_stride + i] = from_f32<AT>(sum_parts(row + i, in_stride, n_in));
        }
    }
    for (int i = threadIdx.x; i < n_gate; i += blockDim.x) {
        const float v = sum_parts(row + q_width + rank + i, in_stride, n_in);
        gate_out[(size_t)t * n_gate + i] = 1.f / (1.f + expf(-v));
    }
}

// The same for a layer whose queries pass through a latent of their own and whose keys carry a rotated part:
// rows are [query latent (q_rank) | latent (rank) | rotated key part (rot) | gate logits (n_gate)].  The query latent
// is normalised with wq and written out for the product that unfolds it; the latent is normalised with wc and
// written to the token's place in the cache, followed by the rotated key part (pairs (i, i + rot / 2) turned by the
// step's table of cosines and sines) and zeros up to the cache's row width `dp`.  All 32-bit until the stores.
template <typename IT, typename AT>
__global__ void __launch_bounds__(256)
latent_rot_prep_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int q_rank, int rank, int rot,
                       int n_gate, const float* __restrict__ wq, const float* __restrict__ wc, float eps,
                       AT* __restrict__ cq_out, int cq_stride, float* __restrict__ gate_out, AT* __restrict__ cache, int dp,
                       const float* __restrict__ cos_sin, const int* __restrict__ positions,
                       const int* __restrict__ slot_of_token, const int* __restrict__ block_table, int max_pages) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float buf[];          // q_rank + rank + rot floats + 33
    float* cb = buf + q_rank;
    float* red = cb + rank + rot;
    const int t = blockIdx.x;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    const IT* row = in + (size_t)t * row_stride;
    float sq = 0.f, sc = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
        const float v = sum_parts(row + i, in_stride, n_in);
        buf[i] = v;
        sq += v * v;
    }
    for (int i = threadIdx.x; i < rank + rot; i += blockDim.x) {
        const float v = sum_parts(row + q_rank + i, in_stride, n_in);
        cb[i] = v;
        if (i < rank) sc += v * v;
    }
    const float inv_q = q_rank > 0 ? rsqrtf(block_sum(sq, red) / (float)q_rank + eps) : 0.f;
    const float inv_c = rsqrtf(block_sum(sc, red) / (float)rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
        cq_out[(size_t)t * cq_stride + i] = from_f32<AT>(buf[i] * inv_q * wq[i]);
    const int pos = positions[t];
    const int page = block_table[(size_t)slot * max_pages + pos / RB_PAGE];
    if (page >= 0) {
        AT* dst = cache + ((size_t)page * RB_PAGE + (pos % RB_PAGE)) * dp;
        const int half = rot >> 1;
        const float* cs = cos_sin + (size_t)t * half * 2;
        for (int i = threadIdx.x; i < dp; i += blockDim.x) {
            float v = 0.f;
            if (i < rank) {
                v = cb[i] * inv_c * wc[i];
            } else if (i < rank + rot) {
                const int d = i - rank, j = d < half ? d : d - half;
                const float c = cs[2 * j], sn = cs[2 * j + 1];
                v = d < half ? cb[rank + d] * c - cb[rank + d + half] * sn : cb[rank + d] * c + cb[rank + d - half] * sn;
            }
            dst[i] = from_f32<AT>(v);
        }
    }
    for (int i = threadIdx.x; i < n_gate; i += blockDim.x) {
        const float v = sum_parts(row + q_rank + rank + rot + i, in_stride, n_in);
        gate_out[(size_t)t * n_gate + i] = 1.f / (1.f + expf(-v));
    }
}

// The rotated part of every query head, turned and placed behind the folded part of its row: head h of `q` is
// [dim plain | rot rotated]; folded[t][h * dp + rank + i] receives the turned entries, zeros follow up to dp.
template <typename AT>
__global__ void latent_q_rot_kernel(const AT* __restrict__ q, int q_stride, int heads, int dim, int rot, int rank, int dp,
                                    const float* __restrict__ cos_sin, AT* __restrict__ folded, int f_stride,
                                    const int* __restrict__ slot_of_token, int T) {
    pdl_trigger();
    pdl_wait();
    const int tail = dp - rank;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T * heads * tail) return;
    const int d = (int)(idx % tail);
    const int h = (int)((idx / tail) % heads);
    const int t = (int)(idx / ((long long)tail * heads));
    if (slot_of_token[t] < 0) return;
    float v = 0.f;
    if (d < rot) {
        const int half = rot >> 1, j = d < half ? d : d - half;
        const float* cs = cos_sin + ((size_t)t * half + j) * 2;
        const AT* src = q + (size_t)t * q_stride + (size_t)h * (dim + rot) + dim;
        const float a = to_f32(src[d]), b = to_f32(src[d < half ? d + half : d - half]);
        v = d < half ? a * cs[0] - b * cs[1] : a * cs[0] + b * cs[1];
    }
    folded[(size_t)t * f_stride + (size_t)h * dp + rank + d] = from_f32<AT>(v);
}

template <typename IT, typename AT, typename WT>
int launch_prep(const void* in, int n_in, long long in_stride, int row_stride, int q_width, int rank, int n_gate,
                const void* w, float eps, void* q_out, int q_stride, float* gate_out, void* cache, const int* positions,
                const int* slot_of_token, const int* block_table, int max_pages, int T, cudaStream_t s) {
    const size_t smem = (size_t)(rank + 33) * sizeof(float);
    if (smem > 48 * 1024) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((latent_prep_kernel<IT, AT, WT>), dim3(T), dim3(256), smem, s, (const IT*)in, n_in, (size_t)in_stride, row_stride,
              q_width, rank, n_gate, (const WT*)w, eps, (AT*)q_out, q_stride, gate_out, (AT*)cache, positions, slot_of_token,
              block_table, max_pages);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

extern "C" int rb_latent_prep(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_width,
                              int rank, int n_gate, const void* w, int w_dtype, float eps, void* q_out, int q_stride,
                              float* gate_out, void* cache, int act_dtype, const int* positions, const int* slot_of_token,
                              const int* block_table, int max_pages, int T, void* stream) {
    if (T <= 0) return RB_OK;
    if (rank <= 0 || n_in < 1 || (n_gate > 0 && !gate_out)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_LP(IT, AT, WT) return launch_prep<IT, AT, WT>(in, n_in, in_stride, row_stride, q_width, rank, n_gate, w, eps, q_out, \
                                                        q_stride, gate_out, cache, positions, slot_of_token, block_table,   \
                                                        max_pages, T, s)
    if (in_dtype == RB_F32 && act_dtype == RB_BF16 && w_dtype == RB_BF16) RB_LP(float, bf, bf);
    if (in_dtype == RB_F32 && act_dtype == RB_BF16 && w_dtype == RB_F32) RB_LP(float, bf, float);
    if (in_dtype == RB_BF16 && act_dtype == RB_BF16 && w_dtype == RB_BF16) RB_LP(bf, bf, bf);
    if (in_dtype == RB_BF16 && act_dtype == RB_BF16 && w_dtype == RB_F32) RB_LP(bf, bf, float);
    if (in_dtype == RB_F32 && act_dtype == RB_F32 && w_dtype == RB_F32) RB_LP(float, float, float);
    if (in_dtype == RB_F32 && act_dtype == RB_F32 && w_dtype == RB_BF16) RB_LP(float, float, bf);
#undef RB_LP
    return RB_ERR_BAD_DTYPE;
}

extern "C" int rb_latent_rot_prep(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_rank,
                                  int rank, int rot, int n_gate, const float* wq, const float* wc, float eps, void* cq_out,
                                  int cq_stride, float* gate_out, void* cache, int dp, int act_dtype, const float* cos_sin,
                                  const int* positions, const int* slot_of_token, const int* block_table, int max_pages,
                                  int T, void* stream) {
    if (T <= 0) return RB_OK;
    if (rank <= 0 || q_rank < 0 || rot < 0 || (rot & 1) || dp < rank + rot || n_in < 1 || (n_gate > 0 && !gate_out) ||
        (rot > 0 && !cos_sin) || (q_rank > 0 && (!cq_out || !wq)))
        return RB_ERR_BAD_SIZE;
    const size_t smem = (size_t)(q_rank + rank + rot + 33) * sizeof(float);
    if (smem > 48 * 1024) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_LR(IT, AT) RB_LAUNCH((latent_rot_prep_kernel<IT, AT>), dim3(T), dim3(256), smem, s, (const IT*)in, n_in,            \
                                (size_t)in_stride, row_stride, q_rank, rank, rot, n_gate, wq, wc, eps, (AT*)cq_out, cq_stride, \
                                gate_out, (AT*)cache, dp, cos_sin, positions, slot_of_token, block_table, max_pages)
    if (in_dtype == RB_F32 && act_dtype == RB_BF16) RB_LR(float, bf);
    else if (in_dtype == RB_BF16 && act_dtype == RB_BF16) RB_LR(bf, bf);
    else if (in_dtype == RB_F32 && act_dtype == RB_F32) RB_LR(float, float);
    else return RB_ERR_BAD_DTYPE;
#undef RB_LR
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_latent_q_rot(const void* q, int q_stride, int heads, int dim, int rot, int rank, int dp,
                               const float* cos_sin, void* folded, int f_stride, int dtype, const int* slot_of_token, int T,
                               void* stream) {
    if (T <= 0 || dp == rank) return RB_OK;
    if (heads <= 0 || dim < 0 || rot < 0 || (rot & 1) || dp < rank + rot || (rot > 0 && !cos_sin)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const long long n = (long long)T * heads * (dp - rank);
    const long long blocks = (n + 255) / 256;
    if (blocks > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
    if (dtype == RB_BF16)
        RB_LAUNCH((latent_q_rot_kernel<__nv_bfloat16>), dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)q, q_stride,
                  heads, dim, rot, rank, dp, cos_sin, (__nv_bfloat16*)folded, f_stride, slot_of_token, T);
    else if (dtype == RB_F32)
        RB_LAUNCH((latent_q_rot_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, s, (const float*)q, q_stride, heads, dim,
                  rot, rank, dp, cos_sin, (float*)folded, f_stride, slot_of_token, T);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
