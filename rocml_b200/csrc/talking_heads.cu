// Attention whose heads' weights are mixed after the softmax, and whose queries and keys are normalised over the
// whole projection.
//
// With a'_h = sum_g M[h][g] a_g and head h reading the values of its own key/value head m(h), the result is
// o_h = sum_g M[h][g] (sum_j a_g(i, j) v_m(h)(j)): every query head's weights applied to the values of every stored
// head (the attention kernels' `cross` mode, result (g, m) for each pair), then a small product over g.
//
//   wide_norm_rope_cache   a token's projection row [q (nq * hd) | k (nkv * hd) | v (nkv * vd)] (in the activations' type,
//                 or 32-bit partial sums added first): q and k are each divided by their root mean square over ALL
//                 their heads together and multiplied by a weight vector of that width; the first rot entries of every
//                 head turn by the step's table (neighbouring pairs, or pairs half a rotation apart); query head h is
//                 multiplied by factor[h] (a temperature on its scores); q goes out padded to hdp a head, k and v into
//                 the token's place in the paged cache, padded alike.  32-bit until the stores.  One block a token.
//   talk_mix      out[t][h][:] = sum_g M[h][g] * o[t][pair (g, m(h))][:], 32-bit sums, padding dropped.  Prompts: a block a
//                 token with the token's pair results in shared memory; few tokens: a thread four values, straight from memory.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
template <typename IT>
__device__ __forceinline__ float sum_parts(const IT* p, size_t stride, int n_in) {
    float v = 0.f;
    for (int s = 0; s < n_in; ++s) v += to_f32(p[(size_t)s * stride]);
    return v;
}

// entry d of a head whose entries x[0 .. rot) turn: cs = (cos, sin) pairs of the token, half = rot / 2
__device__ __forceinline__ float turned(const float* x, int d, int rot, bool neighbours, const float* cs) {
    if (d >= rot) return x[d];
    const int half = rot >> 1;
    if (neighbours) {
        const int i = d >> 1;
        const float c = cs[2 * i], s = cs[2 * i + 1];
        return (d & 1) ? x[d] * c + x[d - 1] * s : x[d] * c - x[d + 1] * s;
    }
    const int i = d < half ? d : d - half;
    const float c = cs[2 * i], s = cs[2 * i + 1];
    return d < half ? x[d] * c - x[d + half] * s : x[d] * c + x[d - half] * s;
}

template <typename IT, typename AT>
__global__ void __launch_bounds__(256)
wide_norm_rope_cache_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int nq, int nkv, int hd,
                            int vd, int hdp, const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                            const float* __restrict__ factor, const float* __restrict__ cos_sin, int rot, int neighbours,
                            AT* __restrict__ q_out, int q_stride, AT* __restrict__ k_cache, AT* __restrict__ v_cache,
                            const int* __restrict__ positions, const int* __restrict__ slot_of_token,
                            const int* __restrict__ block_table, int max_pages) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float buf[];            // (nq + nkv) * hd floats + 33
    const int qw = nq * hd, kw = nkv * hd;
    float* kb = buf + qw;
    float* red = kb + kw;
    const int t = blockIdx.x;
    const int slot = slot_of_token[t];
    if (slot < 0) return;
    const IT* row = in + (size_t)t * row_stride;
    float sq = 0.f, sk = 0.f;
    if (((qw | kw | row_stride) & 3) == 0 && (in_stride & 3) == 0 && ((uintptr_t)in & (4 * sizeof(IT) - 1)) == 0) {
        for (int i = threadIdx.x * 4; i < qw + kw; i += blockDim.x * 4) {      // four values a load; a group of four lies in q or in k
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < n_in; ++s) {
                float p[4];
                load4(row + (size_t)s * in_stride + i, p);
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] += p[u];
            }
            store4(buf + i, v);
            const float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
            if (i < qw) sq += ss; else sk += ss;
        }
    } else {
        for (int i = threadIdx.x; i < qw + kw; i += blockDim.x) {
            const float v = sum_parts(row + i, in_stride, n_in);
            buf[i] = v;
            if (i < qw) sq += v * v; else sk += v * v;
        }
    }
    // both sums of squares in one pass over the block
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = sq; red[8 + (threadIdx.x >> 5)] = sk; }
    __syncthreads();
    sq = sk = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) { sq += red[w]; sk += red[8 + w]; }       // 256 threads: eight warps, added in their order
    const float inv_q = wq ? rsqrtf(sq / (float)qw + eps) : 1.f;
    const float inv_k = wk ? rsqrtf(sk / (float)kw + eps) : 1.f;
    for (int i = threadIdx.x; i < qw + kw; i += blockDim.x) {
        if (i < qw) { if (wq) buf[i] *= inv_q * wq[i]; }
        else if (wk) buf[i] *= inv_k * wk[i - qw];
    }
    __syncthreads();
    const float* cs = cos_sin ? cos_sin + (size_t)t * (rot >> 1) * 2 : nullptr;
    const int r = cs ? rot : 0;
    for (int i = threadIdx.x; i < nq * hdp; i += blockDim.x) {
        const int h = i / hdp, d = i - h * hdp;
        float v = 0.f;
        if (d < hd) v = turned(buf + h * hd, d, r, neighbours != 0, cs) * (factor ? factor[h] : 1.f);
        q_out[(size_t)t * q_stride + i] = from_f32<AT>(v);
    }
    const int pos = positions[t];
    const int page = block_table[(size_t)slot * max_pages + pos / RB_PAGE];
    if (page < 0) return;
    for (int i = threadIdx.x; i < nkv * hdp; i += blockDim.x) {
        const int h = i / hdp, d = i - h * hdp;
        const size_t at = (((size_t)page * nkv + h) * RB_PAGE + (pos % RB_PAGE)) * hdp + d;
        k_cache[at] = from_f32<AT>(d < hd ? turned(kb + h * hd, d, r, neighbours != 0, cs) : 0.f);
        v_cache[at] = from_f32<AT>(d < vd ? sum_parts(row + qw + kw + h * vd + d, in_stride, n_in) : 0.f);
    }
}

// The same, a block a token: the token's pair results are read once into shared memory (every one of them is needed by
// all the heads of its key/value group), then every thread forms four neighbouring values of a result head.
template <typename AT>
__global__ void __launch_bounds__(256)
talk_mix_row_kernel(const AT* __restrict__ o, int o_stride, const float* __restrict__ mix, AT* __restrict__ out, int out_stride,
                    int nq, int nkv, int hdp, int vd, const int* __restrict__ slot_of_token) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) uint8_t raw_sm[];
    AT* row = reinterpret_cast<AT*>(raw_sm);                              // [nq * nkv][hdp]
    float* m_s = reinterpret_cast<float*>(raw_sm + (((size_t)nq * nkv * hdp * sizeof(AT) + 15) & ~(size_t)15));   // [nq][nq]
    const int t = blockIdx.x;
    if (slot_of_token[t] < 0) return;
    const int width = nq * nkv * hdp;
    const AT* src = o + (size_t)t * o_stride;
    for (int i = threadIdx.x * 4; i < width; i += 256 * 4) {
        float x[4];
        load4(src + i, x);
        store4(row + i, x);
    }
    for (int i = threadIdx.x; i < nq * nq; i += 256) m_s[i] = mix[i];
    __syncthreads();
    const int gs = nq / nkv, vd4 = vd >> 2;
    for (int idx = threadIdx.x; idx < nq * vd4; idx += 256) {
        const int h = idx / vd4, d = (idx - h * vd4) * 4;
        const int m = h / gs;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int g = 0; g < nq; ++g) {
            const int a = g / gs;
            float x[4];
            load4(row + (size_t)((a * nkv + m) * gs + (g - a * gs)) * hdp + d, x);
            const float f = m_s[h * nq + g];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(f, x[j], acc[j]);
        }
        store4(out + (size_t)t * out_stride + (size_t)h * vd + d, acc);
    }
}

// The same, four neighbouring values a thread (sizes and addresses allow 4-element accesses).
template <typename AT>
__global__ void talk_mix4_kernel(const AT* __restrict__ o, int o_stride, const float* __restrict__ mix, AT* __restrict__ out,
                                 int out_stride, int nq, int nkv, int hdp, int vd, const int* __restrict__ slot_of_token, int T) {
    pdl_trigger();
    pdl_wait();
    const int vd4 = vd >> 2;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T * nq * vd4) return;
    const int d = (int)(idx % vd4) * 4;
    const int h = (int)((idx / vd4) % nq);
    const int t = (int)(idx / ((long long)vd4 * nq));
    if (slot_of_token[t] < 0) return;
    const int gs = nq / nkv, m = h / gs;
    const AT* row = o + (size_t)t * o_stride + d;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g0 = 0; g0 < nq; g0 += 4) {            // four heads' loads in flight
        float x[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int g = g0 + u, a = g / gs;
            if (g < nq) load4(row + (size_t)((a * nkv + m) * gs + (g - a * gs)) * hdp, x[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (g0 + u < nq) {
                const float f = mix[h * nq + g0 + u];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fmaf(f, x[u][j], acc[j]);
            }
        }
    }
    store4(out + (size_t)t * out_stride + (size_t)h * vd + d, acc);
}

template <typename AT>
__global__ void talk_mix_kernel(const AT* __restrict__ o, int o_stride, const float* __restrict__ mix, AT* __restrict__ out,
                                int out_stride, int nq, int nkv, int hdp, int vd, const int* __restrict__ slot_of_token, int T) {
    pdl_trigger();
    pdl_wait();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)T * nq * vd) return;
    const int d = (int)(idx % vd);
    const int h = (int)((idx / vd) % nq);
    const int t = (int)(idx / ((long long)vd * nq));
    if (slot_of_token[t] < 0) return;
    const int gs = nq / nkv, m = h / gs;
    const AT* row = o + (size_t)t * o_stride + d;
    float acc = 0.f;
    for (int g = 0; g < nq; ++g) {
        const int a = g / gs;
        const int pair = (a * nkv + m) * gs + (g - a * gs);
        acc = fmaf(mix[h * nq + g], to_f32(row[(size_t)pair * hdp]), acc);
    }
    out[(size_t)t * out_stride + (size_t)h * vd + d] = from_f32<AT>(acc);
}
}  // namespace

extern "C" int rb_wide_norm_rope_cache(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int nq,
                                       int nkv, int hd, int vd, int hdp, const float* wq, const float* wk, float eps,
                                       const float* factor, const float* cos_sin, int rot, int neighbours, void* q_out,
                                       int q_stride, void* k_cache, void* v_cache, int act_dtype, const int* positions,
                                       const int* slot_of_token, const int* block_table, int max_pages, int T, void* stream) {
    if (T <= 0) return RB_OK;
    if (nq <= 0 || nkv <= 0 || hd <= 0 || vd <= 0 || hdp < hd || hdp < vd || rot < 0 || (rot & 1) || rot > hd || n_in < 1)
        return RB_ERR_BAD_SIZE;
    const size_t smem = (size_t)((nq + nkv) * hd + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_WN(IT, AT)                                                                                                    \
    do {                                                                                                                 \
        auto k = wide_norm_rope_cache_kernel<IT, AT>;                                                                    \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
            if (e != cudaSuccess) return (int)e;                                                                         \
        }                                                                                                                \
        RB_LAUNCH((k), dim3(T), dim3(256), smem, s, (const IT*)in, n_in, (size_t)in_stride, row_stride, nq, nkv, hd, vd, \
                  hdp, wq, wk, eps, factor, cos_sin, rot, neighbours, (AT*)q_out, q_stride, (AT*)k_cache, (AT*)v_cache,  \
                  positions, slot_of_token, block_table, max_pages);                                                     \
    } while (0)
    if (in_dtype == RB_F32 && act_dtype == RB_BF16) RB_WN(float, bf);
    else if (in_dtype == RB_BF16 && act_dtype == RB_BF16) RB_WN(bf, bf);
    else if (in_dtype == RB_F32 && act_dtype == RB_F32) RB_WN(float, float);
    else return RB_ERR_BAD_DTYPE;
#undef RB_WN
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_talk_mix(const void* o, int o_stride, const float* mix, void* out, int out_stride, int nq, int nkv, int hdp,
                           int vd, int dtype, const int* slot_of_token, int T, void* stream) {
    if (T <= 0) return RB_OK;
    if (nq <= 0 || nkv <= 0 || nq % nkv || vd <= 0 || hdp < vd) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t esz = dtype == RB_BF16 ? 2 : 4;
    if ((vd & 3) == 0 && (hdp & 3) == 0 && (o_stride & 3) == 0 && (out_stride & 3) == 0 && ((uintptr_t)o & (4 * esz - 1)) == 0 &&
        ((uintptr_t)out & (4 * esz - 1)) == 0 && (dtype == RB_BF16 || dtype == RB_F32)) {
        // a block a token while the token's pair results fit shared memory
        const size_t row_bytes = (((size_t)nq * nkv * hdp * esz + 15) & ~(size_t)15) + (size_t)nq * nq * sizeof(float);
        if (row_bytes <= 160 * 1024 && T >= 64) {
            if (dtype == RB_BF16) {
                auto k = talk_mix_row_kernel<__nv_bfloat16>;
                if (row_bytes > 48 * 1024) {
                    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
                    if (e != cudaSuccess) return (int)e;
                }
                RB_LAUNCH((k), dim3(T), dim3(256), row_bytes, s, (const __nv_bfloat16*)o, o_stride, mix, (__nv_bfloat16*)out, out_stride,
                          nq, nkv, hdp, vd, slot_of_token);
            } else {
                auto k = talk_mix_row_kernel<float>;
                if (row_bytes > 48 * 1024) {
                    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
                    if (e != cudaSuccess) return (int)e;
                }
                RB_LAUNCH((k), dim3(T), dim3(256), row_bytes, s, (const float*)o, o_stride, mix, (float*)out, out_stride, nq, nkv, hdp,
                          vd, slot_of_token);
            }
            RB_LAUNCH_CHECK();
            return RB_OK;
        }
        const long long blocks4 = ((long long)T * nq * (vd >> 2) + 255) / 256;
        if (blocks4 > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
        if (dtype == RB_BF16)
            RB_LAUNCH((talk_mix4_kernel<__nv_bfloat16>), dim3((unsigned)blocks4), dim3(256), 0, s, (const __nv_bfloat16*)o, o_stride,
                      mix, (__nv_bfloat16*)out, out_stride, nq, nkv, hdp, vd, slot_of_token, T);
        else
            RB_LAUNCH((talk_mix4_kernel<float>), dim3((unsigned)blocks4), dim3(256), 0, s, (const float*)o, o_stride, mix,
                      (float*)out, out_stride, nq, nkv, hdp, vd, slot_of_token, T);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    const long long blocks = ((long long)T * nq * vd + 255) / 256;
    if (blocks > 0x7fffffffLL) return RB_ERR_BAD_SIZE;
    if (dtype == RB_BF16)
        RB_LAUNCH((talk_mix_kernel<__nv_bfloat16>), dim3((unsigned)blocks), dim3(256), 0, s, (const __nv_bfloat16*)o, o_stride, mix,
                  (__nv_bfloat16*)out, out_stride, nq, nkv, hdp, vd, slot_of_token, T);
    else if (dtype == RB_F32)
        RB_LAUNCH((talk_mix_kernel<float>), dim3((unsigned)blocks), dim3(256), 0, s, (const float*)o, o_stride, mix, (float*)out,
                  out_stride, nq, nkv, hdp, vd, slot_of_token, T);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
