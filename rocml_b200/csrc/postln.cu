// A layer whose norm follows the sum, and the blend of a token with the one before it.
//
//   postln        x <- rmsnorm(alpha * x + g * d) * w      per row of the 32-bit stream, in place; d is the sum of the
//                 sublayer's partial sums (added in their order), g an optional vector (the layer's scale on the
//                 sublayer's result), alpha a constant.  The sum, the statistics and the stream are 32-bit; the
//                 normalised row is also written in the activations' type when a product reads it next.
//                 One block a row, the row in shared memory; 16-byte accesses when the width allows.  In a step of one
//                 token a sequence the kernel can also blend the new row with the one the NEXT layer kept for the
//                 row's sequence (token_shift below, whose row before is then always the slot's), so that the next
//                 layer's blend needs no kernel of its own.
//   token_shift   h_t = x_t + (x_(t-1) - x_t) * mu   with x_(t-1) the row before in the same sequence; for the first
//                 row of a sequence's tokens in this step it is the row the sequence's slot kept from the step
//                 before (zeros at the start of a sequence).  The slot then receives the last row of this step.
//                 A block of the grid is (sequence, a share of its rows); the block that takes a sequence's
//                 first row is the only one that reads the slot's row, and it writes the new one after all its
//                 threads have read the old, so neither an earlier nor a later launch is needed for the hand-over.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int PL_THREADS = 256;

template <typename AT>
__global__ void __launch_bounds__(PL_THREADS)
postln_kernel(float* __restrict__ resid, const float* __restrict__ delta, int n_delta, size_t delta_stride,
              const float* __restrict__ gain, const float* __restrict__ w, float alpha, float eps,
              AT* __restrict__ out, const int* __restrict__ slot_of_token, int H, const float* __restrict__ next_mu,
              float* __restrict__ next_kept, AT* __restrict__ next_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row[];      // H floats + 33
    float* red = row + ((H + 3) & ~3);
    const int t = blockIdx.x;
    if (slot_of_token && slot_of_token[t] < 0) return;
    float* x = resid + (size_t)t * H;
    const float* d = delta ? delta + (size_t)t * H : nullptr;
    float ss = 0.f;
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += PL_THREADS * 4) {
            float v[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
            load4(x + i, v);
            for (int s = 0; s < n_delta; ++s) {
                float p[4];
                load4(d + (size_t)s * delta_stride + i, p);
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] += p[u];
            }
            if (gain) {
                float g[4];
                load4(gain + i, g);
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] *= g[u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                v[u] = fmaf(alpha, v[u], acc[u]);
                ss = fmaf(v[u], v[u], ss);
            }
            store4(row + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += PL_THREADS) {
            float acc = 0.f;
            for (int s = 0; s < n_delta; ++s) acc += d[(size_t)s * delta_stride + i];
            if (gain) acc *= gain[i];
            const float v = fmaf(alpha, x[i], acc);
            ss = fmaf(v, v, ss);
            row[i] = v;
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    float* kept = next_out ? next_kept + (size_t)slot_of_token[t] * H : nullptr;
    if ((H & 3) == 0) {
        for (int i = threadIdx.x * 4; i < H; i += PL_THREADS * 4) {
            float v[4], ww[4];
            load4(row + i, v);
            load4(w + i, ww);
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = v[u] * inv * ww[u];
            store4(x + i, v);
            if (out) store4(out + (size_t)t * H + i, v);
            if (next_out) {
                float before[4], m[4], hrow[4];
                load4(kept + i, before);
                load4(next_mu + i, m);
#pragma unroll
                for (int u = 0; u < 4; ++u) hrow[u] = fmaf(before[u] - v[u], m[u], v[u]);
                store4(next_out + (size_t)t * H + i, hrow);
                store4(kept + i, v);
            }
        }
    } else {
        for (int i = threadIdx.x; i < H; i += PL_THREADS) {
            const float v = row[i] * inv * w[i];
            x[i] = v;
            if (out) out[(size_t)t * H + i] = from_f32<AT>(v);
            if (next_out) {
                next_out[(size_t)t * H + i] = from_f32<AT>(fmaf(kept[i] - v, next_mu[i], v));
                kept[i] = v;
            }
        }
    }
}

template <typename AT>
__global__ void __launch_bounds__(PL_THREADS)
token_shift_kernel(const float* __restrict__ x, const float* __restrict__ mu, float* __restrict__ kept,
                   const int* __restrict__ seq_slot, const int* __restrict__ cu_q, AT* __restrict__ out, int H) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    if (t_end <= t_begin) return;
    float* mine = kept + (size_t)slot * H;
    const bool vec = (H & 3) == 0 && ((((uintptr_t)x | (uintptr_t)mu | (uintptr_t)kept) & 15) == 0) && ((uintptr_t)out & (4 * sizeof(AT) - 1)) == 0;
    for (int t = t_begin + blockIdx.y; t < t_end; t += gridDim.y) {
        const float* cur = x + (size_t)t * H;
        const float* before = t == t_begin ? mine : cur - H;
        if (vec) {
            for (int i = threadIdx.x * 4; i < H; i += PL_THREADS * 4) {
                float c[4], p[4], m[4];
                load4(cur + i, c);
                load4(before + i, p);
                load4(mu + i, m);
#pragma unroll
                for (int u = 0; u < 4; ++u) c[u] = fmaf(p[u] - c[u], m[u], c[u]);
                store4(out + (size_t)t * H + i, c);
            }
        } else {
            for (int i = threadIdx.x; i < H; i += PL_THREADS) {
                const float c = cur[i];
                out[(size_t)t * H + i] = from_f32<AT>(fmaf(before[i] - c, mu[i], c));
            }
        }
    }
    if (blockIdx.y == 0) {
        __syncthreads();           // every thread of this block has read the slot's old row
        const float* last = x + (size_t)(t_end - 1) * H;
        for (int i = threadIdx.x; i < H; i += PL_THREADS) mine[i] = last[i];
    }
}
}  // namespace

extern "C" int rb_postln(float* resid, const float* delta, int n_delta, long long delta_stride, const float* gain,
                         const float* w, float alpha, float eps, void* out, int out_dtype, const int* slot_of_token,
                         int n_rows, int H, const float* next_mu, float* next_kept, void* next_out, void* stream) {
    if (n_rows <= 0) return RB_OK;
    if (H <= 0 || n_delta < 0 || (n_delta > 0 && !delta) || !w) return RB_ERR_BAD_SIZE;
    if (next_out && (!next_mu || !next_kept || !slot_of_token)) return RB_ERR_BAD_SIZE;
    if ((H & 3) == 0 && next_out && ((((uintptr_t)next_mu | (uintptr_t)next_kept) & 15) || ((uintptr_t)next_out & 7)))
        return RB_ERR_BAD_ALIGN;
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    if ((H & 3) == 0 && ((((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)w) & 15) ||
                         (n_delta > 1 && (delta_stride & 3)) || (out && ((uintptr_t)out & 7))))
        return RB_ERR_BAD_ALIGN;
    cudaStream_t s = (cudaStream_t)stream;
    if ((!out && !next_out) || out_dtype == RB_F32) {
        auto k = postln_kernel<float>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        RB_LAUNCH((k), dim3(n_rows), dim3(PL_THREADS), smem, s, resid, delta, n_delta, (size_t)delta_stride, gain, w, alpha, eps,
                  (float*)out, slot_of_token, H, next_mu, next_kept, (float*)next_out);
    } else if (out_dtype == RB_BF16) {
        auto k = postln_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        RB_LAUNCH((k), dim3(n_rows), dim3(PL_THREADS), smem, s, resid, delta, n_delta, (size_t)delta_stride, gain, w, alpha, eps,
                  (__nv_bfloat16*)out, slot_of_token, H, next_mu, next_kept, (__nv_bfloat16*)next_out);
    } else {
        return RB_ERR_BAD_DTYPE;
    }
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_token_shift(const float* x, const float* mu, float* kept, const int* seq_slot, const int* cu_q,
                              int n_seqs, int max_q_len, void* out, int out_dtype, int H, void* stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return RB_OK;
    if (H <= 0 || n_seqs > 0x7fffffff) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid(n_seqs, max_q_len < 2048 ? max_q_len : 2048);
    if (out_dtype == RB_F32)
        RB_LAUNCH((token_shift_kernel<float>), grid, dim3(PL_THREADS), 0, s, x, mu, kept, seq_slot, cu_q, (float*)out, H);
    else if (out_dtype == RB_BF16)
        RB_LAUNCH((token_shift_kernel<__nv_bfloat16>), grid, dim3(PL_THREADS), 0, s, x, mu, kept, seq_slot, cu_q,
                  (__nv_bfloat16*)out, H);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
