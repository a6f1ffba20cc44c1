// Embedding gather, fused residual-add + RMSNorm, SiLU(gate) * up, casts.
//
// All arithmetic is 32-bit; only loads and stores use the storage types.
#include "common.cuh"
#include "api.h"

using namespace rb;

// ---- embedding: resid[t, :] = f32(table[ids[t], :]) --------------------------------------
// Replaces the reference's embedding_f16_f32 (rocml-kernels/kernels/embedding.hip:6-18).
template <typename WT>
__global__ void embedding_kernel(const int* __restrict__ ids, const WT* __restrict__ table,
                                 float* __restrict__ out, int H, int vocab, int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= vocab) {  // a token id outside the table: record it, write zeros
        if (threadIdx.x == 0 && status) atomicExch(status, RB_ERR_BAD_SIZE);
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const WT* row = table + (size_t)id * H;
    if (sizeof(WT) == 2 && H % 8 == 0 && (((uintptr_t)table | (uintptr_t)out) & 15) == 0) {
        // 16 bytes a load, and a thread's loads all requested before the first is used: a row of a table of a
        // gigabyte comes from memory, and loads taken one after the other would each wait for it
        constexpr int UNROLL = 4;
        const int n8 = H / 8;
        for (int i0 = threadIdx.x; i0 < n8; i0 += blockDim.x * UNROLL) {
            uint4 raw[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * blockDim.x;
                raw[u] = i < n8 ? reinterpret_cast<const uint4*>(row)[i] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int i = i0 + u * blockDim.x;
                if (i >= n8) continue;
                const uint32_t ws[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
                float4 lo, hi;
                lo.x = __uint_as_float(ws[0] << 16); lo.y = __uint_as_float(ws[0] & 0xFFFF0000u);
                lo.z = __uint_as_float(ws[1] << 16); lo.w = __uint_as_float(ws[1] & 0xFFFF0000u);
                hi.x = __uint_as_float(ws[2] << 16); hi.y = __uint_as_float(ws[2] & 0xFFFF0000u);
                hi.z = __uint_as_float(ws[3] << 16); hi.w = __uint_as_float(ws[3] & 0xFFFF0000u);
                reinterpret_cast<float4*>(o)[2 * i] = lo;
                reinterpret_cast<float4*>(o)[2 * i + 1] = hi;
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

extern "C" int rb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T,
                            int H, int vocab, int* status, void* stream) {
    if (T <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == RB_BF16)
        RB_LAUNCH((embedding_kernel<__nv_bfloat16>), dim3(T), dim3(threads), 0, s, ids, (const __nv_bfloat16*)table, out, H, vocab, status);
    else if (table_dtype == RB_F32)
        RB_LAUNCH((embedding_kernel<float>), dim3(T), dim3(threads), 0, s, ids, (const float*)table, out, H, vocab, status);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- fused residual add + RMSNorm ---------------------------------------------------------
// r = resid[row] + sum_s delta[s][row] (+ sum_s delta_b[s][row])   (s in fixed order, first all of delta, then all of
// delta_b, so the sum never depends on the batch and equals adding the two groups one after the other)
// if write_back: resid[row] = r
// out[i] = r * rsqrt(mean(r^2) + eps) * w      (and out2[i] = the same row times w2, when a second weight is given:
//                                               two norms of one row that differ in their weights only)
// `rows` (optional) picks the source rows; output row i is compact.  One block per output row.
// Replaces add_inplace_f32 + rmsnorm_f32 (rocml-kernels/kernels/elementwise.hip:7-26,
// rmsnorm.hip:7-43); product order x * inv_rms * w as there.
// Four consecutive outputs: one 8- or 16-byte store when the row allows it.
__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d, bool vec) {
    if (vec) *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
    else { p[0] = a; p[1] = b; p[2] = c; p[3] = d; }
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, float a, float b, float c, float d, bool vec) {
    if (vec) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&lo);
        raw.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = raw;
    } else {
        p[0] = __float2bfloat16_rn(a); p[1] = __float2bfloat16_rn(b);
        p[2] = __float2bfloat16_rn(c); p[3] = __float2bfloat16_rn(d);
    }
}

template <typename OT, typename WT>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                   int n_delta, size_t delta_stride, const WT* __restrict__ w,
                                   OT* __restrict__ out, const int* __restrict__ rows, int H,
                                   float eps, int write_back, const WT* __restrict__ w2, OT* __restrict__ out2,
                                   const float* __restrict__ delta_b, int n_delta_b, size_t delta_b_stride) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];  // H floats (padded to 4) + 33 for the reduction
    float* red = row_buf + ((H + 3) & ~3);
    const int orow = blockIdx.x;
    const int row = rows ? rows[orow] : orow;
    if (row < 0) return;  // a padded entry
    float* r = resid + (size_t)row * H;
    float ss = 0.f;
    const bool vec = (H & 3) == 0 && ((delta_stride | delta_b_stride) & 3) == 0 &&
                     (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)delta_b) & 15) == 0;
    if (vec) {
        const int H4 = H >> 2;
        float4* rb4 = reinterpret_cast<float4*>(row_buf);
        const float4* r4 = reinterpret_cast<const float4*>(r);
        for (int i = threadIdx.x; i < H4; i += blockDim.x) {
            float4 v = r4[i];
            // the first group of partial sums, then the second (a layer's two sublayers), each in its order
            for (int part = 0; part < 2; ++part) {
                const int nd = part ? n_delta_b : n_delta;
                const float4* d4 = reinterpret_cast<const float4*>((part ? delta_b : delta) + (size_t)row * H) + i;
                const size_t ds4 = (part ? delta_b_stride : delta_stride) >> 2;
                // eight partial sums at a time: every load is issued before the first addition, and the
                // additions keep the partial sums' order (an absent one adds zero)
                for (int s = 0; s < nd; s += 8) {
                    float4 d[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        d[j] = s + j < nd ? d4[(size_t)(s + j) * ds4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) { v.x += d[j].x; v.y += d[j].y; v.z += d[j].z; v.w += d[j].w; }
                }
            }
            rb4[i] = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = r[i];
            for (int s = 0; s < n_delta; ++s) v += delta[(size_t)s * delta_stride + (size_t)row * H + i];
            for (int s = 0; s < n_delta_b; ++s) v += delta_b[(size_t)s * delta_b_stride + (size_t)row * H + i];
            row_buf[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, red);
    const float inv = rsqrtf(total / (float)H + eps);
    OT* o = out + (size_t)orow * H;
    const bool out_vec = (((uintptr_t)out | ((size_t)H * sizeof(OT))) & 15) == 0;
    if (vec) {
        const int H4 = H >> 2;
        const float4* rb4 = reinterpret_cast<const float4*>(row_buf);
        float4* r4 = reinterpret_cast<float4*>(r);
        for (int i = threadIdx.x; i < H4; i += blockDim.x) {
            const float4 v = rb4[i];
            if (write_back) r4[i] = v;
            store4(o + 4 * i, v.x * inv * to_f32(w[4 * i]), v.y * inv * to_f32(w[4 * i + 1]),
                   v.z * inv * to_f32(w[4 * i + 2]), v.w * inv * to_f32(w[4 * i + 3]), out_vec);
            if (out2)
                store4(out2 + (size_t)orow * H + 4 * i, v.x * inv * to_f32(w2[4 * i]), v.y * inv * to_f32(w2[4 * i + 1]),
                       v.z * inv * to_f32(w2[4 * i + 2]), v.w * inv * to_f32(w2[4 * i + 3]),
                       out_vec && ((uintptr_t)out2 & 15) == 0);
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float v = row_buf[i];
            if (write_back) r[i] = v;
            o[i] = from_f32<OT>(v * inv * to_f32(w[i]));
            if (out2) out2[(size_t)orow * H + i] = from_f32<OT>(v * inv * to_f32(w2[i]));
        }
    }
}

// The same for many rows (prompts): a row per block of 128 or 256 threads, each thread keeping up to
// eight 16-byte groups of the row in registers, so that the row is read once, all its loads are in
// flight together, and several rows share a multiprocessor.  Needs 16-byte alignment throughout and
// H <= 8 * 4 * threads.
template <typename OT, typename WT, int THREADS>
__global__ void __launch_bounds__(THREADS) add_rmsnorm_rows_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                                                   int n_delta, size_t delta_stride,
                                                                   const WT* __restrict__ w, OT* __restrict__ out,
                                                                   const int* __restrict__ rows, int H, float eps,
                                                                   int write_back, const WT* __restrict__ w2,
                                                                   OT* __restrict__ out2, const float* __restrict__ delta_b,
                                                                   int n_delta_b, size_t delta_b_stride) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[33];
    const int orow = blockIdx.x;
    const int row = rows ? rows[orow] : orow;
    if (row < 0) return;  // a padded entry
    const int H4 = H >> 2;
    float4* r4 = reinterpret_cast<float4*>(resid + (size_t)row * H);
    float4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * THREADS;
        v[j] = i < H4 ? r4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int part = 0; part < 2; ++part) {                      // the first group of partial sums, then the second
        const float* dp = part ? delta_b : delta;
        const int nd = part ? n_delta_b : n_delta;
        const size_t dst = part ? delta_b_stride : delta_stride;
        for (int s = 0; s < nd; s += 2) {                       // partial sums in their order, two in flight
            const float4* d4 = reinterpret_cast<const float4*>(dp + (size_t)s * dst + (size_t)row * H);
            const float4* e4 = reinterpret_cast<const float4*>(dp + (size_t)(s + 1) * dst + (size_t)row * H);
            const bool second = s + 1 < nd;
            float4 d[8], e[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = threadIdx.x + j * THREADS;
                d[j] = i < H4 ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                e[j] = second && i < H4 ? e4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[j].x += d[j].x; v[j].y += d[j].y; v[j].z += d[j].z; v[j].w += d[j].w; }
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[j].x += e[j].x; v[j].y += e[j].y; v[j].z += e[j].z; v[j].w += e[j].w; }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps);
    OT* o = out + (size_t)orow * H;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int i = threadIdx.x + j * THREADS;
        if (i < H4) {
            if (write_back) r4[i] = v[j];
            store4(o + 4 * i, v[j].x * inv * to_f32(w[4 * i]), v[j].y * inv * to_f32(w[4 * i + 1]),
                   v[j].z * inv * to_f32(w[4 * i + 2]), v[j].w * inv * to_f32(w[4 * i + 3]), true);
            if (out2)
                store4(out2 + (size_t)orow * H + 4 * i, v[j].x * inv * to_f32(w2[4 * i]), v[j].y * inv * to_f32(w2[4 * i + 1]),
                       v[j].z * inv * to_f32(w2[4 * i + 2]), v[j].w * inv * to_f32(w2[4 * i + 3]), true);
        }
    }
}

template <typename OT, typename WT>
static int launch_add_rmsnorm(float* resid, const float* delta, int n_delta, size_t delta_stride,
                              const void* w, void* out, const int* rows, int n_rows, int H, float eps,
                              int write_back, const void* w2, void* out2, const float* delta_b, int n_delta_b,
                              size_t delta_b_stride, cudaStream_t s) {
    // many rows: the register kernel, when everything is 16-byte aligned and a row fits its threads
    // (up to 256 rows are at most one wave of the kernel below, whose 1,024 threads a row finish sooner)
    const bool aligned = (H & 3) == 0 && ((delta_stride | delta_b_stride) & 3) == 0 &&
                         ((((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)delta_b) & 15) == 0) &&
                         ((((uintptr_t)out | (uintptr_t)out2 | ((size_t)H * sizeof(OT))) & 15) == 0) &&
                         ((((uintptr_t)w | (uintptr_t)w2) & (4 * sizeof(WT) - 1)) == 0);
    if (n_rows > (H >= 4096 ? 256 : 64) && aligned && H <= 8 * 4 * 256) {
        if (H <= 8 * 4 * 128)
            RB_LAUNCH((add_rmsnorm_rows_kernel<OT, WT, 128>), dim3(n_rows), dim3(128), 0, s, resid, delta, n_delta,
                      delta_stride, (const WT*)w, (OT*)out, rows, H, eps, write_back, (const WT*)w2, (OT*)out2, delta_b,
                      n_delta_b, delta_b_stride);
        else
            RB_LAUNCH((add_rmsnorm_rows_kernel<OT, WT, 256>), dim3(n_rows), dim3(256), 0, s, resid, delta, n_delta,
                      delta_stride, (const WT*)w, (OT*)out, rows, H, eps, write_back, (const WT*)w2, (OT*)out2, delta_b,
                      n_delta_b, delta_b_stride);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    auto k = add_rmsnorm_kernel<OT, WT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    // one 16-byte column group per thread where the row allows it: a row's loads are all in flight at once
    const int threads = H >= 4096 ? 1024 : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
    RB_LAUNCH((k), dim3(n_rows), dim3(threads), smem, s, resid, delta, n_delta, delta_stride, (const WT*)w, (OT*)out, rows, H,
                                    eps, write_back, (const WT*)w2, (OT*)out2, delta_b, n_delta_b, delta_b_stride);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_add_rmsnorm(float* resid, const float* delta, int n_delta, long long delta_stride,
                              const void* w, int w_dtype, void* out, int out_dtype, const int* rows,
                              int n_rows, int H, float eps, int write_back, const void* w2, void* out2,
                              const float* delta_b, int n_delta_b, long long delta_b_stride, void* stream) {
    if (n_rows <= 0) return RB_OK;
    if ((w2 == nullptr) != (out2 == nullptr)) return RB_ERR_BAD_SIZE;
    if (delta_b == nullptr) n_delta_b = 0;
    if (n_delta_b == 0) { delta_b = nullptr; delta_b_stride = 0; }
    cudaStream_t s = (cudaStream_t)stream;
    const size_t ds = (size_t)delta_stride;
    const size_t dbs = (size_t)delta_b_stride;
    if (out_dtype == RB_BF16 && w_dtype == RB_BF16)
        return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, w2, out2, delta_b, n_delta_b, dbs, s);
    if (out_dtype == RB_BF16 && w_dtype == RB_F32)
        return launch_add_rmsnorm<__nv_bfloat16, float>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, w2, out2, delta_b, n_delta_b, dbs, s);
    if (out_dtype == RB_F32 && w_dtype == RB_BF16)
        return launch_add_rmsnorm<float, __nv_bfloat16>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, w2, out2, delta_b, n_delta_b, dbs, s);
    if (out_dtype == RB_F32 && w_dtype == RB_F32)
        return launch_add_rmsnorm<float, float>(resid, delta, n_delta, ds, w, out, rows, n_rows, H, eps, write_back, w2, out2, delta_b, n_delta_b, dbs, s);
    return RB_ERR_BAD_DTYPE;
}

// ---- SiLU(gate) * up ------------------------------------------------------------------------
// in: [S][T, 2*I] (S partial sums that are added first, in order); out: [T, I].  The gate of output
// i sits in column i and its up in column I + i, or, when `paired`, columns alternate in blocks of
// 16 between gates and ups (gate of output i at (i / 16) * 32 + i % 16, its up 16 columns on).  silu(g) = g / (1 + exp(-g)) as in
// rocml-kernels/kernels/silu_mul.hip:15-18.  Four outputs per thread when I is a multiple of 4.
template <typename IT, typename OT>
__global__ void silu_mul_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, OT* __restrict__ out,
                                int rows, int I, int paired) {
    pdl_trigger();
    pdl_wait();
    const int I4 = I >> 2;
    const bool vec = (I & 3) == 0;
    const bool in16 = ((uintptr_t)in & 15) == 0 && (in_stride & 3) == 0;     // with I a multiple of 4: every group of 4 on 16 bytes
    const size_t n = vec ? (size_t)rows * I4 : (size_t)rows * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (size_t)gridDim.x * blockDim.x) {
        if (vec) {
            const size_t t = idx / I4;
            const int i = (int)(idx - t * I4) * 4;
            float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
            const int gi = paired ? (i >> 4) * 32 + (i & 15) : i;
            const int up = paired ? 16 : I;
            if (sizeof(IT) == 4 && in16) {
                // 16-byte loads, two partial sums' worth in flight together; added in the partial sums' order
                for (int s = 0; s < n_in; s += 2) {
                    const float* p = reinterpret_cast<const float*>(in) + (size_t)s * in_stride + t * 2 * I + gi;
                    const bool second = s + 1 < n_in;
                    const float4 g0 = *reinterpret_cast<const float4*>(p), u0 = *reinterpret_cast<const float4*>(p + up);
                    const float4 g1 = second ? *reinterpret_cast<const float4*>(p + in_stride) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 u1 = second ? *reinterpret_cast<const float4*>(p + in_stride + up) : make_float4(0.f, 0.f, 0.f, 0.f);
                    g[0] += g0.x; g[1] += g0.y; g[2] += g0.z; g[3] += g0.w;
                    u[0] += u0.x; u[1] += u0.y; u[2] += u0.z; u[3] += u0.w;
                    g[0] += g1.x; g[1] += g1.y; g[2] += g1.z; g[3] += g1.w;
                    u[0] += u1.x; u[1] += u1.y; u[2] += u1.z; u[3] += u1.w;
                }
            } else {
                for (int s = 0; s < n_in; ++s) {
                    const IT* p = in + (size_t)s * in_stride + t * 2 * I + gi;
#pragma unroll
                    for (int j = 0; j < 4; ++j) { g[j] += to_f32(p[j]); u[j] += to_f32(p[up + j]); }
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) out[t * I + i + j] = from_f32<OT>(g[j] / (1.f + expf(-g[j])) * u[j]);
        } else {
            const size_t t = idx / I;
            const int i = (int)(idx - t * I);
            float g = 0.f, u = 0.f;
            for (int s = 0; s < n_in; ++s) {
                const int gi = paired ? (i >> 4) * 32 + (i & 15) : i;
                g += to_f32(in[(size_t)s * in_stride + t * 2 * I + gi]);
                u += to_f32(in[(size_t)s * in_stride + t * 2 * I + gi + (paired ? 16 : I)]);
            }
            out[idx] = from_f32<OT>(g / (1.f + expf(-g)) * u);
        }
    }
}

extern "C" int rb_silu_mul(const void* in, int in_dtype, int n_in, long long in_stride, void* out, int out_dtype,
                           int rows, int I, int paired, void* stream) {
    if (rows <= 0) return RB_OK;
    if (n_in < 1 || (paired && I % 16)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (I & 3) == 0 ? (size_t)rows * (I >> 2) : (size_t)rows * I;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    typedef __nv_bfloat16 bf;
    if (in_dtype == RB_BF16 && out_dtype == RB_BF16)
        RB_LAUNCH((silu_mul_kernel<bf, bf>), dim3(blocks), dim3(threads), 0, s, (const bf*)in, n_in, (size_t)in_stride, (bf*)out, rows, I, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_BF16)
        RB_LAUNCH((silu_mul_kernel<float, bf>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride, (bf*)out, rows, I, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_F32)
        RB_LAUNCH((silu_mul_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride, (float*)out, rows, I, paired);
    else
        return RB_ERR_BAD_DTYPE;
    return RB_OK;
}

// ---- casts ------------------------------------------------------------------------------------
template <typename A, typename B>
__global__ void cast_kernel(const A* __restrict__ in, B* __restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = from_f32<B>(to_f32(in[i]));
}

extern "C" int rb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream) {
    if (n <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (in_dtype == RB_F32 && out_dtype == RB_BF16)
        RB_LAUNCH((cast_kernel<float, __nv_bfloat16>), dim3(blocks), dim3(threads), 0, s, (const float*)in, (__nv_bfloat16*)out, (size_t)n);
    else if (in_dtype == RB_BF16 && out_dtype == RB_F32)
        RB_LAUNCH((cast_kernel<__nv_bfloat16, float>), dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)in, (float*)out, (size_t)n);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- embedding with a multiplier and an added sinusoid position vector ----------------------------
// out[t, i] = f32(table[ids[t], i]) * scale + (i even ? sin : cos)(positions[t] * inv_freq[i / 2]);
// inv_freq (float32 [ceil(H / 2)]) may be absent: then nothing is added.  `copy` (optional) receives the
// same rows (a model that adds its embedding output back in later keeps them).  Angle, sine and cosine
// are 32-bit and full precision.
template <typename WT>
__global__ void embedding_pos_kernel(const int* __restrict__ ids, const WT* __restrict__ table, float* __restrict__ out,
                                     float* __restrict__ copy, int H, int vocab, float scale,
                                     const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     int* __restrict__ status) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool bad = id < 0 || id >= vocab;
    if (bad && threadIdx.x == 0 && status) atomicExch(status, RB_ERR_BAD_SIZE);
    const WT* row = table + (size_t)(bad ? 0 : id) * H;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = bad ? 0.f : to_f32(row[i]) * scale;
        if (inv_freq) {
            const float a = pos * inv_freq[i >> 1];
            v += (i & 1) ? cosf(a) : sinf(a);
        }
        out[(size_t)t * H + i] = v;
        if (copy) copy[(size_t)t * H + i] = v;
    }
}

extern "C" int rb_embedding_pos(const int* ids, const void* table, int table_dtype, float* out, float* copy, int T,
                                int H, int vocab, float scale, const int* positions, const float* inv_freq,
                                int* status, void* stream) {
    if (T <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == RB_BF16)
        RB_LAUNCH((embedding_pos_kernel<__nv_bfloat16>), dim3(T), dim3(threads), 0, s, ids, (const __nv_bfloat16*)table, out,
                  copy, H, vocab, scale, positions, inv_freq, status);
    else if (table_dtype == RB_F32)
        RB_LAUNCH((embedding_pos_kernel<float>), dim3(T), dim3(threads), 0, s, ids, (const float*)table, out, copy, H, vocab,
                  scale, positions, inv_freq, status);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- additions into the residual stream between layers -----------------------------------------------
// resid[t, :] = ((resid[t, :] + sum_s delta[s][t, :]) + other[t, :]) + vec[:]; each of delta, other, vec may
// be absent.  The additions are 32-bit and in this order for every element.
template <typename WT>
__global__ void residual_inject_kernel(float* __restrict__ resid, const float* __restrict__ delta, int n_delta,
                                       size_t delta_stride, const float* __restrict__ other, const WT* __restrict__ vec,
                                       size_t n, int H) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = resid[i];
        for (int s = 0; s < n_delta; ++s) v += delta[(size_t)s * delta_stride + i];
        if (other) v += other[i];
        if (vec) v += to_f32(vec[i % H]);
        resid[i] = v;
    }
}

extern "C" int rb_residual_inject(float* resid, const float* delta, int n_delta, long long delta_stride,
                                  const float* other, const void* vec, int vec_dtype, int T, int H, void* stream) {
    if (T <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)T * H;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    if (vec_dtype == RB_BF16)
        RB_LAUNCH((residual_inject_kernel<__nv_bfloat16>), dim3(blocks), dim3(threads), 0, s, resid, delta, n_delta,
                  (size_t)delta_stride, other, (const __nv_bfloat16*)vec, n, H);
    else if (vec_dtype == RB_F32)
        RB_LAUNCH((residual_inject_kernel<float>), dim3(blocks), dim3(threads), 0, s, resid, delta, n_delta,
                  (size_t)delta_stride, other, (const float*)vec, n, H);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- a norm on a sublayer's output, the addition, and the next sublayer's norm --------------------------
// d = sum_s delta[s][row]  (s in order), or, with row_of, sum_j weights[row, j] * delta[row_of[row, j]] (j in order: a
// routed feed-forward's rows, summed here instead of in a kernel of their own);
// resid[row] += d * rsqrt(mean(d^2) + eps_post) * w_post;
// if w_next: out[row] = resid[row] * rsqrt(mean(resid[row]^2) + eps_next) * w_next.
// One block a row; the row stays in shared memory between the passes.  All arithmetic is 32-bit.
template <typename OT, typename WT>
__global__ void __launch_bounds__(1024) postnorm_add_norm_kernel(float* __restrict__ resid, const float* __restrict__ delta,
                                                                 int n_delta, size_t delta_stride,
                                                                 const int* __restrict__ row_of,
                                                                 const float* __restrict__ weights, int top,
                                                                 const WT* __restrict__ w_post, float eps_post,
                                                                 const WT* __restrict__ w_next, float eps_next,
                                                                 OT* __restrict__ out, int H) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float row_buf[];  // H floats (padded to 4) + 33 for the reductions
    float* red = row_buf + ((H + 3) & ~3);
    const int row = blockIdx.x;
    float* r = resid + (size_t)row * H;
    float ss = 0.f;
    if (row_of) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = 0.f;
            for (int j = 0; j < top; ++j) {
                const int src = row_of[(size_t)row * top + j];
                if (src >= 0) v = fmaf(weights[(size_t)row * top + j], delta[(size_t)src * delta_stride + i], v);
            }
            row_buf[i] = v;
            ss += v * v;
        }
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            float v = 0.f;
            for (int s = 0; s < n_delta; ++s) v += delta[(size_t)s * delta_stride + (size_t)row * H + i];
            row_buf[i] = v;
            ss += v * v;
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)H + eps_post);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = r[i] + row_buf[i] * inv * to_f32(w_post[i]);
        r[i] = v;
        row_buf[i] = v;
        ss2 += v * v;
    }
    if (!w_next) return;
    const float inv2 = rsqrtf(block_sum(ss2, red) / (float)H + eps_next);
    OT* o = out + (size_t)row * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<OT>(row_buf[i] * inv2 * to_f32(w_next[i]));
}

template <typename OT, typename WT>
static int launch_postnorm(float* resid, const float* delta, int n_delta, size_t delta_stride, const int* row_of,
                           const float* weights, int top, const void* w_post,
                           float eps_post, const void* w_next, float eps_next, void* out, int n_rows, int H,
                           cudaStream_t s) {
    const size_t smem = (size_t)(((H + 3) & ~3) + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    auto k = postnorm_add_norm_kernel<OT, WT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = H >= 4096 ? 1024 : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
    RB_LAUNCH((k), dim3(n_rows), dim3(threads), smem, s, resid, delta, n_delta, delta_stride, row_of, weights, top,
              (const WT*)w_post, eps_post, (const WT*)w_next, eps_next, (OT*)out, H);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_postnorm_add_norm(float* resid, const float* delta, int n_delta, long long delta_stride,
                                    const int* row_of, const float* weights, int top,
                                    const void* w_post, float eps_post, const void* w_next, float eps_next, int w_dtype,
                                    void* out, int out_dtype, int n_rows, int H, void* stream) {
    if (n_rows <= 0) return RB_OK;
    if (n_delta < 1 || !delta || !w_post || (row_of && (!weights || top < 1))) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t ds = (size_t)delta_stride;
    if (out_dtype == RB_BF16 && w_dtype == RB_BF16)
        return launch_postnorm<__nv_bfloat16, __nv_bfloat16>(resid, delta, n_delta, ds, row_of, weights, top, w_post, eps_post, w_next, eps_next, out, n_rows, H, s);
    if (out_dtype == RB_BF16 && w_dtype == RB_F32)
        return launch_postnorm<__nv_bfloat16, float>(resid, delta, n_delta, ds, row_of, weights, top, w_post, eps_post, w_next, eps_next, out, n_rows, H, s);
    if (out_dtype == RB_F32 && w_dtype == RB_BF16)
        return launch_postnorm<float, __nv_bfloat16>(resid, delta, n_delta, ds, row_of, weights, top, w_post, eps_post, w_next, eps_next, out, n_rows, H, s);
    if (out_dtype == RB_F32 && w_dtype == RB_F32)
        return launch_postnorm<float, float>(resid, delta, n_delta, ds, row_of, weights, top, w_post, eps_post, w_next, eps_next, out, n_rows, H, s);
    return RB_ERR_BAD_DTYPE;
}

// ---- gated activations on a stacked [gate | up] product ------------------------------------------------
// in: [S][rows, 2 * I] (S partial sums, added first, in order), gates in columns 0 .. I - 1 and ups in
// I .. 2 I - 1, or, when `paired`, alternating in blocks of 16 columns (gate of output i at
// (i / 16) * 32 + i % 16, its up 16 columns on); out: [rows, I].
//   kind 0: silu(g) * u, silu(g) = g / (1 + exp(-g))
//   kind 1: g' = min(g, limit), u' = clamp(u, -limit, limit); g' * sigmoid(alpha * g') * (u' + 1)
//   kind 2: gelu(g) * u in its tanh form, gelu(g) = g / 2 * (1 + tanh(sqrt(2 / pi) * (g + 0.044715 g^3)))
template <typename IT, typename OT>
__global__ void gated_act_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, size_t in_ld, OT* __restrict__ out,
                                 size_t out_ld, int rows, int I, int kind, float limit, float alpha, int paired) {
    pdl_trigger();
    pdl_wait();
    const size_t n = (size_t)rows * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const int gi = paired ? (i >> 4) * 32 + (i & 15) : i;
        const int up = paired ? 16 : I;
        float g = 0.f, u = 0.f;
        for (int s = 0; s < n_in; ++s) {
            g += to_f32(in[(size_t)s * in_stride + t * in_ld + gi]);
            u += to_f32(in[(size_t)s * in_stride + t * in_ld + gi + up]);
        }
        float v;
        if (kind == 0) {
            v = g / (1.f + expf(-g)) * u;
        } else if (kind == 2) {
            v = gelu_tanh(g) * u;
        } else {
            g = fminf(g, limit);
            u = fminf(fmaxf(u, -limit), limit);
            v = g / (1.f + expf(-alpha * g)) * (u + 1.f);
        }
        out[t * out_ld + i] = from_f32<OT>(v);
    }
}

extern "C" int rb_gated_act(const void* in, int in_dtype, int n_in, long long in_stride, long long in_ld, void* out,
                            int out_dtype, long long out_ld, int rows, int I, int kind, float limit, float alpha,
                            int paired, void* stream) {
    if (rows <= 0 || I <= 0) return RB_OK;
    if (n_in < 1 || kind < 0 || kind > 2 || (paired && I % 16)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * I;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    typedef __nv_bfloat16 bf;
    if (in_dtype == RB_BF16 && out_dtype == RB_BF16)
        RB_LAUNCH((gated_act_kernel<bf, bf>), dim3(blocks), dim3(threads), 0, s, (const bf*)in, n_in, (size_t)in_stride,
                  (size_t)in_ld, (bf*)out, (size_t)out_ld, rows, I, kind, limit, alpha, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_BF16)
        RB_LAUNCH((gated_act_kernel<float, bf>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride,
                  (size_t)in_ld, (bf*)out, (size_t)out_ld, rows, I, kind, limit, alpha, paired);
    else if (in_dtype == RB_F32 && out_dtype == RB_F32)
        RB_LAUNCH((gated_act_kernel<float, float>), dim3(blocks), dim3(threads), 0, s, (const float*)in, n_in, (size_t)in_stride,
                  (size_t)in_ld, (float*)out, (size_t)out_ld, rows, I, kind, limit, alpha, paired);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- heads of an attention result times a gate, narrowed to the values' width ----------------------------------
// in [T, heads, in_w] -> out [T, heads, out_w] (out_w <= in_w: what lies beyond is padding), multiplied by a gate
// formed in 32-bit.  The gate is either finished, float32 [T, heads * gate_w] (gate_w 1: one a head; gate_w = out_w:
// one a value), or `raw`: columns of the projection rows (n_in partial sums added first, in order), of which the
// kernel takes the sigmoid itself.  Absent: 1.
template <typename AT, typename RT>
__global__ void head_gate_kernel(const AT* __restrict__ in, long long ld_in, int in_w, AT* __restrict__ out, long long ld_out,
                                 int out_w, const float* __restrict__ gate, int gate_w, const RT* __restrict__ raw, int n_in,
                                 long long in_stride, long long row_stride, int heads, int T) {
    pdl_trigger();
    pdl_wait();
    const bool each = gate_w > 1;
    if ((in_w & 3) == 0 && (out_w & 3) == 0 && (ld_in & 3) == 0 && (ld_out & 3) == 0 &&
        (((uintptr_t)in | (uintptr_t)out) & (4 * sizeof(AT) - 1)) == 0 &&
        (!raw || !each || ((row_stride & 3) == 0 && (in_stride & 3) == 0 && ((uintptr_t)raw & (4 * sizeof(RT) - 1)) == 0)) &&
        (!gate || !each || ((uintptr_t)gate & 15) == 0)) {
        // four neighbouring values a thread
        const int w4 = out_w >> 2;
        const size_t n4 = (size_t)T * heads * w4;
        for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n4; idx += (size_t)gridDim.x * blockDim.x) {
            const size_t th = idx / w4;
            const int d = (int)(idx - th * w4) * 4;
            const size_t t = th / heads;
            const int h = (int)(th - t * heads);
            float g[4] = {1.f, 1.f, 1.f, 1.f};
            if (raw && each) {
                float z[4] = {0.f, 0.f, 0.f, 0.f};
                for (int s = 0; s < n_in; ++s) {
                    float r[4];
                    load4(raw + (size_t)s * in_stride + t * row_stride + (size_t)h * out_w + d, r);
                    z[0] += r[0]; z[1] += r[1]; z[2] += r[2]; z[3] += r[3];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) g[j] = 1.f / (1.f + expf(-z[j]));
            } else if (raw) {
                float z = 0.f;
                for (int s = 0; s < n_in; ++s) z += to_f32(raw[(size_t)s * in_stride + t * row_stride + h]);
                g[0] = g[1] = g[2] = g[3] = 1.f / (1.f + expf(-z));
            } else if (gate && each) {
                load4(gate + th * out_w + d, g);
            } else if (gate) {
                g[0] = g[1] = g[2] = g[3] = gate[th];
            }
            float x[4];
            load4(in + t * ld_in + (size_t)h * in_w + d, x);
            x[0] *= g[0]; x[1] *= g[1]; x[2] *= g[2]; x[3] *= g[3];
            store4(out + t * ld_out + (size_t)h * out_w + d, x);
        }
        return;
    }
    const size_t n = (size_t)T * heads * out_w;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t th = idx / out_w;
        const int d = (int)(idx - th * out_w);
        const size_t t = th / heads;
        const int h = (int)(th - t * heads);
        float g = 1.f;
        if (raw) {
            float z = 0.f;
            const size_t col = each ? (size_t)h * out_w + d : (size_t)h;
            for (int s = 0; s < n_in; ++s) z += to_f32(raw[(size_t)s * in_stride + t * row_stride + col]);
            g = 1.f / (1.f + expf(-z));
        } else if (gate) {
            g = each ? gate[th * out_w + d] : gate[th];
        }
        out[t * ld_out + (size_t)h * out_w + d] = from_f32<AT>(to_f32(in[t * ld_in + (size_t)h * in_w + d]) * g);
    }
}

extern "C" int rb_head_gate(const void* in, long long ld_in, int in_w, void* out, long long ld_out, int out_w,
                            const float* gate, int gate_w, const void* raw, int raw_dtype, int n_in, long long in_stride,
                            long long row_stride, int heads, int T, int dtype, void* stream) {
    if (T <= 0 || heads <= 0) return RB_OK;
    if (out_w <= 0 || out_w > in_w || (gate_w != 1 && gate_w != out_w) || (raw && (gate || n_in < 1))) return RB_ERR_BAD_SIZE;
    const size_t n = (size_t)T * heads * out_w;
    const int threads = 256;
    const size_t want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_HG(AT, RT)                                                                                                   \
    RB_LAUNCH((head_gate_kernel<AT, RT>), dim3(blocks), dim3(threads), 0, s, (const AT*)in, ld_in, in_w, (AT*)out, ld_out, \
              out_w, gate, gate_w, (const RT*)raw, n_in, in_stride, row_stride, heads, T)
    if (dtype == RB_BF16 && (!raw || raw_dtype == RB_BF16)) RB_HG(bf, bf);
    else if (dtype == RB_BF16 && raw_dtype == RB_F32) RB_HG(bf, float);
    else if (dtype == RB_F32 && (!raw || raw_dtype == RB_F32)) RB_HG(float, float);
    else return RB_ERR_BAD_DTYPE;
#undef RB_HG
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// ---- x *= factor (32-bit, in place) ----------------------------------------------------------------------
__global__ void scale_kernel(float* __restrict__ x, size_t n, float factor) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] *= factor;
}

extern "C" int rb_scale(float* x, long long n, float factor, void* stream) {
    if (n <= 0) return RB_OK;
    const int threads = 256;
    const long long want = (n + threads - 1) / threads;
    const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
    RB_LAUNCH((scale_kernel), dim3(blocks), dim3(threads), 0, (cudaStream_t)stream, x, (size_t)n, factor);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
