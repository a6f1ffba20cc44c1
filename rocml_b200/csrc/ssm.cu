// A state-space mixer's recurrence with a step size per token and head, and the short causal convolution before it.
//
//   causal_conv   y_t[c] = act(b[c] + sum_j w[c][j] * u_(t - taps + 1 + j)[c])      j = 0 .. taps-1, the last tap is the
//                 current token's.  u are columns of the layer's stacked projection (in the activations' type, or 32-bit
//                 partial sums that are added first).  What lies before a sequence's first token of this step comes
//                 from the sequence's slot ([taps - 1][channels], zeros at the start of a sequence), which then
//                 receives the step's last taps - 1 inputs.  A block is (sequence, 32 tokens, 128 channels); the block
//                 of a sequence's first tokens is the only one that reads the slot and rewrites it after its reads.
//   ssm_scan      per (sequence, head h of group g):  dt = softplus(r_t + bias_h),  a = exp(-exp(A_h) * dt)
//                 S_t = a S_(t-1) + dt B_t x_t^T          S [n][p], 32-bit, in the slot
//                 y_t = S_t^T C_t + D_h x_t
//                 x [heads][p], B and C [groups][n] are columns of the convolution's 32-bit output, r columns of the
//                 projection.  A block owns a (sequence, head) and a tile of the state's columns, which stays in
//                 shared memory for the step; eight tokens are staged at a time and every thread walks them over
//                 its own rows of a column, so no barrier separates tokens.  The order of a token's operations does
//                 not depend on how the prompt was cut or on the batch.
//   ssm_scan_blocks   the same for prompts, blocks of 64 tokens side by side.  With c_t = sum_{r <= t} log a_r inside a
//                 block that starts from S0:
//                   y_t   = e^(c_t) S0^T C_t + sum_{s <= t} e^(c_t - c_s) (C_t . B_s) dt_s x_s + D x_t
//                   S_end = e^(c_m) S0 + sum_s e^(c_m - c_s) dt_s B_s x_s^T
//                 every exponent is <= 0.  Four kernels: C_t . B_s per block and group (what a group's heads share); each
//                 block's own sum; the states the blocks start from, along each sequence; each block's outputs.  All
//                 32-bit FMA.
//   ssm_step      one token a sequence: the state streams through registers (a warp every eighth row, a lane a column),
//                 read, decayed, updated and written once; nothing of it passes through shared memory.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
template <typename IT>
__device__ __forceinline__ float sum_in(const IT* p, int n_in, size_t in_stride) {
    float v = 0.f;
    for (int s = 0; s < n_in; ++s) v += to_f32(p[(size_t)s * in_stride]);
    return v;
}

__device__ __forceinline__ float softplus_f32(float z) { return z > 20.f ? z : log1pf(expf(z)); }

constexpr int CONV_TOK = 32;
constexpr int CONV_CH = 128;
constexpr int CONV_MAX_TAPS = 16;

// TAPS > 0: the taps as a constant (the window and the taps live in registers); TAPS == 0: any number up to CONV_MAX_TAPS.
template <typename IT, int TAPS>
__global__ void __launch_bounds__(CONV_CH)
causal_conv_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int col0, int channels, int taps_arg,
                   const float* __restrict__ w, const float* __restrict__ bias, int act, float* __restrict__ kept,
                   const int* __restrict__ seq_slot, const int* __restrict__ cu_q, float* __restrict__ out, int ld_out) {
    pdl_trigger();
    pdl_wait();
    constexpr int MAXT = TAPS > 0 ? TAPS : CONV_MAX_TAPS;
    const int taps = TAPS > 0 ? TAPS : taps_arg;
    const int b = blockIdx.z;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    const int t0 = t_begin + blockIdx.y * CONV_TOK;
    if (t0 >= t_end) return;
    const int c = blockIdx.x * CONV_CH + threadIdx.x;
    if (c >= channels) return;
    const int back = taps - 1;
    float* mine = kept + (size_t)slot * back * channels;          // [taps - 1][channels]
    float wt[MAXT], win[MAXT];                                    // the taps, and the last inputs (win[taps - 1]: the newest)
    const float bc = bias ? bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < MAXT; ++j) {
        if (j < taps) wt[j] = w[(size_t)c * taps + j];
        win[j] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < MAXT - 1; ++j) {
        if (j < back) {
            const int t = t0 - back + j;                          // the row `back - j` before the block's first
            win[j + 1] = t >= t_begin ? sum_in(in + (size_t)t * row_stride + col0 + c, n_in, in_stride)
                                      : mine[(size_t)(back + (t - t_begin)) * channels + c];
        }
    }
    const int n = min(CONV_TOK, t_end - t0);
    const IT* src = in + (size_t)t0 * row_stride + col0 + c;
    for (int tt = 0; tt < n; tt += 4) {
        float fresh[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) fresh[u] = tt + u < n ? sum_in(src + (size_t)(tt + u) * row_stride, n_in, in_stride) : 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (tt + u < n) {
#pragma unroll
                for (int j = 0; j < MAXT - 1; ++j)
                    if (j < back) win[j] = win[j + 1];
#pragma unroll
                for (int j = 0; j < MAXT; ++j)
                    if (j == back) win[j] = fresh[u];
                float acc = bc;
#pragma unroll
                for (int j = 0; j < MAXT; ++j)
                    if (j < taps) acc = fmaf(wt[j], win[j], acc);
                if (act == 1) acc = silu(acc);
                out[(size_t)(t0 + tt + u) * ld_out + c] = acc;
            }
        }
    }
    // Only the block of a sequence's first tokens reads the slot (a block spans more tokens than there are taps), and
    // a channel's rows are read and written by one thread alone: that thread leaves the step's last inputs there.
    if (blockIdx.y == 0 && back > 0) {
        // new rows of the slot: the last `back` inputs of (old rows, this step's rows)
        const int len = t_end - t_begin;
        float last[MAXT];
#pragma unroll
        for (int j = 0; j < MAXT - 1; ++j) {
            if (j < back) {
                const int at = len + j;                            // index into the concatenation of old and new rows
                last[j] = at < back ? mine[(size_t)at * channels + c]
                                    : sum_in(in + (size_t)(t_begin + at - back) * row_stride + col0 + c, n_in, in_stride);
            }
        }
#pragma unroll
        for (int j = 0; j < MAXT - 1; ++j)
            if (j < back) mine[(size_t)j * channels + c] = last[j];
    }
}

constexpr int SCAN_THREADS = 256;
constexpr int SCAN_TB = 8;

template <typename IT>
__global__ void __launch_bounds__(SCAN_THREADS)
ssm_scan_kernel(const float* __restrict__ u, int ld_u, int x_off, int b_off, int c_off, const IT* __restrict__ raw, int n_in,
                size_t in_stride, int row_stride, int dt_off, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const float* __restrict__ skip, int heads, int groups, int n, int p, float* __restrict__ state,
                const int* __restrict__ seq_slot, const int* __restrict__ cu_q, float* __restrict__ out, int ld_out, int VT, int P) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                              // [n][VT]
    float* cs = S + (size_t)n * VT;             // [TB][n]   C_t
    float* bs = cs + SCAN_TB * n;               // [TB][n]   dt_t * B_t
    float* xs = bs + SCAN_TB * n;               // [TB][VT]
    float* part = xs + SCAN_TB * VT;            // [TB][P][VT]
    float* dec = part + SCAN_TB * P * VT;       // [TB] decays, [TB] step sizes
    const int b = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * VT;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    if (t_end <= t_begin) return;
    const int g = h / (heads / groups);
    const int vt = min(VT, p - v0);
    const int tid = threadIdx.x;
    const float rate = expf(a_log[h]), db = dt_bias[h], dskip = skip[h];
    float* st = state + (((size_t)slot * heads + h) * n) * p + v0;
    for (int idx = tid; idx < n * VT; idx += SCAN_THREADS) {
        const int i = idx / VT, j = idx - i * VT;
        S[idx] = j < vt ? st[(size_t)i * p + j] : 0.f;
    }
    const int pp = tid / VT, j = tid - pp * VT;
    const bool works = pp < P && j < vt;
    for (int t0 = t_begin; t0 < t_end; t0 += SCAN_TB) {
        const int nb = min(SCAN_TB, t_end - t0);
        __syncthreads();                        // the tokens before are done with the staging buffers
        if (tid < nb) {
            const float dt = softplus_f32(sum_in(raw + (size_t)(t0 + tid) * row_stride + dt_off + h, n_in, in_stride) + db);
            dec[tid] = expf(-rate * dt);
            dec[SCAN_TB + tid] = dt;
        }
        __syncthreads();
        for (int idx = tid; idx < nb * n; idx += SCAN_THREADS) {
            const int tt = idx / n, i = idx - tt * n;
            const float* row = u + (size_t)(t0 + tt) * ld_u + (size_t)g * n + i;
            cs[idx] = row[c_off];
            bs[idx] = row[b_off] * dec[SCAN_TB + tt];
        }
        for (int idx = tid; idx < nb * VT; idx += SCAN_THREADS) {
            const int tt = idx / VT, jj = idx - tt * VT;
            xs[idx] = jj < vt ? u[(size_t)(t0 + tt) * ld_u + x_off + (size_t)h * p + v0 + jj] : 0.f;
        }
        __syncthreads();
        if (works) {
            for (int tt = 0; tt < nb; ++tt) {
                const float x = xs[tt * VT + j], a = dec[tt];
                const float* cc = cs + tt * n;
                const float* bb = bs + tt * n;
                float acc = 0.f;
                for (int i = pp; i < n; i += P) {
                    const float s = fmaf(bb[i], x, a * S[i * VT + j]);
                    S[i * VT + j] = s;
                    acc = fmaf(s, cc[i], acc);
                }
                part[(tt * P + pp) * VT + j] = acc;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < nb * VT; idx += SCAN_THREADS) {
            const int tt = idx / VT, jj = idx - tt * VT;
            if (jj >= vt) continue;
            float o = 0.f;
            for (int q = 0; q < P; ++q) o += part[(tt * P + q) * VT + jj];
            out[(size_t)(t0 + tt) * ld_out + (size_t)h * p + v0 + jj] = fmaf(dskip, xs[idx], o);
        }
    }
    __syncthreads();
    for (int idx = tid; idx < n * VT; idx += SCAN_THREADS) {
        const int i = idx / VT, jj = idx - i * VT;
        if (jj < vt) st[(size_t)i * p + jj] = S[idx];
    }
}
// ---- one token a sequence: the state streams through registers ---------------------------------------------------------
template <typename IT>
__global__ void __launch_bounds__(256)
ssm_step_kernel(const float* __restrict__ u, int ld_u, int x_off, int b_off, int c_off, const IT* __restrict__ raw, int n_in,
                size_t in_stride, int row_stride, int dt_off, const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                const float* __restrict__ skip, int heads, int groups, int n, int p, float* __restrict__ state,
                const int* __restrict__ seq_slot, const int* __restrict__ cu_q, float* __restrict__ out, int ld_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    __shared__ float part[8][32];
    float* cs = sm;            // [n]  C
    float* bs = sm + n;        // [n]  dt * B
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t = cu_q[b];
    if (cu_q[b + 1] <= t) return;
    const int g = h / (heads / groups);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * 32 + lane;
    const float dt = softplus_f32(sum_in(raw + (size_t)t * row_stride + dt_off + h, n_in, in_stride) + dt_bias[h]);
    const float a = expf(-expf(a_log[h]) * dt);
    const float* row = u + (size_t)t * ld_u;
    for (int i = threadIdx.x; i < n; i += 256) {
        cs[i] = row[c_off + g * n + i];
        bs[i] = row[b_off + g * n + i] * dt;
    }
    const float x = j < p ? row[x_off + h * p + j] : 0.f;
    __syncthreads();
    float* S = state + (((size_t)slot * heads + h) * n) * p + j;
    float acc = 0.f;
    if (j < p) {
        int i = warp;
        for (; i + 24 < n; i += 32) {             // four rows' loads in flight
            float s0 = S[(size_t)i * p], s1 = S[(size_t)(i + 8) * p], s2 = S[(size_t)(i + 16) * p], s3 = S[(size_t)(i + 24) * p];
            s0 = fmaf(bs[i], x, a * s0); s1 = fmaf(bs[i + 8], x, a * s1); s2 = fmaf(bs[i + 16], x, a * s2); s3 = fmaf(bs[i + 24], x, a * s3);
            S[(size_t)i * p] = s0; S[(size_t)(i + 8) * p] = s1; S[(size_t)(i + 16) * p] = s2; S[(size_t)(i + 24) * p] = s3;
            acc = fmaf(s0, cs[i], acc); acc = fmaf(s1, cs[i + 8], acc); acc = fmaf(s2, cs[i + 16], acc); acc = fmaf(s3, cs[i + 24], acc);
        }
        for (; i < n; i += 8) {
            const float s0 = fmaf(bs[i], x, a * S[(size_t)i * p]);
            S[(size_t)i * p] = s0;
            acc = fmaf(s0, cs[i], acc);
        }
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && j < p) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) o += part[w][lane];
        out[(size_t)t * ld_out + (size_t)h * p + j] = fmaf(skip[h], x, o);
    }
}

// ---- prompts: the same recurrence by blocks of 64 tokens, all blocks at once ------------------------------------------------
constexpr int CB = 64;              // tokens a block
constexpr int CT = 256;             // threads: a 16 x 16 grid, each thread a 4 x 4 tile of a 64 x 64 result
constexpr int CP = 64;              // columns of the state a block of the grid takes
constexpr int CN = 64;              // rows of the state staged at a time
constexpr int CL = CB + 4;          // row length of the transposed tiles (a multiple of 4 that is no multiple of 32)

// Which sequence and which of its blocks of tokens the grid's block `g` is (blocks are numbered sequence after sequence).
__device__ __forceinline__ bool find_tokens(int g, const int* seq_slot, const int* cu_q, int n_seqs, int* t0, int* m, int* slot) {
    int base = 0;
    for (int b = 0; b < n_seqs; ++b) {
        const int n = cu_q[b + 1] - cu_q[b];
        const int nb = seq_slot[b] >= 0 ? (n + CB - 1) / CB : 0;
        if (g < base + nb) {
            const int c = g - base;
            *t0 = cu_q[b] + c * CB; *m = min(CB, n - c * CB); *slot = seq_slot[b];
            return true;
        }
        base += nb;
    }
    return false;
}

// The block's step sizes and the running sums of its log decays: dt[t], cum[t] = sum_{r <= t} -rate * dt[r]; rows past m
// repeat the last sum and have step size 0.
template <typename IT>
__device__ __forceinline__ void block_steps(const IT* raw, int n_in, size_t in_stride, int row_stride, int col, int t0, int m,
                                            float rate, float bias, float* dt, float* cum, float* la) {
    const int t = threadIdx.x;
    if (t < CB) {
        float d = 0.f;
        if (t < m) d = softplus_f32(sum_in(raw + (size_t)(t0 + t) * row_stride + col, n_in, in_stride) + bias);
        dt[t] = d;
        la[t] = -rate * d;
    }
    __syncthreads();
    if (t < CB) {
        float c = 0.f;
        for (int r = 0; r <= t; ++r) c += la[r];
        cum[t] = c;
    }
    __syncthreads();
}

// acc[4][4] += A^T[k][rows] . B[k][cols] over k < K: At is [K][lda] (the thread's rows at 4 * ty), Bm is [K][ldb].
__device__ __forceinline__ void tile_mm(float (&acc)[4][4], const float* At, int lda, const float* Bm, int ldb, int K, int ty, int tx) {
#pragma unroll 4
    for (int k = 0; k < K; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(At + k * lda + 4 * ty);
        const float4 b = *reinterpret_cast<const float4*>(Bm + k * ldb + 4 * tx);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
}

// (1) every block's own sum: L[n][p] = sum_s e^(cum_last - cum_s) dt_s B_s[n] x_s[p]; and e^(cum_last) per (block, head).
template <typename IT>
__global__ void __launch_bounds__(CT)
ssm_block_sum_kernel(const float* __restrict__ u, int ld_u, int x_off, int b_off, const IT* __restrict__ raw, int n_in,
                     size_t in_stride, int row_stride, int dt_off, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, int heads, int groups, int n, int p, const int* __restrict__ seq_slot,
                     const int* __restrict__ cu_q, int n_seqs, float* __restrict__ work, float* __restrict__ block_decay) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float Bw[CB][CN];        // [s][n]: B_s[n] * w_s
    __shared__ __align__(16) float Xs[CB][CP];        // [s][p]
    __shared__ float dt[CB], cum[CB], la[CB];
    int t0, m, slot;
    if (!find_tokens(blockIdx.z, seq_slot, cu_q, n_seqs, &t0, &m, &slot)) return;
    const int h = blockIdx.y, p0 = blockIdx.x * CP, g = h / (heads / groups);
    block_steps(raw, n_in, in_stride, row_stride, dt_off + h, t0, m, expf(a_log[h]), dt_bias[h], dt, cum, la);
    const float last = cum[CB - 1];
    if (threadIdx.x == 0 && blockIdx.x == 0) block_decay[(size_t)blockIdx.z * heads + h] = expf(last);
    if (threadIdx.x < CB) la[threadIdx.x] = expf(last - cum[threadIdx.x]) * dt[threadIdx.x];     // token s's weight in the block's sum
    for (int idx = threadIdx.x; idx < CB * CP; idx += CT) {
        const int s = idx / CP, j = idx - s * CP;
        Xs[s][j] = (s < m && p0 + j < p) ? u[(size_t)(t0 + s) * ld_u + x_off + (size_t)h * p + p0 + j] : 0.f;
    }
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float* dst = work + (((size_t)blockIdx.z * heads + h) * n) * p;
    for (int n0 = 0; n0 < n; n0 += CN) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < CB * CN; idx += CT) {
            const int s = idx / CN, i = idx - s * CN;
            Bw[s][i] = (s < m && n0 + i < n) ? u[(size_t)(t0 + s) * ld_u + b_off + (size_t)g * n + n0 + i] * la[s] : 0.f;
        }
        __syncthreads();
        float acc[4][4] = {};
        tile_mm(acc, &Bw[0][0], CN, &Xs[0][0], CP, CB, ty, tx);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int row = n0 + 4 * ty + i, col = p0 + 4 * tx + j;
                if (row < n && col < p) dst[(size_t)row * p + col] = acc[i][j];
            }
    }
}

// (2) along each sequence: the state every block starts from takes the place of the block's own sum; the slot receives the
// state after the last block.  Elementwise; a thread walks its element through the sequence's blocks.
__global__ void __launch_bounds__(256)
ssm_block_states_kernel(float* __restrict__ work, const float* __restrict__ block_decay, float* __restrict__ state, int heads,
                        int np, const int* __restrict__ seq_slot, const int* __restrict__ cu_q) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    int first = 0;
    for (int i = 0; i < b; ++i) first += seq_slot[i] >= 0 ? (cu_q[i + 1] - cu_q[i] + CB - 1) / CB : 0;
    const int nb = (cu_q[b + 1] - cu_q[b] + CB - 1) / CB;
    if (nb <= 0) return;
    const int e = blockIdx.x * 256 + threadIdx.x;
    if (e >= np) return;
    float* st = state + ((size_t)slot * heads + h) * np + e;
    float S = *st;
    for (int c0 = 0; c0 < nb; c0 += 8) {            // eight blocks' sums in flight
        float own[8], dec[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = first + c0 + j;
            own[j] = c0 + j < nb ? work[((size_t)c * heads + h) * np + e] : 0.f;
            dec[j] = c0 + j < nb ? block_decay[(size_t)c * heads + h] : 1.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (c0 + j < nb) {
                work[((size_t)(first + c0 + j) * heads + h) * np + e] = S;
                S = fmaf(dec[j], S, own[j]);
            }
        }
    }
    *st = S;
}

// (0) what the heads of a group share: W[t][s] = C_t . B_s for every block of tokens and group, stored [s][t].
__global__ void __launch_bounds__(CT)
ssm_block_cb_kernel(const float* __restrict__ u, int ld_u, int b_off, int c_off, int groups, int n,
                    const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int n_seqs, float* __restrict__ cb) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float Ct[CN * CL];
    __shared__ __align__(16) float Bt[CN * CL];
    int t0, m, slot;
    if (!find_tokens(blockIdx.y, seq_slot, cu_q, n_seqs, &t0, &m, &slot)) return;
    const int g = blockIdx.x;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[4][4] = {};
    for (int n0 = 0; n0 < n; n0 += CN) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < CB * CN; idx += CT) {
            const int s = idx / CN, i = idx - s * CN;
            const bool in = s < m && n0 + i < n;
            const float* row = u + (size_t)(t0 + s) * ld_u + (size_t)g * n + n0 + i;
            Ct[i * CL + s] = in ? row[c_off] : 0.f;
            Bt[i * CL + s] = in ? row[b_off] : 0.f;
        }
        __syncthreads();
        tile_mm(acc, Ct, CL, Bt, CL, CN, ty, tx);            // rows t, columns s
    }
    float* dst = cb + ((size_t)blockIdx.y * groups + g) * CB * CB;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int sidx = 4 * tx + j;
        *reinterpret_cast<float4*>(dst + sidx * CB + 4 * ty) = make_float4(acc[0][j], acc[1][j], acc[2][j], acc[3][j]);
    }
}

// (3) every block's outputs: y_t = e^(cum_t) C_t S0 + sum_{s <= t} e^(cum_t - cum_s) dt_s (C_t . B_s) x_s + D x_t.
template <typename IT>
__global__ void __launch_bounds__(CT)
ssm_block_out_kernel(const float* __restrict__ u, int ld_u, int x_off, int c_off, const IT* __restrict__ raw, int n_in,
                     size_t in_stride, int row_stride, int dt_off, const float* __restrict__ dt_bias,
                     const float* __restrict__ a_log, const float* __restrict__ skip, int heads, int groups, int n, int p,
                     const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int n_seqs, const float* __restrict__ work,
                     const float* __restrict__ cb, float* __restrict__ out, int ld_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    float* Ct = sm;                     // [CN][CL]: C_t[n] at [n][t]
    float* S0 = Ct + CN * CL;           // [CN][CP]
    float* Xs = S0 + CN * CP;           // [CB][CP]
    float* Gt = Ct;                     // [CB][CB]: the weight of token s in token t's result at [s][t], after the C tiles
    float* dt = Xs + CB * CP;
    float* cum = dt + CB;
    float* la = cum + CB;
    int t0, m, slot;
    if (!find_tokens(blockIdx.z, seq_slot, cu_q, n_seqs, &t0, &m, &slot)) return;
    const int h = blockIdx.y, p0 = blockIdx.x * CP, g = h / (heads / groups);
    block_steps(raw, n_in, in_stride, row_stride, dt_off + h, t0, m, expf(a_log[h]), dt_bias[h], dt, cum, la);
    for (int idx = threadIdx.x; idx < CB * CP; idx += CT) {
        const int s = idx / CP, j = idx - s * CP;
        Xs[idx] = (s < m && p0 + j < p) ? u[(size_t)(t0 + s) * ld_u + x_off + (size_t)h * p + p0 + j] : 0.f;
    }
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const float* start = work + (((size_t)blockIdx.z * heads + h) * n) * p;
    float sacc[4][4] = {};
    for (int n0 = 0; n0 < n; n0 += CN) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < CB * CN; idx += CT) {
            const int s = idx / CN, i = idx - s * CN;         // consecutive threads read consecutive n of one token
            Ct[i * CL + s] = (s < m && n0 + i < n) ? u[(size_t)(t0 + s) * ld_u + c_off + (size_t)g * n + n0 + i] : 0.f;
        }
        for (int idx = threadIdx.x; idx < CN * CP; idx += CT) {
            const int i = idx / CP, j = idx - i * CP;
            S0[idx] = (n0 + i < n && p0 + j < p) ? start[(size_t)(n0 + i) * p + p0 + j] : 0.f;
        }
        __syncthreads();
        tile_mm(sacc, Ct, CL, S0, CP, CN, ty, tx);           // rows t, columns p
    }
    __syncthreads();                    // the C tile is done with: the weights take its room
    // the weight of token s in token t's result, [s][t]: what the group's heads share, times this head's decays and step sizes
    {
        const float* shared_w = cb + ((size_t)blockIdx.z * groups + g) * CB * CB;
        for (int idx = threadIdx.x * 4; idx < CB * CB; idx += CT * 4) {
            const int sidx = idx / CB, t = idx - sidx * CB;
            const float4 w4 = *reinterpret_cast<const float4*>(shared_w + idx);
            const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
            float o4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) o4[j] = (sidx <= t + j && t + j < m) ? wv[j] * expf(cum[t + j] - cum[sidx]) * dt[sidx] : 0.f;
            *reinterpret_cast<float4*>(Gt + idx) = make_float4(o4[0], o4[1], o4[2], o4[3]);
        }
    }
    __syncthreads();
    float yacc[4][4] = {};
    tile_mm(yacc, Gt, CB, Xs, CP, CB, ty, tx);
    const float dskip = skip[h];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = 4 * ty + i;
        if (t >= m) continue;
        const float e = expf(cum[t]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = p0 + 4 * tx + j;
            if (col < p) out[(size_t)(t0 + t) * ld_out + (size_t)h * p + col] = fmaf(e, sacc[i][j], yacc[i][j]) + dskip * Xs[t * CP + 4 * tx + j];
        }
    }
}

// What follows the recurrence: y times act(z), z columns of the projection (the gate comes first), then divided by
// the root mean square of each of `groups` equal parts of the row (eps inside the root), times a weight vector;
// written in the activations' type for the output product.  One block a token, the gated row in shared memory; few
// groups are summed by the whole block one after another, many by a warp each.
template <typename IT, typename AT>
__global__ void __launch_bounds__(256)
gate_group_norm_kernel(const float* __restrict__ y, int ld_y, const IT* __restrict__ proj, int n_in, size_t in_stride,
                       int row_stride, int z_off, const float* __restrict__ w, float eps, int groups, int W, int gate_act,
                       AT* __restrict__ out, int ld_out, const int* __restrict__ slot_of_token) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float rowbuf[];       // W floats + 33
    float* red = rowbuf + W;
    const int t = blockIdx.x;
    if (slot_of_token[t] < 0) return;
    const float* src = y + (size_t)t * ld_y;
    const IT* z = proj + (size_t)t * row_stride + z_off;
    const int gw = W / groups;
    AT* dst = out + (size_t)t * ld_out;
    // four columns a thread where sizes and addresses allow
    const bool vec = (gw & 3) == 0 && (ld_y & 3) == 0 && (row_stride & 3) == 0 && (z_off & 3) == 0 && (in_stride & 3) == 0 &&
                     (ld_out & 3) == 0 && ((uintptr_t)y & 15) == 0 && ((uintptr_t)proj & (4 * sizeof(IT) - 1)) == 0 &&
                     ((uintptr_t)out & (4 * sizeof(AT) - 1)) == 0 && (!w || ((uintptr_t)w & 15) == 0);
    if (vec) {
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
            float v[4], g[4] = {0.f, 0.f, 0.f, 0.f};
            load4(src + i, v);
            for (int s = 0; s < n_in; ++s) {
                float p[4];
                load4(z + (size_t)s * in_stride + i, p);
#pragma unroll
                for (int u = 0; u < 4; ++u) g[u] += p[u];
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] *= gate_act == 1 ? silu(g[u]) : (gate_act == 2 ? sigmoid_f32(g[u]) : 1.f);
            store4(rowbuf + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            const float g = sum_in(z + i, n_in, in_stride);
            rowbuf[i] = src[i] * (gate_act == 1 ? silu(g) : (gate_act == 2 ? sigmoid_f32(g) : 1.f));
        }
    }
    __syncthreads();
    if (vec && groups <= 8) {
        for (int gi = 0; gi < groups; ++gi) {
            float ss = 0.f;
            for (int i = threadIdx.x * 4; i < gw; i += blockDim.x * 4) {
                float v[4];
                load4(rowbuf + gi * gw + i, v);
                ss += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
            }
            const float inv = rsqrtf(block_sum(ss, red) / (float)gw + eps);
            for (int i = threadIdx.x * 4; i < gw; i += blockDim.x * 4) {
                const int c = gi * gw + i;
                float v[4], ww[4] = {1.f, 1.f, 1.f, 1.f};
                load4(rowbuf + c, v);
                if (w) load4(w + c, ww);
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = v[u] * inv * ww[u];
                store4(dst + c, v);
            }
        }
        return;
    }
    if (groups <= 8) {
        for (int gi = 0; gi < groups; ++gi) {
            float ss = 0.f;
            for (int i = threadIdx.x; i < gw; i += blockDim.x) { const float v = rowbuf[gi * gw + i]; ss = fmaf(v, v, ss); }
            const float inv = rsqrtf(block_sum(ss, red) / (float)gw + eps);
            for (int i = threadIdx.x; i < gw; i += blockDim.x) {
                const int c = gi * gw + i;
                dst[c] = from_f32<AT>(rowbuf[c] * inv * (w ? w[c] : 1.f));
            }
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int gi = warp; gi < groups; gi += nwarps) {
        float ss = 0.f;
        for (int i = lane; i < gw; i += 32) { const float v = rowbuf[gi * gw + i]; ss = fmaf(v, v, ss); }
        const float inv = rsqrtf(warp_sum(ss) / (float)gw + eps);
        for (int i = lane; i < gw; i += 32) {
            const int c = gi * gw + i;
            dst[c] = from_f32<AT>(rowbuf[c] * inv * (w ? w[c] : 1.f));
        }
    }
}
}  // namespace

extern "C" int rb_gate_group_norm(const float* y, int ld_y, const void* proj, int proj_dtype, int n_in, long long in_stride,
                                  int row_stride, int z_off, const float* w, float eps, int groups, int W, int gate_act,
                                  void* out, int out_dtype, int ld_out, const int* slot_of_token, int T, void* stream) {
    if (T <= 0) return RB_OK;
    if (groups <= 0 || W <= 0 || W % groups || n_in < 1) return RB_ERR_BAD_SIZE;
    const size_t smem = (size_t)(W + 33) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_GGN(IT, AT)                                                                                                    \
    do {                                                                                                                  \
        auto k = gate_group_norm_kernel<IT, AT>;                                                                          \
        if (smem > 48 * 1024) {                                                                                           \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        RB_LAUNCH((k), dim3(T), dim3(256), smem, s, y, ld_y, (const IT*)proj, n_in, (size_t)in_stride, row_stride, z_off, w, \
                  eps, groups, W, gate_act, (AT*)out, ld_out, slot_of_token);                                              \
    } while (0)
    if (proj_dtype == RB_BF16 && out_dtype == RB_BF16) RB_GGN(bf, bf);
    else if (proj_dtype == RB_F32 && out_dtype == RB_BF16) RB_GGN(float, bf);
    else if (proj_dtype == RB_F32 && out_dtype == RB_F32) RB_GGN(float, float);
    else return RB_ERR_BAD_DTYPE;
#undef RB_GGN
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_causal_conv(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int col0,
                              int channels, int taps, const float* w, const float* bias, int act, float* kept,
                              const int* seq_slot, const int* cu_q, int n_seqs, int max_q_len, float* out, int ld_out,
                              void* stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return RB_OK;
    if (channels <= 0 || taps < 1 || taps > CONV_MAX_TAPS || n_in < 1 || n_seqs > 65535) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((channels + CONV_CH - 1) / CONV_CH, (max_q_len + CONV_TOK - 1) / CONV_TOK, n_seqs);
    if (grid.y > 65535) return RB_ERR_BAD_SIZE;
#define RB_CONV(IT, TAPS)                                                                                                      \
    RB_LAUNCH((causal_conv_kernel<IT, TAPS>), grid, dim3(CONV_CH), 0, s, (const IT*)in, n_in, (size_t)in_stride, row_stride, col0, \
              channels, taps, w, bias, act, kept, seq_slot, cu_q, out, ld_out)
#define RB_CONV_T(IT)                                                                                                          \
    do {                                                                                                                       \
        if (taps == 4) RB_CONV(IT, 4);                                                                                         \
        else if (taps == 3) RB_CONV(IT, 3);                                                                                    \
        else if (taps == 2) RB_CONV(IT, 2);                                                                                    \
        else RB_CONV(IT, 0);                                                                                                   \
    } while (0)
    if (in_dtype == RB_F32) RB_CONV_T(float);
    else if (in_dtype == RB_BF16) RB_CONV_T(__nv_bfloat16);
    else return RB_ERR_BAD_DTYPE;
#undef RB_CONV_T
#undef RB_CONV
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_ssm_scan(const float* u, int ld_u, int x_off, int b_off, int c_off, const void* raw, int raw_dtype, int n_in,
                           long long in_stride, int row_stride, int dt_off, const float* dt_bias, const float* a_log,
                           const float* skip, int heads, int groups, int n, int p, float* state, const int* seq_slot,
                           const int* cu_q, int n_seqs, int one_token_each, float* out, int ld_out, void* stream) {
    if (n_seqs <= 0) return RB_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || n <= 0 || p <= 0 || n_in < 1 || n_seqs > 65535 || heads > 65535)
        return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    if (one_token_each && (size_t)2 * n * sizeof(float) <= 40 * 1024) {
        const dim3 grid1((p + 31) / 32, heads, n_seqs);
        const size_t smem1 = (size_t)2 * n * sizeof(float);
        if (raw_dtype == RB_F32)
            RB_LAUNCH((ssm_step_kernel<float>), grid1, dim3(256), smem1, s, u, ld_u, x_off, b_off, c_off, (const float*)raw, n_in,
                      (size_t)in_stride, row_stride, dt_off, dt_bias, a_log, skip, heads, groups, n, p, state, seq_slot, cu_q, out, ld_out);
        else if (raw_dtype == RB_BF16)
            RB_LAUNCH((ssm_step_kernel<__nv_bfloat16>), grid1, dim3(256), smem1, s, u, ld_u, x_off, b_off, c_off,
                      (const __nv_bfloat16*)raw, n_in, (size_t)in_stride, row_stride, dt_off, dt_bias, a_log, skip, heads, groups, n, p,
                      state, seq_slot, cu_q, out, ld_out);
        else
            return RB_ERR_BAD_DTYPE;
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    // a tile of the state's columns: as wide as 64 KB of shared memory hold with n rows, at most 64, at most p
    int VT = p < 64 ? p : 64;
    while (VT > 1 && (size_t)n * VT * sizeof(float) > 64 * 1024) VT = (VT + 1) / 2;
    int P = SCAN_THREADS / VT;
    if (P > n) P = n;
    if (P < 1) P = 1;
    const size_t smem = ((size_t)n * VT + 2 * SCAN_TB * n + SCAN_TB * VT + (size_t)SCAN_TB * P * VT + 2 * SCAN_TB) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    const dim3 grid((p + VT - 1) / VT, heads, n_seqs);
#define RB_SCAN(IT)                                                                                                          \
    do {                                                                                                                     \
        auto k = ssm_scan_kernel<IT>;                                                                                        \
        if (smem > 48 * 1024) {                                                                                              \
            cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                 \
            if (e != cudaSuccess) return (int)e;                                                                             \
        }                                                                                                                    \
        RB_LAUNCH((k), grid, dim3(SCAN_THREADS), smem, s, u, ld_u, x_off, b_off, c_off, (const IT*)raw, n_in, (size_t)in_stride, \
                  row_stride, dt_off, dt_bias, a_log, skip, heads, groups, n, p, state, seq_slot, cu_q, out, ld_out, VT, P);  \
    } while (0)
    if (raw_dtype == RB_F32) RB_SCAN(float);
    else if (raw_dtype == RB_BF16) RB_SCAN(__nv_bfloat16);
    else return RB_ERR_BAD_DTYPE;
#undef RB_SCAN
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_ssm_scan_blocks(const float* u, int ld_u, int x_off, int b_off, int c_off, const void* raw, int raw_dtype,
                                  int n_in, long long in_stride, int row_stride, int dt_off, const float* dt_bias,
                                  const float* a_log, const float* skip, int heads, int groups, int n, int p, float* state,
                                  const int* seq_slot, const int* cu_q, int n_seqs, int n_blocks, float* work,
                                  float* block_decay, float* cb, float* out, int ld_out, void* stream) {
    if (n_seqs <= 0 || n_blocks <= 0) return RB_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || n <= 0 || p <= 0 || n_in < 1 || n_seqs > 65535 || heads > 65535 ||
        n_blocks > 65535)
        return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const dim3 grid((p + CP - 1) / CP, heads, n_blocks);
    const size_t smem = (size_t)(CN * CL + CN * CP + CB * CP + 3 * CB) * sizeof(float);
    RB_LAUNCH((ssm_block_cb_kernel), dim3(groups, n_blocks), dim3(CT), 0, s, u, ld_u, b_off, c_off, groups, n, seq_slot, cu_q, n_seqs, cb);
    RB_LAUNCH_CHECK();
#define RB_SSB(IT)                                                                                                              \
    do {                                                                                                                        \
        RB_LAUNCH((ssm_block_sum_kernel<IT>), grid, dim3(CT), 0, s, u, ld_u, x_off, b_off, (const IT*)raw, n_in, (size_t)in_stride, \
                  row_stride, dt_off, dt_bias, a_log, heads, groups, n, p, seq_slot, cu_q, n_seqs, work, block_decay);           \
        RB_LAUNCH_CHECK();                                                                                                      \
        RB_LAUNCH((ssm_block_states_kernel), dim3((n * p + 255) / 256, heads, n_seqs), dim3(256), 0, s, work, block_decay, state, \
                  heads, n * p, seq_slot, cu_q);                                                                                 \
        RB_LAUNCH_CHECK();                                                                                                      \
        auto k = ssm_block_out_kernel<IT>;                                                                                      \
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                        \
        if (e != cudaSuccess) return (int)e;                                                                                    \
        RB_LAUNCH((k), grid, dim3(CT), smem, s, u, ld_u, x_off, c_off, (const IT*)raw, n_in, (size_t)in_stride, row_stride,       \
                  dt_off, dt_bias, a_log, skip, heads, groups, n, p, seq_slot, cu_q, n_seqs, work, cb, out, ld_out);             \
    } while (0)
    if (raw_dtype == RB_F32) RB_SSB(float);
    else if (raw_dtype == RB_BF16) RB_SSB(__nv_bfloat16);
    else return RB_ERR_BAD_DTYPE;
#undef RB_SSB
    RB_LAUNCH_CHECK();
    return RB_OK;
}
