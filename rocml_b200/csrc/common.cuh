// Shared helpers of the kernels: element types, conversions, reductions, launch checks.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

// Element type codes of the C interface.
#define RB_F32 0
#define RB_BF16 1

// Return codes of the C interface beyond cudaError_t values (which are returned as they are).
#define RB_OK 0
#define RB_ERR_BAD_SIZE 10001      // a size the kernel does not take
#define RB_ERR_BAD_DTYPE 10002     // an element type combination that is not built
#define RB_ERR_BAD_ALIGN 10003     // a pointer or stride that breaks an alignment rule
#define RB_ERR_TIMEOUT 10004       // a bounded wait inside a kernel ran out
#define RB_ERR_NO_DRIVER_FN 10005  // a driver entry point could not be found
#define RB_ERR_IO 10006            // a file could not be read

#define RB_PAGE 64  // tokens per cache page

#define RB_LAUNCH_CHECK()                         \
    do {                                          \
        cudaError_t e__ = cudaGetLastError();     \
        if (e__ != cudaSuccess) return (int)e__;  \
    } while (0)
#define RB_LAUNCH(...)                                       \
    do {                                                     \
        cudaError_t e__ = rb::launch(__VA_ARGS__);           \
        if (e__ != cudaSuccess) return (int)e__;             \
    } while (0)

namespace rb {

// ---- programmatic dependent launch ------------------------------------------------------------
// Every kernel of the library is launched so that it may be scheduled while its predecessor in the
// stream is still running: it signals at once that its own successor may be scheduled
// (pdl_trigger), does whatever does not depend on the predecessor (set-up, and for the matrix
// products the first tiles of the weights), and only then waits for the predecessor's results
// (pdl_wait, which returns once the predecessor has finished and its writes are visible).  Without
// the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool pdl_enabled();  // defined in launch.cu: on unless RB_PDL=0 is set

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the grid's blocks grouped into clusters (every grid extent a multiple of the cluster's):
// the blocks of a cluster run at the same time and can read and write each other's shared memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem,
                                    cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The lowest key position a query at `pos` sees under a layer's mask, carried in one integer `window`:
// 0: every earlier key; n > 0: the last n keys (its own included); -n: the keys of its own block of n
// positions, blocks counted from position 0 of the sequence.  Never decreases as pos grows.
__device__ __forceinline__ int span_lo(int pos, int window) {
    return window > 0 ? max(0, pos - window + 1) : (window < 0 ? pos - pos % (-window) : 0);
}

// Two more parts of a layer's mask and weights, beside `window`.  `keep` (>= 0): the keys at positions below it
// stay visible to every later query whatever the window says (they keep their own positions).  `sink`: one more
// term exp(sink) in the softmax's denominator, with no value of its own (RB_NO_SINK: none); a row's weights then
// sum to less than one.
#define RB_NO_SINK (-3.0e38f)
__device__ __forceinline__ bool has_sink(float sink) { return sink > -1.0e38f; }
// What the sink does to a finished row: with running maximum m and sum l, the factor for the accumulated values
// (returned) and the new sum (through l): m' = max(m, sink), l' = l e^(m - m') + e^(sink - m').
__device__ __forceinline__ float add_sink(float m, float& l, float sink) {
    const float m2 = fmaxf(m, sink);
    const float a = expf(m - m2);
    l = l * a + expf(sink - m2);
    return a;
}

// Columns of the step's projection rows that gate an attention kernel's result value by value, so that no kernel
// of its own has to: out[t][c] *= sigmoid(sum over the partial sums of raw[s][t][c]), formed in 32-bit.
struct GateCols {
    const void* raw;        // the first gate column of the first token's row; null: no gate
    int f32;                // the columns' type: float32, or bfloat16
    int n_in;               // partial sums, added in order
    long long in_stride;    // elements between two partial sums
    long long row_stride;   // elements between two tokens
};
__device__ __forceinline__ float sigmoid_f32(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float gate_factor(const GateCols& g, size_t t, size_t col) {
    float z = 0.f;
    if (g.f32) {
        const float* p = static_cast<const float*>(g.raw) + t * g.row_stride + col;
        for (int s = 0; s < g.n_in; ++s) z += p[(size_t)s * g.in_stride];
    } else {
        const __nv_bfloat16* p = static_cast<const __nv_bfloat16*>(g.raw) + t * g.row_stride + col;
        for (int s = 0; s < g.n_in; ++s) z += __bfloat162float(p[(size_t)s * g.in_stride]);
    }
    return sigmoid_f32(z);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// gelu in its tanh form: z / 2 * (1 + tanh(sqrt(2 / pi) * (z + 0.044715 z^3))), 32-bit
__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }

// Four neighbouring elements at once (the pointer on 4 elements' alignment).
__device__ __forceinline__ void load4(const float* p, float* x) {
    const float4 f = *reinterpret_cast<const float4*>(p);
    x[0] = f.x; x[1] = f.y; x[2] = f.z; x[3] = f.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* x) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    x[0] = __uint_as_float(raw.x << 16); x[1] = __uint_as_float(raw.x & 0xFFFF0000u);
    x[2] = __uint_as_float(raw.y << 16); x[3] = __uint_as_float(raw.y & 0xFFFF0000u);
}
__device__ __forceinline__ void store4(float* p, const float* x) {
    *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float* x) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace rb
