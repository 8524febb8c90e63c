// Shared helpers for the tango_b200 kernels (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "tango_b200.h"

namespace tango {

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return TANGO_ECUDA;
}

#define TANGO_CUDA_TRY(expr)                                   \
    do {                                                       \
        cudaError_t _e = (expr);                               \
        if (_e != cudaSuccess) return ::tango::cuda_fail(_e);  \
    } while (0)

#define TANGO_LAUNCH_CHECK() TANGO_CUDA_TRY(cudaPeekAtLastError())

inline bool aligned(const void *p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline int64_t ceil_div(int64_t x, int64_t m) { return (x + m - 1) / m; }

constexpr int kNumSMs = 148;  // B200

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Non-negative floats order like their bit patterns, so an integer atomicMax is an exact float max.
__device__ __forceinline__ void atomic_max_nonneg(float *addr, float v) {
    atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
}

// Block-wide max of a non-negative value, then one atomic per block of (max / 127).
__device__ __forceinline__ void block_absmax_to_scale(float thread_max, float *scale_out) {
    __shared__ float s_warp[32];
    float m = warp_max(thread_max);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    if (lane == 0) s_warp[warp] = m;
    __syncthreads();
    if (warp == 0) {
        m = lane < nwarp ? s_warp[lane] : 0.f;
        m = warp_max(m);
        if (lane == 0) atomic_max_nonneg(scale_out, __fdiv_rn(m, 127.0f));
    }
}

// 1/s; 0 when s is 0 or so small (subnormal) that the reciprocal overflows, so such tensors quantize to zeros.
__device__ __forceinline__ float inv_scale(float s) {
    if (s == 0.f) return 0.f;
    const float inv = __fdiv_rn(1.0f, s);
    return isinf(inv) ? 0.f : inv;
}

// Internal (not exported): the dense hub region of the SpMM on the tcgen05 int8 GEMM.  `tiles` holds n_tiles stored
// 128 x 128 int8 tiles ([n_tiles * 128, 128], row-major); work item u = (row tile, first stored tile, first column
// tile, tiles) adds sum_t tile[first + t] . b[128 (col tile + t) .. , :] into ws rows 128 * row tile .. with integer
// atomics.  b is [k, ldb] (k a multiple of 128, ldb a multiple of 16), ws has m rows.  Defined in igemm_tcgen05.cu.
int igemm_accumulate_tiles_i32(const int8_t *tiles, int64_t n_tiles, const int32_t *units, int64_t n_units,
                               const int8_t *b, int64_t ldb, int64_t m, int64_t n, int64_t k, int32_t *ws,
                               int64_t ldws, int *status, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------- Philox4x32-10
struct Philox {
    uint32_t k0, k1;
    __device__ __forceinline__ uint4 operator()(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) const {
        uint32_t a = k0, b = k1;
#pragma unroll
        for (int r = 0; r < 10; ++r) {
            const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
            const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
            const uint32_t n0 = hi1 ^ c1 ^ a, n2 = hi0 ^ c3 ^ b;
            c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
            a += 0x9E3779B9u; b += 0xBB67AE85u;
        }
        return make_uint4(c0, c1, c2, c3);
    }
};

__device__ __forceinline__ int round_to_i8(float t, int mode, float u) {
    float r;
    if (mode == TANGO_ROUND_NEAREST) r = rintf(t);
    else if (mode == TANGO_ROUND_TRUNC) r = truncf(t);
    else r = floorf(__fadd_rn(t, u));
    r = fminf(fmaxf(r, -127.f), 127.f);
    return (int)r;
}

// Call counter of a stochastic-rounding draw: the host's per-call number in the low 32 bits plus, in the high 32 bits,
// a step number read from device memory -- the one part of the counter that can change between replays of a captured
// CUDA graph, whose scalar arguments are frozen at capture time.
__device__ __forceinline__ uint64_t effective_call(uint64_t call, const unsigned long long *step) {
    return step ? call + ((uint64_t)__ldg(step) << 32) : call;
}

// Stochastic-rounding uniform in [0,1) of flat element index `flat`: lane flat%4 of Philox block flat/4, keyed by
// (seed, call).  `cached_blk` / `rnd` let consecutive elements of one thread share a block.
__device__ __forceinline__ float sr_uniform(const Philox &ph, uint64_t flat, uint64_t call, uint64_t &cached_blk,
                                            uint4 &rnd) {
    const uint64_t blk = flat >> 2;
    if (blk != cached_blk) {
        rnd = ph((uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)call, (uint32_t)(call >> 32));
        cached_blk = blk;
    }
    const uint32_t lane = (uint32_t)flat & 3u;
    const uint32_t rr = lane == 0 ? rnd.x : lane == 1 ? rnd.y : lane == 2 ? rnd.z : rnd.w;
    return __fmul_rn((float)(rr >> 8), 5.9604644775390625e-08f);  // 2^-24
}

// sign-extended byte i (0..3) of a packed word, added into acc: dp4a with a one-hot selector.
template <int I>
__device__ __forceinline__ int add_byte(uint32_t w, int acc) {
    return __dp4a((int)w, (int)(1u << (8 * I)), acc);
}

}  // namespace tango
