// Per-tensor symmetric int8 quantisation: absmax scale, three rounding modes, transposing variant.
// All kernels are HBM-streaming: 128-bit loads, 128-bit packed stores, grids sized in multiples of the SM count.
#include "common.cuh"

namespace tango {

thread_local int g_last_cuda_error = 0;

// ---------------------------------------------------------------------------------------------- absmax
// LW = floats per load (4, 2 or 1): rows must start on an LW-float boundary (base aligned, ld % LW == 0); the columns
// past the last full vector of a row are read one by one.
template <int LW>
__global__ void __launch_bounds__(256) absmax_kernel(const float *__restrict__ x, int64_t rows, int64_t cols,
                                                     int64_t ld, const float *__restrict__ row_scale,
                                                     float *__restrict__ scale) {
    float m = 0.f;
    const int64_t cv = cols / LW, total = rows * cv;
    // four independent loads in flight per thread (an 8-byte load per trip alone leaves HBM half idle)
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
        float t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            t[u] = 0.f;
            if (i < total) {
                int64_t r, c;
                if (total <= 0x7fffffff) {      // 32-bit division where it suffices
                    const uint32_t r32 = (uint32_t)i / (uint32_t)cv;
                    r = r32; c = (int64_t)((uint32_t)i - r32 * (uint32_t)cv) * LW;
                } else {
                    r = i / cv; c = (i - r * cv) * LW;
                }
                if (LW == 4) {
                    const float4 v = __ldcs(reinterpret_cast<const float4 *>(x + r * ld + c));
                    t[u] = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
                } else if (LW == 2) {
                    const float2 v = __ldcs(reinterpret_cast<const float2 *>(x + r * ld + c));
                    t[u] = fmaxf(fabsf(v.x), fabsf(v.y));
                } else {
                    t[u] = fabsf(x[r * ld + c]);
                }
                if (row_scale) t[u] = __fmul_rn(t[u], fabsf(__ldg(row_scale + r)));
            }
        }
        m = fmaxf(fmaxf(m, fmaxf(t[0], t[1])), fmaxf(t[2], t[3]));
    }
    const int64_t rem = cols - cv * LW;  // < LW columns per row left over
    if (rem > 0) {
        for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < rows * rem;
             i += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = i / rem, c = cv * LW + (i - r * rem);
            float t = fabsf(x[r * ld + c]);
            if (row_scale) t = __fmul_rn(t, fabsf(__ldg(row_scale + r)));
            m = fmaxf(m, t);
        }
    }
    block_absmax_to_scale(m, scale);
}

// Contiguous matrix whose rows do not start on 16-byte boundaries (e.g. 602 columns), with a per-row factor: the data
// is read as one flat stream of aligned 128-bit loads; a vector that straddles a row boundary (cols >= 4: at most one)
// takes the factor of the next row for its trailing elements.
__global__ void __launch_bounds__(256) absmax_flat_rows_kernel(const float *__restrict__ x, int64_t numel, int64_t cols,
                                                               const float *__restrict__ row_scale,
                                                               float *__restrict__ scale) {
    float m = 0.f;
    const int64_t n4 = numel >> 2;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const bool small = numel <= 0x7fffffff;
    for (int64_t i0 = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i0 < n4; i0 += 4 * stride) {
        float t[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int64_t i = i0 + u * stride;
            t[u] = 0.f;
            if (i < n4) {
                const float4 v = __ldcs(reinterpret_cast<const float4 *>(x) + i);
                const int64_t e = i << 2;
                int64_t r, off;
                if (small) {
                    const uint32_t r32 = (uint32_t)e / (uint32_t)cols;
                    r = r32; off = (uint32_t)e - r32 * (uint32_t)cols;
                } else {
                    r = e / cols; off = e - r * cols;
                }
                const float s0 = fabsf(__ldg(row_scale + r));
                if (off + 3 < cols) {
                    t[u] = __fmul_rn(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))), s0);
                } else {
                    const float s1 = fabsf(__ldg(row_scale + r + 1));   // r + 1 exists: the vector ends inside it
                    const float a0 = __fmul_rn(fabsf(v.x), s0);
                    const float a1 = __fmul_rn(fabsf(v.y), off + 1 < cols ? s0 : s1);
                    const float a2 = __fmul_rn(fabsf(v.z), off + 2 < cols ? s0 : s1);
                    const float a3 = __fmul_rn(fabsf(v.w), s1);
                    t[u] = fmaxf(fmaxf(a0, a1), fmaxf(a2, a3));
                }
            }
        }
        m = fmaxf(fmaxf(m, fmaxf(t[0], t[1])), fmaxf(t[2], t[3]));
    }
    const int64_t tail = (n4 << 2) + blockIdx.x * (int64_t)blockDim.x + threadIdx.x;   // numel % 4 last elements
    if (tail < numel) m = fmaxf(m, __fmul_rn(fabsf(x[tail]), fabsf(__ldg(row_scale + tail / cols))));
    block_absmax_to_scale(m, scale);
}

// ---------------------------------------------------------------------------------------------- quantize

// Optional destinations of a quantizer launch in a multi-GPU run: instead of (only) the local tensor q, every 16-byte
// piece of row r is stored at bases[k] + (row0 + r) * ldq + c0 for k < n -- the same place in the gathered table of
// every GPU of the node (peer memory mapped into this process; plain stores over NVLink).  n == 0: store to q.
struct PushTargets {
    int8_t *const *bases;
    int n;
    int64_t row0;
};

__device__ __forceinline__ void store_piece(int8_t *q, const PushTargets &push, int64_t r, int64_t ldq, int64_t c0,
                                            const uint4 &piece) {
    if (push.n == 0) {
        __stcs(reinterpret_cast<uint4 *>(q + r * ldq + c0), piece);
    } else {
        for (int k = 0; k < push.n; ++k)
            __stcs(reinterpret_cast<uint4 *>(push.bases[k] + (push.row0 + r) * ldq + c0), piece);
    }
}

// One thread produces 16 consecutive output bytes of one row (a 128-bit store).  LW = floats per input load.
template <int LW>
__global__ void __launch_bounds__(256) quantize_kernel(const float *__restrict__ x, int64_t rows, int64_t cols,
                                                       int64_t ldx, const float *__restrict__ row_scale,
                                                       const float *__restrict__ scale, int8_t *__restrict__ q,
                                                       int64_t ldq, int mode, uint64_t seed, uint64_t call0,
                                                       const unsigned long long *__restrict__ step,
                                                       const PushTargets push) {
    const uint64_t call = effective_call(call0, step);
    const float inv = inv_scale(__ldg(scale));
    const int64_t groups = (ldq + 15) >> 4, total = rows * groups;
    const Philox ph{(uint32_t)seed, (uint32_t)(seed >> 32)};
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / groups, c0 = (i - r * groups) << 4;
        const float rs = row_scale ? __ldg(row_scale + r) : 1.f;
        float v[16];
        if (LW == 4 && c0 + 16 <= cols) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 t = __ldcs(reinterpret_cast<const float4 *>(x + r * ldx + c0 + 4 * k));
                v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
            }
        } else if (LW == 2 && c0 + 16 <= cols) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float2 t = __ldcs(reinterpret_cast<const float2 *>(x + r * ldx + c0 + 2 * k));
                v[2 * k] = t.x; v[2 * k + 1] = t.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) v[k] = (c0 + k < cols) ? x[r * ldx + c0 + k] : 0.f;
        }
        uint32_t packed[4] = {0, 0, 0, 0};
        uint64_t cached_blk = ~0ull;
        uint4 rnd = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float t = row_scale ? __fmul_rn(v[k], rs) : v[k];
            t = __fmul_rn(t, inv);
            float u = 0.f;
            if (mode == TANGO_ROUND_STOCHASTIC) {
                const uint64_t flat = (uint64_t)(r * cols + c0 + k);
                const uint64_t blk = flat >> 2;
                if (blk != cached_blk) {
                    rnd = ph((uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)call, (uint32_t)(call >> 32));
                    cached_blk = blk;
                }
                const uint32_t lane = (uint32_t)flat & 3u;
                const uint32_t rr = lane == 0 ? rnd.x : lane == 1 ? rnd.y : lane == 2 ? rnd.z : rnd.w;
                u = __fmul_rn((float)(rr >> 8), 5.9604644775390625e-08f);  // 2^-24
            }
            const int qi = (c0 + k < cols) ? round_to_i8(t, mode, u) : 0;
            packed[k >> 2] |= ((uint32_t)qi & 0xffu) << (8 * (k & 3));
        }
        if (c0 + 16 <= ldq) {
            store_piece(q, push, r, ldq, c0, make_uint4(packed[0], packed[1], packed[2], packed[3]));
        } else {  // ragged end of a flat (single-row) tensor
            for (int k = 0; c0 + k < ldq; ++k) q[r * ldq + c0 + k] = (int8_t)(packed[k >> 2] >> (8 * (k & 3)));
        }
    }
}

// Contiguous fp32 input of any row width (ldx == cols, e.g. 602 columns: rows that are only 8-byte aligned) to int8
// rows padded to ldq: a CTA takes R consecutive rows, whose floats are ONE contiguous, 16-byte aligned span -- read
// with perfectly coalesced 128-bit loads whatever the row width -- rounds them, lays the bytes out at the padded
// pitch in shared memory (pad bytes zero), and writes the block, which is contiguous in the output too, with
// coalesced 128-bit stores.  R is a multiple of 16, so a block starts on a multiple of four elements and a float4
// never straddles two Philox blocks.
__global__ void __launch_bounds__(256) quantize_repitch_kernel(const float *__restrict__ x, int64_t rows, int cols,
                                                               const float *__restrict__ row_scale,
                                                               const float *__restrict__ scale, int8_t *__restrict__ q,
                                                               int ldq, int R, int mode, uint64_t seed, uint64_t call0,
                                                               const unsigned long long *__restrict__ step,
                                                               const PushTargets push) {
    extern __shared__ __align__(16) int8_t rp_tile[];
    const uint64_t call = effective_call(call0, step);
    const float inv = inv_scale(__ldg(scale));
    const Philox ph{(uint32_t)seed, (uint32_t)(seed >> 32)};
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int pad = ldq - cols;
    for (int64_t r0 = (int64_t)blockIdx.x * R; r0 < rows; r0 += (int64_t)gridDim.x * R) {
        const int nr = (int)min((int64_t)R, rows - r0);
        const int n_el = nr * cols;
        for (int i = tid; i < nr * pad; i += nthr) rp_tile[(i / pad) * ldq + cols + i % pad] = 0;
        const float *base = x + r0 * cols;
        const uint64_t flat_base = (uint64_t)r0 * (uint64_t)cols;      // multiple of 16 elements
        const int n4 = n_el >> 2;
        for (int i = tid; i < n4; i += nthr) {
            const float4 v4 = __ldcs(reinterpret_cast<const float4 *>(base) + i);
            const float v[4] = {v4.x, v4.y, v4.z, v4.w};
            int r = (4 * i) / cols, c = 4 * i - r * cols;
            uint4 rnd = make_uint4(0, 0, 0, 0);
            if (mode == TANGO_ROUND_STOCHASTIC) {
                const uint64_t blk = (flat_base >> 2) + (uint64_t)i;
                rnd = ph((uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)call, (uint32_t)(call >> 32));
            }
            const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
            float rs = row_scale ? __ldg(row_scale + r0 + r) : 1.f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float t = row_scale ? __fmul_rn(v[e], rs) : v[e];
                t = __fmul_rn(t, inv);
                const float u = (mode == TANGO_ROUND_STOCHASTIC) ? __fmul_rn((float)(rr[e] >> 8), 5.9604644775390625e-08f) : 0.f;
                rp_tile[r * ldq + c] = (int8_t)round_to_i8(t, mode, u);
                if (++c == cols) {
                    c = 0; ++r;
                    if (row_scale && e < 3 && r < nr) rs = __ldg(row_scale + r0 + r);
                }
            }
        }
        for (int k = (n4 << 2) + tid; k < n_el; k += nthr) {          // last block only: up to three leftover elements
            const int r = k / cols, c = k - r * cols;
            float t = base[k];
            if (row_scale) t = __fmul_rn(t, __ldg(row_scale + r0 + r));
            t = __fmul_rn(t, inv);
            float u = 0.f;
            if (mode == TANGO_ROUND_STOCHASTIC) {
                uint64_t cached = ~0ull;
                uint4 rnd;
                u = sr_uniform(ph, flat_base + (uint64_t)k, call, cached, rnd);
            }
            rp_tile[r * ldq + c] = (int8_t)round_to_i8(t, mode, u);
        }
        __syncthreads();
        const int ppr = ldq >> 4, pieces = nr * ppr;
        for (int i = tid; i < pieces; i += nthr) {
            const int r = i / ppr, c0 = (i - r * ppr) << 4;
            store_piece(q, push, r0 + r, ldq, c0, *reinterpret_cast<const uint4 *>(rp_tile + (size_t)i * 16));
        }
        __syncthreads();
    }
}

// Generic (unaligned output) version: one thread per output byte.
__global__ void __launch_bounds__(256) quantize_scalar_kernel(const float *__restrict__ x, int64_t rows, int64_t cols,
                                                              int64_t ldx, const float *__restrict__ row_scale,
                                                              const float *__restrict__ scale, int8_t *__restrict__ q,
                                                              int64_t ldq, int mode, uint64_t seed, uint64_t call0,
    const unsigned long long *__restrict__ step) {
    const uint64_t call = effective_call(call0, step);
    const float inv = inv_scale(__ldg(scale));
    const int64_t total = rows * ldq;
    const Philox ph{(uint32_t)seed, (uint32_t)(seed >> 32)};
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / ldq, c = i - r * ldq;
        int qi = 0;
        if (c < cols) {
            float t = x[r * ldx + c];
            if (row_scale) t = __fmul_rn(t, __ldg(row_scale + r));
            t = __fmul_rn(t, inv);
            float u = 0.f;
            if (mode == TANGO_ROUND_STOCHASTIC) {
                const uint64_t flat = (uint64_t)(r * cols + c), blk = flat >> 2;
                const uint4 rnd = ph((uint32_t)blk, (uint32_t)(blk >> 32), (uint32_t)call, (uint32_t)(call >> 32));
                const uint32_t lane = (uint32_t)flat & 3u;
                const uint32_t rr = lane == 0 ? rnd.x : lane == 1 ? rnd.y : lane == 2 ? rnd.z : rnd.w;
                u = __fmul_rn((float)(rr >> 8), 5.9604644775390625e-08f);
            }
            qi = round_to_i8(t, mode, u);
        }
        q[r * ldq + c] = (int8_t)qi;
    }
}

// fp32 [nrow, ncol] -> int8 [ncol, nrow] through a padded shared tile (32 x 32 elements per block step).
__global__ void __launch_bounds__(256) quantize_transpose_kernel(const float *__restrict__ x, int64_t nrow,
                                                                 int64_t ncol, const float *__restrict__ scale,
                                                                 int8_t *__restrict__ out) {
    __shared__ int8_t tile[32][33];
    const float inv = inv_scale(__ldg(scale));
    const int64_t r0 = (int64_t)blockIdx.x * 32, c0 = (int64_t)blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t r = r0 + ty + 8 * k, c = c0 + tx;
        int qi = 0;
        if (r < nrow && c < ncol) qi = round_to_i8(__fmul_rn(x[r * ncol + c], inv), TANGO_ROUND_NEAREST, 0.f);
        tile[ty + 8 * k][tx] = (int8_t)qi;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int64_t c = c0 + ty + 8 * k, r = r0 + tx;
        if (r < nrow && c < ncol) out[c * nrow + r] = tile[tx][ty + 8 * k];
    }
}

static inline int stream_grid(int64_t work_items, int threads, int per_sm) {
    int64_t blocks = ceil_div(work_items, threads);
    const int64_t cap = (int64_t)kNumSMs * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace tango

using namespace tango;

extern "C" int tango_version(void) { return 100; }

extern "C" const char *tango_strerror(int code) {
    switch (code) {
        case TANGO_OK: return "ok";
        case TANGO_EINVAL: return "invalid argument";
        case TANGO_EALIGN: return "pointer or leading dimension not aligned as required";
        case TANGO_ECUDA: return "CUDA call failed";
        case TANGO_ETIMEOUT: return "bounded device-side wait expired";
        case TANGO_ESIZE: return "size not supported by this entry point";
        default: return "unknown error";
    }
}

extern "C" int tango_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int tango_absmax_scale(const float *x, int64_t rows, int64_t cols, int64_t ld, const float *row_scale,
                                  float *scale, tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!scale || rows < 0 || cols < 0 || ld < cols) return TANGO_EINVAL;
    TANGO_CUDA_TRY(cudaMemsetAsync(scale, 0, sizeof(float), stream));
    if (rows == 0 || cols == 0) return TANGO_OK;
    if (!x) return TANGO_EINVAL;
    if (ld == cols && !row_scale) {  // contiguous: treat as one long row so the vector path applies to any shape
        cols = rows * cols; rows = 1; ld = cols;
    }
    if (row_scale && ld == cols && cols >= 4 && cols % 4 != 0 && aligned(x, 16)) {
        const int grid = stream_grid(rows * cols / 4, 256, 16);
        absmax_flat_rows_kernel<<<grid, 256, 0, stream>>>(x, rows * cols, cols, row_scale, scale);
        TANGO_LAUNCH_CHECK();
        return TANGO_OK;
    }
    const int lw = (aligned(x, 16) && (rows == 1 || ld % 4 == 0)) ? 4 : (aligned(x, 8) && (rows == 1 || ld % 2 == 0)) ? 2 : 1;
    const int grid = stream_grid(rows * ceil_div(cols, lw), 256, 16);
    if (lw == 4) absmax_kernel<4><<<grid, 256, 0, stream>>>(x, rows, cols, ld, row_scale, scale);
    else if (lw == 2) absmax_kernel<2><<<grid, 256, 0, stream>>>(x, rows, cols, ld, row_scale, scale);
    else absmax_kernel<1><<<grid, 256, 0, stream>>>(x, rows, cols, ld, row_scale, scale);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

static int launch_quantize(const float *x, int64_t rows, int64_t cols, int64_t ldx, const float *row_scale,
                           const float *scale, int8_t *q, int64_t ldq, int mode, uint64_t seed, uint64_t call,
                           const uint64_t *step_, const PushTargets &push, cudaStream_t stream) {
    const unsigned long long *step = reinterpret_cast<const unsigned long long *>(step_);
    if (rows < 0 || cols < 0 || ldx < cols || ldq < cols || mode < 0 || mode > 2) return TANGO_EINVAL;
    if (rows == 0 || ldq == 0) return TANGO_OK;
    if (!x || !scale || (push.n == 0 && !q)) return TANGO_EINVAL;
    if (push.n > 0) {
        if (!push.bases || push.row0 < 0) return TANGO_EINVAL;
        if (ldq % 16 != 0) return TANGO_EALIGN;      // every piece of a pushed row is one aligned 128-bit store
    } else if (ldq == cols && ldx == cols && !row_scale) {  // contiguous in and out: one flat row (same flat index)
        cols = rows * cols; rows = 1; ldx = ldq = cols;
    }
    // contiguous rows of any width, padded int8 rows: the block-repitching kernel streams both sides fully coalesced
    if (rows >= 16 && ldx == cols && aligned(x, 16) && ldq % 16 == 0 && ldq <= 4096 && cols < (1 << 24) &&
        (push.n > 0 || aligned(q, 16))) {
        int R = (int)((12288 / cols) / 16 * 16);
        if (R < 16) R = 16;
        while ((int64_t)R * ldq > 40960 && R > 16) R -= 16;
        if ((int64_t)R * cols < (1 << 28)) {
            const int grid = stream_grid(ceil_div(rows, R) * 256, 256, 8);
            quantize_repitch_kernel<<<grid, 256, (size_t)R * ldq, stream>>>(x, rows, (int)cols, row_scale, scale, q, (int)ldq, R,
                                                                       mode, seed, call, step, push);
            TANGO_LAUNCH_CHECK();
            return TANGO_OK;
        }
    }
    if (push.n > 0 || ((ldq % 16 == 0 || rows == 1) && aligned(q, 16))) {
        const int lw = (aligned(x, 16) && (rows == 1 || ldx % 4 == 0)) ? 4 : (aligned(x, 8) && (rows == 1 || ldx % 2 == 0)) ? 2 : 1;
        const int grid = stream_grid(rows * ceil_div(ldq, 16), 256, 16);
        if (lw == 4)
            quantize_kernel<4><<<grid, 256, 0, stream>>>(x, rows, cols, ldx, row_scale, scale, q, ldq, mode, seed, call, step, push);
        else if (lw == 2)
            quantize_kernel<2><<<grid, 256, 0, stream>>>(x, rows, cols, ldx, row_scale, scale, q, ldq, mode, seed, call, step, push);
        else
            quantize_kernel<1><<<grid, 256, 0, stream>>>(x, rows, cols, ldx, row_scale, scale, q, ldq, mode, seed, call, step, push);
    } else {
        const int grid = stream_grid(rows * ldq, 256, 8);
        quantize_scalar_kernel<<<grid, 256, 0, stream>>>(x, rows, cols, ldx, row_scale, scale, q, ldq, mode, seed, call, step);
    }
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

extern "C" int tango_quantize(const float *x, int64_t rows, int64_t cols, int64_t ldx, const float *row_scale,
                              const float *scale, int8_t *q, int64_t ldq, int mode, uint64_t seed, uint64_t call,
                              const uint64_t *step, tango_stream_t stream) {
    return launch_quantize(x, rows, cols, ldx, row_scale, scale, q, ldq, mode, seed, call, step, PushTargets{nullptr, 0, 0},
                           (cudaStream_t)stream);
}

extern "C" int tango_quantize_push(const float *x, int64_t rows, int64_t cols, int64_t ldx, const float *row_scale,
                                   const float *scale, int8_t *const *tables, int n_tables, int64_t row0, int64_t ldq,
                                   int mode, uint64_t seed, uint64_t call, const uint64_t *step,
                                   tango_stream_t stream) {
    if (n_tables < 1 || n_tables > 64) return TANGO_EINVAL;
    return launch_quantize(x, rows, cols, ldx, row_scale, scale, nullptr, ldq, mode, seed, call, step,
                           PushTargets{tables, n_tables, row0}, (cudaStream_t)stream);
}

extern "C" int tango_quantize_transpose(const float *x, int64_t nrow, int64_t ncol, const float *scale, int8_t *out,
                                        tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (nrow < 0 || ncol < 0) return TANGO_EINVAL;
    if (nrow == 0 || ncol == 0) return TANGO_OK;
    if (!x || !scale || !out) return TANGO_EINVAL;
    const int64_t gx = ceil_div(nrow, 32), gy = ceil_div(ncol, 32);
    if (gy > 65535) return TANGO_ESIZE;
    quantize_transpose_kernel<<<dim3((unsigned)gx, (unsigned)gy), 256, 0, stream>>>(x, nrow, ncol, scale, out);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

// ------------------------------------------------------------------------------------------------ ReLU-gradient fusion
// Backward of  y = relu(...):  the incoming gradient g is masked by (y > 0) before anything else uses it.  The two
// kernels below read g and y directly, so the masked gradient is never written to memory:
//   relu_grad_stats : scale = max |m| / 127 with m = (y > 0 ? g : 0) * row_scale[r], and the column sums of the masked
//                     gradient (the bias gradient), summed in a fixed order (block partials, then one pass over them)
//   relu_grad_quant : int8 m / scale, same layout rules as tango_quantize
namespace tango {

// Column c of the tile is owned by thread tx (VW consecutive columns per thread: 4 with 128-bit loads, else 1), rows
// are dealt to the ty groups; four row-steps are kept in flight per thread.
template <int VW>
__global__ void __launch_bounds__(256) relu_grad_stats_kernel(const float *__restrict__ g, int64_t ldg,
                                                              const float *__restrict__ y, int64_t ldy, int64_t rows,
                                                              int64_t cols, const float *__restrict__ row_scale,
                                                              float *__restrict__ scale, float *__restrict__ partial,
                                                              int cw, int64_t rows_per_block) {
    __shared__ float s_part[256 * VW];
    const int tx = threadIdx.x % cw, ty = threadIdx.x / cw, nty = 256 / cw;
    const int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
    const int64_t r1 = min(rows, r0 + rows_per_block);
    float amax = 0.f;
    for (int64_t c0 = 0; c0 < cols; c0 += (int64_t)cw * VW) {
        const int64_t c = c0 + (int64_t)tx * VW;
        float sum[VW];
#pragma unroll
        for (int k = 0; k < VW; ++k) sum[k] = 0.f;
        if (c < cols) {
#pragma unroll 4
            for (int64_t r = r0 + ty; r < r1; r += nty) {
                float gv[VW], yv[VW];
                if (VW == 4) {
                    const float4 a = __ldcs(reinterpret_cast<const float4 *>(g + r * ldg + c));
                    const float4 m = __ldcs(reinterpret_cast<const float4 *>(y + r * ldy + c));
                    gv[0] = a.x; gv[VW > 1 ? 1 : 0] = a.y; gv[VW > 2 ? 2 : 0] = a.z; gv[VW > 3 ? 3 : 0] = a.w;
                    yv[0] = m.x; yv[VW > 1 ? 1 : 0] = m.y; yv[VW > 2 ? 2 : 0] = m.z; yv[VW > 3 ? 3 : 0] = m.w;
                } else {
                    gv[0] = __ldcs(g + r * ldg + c);
                    yv[0] = __ldcs(y + r * ldy + c);
                }
                const float rs = row_scale ? fabsf(__ldg(row_scale + r)) : 1.f;
#pragma unroll
                for (int k = 0; k < VW; ++k) {
                    const float v = yv[k] > 0.f ? gv[k] : 0.f;
                    sum[k] = __fadd_rn(sum[k], v);
                    float a = fabsf(v);
                    if (row_scale) a = __fmul_rn(a, rs);
                    amax = fmaxf(amax, a);
                }
            }
        }
        if (partial) {
            __syncthreads();
#pragma unroll
            for (int k = 0; k < VW; ++k) s_part[threadIdx.x * VW + k] = sum[k];
            __syncthreads();
            if (ty == 0 && c < cols) {
#pragma unroll
                for (int k = 0; k < VW; ++k) {
                    float t = 0.f;
                    for (int j = 0; j < nty; ++j) t = __fadd_rn(t, s_part[(j * cw + tx) * VW + k]);
                    partial[(int64_t)blockIdx.x * cols + c + k] = t;
                }
            }
        }
    }
    block_absmax_to_scale(amax, scale);
}

// Adds the per-block partial column sums in a fixed order (32 interleaved chains per column, then the 32 chain totals
// in order), so the bias gradient does not depend on scheduling.
__global__ void __launch_bounds__(1024) colsum_finish_kernel(const float *__restrict__ partial, int nblocks,
                                                             int64_t cols, float *__restrict__ colsum) {
    __shared__ float part[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * 32 + tx;
    float t = 0.f;
    if (c < cols)
        for (int b = ty; b < nblocks; b += 32) t = __fadd_rn(t, partial[(int64_t)b * cols + c]);
    part[ty][tx] = t;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float r = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) r = __fadd_rn(r, part[k][tx]);
        colsum[c] = r;
    }
}

template <bool VEC4>
__global__ void __launch_bounds__(256) relu_grad_quant_kernel(const float *__restrict__ g, int64_t ldg,
                                                              const float *__restrict__ y, int64_t ldy, int64_t rows,
                                                              int64_t cols, const float *__restrict__ row_scale,
                                                              const float *__restrict__ scale, int8_t *__restrict__ q,
                                                              int64_t ldq, int mode, uint64_t seed, uint64_t call0,
                                                              const unsigned long long *__restrict__ step,
                                                              const PushTargets push) {
    const uint64_t call = effective_call(call0, step);
    const float inv = inv_scale(__ldg(scale));
    const int64_t groups = ldq >> 4, total = rows * groups;   // ldq % 16 == 0
    const Philox ph{(uint32_t)seed, (uint32_t)(seed >> 32)};
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / groups, c0 = (i - r * groups) << 4;
        const float rs = row_scale ? __ldg(row_scale + r) : 1.f;
        float v[16];
        if (VEC4 && c0 + 16 <= cols) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 a = __ldcs(reinterpret_cast<const float4 *>(g + r * ldg + c0 + 4 * k));
                const float4 m = __ldcs(reinterpret_cast<const float4 *>(y + r * ldy + c0 + 4 * k));
                v[4 * k] = m.x > 0.f ? a.x : 0.f; v[4 * k + 1] = m.y > 0.f ? a.y : 0.f;
                v[4 * k + 2] = m.z > 0.f ? a.z : 0.f; v[4 * k + 3] = m.w > 0.f ? a.w : 0.f;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k)
                v[k] = (c0 + k < cols && y[r * ldy + c0 + k] > 0.f) ? g[r * ldg + c0 + k] : 0.f;
        }
        uint32_t packed[4] = {0, 0, 0, 0};
        uint64_t cached_blk = ~0ull;
        uint4 rnd = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float t = row_scale ? __fmul_rn(v[k], rs) : v[k];
            t = __fmul_rn(t, inv);
            float u = 0.f;
            if (mode == TANGO_ROUND_STOCHASTIC) u = sr_uniform(ph, (uint64_t)(r * cols + c0 + k), call, cached_blk, rnd);
            const int qi = (c0 + k < cols) ? round_to_i8(t, mode, u) : 0;
            packed[k >> 2] |= ((uint32_t)qi & 0xffu) << (8 * (k & 3));
        }
        store_piece(q, push, r, ldq, c0, make_uint4(packed[0], packed[1], packed[2], packed[3]));
    }
}

static int stats_blocks(int64_t rows) {
    int64_t b = ceil_div(rows, 64);
    if (b > kNumSMs * 8) b = kNumSMs * 8;
    return (int)(b < 1 ? 1 : b);
}

}  // namespace tango

extern "C" int64_t tango_relu_grad_stats_scratch_bytes(int64_t rows, int64_t cols) {
    if (rows < 0 || cols < 0) return 0;
    return (int64_t)stats_blocks(rows) * cols * (int64_t)sizeof(float);
}

extern "C" int tango_relu_grad_stats(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows,
                                     int64_t cols, const float *row_scale, float *scale, float *colsum, void *scratch,
                                     int64_t scratch_bytes, tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (rows < 0 || cols < 0 || ldg < cols || ldy < cols || !scale) return TANGO_EINVAL;
    TANGO_CUDA_TRY(cudaMemsetAsync(scale, 0, sizeof(float), stream));
    if (colsum && cols > 0 && rows == 0) TANGO_CUDA_TRY(cudaMemsetAsync(colsum, 0, sizeof(float) * (size_t)cols, stream));
    if (rows == 0 || cols == 0) return TANGO_OK;
    if (!g || !y) return TANGO_EINVAL;
    const int nb = stats_blocks(rows);
    if (colsum && (!scratch || scratch_bytes < tango_relu_grad_stats_scratch_bytes(rows, cols))) return TANGO_ESIZE;
    const bool vec = cols % 4 == 0 && ldg % 4 == 0 && ldy % 4 == 0 && aligned(g, 16) && aligned(y, 16);
    const int64_t tcols = vec ? cols / 4 : cols;   // columns in units of one thread's share
    int cw = 1;
    while (cw < tcols && cw < 256) cw <<= 1;
    const int64_t rpb = ceil_div(rows, nb);
    float *part = colsum ? (float *)scratch : nullptr;
    if (vec) relu_grad_stats_kernel<4><<<nb, 256, 0, stream>>>(g, ldg, y, ldy, rows, cols, row_scale, scale, part, cw, rpb);
    else relu_grad_stats_kernel<1><<<nb, 256, 0, stream>>>(g, ldg, y, ldy, rows, cols, row_scale, scale, part, cw, rpb);
    TANGO_LAUNCH_CHECK();
    if (colsum) {
        colsum_finish_kernel<<<(unsigned)ceil_div(cols, 32), 1024, 0, stream>>>((const float *)scratch, nb, cols, colsum);
        TANGO_LAUNCH_CHECK();
    }
    return TANGO_OK;
}

static int launch_relu_grad_quant(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows, int64_t cols,
                                  const float *row_scale, const float *scale, int8_t *q, int64_t ldq, int mode,
                                  uint64_t seed, uint64_t call, const uint64_t *step_, const PushTargets &push,
                                  cudaStream_t stream) {
    const unsigned long long *step = reinterpret_cast<const unsigned long long *>(step_);
    if (rows < 0 || cols < 0 || ldg < cols || ldy < cols || ldq < cols || mode < 0 || mode > 2) return TANGO_EINVAL;
    if (rows == 0 || ldq == 0) return TANGO_OK;
    if (!g || !y || !scale || (push.n == 0 && !q)) return TANGO_EINVAL;
    if (push.n > 0 && (!push.bases || push.row0 < 0)) return TANGO_EINVAL;
    if (ldq % 16 != 0 || (push.n == 0 && !aligned(q, 16))) return TANGO_EALIGN;
    const bool vec = ldg % 4 == 0 && ldy % 4 == 0 && aligned(g, 16) && aligned(y, 16);
    const int grid = stream_grid(rows * (ldq / 16), 256, 16);
    if (vec) relu_grad_quant_kernel<true><<<grid, 256, 0, stream>>>(g, ldg, y, ldy, rows, cols, row_scale, scale, q, ldq, mode, seed, call, step, push);
    else relu_grad_quant_kernel<false><<<grid, 256, 0, stream>>>(g, ldg, y, ldy, rows, cols, row_scale, scale, q, ldq, mode, seed, call, step, push);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

extern "C" int tango_quantize_relu_grad(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows,
                                        int64_t cols, const float *row_scale, const float *scale, int8_t *q,
                                        int64_t ldq, int mode, uint64_t seed, uint64_t call, const uint64_t *step,
                                        tango_stream_t stream) {
    return launch_relu_grad_quant(g, ldg, y, ldy, rows, cols, row_scale, scale, q, ldq, mode, seed, call, step,
                                  PushTargets{nullptr, 0, 0}, (cudaStream_t)stream);
}

extern "C" int tango_quantize_relu_grad_push(const float *g, int64_t ldg, const float *y, int64_t ldy, int64_t rows,
                                             int64_t cols, const float *row_scale, const float *scale,
                                             int8_t *const *tables, int n_tables, int64_t row0, int64_t ldq, int mode,
                                             uint64_t seed, uint64_t call, const uint64_t *step,
                                             tango_stream_t stream) {
    if (n_tables < 1 || n_tables > 64) return TANGO_EINVAL;
    return launch_relu_grad_quant(g, ldg, y, ldy, rows, cols, row_scale, scale, nullptr, ldq, mode, seed, call, step,
                                  PushTargets{tables, n_tables, row0}, (cudaStream_t)stream);
}
