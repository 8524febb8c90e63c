// Measurement aid: how fast can this GPU gather random rows of an L2-resident table into registers?
//
// The aggregation kernels of a high-degree graph read every int8 feature row hundreds of times; those reads are
// served by L2, not HBM, so the HBM roofline says little about them.  This probe gives the matching ceiling: every
// group of row_bytes / 16 lanes reads pseudo-random rows of the table with 128-bit loads, eight loads in flight per
// lane, and XORs them into a register (no arithmetic to speak of, no stores).  The benchmark divides the bytes it
// gathered by the CUDA-event time of the launch.
#include "common.cuh"

namespace tango {

__global__ void __launch_bounds__(256) row_gather_probe_kernel(const uint4 *__restrict__ table, int rows, int lanes_per_row,
                                                               int iters, uint32_t *sink) {
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    uint32_t seed = (uint32_t)(tid / lanes_per_row) * 2654435761u + 12345u;   // lanes of a group draw the same rows
    const int sub = tid % lanes_per_row;
    uint4 acc = make_uint4(0, 0, 0, 0);
    for (int it = 0; it < iters; ++it) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            seed = seed * 1664525u + 1013904223u;
            const uint32_t r = (seed >> 8) % (uint32_t)rows;
            v[u] = __ldg(table + (size_t)r * lanes_per_row + sub);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) { acc.x ^= v[u].x; acc.y ^= v[u].y; acc.z ^= v[u].z; acc.w ^= v[u].w; }
    }
    if ((acc.x ^ acc.y ^ acc.z ^ acc.w) == 0x12345678u) sink[0] = 1;   // keeps the loads alive
}

}  // namespace tango

using namespace tango;

extern "C" int64_t tango_probe_row_gather(const void *table, int64_t rows, int64_t row_bytes, int iters,
                                          int ctas_per_sm, int threads, uint32_t *sink, tango_stream_t stream) {
    if (!table || !sink || rows < 1 || rows > 0x7fffffff || iters < 1) return TANGO_EINVAL;
    if (ctas_per_sm < 1 || ctas_per_sm > 32 || threads < 32 || threads > 256 || threads % 32) return TANGO_EINVAL;
    if (row_bytes < 16 || row_bytes > 512 || (row_bytes & (row_bytes - 1)) != 0 || !aligned(table, 16)) return TANGO_EALIGN;
    const int lanes = (int)(row_bytes / 16);
    const int blocks = kNumSMs * ctas_per_sm;
    row_gather_probe_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint4 *)table, (int)rows, lanes, iters, sink);
    TANGO_LAUNCH_CHECK();
    return (int64_t)blocks * threads * iters * 8 * 16;   // bytes gathered by the launch
}
