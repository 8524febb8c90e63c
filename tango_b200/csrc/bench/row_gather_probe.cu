// Measurement aid: how fast can this GPU gather random rows of an L2-resident table into registers?
//
// The aggregation kernels of a high-degree graph read every int8 feature row hundreds of times; those reads are
// served by L2, not HBM, so the HBM roofline says little about them.  This probe gives the matching ceiling: every
// group of row_bytes / 16 lanes reads pseudo-random rows of the table with 128-bit loads, eight loads in flight per
// lane, and XORs them into a register (no arithmetic to speak of, no stores).  The benchmark divides the bytes it
// gathered by the CUDA-event time of the launch.
//
// Not part of the product library: built on its own into lib/libtango_bench_probe.so, loaded only by the benchmark.
#include <cuda_runtime.h>
#include <stdint.h>

namespace tango_bench {

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

}  // namespace tango_bench

// Gathers pseudo-random rows (row_bytes a power of two in [16, 512]) of `table` [rows, row_bytes] with 148 x
// ctas_per_sm CTAs of `threads` threads (a multiple of 32, at most 256) and returns the number of bytes the launch
// gathers, or -1 for arguments it does not take.  `sink` is a 4-byte device word that is never actually written.
extern "C" int64_t bench_probe_row_gather(const void *table, int64_t rows, int64_t row_bytes, int iters,
                                          int ctas_per_sm, int threads, uint32_t *sink, void *stream) {
    if (!table || !sink || rows < 1 || rows > 0x7fffffff || iters < 1) return -1;
    if (ctas_per_sm < 1 || ctas_per_sm > 32 || threads < 32 || threads > 256 || threads % 32) return -1;
    if (row_bytes < 16 || row_bytes > 512 || (row_bytes & (row_bytes - 1)) != 0 ||
        (reinterpret_cast<uintptr_t>(table) & 15) != 0) return -1;
    const int lanes = (int)(row_bytes / 16);
    const int blocks = 148 * ctas_per_sm;
    tango_bench::row_gather_probe_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>((const uint4 *)table, (int)rows,
                                                                                       lanes, iters, sink);
    if (cudaPeekAtLastError() != cudaSuccess) return -1;
    return (int64_t)blocks * threads * iters * 8 * 16;   // bytes gathered by the launch
}
