// int8 x int8 -> int32 GEMMs for the quantized linear layer on sm_100a:
// tcgen05.mma kind::i8 (M=128, N<=256, K=32 per instruction), operands staged in shared memory by TMA with the
// 128-byte swizzle, accumulators in tensor memory, read back with tcgen05.ld for the dequantising epilogue.
//
// One kernel serves the three products of the layer by choosing the operand "major" per call:
//   forward  Y [M,N]  = Xq[M,K]  . Wq[N,K]^T   A K-major,  B K-major
//   dX       dX[M,K]  = dYq[M,N] . Wq[N,K]     A K-major,  B MN-major (reduction index is the row of Wq)
//   dW       dW[N,K]  = dYq^T    . Xq[M,K]     A MN-major, B MN-major, split over the long reduction (M) with
//                                              int32 atomics into scratch, then a small dequantising kernel.
// so no transposed copies of the quantized tensors are ever written.
//
// Two kernels.  igemm_kernel (split-K dW, and the fallback): CTA = 6 warps, one output tile per CTA -- warp 0 issues
// TMA loads, warp 1 owns tensor memory and issues the MMAs (one lane), warps 2-5 run the epilogue (each reads the 32
// TMEM lanes it may access).  igemm_persistent_kernel (forward and dX): one CTA of 10 warps per SM keeps its tile of
// the B operand resident in shared memory, streams 128-row A tiles through a 3-stage TMA ring, alternates between
// two TMEM accumulators so the epilogue of one tile overlaps the MMAs of the next, and runs 8 epilogue warps.
// Every mbarrier wait is bounded: after ~2 s without progress the kernel records TANGO_ETIMEOUT in the status word,
// lets outstanding copies land, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace tango {

constexpr int kBlockK = 128;          // bytes of reduction per pipeline stage
constexpr int kTileM = 128;           // UMMA M
constexpr int kABytes = kTileM * kBlockK;  // 16 KiB either major
constexpr int kMaxStages = 8;
constexpr uint64_t kWaitTimeoutNs = 2000000000ull;

struct GemmParams {
    int M, N, K;     // D is [M, N], reduction length K
    int n_tile;      // UMMA N: multiple of 16, <= 256
    int kb_total;    // ceil(K / 128)
    int kb_per_split;
    int a_mn, b_mn;  // 1 = the operand is stored with the reduction index as its row (MN-major)
    int b_boxes;     // MN-major B: number of 128-column TMA boxes per stage; K-major: 1
    int b_bytes;     // bytes of B per stage
    int stages;
    int mode;        // 0: dequantise and store fp32; 1: atomically add int32 partial sums into ws
    float *out;
    int64_t ldo;
    int32_t *ws;
    int64_t ldws;
    const float *sa, *sb, *bias;
    const float *out_row_scale;  // optional: output row r is multiplied by out_row_scale[r] after dequantisation
    float *absmax;
    int *status;
    uint32_t tmem_cols;
    const int4 *tile_units;   // igemm_kernel: CTA x works on unit x = (row tile, first stored A tile, first k block, k blocks)
    int tma_store;   // persistent kernel: the epilogue hands 32 x 16 fp32 boxes to the TMA engine (needs ldo % 4 == 0)
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the wait was abandoned (timeout here or abort raised by another role).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    // hand-offs between the roles are short (a pipeline stage): poll for a while before starting to sleep
#pragma unroll 1
    for (int i = 0; i < 4096; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
#pragma unroll 1
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > kWaitTimeoutNs) {
            *abort_flag = 1;
            return false;
        }
        __nanosleep(64);
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Bulk tensor store shared -> global (this GPU's memory only) of one box, tracked by the issuing thread's bulk
// async-group; wait_read returns once the engine has read the shared-memory source of every committed store,
// wait_all once the stores have been performed.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (sm_100).
// Bits [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
// [46,48) version, [61,64) layout type (2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
        "[%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, "
        "[%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(192, 1)
igemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages];
    __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_acc;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // the swizzle needs 1024-byte aligned tiles
    const uint32_t stage_bytes = kABytes + p.b_bytes;
    // Regular mode: CTA (x, y, z) = (row tile, column tile, slice of the reduction).  Tile-list mode (the SpMM's dense
    // hub region): CTA x takes work item x; its A tiles are stored one after the other as [128, 128] boxes.
    int m0 = blockIdx.x * kTileM;
    const int n0 = blockIdx.y * p.n_tile;
    int kb_begin = blockIdx.z * p.kb_per_split;
    int n_iter = min(p.kb_total, kb_begin + p.kb_per_split) - kb_begin;
    int a_tile0 = -1;
    if (p.tile_units) {
        const int4 u = __ldg(p.tile_units + blockIdx.x);
        m0 = u.x * kTileM; a_tile0 = u.y; kb_begin = u.z; n_iter = u.w;
    }

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_full[s]), 1);
            mbar_init(smem_u32(&bar_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_acc), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;
    volatile int *abort_flag = &s_abort;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0 && n_iter > 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_b) : "memory");
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % p.stages;
                const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
                if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1u, abort_flag)) break;
                const uint32_t full = smem_u32(&bar_full[s]);
                const uint32_t a_dst = smem_base + s * stage_bytes, b_dst = a_dst + kABytes;
                const int kc = (kb_begin + it) * kBlockK;
                mbar_expect_tx(full, stage_bytes);
                if (a_tile0 >= 0) tma_load_2d(a_dst, &tm_a, full, 0, (a_tile0 + it) * kTileM);
                else if (!p.a_mn) tma_load_2d(a_dst, &tm_a, full, kc, m0);
                else tma_load_2d(a_dst, &tm_a, full, m0, kc);
                if (!p.b_mn) {
                    tma_load_2d(b_dst, &tm_b, full, kc, n0);
                } else {
                    for (int j = 0; j < p.b_boxes; ++j) tma_load_2d(b_dst + j * kABytes, &tm_b, full, n0 + j * 128, kc);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_iter > 0) {
            // Instruction descriptor: D = s32 (bits 4-5 = 2), A and B signed int8 (bits 7-9, 10-12 = 1),
            // operand majors (bits 15, 16), N >> 3 (bits 17-22), M >> 4 (bits 24-28).
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) |
                                   ((uint32_t)p.b_mn << 16) | ((uint32_t)(p.n_tile >> 3) << 17) |
                                   ((uint32_t)(kTileM >> 4) << 24);
            const uint32_t a_kstep = p.a_mn ? 32u * 128u : 32u;  // bytes to advance per K=32 instruction
            const uint32_t b_kstep = p.b_mn ? 32u * 128u : 32u;
            const uint32_t a_lbo = p.a_mn ? (uint32_t)kABytes : 16u, b_lbo = p.b_mn ? (uint32_t)kABytes : 16u;
            bool ok = true;
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % p.stages;
                const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
                if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_src = smem_base + s * stage_bytes, b_src = a_src + kABytes;
                const int k_rem = p.K - (kb_begin + it) * kBlockK;
                const int nk = min(4, (k_rem + 31) >> 5);
                for (int k = 0; k < nk; ++k) {
                    const uint64_t da = make_smem_desc(a_src + k * a_kstep, a_lbo, 1024u);
                    const uint64_t db = make_smem_desc(b_src + k * b_kstep, b_lbo, 1024u);
                    umma_i8(tmem_base, da, db, idesc, (it > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(&bar_empty[s]));  // frees the stage once the MMAs above have read it
            }
            if (ok) umma_commit(smem_u32(&bar_acc));   // accumulator complete
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        // Each warp drains the 32 accumulator rows it may read, 32 columns at a time: TMEM -> registers (one row per
        // lane) -> dequantise -> a padded shared-memory tile -> registers (8 lanes per row) -> 128-bit coalesced
        // global stores (or coalesced int32 atomics for the split-K mode).  The tile reuses pipeline-stage memory,
        // which is idle once the accumulator barrier has fired.
        const int q = warp & 3;  // the 32-lane quarter of tensor memory this warp may read
        const int row = m0 + q * 32 + lane;
        constexpr int kTileLd = 36;  // words per staged row: 16-byte aligned, conflict-free for 128-bit accesses
        uint32_t *tile = reinterpret_cast<uint32_t *>(smem_raw + (smem_base - smem_u32(smem_raw))) + q * 32 * kTileLd;
        bool ok = n_iter > 0;
        if (ok) ok = mbar_wait(smem_u32(&bar_acc), 0u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        float amax = 0.f;
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc = 0.f;
            if (p.mode == 0) sc = __fmul_rn(__ldg(p.sa), __ldg(p.sb));
            const bool vec_ok = p.mode == 0 ? ((p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0)
                                            : false;
            // n0 and every 32-column chunk start are even, so an even ldo keeps each row's chunk 8-byte aligned
            const bool vec2_ok = p.mode == 0 && (p.ldo & 1) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0;
            for (int c0 = 0; c0 < p.n_tile; c0 += 32) {
                const int col0 = n0 + c0;
                const int width = min(32, p.n_tile - c0);  // 32, or 16 for the last chunk
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half * 16 < width) {  // warp-uniform
                        uint32_t r[16];
                        tmem_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c0 + half * 16), r);
                        if (p.mode == 0) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const int col = col0 + half * 16 + i;
                                float v = __fmul_rn((float)(int)r[i], sc);
                                if (p.out_row_scale && row < p.M) v = __fmul_rn(v, __ldg(p.out_row_scale + row));
                                if (p.bias && col < p.N) v = __fadd_rn(v, __ldg(p.bias + col));
                                if (col < p.N && row < p.M) amax = fmaxf(amax, fabsf(v));
                                r[i] = __float_as_uint(v);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *reinterpret_cast<uint4 *>(tile + lane * kTileLd + half * 16 + 4 * i) =
                                make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                    }
                }
                __syncwarp();
                if (p.mode == 0 && vec_ok) {
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3), cv = (lane & 7) * 4;
                        const int grow = m0 + q * 32 + rr, gcol = col0 + cv;
                        if (grow < p.M && cv < width && gcol < p.N) {
                            const uint4 t = *reinterpret_cast<const uint4 *>(tile + rr * kTileLd + cv);
                            float *o = p.out + (int64_t)grow * p.ldo + gcol;
                            if (gcol + 4 <= p.N) {
                                *reinterpret_cast<uint4 *>(o) = t;
                            } else {
                                const uint32_t e[4] = {t.x, t.y, t.z, t.w};
                                for (int i = 0; i < 4 && gcol + i < p.N; ++i) o[i] = __uint_as_float(e[i]);
                            }
                        }
                    }
                } else if (p.mode == 0 && vec2_ok) {
                    // rows that are only 8-byte aligned (e.g. ldo = 602): half a warp per row, 64-bit stores
#pragma unroll 4
                    for (int it = 0; it < 16; ++it) {
                        const int rr = it * 2 + (lane >> 4), cv = (lane & 15) * 2;
                        const int grow = m0 + q * 32 + rr, gcol = col0 + cv;
                        if (grow < p.M && cv < width && gcol < p.N) {
                            const uint2 t = *reinterpret_cast<const uint2 *>(tile + rr * kTileLd + cv);
                            float *o = p.out + (int64_t)grow * p.ldo + gcol;
                            if (gcol + 2 <= p.N) *reinterpret_cast<uint2 *>(o) = t;
                            else o[0] = __uint_as_float(t.x);
                        }
                    }
                } else {
                    // one staged row per step, one column per lane: 128-byte coalesced scalar stores / atomics
                    for (int rr = 0; rr < 32; ++rr) {
                        const int grow = m0 + q * 32 + rr, gcol = col0 + lane;
                        if (grow < p.M && lane < width && gcol < p.N) {
                            const uint32_t t = tile[rr * kTileLd + lane];
                            if (p.mode == 0) p.out[(int64_t)grow * p.ldo + gcol] = __uint_as_float(t);
                            else if (t != 0) atomicAdd(p.ws + (int64_t)grow * p.ldws + gcol, (int)t);
                        }
                    }
                }
                __syncwarp();
            }
        }
        if (p.absmax && p.mode == 0) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) {
                const float s = __fdiv_rn(amax, 127.0f);
                if (s > __ldcg(p.absmax)) atomic_max_nonneg(p.absmax, s);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        // give copies that are still in flight time to land before the CTA's shared memory is released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, TANGO_ETIMEOUT);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Persistent, B-stationary variant for the products whose B operand (one N-tile of it, all of K) fits in shared
// memory next to a ring of A tiles -- the forward and dX products of the layer (W_q is a few hundred KB at most).
// One CTA per SM keeps its B tile resident, streams 128-row A tiles through a TMA ring, and alternates between two
// accumulators in tensor memory so that the epilogue of tile i (TMEM -> registers -> shared -> coalesced stores)
// overlaps the loads and MMAs of tile i+1.  Same roles and the same bounded waits as igemm_kernel.
constexpr int kStageLd = 16;  // words per staged epilogue row (16 columns, no padding needed for 128-bit accesses)

__global__ void __launch_bounds__(320, 1)
igemm_persistent_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bar_a_full[kMaxStages];
    __shared__ __align__(8) uint64_t bar_a_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_b_full;
    __shared__ __align__(8) uint64_t bar_acc_full[2];
    __shared__ __align__(8) uint64_t bar_acc_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t b_base = smem_base;                                   // kb_total x b_bytes, resident
    const uint32_t a_base = b_base + (uint32_t)p.kb_total * p.b_bytes;   // stages x 16 KiB ring
    const uint32_t st_off = (a_base - smem_u32(smem_raw)) + (uint32_t)p.stages * kABytes;  // epilogue staging
    const int n0 = blockIdx.y * p.n_tile;
    const int m_tiles = (p.M + kTileM - 1) / kTileM;
    const uint32_t acc_cols = p.tmem_cols >> 1;   // two accumulators side by side

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&bar_a_full[s]), 1);
            mbar_init(smem_u32(&bar_a_empty[s]), 1);
        }
        mbar_init(smem_u32(&bar_b_full), 1);
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&bar_acc_full[b]), 1);
            mbar_init(smem_u32(&bar_acc_empty[b]), 8);   // one arrival per epilogue warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)),
                     "r"(p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = s_tmem_base;
    volatile int *abort_flag = &s_abort;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_b) : "memory");
            const uint32_t bfull = smem_u32(&bar_b_full);
            mbar_expect_tx(bfull, (uint32_t)p.kb_total * p.b_bytes);
            for (int kb = 0; kb < p.kb_total; ++kb) {
                const uint32_t dst = b_base + kb * p.b_bytes;
                if (!p.b_mn) {
                    tma_load_2d(dst, &tm_b, bfull, kb * kBlockK, n0);
                } else {
                    for (int j = 0; j < p.b_boxes; ++j)
                        tma_load_2d(dst + j * kABytes, &tm_b, bfull, n0 + j * 128, kb * kBlockK);
                }
            }
            int it = 0;
            bool ok = true;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x) {
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const int s = it % p.stages;
                    const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_a_empty[s]), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t full = smem_u32(&bar_a_full[s]);
                    mbar_expect_tx(full, kABytes);
                    if (!p.a_mn) tma_load_2d(a_base + s * kABytes, &tm_a, full, kb * kBlockK, mt * kTileM);
                    else tma_load_2d(a_base + s * kABytes, &tm_a, full, mt * kTileM, kb * kBlockK);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)p.a_mn << 15) |
                                   ((uint32_t)p.b_mn << 16) | ((uint32_t)(p.n_tile >> 3) << 17) |
                                   ((uint32_t)(kTileM >> 4) << 24);
            const uint32_t a_kstep = p.a_mn ? 32u * 128u : 32u, b_kstep = p.b_mn ? 32u * 128u : 32u;
            const uint32_t a_lbo = p.a_mn ? (uint32_t)kABytes : 16u, b_lbo = p.b_mn ? (uint32_t)kABytes : 16u;
            bool ok = mbar_wait(smem_u32(&bar_b_full), 0u, abort_flag);
            int it = 0, t = 0;
            for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x, ++t) {
                const int buf = t & 1;
                const uint32_t acc_ph = (uint32_t)(t >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bar_acc_empty[buf]), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + buf * acc_cols;
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const int s = it % p.stages;
                    const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
                    if (!mbar_wait(smem_u32(&bar_a_full[s]), ph, abort_flag)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_src = a_base + s * kABytes, b_src = b_base + kb * p.b_bytes;
                    const int nk = min(4, (p.K - kb * kBlockK + 31) >> 5);
                    for (int k = 0; k < nk; ++k)
                        umma_i8(tmem_d, make_smem_desc(a_src + k * a_kstep, a_lbo, 1024u),
                                make_smem_desc(b_src + k * b_kstep, b_lbo, 1024u), idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(smem_u32(&bar_a_empty[s]));
                }
                if (ok) umma_commit(smem_u32(&bar_acc_full[buf]));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..9)
        // Eight warps drain an accumulator -- one warp runs a long dependent chain per chunk (TMEM load, convert,
        // stage, store), so four warps alone were the kernel's bottleneck.  Warp w reads TMEM lanes 32*(w%4).. and
        // every other 16-column chunk; the next chunk's tcgen05.ld is issued before the current chunk is processed.
        // Values go through a 32 x 16 word tile in shared memory (unpadded: 128-bit accesses of 8 lanes cover whole
        // 128-byte lines) so that four lanes write one row's 64 contiguous bytes.
        const int q = warp & 3, half = (warp - 2) >> 2;
        uint32_t *tile = reinterpret_cast<uint32_t *>(smem_raw + st_off) + (warp - 2) * 32 * kStageLd;
        const float sc = __fmul_rn(__ldg(p.sa), __ldg(p.sb));
        const bool vec_ok = (p.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
        const bool vec2_ok = (p.ldo & 1) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 7) == 0;
        const bool has_bias = p.bias != nullptr, want_max = p.absmax != nullptr;
        float amax = 0.f;
        int t = 0;
        bool ok = true;
        for (int mt = blockIdx.x; mt < m_tiles && ok; mt += gridDim.x, ++t) {
            const int buf = t & 1;
            const uint32_t acc_ph = (uint32_t)(t >> 1) & 1u;
            ok = mbar_wait(smem_u32(&bar_acc_full[buf]), acc_ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m0 = mt * kTileM;
            const int row = m0 + q * 32 + lane;
            const bool has_rs = p.out_row_scale != nullptr;
            const float rs_row = (has_rs && row < p.M) ? __ldg(p.out_row_scale + row) : 1.f;
            const uint32_t tbase = tmem_base + buf * acc_cols + ((uint32_t)(q * 32) << 16);
            uint32_t nxt[16];
            if (half * 16 < p.n_tile) tmem_ld16_nowait(tbase + (uint32_t)(half * 16), nxt);
            for (int c0 = half * 16; c0 < p.n_tile; c0 += 32) {
                const int col0 = n0 + c0;
                uint32_t r[16];
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) r[i] = nxt[i];
                if (c0 + 32 < p.n_tile) tmem_ld16_nowait(tbase + (uint32_t)(c0 + 32), nxt);   // overlaps the work below
                const bool full_cols = col0 + 16 <= p.N;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float v = __fmul_rn((float)(int)r[i], sc);
                    if (has_rs) v = __fmul_rn(v, rs_row);
                    if (has_bias && (full_cols || col0 + i < p.N)) v = __fadd_rn(v, __ldg(p.bias + col0 + i));
                    if (want_max && row < p.M && (full_cols || col0 + i < p.N)) amax = fmaxf(amax, fabsf(v));
                    r[i] = __float_as_uint(v);
                }
                if (p.tma_store) {
                    // The 32 x 16 fp32 box goes out as ONE bulk tensor store: lane = row writes its 64 bytes into the
                    // warp's tile in the 64-byte swizzle the tensor map expects (16-byte chunk c of row r sits at chunk
                    // c ^ ((r >> 1) & 3): conflict-free for a quarter warp), the writes are made visible to the async
                    // proxy, and lane 0 issues the store.  Rows >= M and columns >= N are clipped by the tensor map.
                    // The tile is rewritten only after the engine has read the previous box.
                    if (lane == 0) tma_store_wait_read();
                    __syncwarp();
                    const uint32_t row_addr = smem_u32(tile) + (uint32_t)lane * 64u;
                    const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)i ^ sw) << 4)),
                                     "r"(r[4 * i]), "r"(r[4 * i + 1]), "r"(r[4 * i + 2]), "r"(r[4 * i + 3])
                                     : "memory");
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tma_store_2d(&tm_out, smem_u32(tile), col0, m0 + q * 32);
                    continue;
                }
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    *reinterpret_cast<uint4 *>(tile + lane * kStageLd + 4 * i) =
                        make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
                __syncwarp();
                if (vec_ok) {
#pragma unroll
                    for (int itr = 0; itr < 4; ++itr) {      // 4 lanes x 16 B per row, 8 rows per step
                        const int rr = itr * 8 + (lane >> 2), cv = (lane & 3) * 4;
                        const int grow = m0 + q * 32 + rr, gcol = col0 + cv;
                        if (grow < p.M && gcol < p.N) {
                            const uint4 v4 = *reinterpret_cast<const uint4 *>(tile + rr * kStageLd + cv);
                            float *o = p.out + (int64_t)grow * p.ldo + gcol;
                            if (gcol + 4 <= p.N) {
                                *reinterpret_cast<uint4 *>(o) = v4;
                            } else {
                                const uint32_t e[4] = {v4.x, v4.y, v4.z, v4.w};
                                for (int i = 0; i < 4 && gcol + i < p.N; ++i) o[i] = __uint_as_float(e[i]);
                            }
                        }
                    }
                } else if (vec2_ok) {
#pragma unroll
                    for (int itr = 0; itr < 8; ++itr) {      // 8 lanes x 8 B per row, 4 rows per step
                        const int rr = itr * 4 + (lane >> 3), cv = (lane & 7) * 2;
                        const int grow = m0 + q * 32 + rr, gcol = col0 + cv;
                        if (grow < p.M && gcol < p.N) {
                            const uint2 v2 = *reinterpret_cast<const uint2 *>(tile + rr * kStageLd + cv);
                            float *o = p.out + (int64_t)grow * p.ldo + gcol;
                            if (gcol + 2 <= p.N) *reinterpret_cast<uint2 *>(o) = v2;
                            else o[0] = __uint_as_float(v2.x);
                        }
                    }
                } else {
                    for (int itr = 0; itr < 16; ++itr) {     // 16 lanes x 4 B per row, 2 rows per step
                        const int rr = itr * 2 + (lane >> 4), cv = lane & 15;
                        const int grow = m0 + q * 32 + rr, gcol = col0 + cv;
                        if (grow < p.M && gcol < p.N)
                            p.out[(int64_t)grow * p.ldo + gcol] = __uint_as_float(tile[rr * kStageLd + cv]);
                    }
                }
                __syncwarp();
            }
            // this warp has read its share of the accumulator: hand the buffer back to the MMA issuer
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0)
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_acc_empty[buf])) : "memory");
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();   // this lane's bulk stores, before shared memory goes away
        if (p.absmax) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.f) {
                const float s = __fdiv_rn(amax, 127.0f);
                if (s > __ldcg(p.absmax)) atomic_max_nonneg(p.absmax, s);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) __nanosleep(1000);
        if (threadIdx.x == 0 && p.status) atomicExch(p.status, TANGO_ETIMEOUT);
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(p.tmem_cols)
                     : "memory");
    }
}

__global__ void __launch_bounds__(256) dequant_ws_kernel(const int32_t *__restrict__ ws, int64_t ldws, int64_t rows,
                                                         int64_t cols, const float *__restrict__ sa,
                                                         const float *__restrict__ sb, float *__restrict__ out,
                                                         int64_t ldo) {
    const float sc = __fmul_rn(__ldg(sa), __ldg(sb));
    const int64_t total = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i - r * cols;
        out[r * ldo + c] = __fmul_rn((float)ws[r * ldws + c], sc);
    }
}

// ------------------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;  // benign race: every thread resolves the same pointer
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D uint8 tensor map over a row-major [outer, inner] byte matrix with leading dimension ld; 128-byte swizzle.
static int make_map(CUtensorMap *map, const void *base, int64_t inner, int64_t outer, int64_t ld, int box_inner,
                    int box_outer) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return TANGO_ECUDA;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return TANGO_ECUDA;
    }
    return TANGO_OK;
}

// 2-D fp32 tensor map over the row-major output [rows, cols] (leading dimension ld floats) for the epilogue's bulk
// stores: boxes of 32 rows x 16 columns, 64-byte swizzle.
static int make_out_map(CUtensorMap *map, const float *base, int64_t cols, int64_t rows, int64_t ld) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return TANGO_ECUDA;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(float)};
    cuuint32_t box[2] = {16, 32};
    cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return TANGO_ECUDA;
    }
    return TANGO_OK;
}

struct GemmCall {
    const int8_t *a; int64_t lda; int a_mn;
    const int8_t *b; int64_t ldb; int b_mn;
    int64_t M, N, K;
    int mode; int splits;
    float *out; int64_t ldo; int32_t *ws; int64_t ldws;
    const float *sa, *sb, *bias; float *absmax; int *status;
    const float *out_row_scale = nullptr;
};

static int launch_gemm(const GemmCall &c, cudaStream_t stream) {
    if (c.M <= 0 || c.N <= 0) return TANGO_OK;
    if (c.M > 0x7fffffff || c.N > 0x7fffffff || c.K > 0x7fffffff) return TANGO_ESIZE;
    if (!aligned(c.a, 16) || !aligned(c.b, 16) || c.lda % 16 || c.ldb % 16) return TANGO_EALIGN;
    GemmParams p{};
    p.M = (int)c.M; p.N = (int)c.N; p.K = (int)c.K;
    const int n_tiles = (int)ceil_div(c.N, 256);
    p.n_tile = (int)round_up(ceil_div(c.N, n_tiles), 16);
    p.kb_total = (int)ceil_div(c.K, kBlockK);
    int splits = c.splits < 1 ? 1 : c.splits;
    if (splits > p.kb_total) splits = p.kb_total > 0 ? p.kb_total : 1;
    p.kb_per_split = (int)ceil_div(p.kb_total, splits);
    splits = p.kb_per_split > 0 ? (int)ceil_div(p.kb_total, p.kb_per_split) : 1;
    p.a_mn = c.a_mn; p.b_mn = c.b_mn;
    p.b_boxes = c.b_mn ? (int)ceil_div(p.n_tile, 128) : 1;
    p.b_bytes = c.b_mn ? p.b_boxes * kABytes : (int)round_up((int64_t)p.n_tile * kBlockK, 1024);
    const int stage_bytes = kABytes + p.b_bytes;
    p.stages = 98304 / stage_bytes;
    if (p.stages < 2) p.stages = 2;
    if (p.stages > 6) p.stages = 6;
    p.mode = c.mode; p.out = c.out; p.ldo = c.ldo; p.ws = c.ws; p.ldws = c.ldws;
    p.sa = c.sa; p.sb = c.sb; p.bias = c.bias; p.absmax = c.absmax; p.status = c.status;
    p.out_row_scale = c.out_row_scale;
    p.tmem_cols = 32;
    while ((int)p.tmem_cols < p.n_tile) p.tmem_cols <<= 1;
    if (c.K <= 0) return TANGO_EINVAL;

    CUtensorMap tm_a, tm_b;
    int rc;
    // A: K-major [M rows, K bytes] box {128 k, 128 m};  MN-major [K rows, M bytes] box {128 m, 128 k}
    if (!c.a_mn) rc = make_map(&tm_a, c.a, c.K, c.M, c.lda, kBlockK, kTileM);
    else rc = make_map(&tm_a, c.a, c.M, c.K, c.lda, 128, kBlockK);
    if (rc) return rc;
    // B: K-major [N rows, K bytes] box {128 k, n_tile};  MN-major [K rows, N bytes] boxes {128 n, 128 k}
    if (!c.b_mn) rc = make_map(&tm_b, c.b, c.K, c.N, c.ldb, kBlockK, p.n_tile);
    else rc = make_map(&tm_b, c.b, c.N, c.K, c.ldb, 128, kBlockK);
    if (rc) return rc;

    // Persistent B-stationary kernel when one N-tile of B (all of K) fits in shared memory beside >= 3 A stages.
    if (c.mode == 0 && splits == 1) {
        const int64_t budget = 227 * 1024 - 2048;   // dynamic limit minus static barriers and alignment slack
        const int64_t b_res = (int64_t)p.kb_total * p.b_bytes;
        const int64_t staging = 8 * 32 * kStageLd * 4;
        int64_t st = (budget - 1024 - b_res - staging) / kABytes;
        if (st > kMaxStages) st = kMaxStages;
        if (st >= 3) {
            GemmParams pp = p;
            pp.stages = (int)st;
            uint32_t cols = 32;
            while ((int)cols < p.n_tile) cols <<= 1;
            pp.tmem_cols = cols * 2;
            CUtensorMap tm_out = tm_a;   // placeholder when the bulk-store path is off (never dereferenced then)
            pp.tma_store = (c.ldo % 4 == 0 && aligned(c.out, 16)) ? 1 : 0;
            if (pp.tma_store) {
                rc = make_out_map(&tm_out, c.out, c.N, c.M, c.ldo);
                if (rc) return rc;
            }
            const size_t smem_p = (size_t)(1024 + b_res + st * kABytes + staging);
            TANGO_CUDA_TRY(cudaFuncSetAttribute(igemm_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)(227 * 1024 - 1024)));
            const int64_t m_tiles = ceil_div(c.M, kTileM);
            int64_t gx = kNumSMs / n_tiles;
            if (gx < 1) gx = 1;
            if (gx > m_tiles) gx = m_tiles;
            const dim3 pgrid((unsigned)gx, (unsigned)n_tiles, 1);
            if (pgrid.y > 65535) return TANGO_ESIZE;
            igemm_persistent_kernel<<<pgrid, 320, smem_p, stream>>>(tm_a, tm_b, tm_out, pp);
            TANGO_LAUNCH_CHECK();
            return TANGO_OK;
        }
    }
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;
    // per-device attribute; setting it on every call keeps the entry point free of global state
    TANGO_CUDA_TRY(cudaFuncSetAttribute(igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const dim3 grid((unsigned)ceil_div(c.M, kTileM), (unsigned)n_tiles, (unsigned)splits);
    if (grid.y > 65535 || grid.z > 65535) return TANGO_ESIZE;
    igemm_kernel<<<grid, 192, smem, stream>>>(tm_a, tm_b, p);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

int igemm_accumulate_tiles_i32(const int8_t *tiles, int64_t n_tiles, const int32_t *units, int64_t n_units,
                               const int8_t *b, int64_t ldb, int64_t m, int64_t n, int64_t k, int32_t *ws,
                               int64_t ldws, int *status, cudaStream_t stream) {
    if (n_units <= 0 || n <= 0) return TANGO_OK;
    if (m <= 0 || k <= 0 || n_tiles <= 0 || m % kTileM || k % kBlockK) return TANGO_EINVAL;
    if (m > 0x7fffffff || k > 0x7fffffff || n_tiles * kTileM > 0x7fffffff || n_units > 0x7fffffff) return TANGO_ESIZE;
    if (!aligned(tiles, 16) || !aligned(b, 16) || ldb % 16 || !aligned(units, 16)) return TANGO_EALIGN;
    GemmParams p{};
    p.M = (int)m; p.N = (int)n; p.K = (int)k;
    const int n_tiles_n = (int)ceil_div(n, 256);
    p.n_tile = (int)round_up(ceil_div(n, n_tiles_n), 16);
    p.kb_total = (int)(k / kBlockK);
    p.kb_per_split = p.kb_total;
    p.a_mn = 0; p.b_mn = 1;
    p.b_boxes = (int)ceil_div(p.n_tile, 128);
    p.b_bytes = p.b_boxes * kABytes;
    const int stage_bytes = kABytes + p.b_bytes;
    // work items outnumber the SMs several times: two CTAs per SM when the ring still gets three stages each
    p.stages = 98304 / stage_bytes;
    if (p.stages < 3) p.stages = 196608 / stage_bytes;
    if (p.stages > 6) p.stages = 6;
    if (p.stages < 2) p.stages = 2;
    p.mode = 1; p.ws = ws; p.ldws = ldws; p.status = status;
    p.tile_units = reinterpret_cast<const int4 *>(units);
    p.tmem_cols = 32;
    while ((int)p.tmem_cols < p.n_tile) p.tmem_cols <<= 1;
    CUtensorMap tm_a, tm_b;
    int rc = make_map(&tm_a, tiles, kBlockK, n_tiles * kTileM, kBlockK, kBlockK, kTileM);   // one box = one stored tile
    if (rc) return rc;
    rc = make_map(&tm_b, b, n, k, ldb, 128, kBlockK);
    if (rc) return rc;
    const size_t smem = (size_t)p.stages * stage_bytes + 1024;
    TANGO_CUDA_TRY(cudaFuncSetAttribute(igemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    const dim3 grid((unsigned)n_units, (unsigned)n_tiles_n, 1);
    if (grid.y > 65535) return TANGO_ESIZE;
    igemm_kernel<<<grid, 192, smem, stream>>>(tm_a, tm_b, p);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

}  // namespace tango

using namespace tango;

extern "C" int64_t tango_qgemm_dw_workspace_bytes(int64_t n, int64_t k) {
    if (n < 0 || k < 0) return 0;
    if (n == 0 || k == 0) return 0;
    // n * round_up(k, 4) * 4 must fit in int64: saturate instead of wrapping around
    if (k > INT64_MAX - 3) return INT64_MAX;
    const int64_t ldws = round_up(k, 4);
    if (n > INT64_MAX / 4 / ldws) return INT64_MAX;
    return n * ldws * (int64_t)sizeof(int32_t);
}

extern "C" int tango_qgemm_nt(const int8_t *xq, int64_t ldx, const int8_t *wq, int64_t ldw, int64_t m, int64_t n,
                              int64_t k, const float *sx, const float *sw, const float *bias, float *y, int64_t ldy,
                              float *scale_y, int *status, tango_stream_t stream) {
    if (m < 0 || n < 0 || k <= 0 || ldx < k || ldw < k || ldy < n) return TANGO_EINVAL;
    if (m == 0 || n == 0) return TANGO_OK;
    if (!xq || !wq || !sx || !sw || !y) return TANGO_EINVAL;
    GemmCall c{xq, ldx, 0, wq, ldw, 0, m, n, k, 0, 1, y, ldy, nullptr, 0, sx, sw, bias, scale_y, status};
    return launch_gemm(c, (cudaStream_t)stream);
}

extern "C" int tango_qgemm_forward(const float *x, int64_t ldx_f, const float *row_scale, const float *w,
                                   int64_t ldw_f, int64_t m, int64_t n, int64_t k, const float *sx, const float *sw,
                                   int8_t *xq, int64_t ldxq, int8_t *wq, int64_t ldwq, const float *bias, float *y,
                                   int64_t ldy, float *scale_y, int mode, uint64_t seed, uint64_t call,
                                   const uint64_t *step, int *status, tango_stream_t stream) {
    int rc = tango_quantize(x, m, k, ldx_f, row_scale, sx, xq, ldxq, mode, seed, call, step, stream);
    if (rc) return rc;
    rc = tango_quantize(w, n, k, ldw_f, nullptr, sw, wq, ldwq, mode, seed, call + 1, step, stream);
    if (rc) return rc;
    return tango_qgemm_nt(xq, ldxq, wq, ldwq, m, n, k, sx, sw, bias, y, ldy, scale_y, status, stream);
}

extern "C" int tango_qgemm_dx(const int8_t *dyq, int64_t lddy, const int8_t *wq, int64_t ldw, int64_t m, int64_t n,
                              int64_t k, const float *sdy, const float *sw, const float *row_scale, float *dx,
                              int64_t lddx, int *status, tango_stream_t stream) {
    if (m < 0 || n <= 0 || k < 0 || lddy < n || ldw < k || lddx < k) return TANGO_EINVAL;
    if (m == 0 || k == 0) return TANGO_OK;
    if (!dyq || !wq || !sdy || !sw || !dx) return TANGO_EINVAL;
    // D[m, k] = A[m, n] . B[n, k]: reduction n; B is stored with the reduction index as its row
    GemmCall c{dyq, lddy, 0, wq, ldw, 1, m, k, n, 0, 1, dx, lddx, nullptr, 0, sdy, sw, nullptr, nullptr, status};
    c.out_row_scale = row_scale;
    return launch_gemm(c, (cudaStream_t)stream);
}

extern "C" int tango_qgemm_dw(const int8_t *dyq, int64_t lddy, const int8_t *xq, int64_t ldx, int64_t m, int64_t n,
                              int64_t k, const float *sdy, const float *sx, float *dw, int64_t lddw, void *workspace,
                              int64_t workspace_bytes, int *status, tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (m <= 0 || n < 0 || k < 0 || lddy < n || ldx < k || lddw < k) return TANGO_EINVAL;
    if (n == 0 || k == 0) return TANGO_OK;
    if (!dyq || !xq || !sdy || !sx || !dw || !workspace) return TANGO_EINVAL;
    if (workspace_bytes < tango_qgemm_dw_workspace_bytes(n, k)) return TANGO_ESIZE;
    if (!aligned(workspace, 16)) return TANGO_EALIGN;
    const int64_t ldws = round_up(k, 4);
    TANGO_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)(n * ldws) * sizeof(int32_t), stream));
    // D[n, k] = A[n, m] . B[m, k]^T-free form: both operands are stored with the reduction index m as their row
    const int64_t tiles = ceil_div(n, kTileM) * ceil_div(k, 256);
    int splits = (int)(kNumSMs / (tiles > 0 ? tiles : 1));
    if (splits < 1) splits = 1;
    GemmCall c{dyq, lddy, 1, xq, ldx, 1, n, k, m, 1, splits, nullptr, 0, (int32_t *)workspace, ldws,
               sdy, sx, nullptr, nullptr, status};
    int rc = launch_gemm(c, stream);
    if (rc) return rc;
    int64_t blocks = ceil_div(n * k, 256);
    if (blocks > kNumSMs * 8) blocks = kNumSMs * 8;
    dequant_ws_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const int32_t *)workspace, ldws, n, k, sdy, sx, dw, lddw);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

// ------------------------------------------------------------------------------------------------ no-allocation dW
// Scratch for tango_qgemm_dw_noalloc: a fixed array inside the library image instead of caller-provided memory.
// Every GPU that loads the library keeps these 4 MiB until the process exits.
namespace tango {
constexpr int64_t kStaticDwScratchElems = 1 << 20;  // int32 elements: n * round_up(k, 4) must not exceed this
static __device__ __align__(256) int32_t g_dw_scratch[kStaticDwScratchElems];

constexpr int kMaxDevices = 64;
static std::mutex g_dw_scratch_mutex;
static void *g_dw_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_dw_scratch on the current device.  In host code the array's name is only a handle, so the
// address is looked up once per device (with that device current) and cached.
static int dw_scratch_address(void **out) {
    int dev = -1;
    TANGO_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return TANGO_ESIZE;
    std::lock_guard<std::mutex> lock(g_dw_scratch_mutex);
    if (!g_dw_scratch_ptr[dev]) {
        void *p = nullptr;
        TANGO_CUDA_TRY(cudaGetSymbolAddress(&p, g_dw_scratch));
        if (!p) return TANGO_ECUDA;
        g_dw_scratch_ptr[dev] = p;
    }
    *out = g_dw_scratch_ptr[dev];
    return TANGO_OK;
}
}  // namespace tango

extern "C" int64_t tango_qgemm_dw_noalloc_max_elems(void) { return tango::kStaticDwScratchElems; }

extern "C" int tango_qgemm_dw_noalloc(const int8_t *dyq, int64_t lddy, const int8_t *xq, int64_t ldx, int64_t m,
                                      int64_t n, int64_t k, const float *sdy, const float *sx, float *dw,
                                      int64_t lddw, int *status, tango_stream_t stream) {
    if (n < 0 || k < 0) return TANGO_EINVAL;
    // compared in elements and by division, so that no product of caller-given sizes can wrap around
    if (k > tango::kStaticDwScratchElems) return TANGO_ESIZE;
    if (n > 0 && k > 0 && n > tango::kStaticDwScratchElems / round_up(k, 4)) return TANGO_ESIZE;
    void *scratch = nullptr;
    const int rc = tango::dw_scratch_address(&scratch);
    if (rc) return rc;
    // The regular entry point clears the part of the scratch it uses before accumulating into it.
    return tango_qgemm_dw(dyq, lddy, xq, ldx, m, n, k, sdy, sx, dw, lddw, scratch,
                          tango::kStaticDwScratchElems * (int64_t)sizeof(int32_t), status, stream);
}
