// CSR SpMM over int8 node (or edge) features with exact int32 accumulation.
//
// One warp owns one output row (or one "unit" = slice of a long row).  Within the warp, G lanes cover one
// neighbour's feature row with VEC-byte loads (G * VEC >= padded feature width) and 32/G neighbours are gathered per
// step.  Neighbour ids are fetched 32 at a time with one coalesced load (the next batch is prefetched) and handed out
// by shuffle; four gathers are in flight per lane (eight for narrow rows).  The same word of four neighbours is
// byte-transposed with PRMT and added with a 4-way dp4a against (1,1,1,1) (copy-u) or the four neighbours' int8
// weights (u_mul_e), so every accumulator is an exact int32.  Rows longer than the plan's threshold are cut into
// units that add into an int32 scratch row with integer atomics (order independent => deterministic) and a second
// kernel finishes them; rows of at most 48 neighbours are handled by lane groups (spmm_short_kernel); in-edge sums
// over contiguous edge rows have their own streaming kernel (incidence_contig_kernel).
#include "common.cuh"

namespace tango {

struct SpmmArgs {
    const int32_t *indptr;
    const int32_t *indices;   // feature-row id per slot; NULL => the slot number itself
    const int32_t *edge_ids;  // edge id per slot for the weight lookup; NULL => the slot number itself
    int64_t n_rows;
    int nseg;
    const int8_t *feat;
    int64_t ld;
    int f;      // logical feature bytes per row
    int f_pad;  // bytes the lanes may read (multiple of VEC, <= ld)
    const int8_t *ew;  // [E, H] int8 edge weights (weighted modes)
    int H, D;
    const float *scales;  // [nseg]
    const float *row_scale;
    const float *bias;
    int relu;
    float *out;
    int64_t ldo;
    float *out_absmax;
    const int32_t *units;
    int64_t n_units;
    const int32_t *heavy_rows;
    int64_t n_heavy;
    int32_t *ws;
    int64_t ws_ld;
    int split_threshold;
    const int32_t *row_order;
    int64_t n_long;   // rows row_order[0, n_long) go to the warp-per-row kernel, the rest to the lane-group kernel
    int G;  // lanes per neighbour (power of two)
};

enum { MODE_COPY = 0, MODE_WEIGHT_LANE = 1, MODE_WEIGHT_ELEM = 2 };

template <int VEC> struct VecLoad;
template <> struct VecLoad<16> {
    uint32_t w[4];
    __device__ __forceinline__ void load(const int8_t *p) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
    __device__ __forceinline__ void zero() { w[0] = w[1] = w[2] = w[3] = 0; }
};
template <> struct VecLoad<4> {
    uint32_t w[1];
    __device__ __forceinline__ void load(const int8_t *p) { w[0] = __ldg(reinterpret_cast<const uint32_t *>(p)); }
    __device__ __forceinline__ void zero() { w[0] = 0; }
};
template <> struct VecLoad<1> {
    uint32_t w[1];
    __device__ __forceinline__ void load(const int8_t *p) { w[0] = (uint32_t)(uint8_t)__ldg(p); }
    __device__ __forceinline__ void zero() { w[0] = 0; }
};

// Adds one byte of one neighbour (VEC == 1) or, for the per-element weight mode, VEC bytes with their own weights.
template <int VEC, int MODE>
__device__ __forceinline__ void accumulate_one(int (&acc)[VEC], const VecLoad<VEC> &v, uint32_t wsel,
                                               const int8_t *wrow, int off, const SpmmArgs &a) {
    if (VEC == 1) {
        const int b = (int)(int8_t)(v.w[0] & 0xff);
        if (MODE == MODE_COPY) acc[0] += b;
        else acc[0] += b * (int)(int8_t)wsel;
        return;
    }
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const uint32_t word = v.w[i >> 2];
        const int col = off + i;
        const int wv = (wrow && col < a.f) ? (int)__ldg(wrow + col / a.D) : 0;
        acc[i] += (int)(int8_t)((word >> (8 * (i & 3))) & 0xff) * wv;
    }
}

// Adds four neighbours at once.  The same word of the four rows is byte-transposed with 8 PRMTs so that each result
// word holds one feature of the four neighbours; one 4-way dp4a against (1,1,1,1) -- or against the four neighbours'
// int8 weights -- then adds all four into the int32 accumulator: 12 instructions per 16 gathered bytes.
template <int VEC>
__device__ __forceinline__ void accumulate_four(int (&acc)[VEC], const VecLoad<VEC> *v, uint32_t wvec) {
#pragma unroll
    for (int wp = 0; wp < VEC / 4; ++wp) {
        const uint32_t a = v[0].w[wp], b = v[1].w[wp], c = v[2].w[wp], d = v[3].w[wp];
        const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
        const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
        acc[4 * wp + 0] = __dp4a((int)__byte_perm(t0, t1, 0x5410), (int)wvec, acc[4 * wp + 0]);
        acc[4 * wp + 1] = __dp4a((int)__byte_perm(t0, t1, 0x7632), (int)wvec, acc[4 * wp + 1]);
        acc[4 * wp + 2] = __dp4a((int)__byte_perm(t2, t3, 0x5410), (int)wvec, acc[4 * wp + 2]);
        acc[4 * wp + 3] = __dp4a((int)__byte_perm(t2, t3, 0x7632), (int)wvec, acc[4 * wp + 3]);
    }
}

// Sums the neighbours of slots [beg, end) into acc for the feature bytes [off, off + VEC) handled by this lane.
// On return every lane of group 0 (lane < G) holds the full sum for its bytes.  Lanes whose bytes lie beyond the
// feature width run the same instruction stream on the row's first bytes (their sums are never stored), so the hot
// loop over full batches of 32 neighbours carries no predicates at all.
template <int VEC, int MODE, bool DEEP = false>
__device__ __forceinline__ void gather_segment(int (&acc)[VEC], int beg, int end, int off, bool active,
                                               const SpmmArgs &a) {
    const int lane = threadIdx.x & 31;
    const int G = a.G, NB = 32 / G, grp = lane / G;
    constexpr int U = 4;
    constexpr bool kFour = (VEC >= 4) && (MODE != MODE_WEIGHT_ELEM);
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0;
    const int ld_off = active ? off : 0;
    const int head = (MODE == MODE_WEIGHT_LANE) ? ld_off / a.D : 0;
    const int8_t *base = a.feat + ld_off;
    const int8_t *wbase = (MODE == MODE_WEIGHT_LANE) ? a.ew + head : a.ew;
    const uint32_t ld = (uint32_t)a.ld;   // 32 x 32 -> 64-bit products: one wide multiply per gathered row
    const int H = a.H;
    int j0 = beg;
    if (DEEP && kFour && G == 4) {
        // ---- narrow rows (four lanes per neighbour): a batch of 32 ids is only four gathers per lane, so two batches
        // are taken together to keep eight gathers in flight per lane.
        int nxt_a = 0, nxt_b = 0, nxt_ea = 0, nxt_eb = 0;
        if (j0 + 64 <= end) {
            nxt_a = a.indices ? __ldg(a.indices + j0 + lane) : j0 + lane;
            nxt_b = a.indices ? __ldg(a.indices + j0 + 32 + lane) : j0 + 32 + lane;
            if (MODE != MODE_COPY) {
                nxt_ea = a.edge_ids ? __ldg(a.edge_ids + j0 + lane) : j0 + lane;
                nxt_eb = a.edge_ids ? __ldg(a.edge_ids + j0 + 32 + lane) : j0 + 32 + lane;
            }
        }
        for (; j0 + 64 <= end; j0 += 64) {
            const int idx_a = nxt_a, idx_b = nxt_b, eid_a = nxt_ea, eid_b = nxt_eb;
            if (j0 + 128 <= end) {
                nxt_a = a.indices ? __ldg(a.indices + j0 + 64 + lane) : j0 + 64 + lane;
                nxt_b = a.indices ? __ldg(a.indices + j0 + 96 + lane) : j0 + 96 + lane;
                if (MODE != MODE_COPY) {
                    nxt_ea = a.edge_ids ? __ldg(a.edge_ids + j0 + 64 + lane) : j0 + 64 + lane;
                    nxt_eb = a.edge_ids ? __ldg(a.edge_ids + j0 + 96 + lane) : j0 + 96 + lane;
                }
            }
            VecLoad<VEC> v[8];
            uint32_t wv0 = 0x01010101u, wv1 = 0x01010101u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int src_lane = grp + (u & 3) * 8;
                const int idx = __shfl_sync(0xffffffffu, u < 4 ? idx_a : idx_b, src_lane);
                v[u].load(base + (uint64_t)(uint32_t)idx * ld);
                if (MODE == MODE_WEIGHT_LANE) {
                    const int eid = __shfl_sync(0xffffffffu, u < 4 ? eid_a : eid_b, src_lane);
                    const uint32_t wb = (uint32_t)(uint8_t)__ldg(wbase + (uint64_t)(uint32_t)eid * (uint32_t)H);
                    if (u < 4) wv0 = (u == 0) ? wb : (wv0 | (wb << (8 * u)));
                    else wv1 = (u == 4) ? wb : (wv1 | (wb << (8 * (u - 4))));
                }
            }
            accumulate_four<VEC>(acc, v, wv0);
            accumulate_four<VEC>(acc, v + 4, wv1);
        }
    }
    if (kFour && G >= U) {
        // ---- full batches: every shuffled index is valid, four loads in flight per lane, no predicates.
        // The indices of the next batch are fetched while the current one is processed.
        int nxt_idx = 0, nxt_eid = 0;
        if (j0 + 32 <= end) {
            nxt_idx = a.indices ? __ldg(a.indices + j0 + lane) : j0 + lane;
            if (MODE != MODE_COPY) nxt_eid = a.edge_ids ? __ldg(a.edge_ids + j0 + lane) : j0 + lane;
        }
        for (; j0 + 32 <= end; j0 += 32) {
            const int my_idx = nxt_idx, my_eid = nxt_eid;
            if (j0 + 64 <= end) {
                nxt_idx = a.indices ? __ldg(a.indices + j0 + 32 + lane) : j0 + 32 + lane;
                if (MODE != MODE_COPY) nxt_eid = a.edge_ids ? __ldg(a.edge_ids + j0 + 32 + lane) : j0 + 32 + lane;
            }
            for (int s = 0, lane0 = grp; s < G; s += U, lane0 += U * NB) {
                VecLoad<VEC> v[U];
                uint32_t wvec = 0x01010101u;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int src_lane = lane0 + u * NB;
                    const int idx = __shfl_sync(0xffffffffu, my_idx, src_lane);
                    v[u].load(base + (uint64_t)(uint32_t)idx * ld);
                    if (MODE == MODE_WEIGHT_LANE) {
                        const int eid = __shfl_sync(0xffffffffu, my_eid, src_lane);
                        const uint32_t wb = (uint32_t)(uint8_t)__ldg(wbase + (uint64_t)(uint32_t)eid * (uint32_t)H);
                        wvec = (u == 0) ? wb : (wvec | (wb << (8 * u)));
                    }
                }
                accumulate_four<VEC>(acc, v, wvec);
            }
        }
    }
    // ---- ragged tail (and every batch of the narrow or per-element-weight configurations): predicated
    for (; j0 < end; j0 += 32) {
        const int j = j0 + lane;
        int my_idx = -1, my_eid = 0;
        if (j < end) {
            my_idx = a.indices ? __ldg(a.indices + j) : j;
            if (MODE != MODE_COPY) my_eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        }
        const int steps = min(G, (end - j0 + NB - 1) / NB);
        for (int s = 0; s < steps; s += U) {
            VecLoad<VEC> v[U];
            uint32_t wsel[U];
            const int8_t *wrow[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int src_lane = ((s + u) * NB + grp) & 31;
                int idx = __shfl_sync(0xffffffffu, my_idx, src_lane);
                int eid = 0;
                if (MODE != MODE_COPY) eid = __shfl_sync(0xffffffffu, my_eid, src_lane);
                if (s + u >= steps) idx = -1;
                wsel[u] = 0; wrow[u] = nullptr;
                if (idx >= 0) {
                    v[u].load(base + (uint64_t)(uint32_t)idx * ld);
                    if (MODE == MODE_WEIGHT_LANE) wsel[u] = (uint32_t)(uint8_t)__ldg(wbase + (uint64_t)(uint32_t)eid * (uint32_t)H);
                    if (MODE == MODE_WEIGHT_ELEM) wrow[u] = a.ew + (uint64_t)(uint32_t)eid * (uint32_t)H;
                } else {
                    v[u].zero();
                }
            }
            if (kFour) {
                uint32_t wvec = 0x01010101u;
                if (MODE == MODE_WEIGHT_LANE) wvec = wsel[0] | (wsel[1] << 8) | (wsel[2] << 16) | (wsel[3] << 24);
                accumulate_four<VEC>(acc, v, wvec);
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) accumulate_one<VEC, MODE>(acc, v[u], wsel[u], wrow[u], ld_off, a);
            }
        }
    }
    for (int o = G; o < 32; o <<= 1) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
}

__device__ __forceinline__ float finish_value(float v, int64_t row, int col, const SpmmArgs &a) {
    if (a.row_scale) v = __fmul_rn(v, __ldg(a.row_scale + row));
    if (a.bias) v = __fadd_rn(v, __ldg(a.bias + col));
    if (a.relu) v = fmaxf(v, 0.f);
    return v;
}

constexpr int kSpmmThreads = 128;   // four warps (four rows or slices) per CTA

template <int VEC, int MODE, bool DEEP = false>
__global__ void __launch_bounds__(kSpmmThreads, DEEP ? 6 : 8) spmm_kernel(const SpmmArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int sub = lane % a.G;
    float amax = 0.f;
    if (w < a.n_units) {
        // ---- one slice of a long row: integer partial sums into scratch
        const int4 u = __ldg(reinterpret_cast<const int4 *>(a.units) + w);  // (vrow, beg, end, slot)
        for (int fb = 0; fb < a.f_pad; fb += 32 * VEC) {
            const int off = fb + sub * VEC;
            const bool active = off < a.f_pad;
            int acc[VEC];
            gather_segment<VEC, MODE, DEEP>(acc, u.y, u.z, off, active, a);
            if (active && lane < a.G) {
#pragma unroll
                for (int i = 0; i < VEC; ++i)
                    if (off + i < a.f && acc[i] != 0) atomicAdd(a.ws + (int64_t)u.w * a.ws_ld + off + i, acc[i]);
            }
        }
    } else if (w - a.n_units < a.n_long) {
        int64_t row = w - a.n_units;
        if (a.row_order) row = __ldg(a.row_order + row);
        const int32_t *ip = a.indptr + row * a.nseg;
        const int row_beg = __ldg(ip), row_end = __ldg(ip + a.nseg);
        if (a.n_heavy > 0 && row_end - row_beg > a.split_threshold) return;  // finished by spmm_finalize_kernel
        for (int fb = 0; fb < a.f_pad; fb += 32 * VEC) {
            const int off = fb + sub * VEC;
            const bool active = off < a.f_pad;
            float facc[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = 0.f;
            for (int k = 0; k < a.nseg; ++k) {
                int acc[VEC];
                gather_segment<VEC, MODE, DEEP>(acc, __ldg(ip + k), __ldg(ip + k + 1), off, active, a);
                const float sc = __ldg(a.scales + k);
#pragma unroll
                for (int i = 0; i < VEC; ++i) facc[i] = __fadd_rn(facc[i], __fmul_rn((float)acc[i], sc));
            }
            if (active && lane < a.G) {
                float *o = a.out + row * a.ldo + off;
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    facc[i] = finish_value(facc[i], row, min(off + i, a.f - 1), a);
                    if (off + i < a.f) amax = fmaxf(amax, fabsf(facc[i]));
                }
                if (VEC == 16 && off + 16 <= a.f && (a.ldo & 3) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        reinterpret_cast<float4 *>(o)[i] =
                            make_float4(facc[4 * i], facc[4 * i + 1], facc[4 * i + 2], facc[4 * i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < VEC; ++i)
                        if (off + i < a.f) o[i] = facc[i];
                }
            }
        }
    }
    if (a.out_absmax) {
        amax = warp_max(amax);
        if (lane == 0 && amax > 0.f) {
            const float s = __fdiv_rn(amax, 127.0f);
            if (s > __ldcg(a.out_absmax)) atomic_max_nonneg(a.out_absmax, s);
        }
    }
}

// Short rows: a group of G lanes owns one row (32 / G rows per warp) and needs no cross-lane reduction -- the
// warp-per-row kernel would spend most of its time in the ragged tail on rows with a handful of neighbours.  Such a
// row is a short dependent chain (row bounds -> neighbour ids -> gathers -> store), so what matters is how few round
// trips it takes and how many rows are in flight: with four or more lanes per row the group fetches G neighbour ids
// (and edge ids) with ONE coalesced load and hands them out by shuffles restricted to the group, so an 8-neighbour
// row costs one index round trip and two gather round trips; narrower groups read the ids one by one.
// MULTI: rows cut into per-shard segments with a scale each (row-partitioned multi-GPU aggregation).
template <int VEC, int MODE, bool MULTI>
__global__ void __launch_bounds__(128, MULTI ? 8 : 10) spmm_short_kernel(const SpmmArgs a) {
    const int lane = threadIdx.x & 31;
    const int G = a.G, sub = lane % G;
    const int64_t gid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int64_t n_short = a.n_rows - a.n_long;
    const int off = sub * VEC;
    const bool in_range = gid < n_short;
    const bool active = in_range && off < a.f_pad;
    const unsigned gmask = (G >= 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane - sub));
    const int base_lane = lane - sub;
    float amax = 0.f;
    int64_t row = 0;
    const int32_t *ip = a.indptr;
    if (in_range) {
        row = a.row_order ? (int64_t)__ldg(a.row_order + a.n_long + gid) : a.n_long + gid;
        ip = a.indptr + row * a.nseg;
    }
    const int8_t *base = a.feat + (active ? off : 0);
    const int head = (MODE == MODE_WEIGHT_LANE) ? (active ? off : 0) / a.D : 0;
    float facc[VEC];
    if (MULTI) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) facc[i] = 0.f;
    }
    const int nseg = in_range ? (MULTI ? a.nseg : 1) : 0;
    int acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0;
    for (int k = 0; k < nseg; ++k) {
        const int beg = __ldg(ip + k), end = __ldg(ip + k + 1);
        if (MULTI) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = 0;
        }
        if (G >= 4) {
            for (int j0 = beg; j0 < end; j0 += G) {
                const int j = j0 + sub;
                int my_idx = 0, my_eid = 0;
                if (j < end) {
                    my_idx = a.indices ? __ldg(a.indices + j) : j;
                    if (MODE == MODE_WEIGHT_LANE) my_eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
                }
                const int cnt = min(G, end - j0);
                for (int s0 = 0; s0 < cnt; s0 += 4) {
                    VecLoad<VEC> v[4];
                    uint32_t wvec = (MODE == MODE_WEIGHT_LANE) ? 0u : 0x01010101u;
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int idx = __shfl_sync(gmask, my_idx, base_lane + ((s0 + u) & (G - 1)));
                        int eid = 0;
                        if (MODE == MODE_WEIGHT_LANE) eid = __shfl_sync(gmask, my_eid, base_lane + ((s0 + u) & (G - 1)));
                        if (s0 + u < cnt) {
                            v[u].load(base + (uint64_t)(uint32_t)idx * (uint32_t)a.ld);
                            if (MODE == MODE_WEIGHT_LANE)
                                wvec |= (uint32_t)(uint8_t)__ldg(a.ew + (uint64_t)(uint32_t)eid * (uint32_t)a.H + head) << (8 * u);
                        } else {
                            v[u].zero();
                        }
                    }
                    accumulate_four<VEC>(acc, v, wvec);
                }
            }
        } else {
            for (int j = beg; j < end; j += 4) {
                VecLoad<VEC> v[4];
                uint32_t wvec = (MODE == MODE_WEIGHT_LANE) ? 0u : 0x01010101u;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (j + u < end) {
                        const int idx = a.indices ? __ldg(a.indices + j + u) : j + u;
                        v[u].load(base + (uint64_t)(uint32_t)idx * (uint32_t)a.ld);
                        if (MODE == MODE_WEIGHT_LANE) {
                            const int eid = a.edge_ids ? __ldg(a.edge_ids + j + u) : j + u;
                            wvec |= (uint32_t)(uint8_t)__ldg(a.ew + (uint64_t)(uint32_t)eid * (uint32_t)a.H + head) << (8 * u);
                        }
                    } else {
                        v[u].zero();
                    }
                }
                accumulate_four<VEC>(acc, v, wvec);
            }
        }
        if (MULTI) {
            const float sc = __ldg(a.scales + k);
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = __fadd_rn(facc[i], __fmul_rn((float)acc[i], sc));
        }
    }
    if (active) {
        float *o = a.out + row * a.ldo + off;
        if (!MULTI) {
            // one segment: 0 + acc * scale, the same two roundings as the segmented form
            const float sc = __ldg(a.scales);
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = __fadd_rn(0.f, __fmul_rn((float)acc[i], sc));
        }
        // short rows are as much epilogue as gather: the optional per-element steps are decided once, not per element
        if (a.row_scale) {
            const float rs = __ldg(a.row_scale + row);
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = __fmul_rn(facc[i], rs);
        }
        if (a.bias) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = __fadd_rn(facc[i], __ldg(a.bias + min(off + i, a.f - 1)));
        }
        if (a.relu) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) facc[i] = fmaxf(facc[i], 0.f);
        }
        if (a.out_absmax) {
#pragma unroll
            for (int i = 0; i < VEC; ++i)
                if (off + i < a.f) amax = fmaxf(amax, fabsf(facc[i]));
        }
        if (VEC == 16 && off + 16 <= a.f && (a.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                __stcs(reinterpret_cast<float4 *>(o) + i, make_float4(facc[4 * i], facc[4 * i + 1], facc[4 * i + 2], facc[4 * i + 3]));
        } else {
#pragma unroll
            for (int i = 0; i < VEC; ++i)
                if (off + i < a.f) o[i] = facc[i];
        }
    }
    if (a.out_absmax) {
        amax = warp_max(amax);
        if (lane == 0 && amax > 0.f) {
            const float s = __fdiv_rn(amax, 127.0f);
            if (s > __ldcg(a.out_absmax)) atomic_max_nonneg(a.out_absmax, s);
        }
    }
}

// ---- incidence sums over contiguous edge rows: when slot j of a row IS edge j (edge ids follow the row order) and
// the edge features are packed [E, F] with F dividing 16, the edges of a row are one contiguous byte range.  It is
// streamed with aligned 128-bit loads, four in flight per lane; byte b of an aligned chunk belongs to column b % F.
template <int F>
__device__ __forceinline__ void add_chunk(int (&acc)[F], const uint4 &w) {
    if (F == 1) {
        acc[0] = __dp4a((int)w.x, 0x01010101, acc[0]); acc[0] = __dp4a((int)w.y, 0x01010101, acc[0]);
        acc[0] = __dp4a((int)w.z, 0x01010101, acc[0]); acc[0] = __dp4a((int)w.w, 0x01010101, acc[0]);
    } else if (F == 4) {
        const uint32_t t0 = __byte_perm(w.x, w.y, 0x5140), t1 = __byte_perm(w.z, w.w, 0x5140);
        const uint32_t t2 = __byte_perm(w.x, w.y, 0x7362), t3 = __byte_perm(w.z, w.w, 0x7362);
        acc[0 % F] = __dp4a((int)__byte_perm(t0, t1, 0x5410), 0x01010101, acc[0 % F]);
        acc[1 % F] = __dp4a((int)__byte_perm(t0, t1, 0x7632), 0x01010101, acc[1 % F]);
        acc[2 % F] = __dp4a((int)__byte_perm(t2, t3, 0x5410), 0x01010101, acc[2 % F]);
        acc[3 % F] = __dp4a((int)__byte_perm(t2, t3, 0x7632), 0x01010101, acc[3 % F]);
    } else {
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i % F] += (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
    }
}

template <int F>
__device__ __forceinline__ void contig_segment(int (&acc)[F], int beg, int end, const SpmmArgs &a) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int c = 0; c < F; ++c) acc[c] = 0;
    const int64_t b0 = (int64_t)beg * F, b1 = (int64_t)end * F;
    const int64_t a0 = min(b1, (b0 + 15) & ~(int64_t)15), a1 = max(a0, b1 & ~(int64_t)15);
    // ragged head [b0, a0) and tail [a1, b1): fewer than 16 bytes each; both start on a multiple of F
    const int nh = (int)(a0 - b0), nt = (int)(b1 - a1);
    if (lane < nh || lane < nt) {
        const int vh = lane < nh ? (int)__ldg(a.feat + b0 + lane) : 0;
        const int vt = lane < nt ? (int)__ldg(a.feat + a1 + lane) : 0;
#pragma unroll
        for (int c = 0; c < F; ++c)
            if (lane % F == c) acc[c] += vh + vt;
    }
    const uint4 *chunks = reinterpret_cast<const uint4 *>(a.feat);
    const int64_t c1 = a1 >> 4;
    for (int64_t c = (a0 >> 4) + lane; c < c1; c += 128) {
        uint4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) w[u] = (c + 32 * u < c1) ? __ldcs(chunks + c + 32 * u) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; ++u) add_chunk<F>(acc, w[u]);
    }
#pragma unroll
    for (int c = 0; c < F; ++c)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], o);
}

template <int F>
__global__ void __launch_bounds__(128) incidence_contig_kernel(const SpmmArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int acc[F];
    if (w < a.n_units) {
        const int4 u = __ldg(reinterpret_cast<const int4 *>(a.units) + w);
        contig_segment<F>(acc, u.y, u.z, a);
#pragma unroll
        for (int c = 0; c < F; ++c)
            if (lane == c && acc[c] != 0) atomicAdd(a.ws + (int64_t)u.w * a.ws_ld + c, acc[c]);
    } else if (w - a.n_units < a.n_long) {
        int64_t row = w - a.n_units;
        if (a.row_order) row = __ldg(a.row_order + row);
        const int beg = __ldg(a.indptr + row), end = __ldg(a.indptr + row + 1);
        if (a.n_heavy > 0 && end - beg > a.split_threshold) return;   // finished by spmm_finalize_kernel
        contig_segment<F>(acc, beg, end, a);
        const float sc = __ldg(a.scales);
#pragma unroll
        for (int c = 0; c < F; ++c)
            if (lane == c) a.out[row * a.ldo + c] = __fadd_rn(0.f, __fmul_rn((float)acc[c], sc));
    }
}

// Finishes the rows that went through the int32 scratch (rows cut into units, rows of the dense hub region): one
// thread per (heavy row, four features) -- 128-bit scratch loads and output stores when the row pitch allows.
__global__ void __launch_bounds__(256) spmm_finalize_kernel(const SpmmArgs a) {
    const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int f4 = (a.f + 3) >> 2;
    float amax = 0.f;
    if (t < a.n_heavy * f4) {
        const int64_t hs = t / f4;
        const int col0 = (int)(t - hs * f4) << 2;
        const int64_t row = __ldg(a.heavy_rows + hs);
        float facc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int k = 0; k < a.nseg; ++k) {
            const int32_t *w = a.ws + (hs * a.nseg + k) * a.ws_ld + col0;
            const int4 v = *reinterpret_cast<const int4 *>(w);       // ws_ld is a multiple of 16: always in bounds
            const float sc = __ldg(a.scales + k);
            facc[0] = __fadd_rn(facc[0], __fmul_rn((float)v.x, sc));
            facc[1] = __fadd_rn(facc[1], __fmul_rn((float)v.y, sc));
            facc[2] = __fadd_rn(facc[2], __fmul_rn((float)v.z, sc));
            facc[3] = __fadd_rn(facc[3], __fmul_rn((float)v.w, sc));
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            facc[i] = finish_value(facc[i], row, min(col0 + i, a.f - 1), a);
            if (col0 + i < a.f) amax = fmaxf(amax, fabsf(facc[i]));
        }
        float *o = a.out + row * a.ldo + col0;
        if (col0 + 4 <= a.f && (a.ldo & 3) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
            *reinterpret_cast<float4 *>(o) = make_float4(facc[0], facc[1], facc[2], facc[3]);
        } else {
            for (int i = 0; i < 4 && col0 + i < a.f; ++i) o[i] = facc[i];
        }
    }
    if (a.out_absmax) {
        amax = warp_max(amax);
        if ((threadIdx.x & 31) == 0 && amax > 0.f) {
            const float s = __fdiv_rn(amax, 127.0f);
            if (s > __ldcg(a.out_absmax)) atomic_max_nonneg(a.out_absmax, s);
        }
    }
}

// Packs the feature rows ids[0..n) of `src` ([*, ld] int8, ld a multiple of 16) into dst [n, ld]: the B operand of
// the dense hub block.
__global__ void __launch_bounds__(256) gather_rows_kernel(const int8_t *__restrict__ src, int64_t ld,
                                                          const int32_t *__restrict__ ids, int64_t n,
                                                          int8_t *__restrict__ dst) {
    const int64_t pieces = ld >> 4, total = n * pieces;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / pieces, c = i - r * pieces;
        reinterpret_cast<uint4 *>(dst + r * ld)[c] =
            __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)__ldg(ids + r) * ld) + c);
    }
}

static int pow2_ceil(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

template <int MODE>
static int launch_spmm(SpmmArgs &a, const tango_spmm_plan *plan, cudaStream_t stream) {
    if (a.n_rows == 0 || a.f == 0) return TANGO_OK;
    if (a.ld > 0x7fffffff) return TANGO_ESIZE;
    a.n_long = a.n_rows;
    if (plan) a.row_order = plan->row_order;
    if (plan && plan->n_units > 0) {
        if (!plan->units || !plan->heavy_rows || !plan->ws || plan->ws_ld < a.f || plan->n_heavy <= 0)
            return TANGO_EINVAL;
        if (!aligned(plan->units, 16) || !aligned(plan->ws, 16) || plan->ws_ld % 4) return TANGO_EALIGN;
        a.units = plan->units; a.n_units = plan->n_units; a.heavy_rows = plan->heavy_rows;
        a.n_heavy = plan->n_heavy; a.ws = plan->ws; a.ws_ld = plan->ws_ld; a.split_threshold = plan->split_threshold;
        TANGO_CUDA_TRY(cudaMemsetAsync(a.ws, 0, sizeof(int32_t) * (size_t)(a.n_heavy * a.nseg * a.ws_ld), stream));
    }
    const bool dense = plan && plan->dense_a && plan->dense_rows > 0 && plan->dense_n_cols > 0 && plan->dense_n_units > 0;
    if (dense) {
        // dense hub block: pack the block's feature rows, multiply on the tensor cores, add into the heavy rows'
        // int32 scratch (cleared above); the gather kernels below then cover only the edges outside the block
        if (MODE != MODE_COPY || a.nseg != 1 || plan->n_units < 0 || !plan->heavy_rows || !plan->ws ||
            plan->dense_rows > plan->n_heavy || !plan->dense_cols || !plan->dense_b || !plan->dense_units ||
            plan->dense_n_tiles <= 0 || plan->dense_rows % 128 || plan->dense_n_cols % 128 ||
            plan->n_skip_rows != plan->n_heavy || !plan->row_order || plan->ws_ld < a.f)
            return TANGO_EINVAL;
        if (a.ld % 16 || !aligned(a.feat, 16) || !aligned(plan->dense_a, 16) || !aligned(plan->dense_b, 16) ||
            !aligned(plan->dense_units, 16) || !aligned(plan->ws, 16) || plan->ws_ld % 4)
            return TANGO_EALIGN;
        if (plan->n_units == 0) {      // no unit set the scratch fields above
            a.heavy_rows = plan->heavy_rows; a.n_heavy = plan->n_heavy; a.ws = plan->ws; a.ws_ld = plan->ws_ld;
            a.split_threshold = plan->split_threshold;
            TANGO_CUDA_TRY(cudaMemsetAsync(a.ws, 0, sizeof(int32_t) * (size_t)(a.n_heavy * a.ws_ld), stream));
        }
        const int64_t ldb = round_up(a.f, 16);
        if (ldb > a.ld) return TANGO_EINVAL;
        {
            const int64_t pieces = plan->dense_n_cols * (ldb >> 4);
            int64_t gb = ceil_div(pieces, 256);
            if (gb > kNumSMs * 8) gb = kNumSMs * 8;
            if (ldb == a.ld) {
                gather_rows_kernel<<<(unsigned)gb, 256, 0, stream>>>(a.feat, a.ld, plan->dense_cols, plan->dense_n_cols,
                                                                    plan->dense_b);
            } else {
                return TANGO_EINVAL;   // feature rows wider than their padded width: not a layout the quantizers make
            }
            TANGO_LAUNCH_CHECK();
        }
        const int rc = igemm_accumulate_tiles_i32(plan->dense_a, plan->dense_n_tiles, plan->dense_units,
                                                  plan->dense_n_units, plan->dense_b, ldb, plan->dense_rows, a.f,
                                                  plan->dense_n_cols, a.ws, a.ws_ld, plan->dense_status, stream);
        if (rc) return rc;
    }
    if (plan && plan->n_skip_rows > 0) {
        // the leading rows of row_order belong to units + finalize: the row kernels start after them
        if (!plan->row_order || plan->n_skip_rows > a.n_rows || plan->n_long_rows < plan->n_skip_rows) return TANGO_EINVAL;
        a.row_order = plan->row_order + plan->n_skip_rows;
        a.n_rows -= plan->n_skip_rows;
    }
    if (MODE == MODE_WEIGHT_LANE && a.H == 1) a.D = 1 << 20;  // one head: every byte shares the weight
    int vec = 1;
    if (a.ld % 16 == 0 && aligned(a.feat, 16)) vec = 16;
    else if (a.ld % 4 == 0 && aligned(a.feat, 4)) vec = 4;
    // narrow rows: prefer one lane per neighbour over mostly idle 16-byte lanes
    if (vec == 16 && a.f <= 4) vec = 4;
    a.f_pad = (int)round_up(a.f, vec);
    if (a.f_pad > a.ld) return TANGO_EINVAL;
    a.G = pow2_ceil((a.f_pad + vec - 1) / vec);
    if (a.G > 32) a.G = 32;
    if (MODE == MODE_WEIGHT_LANE && (a.D % vec) != 0) {
        // a lane's bytes must stay inside one head; fall back to narrower loads, else to the per-element mode
        if (vec == 16 && a.D % 4 == 0 && a.ld % 4 == 0) {
            vec = 4; a.f_pad = (int)round_up(a.f, 4); a.G = pow2_ceil(a.f_pad / 4); if (a.G > 32) a.G = 32;
        }
    }
    // short rows (the tail of the degree-sorted order) go to the lane-group kernel when one pass of G lanes covers a row
    const bool four = vec >= 4 && !(MODE == MODE_WEIGHT_LANE && (a.D % vec) != 0);
    const int64_t n_skip = plan ? plan->n_skip_rows : 0;
    if (plan && plan->row_order && plan->n_long_rows >= n_skip && plan->n_long_rows - n_skip <= a.n_rows && four &&
        a.f_pad <= 32 * vec)
        a.n_long = plan->n_long_rows - n_skip;
    else if (n_skip > 0) a.n_long = a.n_rows;
    const int64_t warps = a.n_units + a.n_long;
    const int64_t blocks = ceil_div(warps, kSpmmThreads / 32);
    if (blocks > 0x7fffffff) return TANGO_ESIZE;
#define TANGO_SPMM_LAUNCH(V, M)                                                                  \
    do {                                                                                         \
        if (blocks > 0) spmm_kernel<V, M><<<(unsigned)blocks, kSpmmThreads, 0, stream>>>(a);     \
    } while (0)
    if (MODE == MODE_WEIGHT_LANE && (a.D % vec) != 0) {
        if (vec == 16) TANGO_SPMM_LAUNCH(16, MODE_WEIGHT_ELEM);
        else if (vec == 4) TANGO_SPMM_LAUNCH(4, MODE_WEIGHT_ELEM);
        else TANGO_SPMM_LAUNCH(1, MODE_WEIGHT_LANE);  // VEC == 1: a lane holds one byte, always inside one head
    } else {
        if (vec == 16 && a.G == 4) {
            if (blocks > 0) spmm_kernel<16, MODE, true><<<(unsigned)blocks, kSpmmThreads, 0, stream>>>(a);
        } else if (vec == 16) TANGO_SPMM_LAUNCH(16, MODE);
        else if (vec == 4) TANGO_SPMM_LAUNCH(4, MODE);
        else TANGO_SPMM_LAUNCH(1, MODE);
    }
#undef TANGO_SPMM_LAUNCH
    TANGO_LAUNCH_CHECK();
    if (a.n_long < a.n_rows) {
        const int64_t threads = (a.n_rows - a.n_long) * a.G;
        const int64_t sb = ceil_div(threads, 128);
        if (sb > 0x7fffffff) return TANGO_ESIZE;
        if (a.nseg > 1) {
            if (vec == 16) spmm_short_kernel<16, MODE, true><<<(unsigned)sb, 128, 0, stream>>>(a);
            else spmm_short_kernel<4, MODE, true><<<(unsigned)sb, 128, 0, stream>>>(a);
        } else {
            if (vec == 16) spmm_short_kernel<16, MODE, false><<<(unsigned)sb, 128, 0, stream>>>(a);
            else spmm_short_kernel<4, MODE, false><<<(unsigned)sb, 128, 0, stream>>>(a);
        }
        TANGO_LAUNCH_CHECK();
    }
    if (a.n_units > 0 || dense) {
        const int64_t fb = ceil_div(a.n_heavy * ((a.f + 3) / 4), 256);
        spmm_finalize_kernel<<<(unsigned)fb, 256, 0, stream>>>(a);
        TANGO_LAUNCH_CHECK();
    }
    return TANGO_OK;
}

// Contiguous incidence sums (see incidence_contig_kernel); returns false when the layout does not qualify.
static bool try_incidence_contig(SpmmArgs &a, const tango_spmm_plan *plan, cudaStream_t stream, int &rc) {
    const int f = a.f;
    if (a.indices || a.ld != f || !(f == 1 || f == 2 || f == 4 || f == 8 || f == 16) || !aligned(a.feat, 16)) return false;
    rc = TANGO_OK;
    a.n_long = a.n_rows;
    if (plan) a.row_order = plan->row_order;
    // rows with a handful of edges (the tail of the degree-sorted order) are cheaper with one lane group per row than
    // with a whole warp and its cross-lane reduction: they go to spmm_short_kernel, which needs 4- or 16-byte pieces
    const int short_vec = (f == 16) ? 16 : (f == 4 || f == 8) ? 4 : 0;
    if (short_vec && plan && plan->row_order && plan->n_long_rows >= 0 && plan->n_long_rows <= a.n_rows) {
        a.n_long = plan->n_long_rows;
        a.f_pad = f;
        a.G = f / short_vec;          // 1 or 2 lanes per row
    }
    if (plan && plan->n_units > 0) {
        if (!plan->units || !plan->heavy_rows || !plan->ws || plan->ws_ld < f || plan->n_heavy <= 0 ||
            !aligned(plan->units, 16)) { rc = TANGO_EINVAL; return true; }
        if (!aligned(plan->ws, 16) || plan->ws_ld % 4) { rc = TANGO_EALIGN; return true; }
        a.units = plan->units; a.n_units = plan->n_units; a.heavy_rows = plan->heavy_rows;
        a.n_heavy = plan->n_heavy; a.ws = plan->ws; a.ws_ld = plan->ws_ld; a.split_threshold = plan->split_threshold;
        if (cudaMemsetAsync(a.ws, 0, sizeof(int32_t) * (size_t)(a.n_heavy * a.ws_ld), stream) != cudaSuccess) {
            rc = TANGO_ECUDA; return true;
        }
    }
    const int64_t blocks = ceil_div(a.n_units + a.n_long, 4);
    if (blocks > 0x7fffffff) { rc = TANGO_ESIZE; return true; }
    if (blocks > 0) {
        switch (f) {
            case 1: incidence_contig_kernel<1><<<(unsigned)blocks, 128, 0, stream>>>(a); break;
            case 2: incidence_contig_kernel<2><<<(unsigned)blocks, 128, 0, stream>>>(a); break;
            case 4: incidence_contig_kernel<4><<<(unsigned)blocks, 128, 0, stream>>>(a); break;
            case 8: incidence_contig_kernel<8><<<(unsigned)blocks, 128, 0, stream>>>(a); break;
            default: incidence_contig_kernel<16><<<(unsigned)blocks, 128, 0, stream>>>(a); break;
        }
        if (cudaPeekAtLastError() != cudaSuccess) { rc = TANGO_ECUDA; return true; }
    }
    if (a.n_long < a.n_rows) {
        const int64_t sb = ceil_div((a.n_rows - a.n_long) * a.G, 128);
        if (sb > 0x7fffffff) { rc = TANGO_ESIZE; return true; }
        if (short_vec == 16) spmm_short_kernel<16, MODE_COPY, false><<<(unsigned)sb, 128, 0, stream>>>(a);
        else spmm_short_kernel<4, MODE_COPY, false><<<(unsigned)sb, 128, 0, stream>>>(a);
        if (cudaPeekAtLastError() != cudaSuccess) { rc = TANGO_ECUDA; return true; }
    }
    if (a.n_units > 0) {
        const int64_t fb = ceil_div(a.n_heavy * ((a.f + 3) / 4), 256);
        spmm_finalize_kernel<<<(unsigned)fb, 256, 0, stream>>>(a);
        if (cudaPeekAtLastError() != cudaSuccess) rc = TANGO_ECUDA;
    }
    return true;
}

}  // namespace tango

using namespace tango;

extern "C" int tango_spmm_copy_u(const int32_t *indptr, const int32_t *indices, int64_t n_rows, int nseg,
                                 const int8_t *nq, int64_t ldn, int64_t f, const float *scales, const float *row_scale,
                                 const float *bias, int relu, float *out, int64_t ldo, float *out_absmax,
                                 const tango_spmm_plan *plan, tango_stream_t stream) {
    if (n_rows < 0 || nseg < 1 || f < 0 || ldn < f || ldo < f || f > (1 << 20)) return TANGO_EINVAL;
    if (n_rows == 0 || f == 0) return TANGO_OK;
    if (!indptr || !indices || !nq || !scales || !out) return TANGO_EINVAL;
    SpmmArgs a{};
    a.indptr = indptr; a.indices = indices; a.edge_ids = nullptr; a.n_rows = n_rows; a.nseg = nseg;
    a.feat = nq; a.ld = ldn; a.f = (int)f; a.ew = nullptr; a.H = 1; a.D = (int)f;
    a.scales = scales; a.row_scale = row_scale; a.bias = bias; a.relu = relu;
    a.out = out; a.ldo = ldo; a.out_absmax = out_absmax;
    return launch_spmm<MODE_COPY>(a, plan, (cudaStream_t)stream);
}

extern "C" int tango_spmm_u_mul_e(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                  int64_t n_rows, const int8_t *nq, int64_t ldn, int h, int d, const int8_t *eq,
                                  const float *scale, float *out, int64_t ldo, const tango_spmm_plan *plan,
                                  tango_stream_t stream) {
    if (n_rows < 0 || h < 1 || d < 1) return TANGO_EINVAL;
    const int64_t f = (int64_t)h * d;
    if (ldn < f || ldo < f || f > (1 << 20)) return TANGO_EINVAL;
    if (n_rows == 0) return TANGO_OK;
    if (!indptr || !indices || !nq || !eq || !scale || !out) return TANGO_EINVAL;
    SpmmArgs a{};
    a.indptr = indptr; a.indices = indices; a.edge_ids = edge_ids; a.n_rows = n_rows; a.nseg = 1;
    a.feat = nq; a.ld = ldn; a.f = (int)f; a.ew = eq; a.H = h; a.D = d;
    a.scales = scale; a.out = out; a.ldo = ldo;
    return launch_spmm<MODE_WEIGHT_LANE>(a, plan, (cudaStream_t)stream);
}

extern "C" int tango_spmm_incidence(const int32_t *indptr, const int32_t *edge_ids, int64_t n_rows, const int8_t *zq,
                                    int64_t ldz, int64_t f, const float *scale, float *out, int64_t ldo,
                                    const tango_spmm_plan *plan, tango_stream_t stream) {
    if (n_rows < 0 || f < 0 || ldz < f || ldo < f || f > (1 << 20)) return TANGO_EINVAL;
    if (n_rows == 0 || f == 0) return TANGO_OK;
    if (!indptr || !zq || !scale || !out) return TANGO_EINVAL;
    SpmmArgs a{};
    a.indptr = indptr; a.indices = edge_ids; a.edge_ids = nullptr; a.n_rows = n_rows; a.nseg = 1;
    a.feat = zq; a.ld = ldz; a.f = (int)f; a.H = 1; a.D = (int)f;
    a.scales = scale; a.out = out; a.ldo = ldo;
    int rc = TANGO_OK;
    if (try_incidence_contig(a, plan, (cudaStream_t)stream, rc)) return rc;
    return launch_spmm<MODE_COPY>(a, plan, (cudaStream_t)stream);
}
