// SDDMM over int8 node features: per-edge dot products and element-wise ops.
//
// dot: a group of G lanes owns one (edge, head) pair; every lane loads VEC bytes of the source row and of the
// destination row, multiplies them with dp4a into an exact int32 and the group reduces by shuffle.  Edge endpoints
// are read 32 at a time with coalesced loads and handed out by shuffle.
#include "common.cuh"

namespace tango {

struct DotArgs {
    const int32_t *src, *dst;
    int64_t n_edges;
    const int8_t *u, *v;
    int64_t ldu, ldv;
    int H, D;
    int d_pad;  // bytes per head the lanes may read (multiple of VEC)
    int G;      // lanes per (edge, head), power of two
    const float *su, *sv;
    float *out;
    float *out_absmax;
};

template <int VEC>
__device__ __forceinline__ int dot_bytes(const int8_t *pu, const int8_t *pv) {
    if (VEC == 16) {
        const uint4 a = __ldg(reinterpret_cast<const uint4 *>(pu));
        const uint4 b = __ldg(reinterpret_cast<const uint4 *>(pv));
        int s = __dp4a((int)a.x, (int)b.x, 0);
        s = __dp4a((int)a.y, (int)b.y, s);
        s = __dp4a((int)a.z, (int)b.z, s);
        return __dp4a((int)a.w, (int)b.w, s);
    } else if (VEC == 4) {
        return __dp4a((int)__ldg(reinterpret_cast<const uint32_t *>(pu)),
                      (int)__ldg(reinterpret_cast<const uint32_t *>(pv)), 0);
    } else {
        return (int)__ldg(pu) * (int)__ldg(pv);
    }
}

template <int VEC> struct DotVec;
template <> struct DotVec<16> { typedef uint4 T; };
template <> struct DotVec<4> { typedef uint32_t T; };
template <> struct DotVec<1> { typedef int8_t T; };

template <int VEC>
__device__ __forceinline__ int dot_regs(const typename DotVec<VEC>::T &a, const typename DotVec<VEC>::T &b);
template <> __device__ __forceinline__ int dot_regs<16>(const uint4 &a, const uint4 &b) {
    int s = __dp4a((int)a.x, (int)b.x, 0);
    s = __dp4a((int)a.y, (int)b.y, s);
    s = __dp4a((int)a.z, (int)b.z, s);
    return __dp4a((int)a.w, (int)b.w, s);
}
template <> __device__ __forceinline__ int dot_regs<4>(const uint32_t &a, const uint32_t &b) {
    return __dp4a((int)a, (int)b, 0);
}
template <> __device__ __forceinline__ int dot_regs<1>(const int8_t &a, const int8_t &b) { return (int)a * (int)b; }

template <int VEC>
__global__ void __launch_bounds__(256) sddmm_dot_kernel(const DotArgs a) {
    typedef typename DotVec<VEC>::T V;
    const int lane = threadIdx.x & 31;
    const int G = a.G, IPS = 32 / G, grp = lane / G, sub = lane % G;
    const float sc = __fmul_rn(__ldg(a.su), __ldg(a.sv));
    const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t nwarp = (int64_t)gridDim.x * (blockDim.x >> 5);
    const bool single_trip = a.d_pad <= G * VEC;   // one load per operand covers a head: keep 4 items in flight
    constexpr int UN = 4;
    float amax = 0.f;
    for (int64_t e0 = warp * 32; e0 < a.n_edges; e0 += nwarp * 32) {
        const int64_t e = e0 + lane;
        int my_s = 0, my_d = 0;
        if (e < a.n_edges) { my_s = __ldg(a.src + e); my_d = __ldg(a.dst + e); }
        const int n_e = (int)min((int64_t)32, a.n_edges - e0);
        const int items = n_e * a.H;
        for (int it0 = 0; it0 < items; it0 += IPS * UN) {
            int acc[UN], el[UN], hd[UN];
            V ru[UN], rv[UN];
            bool ok[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const int item = it0 + u * IPS + grp;
                el[u] = item / a.H; hd[u] = item - el[u] * a.H;
                const int s_id = __shfl_sync(0xffffffffu, my_s, el[u] & 31);
                const int d_id = __shfl_sync(0xffffffffu, my_d, el[u] & 31);
                ok[u] = item < items;
                acc[u] = 0;
                const int8_t *pu = a.u + (int64_t)s_id * a.ldu + (int64_t)hd[u] * a.D;
                const int8_t *pv = a.v + (int64_t)d_id * a.ldv + (int64_t)hd[u] * a.D;
                if (single_trip) {
                    const bool ld = ok[u] && sub * VEC < a.d_pad;
                    ru[u] = ld ? __ldg(reinterpret_cast<const V *>(pu + sub * VEC)) : V();
                    rv[u] = ld ? __ldg(reinterpret_cast<const V *>(pv + sub * VEC)) : V();
                } else if (ok[u]) {
                    for (int off = sub * VEC; off < a.d_pad; off += G * VEC)
                        acc[u] += dot_bytes<VEC>(pu + off, pv + off);
                }
            }
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                if (single_trip) acc[u] = dot_regs<VEC>(ru[u], rv[u]);
                for (int o = G >> 1; o > 0; o >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], o);
                if (ok[u] && sub == 0) {
                    const float r = __fmul_rn((float)acc[u], sc);
                    __stcs(a.out + (e0 + el[u]) * a.H + hd[u], r);
                    amax = fmaxf(amax, fabsf(r));
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

// ---- row-wise dot: out[eid(j), h] = <U[indices[j], h, :], V[row, h, :]> for every slot j of a CSR/CSC row.
// The fixed operand's row is loaded once per row and stays in registers; only the other operand is gathered, which
// halves the gathered bytes of the endpoint-list kernel above, and the index stream is read once, coalesced.  A warp
// owns a row (or a slice of a long row: slices need no merging, every edge has its own output); G lanes share a
// neighbour, 32 / G neighbours per step, four steps in flight.  A head occupies LH = D / VEC adjacent lanes (or the
// whole group when there is one head) and is reduced with log2(LH) shuffles.
struct DotRowArgs {
    const int32_t *indptr, *indices, *edge_ids, *row_order;
    const int32_t *units;   // (row, begin, end, -) slices of the rows longer than split_threshold
    int64_t n_units, n_rows;
    int split_threshold;    // rows longer than this are covered by units (0: none)
    const int8_t *u, *v;    // u is gathered through indices, v is read at the row
    int64_t ldu, ldv;
    int H, f, f_pad, G, LH;
    const float *su, *sv;
    float *out;
    float *out_absmax;
    int64_t n_long;         // rows row_order[0, n_long) get a warp each; the shorter rows after them a lane group
};

template <int VEC, bool QUAD>
__device__ __forceinline__ void dot_row_segment(const DotRowArgs &a, int64_t row, int beg, int end, float sc,
                                                float &amax) {
    typedef typename DotVec<VEC>::T V;
    const int lane = threadIdx.x & 31;
    const int G = a.G, NB = 32 / G, grp = lane / G, sub = lane % G;
    const bool active = sub * VEC < a.f_pad;
    const int off = active ? sub * VEC : 0;
    V vr = V();
    if (active) vr = __ldg(reinterpret_cast<const V *>(a.v + row * a.ldv + off));
    const int8_t *ubase = a.u + off;
    const uint32_t ld = (uint32_t)a.ldu;
    const int head = (sub * VEC) / (a.LH * VEC);            // LH lanes per head
    const bool writer = active && (sub % a.LH) == 0 && head < a.H;
    const bool quad_writer = (sub % a.LH) < 4 && head < a.H;   // QUAD: lane r of the head's first quad stores step r
    constexpr int U = 4;
    int j0 = beg;
    int nxt_idx = 0, nxt_eid = 0;
    if (j0 + 32 <= end) {
        nxt_idx = __ldg(a.indices + j0 + lane);
        nxt_eid = a.edge_ids ? __ldg(a.edge_ids + j0 + lane) : j0 + lane;
    }
    if (G >= U) {
        for (; j0 + 32 <= end; j0 += 32) {
            const int my_idx = nxt_idx, my_eid = nxt_eid;
            if (j0 + 64 <= end) {
                nxt_idx = __ldg(a.indices + j0 + 32 + lane);
                nxt_eid = a.edge_ids ? __ldg(a.edge_ids + j0 + 32 + lane) : j0 + 32 + lane;
            }
            for (int s = 0, lane0 = grp; s < G; s += U, lane0 += U * NB) {
                V ur[U];
#pragma unroll
                for (int k = 0; k < U; ++k) {
                    const int idx = __shfl_sync(0xffffffffu, my_idx, lane0 + k * NB);
                    ur[k] = __ldg(reinterpret_cast<const V *>(ubase + (uint64_t)(uint32_t)idx * ld));
                }
                int p[U];
#pragma unroll
                for (int k = 0; k < U; ++k) p[k] = active ? dot_regs<VEC>(ur[k], vr) : 0;
                if (QUAD) {
                    // Four lanes or more per head: three exchanges leave lane r = sub % 4 of every aligned lane quad
                    // with step r's sum over the quad (instead of 2 x 4 shuffles that leave 3 of 4 lanes idle), the
                    // remaining lanes of the head are folded in, and every one of those four lanes stores one value.
                    const bool b0 = sub & 1, b1 = sub & 2;
                    const int s01 = (b0 ? p[1] : p[0]) + __shfl_xor_sync(0xffffffffu, b0 ? p[0] : p[1], 1);
                    const int s23 = (b0 ? p[3] : p[2]) + __shfl_xor_sync(0xffffffffu, b0 ? p[2] : p[3], 1);
                    int t = (b1 ? s23 : s01) + __shfl_xor_sync(0xffffffffu, b1 ? s01 : s23, 2);
                    for (int o = 4; o < a.LH; o <<= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
                    const int e = __shfl_sync(0xffffffffu, my_eid, lane0 + (sub & 3) * NB);   // edge of step sub % 4
                    if (quad_writer) {
                        const float r = __fmul_rn((float)t, sc);
                        __stcs(a.out + (int64_t)e * a.H + head, r);
                        amax = fmaxf(amax, fabsf(r));
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < U; ++k) {
                        int acc = p[k];
                        for (int o = a.LH >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                        const int e = __shfl_sync(0xffffffffu, my_eid, lane0 + k * NB);
                        if (writer) {
                            const float r = __fmul_rn((float)acc, sc);
                            __stcs(a.out + (int64_t)e * a.H + head, r);
                            amax = fmaxf(amax, fabsf(r));
                        }
                    }
                }
            }
        }
    }
    // ragged tail, and every batch when fewer than four lanes share a neighbour
    for (; j0 < end; j0 += 32) {
        const int j = j0 + lane;
        int my_idx = -1, my_eid = 0;
        if (j < end) {
            my_idx = __ldg(a.indices + j);
            my_eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        }
        const int steps = min(G, (end - j0 + NB - 1) / NB);
        for (int s = 0; s < steps; ++s) {
            const int src_lane = (s * NB + grp) & 31;
            const int idx = __shfl_sync(0xffffffffu, my_idx, src_lane);
            const int eid = __shfl_sync(0xffffffffu, my_eid, src_lane);
            int acc = 0;
            if (idx >= 0 && active)
                acc = dot_regs<VEC>(__ldg(reinterpret_cast<const V *>(ubase + (uint64_t)(uint32_t)idx * ld)), vr);
            for (int o = a.LH >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (writer && idx >= 0) {
                const float r = __fmul_rn((float)acc, sc);
                __stcs(a.out + (int64_t)eid * a.H + head, r);
                amax = fmaxf(amax, fabsf(r));
            }
        }
    }
}

template <int VEC, bool QUAD>
__global__ void __launch_bounds__(128, 8) sddmm_dot_rows_kernel(const DotRowArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const float sc = __fmul_rn(__ldg(a.su), __ldg(a.sv));
    float amax = 0.f;
    if (w < a.n_units) {
        const int4 u = __ldg(reinterpret_cast<const int4 *>(a.units) + w);
        dot_row_segment<VEC, QUAD>(a, u.x, u.y, u.z, sc, amax);
    } else if (w - a.n_units < a.n_rows) {
        int64_t row = w - a.n_units;
        if (a.row_order) row = __ldg(a.row_order + row);
        const int beg = __ldg(a.indptr + row), end = __ldg(a.indptr + row + 1);
        if (!(a.n_units > 0 && end - beg > a.split_threshold)) dot_row_segment<VEC, QUAD>(a, row, beg, end, sc, amax);
    }
    if (a.out_absmax) {
        amax = warp_max(amax);
        if (lane == 0 && amax > 0.f) {
            const float s = __fdiv_rn(amax, 127.0f);
            if (s > __ldcg(a.out_absmax)) atomic_max_nonneg(a.out_absmax, s);
        }
    }
}

// Short rows (a handful of edges): a group of G lanes owns one row, keeps its piece of V[row] in registers, fetches
// G neighbour ids with one coalesced load, gathers four neighbours' pieces of U at a time, and the LH lanes of a head
// reduce with shuffles restricted to the group.  Several rows per warp, no lane idles on a 7-edge row.
template <int VEC>
__global__ void __launch_bounds__(128, 12) sddmm_dot_short_kernel(const DotRowArgs a) {
    typedef typename DotVec<VEC>::T V;
    const int lane = threadIdx.x & 31;
    const int G = a.G, sub = lane % G;
    const int64_t gid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int64_t n_short = a.n_rows - a.n_long;
    const bool in_range = gid < n_short;
    const bool active = in_range && sub * VEC < a.f_pad;
    const int off = active ? sub * VEC : 0;
    const unsigned gmask = (G >= 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane - sub));
    const int base_lane = lane - sub;
    const float sc = __fmul_rn(__ldg(a.su), __ldg(a.sv));
    const int head = (sub * VEC) / (a.LH * VEC);
    const bool writer = active && (sub % a.LH) == 0 && head < a.H;
    float amax = 0.f;
    int beg = 0, end = 0;
    V vr = V();
    if (in_range) {
        const int64_t row = a.row_order ? (int64_t)__ldg(a.row_order + a.n_long + gid) : a.n_long + gid;
        beg = __ldg(a.indptr + row); end = __ldg(a.indptr + row + 1);
        if (active) vr = __ldg(reinterpret_cast<const V *>(a.v + row * a.ldv + off));
    }
    const int8_t *ubase = a.u + off;
    const uint32_t ld = (uint32_t)a.ldu;
    const int CH = G < 4 ? 4 : G;           // ids fetched per step (narrow groups: lane `sub` fetches several)
    for (int j0 = beg; j0 < end; j0 += CH) {
        int my_idx = 0, my_eid = 0;
        int idx4[4] = {0, 0, 0, 0}, eid4[4] = {0, 0, 0, 0};
        if (G >= 4) {
            const int j = j0 + sub;
            if (j < end) {
                my_idx = __ldg(a.indices + j);
                my_eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (j0 + k < end) {
                    idx4[k] = __ldg(a.indices + j0 + k);
                    eid4[k] = a.edge_ids ? __ldg(a.edge_ids + j0 + k) : j0 + k;
                }
        }
        const int cnt = min(CH, end - j0);
        for (int s0 = 0; s0 < cnt; s0 += 4) {
            V ur[4];
            int e[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int idx;
                if (G >= 4) {
                    idx = __shfl_sync(gmask, my_idx, base_lane + ((s0 + k) & (G - 1)));
                    e[k] = __shfl_sync(gmask, my_eid, base_lane + ((s0 + k) & (G - 1)));
                } else {
                    idx = idx4[k]; e[k] = eid4[k];
                }
                ur[k] = (s0 + k < cnt && active) ? __ldg(reinterpret_cast<const V *>(ubase + (uint64_t)(uint32_t)idx * ld)) : V();
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int acc = dot_regs<VEC>(ur[k], vr);
                for (int o = a.LH >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(gmask, acc, o);
                if (writer && s0 + k < cnt) {
                    const float r = __fmul_rn((float)acc, sc);
                    __stcs(a.out + (int64_t)e[k] * a.H + head, r);
                    amax = fmaxf(amax, fabsf(r));
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

struct ElemArgs {
    const int32_t *src, *dst;
    int64_t n_edges;
    const int8_t *u, *v;
    int64_t ldu, ldv;
    int64_t dim;
    const float *su, *sv;
    float *out;
    float *out_absmax;
};

template <int OP>
__device__ __forceinline__ float apply_op(float x, float y) {
    if (OP == TANGO_OP_ADD) return __fadd_rn(x, y);
    if (OP == TANGO_OP_SUB) return __fsub_rn(x, y);
    if (OP == TANGO_OP_MUL) return __fmul_rn(x, y);
    return __fdiv_rn(x, y);
}

// One thread per (edge, group of 4 features).  VEC4: 32-bit loads of both rows, 128-bit store when dim % 4 == 0.
template <int OP, bool VEC4>
__global__ void __launch_bounds__(256) sddmm_elem_kernel(const ElemArgs a) {
    const float su = __ldg(a.su), sv = __ldg(a.sv);
    const int64_t groups = (a.dim + 3) >> 2, total = a.n_edges * groups;
    float amax = 0.f;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t e = i / groups, c0 = (i - e * groups) << 2;
        const int64_t s = __ldg(a.src + e), d = __ldg(a.dst + e);
        const int8_t *pu = a.u + s * a.ldu + c0, *pv = a.v + d * a.ldv + c0;
        int8_t bu[4], bv[4];
        if (VEC4) {
            const uint32_t wu = __ldg(reinterpret_cast<const uint32_t *>(pu));
            const uint32_t wv = __ldg(reinterpret_cast<const uint32_t *>(pv));
#pragma unroll
            for (int k = 0; k < 4; ++k) { bu[k] = (int8_t)(wu >> (8 * k)); bv[k] = (int8_t)(wv >> (8 * k)); }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const bool ok = c0 + k < a.dim;
                bu[k] = ok ? __ldg(pu + k) : (int8_t)0;
                bv[k] = ok ? __ldg(pv + k) : (int8_t)1;
            }
        }
        float r[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            r[k] = apply_op<OP>(__fmul_rn((float)bu[k], su), __fmul_rn((float)bv[k], sv));
            if (c0 + k < a.dim) amax = fmaxf(amax, fabsf(r[k]));
        }
        float *o = a.out + e * a.dim + c0;
        if (VEC4 && (a.dim & 3) == 0) {
            __stcs(reinterpret_cast<float4 *>(o), make_float4(r[0], r[1], r[2], r[3]));
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                if (c0 + k < a.dim) o[k] = r[k];
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

static int pow2_ceil(int x) {
    int p = 1;
    while (p < x) p <<= 1;
    return p;
}

}  // namespace tango

using namespace tango;

extern "C" int tango_sddmm_dot(const int32_t *src, const int32_t *dst, int64_t n_edges, const int8_t *uq, int64_t ldu,
                               const int8_t *vq, int64_t ldv, int h, int d, const float *su, const float *sv,
                               float *out, float *out_absmax, tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_edges < 0 || h < 1 || d < 1 || ldu < (int64_t)h * d || ldv < (int64_t)h * d) return TANGO_EINVAL;
    if (n_edges == 0) return TANGO_OK;
    if (!src || !dst || !uq || !vq || !su || !sv || !out) return TANGO_EINVAL;
    DotArgs a{};
    a.src = src; a.dst = dst; a.n_edges = n_edges; a.u = uq; a.v = vq; a.ldu = ldu; a.ldv = ldv; a.H = h; a.D = d;
    a.su = su; a.sv = sv; a.out = out; a.out_absmax = out_absmax;
    // widest load for which every head starts on a VEC boundary of both operands
    int vec = 1;
    const bool single = (h == 1);
    auto fits = [&](int v) {
        return ldu % v == 0 && ldv % v == 0 && aligned(uq, v) && aligned(vq, v) &&
               (single ? (round_up(d, v) <= ldu && round_up(d, v) <= ldv) : d % v == 0);
    };
    if (fits(16)) vec = 16; else if (fits(4)) vec = 4;
    a.d_pad = (int)round_up(d, vec);  // single head: pad bytes are zero by the layout convention
    a.G = pow2_ceil(a.d_pad / vec);
    if (a.G > 32) a.G = 32;
    int64_t blocks = ceil_div(ceil_div(n_edges, 32), 8);
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (vec == 16) sddmm_dot_kernel<16><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (vec == 4) sddmm_dot_kernel<4><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else sddmm_dot_kernel<1><<<(unsigned)blocks, 256, 0, stream>>>(a);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

extern "C" int tango_sddmm_dot_rows(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                    int64_t n_rows, const int8_t *uq, int64_t ldu, const int8_t *vq, int64_t ldv,
                                    int h, int d, const float *su, const float *sv, float *out, float *out_absmax,
                                    const tango_spmm_plan *plan, tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    const int64_t f = (int64_t)h * d;
    if (n_rows < 0 || h < 1 || d < 1 || ldu < f || ldv < f || ldu > 0x7fffffff) return TANGO_EINVAL;
    if (n_rows == 0) return TANGO_OK;
    if (!indptr || !indices || !uq || !vq || !su || !sv || !out) return TANGO_EINVAL;
    // one 16-byte (or 4-byte) piece per lane; a head must cover a power-of-two number of whole pieces
    int vec = 0;
    auto fits = [&](int v) {
        if (ldu % v || ldv % v || !aligned(uq, v) || !aligned(vq, v)) return false;
        if (round_up(f, v) > ldu || round_up(f, v) > ldv || round_up(f, v) > 32 * v) return false;
        if (h == 1) return true;
        const int lh = d / v;
        return d % v == 0 && (lh & (lh - 1)) == 0;
    };
    if (fits(16)) vec = 16; else if (fits(4)) vec = 4;
    if (vec == 0) return TANGO_EALIGN;   // the caller falls back to the endpoint-list kernel
    DotRowArgs a{};
    a.indptr = indptr; a.indices = indices; a.edge_ids = edge_ids; a.n_rows = n_rows;
    a.u = uq; a.v = vq; a.ldu = ldu; a.ldv = ldv; a.H = h; a.f = (int)f; a.f_pad = (int)round_up(f, vec);
    a.G = pow2_ceil(a.f_pad / vec);
    a.LH = (h == 1) ? a.G : d / vec;
    a.su = su; a.sv = sv; a.out = out; a.out_absmax = out_absmax;
    a.n_long = n_rows;
    if (plan) {
        a.row_order = plan->row_order;
        if (plan->n_units > 0) {
            if (!plan->units || !aligned(plan->units, 16)) return TANGO_EINVAL;
            a.units = plan->units; a.n_units = plan->n_units; a.split_threshold = plan->split_threshold;
        }
        // rows of a few edges (the tail of the degree-sorted order) go to the lane-group kernel
        if (plan->row_order && plan->n_long_rows >= 0 && plan->n_long_rows <= n_rows) a.n_long = plan->n_long_rows;
    }
    const int64_t n_short = n_rows - a.n_long;
    DotRowArgs al = a;
    al.n_rows = a.n_long;        // the warp-per-row kernel walks row_order[0, n_long)
    const int64_t blocks = ceil_div(al.n_units + al.n_rows, 4);
    if (blocks > 0x7fffffff) return TANGO_ESIZE;
    const bool quad = a.LH >= 4;
    if (blocks > 0) {
        if (vec == 16 && quad) sddmm_dot_rows_kernel<16, true><<<(unsigned)blocks, 128, 0, stream>>>(al);
        else if (vec == 16) sddmm_dot_rows_kernel<16, false><<<(unsigned)blocks, 128, 0, stream>>>(al);
        else if (quad) sddmm_dot_rows_kernel<4, true><<<(unsigned)blocks, 128, 0, stream>>>(al);
        else sddmm_dot_rows_kernel<4, false><<<(unsigned)blocks, 128, 0, stream>>>(al);
        TANGO_LAUNCH_CHECK();
    }
    if (n_short > 0) {
        const int64_t sb = ceil_div(n_short * a.G, 128);
        if (sb > 0x7fffffff) return TANGO_ESIZE;
        if (vec == 16) sddmm_dot_short_kernel<16><<<(unsigned)sb, 128, 0, stream>>>(a);
        else sddmm_dot_short_kernel<4><<<(unsigned)sb, 128, 0, stream>>>(a);
        TANGO_LAUNCH_CHECK();
    }
    return TANGO_OK;
}

template <int OP>
static int launch_elem(const ElemArgs &a, bool vec4, cudaStream_t stream) {
    const int64_t total = a.n_edges * ((a.dim + 3) / 4);
    int64_t blocks = ceil_div(total, 256);
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (vec4) sddmm_elem_kernel<OP, true><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else sddmm_elem_kernel<OP, false><<<(unsigned)blocks, 256, 0, stream>>>(a);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

extern "C" int tango_sddmm_elementwise(int op, const int32_t *src, const int32_t *dst, int64_t n_edges,
                                       const int8_t *uq, int64_t ldu, const int8_t *vq, int64_t ldv, int64_t dim,
                                       const float *su, const float *sv, float *out, float *out_absmax,
                                       tango_stream_t stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    if (n_edges < 0 || dim < 1 || ldu < dim || ldv < dim || op < 0 || op > 3) return TANGO_EINVAL;
    if (n_edges == 0) return TANGO_OK;
    if (!src || !dst || !uq || !vq || !su || !sv || !out) return TANGO_EINVAL;
    ElemArgs a{src, dst, n_edges, uq, vq, ldu, ldv, dim, su, sv, out, out_absmax};
    const bool vec4 = ldu % 4 == 0 && ldv % 4 == 0 && aligned(uq, 4) && aligned(vq, 4) && aligned(out, 16) &&
                      round_up(dim, 4) <= ldu && round_up(dim, 4) <= ldv;
    switch (op) {
        case TANGO_OP_ADD: return launch_elem<TANGO_OP_ADD>(a, vec4, stream);
        case TANGO_OP_SUB: return launch_elem<TANGO_OP_SUB>(a, vec4, stream);
        case TANGO_OP_MUL: return launch_elem<TANGO_OP_MUL>(a, vec4, stream);
        default: return launch_elem<TANGO_OP_DIV>(a, vec4, stream);
    }
}
