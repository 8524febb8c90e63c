// Edge softmax over the incoming edges of every destination, forward and gradient, in two flavours.
//
// fused GAT attention:
//   forward : a[e,h]  = softmax over the incoming edges of dst(e) of leaky_relu(el_q[src(e),h]*sl + er_q[dst(e),h]*sr)
//   backward: dz[e,h] = a * (da - sum_row a*da) * (z > 0 ? 1 : slope)   (PyTorch's LeakyReLU gradient convention at 0)
// plain scores (zin given):
//   forward : a[e,h]  = softmax over the incoming edges of dst(e) of zin[e,h] * zmul
//   backward: dz[e,h] = a * (da - sum_row a*da) * zmul
//
// two-step forward without an fp32 copy of the attention weights (stats / quantized):
//   stats     : per (row, head) the softmax statistics m = max z and inv = 1 / sum exp(z - m); the largest weight of a
//               row is exp(0) * inv = inv, so max over rows of inv is max|a| and fixes the int8 scale of a up front
//   quantized : a_q[e,h] = round(exp(z - m) * inv / scale) -- the int8 weights the aggregation consumes, written once
//   backward  : the same gradient as above with a recomputed from (z, m, inv) instead of being read
//
// A destination row is owned by a thread team: a whole CTA for the rows at the head of the degree-sorted order (a
// power-law graph has rows with 10^5 incoming edges; one warp would serialise them), a warp for the rest.  All heads
// of an edge are handled together (one 128-bit access per edge when H == 4).  The softmax statistics are
// accumulated "online" (running maximum with rescaling), so the forward needs two sweeps over a row, and every
// reduction runs in a fixed order, which makes the result deterministic.
#include "common.cuh"

namespace tango {

constexpr int kMaxHeads = 8;

struct GatArgs {
    const int32_t *indptr, *indices, *edge_ids, *row_order;
    int64_t n_rows, n_block_rows;
    const int8_t *elq, *erq;
    int H;
    const float *sl, *sr;
    float slope;
    float *att;          // forward: output; backward: input
    const float *datt;   // backward
    float *dz;           // backward
    const float *zin;    // plain-score flavour: fp32 scores [E, H] in edge-id order (elq / erq / sl / sr unused)
    float zmul;          // factor applied to zin before the softmax
    float *out_absmax;   // optional: receives max|output| / 127 (forward: of a, backward: of dz); must hold 0
    // two-step forward / recomputing backward
    float *row_m, *row_inv;        // [n_rows, H] softmax statistics (written by STATS, read by QUANT and by BWD)
    int8_t *att_q;                 // QUANT: int8 output [E, H] in edge-id order
    const float *att_scale;        // QUANT: scale of a (device, 1 element)
    int round_mode;
    uint64_t seed, call;
    const unsigned long long *step;
};

enum { FWD_FLOAT = 0, FWD_STATS = 1, FWD_QUANT = 2 };

__device__ __forceinline__ float leaky(float z, float slope) { return z >= 0.f ? z : __fmul_rn(z, slope); }

// z for all heads of slot j of row `row`
template <int HT>
__device__ __forceinline__ void edge_logits(const GatArgs &a, int j, const float (&er)[kMaxHeads], float sl,
                                            float (&z)[kMaxHeads]) {
    if (a.zin) {
        const int64_t eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        if (HT == 4) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(a.zin + eid * 4));
            z[0] = __fmul_rn(v.x, a.zmul); z[1] = __fmul_rn(v.y, a.zmul);
            z[2] = __fmul_rn(v.z, a.zmul); z[3] = __fmul_rn(v.w, a.zmul);
        } else {
            const int H = HT ? HT : a.H;
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h)
                if (h < H) z[h] = __fmul_rn(__ldg(a.zin + eid * H + h), a.zmul);
        }
        return;
    }
    const int64_t s = __ldg(a.indices + j);
    if (HT == 4) {
        const uint32_t w = __ldg(reinterpret_cast<const uint32_t *>(a.elq + s * 4));
#pragma unroll
        for (int h = 0; h < 4; ++h)
            z[h] = leaky(__fadd_rn(__fmul_rn((float)(int8_t)(w >> (8 * h)), sl), er[h]), a.slope);
    } else {
        const int H = HT ? HT : a.H;
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h)
            if (h < H) z[h] = leaky(__fadd_rn(__fmul_rn((float)__ldg(a.elq + s * H + h), sl), er[h]), a.slope);
    }
}

// Fixed-order reductions over a team of NT threads (NT = 32: one warp; else the whole CTA through shared memory).
template <int NT>
__device__ __forceinline__ float team_sum(float v, float *smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (NT == 32) return v;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < NT / 32; ++w) t += smem[w];
    return t;
}

// merges online-softmax states (m, s): fixed butterfly inside a warp, then warp 0..n in order
template <int NT>
__device__ __forceinline__ void team_softmax_merge(float &m, float &s, float *smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mm = fmaxf(m, m2);
        s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
        m = mm;
    }
    if (NT == 32) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { smem[warp] = m; smem[32 + warp] = s; }
    __syncthreads();
    float mm = -INFINITY, ss = 0.f;
    for (int w = 0; w < NT / 32; ++w) {
        const float m2 = smem[w], s2 = smem[32 + w];
        const float mx = fmaxf(mm, m2);
        ss = (mm == -INFINITY ? 0.f : ss * __expf(mm - mx)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mx));
        mm = mx;
    }
    m = mm; s = ss;
}

template <int NT, int HT, int STAGE>
__device__ __forceinline__ void softmax_row(const GatArgs &a, int64_t row, int tid, float *smem, float &amax) {
    const float sl = a.zin ? 0.f : __ldg(a.sl), sr = a.zin ? 0.f : __ldg(a.sr);
    const int beg = __ldg(a.indptr + row), end = __ldg(a.indptr + row + 1);
    const int H = HT ? HT : a.H;
    float er[kMaxHeads], m[kMaxHeads], s[kMaxHeads];
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h) {
        er[h] = (h < H && !a.zin) ? __fmul_rn((float)__ldg(a.erq + row * H + h), sr) : 0.f;
        m[h] = -INFINITY; s[h] = 0.f;
    }
    if (STAGE == FWD_QUANT) {
        // second step: statistics from the first step, int8 weights out
        float inv[kMaxHeads];
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h) {
            m[h] = h < H ? __ldg(a.row_m + row * H + h) : 0.f;
            inv[h] = h < H ? __ldg(a.row_inv + row * H + h) : 0.f;
        }
        const float inv_s = inv_scale(__ldg(a.att_scale));
        const uint64_t call = effective_call(a.call, a.step);
        const Philox ph{(uint32_t)a.seed, (uint32_t)(a.seed >> 32)};
        for (int j = beg + tid; j < end; j += NT) {
            float z[kMaxHeads];
            edge_logits<HT>(a, j, er, sl, z);
            const int64_t eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
            uint32_t packed = 0;
            uint64_t cached_blk = ~0ull;
            uint4 rnd = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h) {
                if (h < H) {
                    const float t = __fmul_rn(__expf(z[h] - m[h]) * inv[h], inv_s);
                    float u = 0.f;
                    if (a.round_mode == TANGO_ROUND_STOCHASTIC)
                        u = sr_uniform(ph, (uint64_t)eid * (uint64_t)H + (uint64_t)h, call, cached_blk, rnd);
                    const int qi = round_to_i8(t, a.round_mode, u);
                    if (HT == 4) packed |= ((uint32_t)qi & 0xffu) << (8 * h);
                    else a.att_q[eid * H + h] = (int8_t)qi;
                }
            }
            if (HT == 4) *reinterpret_cast<uint32_t *>(a.att_q + eid * 4) = packed;
        }
        return;
    }
    for (int j = beg + tid; j < end; j += NT) {
        float z[kMaxHeads];
        edge_logits<HT>(a, j, er, sl, z);
#pragma unroll
        for (int h = 0; h < kMaxHeads; ++h) {
            if (h < H) {
                if (z[h] > m[h]) { s[h] = s[h] * __expf(m[h] - z[h]) + 1.f; m[h] = z[h]; }
                else s[h] += __expf(z[h] - m[h]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
        if (h < H) team_softmax_merge<NT>(m[h], s[h], smem);
    float inv[kMaxHeads];
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h) inv[h] = h < H ? 1.f / s[h] : 0.f;
    if (STAGE == FWD_STATS) {
        // first step: keep (m, inv); the row's largest weight is exp(0) * inv = inv
        if (tid == 0 && end > beg) {
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h) {
                if (h < H) {
                    a.row_m[row * H + h] = m[h];
                    a.row_inv[row * H + h] = inv[h];
                    amax = fmaxf(amax, inv[h]);
                }
            }
        }
        return;
    }
    for (int j = beg + tid; j < end; j += NT) {
        float z[kMaxHeads];
        edge_logits<HT>(a, j, er, sl, z);
        const int64_t eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        if (HT == 4) {
            const float4 o = make_float4(__expf(z[0] - m[0]) * inv[0], __expf(z[1] - m[1]) * inv[1],
                                         __expf(z[2] - m[2]) * inv[2], __expf(z[3] - m[3]) * inv[3]);
            *reinterpret_cast<float4 *>(a.att + eid * 4) = o;
            amax = fmaxf(fmaxf(amax, fmaxf(o.x, o.y)), fmaxf(o.z, o.w));
        } else {
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h) {
                if (h < H) {
                    const float o = __expf(z[h] - m[h]) * inv[h];
                    a.att[eid * H + h] = o;
                    amax = fmaxf(amax, o);
                }
            }
        }
    }
}

// RECOMPUTE: the attention weights are not read but recomputed as exp(z - m) * inv from the forward's statistics.
template <int NT, int HT, bool RECOMPUTE>
__device__ __forceinline__ void softmax_bwd_row(const GatArgs &a, int64_t row, int tid, float *smem, float &amax) {
    const bool plain = a.zin != nullptr;   // backward of the plain flavour: zin is only a marker, never read
    const float sl = plain ? 0.f : __ldg(a.sl), sr = plain ? 0.f : __ldg(a.sr);
    const int beg = __ldg(a.indptr + row), end = __ldg(a.indptr + row + 1);
    const int H = HT ? HT : a.H;
    float er[kMaxHeads], dot[kMaxHeads], m[kMaxHeads], inv[kMaxHeads];
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h) {
        er[h] = (h < H && !plain) ? __fmul_rn((float)__ldg(a.erq + row * H + h), sr) : 0.f;
        dot[h] = 0.f;
        m[h] = (RECOMPUTE && h < H) ? __ldg(a.row_m + row * H + h) : 0.f;
        inv[h] = (RECOMPUTE && h < H) ? __ldg(a.row_inv + row * H + h) : 0.f;
    }
    for (int j = beg + tid; j < end; j += NT) {
        const int64_t eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        if (RECOMPUTE) {
            float z[kMaxHeads];
            edge_logits<HT>(a, j, er, sl, z);
            if (HT == 4) {
                const float4 g = __ldg(reinterpret_cast<const float4 *>(a.datt + eid * 4));
                dot[0] += __expf(z[0] - m[0]) * inv[0] * g.x; dot[1] += __expf(z[1] - m[1]) * inv[1] * g.y;
                dot[2] += __expf(z[2] - m[2]) * inv[2] * g.z; dot[3] += __expf(z[3] - m[3]) * inv[3] * g.w;
            } else {
#pragma unroll
                for (int h = 0; h < kMaxHeads; ++h)
                    if (h < H) dot[h] += __expf(z[h] - m[h]) * inv[h] * __ldg(a.datt + eid * H + h);
            }
        } else if (HT == 4) {
            const float4 p = __ldg(reinterpret_cast<const float4 *>(a.att + eid * 4));
            const float4 g = __ldg(reinterpret_cast<const float4 *>(a.datt + eid * 4));
            dot[0] += p.x * g.x; dot[1] += p.y * g.y; dot[2] += p.z * g.z; dot[3] += p.w * g.w;
        } else {
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h)
                if (h < H) dot[h] += __ldg(a.att + eid * H + h) * __ldg(a.datt + eid * H + h);
        }
    }
#pragma unroll
    for (int h = 0; h < kMaxHeads; ++h)
        if (h < H) dot[h] = team_sum<NT>(dot[h], smem);
    for (int j = beg + tid; j < end; j += NT) {
        float z[kMaxHeads];
        if (!plain) edge_logits<HT>(a, j, er, sl, z);   // leaky(z) has the sign of z
        const int64_t eid = a.edge_ids ? __ldg(a.edge_ids + j) : j;
        if (HT == 4) {
            const float4 p = RECOMPUTE ? make_float4(__expf(z[0] - m[0]) * inv[0], __expf(z[1] - m[1]) * inv[1],
                                                     __expf(z[2] - m[2]) * inv[2], __expf(z[3] - m[3]) * inv[3])
                                       : __ldg(reinterpret_cast<const float4 *>(a.att + eid * 4));
            const float4 g = __ldg(reinterpret_cast<const float4 *>(a.datt + eid * 4));
            float4 o = make_float4(p.x * (g.x - dot[0]), p.y * (g.y - dot[1]), p.z * (g.z - dot[2]),
                                   p.w * (g.w - dot[3]));
            if (plain) {
                o.x *= a.zmul; o.y *= a.zmul; o.z *= a.zmul; o.w *= a.zmul;
            } else {
                if (!(z[0] > 0.f)) o.x *= a.slope;
                if (!(z[1] > 0.f)) o.y *= a.slope;
                if (!(z[2] > 0.f)) o.z *= a.slope;
                if (!(z[3] > 0.f)) o.w *= a.slope;
            }
            *reinterpret_cast<float4 *>(a.dz + eid * 4) = o;
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(o.x), fabsf(o.y))), fmaxf(fabsf(o.z), fabsf(o.w)));
        } else {
#pragma unroll
            for (int h = 0; h < kMaxHeads; ++h) {
                if (h < H) {
                    const float p = RECOMPUTE ? __expf(z[h] - m[h]) * inv[h] : __ldg(a.att + eid * H + h);
                    float o = p * (__ldg(a.datt + eid * H + h) - dot[h]);
                    if (plain) o *= a.zmul;
                    else if (!(z[h] > 0.f)) o *= a.slope;
                    a.dz[eid * H + h] = o;
                    amax = fmaxf(amax, fabsf(o));
                }
            }
        }
    }
}

// blocks [0, n_block_rows): one CTA per row; the remaining blocks: one warp per row
// BWD: gradient kernel; STAGE: forward flavour (FWD_*) or, for BWD, 1 = recompute the weights from the statistics
template <int HT, bool BWD, int STAGE>
__global__ void __launch_bounds__(256) gat_softmax_kernel(const GatArgs a) {
    __shared__ float smem[64];
    float amax = 0.f;
    if ((int64_t)blockIdx.x < a.n_block_rows) {
        const int64_t row = a.row_order ? (int64_t)__ldg(a.row_order + blockIdx.x) : (int64_t)blockIdx.x;
        if (BWD) softmax_bwd_row<256, HT, STAGE != 0>(a, row, threadIdx.x, smem, amax);
        else softmax_row<256, HT, STAGE>(a, row, threadIdx.x, smem, amax);
    } else {
        const int64_t i = a.n_block_rows + ((int64_t)blockIdx.x - a.n_block_rows) * 8 + (threadIdx.x >> 5);
        if (i < a.n_rows) {
            const int64_t row = a.row_order ? (int64_t)__ldg(a.row_order + i) : i;
            if (BWD) softmax_bwd_row<32, HT, STAGE != 0>(a, row, threadIdx.x & 31, smem, amax);
            else softmax_row<32, HT, STAGE>(a, row, threadIdx.x & 31, smem, amax);
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

template <bool BWD, int STAGE = 0>
static int launch_gat(GatArgs &a, cudaStream_t stream) {
    if (a.n_rows < 0 || a.H < 1 || a.H > kMaxHeads) return TANGO_EINVAL;
    if (a.n_rows == 0) return TANGO_OK;
    if (!a.row_order) a.n_block_rows = 0;
    if (a.n_block_rows < 0 || a.n_block_rows > a.n_rows) return TANGO_EINVAL;
    const int64_t blocks = a.n_block_rows + ceil_div(a.n_rows - a.n_block_rows, 8);
    if (blocks > 0x7fffffff) return TANGO_ESIZE;
    const bool h4 = a.H == 4 && aligned(a.att, 16) && (a.zin ? aligned(a.zin, 16) : aligned(a.elq, 4)) &&
                    (!BWD || (aligned(a.datt, 16) && aligned(a.dz, 16))) && aligned(a.att_q, 4);
    if (h4) gat_softmax_kernel<4, BWD, STAGE><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (a.H == 1) gat_softmax_kernel<1, BWD, STAGE><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else if (a.H == 2) gat_softmax_kernel<2, BWD, STAGE><<<(unsigned)blocks, 256, 0, stream>>>(a);
    else gat_softmax_kernel<0, BWD, STAGE><<<(unsigned)blocks, 256, 0, stream>>>(a);
    TANGO_LAUNCH_CHECK();
    return TANGO_OK;
}

}  // namespace tango

using namespace tango;

extern "C" int tango_gat_edge_softmax(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                      const int32_t *row_order, int64_t n_block_rows, int64_t n_rows,
                                      const int8_t *elq, const int8_t *erq, int h, const float *sl, const float *sr,
                                      float slope, float *a, float *a_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !indices || !elq || !erq || !sl || !sr || !a)) return TANGO_EINVAL;
    GatArgs g{indptr, indices, edge_ids, row_order, n_rows, n_block_rows, elq, erq, h, sl, sr, slope, a, nullptr, nullptr,
              nullptr, 1.f, a_absmax};
    return launch_gat<false>(g, (cudaStream_t)stream);
}

extern "C" int tango_gat_edge_softmax_bwd(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                          const int32_t *row_order, int64_t n_block_rows, int64_t n_rows,
                                          const int8_t *elq, const int8_t *erq, int h, const float *sl,
                                          const float *sr, float slope, const float *a, const float *da, float *dz,
                                          float *dz_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !indices || !elq || !erq || !sl || !sr || !a || !da || !dz)) return TANGO_EINVAL;
    GatArgs g{indptr, indices, edge_ids, row_order, n_rows, n_block_rows, elq, erq, h, sl, sr, slope,
              const_cast<float *>(a), da, dz, nullptr, 1.f, dz_absmax};
    return launch_gat<true>(g, (cudaStream_t)stream);
}

extern "C" int tango_gat_edge_softmax_stats(const int32_t *indptr, const int32_t *indices, const int32_t *row_order,
                                            int64_t n_block_rows, int64_t n_rows, const int8_t *elq, const int8_t *erq,
                                            int h, const float *sl, const float *sr, float slope, float *row_m,
                                            float *row_inv, float *a_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !indices || !elq || !erq || !sl || !sr || !row_m || !row_inv)) return TANGO_EINVAL;
    GatArgs g{};
    g.indptr = indptr; g.indices = indices; g.row_order = row_order; g.n_rows = n_rows; g.n_block_rows = n_block_rows;
    g.elq = elq; g.erq = erq; g.H = h; g.sl = sl; g.sr = sr; g.slope = slope; g.zmul = 1.f;
    g.row_m = row_m; g.row_inv = row_inv; g.out_absmax = a_absmax;
    return launch_gat<false, FWD_STATS>(g, (cudaStream_t)stream);
}

extern "C" int tango_gat_edge_softmax_quantized(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                                const int32_t *row_order, int64_t n_block_rows, int64_t n_rows,
                                                const int8_t *elq, const int8_t *erq, int h, const float *sl,
                                                const float *sr, float slope, const float *row_m, const float *row_inv,
                                                const float *a_scale, int8_t *aq, int mode, uint64_t seed,
                                                uint64_t call, const uint64_t *step, tango_stream_t stream) {
    if (mode < 0 || mode > 2) return TANGO_EINVAL;
    if (n_rows > 0 && (!indptr || !indices || !elq || !erq || !sl || !sr || !row_m || !row_inv || !a_scale || !aq))
        return TANGO_EINVAL;
    GatArgs g{};
    g.indptr = indptr; g.indices = indices; g.edge_ids = edge_ids; g.row_order = row_order; g.n_rows = n_rows;
    g.n_block_rows = n_block_rows; g.elq = elq; g.erq = erq; g.H = h; g.sl = sl; g.sr = sr; g.slope = slope; g.zmul = 1.f;
    g.row_m = const_cast<float *>(row_m); g.row_inv = const_cast<float *>(row_inv); g.att_q = aq; g.att_scale = a_scale;
    g.round_mode = mode; g.seed = seed; g.call = call; g.step = reinterpret_cast<const unsigned long long *>(step);
    return launch_gat<false, FWD_QUANT>(g, (cudaStream_t)stream);
}

extern "C" int tango_gat_edge_softmax_bwd_stats(const int32_t *indptr, const int32_t *indices, const int32_t *edge_ids,
                                                const int32_t *row_order, int64_t n_block_rows, int64_t n_rows,
                                                const int8_t *elq, const int8_t *erq, int h, const float *sl,
                                                const float *sr, float slope, const float *row_m, const float *row_inv,
                                                const float *da, float *dz, float *dz_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !indices || !elq || !erq || !sl || !sr || !row_m || !row_inv || !da || !dz))
        return TANGO_EINVAL;
    GatArgs g{};
    g.indptr = indptr; g.indices = indices; g.edge_ids = edge_ids; g.row_order = row_order; g.n_rows = n_rows;
    g.n_block_rows = n_block_rows; g.elq = elq; g.erq = erq; g.H = h; g.sl = sl; g.sr = sr; g.slope = slope; g.zmul = 1.f;
    g.row_m = const_cast<float *>(row_m); g.row_inv = const_cast<float *>(row_inv); g.datt = da; g.dz = dz;
    g.out_absmax = dz_absmax;
    return launch_gat<true, 1>(g, (cudaStream_t)stream);
}

extern "C" int tango_edge_softmax(const int32_t *indptr, const int32_t *edge_ids, const int32_t *row_order,
                                  int64_t n_block_rows, int64_t n_rows, const float *z, int h, float zmul, float *a,
                                  float *a_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !z || !a)) return TANGO_EINVAL;
    GatArgs g{indptr, nullptr, edge_ids, row_order, n_rows, n_block_rows, nullptr, nullptr, h, nullptr, nullptr, 1.f,
              a, nullptr, nullptr, z, zmul, a_absmax};
    return launch_gat<false>(g, (cudaStream_t)stream);
}

extern "C" int tango_edge_softmax_bwd(const int32_t *indptr, const int32_t *edge_ids, const int32_t *row_order,
                                      int64_t n_block_rows, int64_t n_rows, int h, float zmul, const float *a,
                                      const float *da, float *dz, float *dz_absmax, tango_stream_t stream) {
    if (n_rows > 0 && (!indptr || !a || !da || !dz)) return TANGO_EINVAL;
    GatArgs g{indptr, nullptr, edge_ids, row_order, n_rows, n_block_rows, nullptr, nullptr, h, nullptr, nullptr, 1.f,
              const_cast<float *>(a), da, dz, a, zmul, dz_absmax};
    return launch_gat<true>(g, (cudaStream_t)stream);
}
