/*
 * Plain-C restatement of Tango's quantized primitives (second, independent checker beside tango_oracle.py; used for
 * the sizes NumPy scatter-adds are too slow for).  TEST INFRASTRUCTURE ONLY -- never linked into the product.
 * PARITY UNPINNED: the reference ships no golden vectors; each function cites the reference source it follows.
 * Compile with -ffp-contract=off: every fp32 operation below must stay a single IEEE operation.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

/* Philox4x32-10 (Salmon et al., SC'11). */
static void philox(uint32_t c[4], uint32_t k0, uint32_t k1) {
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
}

/* scale = max|x| / 127 -- cuda/src/quantization.cu:45-93, cuda/src/utils.h:83-99 */
float oc_absmax_scale(const float *x, int64_t n) {
    float m = 0.f;
    for (int64_t i = 0; i < n; ++i) { float a = fabsf(x[i]); if (a > m) m = a; }
    return m / 127.0f;
}

/* mode 0: (int8)(x*inv) truncation -- cuda/src/iterator.h:155-164; mode 1: rintf + clamp --
 * cuda/src/quantization.cu:6-35; mode 2: floor(x*inv + u), u = (philox >> 8) * 2^-24 (not in the reference). */
void oc_quantize(const float *x, int64_t n, float scale, int mode, uint64_t seed, uint64_t call, int8_t *q) {
    float inv = scale == 0.f ? 0.f : 1.0f / scale;
    if (isinf(inv)) inv = 0.f; /* subnormal scale: the tensor quantizes to zeros */
#pragma omp parallel for
    for (int64_t i = 0; i < n; ++i) {
        float t = x[i] * inv, r;
        if (mode == 1) r = rintf(t);
        else if (mode == 0) r = truncf(t);
        else {
            uint32_t c[4] = {(uint32_t)(i >> 2), (uint32_t)((uint64_t)(i >> 2) >> 32), (uint32_t)call,
                             (uint32_t)(call >> 32)};
            philox(c, (uint32_t)seed, (uint32_t)(seed >> 32));
            float u = (float)(c[i & 3] >> 8) * 5.9604644775390625e-08f;
            float v = t + u;
            r = floorf(v);
        }
        if (r > 127.f) r = 127.f;
        if (r < -127.f) r = -127.f;
        q[i] = (int8_t)r;
    }
}

/* acc[m,n] = sum_k a[m,k]*b[n,k] -- cuda/src/QGEMM_forward.cu:22-27 */
void oc_igemm_nt(const int8_t *a, const int8_t *b, int64_t M, int64_t N, int64_t K, int32_t *acc) {
#pragma omp parallel for
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            int32_t s = 0;
            for (int64_t k = 0; k < K; ++k) s += (int32_t)a[m * K + k] * (int32_t)b[n * K + k];
            acc[m * N + n] = s;
        }
}

/* out[v,:] = float(sum_j nq[indices[j],:]) * scale -- cuda/src/SPMM.cu:23-68 (all-ones CSR times int8 dense) */
void oc_spmm_copy_u(const int64_t *indptr, const int64_t *indices, int64_t n_rows, const int8_t *nq, int64_t f,
                    float scale, float *out) {
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t v = 0; v < n_rows; ++v) {
        int32_t acc[1024];
        for (int64_t c0 = 0; c0 < f; c0 += 1024) {
            int64_t w = f - c0 < 1024 ? f - c0 : 1024;
            memset(acc, 0, sizeof(int32_t) * (size_t)w);
            for (int64_t j = indptr[v]; j < indptr[v + 1]; ++j) {
                const int8_t *row = nq + indices[j] * f + c0;
                for (int64_t c = 0; c < w; ++c) acc[c] += row[c];
            }
            for (int64_t c = 0; c < w; ++c) out[v * f + c0 + c] = (float)acc[c] * scale;
        }
    }
}

/* out[v,h,:] = float(sum_j eq[eid[j],h] * nq[indices[j],h,:]) * scale -- cuda/src/SPMM.cu:70-130,
 * cuda/kernels.py:122-136 */
void oc_spmm_u_mul_e(const int64_t *indptr, const int64_t *indices, const int64_t *eids, int64_t n_rows,
                     const int8_t *nq, int64_t H, int64_t D, const int8_t *eq, float scale, float *out) {
    const int64_t f = H * D;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t v = 0; v < n_rows; ++v)
        for (int64_t h = 0; h < H; ++h)
            for (int64_t d = 0; d < D; ++d) {
                int32_t acc = 0;
                for (int64_t j = indptr[v]; j < indptr[v + 1]; ++j) {
                    const int64_t e = eids ? eids[j] : j;
                    acc += (int32_t)eq[e * H + h] * (int32_t)nq[indices[j] * f + h * D + d];
                }
                out[v * f + h * D + d] = (float)acc * scale;
            }
}

/* out[e,h] = float(sum_d u[src,h,d]*v[dst,h,d]) * (su*sv) -- cuda/src/SDDMM.cu:8-47 */
void oc_sddmm_dot(const int64_t *src, const int64_t *dst, int64_t n_edges, const int8_t *u, const int8_t *v, int64_t H,
                  int64_t D, float su, float sv, float *out) {
    const float sc = su * sv;
#pragma omp parallel for
    for (int64_t e = 0; e < n_edges; ++e)
        for (int64_t h = 0; h < H; ++h) {
            int32_t acc = 0;
            const int8_t *pu = u + (src[e] * H + h) * D, *pv = v + (dst[e] * H + h) * D;
            for (int64_t d = 0; d < D; ++d) acc += (int32_t)pu[d] * (int32_t)pv[d];
            out[e * H + h] = (float)acc * sc;
        }
}
