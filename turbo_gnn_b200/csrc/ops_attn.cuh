// Shared pieces of the fused attention ops (GATv2 and graph transformer).
//
// A node row is [heads * head_dim]; a warp (or a group of G lanes) covers it in
// 16-byte chunks, lane-contiguous, so one head occupies `lanes_per_head`
// consecutive lanes of one chunk index v (or, for head_dim > 32 chunks, all 32
// lanes of several v).  Per-head dot products are finished with xor shuffles
// inside that lane range; every lane of a head then holds the head's score and
// runs the softmax bookkeeping for its own accumulators redundantly.
#pragma once

#include "ops_reduce.cuh"

namespace tgnn {

// Head layout of one lane.
template <int kVpl, int kPer>
struct HeadMap {
    int lanes_per_head;  // shuffle span, <= 32
    int v_per_head;      // chunk indices v that belong to one head (1 unless head_dim > 32 chunks)
    int head[kVpl];      // head index of chunk v, -1 if the chunk is beyond the row
    bool writer[kVpl];   // this lane stores the per-head scalars of chunk v's head

    __device__ __forceinline__ HeadMap(const Lanes &L, const ChunkMap<kVpl, kPer> &map, int head_dim) {
        const int cph = head_dim / kPer;
        lanes_per_head = cph > 32 ? 32 : cph;
        v_per_head = cph > 32 ? cph / 32 : 1;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            head[v] = map.off[v] >= 0 ? map.off[v] / head_dim : -1;
            writer[v] = map.off[v] >= 0 && (map.off[v] % head_dim) == 0 && L.grp == 0;
        }
    }

    // pv[v]: this lane's partial dot product over chunk v.  On return pv[v] is the
    // full dot product of chunk v's head, in every lane of that head.
    __device__ __forceinline__ void finish(float (&pv)[kVpl]) const {
        if (v_per_head > 1) {
            float tot[kVpl];
#pragma unroll
            for (int v = 0; v < kVpl; ++v) {
                tot[v] = 0.0f;
#pragma unroll
                for (int u = 0; u < kVpl; ++u)
                    if (u / v_per_head == v / v_per_head) tot[v] += pv[u];
            }
#pragma unroll
            for (int v = 0; v < kVpl; ++v) pv[v] = tot[v];
        }
#pragma unroll
        for (int v = 0; v < kVpl; ++v)
            for (int o = lanes_per_head >> 1; o > 0; o >>= 1) pv[v] += __shfl_xor_sync(kFull, pv[v], o);
    }
};

// Running softmax-weighted sum of gathered rows: per chunk v a running max m,
// a running denominator s and kPer numerators.
template <int kVpl, int kPer>
struct SoftmaxAcc {
    static constexpr int kVals = kVpl * kPer;
    static constexpr int kWords = kVals + 2 * kVpl;
    float acc[kVals];
    float m[kVpl];
    float s[kVpl];

    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < kVals; ++i) acc[i] = 0.0f;
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            m[v] = -INFINITY;
            s[v] = 0.0f;
        }
    }
    // Fold one edge: score of chunk v's head, x = the gathered value chunk.
    __device__ __forceinline__ void push(int v, float score, const float *x) {
        const float m_new = fmaxf(m[v], score);
        const float corr = __expf(m[v] - m_new);  // 0 on the first edge (m = -inf)
        const float p = __expf(score - m_new);
        s[v] = fmaf(s[v], corr, p);
#pragma unroll
        for (int e = 0; e < kPer; ++e) acc[v * kPer + e] = fmaf(acc[v * kPer + e], corr, p * x[e]);
        m[v] = m_new;
    }
    __device__ __forceinline__ void merge(const SoftmaxAcc &o) {
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            const float m_new = fmaxf(m[v], o.m[v]);
            const float c1 = m[v] == -INFINITY ? 0.0f : __expf(m[v] - m_new);
            const float c2 = o.m[v] == -INFINITY ? 0.0f : __expf(o.m[v] - m_new);
            s[v] = s[v] * c1 + o.s[v] * c2;
#pragma unroll
            for (int e = 0; e < kPer; ++e) acc[v * kPer + e] = acc[v * kPer + e] * c1 + o.acc[v * kPer + e] * c2;
            m[v] = m_new;
        }
    }
    __device__ __forceinline__ void to_words(uint32_t *w) const {
#pragma unroll
        for (int i = 0; i < kVals; ++i) w[i] = __float_as_uint(acc[i]);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            w[kVals + v] = __float_as_uint(m[v]);
            w[kVals + kVpl + v] = __float_as_uint(s[v]);
        }
    }
    __device__ __forceinline__ void from_words(const uint32_t *w) {
#pragma unroll
        for (int i = 0; i < kVals; ++i) acc[i] = __uint_as_float(w[i]);
#pragma unroll
        for (int v = 0; v < kVpl; ++v) {
            m[v] = __uint_as_float(w[kVals + v]);
            s[v] = __uint_as_float(w[kVals + kVpl + v]);
        }
    }
};

// Plain per-lane float accumulators (the backward ops).
template <int kN>
struct SumAcc {
    float a[kN];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] = 0.0f;
    }
    __device__ __forceinline__ void merge(const SumAcc &o) {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] += o.a[i];
    }
    __device__ __forceinline__ void to_words(uint32_t *w) const {
#pragma unroll
        for (int i = 0; i < kN; ++i) w[i] = __float_as_uint(a[i]);
    }
    __device__ __forceinline__ void from_words(const uint32_t *w) {
#pragma unroll
        for (int i = 0; i < kN; ++i) a[i] = __uint_as_float(w[i]);
    }
};

// Load the chunks of one row of a [rows, cols] matrix into registers as floats.
template <typename T, int kVpl>
__device__ __forceinline__ void load_row_f32(const T *row, const ChunkMap<kVpl, Elem<T>::kPerChunk> &map, float *dst) {
    constexpr int kPer = Elem<T>::kPerChunk;
#pragma unroll
    for (int v = 0; v < kVpl; ++v) {
        if (map.off[v] >= 0) {
            Elem<T>::unpack(ld_stream16(row + map.off[v]), dst + v * kPer);
        } else {
#pragma unroll
            for (int e = 0; e < kPer; ++e) dst[v * kPer + e] = 0.0f;
        }
    }
}

template <typename T, int kVpl>
__device__ __forceinline__ void store_row_f32(T *row, const ChunkMap<kVpl, Elem<T>::kPerChunk> &map, const float *src) {
    constexpr int kPer = Elem<T>::kPerChunk;
#pragma unroll
    for (int v = 0; v < kVpl; ++v)
        if (map.off[v] >= 0) st_stream16(row + map.off[v], Elem<T>::pack(src + v * kPer));
}

template <typename T, int kVpl>
__device__ __forceinline__ void gather_row(const T *row, const ChunkMap<kVpl, Elem<T>::kPerChunk> &map, uint64_t keep,
                                           uint4 *raw) {
#pragma unroll
    for (int v = 0; v < kVpl; ++v)
        if (map.off[v] >= 0) raw[v] = ld_gather16(row + map.off[v], keep);
}

// Empty hooks for ops that carry nothing across rows.
struct NoCarry {};

}  // namespace tgnn
